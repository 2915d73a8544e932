"""CPU-only checks of the host side: the weight container, the C ABI library's exported symbols (no compute
calls), argument validation that needs no GPU, the synthetic-model calibration, and replica sharding under a
world-size-2 gloo process group."""
import ctypes as C
import os
import re
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_weight_container_round_trip(tmp_path):
    from lightseq_b200 import weights

    tens = {"a.w": np.arange(12, dtype=np.float32).reshape(3, 4), "b": np.ones(7, np.float32) * 0.5}
    p = str(tmp_path / "m.ls100")
    weights.save(p, "QuantTransformer", {"hidden": 4, "beam": 4.0}, {"a.w": 0.25}, tens)
    model, conf, amax, back = weights.load(p)
    assert model == "QuantTransformer" and conf == {"hidden": 4.0, "beam": 4.0} and amax == {"a.w": 0.25}
    assert all(np.array_equal(back[k], v) for k, v in tens.items())
    with open(p, "r+b") as f:
        f.write(b"XX")
    with pytest.raises(ValueError):
        weights.load(p)


def test_library_exports_every_declared_symbol():
    """Every function declared in include/ls100.h must be exported by libls100.so (built by build())."""
    import __graft_entry__ as g

    g.build()
    from lightseq_b200 import _lib

    header = (ROOT / "include" / "ls100.h").read_text()
    names = set(re.findall(r"\b(ls100_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 20
    for n in sorted(names):
        assert hasattr(_lib.lib, n), f"{n} is declared in include/ls100.h but not exported"
    assert _lib.lib.ls100_strerror(-5).decode().startswith("a bounded device-side wait")


def test_ctypes_structures_have_the_layout_of_the_header(tmp_path):
    """The argument structs cross the C ABI by pointer: the ctypes mirror of every one must have the size the C
    compiler gives the declaration in include/ls100.h, and its last member must sit at the same offset (a member
    appended in the header but not in the mirror would leave it unset and go unnoticed otherwise)."""
    import shutil
    import subprocess

    from lightseq_b200 import _lib as L

    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    pairs = {"ls100_gemm_i8_args": L.GemmI8Args, "ls100_embed_args": L.EmbedArgs, "ls100_ln_quant_args": L.LnQuantArgs,
             "ls100_patch_embed_args": L.PatchEmbedArgs, "ls100_attn_self_args": L.AttnSelfArgs,
             "ls100_attn_dec_args": L.AttnDecArgs, "ls100_attn_cross_args": L.AttnCrossArgs, "ls100_proj_f32_args": L.ProjF32Args,
             "ls100_proj_tc_args": L.ProjTcArgs, "ls100_beam_topk_args": L.BeamTopkArgs, "ls100_beam_select_args": L.BeamSelectArgs,
             "ls100_beam_update_args": L.BeamUpdateArgs, "ls100_beam_result_args": L.BeamResultArgs,
             "ls100_sample_topk_args": L.SampleTopkArgs, "ls100_sample_topp_args": L.SampleToppArgs}
    header = (ROOT / "include" / "ls100.h").read_text()
    last = {}
    for name in pairs:  # last member of the C declaration
        body = header[:header.index("} " + name + ";")]
        body = body[body.rindex("typedef struct {"):]
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        decl = [d.strip() for d in body.split(";") if d.strip()][-1]
        last[name] = re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*(?:\[[^\]]*\])?$", decl.split(",")[-1].strip())[0]
    src = ["#include <stdio.h>", "#include <stddef.h>", '#include "ls100.h"', "int main(void) {"]
    for name in pairs:
        src.append(f'  printf("{name} %zu %zu\\n", sizeof({name}), offsetof({name}, {last[name]}));')
    src += ["  return 0;", "}"]
    c = tmp_path / "layout.c"
    c.write_text("\n".join(src))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = 0
    for line in out.splitlines():
        name, size, off = line.split()
        cls = pairs[name]
        assert C.sizeof(cls) == int(size), f"{name}: header {size} bytes, ctypes {C.sizeof(cls)}"
        assert getattr(cls, cls._fields_[-1][0]).offset == int(off), f"{name}: last member at {off} in the header"
        assert cls._fields_[-1][0] == last[name], f"{name}: last member {last[name]} in the header, {cls._fields_[-1][0]} in ctypes"
        seen += 1
    assert seen == len(pairs)


def test_null_arguments_are_rejected_without_a_gpu():
    from lightseq_b200 import _lib as L

    assert L.lib.ls100_ctx_create(None, 0) == L.ERR_BAD_ARG
    assert L.lib.ls100_gemm_i8(None, None, None) == L.ERR_BAD_ARG
    assert L.lib.ls100_ln_quant(None, None, None) == L.ERR_BAD_ARG
    L.lib.ls100_model_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]
    h = C.c_void_p()
    assert L.lib.ls100_model_create(b"NoSuchModel", b"/nonexistent", 1, C.byref(h)) != 0
    L.lib.ls100_model_last_error.restype = C.c_char_p
    assert len(L.lib.ls100_model_last_error()) > 0  # what the C++ API would have thrown


def test_synthetic_model_is_seeded_and_calibrated():
    from lightseq_b200 import synth

    c1, a1, w1 = synth.make_transformer(None, hidden=64, heads=1, ffn=128, n_enc=1, n_dec=1, vocab=50, max_step=16, seed=3)
    c2, a2, w2 = synth.make_transformer(None, hidden=64, heads=1, ffn=128, n_enc=1, n_dec=1, vocab=50, max_step=16, seed=3)
    assert a1 == a2 and all(np.array_equal(w1[k], w2[k]) for k in w1)
    assert abs(a1["enc.0.qkv.w"] - 4 * w1["enc.0.qkv.w"].std()) < 1e-6
    for k in ("enc.0.qkv.in", "enc.0.fc2.out", "dec.0.kv", "dec.0.xq.out", "logits.in", "logits.out", "emb"):
        assert a1[k] > 0


def test_shard_and_merge_single_process():
    from lightseq_b200 import sharding, synth

    ids = synth.transformer_inputs(batch=11, min_len=2, max_len=9, vocab=40, seed=1)
    shards = sharding.shard_batch(ids, 1, 4)
    assert sorted(np.concatenate([r for r, _ in shards]).tolist()) == list(range(11))
    for rows, sub in shards:
        assert sub.shape[0] == len(rows) and (sub[:, -1] != 1).any()
        assert np.array_equal(sub, ids[rows, : sub.shape[1]])
    outs = [(rows, np.full((len(rows), 1, 3 + i), 7, np.int32), np.full((len(rows), 1), float(i), np.float32))
            for i, (rows, _) in enumerate(shards)]
    tok, sc = sharding.merge_results(11, outs, end_id=2)
    assert tok.shape == (11, 1, 6)
    for i, (rows, _) in enumerate(shards):
        assert (sc[rows, 0] == i).all() and (tok[rows, 0, : 3 + i] == 7).all() and (tok[rows, 0, 3 + i:] == 2).all()


_WORKER = r"""
import os, sys
import numpy as np
import torch.distributed as dist
sys.path.insert(0, os.environ["LS100_ROOT"])
from lightseq_b200 import sharding, synth
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
ids = synth.transformer_inputs(batch=10, min_len=2, max_len=9, vocab=40, seed=1)
rows, sub = sharding.shard_batch(ids, 1, world)[rank]
# stand-in for the per-rank engine: "generate" the reversed non-pad source ids
toks = np.full((len(rows), 1, sub.shape[1]), 2, np.int32)
for i in range(len(rows)):
    n = int((sub[i] != 1).sum())
    toks[i, 0, :n] = sub[i, :n][::-1]
gathered = [None] * world
dist.all_gather_object(gathered, (rows, toks, np.full((len(rows), 1), float(rank), np.float32)))
if rank == 0:
    tok, sc = sharding.merge_results(10, gathered, end_id=2)
    for b in range(10):
        n = int((ids[b] != 1).sum())
        assert (tok[b, 0, :n] == ids[b, :n][::-1]).all() and (tok[b, 0, n:] == 2).all()
    assert set(sc[:, 0].tolist()) == {0.0, 1.0}
    print("MERGE_OK")
dist.destroy_process_group()
"""


def test_replica_sharding_world_size_2_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, LS100_ROOT=str(ROOT))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "MERGE_OK" in r.stdout


def test_torch_extension_surface_has_the_reference_entry_points():
    """The names the reference's training-side extension exports for the quantised layers
    (lightseq/csrc/pybind/pybind_layer.cpp:480-571); calling them needs a GPU, importing does not."""
    from lightseq_b200 import torch_ext as te

    for name in ("create_quant_linear_layer_fp32", "create_quant_linear_layer_fp16", "quant_linear_layer_fw_fp32",
                 "quant_linear_layer_fw_fp16", "create_transformer_encoder_layer_fp32", "create_transformer_encoder_layer_fp16",
                 "transformer_encoder_layer_fw_fp32", "transformer_encoder_layer_fw_fp16", "assign_layer_weight_grad"):
        assert callable(getattr(te, name))
    assert te._gen_offset(4, 8)[-1] == 4 * 4 * 3 + 12 + 16 + 4 + 8 + 32 + 8 + 32 + 4 + 8 + 12
    import torch

    assert te.create_quant_linear_layer_fp32(1, 64, 32, 16) == 0
    with pytest.raises(RuntimeError, match="CUDA"):
        te.quant_linear_layer_fw_fp32(1, torch.zeros(1, 4, 64), torch.zeros(32, 64), torch.ones(3), True)
