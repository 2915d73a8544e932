"""Generates tests/golden/*.npz by running the REAL reference modules
(lightseq/training/ops/pytorch/{quantization,torch_transformer_layers}.py) on CPU.

Needs a checkout of bytedance/lightseq, named by $LIGHTSEQ_REF or the first argument;
the tests only read the committed .npz files. Usage:  LIGHTSEQ_REF=<checkout> python tests/golden/gen_golden.py

The reference package's ``lightseq.training`` __init__ JIT-builds CUDA layers at
import, so empty stub packages are registered for ``lightseq.training``,
``.ops`` and ``.ops.pytorch`` before importing the two pure-PyTorch modules.
"""
from __future__ import annotations

import math
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF = os.environ.get("LIGHTSEQ_REF") or (sys.argv[1] if len(sys.argv) > 1 else "")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set LIGHTSEQ_REF (or pass the path) to a checkout of bytedance/lightseq")
sys.path.insert(0, str(ROOT))
sys.path.insert(0, REF)


def import_reference():
    import lightseq  # noqa: F401

    for name in ("lightseq.training", "lightseq.training.ops", "lightseq.training.ops.pytorch"):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(REF, *name.split("."))]
        sys.modules[name] = m
    from lightseq.training.ops.pytorch import quantization as qz
    from lightseq.training.ops.pytorch import torch_transformer_layers as tl

    return qz, tl


qz, tl = import_reference()
from lightseq_b200 import synth  # noqa: E402


def set_qlinear(m, amax, name):
    """Clip-max plumbing: learned quantisers read Clip.clip_value_max, fixed ones ``_amax``
    (tensor_quantizer.py:340-347)."""
    if m.input_quant is not None:
        m.input_quant.clip.clip_value_max.data.fill_(amax[name + ".in"])
    if m.output_quant is not None:
        m.output_quant._amax.fill_(amax[name + ".out"])


def load_linear(m, w, name, amax, w_amax=None):
    m.weight.data.copy_(torch.from_numpy(w[name + ".w"]))
    if m.bias is not None:
        m.bias.data.copy_(torch.from_numpy(w[name + ".b"]))
    m.weight_quant._amax.fill_(amax[w_amax or name + ".w"])
    set_qlinear(m, amax, name)


def load_ln(m, w, name):
    m.weight.data.copy_(torch.from_numpy(w[name + ".g"]))
    m.bias.data.copy_(torch.from_numpy(w[name + ".b"]))


def build_encoder_layer(w, amax, p, hidden, heads, ffn, act="relu", pre_ln=True):
    cfg = tl.TransformerEncoderLayer.get_config(
        max_batch_tokens=4096, max_seq_len=256, hidden_size=hidden, intermediate_size=ffn, nhead=heads,
        attn_prob_dropout_ratio=0.0, activation_dropout_ratio=0.0, hidden_dropout_ratio=0.0,
        pre_layer_norm=pre_ln, fp16=False, local_rank=-1, activation_fn=act)
    lyr = tl.TransformerEncoderLayer(cfg)
    load_linear(lyr.self_attn.qkv_proj, w, p + ".qkv", amax)
    load_linear(lyr.self_attn.out_proj, w, p + ".out", amax)
    load_linear(lyr.fc1, w, p + ".fc1", amax)
    load_linear(lyr.fc2, w, p + ".fc2", amax)
    load_ln(lyr.self_attn_layer_norm, w, p + ".ln1")
    load_ln(lyr.final_layer_norm, w, p + ".ln2")
    lyr.eval()
    lyr.apply(qz.enable_quant)
    return lyr


def build_decoder_layer(w, amax, p, hidden, heads, ffn, n_dec, act="relu"):
    cfg = tl.TransformerDecoderLayer.get_config(
        max_batch_tokens=4096, max_seq_len=256, hidden_size=hidden, intermediate_size=ffn, nhead=heads,
        attn_prob_dropout_ratio=0.0, activation_dropout_ratio=0.0, hidden_dropout_ratio=0.0,
        pre_layer_norm=True, fp16=False, local_rank=-1, nlayer=n_dec, activation_fn=act)
    lyr = tl.TransformerDecoderLayer(cfg)
    load_linear(lyr.self_attn.qkv_proj, w, p + ".qkv", amax)
    lyr.self_attn.attention_quant._amax.fill_(amax[p + ".kv"])
    load_linear(lyr.self_attn.out_proj, w, p + ".out", amax)
    load_linear(lyr.encoder_attn.q_proj, w, p + ".xq", amax)
    load_linear(lyr.encoder_attn.k_proj, w, p + ".xk", amax)
    load_linear(lyr.encoder_attn.v_proj, w, p + ".xv", amax)
    load_linear(lyr.encoder_attn.out_proj, w, p + ".xout", amax)
    load_linear(lyr.fc1, w, p + ".fc1", amax)
    load_linear(lyr.fc2, w, p + ".fc2", amax)
    load_ln(lyr.self_attn_layer_norm, w, p + ".ln1")
    load_ln(lyr.encoder_attn_layer_norm, w, p + ".ln2")
    load_ln(lyr.final_layer_norm, w, p + ".ln3")
    lyr.eval()
    lyr.apply(qz.enable_quant)
    return lyr


def build_embedding(w, amax, hidden, vocab, pad_id):
    cfg = tl.TransformerEmbeddingLayer.get_config(
        vocab_size=vocab, embedding_dim=hidden, max_batch_tokens=4096, max_seq_len=1024, padding_idx=pad_id,
        dropout=0.0, fp16=False, local_rank=-1)
    emb = tl.TransformerEmbeddingLayer(cfg)
    emb.emb_lookup.weight.data.copy_(torch.from_numpy(w["emb"]))
    emb.emb_quant.clip.clip_value_max.data.fill_(amax["emb"])
    emb.eval()
    emb.apply(qz.enable_quant)
    return emb


@torch.no_grad()
def golden_c0():
    """BASELINE config 0: one transformer-base encoder layer, batch 8 x padded seq 64."""
    H, heads, F = 512, 8, 2048
    rng = np.random.default_rng(4321)
    x = rng.standard_normal((8, 64, H), dtype=np.float32)
    lens = rng.integers(16, 65, size=8)
    pad = (np.arange(64)[None, :] >= lens[:, None])
    w = synth.transformer_weights(H, heads, F, 1, 0, vocab=8, seed=1234)
    # calibration: 4*std of every quantised tensor, from the reference layer with quantisers off
    lyr = build_encoder_layer(w, {k: 1.0 for k in _enc_amax_names("enc.0")}, "enc.0", H, heads, F)
    lyr.apply(qz.disable_quant)
    stats = {}
    hooks = []

    def hook(name):
        def f(mod, inp, out):
            stats[name + ".in"] = float(4 * inp[0].std())
            stats[name + ".out"] = float(4 * (out - (mod.bias if mod.bias is not None else 0)).std())
        return f

    for name, m in (("enc.0.qkv", lyr.self_attn.qkv_proj), ("enc.0.out", lyr.self_attn.out_proj),
                    ("enc.0.fc1", lyr.fc1), ("enc.0.fc2", lyr.fc2)):
        hooks.append(m.register_forward_hook(hook(name)))
    lyr(torch.from_numpy(x), torch.from_numpy(pad))
    for h in hooks:
        h.remove()
    amax = dict(stats)
    for n in ("qkv", "out", "fc1", "fc2"):
        amax[f"enc.0.{n}.w"] = float(np.float32(4 * w[f"enc.0.{n}.w"].std()))
    lyr = build_encoder_layer(w, amax, "enc.0", H, heads, F)
    y = lyr(torch.from_numpy(x), torch.from_numpy(pad)).numpy()
    np.savez_compressed(HERE / "c0_encoder_layer.npz", lens=lens, y=y.astype(np.float32),
                        amax_names=np.array(list(amax.keys())), amax_vals=np.array(list(amax.values()), np.float32))
    print("c0: y", y.shape, "mean|y|", float(np.abs(y).mean()))


def _enc_amax_names(p):
    return [f"{p}.{n}.{s}" for n in ("qkv", "out", "fc1", "fc2") for s in ("in", "w", "out")]


@torch.no_grad()
def golden_small_seq2seq():
    """A small enc-dec model (H 64, 4 heads, FFN 128, 2+2 layers, vocab 96): encoder output,
    cross K/V, and 6 teacher-forced incremental decoder steps with beam-like row duplication."""
    H, heads, F, V, n_enc, n_dec, pad_id = 64, 4, 128, 96, 2, 2, 1
    conf, amax, w = synth.make_transformer(None, hidden=H, heads=heads, ffn=F, n_enc=n_enc, n_dec=n_dec, vocab=V,
                                           max_step=32, seed=77)
    src = synth.transformer_inputs(batch=3, min_len=5, max_len=11, vocab=V, pad_id=pad_id, seed=5)
    rng = np.random.default_rng(11)
    steps = 6
    beam = 2
    T = src.shape[0] * beam
    tgt = rng.integers(4, V, size=(T, steps)).astype(np.int64)
    tgt[:, 0] = 2

    emb = build_embedding(w, amax, H, V, pad_id)
    enc_layers = [build_encoder_layer(w, amax, f"enc.{l}", H, heads, F) for l in range(n_enc)]
    dec_layers = [build_decoder_layer(w, amax, f"dec.{l}", H, heads, F, n_dec) for l in range(n_dec)]
    enc_ln = torch.nn.LayerNorm(H)
    load_ln(enc_ln, w, "enc.ln")
    dec_ln = torch.nn.LayerNorm(H)
    load_ln(dec_ln, w, "dec.ln")
    # output projection shares the embedding table and its quantiser (ls_transformer.py:393-400)
    proj = qz.QuantLinear(H, V, bias=False)
    proj.weight_quant = emb.emb_quant
    proj.weight = emb.emb_lookup.weight
    set_qlinear(proj, amax, "logits")
    proj.eval()
    proj.apply(qz.enable_quant)

    tsrc = torch.from_numpy(src.astype(np.int64))
    pad = tsrc.eq(pad_id)
    x = emb(tsrc)
    enc_emb = x.numpy().copy()
    enc_ys = []
    for lyr in enc_layers:
        x = lyr(x, pad)
        enc_ys.append(x.numpy().copy())
    enc_out = enc_ln(x)
    out = {"src": src, "tgt": tgt, "enc_emb": enc_emb, "enc_out": enc_out.numpy()}
    for l, y in enumerate(enc_ys):
        out[f"enc_y{l}"] = y
    enc_tbc = enc_out.transpose(0, 1)  # [S,B,H]
    inc = {}
    logits = []
    dec_x = []
    for s in range(steps):
        tok = torch.from_numpy(tgt[:, s:s + 1])
        x = emb(tok, s)
        for lyr in dec_layers:
            x, _, _ = lyr(x, encoder_out=enc_tbc, encoder_padding_mask=pad, incremental_state=inc)
        x = dec_ln(x)
        dec_x.append(x[:, 0].numpy().copy())
        logits.append(proj(x)[:, 0].numpy().copy())
    out["dec_x"] = np.stack(dec_x, 1)
    out["logits"] = np.stack(logits, 1)
    np.savez_compressed(HERE / "small_seq2seq.npz", **out)
    print("small seq2seq: logits", out["logits"].shape)


@torch.no_grad()
def golden_quantizer():
    """Known-answer vectors of fake_tensor_quant itself, signed and unsigned, incl. half-way points."""
    from lightseq.training.pytorch_quantization.tensor_quant import fake_tensor_quant

    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 3,
                        (np.arange(-130, 131, dtype=np.float32) + 0.5) * np.float32(2.5 / 127),
                        np.array([0.0, 2.5, -2.5, 1e-8, -1e-8, 100.0, -100.0], np.float32)])
    amax = np.float32(2.5)
    ys = fake_tensor_quant(torch.from_numpy(x), torch.tensor(amax)).numpy()
    xu = np.abs(x)
    yu = fake_tensor_quant(torch.from_numpy(xu), torch.tensor(amax), 8, True).numpy()
    np.savez_compressed(HERE / "quantizer.npz", x=x, amax=amax, y_signed=ys, y_unsigned=yu)
    print("quantizer vectors", x.size)


@torch.no_grad()
def golden_small_bert():
    """BertEmbeddingLayer + two post-LN GELU encoder layers (H 64, 1 head... here 2 heads of 32 are not
    supported by the engine, so H 128 / 2 heads), vocab 120, batch 3 x seq 12 with padding."""
    H, heads, F, V, n_layer, pad_id, S = 128, 2, 256, 120, 2, 0, 12
    conf, amax, w = synth.make_bert(None, hidden=H, heads=heads, ffn=F, n_layer=n_layer, vocab=V, max_step=16, seed=21)
    ids = synth.bert_inputs(batch=3, seq=S, vocab=V, pad_id=pad_id, seed=8)
    cfg = tl.BertEmbeddingLayer.get_config(
        vocab_size=V, embedding_dim=H, max_batch_tokens=4096, max_seq_len=16, padding_idx=pad_id, dropout=0.0,
        fp16=False, local_rank=-1)
    cfg.type_vocab_size = 2
    cfg.layer_norm_eps = 1e-5
    emb = tl.BertEmbeddingLayer(cfg)
    emb.word_embeddings.weight.data.copy_(torch.from_numpy(w["emb"]))
    emb.position_embeddings.weight.data.copy_(torch.from_numpy(w["pos"]))
    emb.token_type_embeddings.weight.data.copy_(torch.from_numpy(w["type_emb"]))
    load_ln(emb.LayerNorm, w, "emb.ln")
    emb.emb_quant.clip.clip_value_max.data.fill_(amax["emb"])
    emb.eval()
    emb.apply(qz.enable_quant)
    layers = [build_encoder_layer(w, amax, f"enc.{l}", H, heads, F, act="gelu", pre_ln=False) for l in range(n_layer)]
    t = torch.from_numpy(ids.astype(np.int64))
    x = emb(t)
    out = {"ids": ids, "emb_out": x.numpy().copy()}
    pad = t.eq(pad_id)
    for l, lyr in enumerate(layers):
        x = lyr(x, pad)
        out[f"y{l}"] = x.numpy().copy()
    np.savez_compressed(HERE / "small_bert.npz", **out)
    print("small bert:", out["y1"].shape)


@torch.no_grad()
def golden_small_gpt():
    """GPT-2 layout: quantised token embedding + learned positions, two decoder-only layers
    (TransformerDecoderLayer with has_cross_attn=False -> causal self-attention on attention_quant(qkv)),
    final LayerNorm and the lm_head QuantLinear that shares the embedding table and quantiser
    (examples/training/huggingface/gpt/ls_hf_gpt_layer.py:44-139). Full-sequence forward, batch 3 x 10."""
    H, heads, F, V, n_layer, S = 128, 2, 256, 150, 2, 10
    conf, amax, w = synth.make_gpt(None, hidden=H, heads=heads, ffn=F, n_layer=n_layer, vocab=V, max_step=16, end_id=149, seed=31)
    ids = synth.gpt_inputs(batch=3, prompt=S, vocab=V, seed=6)
    from lightseq.training.pytorch_quantization.nn.modules.tensor_quantizer import TensorQuantizer

    emb_quant = TensorQuantizer(qz.emb_quant_config)
    emb_quant.clip.clip_value_max.data.fill_(amax["emb"])
    emb_quant.apply(qz.enable_quant)
    wte = torch.nn.Parameter(torch.from_numpy(w["emb"]))
    layers = []
    for l in range(n_layer):
        p = f"dec.{l}"
        cfg = tl.TransformerDecoderLayer.get_config(
            max_batch_tokens=4096, max_seq_len=256, hidden_size=H, intermediate_size=F, nhead=heads,
            attn_prob_dropout_ratio=0.0, activation_dropout_ratio=0.0, hidden_dropout_ratio=0.0,
            pre_layer_norm=True, fp16=False, local_rank=-1, nlayer=n_layer, activation_fn="gelu", has_cross_attn=False)
        lyr = tl.TransformerDecoderLayer(cfg)
        load_linear(lyr.self_attn.qkv_proj, w, p + ".qkv", amax)
        lyr.self_attn.attention_quant._amax.fill_(amax[p + ".kv"])
        load_linear(lyr.self_attn.out_proj, w, p + ".out", amax)
        load_linear(lyr.fc1, w, p + ".fc1", amax)
        load_linear(lyr.fc2, w, p + ".fc2", amax)
        load_ln(lyr.self_attn_layer_norm, w, p + ".ln1")
        load_ln(lyr.final_layer_norm, w, p + ".ln2")
        lyr.eval()
        lyr.apply(qz.enable_quant)
        layers.append(lyr)
    ln_f = torch.nn.LayerNorm(H)
    load_ln(ln_f, w, "dec.ln")
    head = qz.QuantLinear(H, V, bias=False)
    head.weight = wte
    head.weight_quant = emb_quant
    set_qlinear(head, amax, "logits")
    head.eval()
    head.apply(qz.enable_quant)
    t = torch.from_numpy(ids.astype(np.int64))
    x = emb_quant(torch.nn.functional.embedding(t, wte)) + torch.from_numpy(w["pos"][:S])
    for lyr in layers:
        x, _, _ = lyr(x)
    h = ln_f(x)
    logits = head(h)
    np.savez_compressed(HERE / "small_gpt.npz", ids=ids, hidden=h.numpy(), logits=logits.numpy())
    print("small gpt: logits", tuple(logits.shape))


@torch.no_grad()
def golden_generation():
    """Beam-4 generation of a small encoder-decoder assembled from the reference's own modules (oracle/ref_torch.py:
    every layer computation is the reference's, the beam step between decoder calls is oracle/beam.py). Pins
    oracle.model.Seq2Seq.generate end to end: tokens, scores and the number of decode steps, with early stop."""
    from oracle import model as om
    from oracle import ref_torch as rt

    kw = dict(hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=300, max_step=32, beam=4, extra_decode_length=8, seed=5)
    conf, amax, w = synth.make_transformer(None, **kw)
    u = np.sign(np.random.default_rng(0).standard_normal(128)).astype(np.float32)
    w["dec.ln.b"] = (0.15 * u).astype(np.float32)      # EOS made competitive: beams finish at different steps
    w["emb"][int(conf["end_id"])] = (0.02 * u).astype(np.float32)
    cfg = om.Config(hidden=128, heads=2, ffn=256, n_enc=2, n_dec=2, vocab=300, max_step=32, beam=4, extra_decode_length=8,
                    length_penalty=float(conf["length_penalty"]), pad_id=int(conf["pad_id"]), start_id=int(conf["start_id"]),
                    end_id=int(conf["end_id"]))
    src = synth.transformer_inputs(batch=6, min_len=3, max_len=9, vocab=300, seed=2)
    tok, score, n = rt.RefSeq2Seq((qz, tl), cfg, w, amax).generate(src)
    np.savez_compressed(HERE / "small_seq2seq_generation.npz", src=src, tokens=tok, scores=score, n=np.int32(n))
    print("generation: tokens", tok.shape, "steps", n)


if __name__ == "__main__":
    torch.manual_seed(0)
    golden_quantizer()
    golden_c0()
    golden_small_seq2seq()
    golden_small_bert()
    golden_small_gpt()
    golden_generation()
