"""Torch-tensor entry points (lightseq_b200.torch_ext) against the oracle's QuantLinear: the fp32 form is bit-exact,
the fp16 form equals the fp32 result rounded to half; error behaviour follows the reference's CHECK_INPUT."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import model as om  # noqa: E402
from oracle import quant as oq  # noqa: E402

F32 = np.float32


def _case(seed, b, s, k, n):
    r = np.random.default_rng(seed)
    x = r.standard_normal((b, s, k)).astype(F32)
    w = (r.standard_normal((n, k)) * 0.02).astype(F32)
    amax = {"l.in": float(F32(4 * x.std())), "l.w": float(F32(4 * w.std())),
            "l.out": float(F32(4 * (x.reshape(-1, k) @ w.T).std()))}
    ref = om.qlinear(om.State(w={"l.w": w}, amax=amax), x.reshape(-1, k), "l", bias=False).reshape(b, s, n)
    return x, w, amax, ref


@pytest.mark.parametrize("b,s,k,n", [(4, 33, 512, 512), (2, 7, 64, 48), (8, 64, 512, 2048)])
def test_quant_linear_layer_fw_fp32_bit_exact(b, s, k, n):
    from lightseq_b200 import torch_ext as te

    x, w, amax, ref = _case(b + s + k, b, s, k, n)
    assert te.create_quant_linear_layer_fp32(7, k, n, b * s) == 0
    cm = torch.tensor([amax["l.in"], amax["l.w"], amax["l.out"]], device="cuda")
    xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = te.quant_linear_layer_fw_fp32(7, xt, wt, cm, True)
    torch.cuda.synchronize()
    assert out.shape == (b, s, n) and out.dtype == torch.float32
    assert np.array_equal(out.cpu().numpy(), ref)
    # the clip-max tensor is re-read after an in-place change
    cm[2] *= 2
    out2 = te.quant_linear_layer_fw_fp32(7, xt, wt, cm, True)
    amax2 = dict(amax)
    amax2["l.out"] = float(F32(amax["l.out"]) * F32(2))
    ref2 = om.qlinear(om.State(w={"l.w": w}, amax=amax2), x.reshape(-1, k), "l", bias=False).reshape(b, s, n)
    assert np.array_equal(out2.cpu().numpy(), ref2)
    # unquantised mode is the plain linear map
    plain = te.quant_linear_layer_fw_fp32(7, xt, wt, cm, False)
    assert torch.allclose(plain, torch.nn.functional.linear(xt, wt))


def test_quant_linear_layer_fw_fp16_and_errors():
    from lightseq_b200 import torch_ext as te

    b, s, k, n = 3, 20, 256, 128
    x, w, amax, _ = _case(5, b, s, k, n)
    xh, wh = torch.from_numpy(x).cuda().half(), torch.from_numpy(w).cuda().half()
    ref = om.qlinear(om.State(w={"l.w": wh.float().cpu().numpy()}, amax=amax), xh.float().cpu().numpy().reshape(-1, k), "l",
                     bias=False).reshape(b, s, n)
    te.create_quant_linear_layer_fp16(9, k, n, 64)
    cm = torch.tensor([amax["l.in"], amax["l.w"], amax["l.out"]], device="cuda", dtype=torch.float16)
    amax_h = {key: float(v) for key, v in zip(("l.in", "l.w", "l.out"), cm.float().cpu().tolist())}
    ref = om.qlinear(om.State(w={"l.w": wh.float().cpu().numpy()}, amax=amax_h), xh.float().cpu().numpy().reshape(-1, k), "l",
                     bias=False).reshape(b, s, n)
    out = te.quant_linear_layer_fw_fp16(9, xh, wh, cm, True)
    assert out.dtype == torch.float16
    assert np.array_equal(out.cpu().numpy(), ref.astype(np.float16))
    with pytest.raises(RuntimeError, match="max_batch_tokens"):
        te.quant_linear_layer_fw_fp16(9, torch.zeros(4, 20, k, device="cuda", dtype=torch.float16), wh, cm, True)
    with pytest.raises(RuntimeError, match="contiguous"):
        te.quant_linear_layer_fw_fp16(9, xh.transpose(0, 1), wh, cm, True)
    with pytest.raises(RuntimeError, match="CUDA"):
        te.quant_linear_layer_fw_fp16(9, xh.cpu(), wh, cm, True)
    with pytest.raises(RuntimeError, match="not been created"):
        te.quant_linear_layer_fw_fp32(12345, xh.float(), wh.float(), cm.float(), True)


def _flat_params(w, amax, prefix):
    """The flat parameter tensor of LSTransformerEncoderLayer (transformer_encoder_layer.py:154-172)."""
    order = ["qkv.w", "qkv.b", "out.w", "out.b", "ln1.g", "ln1.b", "fc1.w", "fc1.b", "fc2.w", "fc2.b", "ln2.g", "ln2.b"]
    parts = [w[f"{prefix}.{n}"].reshape(-1).astype(F32) for n in order]
    cm = [amax[f"{prefix}.{l}.{k}"] for l in ("qkv", "out", "fc1", "fc2") for k in ("in", "w", "out")]
    return np.concatenate(parts + [np.array(cm, F32)])


def test_transformer_encoder_layer_fw_matches_oracle_and_reference_golden():
    """BASELINE config 0 (one pre-LN ReLU encoder layer, 8 x 64 x 512, padding mask) through
    transformer_encoder_layer_fw_fp32: against the numpy oracle (differences only where the fp32 attention sums flip
    an int8 value) and against the output of the reference's own TransformerEncoderLayer stored in the golden file
    (the tolerance the oracle itself is pinned with)."""
    from pathlib import Path

    from lightseq_b200 import synth
    from lightseq_b200 import torch_ext as te

    g = np.load(Path(__file__).parent / "golden" / "c0_encoder_layer.npz")
    amax = dict(zip([str(s) for s in g["amax_names"]], [float(v) for v in g["amax_vals"]]))
    w = synth.transformer_weights(512, 8, 2048, 1, 0, vocab=8, seed=1234)
    r = np.random.default_rng(4321)
    x = r.standard_normal((8, 64, 512), dtype=np.float32)
    lens = r.integers(16, 65, size=8)
    pad = np.arange(64)[None, :] >= lens[:, None]
    cfg = om.Config(hidden=512, heads=8, ffn=2048, n_enc=1, n_dec=0)
    y_or = om.encoder_layer(om.State(w=w, amax=amax), x, pad, "enc.0", cfg)

    assert te.create_transformer_encoder_layer_fp32(3, 8 * 64, 64, 512, 8, 2048, 0.0, 0.0, 0.0, True, "relu", False) == 0
    para = torch.from_numpy(_flat_params(w, amax, "enc.0")).cuda()
    te.assign_layer_weight_grad(3, para, None, "TransformerEncoderLayer")
    (out,) = te.transformer_encoder_layer_fw_fp32(3, torch.from_numpy(x).cuda(), torch.from_numpy(pad.astype(F32)).cuda(),
                                                  False, True, True)
    torch.cuda.synchronize()
    y = out.cpu().numpy()
    valid = ~pad
    d = np.abs(y - y_or)[valid]
    print("vs oracle: max", d.max(), "mean", d.mean(), "frac > 1e-4", (d > 1e-4).mean())
    assert d.mean() < 2e-4 and (d > 1e-4).mean() < 0.01
    dr = np.abs(y - g["y"])[valid]
    step = amax["enc.0.fc2.out"] / 127
    print("vs reference golden: max", dr.max(), "mean", dr.mean())
    assert dr.mean() < 1e-3 and dr.max() < 2e-2 + 2 * step and (dr > 1e-4).mean() < 0.02
    # same parameters, same input: same output; an in-place parameter change is picked up
    (out2,) = te.transformer_encoder_layer_fw_fp32(3, torch.from_numpy(x).cuda(), torch.from_numpy(pad.astype(F32)).cuda(),
                                                   False, True, True)
    assert torch.equal(out, out2)
    with pytest.raises(RuntimeError, match="forward-only"):
        te.transformer_encoder_layer_fw_fp32(3, out, torch.zeros(8, 64, device="cuda"), True, True, True)


def test_transformer_encoder_layer_fw_post_ln_gelu():
    """BERT-style layer (post-LN, GELU) through the same entry point vs the oracle."""
    from lightseq_b200 import synth
    from lightseq_b200 import torch_ext as te

    H, heads, Fd = 128, 2, 256
    conf, amax, w = synth.make_bert(None, hidden=H, heads=heads, ffn=Fd, n_layer=1, vocab=50, max_step=32, seed=3)
    r = np.random.default_rng(8)
    x = r.standard_normal((3, 20, H)).astype(F32)
    pad = np.arange(20)[None, :] >= np.array([20, 11, 5])[:, None]
    cfg = om.Config(hidden=H, heads=heads, ffn=Fd, n_enc=1, n_dec=0, act="gelu", pre_ln=False)
    y_or = om.encoder_layer(om.State(w=w, amax=amax), x, pad, "enc.0", cfg)
    te.create_transformer_encoder_layer_fp32(4, 64, 32, H, heads, Fd, 0.0, 0.0, 0.0, False, "gelu", False)
    te.assign_layer_weight_grad(4, torch.from_numpy(_flat_params(w, amax, "enc.0")).cuda(), None, "TransformerEncoderLayer")
    (out,) = te.transformer_encoder_layer_fw_fp32(4, torch.from_numpy(x).cuda(), torch.from_numpy(pad.astype(F32)).cuda(),
                                                  False, False, True)
    d = np.abs(out.cpu().numpy() - y_or)[~pad]
    print("post-LN vs oracle: max", d.max(), "mean", d.mean())
    assert d.mean() < 1e-3 and (d > 1e-3).mean() < 0.02
