"""Stage-wise parity of every CUDA kernel family against the numpy oracle, called through
the C ABI (ctypes). Integer stages (quantised weights, int32 accumulators, requantised
GEMM outputs, embedding, LayerNorm->int8) must be bit-exact; attention outputs go through
fp32 softmax in a different summation order, so their int8 result may differ by one
quantisation step on a small fraction of elements (bound stated per test)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from lightseq_b200 import _lib as L  # noqa: E402
from oracle import beam as ob  # noqa: E402
from oracle import model as om  # noqa: E402
from oracle import quant as oq  # noqa: E402
from tests.gpu_util import ctx, dev, empty, gemm, ptr, sync_check  # noqa: E402

F32 = np.float32


def rng(seed):
    return np.random.default_rng(seed)


# ----------------------------------------------------------------------------- weights
@pytest.mark.parametrize("rows,cols", [(512, 512), (96, 64), (2048, 512), (37, 128)])
def test_quantize_weight_bit_exact(rows, cols):
    w = (rng(1).standard_normal((rows, cols)) * 0.02).astype(F32)
    amax = float(F32(4 * w.std()))
    q_ref, _ = oq.quantize(w, amax)
    dw = dev(w)
    out = empty((rows, cols), torch.int8)
    off = empty((rows,), torch.int32)
    L.check(L.lib.ls100_quantize_weight(ctx().handle, ptr(dw), rows, cols, amax, ptr(out), ptr(off), None), "quantize")
    sync_check()
    assert np.array_equal(out.cpu().numpy(), q_ref)
    assert np.array_equal(off.cpu().numpy(), 127 * q_ref.astype(np.int64).sum(1))


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("m,n,k", [(512, 1536, 512), (200, 80, 256), (7680, 512, 512), (64, 1024, 1024),
                                   (1, 64, 64), (129, 48, 144), (512, 512, 2048)])
def test_gemm_int32_accumulators_bit_exact(m, n, k):
    r = rng(m + n + k)
    a = r.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = r.integers(-127, 128, size=(n, k), dtype=np.int8)
    out = gemm(dev(a), dev(w), s_acc=1.0, out_kind=L.OUT_I32)
    sync_check()
    assert np.array_equal(out.cpu().numpy().astype(np.int64), oq.int_matmul(a, w))


@pytest.mark.parametrize("m,n,k", [(5000, 2440, 208), (19000, 512, 1040), (4096, 2560, 128), (2500, 4136, 400)])
def test_gemm_many_tiles_int32_bit_exact(m, n, k):
    """Problems of more than two tiles per SM take the persistent kernel (static tile list, double-buffered
    accumulators): ragged M, N ending inside a 32-column group and inside either half of a 256-column tile, K
    ending inside a k-block, more and fewer tiles per CTA than accumulator buffers."""
    r = rng(m + n + k)
    a = r.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = r.integers(-127, 128, size=(n, k), dtype=np.int8)
    out = gemm(dev(a), dev(w), s_acc=1.0, out_kind=L.OUT_I32)
    sync_check()
    assert np.array_equal(out.cpu().numpy().astype(np.int64), oq.int_matmul(a, w))


@pytest.mark.parametrize("m,n,k,in_place", [(6000, 1800, 256, False), (16384, 768, 768, True), (4100, 2564, 384, True),
                                            (9000, 772, 128, False)])
def test_gemm_many_tiles_bias_residual_and_offset_bit_exact(m, n, k, in_place):
    """The persistent kernel with every epilogue input in use: unsigned input offset, bias, residual, fp32 out (the
    path that moves the residual and the result through per-warp staging tiles); N ending 4, 8 and 36 columns into a
    256-column tile, ragged M, and the residual buffer doubling as the output as the engine layers use it."""
    st, x, w, b = _qlinear_case(21, m, n, k, unsigned_in=True)
    st.trace = {}
    xq, s_x = oq.quantize(x, st.amax["l.in"], unsigned=True)
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    s_o = oq.scale_of(st.amax["l.out"])
    acc = oq.int_matmul(xq.astype(np.int64) + 127, wq)
    y = (acc.astype(F32) * F32(s_x * s_w))
    y = oq.quantize(y, st.amax["l.out"])[0].astype(F32) * s_o + b
    resid = rng(22).standard_normal((m, n)).astype(F32)
    off = dev((127 * wq.astype(np.int64).sum(1)).astype(np.int32))
    out = gemm(dev(xq), dev(wq), s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_F32, s_outq=float(s_o), bias=dev(b),
               resid=dev(resid), w_off=off, in_place=in_place)
    sync_check()
    assert np.array_equal(out.cpu().numpy(), resid + y)


def test_gemm_many_tiles_fp32_without_residual_bit_exact():
    m, n, k = 7000, 1284, 256
    st, x, w, b = _qlinear_case(31, m, n, k)
    st.trace = {}
    y = om.qlinear(st, x, "l")
    xq, s_x = oq.quantize(x, st.amax["l.in"])
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    out = gemm(dev(xq), dev(wq), s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_F32, s_outq=float(oq.scale_of(st.amax["l.out"])),
               bias=dev(b))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), y)


def _qlinear_case(seed, m, n, k, unsigned_in=False):
    r = rng(seed)
    w = (r.standard_normal((n, k)) * 0.02).astype(F32)
    x = r.standard_normal((m, k)).astype(F32)
    if unsigned_in:
        x = np.maximum(x, 0)
    b = (r.standard_normal(n) * 0.1).astype(F32)
    st = om.State(w={"l.w": w, "l.b": b}, amax={"l.w": float(F32(4 * w.std())), "l.in": float(F32(4 * x.std())),
                                                  "l.out": float(F32(4 * (x @ w.T).std()))})
    return st, x, w, b


def test_gemm_outq_int8_and_bias_residual_bit_exact():
    """QKV-style (int8 of the output quantiser) and out-proj-style (fake-quant + bias + residual, fp32)."""
    m, n, k = 300, 512, 512
    st, x, w, b = _qlinear_case(5, m, n, k)
    st.trace = {}
    y = om.qlinear(st, x, "l")
    xq, s_x = oq.quantize(x, st.amax["l.in"])
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    s_o = oq.scale_of(st.amax["l.out"])
    out = gemm(dev(xq), dev(wq), s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_OUTQ_I8, s_outq=float(s_o))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), st.trace["l.out_q"])
    resid = rng(6).standard_normal((m, n)).astype(F32)
    out = gemm(dev(xq), dev(wq), s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_F32, s_outq=float(s_o), bias=dev(b),
               resid=dev(resid))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), resid + y)


@pytest.mark.parametrize("m,n,k", [(512, 512, 512), (190, 100, 384), (130, 512, 2048), (448, 288, 640)])
def test_gemm_64_row_tiles_every_epilogue_bit_exact(m, n, k):
    """Problems of several row blocks and at most one CTA per SM run 64-row tiles (an M = 64 MMA, 16 active lanes per
    TMEM lane quarter): the out-projection / FFN2 shapes of a decode step, ragged M (last tile of 62 and of 2 rows),
    N ending inside a 32-column tile, K ending inside a k-block; int32, int8 of the output quantiser, fp32 + bias +
    residual in place, and bias + GELU + requantise."""
    st, x, w, b = _qlinear_case(51, m, n, k)
    st.trace = {}
    y = om.qlinear(st, x, "l")
    xq, s_x = oq.quantize(x, st.amax["l.in"])
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    s_o = oq.scale_of(st.amax["l.out"])
    s_acc = float(F32(s_x * s_w))
    out = gemm(dev(xq), dev(wq), s_acc=1.0, out_kind=L.OUT_I32)
    sync_check()
    assert np.array_equal(out.cpu().numpy().astype(np.int64), oq.int_matmul(xq, wq))
    out = gemm(dev(xq), dev(wq), s_acc=s_acc, out_kind=L.OUT_OUTQ_I8, s_outq=float(s_o))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), st.trace["l.out_q"])
    resid = rng(52).standard_normal((m, n)).astype(F32)
    out = gemm(dev(xq), dev(wq), s_acc=s_acc, out_kind=L.OUT_F32, s_outq=float(s_o), bias=dev(b), resid=dev(resid), in_place=True)
    sync_check()
    assert np.array_equal(out.cpu().numpy(), resid + y)
    act = oq.gelu(y)
    amax2 = float(F32(4 * act.std()))
    ref, s2 = oq.quantize(act, amax2)
    out = gemm(dev(xq), dev(wq), s_acc=s_acc, out_kind=L.OUT_REQ_S8, s_outq=float(s_o), bias=dev(b), act=L.ACT_GELU, s_req=float(s2))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("m,n,k", [(512, 512, 512), (300, 512, 2048), (512, 1024, 1024), (130, 256, 128), (260, 768, 768),
                                   (200, 2048, 256), (64, 1024, 4096)])
def test_gemm_fused_layernorm_bit_exact(m, n, k):
    """Residual GEMM with the LayerNorm + quantise of the next sublayer in the same launch (thread-block cluster per
    128-row block, row sums exchanged through distributed shared memory): the fp32 rows equal the oracle's and the
    int8 LayerNorm output equals quantize(layer_norm(rows)). N = 2048 takes the two-launch fallback."""
    st, x, w, b = _qlinear_case(31 + n, m, n, k)
    y = om.qlinear(st, x, "l")
    xq, s_x = oq.quantize(x, st.amax["l.in"])
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    r = rng(m + n)
    resid = r.standard_normal((m, n)).astype(F32)
    g = (1 + 0.1 * r.standard_normal(n)).astype(F32)
    be = (0.1 * r.standard_normal(n)).astype(F32)
    rows = resid + y
    z = om.layer_norm(rows, g, be)
    amax = float(F32(4 * z.std()))
    q_ref, _ = oq.quantize(z, amax)
    out, ln_out = gemm(dev(xq), dev(wq), s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_F32,
                       s_outq=float(oq.scale_of(st.amax["l.out"])), bias=dev(b), resid=dev(resid), ln=(dev(g), dev(be), amax))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), rows)
    assert np.array_equal(ln_out.cpu().numpy(), q_ref)


def test_gemm_ffn_relu_unsigned_chain_bit_exact():
    """fc1 (+bias, ReLU, unsigned requantise) then fc2 with the 127*rowsum offset."""
    m, h, f = 260, 512, 2048
    r = rng(9)
    w1 = (r.standard_normal((f, h)) * 0.02).astype(F32)
    w2 = (r.standard_normal((h, f)) * 0.02).astype(F32)
    b1 = (r.standard_normal(f) * 0.05).astype(F32)
    b2 = (r.standard_normal(h) * 0.05).astype(F32)
    x = r.standard_normal((m, h)).astype(F32)
    h1 = np.maximum(x @ w1.T + b1, 0)
    st = om.State(w={"p.fc1.w": w1, "p.fc1.b": b1, "p.fc2.w": w2, "p.fc2.b": b2},
                  amax={"p.fc1.w": float(F32(4 * w1.std())), "p.fc2.w": float(F32(4 * w2.std())),
                        "p.fc1.in": float(F32(4 * x.std())), "p.fc1.out": float(F32(4 * (x @ w1.T).std())),
                        "p.fc2.in": float(F32(4 * h1.std())), "p.fc2.out": float(F32(4 * (h1 @ w2.T).std()))})
    st.trace = {}
    y = om.ffn(st, x, "p", om.Config(hidden=h, ffn=f))
    xq, s_x = oq.quantize(x, st.amax["p.fc1.in"])
    w1q, s_w1 = oq.quantize(w1, st.amax["p.fc1.w"])
    w2q, s_w2 = oq.quantize(w2, st.amax["p.fc2.w"])
    s_h = oq.scale_of(st.amax["p.fc2.in"], unsigned=True)
    hq = gemm(dev(xq), dev(w1q), s_acc=float(F32(s_x * s_w1)), out_kind=L.OUT_REQ_U8,
              s_outq=float(oq.scale_of(st.amax["p.fc1.out"])), bias=dev(b1), act=L.ACT_RELU, s_req=float(s_h))
    sync_check()
    assert np.array_equal(hq.cpu().numpy(), st.trace["p.fc2.in_q"])
    off = dev((127 * w2q.astype(np.int64).sum(1)).astype(np.int32))
    out = gemm(hq, dev(w2q), s_acc=float(F32(s_h * s_w2)), out_kind=L.OUT_F32,
               s_outq=float(oq.scale_of(st.amax["p.fc2.out"])), bias=dev(b2), w_off=off)
    sync_check()
    assert np.array_equal(out.cpu().numpy(), y)


@pytest.mark.parametrize("m,n,k", [(256, 768, 768), (4096, 3072, 256)])
def test_gemm_gelu_requant_bit_exact(m, n, k):
    """GELU + requantise: the device uses a branch-free fp32 erf and redoes with the float64 erf every element
    whose quantisation could depend on the difference, so the int8 result equals the oracle's (scipy float64
    erf). The large case has 12.6M outputs: an error bound that was too tight by 1e-5 of a quantisation step
    would show as about a hundred mismatches."""
    st, x, w, b = _qlinear_case(11, m, n, k)
    pre = om.qlinear(st, x, "l")
    act = oq.gelu(pre)
    amax2 = float(F32(4 * act.std()))
    ref, s2 = oq.quantize(act, amax2)
    xq, s_x = oq.quantize(x, st.amax["l.in"])
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    out = gemm(dev(xq), dev(wq), s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_REQ_S8,
               s_outq=float(oq.scale_of(st.amax["l.out"])), bias=dev(b), act=L.ACT_GELU, s_req=float(s2))
    sync_check()
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("m,n,k,act,unsigned_out", [(4096, 3072, 256, "gelu", False), (5000, 2440, 208, "relu", True),
                                                    (9000, 2100, 128, "none", False), (16384, 2304, 768, "none", False),
                                                    (300, 512, 256, "gelu", False)])
def test_gemm_requantisation_table_gives_the_computed_bytes(m, n, k, act, unsigned_out):
    """Bias, activation and requantisation read from the per-column table (built on the device with the scalar forms
    of the same roundings) instead of computed per element: the many-tile kernel walks its tiles column by column
    and keeps one 256-column slice of the table in shared memory. The result must equal the oracle AND the bytes of
    the computing path; N ending inside a 64-column group and a 256-column tile, ragged M, K ending inside a
    k-block, and a problem small enough for the one-tile kernel (which ignores the table)."""
    st, x, w, b = _qlinear_case(41, m, n, k)
    pre = om.qlinear(st, x, "l")
    post = {"gelu": oq.gelu, "relu": lambda t: np.maximum(t, 0), "none": lambda t: t}[act](pre)
    amax2 = float(F32(4 * post.std()))
    ref, s2 = oq.quantize(post, amax2, unsigned=unsigned_out)
    xq, s_x = oq.quantize(x, st.amax["l.in"])
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    kw = dict(s_acc=float(F32(s_x * s_w)), out_kind=L.OUT_REQ_U8 if unsigned_out else L.OUT_REQ_S8,
              s_outq=float(oq.scale_of(st.amax["l.out"])), bias=dev(b),
              act={"gelu": L.ACT_GELU, "relu": L.ACT_RELU, "none": L.ACT_NONE}[act], s_req=float(s2))
    computed = gemm(dev(xq), dev(wq), **kw)
    tabled = gemm(dev(xq), dev(wq), table=True, **kw)
    sync_check()
    assert np.array_equal(computed.cpu().numpy(), ref)
    assert np.array_equal(tabled.cpu().numpy(), ref)


def test_gemm_rejects_bad_arguments():
    a = dev(np.zeros((16, 64), np.int8))
    out = empty((16, 16), torch.int32)
    args = L.GemmI8Args(a=ptr(a), lda=60, w=ptr(a), ldw=64, m=16, n=16, k=64, s_acc=1.0, out_kind=L.OUT_I32,
                        out=ptr(out), ldo=16)
    assert L.lib.ls100_gemm_i8(ctx().handle, C.byref(args), None) == L.ERR_ALIGN
    args.lda = 64
    args.m = 0
    assert L.lib.ls100_gemm_i8(ctx().handle, C.byref(args), None) == L.ERR_BAD_ARG
    args.m = 16
    args.out_kind = L.OUT_OUTQ_I8  # needs s_outq > 0
    assert L.lib.ls100_gemm_i8(ctx().handle, C.byref(args), None) == L.ERR_BAD_ARG


# ----------------------------------------------------------------------------- LayerNorm, embedding
@pytest.mark.parametrize("rows,hidden", [(512, 512), (33, 64), (1000, 768), (7, 1024), (3, 2048), (2, 4096), (3000, 512), (2500, 1024)])
def test_ln_quant_bit_exact(rows, hidden):
    r = rng(rows)
    x = (r.standard_normal((rows, hidden)) * 1.7 + 0.3).astype(F32)
    g = (1 + 0.1 * r.standard_normal(hidden)).astype(F32)
    b = (0.1 * r.standard_normal(hidden)).astype(F32)
    y = om.layer_norm(x, g, b)
    amax = float(F32(4 * y.std()))
    q_ref, _ = oq.quantize(y, amax)
    oq_t, of_t = empty((rows, hidden), torch.int8), empty((rows, hidden), torch.float32)
    dx, dg, db = dev(x), dev(g), dev(b)
    args = L.LnQuantArgs(x=ptr(dx), ldx=hidden, gamma=ptr(dg), beta=ptr(db), rows=rows, hidden=hidden, amax=amax,
                         out_q=ptr(oq_t), ldq=hidden, out_f=ptr(of_t), ldf=hidden)
    L.call("ls100_ln_quant", ctx(), args)
    sync_check()
    assert np.array_equal(of_t.cpu().numpy(), y)
    assert np.array_equal(oq_t.cpu().numpy(), q_ref)


def test_embed_encoder_and_decoder_forms_bit_exact():
    V, H, pad = 500, 128, 1
    r = rng(2)
    tab = (r.standard_normal((V, H)) * 0.02).astype(F32)
    tab[pad] = 0
    amax = float(F32(4 * tab.std()))
    st = om.State(w={"emb": tab}, amax={"emb": amax})
    cfg = om.Config(hidden=H, vocab=V, pad_id=pad)
    pos = om.sinusoid_table(64, H)
    ids = r.integers(4, V, size=(5, 19)).astype(np.int32)
    for i, n in enumerate([19, 3, 11, 1, 8]):
        ids[i, n:] = pad
    ref = om.embed(st, ids, 0, cfg, pos)
    tq, s = oq.quantize(tab, amax)
    dt, dp, di = dev(tq), dev(pos), dev(ids)
    out = empty((5 * 19, H), torch.float32)
    mask = empty((5, 19), torch.uint8)
    args = L.EmbedArgs(ids=ptr(di), ld_ids=19, batch=5, seq=19, hidden=H, step_ptr=None, table_q=ptr(dt), s_emb=float(s),
                       sqrt_h=float(F32(np.sqrt(H))), pos=ptr(dp), n_pos=64, pad_id=pad, vocab=V, out=ptr(out),
                       pad_mask=ptr(mask))
    L.call("ls100_embed", ctx(), args)
    sync_check()
    assert np.array_equal(out.cpu().numpy().reshape(5, 19, H), ref)
    assert np.array_equal(mask.cpu().numpy().astype(bool), ids == pad)
    # decoder form: token of row r at column *step of a [rows, max_step] history, position = step
    hist = r.integers(4, V, size=(6, 32)).astype(np.int32)
    step = 7
    dstep = dev(np.array([step], np.int32))
    dh = dev(hist)
    out = empty((6, H), torch.float32)
    args = L.EmbedArgs(ids=ptr(dh), ld_ids=32, batch=6, seq=1, hidden=H, step_ptr=ptr(dstep), table_q=ptr(dt),
                       s_emb=float(s), sqrt_h=float(F32(np.sqrt(H))), pos=ptr(dp), n_pos=64, pad_id=pad, vocab=V,
                       out=ptr(out), pad_mask=None)
    L.call("ls100_embed", ctx(), args)
    sync_check()
    ref = om.embed(st, hist[:, step:step + 1], step, cfg, pos)[:, 0]
    assert np.array_equal(out.cpu().numpy(), ref)
    # the same lookup inside the LayerNorm launch (head of a decode step): residual stream, fp32 and int8 LN outputs
    hist[2, step] = pad  # a finished row: no position added
    dh = dev(hist)
    ref = om.embed(st, hist[:, step:step + 1], step, cfg, pos)[:, 0]
    g = (1 + 0.1 * r.standard_normal(H)).astype(F32)
    b = (0.1 * r.standard_normal(H)).astype(F32)
    y = om.layer_norm(ref, g, b)
    amax_y = float(F32(4 * y.std()))
    x_out, of_t, oq_t = empty((6, H), torch.float32), empty((6, H), torch.float32), empty((6, H), torch.int8)
    dg, db = dev(g), dev(b)
    args.ids, args.out = ptr(dh), ptr(x_out)
    ln = L.LnQuantArgs(x=None, ldx=H, gamma=ptr(dg), beta=ptr(db), rows=6, hidden=H, amax=amax_y, out_q=ptr(oq_t), ldq=H,
                       out_f=ptr(of_t), ldf=H, emb=args)
    L.call("ls100_ln_quant", ctx(), ln)
    sync_check()
    assert np.array_equal(x_out.cpu().numpy(), ref)
    assert np.array_equal(of_t.cpu().numpy(), y)
    assert np.array_equal(oq_t.cpu().numpy(), oq.quantize(y, amax_y)[0])
    ln.rows = 5  # rows must equal the lookup's batch
    with pytest.raises(RuntimeError):
        L.call("ls100_ln_quant", ctx(), ln)


# ----------------------------------------------------------------------------- attention
def _int8_close(got, ref, max_rate):
    d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
    assert d.max() <= 1, f"int8 outputs differ by {d.max()} steps"
    rate = float((d > 0).mean())
    assert rate < max_rate, f"one-step mismatch rate {rate}"
    return rate


@pytest.mark.parametrize("B,S,heads,causal,with_bias", [(3, 60, 8, 0, 1), (2, 150, 4, 0, 1), (2, 100, 4, 1, 0),
                                                       (1, 1, 2, 0, 1), (4, 64, 2, 0, 1), (2, 512, 12, 0, 1), (2, 300, 4, 1, 1),
                                                       (3, 130, 6, 0, 0), (2, 90, 3, 0, 1), (5, 17, 2, 1, 1)])
def test_attn_self_matches_oracle(B, S, heads, causal, with_bias):
    H = heads * 64
    r = rng(B * S)
    qkv_q = r.integers(-127, 128, size=(B, S, 3 * H), dtype=np.int8)
    s_qkv = F32(0.021)
    bias = (r.standard_normal(3 * H) * 0.2).astype(F32) if with_bias else None
    lens = r.integers(max(1, S // 3), S + 1, size=B)
    pad = np.arange(S)[None, :] >= lens[:, None]
    qkv = qkv_q.astype(F32) * s_qkv
    if bias is not None:
        qkv = qkv + bias
    a = om.attention_core(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads, pad, 64 ** -0.5, bool(causal))
    amax = float(F32(4 * a.std()))
    ref, _ = oq.quantize(a, amax)
    dq, dpad = dev(qkv_q.reshape(B * S, 3 * H)), dev(pad.astype(np.uint8))
    db = dev(bias) if bias is not None else None
    out = empty((B * S, H), torch.int8)
    args = L.AttnSelfArgs(qkv=ptr(dq), ld_qkv=3 * H, s_qkv=float(s_qkv), bias=ptr(db), pad_mask=ptr(dpad), batch=B,
                          seq=S, heads=heads, causal=causal, amax_out=amax, out=ptr(out), ld_out=H, k_cache=None,
                          v_cache=None, max_step=0)
    L.call("ls100_attn_self", ctx(), args)
    sync_check()
    got = out.cpu().numpy().reshape(B, S, H)
    valid = ~pad
    rate = _int8_close(got[valid], ref[valid], 5e-3)
    print(f"attn_self B={B} S={S} heads={heads} causal={causal}: one-step mismatch rate {rate:.2e}")


@pytest.mark.parametrize("B,S,heads,ms", [(3, 40, 4, 64), (2, 200, 2, 256), (2, 9, 2, 16), (2, 50, 3, 64)])
def test_attn_self_causal_prompt_fills_the_kv_cache(B, S, heads, ms):
    """GPT prompt form: causal, no bias, and the int8 keys / values of every position stored into the cache
    [batch, heads, max_step, 64] (tensor-core kernel for even head counts and S >= 16, SIMT otherwise)."""
    H = heads * 64
    r = rng(S + heads)
    qkv_q = r.integers(-127, 128, size=(B, S, 3 * H), dtype=np.int8)
    s_qkv = F32(0.017)
    qkv = qkv_q.astype(F32) * s_qkv
    a = om.attention_core(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads, None, 64 ** -0.5, True)
    amax = float(F32(4 * a.std()))
    ref, _ = oq.quantize(a, amax)
    dq = dev(qkv_q.reshape(B * S, 3 * H))
    out = empty((B * S, H), torch.int8)
    kc, vc = empty((B, heads, ms, 64), torch.int8), empty((B, heads, ms, 64), torch.int8)
    kc.fill_(77)
    vc.fill_(77)
    args = L.AttnSelfArgs(qkv=ptr(dq), ld_qkv=3 * H, s_qkv=float(s_qkv), bias=None, pad_mask=None, batch=B, seq=S, heads=heads,
                          causal=1, amax_out=amax, out=ptr(out), ld_out=H, k_cache=ptr(kc), v_cache=ptr(vc), max_step=ms)
    L.call("ls100_attn_self", ctx(), args)
    sync_check()
    _int8_close(out.cpu().numpy().reshape(B, S, H), ref, 5e-3)
    k_ref = qkv_q[..., H:2 * H].reshape(B, S, heads, 64).transpose(0, 2, 1, 3)
    v_ref = qkv_q[..., 2 * H:].reshape(B, S, heads, 64).transpose(0, 2, 1, 3)
    assert np.array_equal(kc.cpu().numpy()[:, :, :S], k_ref) and np.array_equal(vc.cpu().numpy()[:, :, :S], v_ref)
    assert (kc.cpu().numpy()[:, :, S:] == 77).all() and (vc.cpu().numpy()[:, :, S:] == 77).all()  # nothing past the prompt


@pytest.mark.parametrize("history_static,ms,n_steps", [(0, 16, 5), (1, 16, 5), (1, 48, 40)])
def test_attn_dec_int8_cache_with_beam_ancestry(history_static, ms, n_steps):
    """Decode steps with a random beam reshuffle after each; the oracle permutes its cache physically, the kernel only
    follows the ancestry table. history_static: the step counter, the ancestry table and the cache history are read
    ahead of the grid dependency (every launch here follows a synchronisation, so they are static); 40 steps take the
    history past the 32 positions that are copied early."""
    B, K, heads = 3, 4, 4
    H, T = heads * 64, 3 * 4
    r = rng(17)
    s_kv = F32(0.03)
    kc, vc = empty((T, heads, ms, 64), torch.int8), empty((T, heads, ms, 64), torch.int8)
    kc.zero_()
    vc.zero_()
    anc = np.zeros((T, ms), np.int32)
    danc = dev(anc)
    dstep = dev(np.zeros(1, np.int32))
    ok_k = np.zeros((T, 0, H), np.int8)
    ok_v = np.zeros((T, 0, H), np.int8)
    worst = 0.0
    for step in range(n_steps):
        qkv = r.integers(-127, 128, size=(T, 3 * H), dtype=np.int8)
        ok_k = np.concatenate([ok_k, qkv[:, None, H:2 * H]], 1)
        ok_v = np.concatenate([ok_v, qkv[:, None, 2 * H:]], 1)
        q = qkv[:, :H].astype(F32) * s_kv
        a = om.attention_core(q[:, None], ok_k.astype(F32) * s_kv, ok_v.astype(F32) * s_kv, heads, None, 64 ** -0.5)[:, 0]
        amax = float(F32(4 * a.std()))
        ref, _ = oq.quantize(a, amax)
        dq = dev(qkv)
        dstep.copy_(torch.tensor([step], dtype=torch.int32))
        danc.copy_(torch.from_numpy(anc))
        out = empty((T, H), torch.int8)
        args = L.AttnDecArgs(qkv=ptr(dq), ld_qkv=3 * H, s_kv=float(s_kv), k_cache=ptr(kc), v_cache=ptr(vc), anc=ptr(danc),
                             step_ptr=ptr(dstep), rows=T, heads=heads, max_step=ms, amax_out=amax, out=ptr(out), ld_out=H,
                             history_static=history_static)
        L.call("ls100_attn_dec", ctx(), args)
        sync_check()
        worst = max(worst, _int8_close(out.cpu().numpy(), ref, 5e-3))
        # beam reshuffle: new beam j of batch b continues old beam parent[b, j]
        parent = r.integers(0, K, size=(B, K))
        flat = (parent + np.arange(B)[:, None] * K).reshape(-1)
        ok_k, ok_v = ok_k[flat], ok_v[flat]
        new_anc = anc.copy()
        for t in range(T):
            new_anc[t, :step] = anc[flat[t], :step]
            new_anc[t, step] = flat[t]
        anc = new_anc
    print("attn_dec worst one-step rate", worst)


@pytest.mark.parametrize("B,K,S,heads,kv_static,head_major",
                         [(5, 4, 37, 8, 0, 0), (5, 4, 37, 8, 1, 1), (3, 2, 150, 4, 1, 0), (70, 4, 64, 8, 1, 1),
                          (2, 1, 1, 2, 0, 1), (9, 8, 65, 16, 1, 1), (3, 2, 150, 4, 0, 1)])
def test_attn_cross_matches_oracle(B, K, S, heads, kv_static, head_major):
    """One and several 64-key tiles per (sentence, head), more pairs than resident CTAs (70 x 8 > 3 x SMs), the
    keys fetched before and after the grid dependency, 1 to 8 beams."""
    H = heads * 64
    r = rng(23)
    q_q = r.integers(-127, 128, size=(B * K, H), dtype=np.int8)
    s_q = F32(0.017)
    bias = (r.standard_normal(H) * 0.1).astype(F32)
    k = (r.standard_normal((B, S, H)) * 0.5).astype(F32)
    v = (r.standard_normal((B, S, H)) * 0.5).astype(F32)
    lens = r.integers(1, S + 1, size=B)
    pad = np.arange(S)[None, :] >= lens[:, None]
    q = q_q.astype(F32) * s_q + bias
    a = om.attention_core(q[:, None], np.repeat(k.astype(F32), K, 0), np.repeat(v.astype(F32), K, 0), heads,
                          np.repeat(pad, K, 0), 64 ** -0.5)[:, 0]
    amax = float(F32(4 * a.std()))
    ref, _ = oq.quantize(a, amax)
    if head_major:  # [batch, heads, src_len, 64]
        kd = np.ascontiguousarray(k.reshape(B, S, heads, 64).transpose(0, 2, 1, 3))
        vd = np.ascontiguousarray(v.reshape(B, S, heads, 64).transpose(0, 2, 1, 3))
    else:
        kd, vd = k.reshape(B * S, H), v.reshape(B * S, H)
    dq, db, dk, dv, dp = dev(q_q), dev(bias), dev(kd), dev(vd), dev(pad.astype(np.uint8))
    out = empty((B * K, H), torch.int8)
    args = L.AttnCrossArgs(q=ptr(dq), ld_q=H, s_q=float(s_q), bias=ptr(db), k=ptr(dk), v=ptr(dv), ld_kv=H,
                           pad_mask=ptr(dp), batch=B, beam=K, src_len=S, heads=heads, amax_out=amax, out=ptr(out), ld_out=H,
                           kv_static=kv_static, kv_head_major=head_major)
    L.call("ls100_attn_cross", ctx(), args)
    sync_check()
    _int8_close(out.cpu().numpy(), ref, 5e-3)


def test_proj_f32_weight_only_quant():
    m, n, k = 333, 192, 512
    r = rng(31)
    x = r.standard_normal((m, k)).astype(F32)
    w = (r.standard_normal((n, k)) * 0.02).astype(F32)
    b = (r.standard_normal(n) * 0.1).astype(F32)
    st = om.State(w={"l.w": w, "l.b": b}, amax={"l.w": float(F32(4 * w.std()))})
    ref = om.qlinear(st, x, "l", quant_in=False, quant_out=False)
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    dx, dw, db = dev(x), dev(wq), dev(b)
    out = empty((m, n), torch.float32)
    args = L.ProjF32Args(x=ptr(dx), ldx=k, w=ptr(dw), ldw=k, s_w=float(s_w), bias=ptr(db), m=m, n=n, k=k, out=ptr(out), ldo=n)
    L.call("ls100_proj_f32", ctx(), args)
    sync_check()
    d = np.abs(out.cpu().numpy() - ref)
    # fp32 accumulation in a different order than the oracle's float64 sum
    assert d.max() <= np.abs(ref).max() * 1e-5
    # head-split output [batch, heads, seq, 64]: the same numbers, rearranged
    out2 = empty((9, n // 64, 37, 64), torch.float32)
    args = L.ProjF32Args(x=ptr(dx), ldx=k, w=ptr(dw), ldw=k, s_w=float(s_w), bias=ptr(db), m=m, n=n, k=k, out=ptr(out2), ldo=0,
                         split_seq=37)
    L.call("ls100_proj_f32", ctx(), args)
    sync_check()
    want = out.cpu().numpy().reshape(9, 37, n // 64, 64).transpose(0, 2, 1, 3)
    assert np.array_equal(out2.cpu().numpy(), want)


@pytest.mark.parametrize("m,n,k,seq", [(333, 192, 512, 0), (7680, 512, 512, 60), (300, 1024, 1024, 0), (50, 64, 64, 25),
                                        (1000, 200, 128, 0)])
def test_proj_tc_matches_oracle_and_simt(m, n, k, seq):
    """The K/V projection on the tensor cores (fp32 activations as three bf16 terms x the int8 weight as bf16): within
    1e-5 of the output range of the float64 oracle, like the SIMT kernel, and within the same bound of that kernel;
    row-major and head-split stores, ragged M and N, several tiles per CTA."""
    r = rng(m + n + k)
    x = (r.standard_normal((m, k)) * np.exp(r.standard_normal((m, 1)))).astype(F32)  # rows of different magnitude
    w = (r.standard_normal((n, k)) * 0.02).astype(F32)
    b = (r.standard_normal(n) * 0.1).astype(F32)
    st = om.State(w={"l.w": w, "l.b": b}, amax={"l.w": float(F32(4 * w.std()))})
    ref = om.qlinear(st, x, "l", quant_in=False, quant_out=False)
    wq, s_w = oq.quantize(w, st.amax["l.w"])
    dx, dw, db = dev(x), dev(wq), dev(b)
    x3 = empty((m, 3 * k), torch.bfloat16)
    wb = empty((n, k), torch.bfloat16)
    L.check(L.lib.ls100_split_bf16x3(ctx().handle, ptr(dx), k, m, k, ptr(x3), None), "split")
    L.check(L.lib.ls100_i8_to_bf16(ctx().handle, ptr(dw), k, n, k, ptr(wb), None), "i8->bf16")
    sync_check()
    assert np.array_equal(wb.float().cpu().numpy(), wq.astype(F32))
    parts = x3.float().cpu().numpy().reshape(m, 3, k).astype(np.float64)
    assert np.abs(parts.sum(1) - x.astype(np.float64)).max() <= np.abs(x).max() * 2.0 ** -26
    shape = (m // seq, n // 64, seq, 64) if seq else (m, n)
    out = empty(shape, torch.float32)
    args = L.ProjTcArgs(x3=ptr(x3), w_bf16=ptr(wb), s_w=float(s_w), bias=ptr(db), m=m, n=n, k=k, out=ptr(out), ldo=n,
                        split_seq=seq)
    L.call("ls100_proj_tc", ctx(), args)
    out2 = empty(shape, torch.float32)
    a2 = L.ProjF32Args(x=ptr(dx), ldx=k, w=ptr(dw), ldw=k, s_w=float(s_w), bias=ptr(db), m=m, n=n, k=k, out=ptr(out2), ldo=n,
                       split_seq=seq)
    L.call("ls100_proj_f32", ctx(), a2)
    sync_check()
    got, simt = out.cpu().numpy(), out2.cpu().numpy()
    if seq:
        got = got.transpose(0, 2, 1, 3).reshape(m, n)
        simt = simt.transpose(0, 2, 1, 3).reshape(m, n)
    tol = np.abs(ref).max() * 1e-5
    print("tensor-core vs oracle", np.abs(got - ref).max(), "SIMT vs oracle", np.abs(simt - ref).max(), "tol", tol)
    assert np.abs(got - ref).max() <= tol
    assert np.abs(got - simt).max() <= tol


# ----------------------------------------------------------------------------- beam search
@pytest.mark.parametrize("V,ties", [(32000, False), (1000, True), (37, True), (40000, False)])
def test_beam_step_matches_oracle(V, ties):
    """Several steps of topk+update vs oracle.beam.beam_step, incl. EOS finishing, heavy logit ties and
    the in-place history / ancestry rewrite."""
    B, K, ms, end_id = 6, 4, 24, 2
    r = rng(V)
    ldv = (V + 15) // 16 * 16
    s_l = F32(0.08)
    alive = np.full((B, K, ms), end_id, np.int32)
    probs = np.full((B, K), -1000.0, F32)
    probs[:, 0] = 0
    score = np.zeros((B, K), F32)
    anc = np.zeros((B * K, ms), np.int32)
    ln_tab = np.array([ob.length_norm(i + 1, 0.6) for i in range(ms)], F32)
    d_alive, d_probs, d_score, d_anc = dev(alive), dev(probs), dev(score), dev(anc)
    d_ln = dev(ln_tab)
    d_step = dev(np.zeros(1, np.int32))
    d_fin, d_ticket = dev(np.zeros(ms, np.int32)), dev(np.zeros(ms, np.int32))
    d_stop = dev(np.full(1, -1, np.int32))
    cs, ct = empty((B * K, K), torch.float32), empty((B * K, K), torch.int32)
    for step in range(8):
        if ties:
            lq = r.integers(-3, 4, size=(B, K, V)).astype(np.int8)
        else:
            lq = np.clip(np.rint(r.standard_normal((B, K, V)) * 32), -127, 127).astype(np.int8)
        if step >= 2:  # push EOS so that beams finish
            lq[:, :, end_id] = 127 if ties else 120
        pad = np.full((B * K, ldv), 55, np.int8)
        pad[:, :V] = lq.reshape(B * K, V)
        d_l = dev(pad)
        a1 = L.BeamTopkArgs(logits=ptr(d_l), ld_logits=ldv, s_logits=float(s_l), batch=B, beam=K, vocab=V, max_step=ms,
                            end_id=end_id, step_ptr=ptr(d_step), length_norm=ptr(d_ln), alive=ptr(d_alive),
                            seq_probs=ptr(d_probs), seq_score=ptr(d_score), cand_score=ptr(cs), cand_token=ptr(ct))
        L.call("ls100_beam_topk", ctx(), a1)
        a2 = L.BeamUpdateArgs(cand_score=ptr(cs), cand_token=ptr(ct), batch=B, beam=K, max_step=ms, end_id=end_id,
                              step_ptr=ptr(d_step), length_norm=ptr(d_ln), alive=ptr(d_alive), anc=ptr(d_anc),
                              seq_probs=ptr(d_probs), seq_score=ptr(d_score), fin_count=ptr(d_fin), ticket=ptr(d_ticket),
                              stop_step=ptr(d_stop), stop_host=None)
        L.call("ls100_beam_update", ctx(), a2)
        sync_check()
        alive, probs, score, parent, n_fin = ob.beam_step(lq, s_l, alive, probs, score, step, ln_tab[step], end_id)
        flat = (parent + np.arange(B)[:, None] * K).reshape(-1)
        new_anc = anc.copy()
        for t in range(B * K):
            new_anc[t, :step] = anc[flat[t], :step]
            new_anc[t, step] = flat[t]
        anc = new_anc
        assert int(d_step.cpu()[0]) == step + 1
        g_alive, g_score, g_probs = d_alive.cpu().numpy(), d_score.cpu().numpy(), d_probs.cpu().numpy()
        g_anc = d_anc.cpu().numpy()
        # Beams must be the same set per sentence; their ORDER may differ from the oracle's only between
        # beams whose oracle scores are within a few ulps of each other (float near-ties: the device sums
        # exp() in a different order than the oracle's histogram form).
        for b in range(B):
            perm = []
            for j in range(K):
                match = [k for k in range(K) if k not in perm and np.array_equal(g_alive[b, j], alive[b, k])
                         and abs(float(g_score[b, j]) - float(score[b, k])) <= 2e-5 + 2e-6 * abs(float(score[b, k]))]
                assert match, f"step {step} sentence {b}: device beam {j} is not among the oracle's beams"
                perm.append(match[0])
            for j, k in enumerate(perm):
                if j != k:
                    assert abs(float(score[b, j]) - float(score[b, k])) <= 4e-6 * abs(float(score[b, j])) + 1e-6, \
                        f"step {step} sentence {b}: beams reordered without a score near-tie"
            perm = np.array(perm)
            alive[b], probs[b], score[b] = alive[b, perm], probs[b, perm], score[b, perm]
            rows = b * K + perm
            anc[b * K:(b + 1) * K] = anc[rows]
        assert np.array_equal(g_alive, alive), f"step {step}: token histories differ"
        assert np.array_equal(g_anc[:, :step + 1], anc[:, :step + 1])
        np.testing.assert_allclose(g_score, score, rtol=2e-6, atol=2e-5)
        live = alive[:, :, step + 1] != end_id
        np.testing.assert_allclose(g_probs[live], probs[live], rtol=2e-6, atol=2e-5)
        # continue from the device's values so that rounding differences do not accumulate into new near-ties
        probs[live] = g_probs[live]
        score = g_score.copy()
        assert int(d_fin.cpu()[step]) == n_fin
        if n_fin == B * K:
            assert int(d_stop.cpu()[0]) >= 0
            break
    assert int(d_stop.cpu()[0]) == step if n_fin == B * K else int(d_stop.cpu()[0]) == -1


# ----------------------------------------------------------------------------- top-k sampling
@pytest.mark.parametrize("V,k", [(50257, 8), (1000, 4), (50, 1)])
def test_sample_topk_matches_oracle(V, k):
    """Several sampling steps: tokens equal the oracle's (same Philox counter stream), ended rows keep emitting
    EOS, the position advances on the device and the all-ended position is recorded."""
    rows, ms, end_id = 10, 16, 3
    r = rng(V + k)
    ldv = (V + 15) // 16 * 16
    s_l = F32(0.06)
    seq = np.full((rows, ms), end_id, np.int32)
    seq[:, :2] = r.integers(4, V, size=(rows, 2))
    d_seq = dev(seq)
    d_cur = dev(np.array([1], np.int32))
    d_ticket, d_ended, d_stop = dev(np.zeros(1, np.int32)), dev(np.zeros(1, np.int32)), dev(np.full(1, -1, np.int32))
    seed_lo, seed_hi = 2024, 7
    stop_ref = -1
    for step in range(6):
        cur = 1 + step
        lq = np.clip(np.rint(r.standard_normal((rows, ldv)) * 30), -127, 127).astype(np.int8)
        if step >= 2:
            lq[step % rows::3, end_id] = 127  # make some rows end
        if step == 5:
            lq[:, :] = -100
            lq[:, end_id] = 127          # everything ends
        d_l = dev(lq)
        a = L.SampleTopkArgs(logits=ptr(d_l), ld_logits=ldv, s_logits=float(s_l), rows=rows, vocab=V, k=k, max_step=ms,
                             end_id=end_id, seed_lo=seed_lo, seed_hi=seed_hi, seq=ptr(d_seq), cur=ptr(d_cur),
                             ticket=ptr(d_ticket), n_ended=ptr(d_ended), stop=ptr(d_stop), stop_host=None)
        L.call("ls100_sample_topk", ctx(), a)
        sync_check()
        for row in range(rows):
            if seq[row, cur] == end_id:
                seq[row, cur + 1] = end_id
            else:
                seq[row, cur + 1] = ob.sample_topk_row(lq[row, :V], s_l, k, cur + 1, row, seed_lo, seed_hi)
        if stop_ref < 0 and (seq[:, cur + 1] == end_id).all():
            stop_ref = cur + 1
        assert int(d_cur.cpu()[0]) == cur + 1
        assert np.array_equal(d_seq.cpu().numpy(), seq), f"step {step}: sampled tokens differ"
        assert int(d_stop.cpu()[0]) == stop_ref
    assert stop_ref > 0


@pytest.mark.parametrize("V,p,spread", [(50257, 0.9, 30), (1000, 0.5, 8), (37, 0.3, 2), (32000, 1.0, 30), (5000, 0.02, 40)])
def test_sample_topp_matches_oracle(V, p, spread):
    """Nucleus sampling over several steps: tokens equal the oracle's exact nucleus draw (same Philox counters),
    from nearly flat rows (nucleus = most of the vocabulary) to peaked ones (nucleus inside the top level);
    ended rows keep emitting EOS and the all-ended position is recorded."""
    rows, ms, end_id = 9, 16, 3
    r = rng(V + spread)
    ldv = (V + 15) // 16 * 16
    s_l = F32(0.06)
    seq = np.full((rows, ms), end_id, np.int32)
    seq[:, :2] = r.integers(4, V, size=(rows, 2))
    d_seq = dev(seq)
    d_cur = dev(np.array([1], np.int32))
    d_ticket, d_ended, d_stop = dev(np.zeros(1, np.int32)), dev(np.zeros(1, np.int32)), dev(np.full(1, -1, np.int32))
    seed_lo, seed_hi = 99, 5
    stop_ref = -1
    for step in range(5):
        cur = 1 + step
        lq = np.clip(np.rint(r.standard_normal((rows, ldv)) * spread), -127, 127).astype(np.int8)
        if step >= 2:
            lq[step % rows::3, :] = -127
            lq[step % rows::3, end_id] = 127  # these rows end
        if step == 4:
            lq[:, :] = -127
            lq[:, end_id] = 127
        d_l = dev(lq)
        a = L.SampleToppArgs(logits=ptr(d_l), ld_logits=ldv, s_logits=float(s_l), p=p, rows=rows, vocab=V, max_step=ms,
                             end_id=end_id, seed_lo=seed_lo, seed_hi=seed_hi, seq=ptr(d_seq), cur=ptr(d_cur),
                             ticket=ptr(d_ticket), n_ended=ptr(d_ended), stop=ptr(d_stop), stop_host=None)
        L.call("ls100_sample_topp", ctx(), a)
        sync_check()
        for row in range(rows):
            if seq[row, cur] == end_id:
                seq[row, cur + 1] = end_id
            else:
                seq[row, cur + 1] = ob.sample_topp_row(lq[row, :V], s_l, p, cur + 1, row, seed_lo, seed_hi)
        if stop_ref < 0 and (seq[:, cur + 1] == end_id).all():
            stop_ref = cur + 1
        assert int(d_cur.cpu()[0]) == cur + 1
        assert np.array_equal(d_seq.cpu().numpy(), seq), f"step {step}: sampled tokens differ"
        assert int(d_stop.cpu()[0]) == stop_ref
    assert stop_ref > 0


def test_bounded_wait_runs_out_and_reports_once():
    """A wait that nothing satisfies gives up after its budget: the kernel returns normally, the context's error word
    holds LS100_ERR_TIMEOUT exactly once, and the context keeps working (the next GEMM is bit-exact)."""
    c = ctx()
    assert c.poll_error() == 0
    assert L.lib.ls100_debug_expire_wait(c.handle, None) == 0
    assert c.poll_error() == L.ERR_TIMEOUT
    assert c.poll_error() == 0  # reading clears it
    r = np.random.default_rng(1)
    a = r.integers(-127, 128, size=(128, 256), dtype=np.int8)
    w = r.integers(-127, 128, size=(64, 256), dtype=np.int8)
    out = gemm(dev(a), dev(w), s_acc=1.0, out_kind=L.OUT_I32)
    sync_check()
    assert np.array_equal(out.cpu().numpy().astype(np.int64), oq.int_matmul(a, w))


@pytest.mark.parametrize("B,K,V,Kd,levels", [(3, 4, 37, 64, 40.0), (5, 4, 1000, 128, 40.0), (128, 4, 32000, 512, 40.0),
                                             (9, 8, 40003, 256, 40.0), (33, 2, 32000, 128, 1.5), (4, 1, 5000, 64, 40.0)])
def test_logits_statistics_and_beam_select_match_beam_topk(B, K, V, Kd, levels):
    """The logits GEMM keeps, per row and 64-column group, the largest int8 value and the sum of exponentials;
    ls100_beam_select picks the beam candidates from those statistics and the few groups that matter. The tokens
    must be exactly those of ls100_beam_topk on the same logits, the scores equal to float rounding. `levels` = the
    spread of the int8 logits: 1.5 leaves about seven distinct values, so that hundreds of groups tie for the maximum
    (the path that reads every group) and the token tie-break decides."""
    rows, ms, end_id = B * K, 16, 2
    r = rng(41 + V)
    a = r.integers(-127, 128, size=(rows, Kd), dtype=np.int8)
    w = r.integers(-127, 128, size=(V, Kd), dtype=np.int8)
    acc_std = 127 * 127 / 3.0 * np.sqrt(Kd)
    s_out = F32(0.05)
    s_acc = F32(float(s_out) * levels / acc_std)  # int8 logits ~ N(0, levels^2), clipped at +-127
    ldv = (V + 15) // 16 * 16
    G = (V + 63) // 64
    nrb = (rows + 127) // 128
    da, dw = dev(a), dev(w)
    logits = torch.zeros((rows, ldv), dtype=torch.int8, device="cuda:0")
    st_max = torch.full((nrb, G, 128), -99, dtype=torch.int8, device="cuda:0")
    st_sum = torch.zeros((nrb, G, 128), dtype=torch.float32, device="cuda:0")
    g = L.GemmI8Args(a=ptr(da), lda=Kd, w=ptr(dw), ldw=Kd, m=rows, n=V, k=Kd, s_acc=float(s_acc), s_outq=float(s_out),
                     out_kind=L.OUT_OUTQ_I8, out=ptr(logits), ldo=ldv, stat_max=ptr(st_max), stat_sum=ptr(st_sum))
    L.call("ls100_gemm_i8", ctx(), g)
    sync_check()
    lq = logits.cpu().numpy()[:, :V]
    # the statistics are what numpy computes from the int8 matrix
    pad = np.full((rows, G * 64), -128, np.int32)
    pad[:, :V] = lq
    want_max = pad.reshape(rows, G, 64).max(2)
    e = np.exp((pad.astype(np.float64) - 127.0) * float(s_out))
    e[:, V:] = 0
    want_sum = e.reshape(rows, G, 64).sum(2)
    got_max = st_max.cpu().numpy().transpose(0, 2, 1).reshape(nrb * 128, G)[:rows]
    got_sum = st_sum.cpu().numpy().transpose(0, 2, 1).reshape(nrb * 128, G)[:rows]
    assert np.array_equal(got_max, want_max)
    np.testing.assert_allclose(got_sum, want_sum, rtol=1e-5)
    # candidates: both kernels from the same state, step 1 with one finished beam
    alive = np.full((B, K, ms), end_id, np.int32)
    alive[:, :, 0] = 3
    alive[:, :, 1] = 7
    if K > 1:
        alive[0, 1, 1] = end_id
    probs = (-r.random((B, K)) * 3).astype(F32)
    score = (-r.random((B, K)) * 3).astype(F32)
    d_alive, d_probs, d_score = dev(alive), dev(probs), dev(score)
    step = dev(np.ones(1, np.int32))
    ln = dev(np.array([ob.length_norm(i + 1, 0.6) for i in range(ms)], F32))
    outs = []
    for fused in (False, True):
        cs, ct = empty((rows, K), torch.float32), empty((rows, K), torch.int32)
        t = L.BeamTopkArgs(logits=ptr(logits), ld_logits=ldv, s_logits=float(s_out), batch=B, beam=K, vocab=V, max_step=ms,
                           end_id=end_id, step_ptr=ptr(step), length_norm=ptr(ln), alive=ptr(d_alive), seq_probs=ptr(d_probs),
                           seq_score=ptr(d_score), cand_score=ptr(cs), cand_token=ptr(ct), diverse_lambda=0.25)
        if fused:
            L.call("ls100_beam_select", ctx(), L.BeamSelectArgs(topk=t, stat_max=ptr(st_max), stat_sum=ptr(st_sum), n_groups=G))
        else:
            L.call("ls100_beam_topk", ctx(), t)
        sync_check()
        outs.append((cs.cpu().numpy(), ct.cpu().numpy()))
    assert np.array_equal(outs[0][1], outs[1][1]), "candidate tokens differ"
    np.testing.assert_allclose(outs[1][0], outs[0][0], rtol=2e-6, atol=2e-6)
    print("distinct logit values", len(np.unique(lq)), "rows", rows, "groups", G)
