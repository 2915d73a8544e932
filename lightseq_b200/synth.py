"""Seeded synthetic int8 models for benchmarking and testing.

There are no pretrained checkpoints or datasets in the build environment, so the
benchmark configurations are stated as *shapes plus distributions*: weights
N(0, 0.02^2), biases 0, LayerNorm gamma 1 / beta 0, sinusoidal positions, and every
clip-max = 4 x std of the tensor it clips. The std of a weight comes from the weight
itself; the std of an activation is measured here by one un-quantised fp32
calibration pass over (a sample of) the seeded inputs — the role the reference gives
to its calibrators (lightseq/training/pytorch_quantization/calib/). That pass is plain
fp32 numpy and cannot produce the quantised model's outputs.

Tensor names (shared with the engine's loader):
  emb [V,H];  enc.{l}.{qkv,out,fc1,fc2}.{w,b};  enc.{l}.ln{1,2}.{g,b};  enc.ln.{g,b}
  dec.{l}.{qkv,out,xq,xk,xv,xout,fc1,fc2}.{w,b};  dec.{l}.ln{1,2,3}.{g,b};  dec.ln.{g,b}
Clip-max names: ``<linear>.in`` / ``<linear>.w`` / ``<linear>.out``, ``dec.{l}.kv`` (int8
self-attention cache), ``emb``, ``logits.in`` / ``logits.out``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np

F32 = np.float32


class _Stats:
    def __init__(self):
        self.s: Dict[str, list] = {}

    def see(self, name: str, x: np.ndarray):
        x = np.asarray(x, dtype=np.float64)
        a = self.s.setdefault(name, [0.0, 0.0, 0])
        a[0] += float(x.sum())
        a[1] += float((x * x).sum())
        a[2] += x.size

    def amax(self, k: float = 4.0) -> Dict[str, float]:
        out = {}
        for name, (s, q, n) in self.s.items():
            m = s / n
            out[name] = float(F32(k * math.sqrt(max(q / n - m * m, 1e-12))))
        return out


def sinusoid_table(n: int, dim: int) -> np.ndarray:
    """Sinusoidal positions as SinusoidalPositionalEmbedding.get_embedding
    (lightseq/training/ops/pytorch/torch_transformer_layers.py:1086-1106)."""
    half = dim // 2
    e = F32(math.log(10000) / (half - 1))
    freq = np.exp(np.arange(half, dtype=F32) * -e).astype(F32)
    ang = (np.arange(n, dtype=F32)[:, None] * freq[None, :]).astype(F32)
    tab = np.concatenate([np.sin(ang), np.cos(ang)], axis=1).astype(F32)
    if dim % 2 == 1:
        tab = np.concatenate([tab, np.zeros((n, 1), F32)], axis=1)
    return tab


def _ln(x, g, b):
    m = x.mean(-1, keepdims=True)
    v = ((x - m) ** 2).mean(-1, keepdims=True)
    return ((x - m) / np.sqrt(v + 1e-5) * g + b).astype(F32)


def _ln_offset(x, valid):
    """Mean over the valid tokens of mean(x) / std(x): what LayerNorm subtracts from every element, in output units."""
    m = x.mean(-1)
    sd = np.sqrt(((x - m[..., None]) ** 2).mean(-1) + 1e-5)
    return float((m / sd)[valid].mean())


def _softmax(s):
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(-1, keepdims=True)


def _attn(q, k, v, heads, mask):
    """q [B,Lq,H], k,v [B,Lk,H]; mask broadcastable to [B,heads,Lq,Lk], True = masked."""
    B, Lq, H = q.shape
    Lk = k.shape[1]
    dh = H // heads
    qh = (q * F32(dh ** -0.5)).reshape(B, Lq, heads, dh).transpose(0, 2, 1, 3)
    kh = k.reshape(B, Lk, heads, dh).transpose(0, 2, 3, 1)
    vh = v.reshape(B, Lk, heads, dh).transpose(0, 2, 1, 3)
    s = np.matmul(qh, kh)
    if mask is not None:
        s = np.where(mask, F32(-1e30), s)
    return np.matmul(_softmax(s), vh).transpose(0, 2, 1, 3).reshape(B, Lq, H).astype(F32)


def _act(x, act):
    if act == "relu":
        return np.maximum(x, 0)
    from scipy.special import erf

    return (0.5 * x * (1.0 + erf(x / math.sqrt(2.0)))).astype(F32)


def transformer_weights(hidden=512, heads=8, ffn=2048, n_enc=6, n_dec=6, vocab=32000, pad_id=1, seed=1234,
                        std=0.02) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)

    def nrm(*shape):
        return (rng.standard_normal(shape, dtype=F32) * F32(std)).astype(F32)

    w: Dict[str, np.ndarray] = {}
    w["emb"] = nrm(vocab, hidden)
    w["emb"][pad_id] = 0
    H = hidden

    def lin(name, n_out, n_in):
        w[name + ".w"] = nrm(n_out, n_in)
        w[name + ".b"] = np.zeros(n_out, F32)

    def ln(name):
        w[name + ".g"] = np.ones(H, F32)
        w[name + ".b"] = np.zeros(H, F32)

    for l in range(n_enc):
        p = f"enc.{l}"
        lin(p + ".qkv", 3 * H, H)
        lin(p + ".out", H, H)
        lin(p + ".fc1", ffn, H)
        lin(p + ".fc2", H, ffn)
        ln(p + ".ln1")
        ln(p + ".ln2")
    ln("enc.ln")
    for l in range(n_dec):
        p = f"dec.{l}"
        lin(p + ".qkv", 3 * H, H)
        lin(p + ".out", H, H)
        lin(p + ".xq", H, H)
        lin(p + ".xk", H, H)
        lin(p + ".xv", H, H)
        lin(p + ".xout", H, H)
        lin(p + ".fc1", ffn, H)
        lin(p + ".fc2", H, ffn)
        ln(p + ".ln1")
        ln(p + ".ln2")
        ln(p + ".ln3")
    ln("dec.ln")
    return w


def transformer_inputs(batch=128, min_len=20, max_len=60, vocab=32000, pad_id=1, seed=4321) -> np.ndarray:
    """Source ids [B, max(len)] int32, uniform over [4, vocab), right-padded with ``pad_id``."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(min_len, max_len + 1, size=batch)
    S = int(lens.max())
    ids = np.full((batch, S), pad_id, dtype=np.int32)
    for i, n in enumerate(lens):
        ids[i, :n] = rng.integers(4, vocab, size=n)
    return ids


SAMPLING_METHODS = ("beam_search", "topk", "topp", "topk_greedy")  # the code stored in a model's configuration


def calibrate_transformer(w: Dict[str, np.ndarray], src: np.ndarray, *, heads: int, n_enc: int, n_dec: int,
                          act: str = "relu", pad_id: int = 1, seed: int = 99, k: float = 4.0,
                          ln_offsets: Optional[Dict[str, float]] = None, no_scale_embedding: bool = False,
                          pre_ln: bool = True) -> Dict[str, float]:
    """Clip-max table = k x std, from one fp32 pass: encoder on ``src``; decoder teacher-forced
    on random target ids of the source lengths (causal self-attention). ``ln_offsets``, when given, receives the
    average mean/std ratio of the inputs of the encoder's final LayerNorm and of every decoder ``ln2``."""
    st = _Stats()
    H = w["emb"].shape[1]
    V = w["emb"].shape[0]
    B, S = src.shape
    pos = sinusoid_table(max(1024, S + 64), H)
    rng = np.random.default_rng(seed)

    def lin(name, x, see_in=True, see_out=True):
        if see_in:
            st.see(name + ".in", x)
        y = x @ w[name + ".w"].T
        if see_out:
            st.see(name + ".out", y)
        return (y + w[name + ".b"]).astype(F32)

    def emb(ids):
        mask = ids != pad_id
        p = (np.cumsum(mask, 1) - 1) * mask
        scale = F32(1.0) if no_scale_embedding else F32(math.sqrt(H))
        return (scale * w["emb"][ids] + pos[p] * mask[..., None]).astype(F32)

    pad = src == pad_id
    x = emb(src)
    ln = lambda t, name: _ln(t, w[name + ".g"], w[name + ".b"])  # noqa: E731
    for l in range(n_enc):
        p = f"enc.{l}"
        qkv = lin(p + ".qkv", ln(x, p + ".ln1") if pre_ln else x)
        a = _attn(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads, pad[:, None, None, :])
        x = x + lin(p + ".out", a)
        if not pre_ln:
            x = ln(x, p + ".ln1")
        h = _act(lin(p + ".fc1", ln(x, p + ".ln2") if pre_ln else x), act)
        x = x + lin(p + ".fc2", h)
        if not pre_ln:
            x = ln(x, p + ".ln2")
    if ln_offsets is not None:
        ln_offsets["enc.ln"] = _ln_offset(x, ~pad)
    enc = _ln(x, w["enc.ln.g"], w["enc.ln.b"]) if pre_ln else x

    lens = (~pad).sum(1)
    tgt = np.full((B, S), pad_id, dtype=np.int64)
    for i, n in enumerate(lens):
        tgt[i, :n] = rng.integers(4, V, size=n)
    tpad = tgt == pad_id
    causal = ~np.tril(np.ones((S, S), dtype=bool))
    x = emb(tgt)
    for l in range(n_dec):
        p = f"dec.{l}"
        qkv = lin(p + ".qkv", ln(x, p + ".ln1") if pre_ln else x)
        st.see(p + ".kv", qkv)
        a = _attn(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads,
                  causal[None, None] | tpad[:, None, None, :])
        x = x + lin(p + ".out", a)
        if not pre_ln:
            x = ln(x, p + ".ln1")
        if ln_offsets is not None:
            ln_offsets[p + ".ln2"] = _ln_offset(x, ~tpad)
        q = lin(p + ".xq", ln(x, p + ".ln2") if pre_ln else x)
        kx = lin(p + ".xk", enc, False, False)
        vx = lin(p + ".xv", enc, False, False)
        a = _attn(q, kx, vx, heads, pad[:, None, None, :])
        x = x + lin(p + ".xout", a)
        if not pre_ln:
            x = ln(x, p + ".ln2")
        h = _act(lin(p + ".fc1", ln(x, p + ".ln3") if pre_ln else x), act)
        x = x + lin(p + ".fc2", h)
        if not pre_ln:
            x = ln(x, p + ".ln3")
    if not pre_ln:
        st.see("logits.in", x)
        st.see("logits.out", x[:, : min(S, 8)] @ w["emb"].T)
        amax = st.amax(k)
        for name, t in w.items():
            if name.endswith(".w") and t.ndim == 2:
                amax[name] = float(F32(k * t.std()))
        amax["emb"] = float(F32(k * w["emb"].std()))
        return amax
    x = _ln(x, w["dec.ln.g"], w["dec.ln.b"])
    st.see("logits.in", x)
    st.see("logits.out", x[:, : min(S, 8)] @ w["emb"].T)
    amax = st.amax(k)
    for name, t in w.items():
        if name.endswith(".w") and t.ndim == 2:
            amax[name] = float(F32(k * t.std()))
    amax["emb"] = float(F32(k * w["emb"].std()))
    return amax


def make_transformer(path: Optional[str] = None, *, hidden=512, heads=8, ffn=2048, n_enc=6, n_dec=6, vocab=32000,
                     act="relu", beam=4, length_penalty=0.6, extra_decode_length=50, max_step=256, pad_id=1,
                     start_id=3, end_id=2, seed=1234, calib_src: Optional[np.ndarray] = None,
                     sampling_method: str = "beam_search", topk: int = 1, topp: float = 0.0, output_topk: bool = False,
                     no_scale_embedding: bool = False, rng_seed: int = 0, pre_ln: bool = True, diverse_lambda: float = 0.0
                     ) -> Tuple[Dict[str, float], Dict[str, float], Dict[str, np.ndarray]]:
    """Builds (conf, amax, tensors) of a seeded synthetic QuantTransformer and optionally writes ``path``. The
    generator options are those of the reference's model configuration (sampling_method, topk, topp; every beam in
    the output; embeddings not scaled by sqrt(hidden))."""
    w = transformer_weights(hidden, heads, ffn, n_enc, n_dec, vocab, pad_id, seed)
    if calib_src is None:
        calib_src = transformer_inputs(batch=8, min_len=8, max_len=24, vocab=vocab, pad_id=pad_id, seed=seed + 1)
    amax = calibrate_transformer(w, calib_src, heads=heads, n_enc=n_enc, n_dec=n_dec, act=act, pad_id=pad_id,
                                 no_scale_embedding=no_scale_embedding, pre_ln=pre_ln)
    conf = dict(hidden=hidden, heads=heads, ffn=ffn, n_enc=n_enc, n_dec=n_dec, vocab=vocab,
                act_gelu=float(act == "gelu"), pre_ln=float(pre_ln), beam=beam, length_penalty=length_penalty,
                extra_decode_length=extra_decode_length, max_step=max_step, pad_id=pad_id, start_id=start_id,
                end_id=end_id, sampling_method=float(SAMPLING_METHODS.index(sampling_method)), topk=float(topk),
                topp=float(topp), output_topk=float(output_topk), no_scale_embedding=float(no_scale_embedding),
                rng_seed=float(rng_seed), diverse_lambda=float(diverse_lambda))
    w["pos"] = sinusoid_table(max_step, hidden)
    if path is not None:
        from . import weights

        weights.save(path, "QuantTransformer", conf, amax, w)
    return conf, amax, w


def copy_task_inputs(batch=32, min_len=20, max_len=60, vocab=32000, pad_id=1, end_id=2, seed=4321) -> np.ndarray:
    """Source ids as ``transformer_inputs`` (lengths U{min_len..max_len}, ids U[4, vocab)) whose last token is EOS,
    the way translation sources end: the copy-task model then ends its output where the source ends."""
    src = transformer_inputs(batch, min_len, max_len, vocab, pad_id, seed)
    lens = (src != pad_id).sum(1)
    src[np.arange(batch), lens - 1] = end_id
    return src


def make_copy_transformer(path: Optional[str] = None, *, hidden=512, heads=8, ffn=2048, n_enc=6, n_dec=6, vocab=32000,
                          beam=4, length_penalty=0.6, extra_decode_length=50, max_step=256, pad_id=1, start_id=3,
                          end_id=2, seed=1234, calib_src: Optional[np.ndarray] = None, sharp=5.0, gain=4.0,
                          logits_amax_sigmas=14.0):
    """A seeded Transformer with a PEAKED output distribution, for free-running parity tests.

    A randomly initialised model has an almost flat output distribution: beam search on it is chaotic, and one
    int8 rounding flip anywhere reorders near-tied candidates. Trained translation models are peaked. This builder
    keeps every weight of ``make_transformer`` (N(0, 0.02^2), same seed) except the cross-attention of the LAST
    decoder layer, which is set so that the model copies its source: query and key projections select the sine/cosine
    pairs of the 16 fastest positional frequencies for every head (q.k ~ ``sharp``^2/8 * 2 sum_i cos(w_i (t - s)), peaked at
    source position s = decode position t; the embedding table is zero in those 32 dims), the value projection is the identity and the output
    projection ``gain`` times the identity, so the residual stream going into the output projection is dominated by
    the encoder state of source token t, whose own embedding row then wins the logits by tens of int8 steps.
    Everything still runs through the int8 path (all other layers add their pseudo-random contributions, every
    quantiser is live); the logits clip-max is widened to ``logits_amax_sigmas`` standard deviations so that the
    winning logit is not clipped into a tie with the largest noise logits. Clip-max of the designed matrices is
    their largest magnitude; all others are 4 x std from the calibration pass."""
    w = transformer_weights(hidden, heads, ffn, n_enc, n_dec, vocab, pad_id, seed)
    H, dh = hidden, hidden // heads
    half = H // 2
    p = f"dec.{n_dec - 1}"
    sel = np.zeros((H, H), F32)
    n_f = dh // 2
    n_freq = n_f  # the dh/2 fastest frequencies (1 .. 0.33 rad per position for dh = 64), the same set for every head
    for h in range(heads):
        for j in range(n_f):
            sel[h * dh + j, j] = 1.0                 # sin(w_j * pos)
            sel[h * dh + n_f + j, half + j] = 1.0    # cos(w_j * pos)
    # Those 2 x n_freq dims of the residual stream are kept as a clean positional channel: the token embedding is zero
    # there and no sublayer writes to them (zero rows in every attention-output and second-FFN matrix), so a key's
    # score depends on its position only and not on pseudo-random layer output that would favour some positions.
    chan = np.concatenate([np.arange(n_freq), half + np.arange(n_freq)])
    w["emb"][:, chan] = 0
    for name in list(w):
        if name.endswith((".out.w", ".xout.w", ".fc2.w")):
            w[name][chan, :] = 0
    w[p + ".xq.w"] = (F32(sharp) * sel).astype(F32)
    w[p + ".xk.w"] = (F32(sharp) * sel).astype(F32)
    w[p + ".xv.w"] = np.eye(H, dtype=F32)
    w[p + ".xout.w"] = (F32(gain) * np.eye(H, dtype=F32)).astype(F32)
    if calib_src is None:
        calib_src = copy_task_inputs(batch=8, min_len=8, max_len=24, vocab=vocab, pad_id=pad_id, end_id=end_id, seed=seed + 1)
    # LayerNorm subtracts the row mean (about 0.4: half of the positional table is cosines of slow frequencies, close
    # to 1) from the channel as well; a constant LayerNorm bias on the channel dims puts it back, so that queries and
    # keys are the bare sines and cosines (times 1/std). First pass measures the offset, second pass the clip-max table.
    off: Dict[str, float] = {}
    calibrate_transformer(w, calib_src, heads=heads, n_enc=n_enc, n_dec=n_dec, act="relu", pad_id=pad_id, ln_offsets=off)
    w["enc.ln.b"][chan] = F32(off["enc.ln"])
    w[p + ".ln2.b"][chan] = F32(off[p + ".ln2"])
    amax = calibrate_transformer(w, calib_src, heads=heads, n_enc=n_enc, n_dec=n_dec, act="relu", pad_id=pad_id)
    for name in (".xq.w", ".xk.w", ".xv.w", ".xout.w"):
        amax[p + name] = float(np.abs(w[p + name]).max())
    amax["logits.out"] = float(F32(amax["logits.out"] / 4.0 * logits_amax_sigmas))
    conf = dict(hidden=hidden, heads=heads, ffn=ffn, n_enc=n_enc, n_dec=n_dec, vocab=vocab, act_gelu=0.0, pre_ln=1.0,
                beam=beam, length_penalty=length_penalty, extra_decode_length=extra_decode_length, max_step=max_step,
                pad_id=pad_id, start_id=start_id, end_id=end_id)
    w["pos"] = sinusoid_table(max_step, hidden)
    if path is not None:
        from . import weights

        weights.save(path, "QuantTransformer", conf, amax, w)
    return conf, amax, w


# ------------------------------------------------------------------------------------------- BERT
def bert_weights(hidden=768, heads=12, ffn=3072, n_layer=12, vocab=30522, max_pos=512, seed=1234, std=0.02):
    rng = np.random.default_rng(seed)

    def nrm(*shape):
        return (rng.standard_normal(shape, dtype=F32) * F32(std)).astype(F32)

    w: Dict[str, np.ndarray] = {"emb": nrm(vocab, hidden), "type_emb": nrm(2, hidden), "pos": nrm(max_pos, hidden),
                                "emb.ln.g": np.ones(hidden, F32), "emb.ln.b": np.zeros(hidden, F32)}
    for l in range(n_layer):
        p = f"enc.{l}"
        for name, (no, ni) in (("qkv", (3 * hidden, hidden)), ("out", (hidden, hidden)), ("fc1", (ffn, hidden)),
                               ("fc2", (hidden, ffn))):
            w[f"{p}.{name}.w"] = nrm(no, ni)
            w[f"{p}.{name}.b"] = np.zeros(no, F32)
        for ln in ("ln1", "ln2"):
            w[f"{p}.{ln}.g"] = np.ones(hidden, F32)
            w[f"{p}.{ln}.b"] = np.zeros(hidden, F32)
    return w


def bert_inputs(batch=128, seq=128, vocab=30522, pad_id=0, seed=4321) -> np.ndarray:
    """ids [batch, seq]: valid lengths U{seq/4..seq}, ids U[1000, vocab), right-padded with ``pad_id``."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(max(seq // 4, 1), seq + 1, size=batch)
    ids = np.full((batch, seq), pad_id, dtype=np.int32)
    for i, n in enumerate(lens):
        ids[i, :n] = rng.integers(min(1000, vocab - 1), vocab, size=n)
    return ids


def calibrate_bert(w, ids, *, heads: int, n_layer: int, pad_id: int = 0, k: float = 4.0) -> Dict[str, float]:
    st = _Stats()
    H = w["emb"].shape[1]
    B, S = ids.shape

    def lin(name, x):
        st.see(name + ".in", x)
        y = x @ w[name + ".w"].T
        st.see(name + ".out", y)
        return (y + w[name + ".b"]).astype(F32)

    pad = ids == pad_id
    e = w["emb"][ids] + w["type_emb"][0]
    st.see("emb", w["emb"] + w["type_emb"][0])
    x = _ln(e + w["pos"][np.arange(S)], w["emb.ln.g"], w["emb.ln.b"])
    for l in range(n_layer):
        p = f"enc.{l}"
        qkv = lin(p + ".qkv", x)
        a = _attn(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads, pad[:, None, None, :])
        x = _ln(x + lin(p + ".out", a), w[p + ".ln1.g"], w[p + ".ln1.b"])
        h = _act(lin(p + ".fc1", x), "gelu")
        x = _ln(x + lin(p + ".fc2", h), w[p + ".ln2.g"], w[p + ".ln2.b"])
    amax = st.amax(k)
    for name, t in w.items():
        if name.endswith(".w") and t.ndim == 2:
            amax[name] = float(F32(k * t.std()))
    return amax


def make_bert(path: Optional[str] = None, *, hidden=768, heads=12, ffn=3072, n_layer=12, vocab=30522, max_step=512,
              pad_id=0, seed=1234, calib_ids: Optional[np.ndarray] = None):
    """Builds (conf, amax, tensors) of a seeded synthetic QuantBert (post-LN, GELU, learned positions)."""
    w = bert_weights(hidden, heads, ffn, n_layer, vocab, max_step, seed)
    if calib_ids is None:
        calib_ids = bert_inputs(batch=4, seq=min(32, max_step), vocab=vocab, pad_id=pad_id, seed=seed + 1)
    amax = calibrate_bert(w, calib_ids, heads=heads, n_layer=n_layer, pad_id=pad_id)
    conf = dict(hidden=hidden, heads=heads, ffn=ffn, n_enc=n_layer, vocab=vocab, act_gelu=1.0, pre_ln=0.0,
                max_step=max_step, pad_id=pad_id)
    if path is not None:
        from . import weights

        weights.save(path, "QuantBert", conf, amax, w)
    return conf, amax, w


# ------------------------------------------------------------------------------------------- ViT
def vit_weights(hidden=768, heads=12, ffn=3072, n_layer=12, image=224, patch=16, channels=3, seed=1234, std=0.02):
    rng = np.random.default_rng(seed)

    def nrm(*shape):
        return (rng.standard_normal(shape, dtype=F32) * F32(std)).astype(F32)

    n_tok = 1 + (image // patch) ** 2
    w: Dict[str, np.ndarray] = {"conv.w": nrm(hidden, channels * patch * patch), "conv.b": nrm(hidden), "pos": nrm(n_tok, hidden),
                                "cls": nrm(hidden), "enc.ln.g": np.ones(hidden, F32), "enc.ln.b": np.zeros(hidden, F32)}
    for l in range(n_layer):
        p = f"enc.{l}"
        for name, (no, ni) in (("qkv", (3 * hidden, hidden)), ("out", (hidden, hidden)), ("fc1", (ffn, hidden)),
                               ("fc2", (hidden, ffn))):
            w[f"{p}.{name}.w"] = nrm(no, ni)
            w[f"{p}.{name}.b"] = np.zeros(no, F32)
        for ln in ("ln1", "ln2"):
            w[f"{p}.{ln}.g"] = np.ones(hidden, F32)
            w[f"{p}.{ln}.b"] = np.zeros(hidden, F32)
    return w


def vit_inputs(batch=128, image=224, channels=3, seed=4321) -> np.ndarray:
    """pixels [batch, channels, image, image] fp32, N(0, 1) (normalised images)."""
    return np.random.default_rng(seed).standard_normal((batch, channels, image, image), dtype=F32)


def calibrate_vit(w, pixels, *, heads: int, n_layer: int, patch: int, k: float = 4.0) -> Dict[str, float]:
    st = _Stats()
    H = w["cls"].size
    B, C, I, _ = pixels.shape
    g = I // patch

    def lin(name, x):
        st.see(name + ".in", x)
        y = x @ w[name + ".w"].T
        st.see(name + ".out", y)
        return (y + w[name + ".b"]).astype(F32)

    xp = pixels.reshape(B, C, g, patch, g, patch).transpose(0, 2, 4, 1, 3, 5).reshape(B, g * g, -1)
    y = xp @ w["conv.w"].T + w["conv.b"] + w["pos"][1:]
    x = np.concatenate([np.broadcast_to(w["cls"] + w["pos"][0], (B, 1, H)), y], 1).astype(F32)
    for l in range(n_layer):
        p = f"enc.{l}"
        h = _ln(x, w[p + ".ln1.g"], w[p + ".ln1.b"])
        qkv = lin(p + ".qkv", h)
        a = _attn(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads, None)
        x = x + lin(p + ".out", a)
        h = _ln(x, w[p + ".ln2.g"], w[p + ".ln2.b"])
        x = x + lin(p + ".fc2", _act(lin(p + ".fc1", h), "gelu"))
    amax = st.amax(k)
    for name, t in w.items():
        if name.endswith(".w") and t.ndim == 2 and name != "conv.w":
            amax[name] = float(F32(k * t.std()))
    return amax


def make_vit(path: Optional[str] = None, *, hidden=768, heads=12, ffn=3072, n_layer=12, image=224, patch=16, channels=3,
             seed=1234, calib_pixels: Optional[np.ndarray] = None):
    """Builds (conf, amax, tensors) of a seeded synthetic QuantVit (patch embedding, pre-LN GELU encoder, final LayerNorm)."""
    w = vit_weights(hidden, heads, ffn, n_layer, image, patch, channels, seed)
    if calib_pixels is None:
        calib_pixels = vit_inputs(batch=2, image=image, channels=channels, seed=seed + 1)
    amax = calibrate_vit(w, calib_pixels, heads=heads, n_layer=n_layer, patch=patch)
    conf = dict(hidden=hidden, heads=heads, ffn=ffn, n_enc=n_layer, act_gelu=1.0, pre_ln=1.0, max_step=1 + (image // patch) ** 2,
                image_size=image, patch_size=patch, channels=channels)
    if path is not None:
        from . import weights

        weights.save(path, "QuantVit", conf, amax, w)
    return conf, amax, w


# ------------------------------------------------------------------------------------------- GPT-2
def gpt_weights(hidden=1024, heads=16, ffn=4096, n_layer=24, vocab=50257, max_pos=1024, seed=1234, std=0.02):
    rng = np.random.default_rng(seed)

    def nrm(*shape):
        return (rng.standard_normal(shape, dtype=F32) * F32(std)).astype(F32)

    w: Dict[str, np.ndarray] = {"emb": nrm(vocab, hidden), "pos": nrm(max_pos, hidden),
                                "dec.ln.g": np.ones(hidden, F32), "dec.ln.b": np.zeros(hidden, F32)}
    for l in range(n_layer):
        p = f"dec.{l}"
        for name, (no, ni) in (("qkv", (3 * hidden, hidden)), ("out", (hidden, hidden)), ("fc1", (ffn, hidden)),
                               ("fc2", (hidden, ffn))):
            w[f"{p}.{name}.w"] = nrm(no, ni)
            w[f"{p}.{name}.b"] = np.zeros(no, F32)
        for ln in ("ln1", "ln2"):
            w[f"{p}.{ln}.g"] = np.ones(hidden, F32)
            w[f"{p}.{ln}.b"] = np.zeros(hidden, F32)
    return w


def gpt_inputs(batch=64, prompt=64, vocab=50257, seed=4321) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, vocab, size=(batch, prompt)).astype(np.int32)


def calibrate_gpt(w, ids, *, heads: int, n_layer: int, k: float = 4.0) -> Dict[str, float]:
    st = _Stats()
    H = w["emb"].shape[1]
    B, S = ids.shape

    def lin(name, x):
        st.see(name + ".in", x)
        y = x @ w[name + ".w"].T
        st.see(name + ".out", y)
        return (y + w[name + ".b"]).astype(F32)

    causal = ~np.tril(np.ones((S, S), dtype=bool))
    x = (w["emb"][ids] + w["pos"][np.arange(S)]).astype(F32)
    for l in range(n_layer):
        p = f"dec.{l}"
        qkv = lin(p + ".qkv", _ln(x, w[p + ".ln1.g"], w[p + ".ln1.b"]))
        st.see(p + ".kv", qkv)
        a = _attn(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], heads, causal[None, None])
        x = x + lin(p + ".out", a)
        x = x + lin(p + ".fc2", _act(lin(p + ".fc1", _ln(x, w[p + ".ln2.g"], w[p + ".ln2.b"])), "gelu"))
    x = _ln(x, w["dec.ln.g"], w["dec.ln.b"])
    st.see("logits.in", x)
    st.see("logits.out", x[:, -4:] @ w["emb"].T)
    amax = st.amax(k)
    for name, t in w.items():
        if name.endswith(".w") and t.ndim == 2:
            amax[name] = float(F32(k * t.std()))
    amax["emb"] = float(F32(k * w["emb"].std()))
    return amax


def make_gpt(path: Optional[str] = None, *, hidden=1024, heads=16, ffn=4096, n_layer=24, vocab=50257, max_step=256,
             end_id=50256, topk=8, topp=0.0, pad_id=-1, max_new_tokens=192, seed=1234, rng_seed=2024,
             calib_ids: Optional[np.ndarray] = None):
    """Builds (conf, amax, tensors) of a seeded synthetic QuantGpt (GPT-2 layout: pre-LN, GELU, learned positions)."""
    w = gpt_weights(hidden, heads, ffn, n_layer, vocab, max_step, seed)
    if calib_ids is None:
        calib_ids = gpt_inputs(batch=4, prompt=min(24, max_step), vocab=vocab, seed=seed + 1)
    amax = calibrate_gpt(w, calib_ids, heads=heads, n_layer=n_layer)
    conf = dict(hidden=hidden, heads=heads, ffn=ffn, n_dec=n_layer, vocab=vocab, act_gelu=1.0, pre_ln=1.0,
                max_step=max_step, end_id=end_id, topk=topk, topp=topp, pad_id=pad_id, max_new_tokens=max_new_tokens,
                rng_seed=rng_seed)
    if path is not None:
        from . import weights

        weights.save(path, "QuantGpt", conf, amax, w)
    return conf, amax, w
