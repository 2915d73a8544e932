"""CPU oracle (test infrastructure, not product code): numpy restatement of the
reference's fake-quant Transformer layers on exact integer accumulators.

What follows what (paths inside the bytedance/lightseq tree):

* ``QLinear``            QuantLinear.forward, lightseq/training/ops/pytorch/quantization.py:33-61
* ``layer_norm``         torch.nn.LayerNorm (eps 1e-5) used at torch_transformer_layers.py:556,574
* ``mha_*``              MultiheadAttention.forward, torch_transformer_layers.py:152-396
* ``encoder_layer``      TransformerEncoderLayer.forward, torch_transformer_layers.py:630-679
* ``decoder_layer_step`` TransformerDecoderLayer.forward (incremental), torch_transformer_layers.py:844-965
* ``embed``              TransformerEmbeddingLayer.forward, torch_transformer_layers.py:1027-1036,
                         SinusoidalPositionalEmbedding :1069-1130
* ``Seq2Seq``            the wiring of lightseq/training/cli/fs_modules/ls_transformer.py:253-420
                         (final LayerNorms, output projection sharing the embedding quantiser)

Integer-exact rule: ``F.linear(fq(x), fq(W))`` is evaluated as
``float32(int_matmul(q_x, q_w)) * float32(s_x * s_w)``. The reference evaluates the
same product as an fp32 GEMM of the fake-quantised floats, whose rounding depends
on the BLAS summation order; the two agree to ~1e-6 relative, and the int8 tensor
produced by the next quantiser can differ by one step on a tiny fraction of
elements. tests/test_oracle_golden.py measures that fraction against outputs of
the real reference modules.

LayerNorm statistics are accumulated in float64 so the result does not depend on
summation order (the CUDA kernel does the same).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this package.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import numpy as np

from . import quant as Q

F32 = np.float32
LN_EPS = 1e-5


# --------------------------------------------------------------------------- config
@dataclass
class Config:
    hidden: int = 512
    heads: int = 8
    ffn: int = 2048
    n_enc: int = 6
    n_dec: int = 6
    vocab: int = 32000
    act: str = "relu"          # relu | gelu
    pre_ln: bool = True
    max_step: int = 256
    pad_id: int = 1
    start_id: int = 2
    end_id: int = 2
    beam: int = 4
    length_penalty: float = 0.6
    extra_decode_length: int = 50
    # generator options of the reference's decoder (lightseq/inference/proto/quant_transformer.proto:140-149)
    sampling_method: str = "beam_search"   # beam_search | topk | topp | topk_greedy
    topk: int = 1
    topp: float = 0.0
    output_topk: bool = False              # every beam in the result, last position forced to EOS
    no_scale_embedding: bool = False
    diverse_lambda: float = 0.0
    seed_lo: int = 0
    seed_hi: int = 0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


# --------------------------------------------------------------------------- calibration
class Calib:
    """Collects the std of every tensor that a quantiser will see (quantisers disabled),
    so that clip-max can be set to 4*std as the benchmark configuration prescribes."""

    def __init__(self):
        self.sum: Dict[str, float] = {}
        self.sq: Dict[str, float] = {}
        self.n: Dict[str, int] = {}

    def observe(self, name: str, x: np.ndarray):
        x = np.asarray(x, dtype=np.float64)
        self.sum[name] = self.sum.get(name, 0.0) + float(x.sum())
        self.sq[name] = self.sq.get(name, 0.0) + float((x * x).sum())
        self.n[name] = self.n.get(name, 0) + x.size

    def amax(self, k: float = 4.0) -> Dict[str, float]:
        out = {}
        for name, n in self.n.items():
            mean = self.sum[name] / n
            var = max(self.sq[name] / n - mean * mean, 1e-12)
            out[name] = float(np.float32(k * math.sqrt(var)))
        return out


@dataclass
class State:
    """Weights (fp32), clip-max table, caches of quantised weights; ``calib`` switches to
    the un-quantised fp32 forward that measures activation statistics."""
    w: Dict[str, np.ndarray]
    amax: Dict[str, float] = field(default_factory=dict)
    calib: Optional[Calib] = None
    trace: Optional[Dict[str, np.ndarray]] = None
    _wq: Dict[str, tuple] = field(default_factory=dict)

    def weight_q(self, wname: str, amax_name: str):
        key = wname + "|" + amax_name
        if key not in self._wq:
            q, s = Q.quantize(self.w[wname], self.amax[amax_name])
            self._wq[key] = (q, s, q.astype(np.float64), q.astype(np.int64).sum(axis=1))
        return self._wq[key]

    def rec(self, name: str, x):
        if self.trace is not None:
            self.trace[name] = np.array(x, copy=True)


# --------------------------------------------------------------------------- primitives
def layer_norm(x: np.ndarray, g: np.ndarray, b: np.ndarray) -> np.ndarray:
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=-1, keepdims=True)
    d = x64 - mean
    var = (d * d).mean(axis=-1, keepdims=True)
    y = (d * (1.0 / np.sqrt(var + LN_EPS))).astype(F32)
    return y * g.astype(F32) + b.astype(F32)


def qlinear(st: State, x: np.ndarray, name: str, *, wname: Optional[str] = None, w_amax: Optional[str] = None,
            unsigned_in: bool = False, quant_in: bool = True, quant_out: bool = True, bias: bool = True,
            return_q: bool = False):
    """QuantLinear.forward (quantization.py:50-61). ``name`` keys the clip-max entries
    ``name.in`` / ``name.w`` / ``name.out`` and the weights ``name.w`` / ``name.b``."""
    wname = wname or name + ".w"
    w_amax = w_amax or name + ".w"
    x = np.asarray(x, dtype=F32)
    b = st.w.get(name + ".b") if bias else None
    if st.calib is not None:
        if quant_in:
            st.calib.observe(name + ".in", x)
        y = x @ st.w[wname].T.astype(F32)
        if quant_out:
            st.calib.observe(name + ".out", y)
        return y + b if b is not None else y
    wq, s_w, wq64, w_rowsum = st.weight_q(wname, w_amax)
    if quant_in:
        xq, s_x = Q.quantize(x, st.amax[name + ".in"], unsigned=unsigned_in)
        st.rec(name + ".in_q", xq)
        acc = (xq.astype(np.float64) @ wq64.T).astype(np.int64)
        if unsigned_in:  # sum_k W_q (q+127) = acc + 127 * rowsum(W_q)
            acc = acc + 127 * w_rowsum[None, :]
        st.rec(name + ".acc", acc)
        v = acc.astype(F32) * F32(s_x * s_w)
    else:
        # weight-only quantisation (pre_activation="encoder_out", quantization.py:41-46)
        v = (x.astype(np.float64) @ wq64.T).astype(F32) * s_w
    if quant_out and not st.amax.get(name + ".out", 0.0) > 0.0:
        if return_q:
            raise ValueError(name + ".out: the integer output was asked for but this output is not quantised")
        quant_out = False  # a clip-max of 0 (or none): files of the encoder-only engines hold none for the second FFN output
    if quant_out:
        oq, s_o = Q.quantize(v, st.amax[name + ".out"], clip=False)
        st.rec(name + ".out_q", oq)
        v = oq.astype(F32) * s_o
    if b is not None:
        v = v + b.astype(F32)
    if return_q:
        return v, oq, s_o
    return v


def softmax_rows(s: np.ndarray) -> np.ndarray:
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / e.sum(axis=-1, keepdims=True)


def attention_core(q, k, v, heads: int, key_pad: Optional[np.ndarray], scaling: float, causal: bool = False):
    """q [B,Lq,H], k/v [B,Lk,H] fp32 (already biased); key_pad [B,Lk] True = masked.
    torch_transformer_layers.py:231,332-376: q*scaling, bmm, masked_fill(-inf), fp32 softmax, bmm."""
    B, Lq, H = q.shape
    Lk = k.shape[1]
    dh = H // heads
    qh = (q * F32(scaling)).reshape(B, Lq, heads, dh).transpose(0, 2, 1, 3)
    kh = k.reshape(B, Lk, heads, dh).transpose(0, 2, 1, 3)
    vh = v.reshape(B, Lk, heads, dh).transpose(0, 2, 1, 3)
    s = np.matmul(qh, kh.transpose(0, 1, 3, 2)).astype(F32)
    if causal:  # torch_transformer_layers.py:337-345 (masked_bias = -1e4)
        tri = np.tril(np.ones((Lk, Lk), dtype=bool))[Lk - Lq:Lk, :Lk]
        s = np.where(tri[None, None], s, F32(-1e4))
    if key_pad is not None:
        s = np.where(key_pad[:, None, None, :], F32(-np.inf), s)
    p = softmax_rows(s).astype(F32)
    o = np.matmul(p, vh).astype(F32)
    return o.transpose(0, 2, 1, 3).reshape(B, Lq, H)


def activation(x, act: str):
    if act == "relu":
        return np.maximum(x, F32(0))
    if act == "gelu":
        return Q.gelu(x)
    raise ValueError(act)


def ffn(st: State, x: np.ndarray, p: str, cfg: Config) -> np.ndarray:
    h = activation(qlinear(st, x, p + ".fc1"), cfg.act)
    return qlinear(st, h, p + ".fc2", unsigned_in=(cfg.act == "relu"))


# --------------------------------------------------------------------------- encoder layer
def encoder_layer(st: State, x: np.ndarray, key_pad: Optional[np.ndarray], p: str, cfg: Config,
                  causal: bool = False) -> np.ndarray:
    """x [B,S,H] -> [B,S,H] (torch_transformer_layers.py:630-679)."""
    B, S, H = x.shape
    res = x
    h = layer_norm(x, st.w[p + ".ln1.g"], st.w[p + ".ln1.b"]) if cfg.pre_ln else x
    qkv = qlinear(st, h.reshape(B * S, H), p + ".qkv").reshape(B, S, 3 * H)
    a = attention_core(qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:], cfg.heads, key_pad,
                       cfg.head_dim ** -0.5, causal)
    st.rec(p + ".attn", a)
    o = qlinear(st, a.reshape(B * S, H), p + ".out").reshape(B, S, H)
    x = res + o
    if not cfg.pre_ln:
        x = layer_norm(x, st.w[p + ".ln1.g"], st.w[p + ".ln1.b"])
    res = x
    h = layer_norm(x, st.w[p + ".ln2.g"], st.w[p + ".ln2.b"]) if cfg.pre_ln else x
    f = ffn(st, h.reshape(B * S, H), p, cfg).reshape(B, S, H)
    x = res + f
    if not cfg.pre_ln:
        x = layer_norm(x, st.w[p + ".ln2.g"], st.w[p + ".ln2.b"])
    return x.astype(F32)


# --------------------------------------------------------------------------- embedding
def sinusoid_table(n: int, dim: int) -> np.ndarray:
    """SinusoidalPositionalEmbedding.get_embedding (torch_transformer_layers.py:1086-1106), fp32."""
    half = dim // 2
    e = F32(math.log(10000) / (half - 1))
    freq = np.exp(np.arange(half, dtype=F32) * -e).astype(F32)
    ang = (np.arange(n, dtype=F32)[:, None] * freq[None, :]).astype(F32)
    tab = np.concatenate([np.sin(ang), np.cos(ang)], axis=1).astype(F32)
    if dim % 2 == 1:
        tab = np.concatenate([tab, np.zeros((n, 1), F32)], axis=1)
    return tab


def embed(st: State, ids: np.ndarray, step: int, cfg: Config, pos_table: np.ndarray) -> np.ndarray:
    """ids [B,L] -> [B,L,H]: lookup -> emb_quant -> *sqrt(H) -> + sinusoid (pads zeroed)."""
    e = st.w["emb"][ids]
    if st.calib is not None:
        st.calib.observe("emb", st.w["emb"])
    else:
        eq, s = st.weight_q("emb", "emb")[:2]
        e = eq[ids].astype(F32) * s
    x = e if cfg.no_scale_embedding else F32(math.sqrt(cfg.hidden)) * e
    mask = (ids != cfg.pad_id)
    pos = (np.cumsum(mask, axis=1) - 1 + step) * mask
    return (x + pos_table[pos] * mask[..., None].astype(F32)).astype(F32)


# --------------------------------------------------------------------------- decoder layer
def decoder_layer_step(st: State, x: np.ndarray, p: str, cfg: Config, cache: dict, cross_k: np.ndarray,
                       cross_v: np.ndarray, src_pad: np.ndarray) -> np.ndarray:
    """One incremental step. x [T,H] (T = batch*beam); ``cache`` holds this layer's
    int8 self-attention keys/values [T,L,H] (grown here); cross_k/v [B,S,H] fp32.
    torch_transformer_layers.py:844-965 with MultiheadAttention's incremental branch :262-300."""
    T, H = x.shape
    beam = T // cross_k.shape[0]
    res = x
    h = layer_norm(x, st.w[p + ".ln1.g"], st.w[p + ".ln1.b"]) if cfg.pre_ln else x
    qkv = qlinear(st, h, p + ".qkv")
    if st.calib is not None:
        st.calib.observe(p + ".kv", qkv)
        q, k, v = qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:]
        cache["k"] = k[:, None] if "k" not in cache else np.concatenate([cache["k"], k[:, None]], 1)
        cache["v"] = v[:, None] if "v" not in cache else np.concatenate([cache["v"], v[:, None]], 1)
        K, V = cache["k"], cache["v"]
    else:
        # attention_quant on the whole biased qkv (torch_transformer_layers.py:95-97,203-204)
        qq, s_kv = Q.quantize(qkv, st.amax[p + ".kv"], clip=False)
        st.rec(p + ".qkv_q", qq)
        kq, vq = qq[:, H:2 * H], qq[:, 2 * H:]
        cache["k"] = kq[:, None] if "k" not in cache else np.concatenate([cache["k"], kq[:, None]], 1)
        cache["v"] = vq[:, None] if "v" not in cache else np.concatenate([cache["v"], vq[:, None]], 1)
        q = qq[:, :H].astype(F32) * s_kv
        K = cache["k"].astype(F32) * s_kv
        V = cache["v"].astype(F32) * s_kv
    a = attention_core(q[:, None], K, V, cfg.heads, None, cfg.head_dim ** -0.5)[:, 0]
    st.rec(p + ".attn", a)
    x = res + qlinear(st, a, p + ".out")
    if not cfg.pre_ln:
        x = layer_norm(x, st.w[p + ".ln1.g"], st.w[p + ".ln1.b"])

    res = x
    h = layer_norm(x, st.w[p + ".ln2.g"], st.w[p + ".ln2.b"]) if cfg.pre_ln else x
    q = qlinear(st, h, p + ".xq")
    kx = np.repeat(cross_k, beam, axis=0)
    vx = np.repeat(cross_v, beam, axis=0)
    pad = np.repeat(src_pad, beam, axis=0)
    a = attention_core(q[:, None], kx, vx, cfg.heads, pad, cfg.head_dim ** -0.5)[:, 0]
    st.rec(p + ".xattn", a)
    x = res + qlinear(st, a, p + ".xout")
    if not cfg.pre_ln:
        x = layer_norm(x, st.w[p + ".ln2.g"], st.w[p + ".ln2.b"])

    res = x
    h = layer_norm(x, st.w[p + ".ln3.g"], st.w[p + ".ln3.b"]) if cfg.pre_ln else x
    x = res + ffn(st, h, p, cfg)
    if not cfg.pre_ln:
        x = layer_norm(x, st.w[p + ".ln3.g"], st.w[p + ".ln3.b"])
    return x.astype(F32)


# --------------------------------------------------------------------------- full model
class Seq2Seq:
    """Encoder-decoder with shared embedding / output projection and beam search."""

    def __init__(self, cfg: Config, st: State):
        self.cfg = cfg
        self.st = st
        self.pos = sinusoid_table(max(cfg.max_step, 1024), cfg.hidden)

    # encoder -------------------------------------------------------------
    def encode(self, src: np.ndarray):
        cfg, st = self.cfg, self.st
        pad = (src == cfg.pad_id)
        x = embed(st, src, 0, cfg, self.pos)
        st.rec("enc.emb", x)
        for l in range(cfg.n_enc):
            x = encoder_layer(st, x, pad, f"enc.{l}", cfg)
            st.rec(f"enc.{l}.y", x)
        if cfg.pre_ln:
            x = layer_norm(x, st.w["enc.ln.g"], st.w["enc.ln.b"])
        st.rec("enc.out", x)
        return x.astype(F32), pad

    def cross_kv(self, enc_out: np.ndarray):
        """k_proj / v_proj of every decoder layer: weight-only fake-quant, fp32 activations."""
        B, S, H = enc_out.shape
        flat = enc_out.reshape(B * S, H)
        ks, vs = [], []
        for l in range(self.cfg.n_dec):
            ks.append(qlinear(self.st, flat, f"dec.{l}.xk", quant_in=False, quant_out=False).reshape(B, S, H))
            vs.append(qlinear(self.st, flat, f"dec.{l}.xv", quant_in=False, quant_out=False).reshape(B, S, H))
        return ks, vs

    # one decoder step ----------------------------------------------------
    def decode_step(self, tokens: np.ndarray, step: int, caches, ks, vs, src_pad):
        """tokens [T] -> (int8 logits [T,V], logits scale)."""
        cfg, st = self.cfg, self.st
        x = embed(st, tokens[:, None], step, cfg, self.pos)[:, 0]
        st.rec("dec.emb", x)
        for l in range(cfg.n_dec):
            x = decoder_layer_step(st, x, f"dec.{l}", cfg, caches[l], ks[l], vs[l], src_pad)
            st.rec(f"dec.{l}.y", x)
        if cfg.pre_ln:
            x = layer_norm(x, st.w["dec.ln.g"], st.w["dec.ln.b"])
        if st.calib is not None:
            return qlinear(st, x, "logits", wname="emb", w_amax="emb", bias=False), None
        _, lq, s = qlinear(st, x, "logits", wname="emb", w_amax="emb", bias=False, return_q=True)
        return lq, s

    # beam search ---------------------------------------------------------
    def generate(self, src: np.ndarray, max_len: Optional[int] = None, early_stop: bool = True):
        """Generation following the reference engine's bookkeeping
        (lightseq/inference/model/quant_decoder.cc.cu:415-484,951-1133;
        lightseq/inference/kernels/transformerKernels_int8.cc.cu:1690-1844;
        lightseq/inference/kernels/transformerKernels.cc.cu:1398-1463,1722-1813), with an
        exact per-row top-``beam`` instead of the rough threshold, no float batch offsets,
        and the deterministic tie-break: higher score, then lower beam, then lower token id.

        ``sampling_method`` beam_search: returns (tokens [B, n] of the best beam, scores [B], n); with
        ``output_topk`` (tokens [B, K, n], scores [B, K], n), the last position forced to EOS. A negative length
        penalty picks, per sentence, the beam with the best score per non-EOS token.
        topk / topp: one sequence per sentence sampled token by token (counter-based Philox draw keyed by position and
        row), up to ``max_step`` tokens; returns (tokens [B, 1, n], scores [B, 1] = 0, n).
        topk_greedy: the first step is a beam step (K different first tokens), every later step takes each row's
        best token; returns all K rows like ``output_topk``."""
        from .beam import beam_step, length_norm, sample_topk_row, sample_topp_row

        cfg = self.cfg
        B, S = src.shape
        method = cfg.sampling_method
        sampling = method in ("topk", "topp")
        K = 1 if sampling else cfg.beam
        enc_out, src_pad = self.encode(src)
        ks, vs = self.cross_kv(enc_out)
        max_decode = cfg.max_step if method != "beam_search" else min(cfg.max_step, S + cfg.extra_decode_length) - 1
        if max_len is not None:
            max_decode = min(max_decode, max_len)
        alive = np.full((B, K, cfg.max_step), cfg.end_id, dtype=np.int32)
        alive[:, :, 0] = cfg.start_id
        probs = np.full((B, K), -1000.0, dtype=F32)
        probs[:, 0] = 0.0
        score = np.zeros((B, K), dtype=F32)
        caches = [dict() for _ in range(cfg.n_dec)]
        cur = 0
        for cur in range(max_decode - 1):
            tokens = alive[:, :, cur].reshape(-1)
            lq, s_l = self.decode_step(tokens, cur, caches, ks, vs, src_pad)
            if method == "beam_search" or (method == "topk_greedy" and cur == 0):
                ln = length_norm(cur + 1, cfg.length_penalty)
                alive, probs, score, parent, n_fin = beam_step(
                    lq.reshape(B, K, -1), s_l, alive, probs, score, cur, ln, cfg.end_id,
                    cfg.diverse_lambda if method == "beam_search" else 0.0)
                if early_stop and n_fin == B * K:
                    break
                flat = (parent + np.arange(B)[:, None] * K).reshape(-1)
                for c in caches:
                    c["k"] = c["k"][flat]
                    c["v"] = c["v"][flat]
                continue
            flat_alive = alive.reshape(B * K, -1)
            for r in range(B * K):
                if flat_alive[r, cur] == cfg.end_id and cur != 0:
                    flat_alive[r, cur + 1] = cfg.end_id
                elif method == "topp":
                    flat_alive[r, cur + 1] = sample_topp_row(lq[r], s_l, cfg.topp, cur + 1, r, cfg.seed_lo, cfg.seed_hi)
                else:
                    k = 1 if method == "topk_greedy" else cfg.topk
                    flat_alive[r, cur + 1] = sample_topk_row(lq[r], s_l, k, cur + 1, r, cfg.seed_lo, cfg.seed_hi)
            if early_stop and (flat_alive[:, cur + 1] == cfg.end_id).all():
                break
        else:
            cur = max(max_decode - 1, 0)
        n = min(cur + 1, cfg.max_step - 1)
        if method != "beam_search" or cfg.output_topk:
            tok = alive[:, :, 1:n + 1].copy()
            tok[:, :, n - 1] = cfg.end_id
            return tok, score.copy(), n
        if cfg.length_penalty < 0:
            out_t = np.zeros((B, n), np.int32)
            out_s = np.zeros(B, F32)
            for b in range(B):
                best, pick = F32(-np.inf), 0
                for j in range(K):
                    ln_j = int((alive[b, j, 1:n + 1] != cfg.end_id).sum())
                    sc = F32(score[b, j] / F32(F32(ln_j) + F32(1e-12)))
                    if sc > best:
                        best, pick = sc, j
                out_t[b] = alive[b, pick, 1:n + 1]
                out_s[b] = best
            return out_t, out_s, n
        return alive[:, 0, 1:n + 1].copy(), score[:, 0].copy(), n


# --------------------------------------------------------------------------- BERT
class Bert:
    """BertEmbeddingLayer (torch_transformer_layers.py:1177-1207: word + token-type(0) -> emb_quant -> + learned
    position -> LayerNorm) followed by post-LN GELU encoder layers (:630-679); output [B,S,H] fp32, as
    QuantBertEncoder::run_one_infer returns it (lightseq/inference/model/quant_bert_encoder.cc.cu:214-265)."""

    def __init__(self, cfg: Config, st: State):
        self.cfg = cfg
        self.st = st

    def embed(self, ids: np.ndarray) -> np.ndarray:
        st = self.st
        e = st.w["emb"][ids] + st.w["type_emb"][0]
        eq, s = Q.quantize(e, st.amax["emb"])
        x = eq.astype(F32) * s + st.w["pos"][np.arange(ids.shape[1])]
        return layer_norm(x, st.w["emb.ln.g"], st.w["emb.ln.b"])

    def forward(self, ids: np.ndarray) -> np.ndarray:
        cfg, st = self.cfg, self.st
        pad = ids == cfg.pad_id
        x = self.embed(ids)
        st.rec("emb.out", x)
        for l in range(cfg.n_enc):
            x = encoder_layer(st, x, pad, f"enc.{l}", cfg)
            st.rec(f"enc.{l}.y", x)
        return x


# --------------------------------------------------------------------------- ViT encoder
def patch_embed(w: Dict[str, np.ndarray], pixels: np.ndarray, patch: int) -> np.ndarray:
    """pixels [B,C,I,I] fp32 -> [B, 1+N, H]: token 0 = cls + pos[0]; token 1+n = conv(patch n) + bias + pos[1+n] with
    kernel = stride = patch, patches in row-major order, weight index (hidden, channel, row, col)
    (ker_patch_emb, lightseq/inference/kernels/embKernels.cc.cu:565-606). The dot products are taken in float64 and
    rounded once to fp32 (the reference sums in fp32 in a block-reduction order of its own); bias and position are
    fp32 additions in the reference's order."""
    B, C, I, _ = pixels.shape
    g = I // patch
    x = pixels.reshape(B, C, g, patch, g, patch).transpose(0, 2, 4, 1, 3, 5).reshape(B, g * g, C * patch * patch)
    y = (x.astype(np.float64) @ w["conv.w"].reshape(w["conv.w"].shape[0], -1).astype(np.float64).T).astype(F32)
    y = (y + w["conv.b"].astype(F32)).astype(F32) + w["pos"][1:1 + g * g].astype(F32)
    cls = (w["cls"].astype(F32) + w["pos"][0].astype(F32)).astype(F32)
    return np.concatenate([np.broadcast_to(cls, (B, 1, cls.size)), y.astype(F32)], axis=1).astype(F32)


class Vit:
    """QuantVit: patch embedding (fp32) -> pre-LN int8 encoder layers -> final LayerNorm; output [B, 1+N, H] fp32 as
    QuantVitEncoder::run_one_infer leaves it (lightseq/inference/model/quant_vit_encoder.cc.cu:189-232). No token is
    padding."""

    def __init__(self, cfg: Config, st: State, patch: int):
        self.cfg = cfg
        self.st = st
        self.patch = patch

    def forward(self, pixels: np.ndarray) -> np.ndarray:
        cfg, st = self.cfg, self.st
        x = patch_embed(st.w, pixels, self.patch)
        st.rec("emb.out", x)
        for l in range(cfg.n_enc):
            x = encoder_layer(st, x, None, f"enc.{l}", cfg)
            st.rec(f"enc.{l}.y", x)
        if cfg.pre_ln:
            x = layer_norm(x, st.w["enc.ln.g"], st.w["enc.ln.b"])
        return x.astype(F32)


# --------------------------------------------------------------------------- GPT-2 style decoder-only model
def gpt_layer(st: State, x: np.ndarray, p: str, cfg: Config, cache: dict) -> np.ndarray:
    """Decoder-only layer (TransformerDecoderLayer with has_cross_attn=False, pre-LN, causal;
    torch_transformer_layers.py:682-965 wired as in examples/training/huggingface/gpt/ls_hf_gpt_layer.py:44-83).
    x [B,L,H] holds the L newest positions; ``cache`` keeps the int8 keys/values of all earlier positions
    (attention_quant is applied to the whole biased qkv, :95-97,203-204)."""
    B, L, H = x.shape
    res = x
    h = layer_norm(x, st.w[p + ".ln1.g"], st.w[p + ".ln1.b"])
    qkv = qlinear(st, h.reshape(B * L, H), p + ".qkv").reshape(B, L, 3 * H)
    qq, s_kv = Q.quantize(qkv, st.amax[p + ".kv"], clip=False)
    st.rec(p + ".qkv_q", qq)
    kq, vq = qq[..., H:2 * H], qq[..., 2 * H:]
    cache["k"] = kq if "k" not in cache else np.concatenate([cache["k"], kq], 1)
    cache["v"] = vq if "v" not in cache else np.concatenate([cache["v"], vq], 1)
    a = attention_core(qq[..., :H].astype(F32) * s_kv, cache["k"].astype(F32) * s_kv, cache["v"].astype(F32) * s_kv,
                       cfg.heads, None, cfg.head_dim ** -0.5, causal=True)
    st.rec(p + ".attn", a)
    x = res + qlinear(st, a.reshape(B * L, H), p + ".out").reshape(B, L, H)
    res = x
    h = layer_norm(x, st.w[p + ".ln2.g"], st.w[p + ".ln2.b"])
    return (res + ffn(st, h.reshape(B * L, H), p, cfg).reshape(B, L, H)).astype(F32)


class Gpt:
    """GptEmbedding (token lookup -> emb_quant, ls_hf_gpt_layer.py:85-96) + learned positions + decoder-only
    layers + final LayerNorm + lm_head sharing the embedding table and quantiser (:131-139); generation by
    top-k sampling as QuantGptEncoder::run_one_sample (lightseq/inference/model/quant_gpt_encoder.cc.cu:300-397)."""

    def __init__(self, cfg: Config, st: State):
        self.cfg = cfg
        self.st = st

    def forward(self, ids: np.ndarray, start: int, caches) -> np.ndarray:
        """ids [B,L] at absolute positions start..start+L-1 -> final-LayerNorm hidden states [B,L,H]."""
        cfg, st = self.cfg, self.st
        eq, s = st.weight_q("emb", "emb")[:2]
        x = eq[ids].astype(F32) * s + st.w["pos"][start + np.arange(ids.shape[1])]
        for l in range(cfg.n_dec):
            x = gpt_layer(st, x.astype(F32), f"dec.{l}", cfg, caches[l])
        return layer_norm(x, st.w["dec.ln.g"], st.w["dec.ln.b"])

    def logits(self, h: np.ndarray):
        """h [T,H] -> (int8 logits [T,V], scale)."""
        _, lq, s = qlinear(self.st, h, "logits", wname="emb", w_amax="emb", bias=False, return_q=True)
        return lq, s

    def ppl(self, ids: np.ndarray, pad_id: int = -1) -> np.ndarray:
        """Mean negative log-likelihood of each sequence's own next tokens from the int8 logits, as ker_ppl_i8I
        (lightseq/inference/kernels/gptKernels_int8.cc.cu:108-180): positions t < len - 1 of a sequence of len
        non-pad tokens, each contributing logsumexp(logits_t) - logits_t[ids[t + 1]]."""
        cfg = self.cfg
        B, S = ids.shape
        h = self.forward(ids, 0, [dict() for _ in range(cfg.n_dec)])
        lq, s_l = self.logits(h.reshape(B * S, -1))
        lg = lq.astype(np.float64).reshape(B, S, -1) * float(s_l)
        mx = lg.max(-1, keepdims=True)
        lse = np.log(np.exp(lg - mx).sum(-1)) + mx[..., 0]
        out = np.zeros(B, dtype=F32)
        for b in range(B):
            n = int((ids[b] != pad_id).sum()) if pad_id >= 0 else S
            if n > 1:
                t = np.arange(n - 1)
                out[b] = F32((lse[b, t] - lg[b, t, ids[b, t + 1]]).mean())
        return out

    def generate(self, prompt: np.ndarray, max_new: int, k: int, seed_lo: int, seed_hi: int, topp: float = 0.0):
        from .beam import sample_topk_row, sample_topp_row

        cfg = self.cfg
        B, P = prompt.shape
        caches = [dict() for _ in range(cfg.n_dec)]
        seq = np.full((B, cfg.max_step), cfg.end_id, dtype=np.int32)
        seq[:, :P] = prompt
        h = self.forward(prompt, 0, caches)[:, -1]
        cur = P - 1
        while cur + 1 < min(cfg.max_step, P + max_new):
            lq, s_l = self.logits(h)
            for b in range(B):
                if seq[b, cur] == cfg.end_id:
                    seq[b, cur + 1] = cfg.end_id
                else:
                    seq[b, cur + 1] = (sample_topp_row(lq[b], s_l, topp, cur + 1, b, seed_lo, seed_hi) if topp > 0
                                       else sample_topk_row(lq[b], s_l, k, cur + 1, b, seed_lo, seed_hi))
            cur += 1
            if (seq[:, cur] == cfg.end_id).all():
                break
            if cur + 1 >= min(cfg.max_step, P + max_new):
                break
            h = self.forward(seq[:, cur:cur + 1], cur, caches)[:, 0]
        return seq[:, :cur + 1].copy()
