"""CPU oracle (test infrastructure, not product code): one beam-search step and the
top-k / top-p sampling step, restated from the reference inference engine.

Beam step = ``select_beam_rough_topk_i8I`` (lightseq/inference/kernels/transformerKernels_int8.cc.cu:1690-1844)
+ the global sort of ``QuantDecoder::beam_search`` (lightseq/inference/model/quant_decoder.cc.cu:987-1076)
+ ``ker_refresh_result`` (lightseq/inference/kernels/transformerKernels.cc.cu:1398-1463):

* a beam whose last token is EOS re-emits EOS with its frozen ``seq_score``;
* a live beam scores token v as ``(logit_v + prefix - logsumexp) * length_norm``, with
  ``exp`` arguments clamped at -64 (``logit_thresh_min``, transformerKernels.h:11) and the
  result floored at -1999 (``min_log_probability + 1``);
* per batch the best ``beam`` candidates survive; live ones get ``seq_probs = score / length_norm``.

Differences from the engine, on purpose: exact top-``beam`` per row instead of the
rough threshold of ``blockRoughTopK`` (a superset of the winners, so the winners are
the same); no ``-2000 * batch_id`` float offsets (they only separate batches inside
one global sort and cost precision); ties broken by (higher score, lower beam, lower
token id) instead of the unspecified Thrust order; ``seq_score`` is also refreshed
for live beams (the engine leaves it stale there).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import
this package.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
LOGIT_THRESH_MIN = F32(-64.0)
MIN_LOG_PROB = F32(-2000.0)


def length_norm(length: int, alpha: float) -> np.float32:
    """transformerKernels.h:137-140."""
    if alpha < 0:
        return F32(1.0 / length)
    return F32(np.power(F32((5.0 + length) / 6.0), F32(-alpha)))


def row_logsumexp_base(lq_row: np.ndarray, s_l: np.float32):
    """max logit and log(sum exp) of one dequantised int8 row; sums run over the 255-bin
    histogram of the int8 values from the largest value down (order-independent)."""
    hist = np.bincount(lq_row.astype(np.int32) + 128, minlength=256)
    vals = np.nonzero(hist)[0]
    qmax = vals.max() - 128
    mx = F32(qmax) * s_l
    tot = np.float64(0.0)
    for b in vals[::-1]:
        lg = F32(b - 128) * s_l
        d = max(F32(lg - mx), LOGIT_THRESH_MIN)
        tot += np.float64(hist[b]) * np.float64(np.exp(F32(d), dtype=F32))
    return mx, F32(np.log(F32(tot), dtype=F32))


def candidate_score(lq_row: np.ndarray, s_l, prob, ln, token: int) -> np.float32:
    """Score the engine/oracle assigns to extending a live beam (prefix log-prob ``prob``) with ``token``."""
    s_l = F32(s_l)
    mx, lse = row_logsumexp_base(lq_row, s_l)
    base = F32(F32(F32(prob) - lse) - mx)
    lg = F32(lq_row[token]) * s_l
    return max(F32(F32(lg + base) * F32(ln)), F32(MIN_LOG_PROB + F32(1.0)))


def beam_step(lq: np.ndarray, s_l, alive: np.ndarray, probs: np.ndarray, score: np.ndarray, cur_step: int,
              ln, end_id: int, diverse_lambda: float = 0.0):
    """lq int8 [B,K,V]; alive int32 [B,K,max_step]; probs/score fp32 [B,K].
    Returns (new_alive, new_probs, new_score, parent [B,K], n_finished).
    ``diverse_lambda`` (diverse beam search, ker_diverse_beam_search, lightseq/inference/kernels/
    transformerKernels.cc.cu:312-333): the r-th best candidate of a beam competes with its score minus
    lambda * (r + 1); the stored score and prefix are the unpenalised ones (ker_refresh_result :1430-1458)."""
    lam = F32(diverse_lambda)
    B, K, V = lq.shape
    s_l = F32(s_l)
    ln = F32(ln)
    new_alive = np.full_like(alive, end_id)
    new_probs = probs.copy()
    new_score = score.copy()
    parent = np.zeros((B, K), dtype=np.int64)
    n_fin = 0
    for b in range(B):
        cands = []  # (score, beam, token)
        for k in range(K):
            if cur_step != 0 and alive[b, k, cur_step] == end_id:
                cands.append((F32(F32(score[b, k]) - lam), k, end_id, 0))
                continue
            row = lq[b, k]
            mx, lse = row_logsumexp_base(row, s_l)
            base = F32(F32(probs[b, k] - lse) - mx)
            # exact top-K of the row: larger int8 value first, then lower token id
            order = np.lexsort((np.arange(V), -row.astype(np.int32)))[:K]
            for rank, v in enumerate(order):
                lg = F32(row[v]) * s_l
                sc = max(F32(F32(lg + base) * ln), F32(MIN_LOG_PROB + F32(1.0)))
                cands.append((F32(sc - F32(lam * F32(rank + 1))), k, int(v), rank))
        cands.sort(key=lambda c: (-float(c[0]), c[1], c[2]))
        for j in range(K):
            sc, k, v, rank = cands[j]
            sc = F32(sc + F32(lam * F32(rank + 1)))
            parent[b, j] = k
            new_alive[b, j, :cur_step + 1] = alive[b, k, :cur_step + 1]
            new_alive[b, j, cur_step + 1] = v
            new_score[b, j] = sc
            if v != end_id:
                new_probs[b, j] = F32(sc / ln)
            else:
                n_fin += 1
    return new_alive, new_probs, new_score, parent, n_fin


# --------------------------------------------------------------------------- top-k sampling
def philox4x32_10_first(c0: int, c1: int, c2: int, c3: int, k0: int, k1: int) -> int:
    """First output word of Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11)."""
    M0, M1, W0, W1, MASK = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & MASK, p1 >> 32, p1 & MASK
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & MASK, lo1, (hi0 ^ c3 ^ k1) & MASK, lo0
        k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
    return c0


def sample_topk_row(lq_row: np.ndarray, s_l, k: int, position: int, row: int, seed_lo: int, seed_hi: int) -> int:
    """Top-k sampling of one row of int8 logits, restating ker_topk_sample_i8I
    (lightseq/inference/kernels/gptKernels_int8.cc.cu:252-430) with an exact top-k (logit desc, token asc),
    softmax over the kept logits, cumulative in that order, and a counter-based uniform
    u = ((philox(position, row; seed) >> 8) + 1) * 2^-24 instead of the engine's clock()-seeded cuRAND state."""
    s_l = F32(s_l)
    V = lq_row.shape[0]
    order = np.lexsort((np.arange(V), -lq_row.astype(np.int32)))[:k]
    v0 = int(lq_row[order[0]])
    e = [np.exp(F32(F32(int(lq_row[i]) - v0) * s_l), dtype=F32) for i in order]
    tot = F32(0)
    for x in e:
        tot = F32(tot + x)
    u = F32(F32((philox4x32_10_first(position, row, 0, 0, seed_lo, seed_hi) >> 8) + 1) * F32(2.0 ** -24))
    cum = F32(0)
    pick = len(order) - 1
    for i, x in enumerate(e):
        cum = F32(cum + F32(x / tot))
        if u <= cum:
            pick = i
            break
    return int(order[pick])


def _topp_rank(c, w, n: int, t) -> int:
    """Smallest j in [1, n] with float32(c + float32(j) * w) >= t, n if there is none."""
    for j in range(1, n + 1):
        if F32(c + F32(F32(j) * w)) >= t:
            return j
    return n


def sample_topp_row(lq_row: np.ndarray, s_l, p, position: int, row: int, seed_lo: int, seed_hi: int) -> int:
    """Nucleus sampling of one row of int8 logits: the exact form of what ker_topp_sample_i8I approximates
    (lightseq/inference/kernels/transformerKernels_int8.cc.cu:2131-2294). Tokens are ordered by (logit desc,
    token asc); all float32; masses are accumulated level by level (there are at most 255 levels), a level of
    n tokens of weight w contributing float32(n) * w; the nucleus is the shortest prefix whose mass reaches
    p * total and the draw is the first token whose cumulative mass reaches u * mass(nucleus)."""
    s_l, p = F32(s_l), F32(p)
    lq = lq_row.astype(np.int32)
    levels = sorted(set(lq.tolist()), reverse=True)
    top = levels[0]
    cnt = {q: int((lq == q).sum()) for q in levels}
    wgt = {q: np.exp(F32(F32(q - top) * s_l), dtype=F32) for q in levels}
    total = F32(0)
    for q in levels:
        total = F32(total + F32(F32(cnt[q]) * wgt[q]))
    cut = F32(p * total)
    c = F32(0)
    for q in levels:
        m = F32(F32(cnt[q]) * wgt[q])
        cut_q, cut_n = q, cnt[q]
        if F32(c + m) >= cut:
            cut_n = _topp_rank(c, wgt[q], cnt[q], cut)
            mass = F32(c + F32(F32(cut_n) * wgt[q]))
            break
        c = F32(c + m)
        mass = c
    u = F32(F32((philox4x32_10_first(position, row, 0, 0, seed_lo, seed_hi) >> 8) + 1) * F32(2.0 ** -24))
    target = F32(u * mass)
    c = F32(0)
    for q in levels:
        n = cut_n if q == cut_q else cnt[q]
        m = F32(F32(n) * wgt[q])
        if q == cut_q or F32(c + m) >= target:
            rank = _topp_rank(c, wgt[q], n, target)
            return int(np.flatnonzero(lq == q)[rank - 1])
        c = F32(c + m)
    raise AssertionError("unreachable")
