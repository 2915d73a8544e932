// Top-k sampling step for decoder-only generation (QuantGpt): one CTA of eight warps per sequence streams the row of int8
// logits once (16-byte loads, SIMD byte compares against a warp-wide running threshold, candidate buffer in
// shared memory — the same selection as the beam kernel), then lane 0 draws the token with a counter-based
// Philox4x32-10 stream keyed by (seed, row, position), so results do not depend on launch order or history.
// No host round trip: the kernel appends the token, advances the position and records when every row has ended.
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr int SMP_WARPS = 8;
constexpr int SMP_MAXK = 8;
constexpr int SMP_BUF = 512 + 64;

__device__ __forceinline__ int4 smp_load16(const int8_t* lp, int off, int vocab) {
  if (off + 16 <= vocab && ((reinterpret_cast<uintptr_t>(lp + off) & 15) == 0)) return *reinterpret_cast<const int4*>(lp + off);
  int w[4] = {(int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080};  // -128 = "no token"
  for (int j = 0; j < 16 && off + j < vocab; ++j) {
    const int byte = (int)(uint8_t)lp[off + j];
    w[j >> 2] = (w[j >> 2] & ~(0xff << ((j & 3) * 8))) | (byte << ((j & 3) * 8));
  }
  return make_int4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ int smp_flush(unsigned* buf, int n, int K, int lane, int* n_kept) {
  constexpr int PER = (SMP_BUF + 31) / 32;
  unsigned keys[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    keys[i] = (e < n) ? buf[e] : 0u;
  }
  __syncwarp();
  unsigned winner = 0;
  int thr = -128;
  for (int rnd = 0; rnd < K; ++rnd) {
    unsigned loc = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) loc = max(loc, keys[i]);
    unsigned best = loc;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (best != 0u && loc == best) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (keys[i] == best) keys[i] = 0u;
    }
    if (lane == rnd) winner = best;
    if (rnd == K - 1 && best != 0u) thr = (int)(best >> 22) - 128;
  }
  if (lane < K) buf[lane] = winner;
  __syncwarp();
  *n_kept = min(n, K);
  return thr;
}

__device__ __forceinline__ uint32_t philox4x32_10_first(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                        uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0;
    c1 = n1;
    c2 = n2;
    c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

__global__ void __launch_bounds__(32 * SMP_WARPS) sample_topk_kernel(const ls100_sample_topk_args a) {
  // One CTA per row; the eight warps take every eighth 512-byte chunk of the row (two chunks per warp in flight),
  // each keeps its own k best, warp 0 merges them and draws.
  __shared__ unsigned s_buf[SMP_WARPS][SMP_BUF];
  __shared__ int s_kept[SMP_WARPS];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x;
  const int cur = *a.cur;
  const int K = a.k;
  int32_t* seq = a.seq + (long long)row * a.max_step;
  int token = a.end_id;
  if (seq[cur] != a.end_id) {  // uniform over the CTA
    const int8_t* lp = a.logits + (long long)row * a.ld_logits;
    unsigned* buf = s_buf[warp];
    int n_buf = 0, thr = -128;
    unsigned thr4 = 0x80808080u;
    const int n_chunks = (a.vocab + 511) / 512;
    const int4 none = make_int4((int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080);
    int4 v1 = none, v2 = none;
    if (warp * 512 + lane * 16 < a.vocab) v1 = smp_load16(lp, warp * 512 + lane * 16, a.vocab);
    if ((warp + SMP_WARPS) * 512 + lane * 16 < a.vocab) v2 = smp_load16(lp, (warp + SMP_WARPS) * 512 + lane * 16, a.vocab);
    for (int ch = warp; ch < n_chunks; ch += SMP_WARPS) {
      const int off = ch * 512 + lane * 16;
      const int4 v = v1;
      v1 = v2;
      v2 = none;
      if (off + 2 * SMP_WARPS * 512 < a.vocab) v2 = smp_load16(lp, off + 2 * SMP_WARPS * 512, a.vocab);
      const unsigned w4[4] = {(unsigned)v.x, (unsigned)v.y, (unsigned)v.z, (unsigned)v.w};
      unsigned hit = 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) hit |= __vcmpgts4(w4[w], thr4);
      if (__ballot_sync(0xffffffffu, hit != 0u) != 0u) {
        unsigned qbits = 0;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const unsigned g = __vcmpgts4(w4[w], thr4);
          qbits |= (((g >> 7) & 1u) | ((g >> 14) & 2u) | ((g >> 21) & 4u) | ((g >> 28) & 8u)) << (w * 4);
        }
        const int mine = __popc(qbits);
        int pre = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, pre, o);
          if (lane >= o) pre += t;
        }
        const int total = __shfl_sync(0xffffffffu, pre, 31);
        int pos = n_buf + pre - mine;
        unsigned bits = qbits;
        while (bits) {
          const int bpos = __ffs(bits) - 1;
          bits &= bits - 1;
          const int q = (int)(int8_t)((w4[bpos >> 2] >> ((bpos & 3) * 8)) & 0xff);
          buf[pos++] = ((unsigned)(q + 128) << 22) | (unsigned)(0x3fffff - (off + bpos));
        }
        n_buf += total;
        __syncwarp();
        if (n_buf > 32) {
          thr = smp_flush(buf, n_buf, K, lane, &n_buf);
          thr4 = (unsigned)(thr & 0xff) * 0x01010101u;
        }
      }
    }
    __syncwarp();
    smp_flush(buf, n_buf, K, lane, &n_buf);
    if (lane == 0) s_kept[warp] = n_buf;
    __syncthreads();
    if (warp == 0) {
      int n_all = n_buf;  // warp 0's own list already sits at buf[0 .. n_buf)
      for (int w = 1; w < SMP_WARPS; ++w) {
        const int nk = s_kept[w];
        if (lane < nk) buf[n_all + lane] = s_buf[w][lane];
        n_all += nk;
      }
      __syncwarp();
      smp_flush(buf, n_all, K, lane, &n_buf);
      // softmax over the k kept logits and the draw (lane 0; k <= 8 values)
      if (lane == 0) {
        const int v0 = (int)(buf[0] >> 22) - 128;
        float e[SMP_MAXK];
        float sum = 0.f;
        for (int i = 0; i < n_buf; ++i) {
          const int vi = (int)(buf[i] >> 22) - 128;
          e[i] = expf(__fmul_rn((float)(vi - v0), a.s_logits));
          sum = __fadd_rn(sum, e[i]);
        }
        const uint32_t x = philox4x32_10_first((uint32_t)(cur + 1), (uint32_t)row, 0u, 0u, a.seed_lo, a.seed_hi);
        const float u = __fmul_rn((float)((x >> 8) + 1u), 5.9604644775390625e-8f);  // ((x>>8)+1) * 2^-24 in (0,1]
        float cum = 0.f;
        int pick = n_buf - 1;
        for (int i = 0; i < n_buf; ++i) {
          cum = __fadd_rn(cum, __fdiv_rn(e[i], sum));
          if (u <= cum) {
            pick = i;
            break;
          }
        }
        token = 0x3fffff - (int)(buf[pick] & 0x3fffff);
      }
    }
  }
  if (threadIdx.x == 0) {
    if (cur + 1 < a.max_step) seq[cur + 1] = token;
    if (token == a.end_id) atomicAdd(a.n_ended, 1);
    __threadfence();
    const int ticket = atomicAdd(a.ticket, 1);
    if (ticket == (int)gridDim.x - 1) {
      const int total = atomicAdd(a.n_ended, 0);
      if (total == a.rows) {
        if (atomicCAS(a.stop, -1, cur + 1) == -1 && a.stop_host) *((volatile int*)a.stop_host) = cur + 1;
      }
      *a.n_ended = 0;  // self-cleaning: the next call starts from zero
      *a.ticket = 0;
      __threadfence();
      *a.cur = cur + 1;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Nucleus sampling: CTA per row. Pass 1 builds the 256-bin histogram of the row (one copy per warp in shared
// memory, 16-byte loads); thread 0 walks the levels from the top (at most 255 float additions, in the order
// the contract fixes) to find the cut and the drawn (level, rank); pass 2 finds the rank-th token of that level
// in token order with per-thread segment counts and a scan.
constexpr int TOPP_THREADS = 128;

// smallest j in [1, n] with c + float(j) * w >= t (n if there is none): closed form, then the exact predicate
__device__ __forceinline__ int topp_rank(float c, float w, int n, float t) {
  int j = (int)ceilf(__fdiv_rn(__fsub_rn(t, c), w));
  j = max(1, min(n, j));
  while (j > 1 && __fadd_rn(c, __fmul_rn((float)(j - 1), w)) >= t) --j;
  while (j < n && __fadd_rn(c, __fmul_rn((float)j, w)) < t) ++j;
  return j;
}

__global__ void __launch_bounds__(TOPP_THREADS) sample_topp_kernel(const ls100_sample_topp_args a) {
  __shared__ int s_hist[TOPP_THREADS / 32][256];
  __shared__ int s_cnt[256];
  __shared__ int s_seg[TOPP_THREADS];
  __shared__ int s_level, s_rank, s_token;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = blockIdx.x;
  const int cur = *a.cur;
  int32_t* seq = a.seq + (long long)row * a.max_step;
  const bool ended = seq[cur] == a.end_id;  // uniform over the CTA
  if (tid == 0) s_token = a.end_id;
  if (!ended) {
    const int8_t* lp = a.logits + (long long)row * a.ld_logits;
    for (int i = tid; i < (TOPP_THREADS / 32) * 256; i += TOPP_THREADS) (&s_hist[0][0])[i] = 0;
    __syncthreads();
    for (int off = tid * 16; off < a.vocab; off += TOPP_THREADS * 16) {
      const int4 v = smp_load16(lp, off, a.vocab);  // beyond the vocabulary: -128, a level no logit takes
      const unsigned w4[4] = {(unsigned)v.x, (unsigned)v.y, (unsigned)v.z, (unsigned)v.w};
#pragma unroll
      for (int j = 0; j < 16; ++j) atomicAdd(&s_hist[warp][((w4[j >> 2] >> ((j & 3) * 8)) & 0xff) ^ 0x80], 1);
    }
    __syncthreads();
    for (int b = tid; b < 256; b += TOPP_THREADS) {  // bin b holds level b - 128
      int c = 0;
#pragma unroll
      for (int w = 0; w < TOPP_THREADS / 32; ++w) c += s_hist[w][b];
      s_cnt[b] = (b == 0) ? 0 : c;  // level -128 is padding
    }
    __syncthreads();
    if (tid == 0) {
      int top = 255;
      while (top > 0 && s_cnt[top] == 0) --top;
      float total = 0.f;
      for (int b = top; b >= 1; --b)
        if (s_cnt[b]) total = __fadd_rn(total, __fmul_rn((float)s_cnt[b], expf(__fmul_rn((float)(b - top), a.s_logits))));
      const float cut = __fmul_rn(a.p, total);
      // the nucleus: levels above cut_b whole, cut_n tokens of level cut_b
      int cut_b = 1, cut_n = s_cnt[1];
      float c = 0.f, mass = total;
      for (int b = top; b >= 1; --b) {
        if (!s_cnt[b]) continue;
        const float w = expf(__fmul_rn((float)(b - top), a.s_logits));
        const float m = __fmul_rn((float)s_cnt[b], w);
        cut_b = b;
        cut_n = s_cnt[b];
        if (__fadd_rn(c, m) >= cut) {
          cut_n = topp_rank(c, w, s_cnt[b], cut);
          mass = __fadd_rn(c, __fmul_rn((float)cut_n, w));
          break;
        }
        c = __fadd_rn(c, m);
        mass = c;
      }
      const uint32_t x = philox4x32_10_first((uint32_t)(cur + 1), (uint32_t)row, 0u, 0u, a.seed_lo, a.seed_hi);
      const float u = __fmul_rn((float)((x >> 8) + 1u), 5.9604644775390625e-8f);
      const float target = __fmul_rn(u, mass);
      int lvl = cut_b, rank = cut_n;
      c = 0.f;
      for (int b = top; b >= cut_b; --b) {
        if (!s_cnt[b]) continue;
        const int n = (b == cut_b) ? cut_n : s_cnt[b];
        const float w = expf(__fmul_rn((float)(b - top), a.s_logits));
        const float m = __fmul_rn((float)n, w);
        if (b == cut_b || __fadd_rn(c, m) >= target) {
          lvl = b;
          rank = topp_rank(c, w, n, target);
          break;
        }
        c = __fadd_rn(c, m);
      }
      s_level = lvl - 128;
      s_rank = rank;
    }
    __syncthreads();
    // the rank-th token (1-based, ascending id) whose logit is s_level
    const int level = s_level, rank = s_rank;
    const int seg = (a.vocab + TOPP_THREADS - 1) / TOPP_THREADS;
    const int lo = tid * seg, hi = min(a.vocab, lo + seg);
    int mine = 0;
    for (int i = lo; i < hi; ++i) mine += ((int)lp[i] == level);
    s_seg[tid] = mine;
    __syncthreads();
    if (tid == 0) {
      int before = 0, t = 0;
      while (t < TOPP_THREADS - 1 && before + s_seg[t] < rank) before += s_seg[t++];
      s_seg[0] = t;         // the segment that holds the token
      s_rank = rank - before;  // its rank inside that segment
    }
    __syncthreads();
    if (tid == s_seg[0]) {
      int left = s_rank, tok = a.end_id;
      for (int i = lo; i < hi; ++i)
        if ((int)lp[i] == level && --left == 0) {
          tok = i;
          break;
        }
      s_token = tok;
    }
    __syncthreads();
  }
  if (tid == 0) {
    const int token = s_token;
    if (cur + 1 < a.max_step) seq[cur + 1] = token;
    if (token == a.end_id) atomicAdd(a.n_ended, 1);
    __threadfence();
    const int ticket = atomicAdd(a.ticket, 1);
    if (ticket == (int)gridDim.x - 1) {
      const int total = atomicAdd(a.n_ended, 0);
      if (total == a.rows) {
        if (atomicCAS(a.stop, -1, cur + 1) == -1 && a.stop_host) *((volatile int*)a.stop_host) = cur + 1;
      }
      *a.n_ended = 0;
      *a.ticket = 0;
      __threadfence();
      *a.cur = cur + 1;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Per-token negative log-likelihood from int8 logits: warp per row, two passes over the row (the second is
// served from L1/L2): the row maximum by SIMD byte max, then the sum of exp(-(q_max - q) * s) through a 255-entry
// table shared by the CTA, so no exponential is evaluated per element.
constexpr int NLL_WARPS = 4;

__global__ void __launch_bounds__(32 * NLL_WARPS) token_nll_kernel(const ls100_token_nll_args a) {
  __shared__ float s_lut[256];
  pdl_launch_dependents();
  for (int d = threadIdx.x; d < 256; d += blockDim.x) s_lut[d] = expf(-__fmul_rn((float)d, a.s_logits));
  pdl_wait();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * NLL_WARPS + warp;
  if (r >= a.rows) return;
  const int flat = a.row0 + r;
  const int b = flat / a.seq, t = flat % a.seq;
  const int8_t* lp = a.logits + (long long)r * a.ld_logits;
  unsigned m4 = 0x80808080u;
  for (int off = lane * 16; off < a.vocab; off += 512) {
    const int4 v = smp_load16(lp, off, a.vocab);
    m4 = __vmaxs4(__vmaxs4(m4, (unsigned)v.x), __vmaxs4((unsigned)v.y, __vmaxs4((unsigned)v.z, (unsigned)v.w)));
  }
  int qmax = max(max((int)(int8_t)(m4 & 0xff), (int)(int8_t)((m4 >> 8) & 0xff)),
                 max((int)(int8_t)((m4 >> 16) & 0xff), (int)(int8_t)(m4 >> 24)));
  qmax = warp_max_i(qmax);
  float sum = 0.f;
  for (int off = lane * 16; off < a.vocab; off += 512) {
    const int4 v = smp_load16(lp, off, a.vocab);
    const unsigned w4[4] = {(unsigned)v.x, (unsigned)v.y, (unsigned)v.z, (unsigned)v.w};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = (int)(int8_t)((w4[j >> 2] >> ((j & 3) * 8)) & 0xff);
      sum += (q == -128) ? 0.f : s_lut[min(255, qmax - q)];  // -128 marks the positions beyond the vocabulary
    }
  }
  sum = warp_sum(sum);
  if (lane == 0) {
    float nll = 0.f;
    if (t + 1 < a.seq) {
      int tgt = a.ids[(long long)b * a.seq + t + 1];
      tgt = min(max(tgt, 0), a.vocab - 1);
      nll = logf(sum) + __fmul_rn((float)(qmax - (int)lp[tgt]), a.s_logits);
    }
    a.nll[flat] = nll;
  }
}

__global__ void __launch_bounds__(128) seq_ppl_kernel(const ls100_seq_ppl_args a) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (b >= a.batch) return;
  const int32_t* ids = a.ids + (long long)b * a.seq;
  int len = 0;
  for (int t = lane; t < a.seq; t += 32) len += (a.pad_id < 0 || ids[t] != a.pad_id) ? 1 : 0;
  len = warp_sum_i(len);
  float s = 0.f;
  for (int t = lane; t < len - 1; t += 32) s += a.nll[(long long)b * a.seq + t];
  s = warp_sum(s);
  if (lane == 0) a.ppl[b] = len > 1 ? s / (float)(len - 1) : 0.f;
}

}  // namespace ls100

extern "C" int ls100_sample_topk(ls100_ctx* ctx, const ls100_sample_topk_args* a, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !a->logits || !a->seq || !a->cur || !a->ticket || !a->n_ended || !a->stop) return LS100_ERR_BAD_ARG;
  if (a->rows <= 0 || a->vocab <= 0 || a->k <= 0 || a->max_step <= 0 || !(a->s_logits > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->k > SMP_MAXK || a->vocab < a->k || a->vocab > (1 << 22)) return LS100_ERR_UNSUPPORTED;
  return ls100_launch(sample_topk_kernel, dim3(a->rows), dim3(32 * SMP_WARPS), 0,
                      (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_sample_topp(ls100_ctx* ctx, const ls100_sample_topp_args* a, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !a->logits || !a->seq || !a->cur || !a->ticket || !a->n_ended || !a->stop) return LS100_ERR_BAD_ARG;
  if (a->rows <= 0 || a->vocab <= 0 || a->max_step <= 0 || !(a->s_logits > 0.f)) return LS100_ERR_BAD_ARG;
  if (!(a->p > 0.f) || a->p > 1.f) return LS100_ERR_BAD_ARG;
  if (a->ld_logits < a->vocab) return LS100_ERR_BAD_ARG;
  return ls100_launch(sample_topp_kernel, dim3(a->rows), dim3(TOPP_THREADS), 0, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_token_nll(ls100_ctx* ctx, const ls100_token_nll_args* a, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !a->logits || !a->ids || !a->nll) return LS100_ERR_BAD_ARG;
  if (a->rows <= 0 || a->row0 < 0 || a->vocab <= 0 || a->batch <= 0 || a->seq <= 0 || !(a->s_logits > 0.f))
    return LS100_ERR_BAD_ARG;
  if ((long long)a->row0 + a->rows > (long long)a->batch * a->seq || a->ld_logits < a->vocab) return LS100_ERR_BAD_ARG;
  return ls100_launch(token_nll_kernel, dim3((a->rows + NLL_WARPS - 1) / NLL_WARPS), dim3(32 * NLL_WARPS), 0,
                      (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_seq_ppl(ls100_ctx* ctx, const ls100_seq_ppl_args* a, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !a->nll || !a->ids || !a->ppl || a->batch <= 0 || a->seq <= 0) return LS100_ERR_BAD_ARG;
  return ls100_launch(seq_ppl_kernel, dim3((a->batch + 3) / 4), dim3(128), 0, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}
