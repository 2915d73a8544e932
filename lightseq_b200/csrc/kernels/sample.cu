// Top-k sampling step for decoder-only generation (QuantGpt): one warp per sequence streams the row of int8
// logits once (16-byte loads, SIMD byte compares against a warp-wide running threshold, candidate buffer in
// shared memory — the same selection as the beam kernel), then lane 0 draws the token with a counter-based
// Philox4x32-10 stream keyed by (seed, row, position), so results do not depend on launch order or history.
// No host round trip: the kernel appends the token, advances the position and records when every row has ended.
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr int SMP_WARPS = 4;
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
  __shared__ unsigned s_buf[SMP_WARPS][SMP_BUF];
  __shared__ int s_ended;
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_ended = 0;
  __syncthreads();
  const int row = blockIdx.x * SMP_WARPS + warp;
  const int cur = *a.cur;
  const int K = a.k;
  if (row < a.rows) {
    int32_t* seq = a.seq + (long long)row * a.max_step;
    int token;
    if (seq[cur] == a.end_id) {
      token = a.end_id;
    } else {
      const int8_t* lp = a.logits + (long long)row * a.ld_logits;
      unsigned* buf = s_buf[warp];
      int n_buf = 0, thr = -128;
      unsigned thr4 = 0x80808080u;
      const int n_chunks = (a.vocab + 511) / 512;
      int4 vnext = make_int4((int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080);
      if (lane * 16 < a.vocab) vnext = smp_load16(lp, lane * 16, a.vocab);
      for (int ch = 0; ch < n_chunks; ++ch) {
        const int off = ch * 512 + lane * 16;
        const int4 v = vnext;
        vnext = make_int4((int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080);
        if (off + 512 < a.vocab) vnext = smp_load16(lp, off + 512, a.vocab);
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
      // softmax over the k kept logits and the draw (lane 0; k <= 8 values)
      token = a.end_id;
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
      token = __shfl_sync(0xffffffffu, token, 0);
    }
    if (lane == 0) {
      if (cur + 1 < a.max_step) seq[cur + 1] = token;
      if (token == a.end_id) atomicAdd(&s_ended, 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(a.n_ended, s_ended);
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

}  // namespace ls100

extern "C" int ls100_sample_topk(ls100_ctx* ctx, const ls100_sample_topk_args* a, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !a->logits || !a->seq || !a->cur || !a->ticket || !a->n_ended || !a->stop) return LS100_ERR_BAD_ARG;
  if (a->rows <= 0 || a->vocab <= 0 || a->k <= 0 || a->max_step <= 0 || !(a->s_logits > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->k > SMP_MAXK || a->vocab < a->k || a->vocab > (1 << 22)) return LS100_ERR_UNSUPPORTED;
  return ls100_launch(sample_topk_kernel, dim3((a->rows + SMP_WARPS - 1) / SMP_WARPS), dim3(32 * SMP_WARPS), 0,
                      (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}
