// Beam-search step on the device, no host round trip:
//   beam_topk   one CTA per (batch, beam) row: the row of int8 logits is read ONCE into
//               registers (16-byte loads), a 256-bin histogram gives max / log-sum-exp and
//               the value of the k-th largest logit, and the exact top-k by (logit desc,
//               token asc) is emitted with length-normalised scores.
//   beam_update one CTA per batch element: merges beam*beam candidates, rewrites the
//               token history and the KV-cache ancestry table in place (staged through
//               shared memory), updates probabilities/scores, counts finished beams and
//               advances the device-side step counter.
// Bookkeeping follows select_beam_rough_topk_i8I
// (lightseq/inference/kernels/transformerKernels_int8.cc.cu:1690-1844) and
// ker_refresh_result (lightseq/inference/kernels/transformerKernels.cc.cu:1398-1463);
// the rough threshold + global Thrust sort are replaced by an exact selection with a
// fixed tie-break (higher score, lower beam, lower token id).
#include <float.h>

#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr float LOGIT_THRESH_MIN = -64.f;   // lightseq/inference/kernels/transformerKernels.h:11
constexpr float MIN_LOG_PROB = -2000.f;     // transformerKernels.h:12
constexpr int MAX_BEAM = 8;

template <int NCH>
__global__ void __launch_bounds__(256) beam_topk_kernel(const ls100_beam_topk_args a) {
  __shared__ int whist[8][256];
  __shared__ int hist[256];
  __shared__ double red[256];
  __shared__ int s_qmax, s_thr, s_need, s_nabove, s_best;
  __shared__ int l_val[MAX_BEAM], l_idx[MAX_BEAM];
  const int t = threadIdx.x, warp = t >> 5;
  const int row = blockIdx.x;
  const int step = *a.step_ptr;
  const int K = a.beam;
  float* cs = a.cand_score + (long long)row * K;
  int32_t* ct = a.cand_token + (long long)row * K;
  if (step != 0 && a.alive[(long long)row * a.max_step + step] == a.end_id) {
    if (t < K) {
      cs[t] = (t == 0) ? a.seq_score[row] : -FLT_MAX;
      ct[t] = a.end_id;
    }
    return;
  }
  for (int i = t; i < 8 * 256; i += 256) (&whist[0][0])[i] = 0;
  if (t == 0) {
    s_qmax = 0;
    s_nabove = 0;
  }
  __syncthreads();
  // ---- the row, once: 16 bytes per load, invalid tail bytes become -128
  const int8_t* lp = a.logits + (long long)row * a.ld_logits;
  int4 reg[NCH];
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int off = (t + 256 * i) * 16;
    int4 v = make_int4((int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080);
    if (off + 16 <= a.vocab) v = *reinterpret_cast<const int4*>(lp + off);
    else if (off < a.vocab) {
      int w[4] = {(int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080};
      for (int j = 0; j < a.vocab - off; ++j) {
        const int byte = (int)(uint8_t)lp[off + j];
        w[j >> 2] = (w[j >> 2] & ~(0xff << ((j & 3) * 8))) | (byte << ((j & 3) * 8));
      }
      v = make_int4(w[0], w[1], w[2], w[3]);
    }
    reg[i] = v;
    const int w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = (int)(int8_t)((w4[j >> 2] >> ((j & 3) * 8)) & 0xff);
      if (q != -128) atomicAdd(&whist[warp][q + 128], 1);
    }
  }
  __syncthreads();
  int cnt = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) cnt += whist[w][t];
  hist[t] = cnt;
  if (cnt > 0) atomicMax(&s_qmax, t);
  __syncthreads();
  const int qmax = s_qmax - 128;
  const float mx = __fmul_rn((float)qmax, a.s_logits);
  {
    const float lg = __fmul_rn((float)(t - 128), a.s_logits);
    const float d = fmaxf(__fsub_rn(lg, mx), LOGIT_THRESH_MIN);
    red[t] = cnt > 0 ? (double)cnt * (double)expf(d) : 0.0;
  }
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (t < s) red[t] += red[t + s];
    __syncthreads();
  }
  if (t == 0) {
    int acc = 0, b = s_qmax;
    for (; b > 0; --b) {
      if (acc + hist[b] >= K) break;
      acc += hist[b];
    }
    s_thr = b - 128;
    s_nabove = 0;
    s_need = K - acc;  // how many tokens of value == thr are taken (lowest ids first)
    s_best = 0x7fffffff;
  }
  __syncthreads();
  const int thr = s_thr;
  // ---- tokens above the threshold value, and a bitmap of tokens equal to it
  uint32_t eq[(NCH * 16 + 31) / 32];
#pragma unroll
  for (int i = 0; i < (NCH * 16 + 31) / 32; ++i) eq[i] = 0;
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int w4[4] = {reg[i].x, reg[i].y, reg[i].z, reg[i].w};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int q = (int)(int8_t)((w4[j >> 2] >> ((j & 3) * 8)) & 0xff);
      if (q == -128) continue;
      if (q > thr) {
        const int slot = atomicAdd(&s_nabove, 1);
        if (slot < MAX_BEAM) {
          l_val[slot] = q;
          l_idx[slot] = (t + 256 * i) * 16 + j;
        }
      } else if (q == thr) {
        eq[(i * 16 + j) >> 5] |= 1u << ((i * 16 + j) & 31);
      }
    }
  }
  __syncthreads();
  const int nabove = s_nabove;
  const int need = s_need;
  int last = -1;
  for (int rnd = 0; rnd < need; ++rnd) {
    // this thread's smallest token id with value == thr and id > last
    int mine = 0x7fffffff;
#pragma unroll
    for (int wv = 0; wv < (NCH * 16 + 31) / 32; ++wv) {
      uint32_t bits = eq[wv];
      while (bits && mine == 0x7fffffff) {
        const int bpos = __ffs(bits) - 1;
        bits &= bits - 1;
        const int pos = wv * 32 + bpos;
        const int idx = (t + 256 * (pos >> 4)) * 16 + (pos & 15);
        if (idx > last) mine = idx;
        else eq[wv] &= ~(1u << bpos);
      }
    }
    if (mine != 0x7fffffff) atomicMin(&s_best, mine);
    __syncthreads();
    last = s_best;
    if (t == 0) {
      l_val[nabove + rnd] = thr;
      l_idx[nabove + rnd] = last;
    }
    __syncthreads();
    if (t == 0) s_best = 0x7fffffff;
    __syncthreads();
  }
  if (t == 0) {
    // order the "above" part by (value desc, token asc); the "equal" part is already in token order
    for (int i = 1; i < nabove; ++i) {
      const int v = l_val[i], x = l_idx[i];
      int j = i - 1;
      while (j >= 0 && (l_val[j] < v || (l_val[j] == v && l_idx[j] > x))) {
        l_val[j + 1] = l_val[j];
        l_idx[j + 1] = l_idx[j];
        --j;
      }
      l_val[j + 1] = v;
      l_idx[j + 1] = x;
    }
    const float lse = logf((float)red[0]);
    const float base = __fsub_rn(__fsub_rn(a.seq_probs[row], lse), mx);
    const float ln = a.length_norm[step];
    const int n = min(K, nabove + need);
    for (int j = 0; j < K; ++j) {
      if (j < n) {
        const float lg = __fmul_rn((float)l_val[j], a.s_logits);
        cs[j] = fmaxf(__fmul_rn(__fadd_rn(lg, base), ln), MIN_LOG_PROB + 1.f);
        ct[j] = l_idx[j];
      } else {
        cs[j] = -FLT_MAX;
        ct[j] = a.end_id;
      }
    }
  }
}

__global__ void __launch_bounds__(128) beam_update_kernel(const ls100_beam_update_args a) {
  extern __shared__ int stage[];  // [2][K][max_step]
  __shared__ int s_parent[MAX_BEAM], s_token[MAX_BEAM];
  __shared__ float s_score[MAX_BEAM];
  const int b = blockIdx.x, t = threadIdx.x;
  const int K = a.beam;
  const int step = *a.step_ptr;
  const int ms = a.max_step;
  int* st_alive = stage;
  int* st_anc = stage + K * ms;
  if (t == 0) {
    // best K of K*K candidates by (score desc, beam asc, token asc)
    const float* cs = a.cand_score + (long long)b * K * K;
    const int32_t* ct = a.cand_token + (long long)b * K * K;
    unsigned long long used = 0ull;
    for (int j = 0; j < K; ++j) {
      int best = -1;
      for (int c = 0; c < K * K; ++c) {
        if (used >> c & 1ull) continue;
        if (best < 0) {
          best = c;
          continue;
        }
        const float sc = cs[c], sb = cs[best];
        if (sc > sb) best = c;  // equal scores keep the earlier (lower beam, then lower-token-first) candidate
        else if (sc == sb && (c / K == best / K) && ct[c] < ct[best]) best = c;
      }
      used |= 1ull << best;
      s_parent[j] = best / K;
      s_token[j] = ct[best];
      s_score[j] = cs[best];
    }
  }
  int* alive_b = a.alive + (long long)b * K * ms;
  int* anc_b = a.anc ? a.anc + (long long)b * K * ms : nullptr;
  for (int i = t; i < K * ms; i += 128) {
    const int p = i % ms;
    if (p <= step) {
      st_alive[i] = alive_b[i];
      if (anc_b) st_anc[i] = anc_b[i];
    }
  }
  __syncthreads();
  for (int i = t; i < K * ms; i += 128) {
    const int j = i / ms, p = i % ms;
    const int par = s_parent[j];
    if (p <= step) {
      alive_b[i] = st_alive[par * ms + p];
      if (anc_b) anc_b[i] = (p < step) ? st_anc[par * ms + p] : (b * K + par);
    } else if (p == step + 1) {
      alive_b[i] = s_token[j];
    }
  }
  if (t == 0) {
    const float ln = a.length_norm[step];
    int fin = 0;
    for (int j = 0; j < K; ++j) {
      a.seq_score[b * K + j] = s_score[j];
      if (s_token[j] != a.end_id) a.seq_probs[b * K + j] = __fdiv_rn(s_score[j], ln);
      else ++fin;
    }
    atomicAdd(a.fin_count + step, fin);
    __threadfence();
    const int ticket = atomicAdd(a.ticket + step, 1);
    if (ticket == (int)gridDim.x - 1) {
      const int total = atomicAdd(a.fin_count + step, 0);
      if (total == (int)gridDim.x * K) {
        if (atomicCAS(a.stop_step, -1, step) == -1 && a.stop_host) *((volatile int*)a.stop_host) = step;
      }
      *a.step_ptr = step + 1;
    }
  }
}

}  // namespace ls100

using namespace ls100;

extern "C" int ls100_beam_topk(ls100_ctx* ctx, const ls100_beam_topk_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->logits || !a->step_ptr || !a->length_norm || !a->alive || !a->seq_probs || !a->seq_score ||
      !a->cand_score || !a->cand_token)
    return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->vocab <= 0 || a->max_step <= 0 || !(a->s_logits > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->beam > MAX_BEAM || a->vocab > 65536 || a->vocab < a->beam) return LS100_ERR_UNSUPPORTED;
  if ((((uintptr_t)a->logits) & 15) || (a->ld_logits & 15)) return LS100_ERR_ALIGN;
  const int rows = a->batch * a->beam;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->vocab <= 32768) beam_topk_kernel<8><<<rows, 256, 0, stream>>>(*a);
  else beam_topk_kernel<16><<<rows, 256, 0, stream>>>(*a);
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

extern "C" int ls100_beam_update(ls100_ctx* ctx, const ls100_beam_update_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->cand_score || !a->cand_token || !a->step_ptr || !a->length_norm || !a->alive || !a->seq_probs ||
      !a->seq_score || !a->fin_count || !a->ticket || !a->stop_step)
    return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->max_step <= 0) return LS100_ERR_BAD_ARG;
  if (a->beam > MAX_BEAM) return LS100_ERR_UNSUPPORTED;
  const size_t smem = (size_t)2 * a->beam * a->max_step * sizeof(int);
  if (smem > 48 * 1024) return LS100_ERR_UNSUPPORTED;
  beam_update_kernel<<<a->batch, 128, smem, (cudaStream_t)stream_>>>(*a);
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}
