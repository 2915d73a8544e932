// Attention kernels (head_dim 64):
//   attn_self  — full-sequence masked softmax attention reading the QKV GEMM's int8
//                output (encoder, BERT, GPT prefill); online softmax, fp32 math.
//   attn_dec   — one-token decoder self-attention over the int8 KV cache with beam
//                ancestry indirection (no per-step cache permutation), dp4a scores.
//   attn_cross — decoder cross-attention over fp32 encoder keys/values.
// All three quantise their output with the out-projection's input clip-max, so the
// next GEMM consumes int8 directly.
//
// Arithmetic follows MultiheadAttention.forward
// (lightseq/training/ops/pytorch/torch_transformer_layers.py:201-376): q is scaled by
// head_dim^-0.5 before the dot products, masked keys are excluded (the reference fills
// -inf for padding and -1e4 for the causal mask; both give probability 0 in fp32), softmax
// in fp32. Summation order differs from torch's bmm, so outputs agree to rounding, not
// bit for bit; the int8 result can differ by one step on a small fraction of elements.
#include <cstdlib>

#include "common.cuh"
#include "ctx.h"

#ifndef LS100_TRACE
#define LS100_TRACE(slot)
#endif

namespace ls100 {

constexpr int DH = 64;

// 16 int8 -> 16 floats without the conversion unit (16 lanes per clock per SM): flip the sign bits so that the
// bytes order as unsigned, drop each byte into the mantissa of 2^23 with one byte-permute, subtract 2^23 + 128.
__device__ __forceinline__ void unpack16(const int4 v, float (&f)[16]) {
  const unsigned w[4] = {(unsigned)v.x ^ 0x80808080u, (unsigned)v.y ^ 0x80808080u, (unsigned)v.z ^ 0x80808080u,
                         (unsigned)v.w ^ 0x80808080u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i * 4 + 0] = __fsub_rn(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7440)), 8388736.f);
    f[i * 4 + 1] = __fsub_rn(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7441)), 8388736.f);
    f[i * 4 + 2] = __fsub_rn(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7442)), 8388736.f);
    f[i * 4 + 3] = __fsub_rn(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7443)), 8388736.f);
  }
}

// ------------------------------------------------------------------ attn_self
__global__ void __launch_bounds__(64) attn_self_kernel(const ls100_attn_self_args a, const float s_out, const float rs_out) {
  __shared__ __align__(16) float Ks[64][DH];
  __shared__ __align__(16) float Vs[64][DH];
  __shared__ uint8_t msk[64];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int q0 = blockIdx.x * 64;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hidden = a.heads * DH;
  const int i = q0 + tid;
  const bool valid = i < a.seq;
  const float scaling = 0.125f;  // 64^-0.5
  const int8_t* base = a.qkv + (long long)b * a.seq * a.ld_qkv;

  float qf[DH];
  {
    const int8_t* qp = base + (long long)(valid ? i : 0) * a.ld_qkv + h * DH;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float f[16];
      unpack16(*reinterpret_cast<const int4*>(qp + c * 16), f);
#pragma unroll
      for (int j = 0; j < 16; ++j) f[j] = __fmul_rn(f[j], a.s_qkv);
      if (a.bias) {
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const float4 bb = __ldg(reinterpret_cast<const float4*>(a.bias + h * DH + c * 16 + j));
          f[j] = __fadd_rn(f[j], bb.x);
          f[j + 1] = __fadd_rn(f[j + 1], bb.y);
          f[j + 2] = __fadd_rn(f[j + 2], bb.z);
          f[j + 3] = __fadd_rn(f[j + 3], bb.w);
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) qf[c * 16 + j] = __fmul_rn(f[j], scaling);
    }
  }
  if (a.k_cache && valid) {  // GPT prefill: keep this row's int8 k,v for the decode steps
    const int8_t* kp = base + (long long)i * a.ld_qkv + hidden + h * DH;
    const int8_t* vp = kp + hidden;
    int8_t* kc = a.k_cache + (((long long)b * a.heads + h) * a.max_step + i) * DH;
    int8_t* vc = a.v_cache + (((long long)b * a.heads + h) * a.max_step + i) * DH;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      *reinterpret_cast<int4*>(kc + c * 16) = *reinterpret_cast<const int4*>(kp + c * 16);
      *reinterpret_cast<int4*>(vc + c * 16) = *reinterpret_cast<const int4*>(vp + c * 16);
    }
  }

  float acc[DH];
#pragma unroll
  for (int d = 0; d < DH; ++d) acc[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int k_end = a.causal ? min(a.seq, q0 + 64) : a.seq;
  for (int k0 = 0; k0 < k_end; k0 += 64) {
    __syncthreads();
    // cooperative load of 64 key rows and 64 value rows, dequantised to fp32
    for (int id = tid; id < 64 * 4 * 2; id += 64) {
      const int mat = id >> 8, rem = id & 255, row = rem >> 2, part = rem & 3;
      const int key = k0 + row;
      float f[16];
      if (key < a.seq) {
        const int col = (1 + mat) * hidden + h * DH + part * 16;
        unpack16(*reinterpret_cast<const int4*>(base + (long long)key * a.ld_qkv + col), f);
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = __fmul_rn(f[j], a.s_qkv);
        if (a.bias) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 bb = __ldg(reinterpret_cast<const float4*>(a.bias + col + j));
            f[j] = __fadd_rn(f[j], bb.x);
            f[j + 1] = __fadd_rn(f[j + 1], bb.y);
            f[j + 2] = __fadd_rn(f[j + 2], bb.z);
            f[j + 3] = __fadd_rn(f[j + 3], bb.w);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = 0.f;
      }
      float* dst = (mat == 0 ? &Ks[row][0] : &Vs[row][0]) + part * 16;
#pragma unroll
      for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    }
    {
      const int key = k0 + tid;
      uint8_t mk = 1;
      if (key < a.seq) mk = a.pad_mask ? a.pad_mask[(long long)b * a.seq + key] : 0;
      msk[tid] = mk;
    }
    __syncthreads();
    const int nk = min(64, a.seq - k0);
    for (int c0 = 0; c0 < nk; c0 += 16) {
      float sc[16];
      float cm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int kk = c0 + j;
        const int key = k0 + kk;
        float s = -INFINITY;
        if (kk < nk && !msk[kk] && (!a.causal || key <= i)) {
          s = 0.f;
#pragma unroll
          for (int d = 0; d < DH; d += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(&Ks[kk][d]);
            s = fmaf(qf[d], k4.x, s);
            s = fmaf(qf[d + 1], k4.y, s);
            s = fmaf(qf[d + 2], k4.z, s);
            s = fmaf(qf[d + 3], k4.w, s);
          }
        }
        sc[j] = s;
        cm = fmaxf(cm, s);
      }
      if (cm == -INFINITY) continue;
      if (cm > m) {
        const float r = __expf(m - cm);  // m = -inf gives 0
        l *= r;
#pragma unroll
        for (int d = 0; d < DH; ++d) acc[d] *= r;
        m = cm;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (sc[j] == -INFINITY) continue;
        const float p = expf(sc[j] - m);
        l += p;
        const int kk = c0 + j;
#pragma unroll
        for (int d = 0; d < DH; d += 4) {
          const float4 v4 = *reinterpret_cast<const float4*>(&Vs[kk][d]);
          acc[d] = fmaf(p, v4.x, acc[d]);
          acc[d + 1] = fmaf(p, v4.y, acc[d + 1]);
          acc[d + 2] = fmaf(p, v4.z, acc[d + 2]);
          acc[d + 3] = fmaf(p, v4.w, acc[d + 3]);
        }
      }
    }
  }
  if (!valid) return;
  const float inv = (l > 0.f) ? 1.f / l : 0.f;
  int8_t* op = a.out + ((long long)b * a.seq + i) * a.ld_out + h * DH;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 u;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = c * 16 + j * 4;
      w[j] = pack_i8x4(quant_s(clipf(acc[d] * inv, a.amax_out), s_out, rs_out), quant_s(clipf(acc[d + 1] * inv, a.amax_out), s_out, rs_out),
                       quant_s(clipf(acc[d + 2] * inv, a.amax_out), s_out, rs_out),
                       quant_s(clipf(acc[d + 3] * inv, a.amax_out), s_out, rs_out));
    }
    u.x = w[0];
    u.y = w[1];
    u.z = w[2];
    u.w = w[3];
    *reinterpret_cast<uint4*>(op + c * 16) = u;
  }
}

// ------------------------------------------------------------------ attn_dec
// One warp per (row, head). 4 lanes x 16 bytes cover one cached position, so one warp-wide
// load instruction fetches 8 positions (512 B). Keys AND values of 32 positions are requested
// together (8 x 16-byte loads per lane in flight) and folded in with an online softmax, so a
// 100-token history costs 4 memory round trips instead of a key pass plus a value pass. The
// beam-ancestry slots of all positions are fetched into shared memory first so that the cache
// loads do not wait on them.
__global__ void __launch_bounds__(128, 7) attn_dec_kernel(const ls100_attn_dec_args a, const float s_out,
                                                        const float rs_out, const float score_scale) {
  extern __shared__ int slot_all[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wid = blockIdx.x * 4 + warp;
  const bool live = wid < a.rows * a.heads;
  const int r = live ? wid / a.heads : 0, h = live ? wid % a.heads : 0;
  const int hidden = a.heads * DH;
  int* slot_s = slot_all + warp * a.max_step;
  const int g = lane >> 2, c = lane & 3;
  // With a static history the keys and values of the first 32 positions are copied into this warp's shared-memory
  // block while the preceding kernel is still running (cp.async: no register waits for them).
  uint8_t* kv_s = reinterpret_cast<uint8_t*>(slot_all + 4 * a.max_step) + warp * 4096;
  const bool pre = a.history_static != 0 && live;
  if (pre) {
    const int step0 = *a.step_ptr;
    const int32_t* anc0 = a.anc ? a.anc + (long long)r * a.max_step : nullptr;
    const int mine = (anc0 && lane < step0 && lane < a.max_step) ? anc0[lane] : r;  // slot of position `lane`
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int p = u * 8 + g;
      const int slot = __shfl_sync(0xffffffffu, mine, p);
      if (p < step0) {
        const long long o = (long long)slot * a.heads * a.max_step * DH + (long long)h * a.max_step * DH + (long long)p * DH + c * 16;
        cp_async_16(kv_s + p * 64 + c * 16, a.k_cache + o);
        cp_async_16(kv_s + 2048 + p * 64 + c * 16, a.v_cache + o);
      }
    }
    cp_async_commit();
  }
  pdl_wait();
  if (!live) return;
  // Everything the first cache reads wait for is requested in one go: this row's q / k / v, the step counter, and the
  // ancestry slots of the first 128 positions (read whatever the step is: the table row has max_step entries), so that
  // one round trip to the L2 stands before the cache loads instead of three.
  const int8_t* row = a.qkv + (long long)r * a.ld_qkv + h * DH + c * 16;
  const int4 q4 = *reinterpret_cast<const int4*>(row);
  const int4 knew = *reinterpret_cast<const int4*>(row + hidden);
  const int4 vnew = *reinterpret_cast<const int4*>(row + 2 * hidden);
  const int32_t* anc = a.anc ? a.anc + (long long)r * a.max_step : nullptr;
  int anc_pre[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = lane + 32 * i;
    anc_pre[i] = (anc && p < a.max_step) ? anc[p] : r;
  }
  const int step = *a.step_ptr;
  const int L = step + 1;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = lane + 32 * i;
    if (p < L) slot_s[p] = (p < step) ? anc_pre[i] : r;
  }
  for (int p = lane + 128; p < L; p += 32) slot_s[p] = (anc && p < step) ? anc[p] : r;
  const long long own = (((long long)r * a.heads + h) * a.max_step + step) * DH + c * 16;
  if (g == 0) *reinterpret_cast<int4*>(a.k_cache + own) = knew;
  if (g == 1) *reinterpret_cast<int4*>(a.v_cache + own) = vnew;
  __syncwarp();
  const long long head_off = (long long)h * a.max_step * DH + c * 16;
  const long long slot_stride = (long long)a.heads * a.max_step * DH;

  float m = -INFINITY, l = 0.f;
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  if (pre) cp_async_wait_all();
  for (int p0 = 0; p0 < L; p0 += 32) {
    int4 k4[4], v4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int p = p0 + u * 8 + g;
      k4[u] = make_int4(0, 0, 0, 0);
      v4[u] = make_int4(0, 0, 0, 0);
      if (p < step) {
        if (pre && p0 == 0) {  // copied ahead of the grid dependency (this lane reads back the pieces it copied)
          k4[u] = *reinterpret_cast<const int4*>(kv_s + p * 64 + c * 16);
          v4[u] = *reinterpret_cast<const int4*>(kv_s + 2048 + p * 64 + c * 16);
        } else {
          const long long o = slot_s[p] * slot_stride + head_off + (long long)p * DH;
          k4[u] = __ldcs(reinterpret_cast<const int4*>(a.k_cache + o));  // streamed once per step: evict first
          v4[u] = __ldcs(reinterpret_cast<const int4*>(a.v_cache + o));
        }
      } else if (p == step) {
        k4[u] = knew;
        v4[u] = vnew;
      }
    }
    float sv[4];
    float bm = -INFINITY;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int p = p0 + u * 8 + g;
      int dot = __dp4a(q4.x, k4[u].x, 0);
      dot = __dp4a(q4.y, k4[u].y, dot);
      dot = __dp4a(q4.z, k4[u].z, dot);
      dot = __dp4a(q4.w, k4[u].w, dot);
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      sv[u] = (p < L) ? (float)dot * score_scale : -INFINITY;
      bm = fmaxf(bm, sv[u]);
    }
    bm = warp_max(bm);  // p0 < L, so at least one position of the block is valid
    const float m_new = fmaxf(m, bm);
    const float resc = __expf(m - m_new);  // 0 when m = -inf
    l *= resc;
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] *= resc;
    m = m_new;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float w = (sv[u] == -INFINITY) ? 0.f : expf(sv[u] - m);
      if (c == 0) l += w;  // each position is seen by the 4 lanes of its group
      float f[16];
      unpack16(v4[u], f);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = fmaf(w, f[j], acc[j]);
    }
  }
  const float sum = warp_sum(l);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 4);
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 8);
    acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
  }
  if (g == 0) {
    const float f = a.s_kv / sum;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = pack_i8x4(quant_s(clipf(acc[j * 4] * f, a.amax_out), s_out, rs_out), quant_s(clipf(acc[j * 4 + 1] * f, a.amax_out), s_out, rs_out),
                       quant_s(clipf(acc[j * 4 + 2] * f, a.amax_out), s_out, rs_out),
                       quant_s(clipf(acc[j * 4 + 3] * f, a.amax_out), s_out, rs_out));
    uint4 u;
    u.x = w[0];
    u.y = w[1];
    u.z = w[2];
    u.w = w[3];
    *reinterpret_cast<uint4*>(a.out + (long long)r * a.ld_out + h * DH + c * 16) = u;
  }
}

// ------------------------------------------------------------------ attn_cross
// One CTA of four warps per (sentence, head). The head's fp32 keys and values of a 64-key tile are brought into
// shared memory by four TMA box copies (K and V, each as two 128-byte-wide halves of the 64 head dims, 128-byte
// swizzle) issued by one thread. When the caller declares the keys and values static (kv_static: written once per
// request, before the decode kernels), the copies are issued BEFORE the grid-dependency wait, so that they travel
// while the preceding kernel is still running. One tile buffer per CTA (32 KB) instead of a persistent CTA with
// two: residency is what hides the latency of this kernel (its arithmetic is a chain of dependent shuffles and
// small FMAs), and six CTAs per SM hold nearly every (sentence, head) of a decode step at once. Sources longer than
// 64 tokens reuse the buffer tile after tile.
// Every key and value element is read from shared memory ONCE for all beams: each of the four warps owns 16 keys
// of the tile and keeps one accumulator set per beam. Scores: lane = (key, half of the head dims), 16-byte reads
// that are conflict-free under the swizzle, the two halves added by one shuffle. PV: two head dims per lane. The
// warps' partial softmax results (max, sum, weighted values) are merged through shared memory at the end.
constexpr int XT = 64;                 // keys per tile
constexpr int XHALF = XT * 128;        // bytes of one half tile: 64 rows x 128 B
constexpr int XTILE = 4 * XHALF;       // K lo, K hi, V lo, V hi
constexpr int XCTAS_PER_SM = 6;
constexpr int XWARPS = 4;              // 16 keys of a tile each
constexpr int XQ = 72;                 // floats per q row in shared memory: the two 32-float halves 36 apart,
                                       // so that the two addresses a warp reads at once fall into different banks

__device__ __forceinline__ void xattn_issue(uint8_t* buf, uint64_t* bar, const CUtensorMap* tm_k, const CUtensorMap* tm_v,
                                            int item, int t, int heads, int S) {
  // token-major: the head is a 256-byte column window of row b * S + s; head-major (heads == 0 here): row item * S + s
  int x = 0, y = item * S + t * XT;
  if (heads > 0) {
    const int b = item / heads, h = item - b * heads;
    x = h * DH * 4;
    y = b * S + t * XT;
  }
  const uint64_t once = l2_policy_evict_first();  // read once per step: do not displace the weights
  mbar_expect_tx(bar, XTILE);
  tma_load_2d_hint(buf, tm_k, bar, x, y, once);
  tma_load_2d_hint(buf + XHALF, tm_k, bar, x + 128, y, once);
  tma_load_2d_hint(buf + 2 * XHALF, tm_v, bar, x, y, once);
  tma_load_2d_hint(buf + 3 * XHALF, tm_v, bar, x + 128, y, once);
}

template <int NB>  // beams rounded up to 1, 2, 4 or 8
__global__ void __launch_bounds__(32 * XWARPS, NB <= 4 ? XCTAS_PER_SM : 3)
attn_cross_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                  const ls100_attn_cross_args a, const float s_out, const float rs_out, int* err) {
  extern __shared__ uint8_t xs_raw[];
  uint8_t* xs = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(xs_raw) + 1023) & ~(uintptr_t)1023);
  float* qs = reinterpret_cast<float*>(xs + XTILE);      // [NB][XQ]
  float* ps = qs + NB * XQ;                               // [XWARPS][NB][16]
  float* mg = reinterpret_cast<float*>(xs);               // [XWARPS][NB][DH + 2]: the tile buffer, once the tiles are done
  uint64_t* bar = reinterpret_cast<uint64_t*>(ps + XWARPS * NB * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int key = lane & 15, hf = lane >> 4;
  const int S = a.src_len;
  const int tiles = (S + XT - 1) / XT;
  const int tm_heads = a.kv_head_major ? 0 : a.heads;
  const int item = blockIdx.x;
  const int b = item / a.heads, h = item - b * a.heads;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    mbar_init(bar, 1);
    fence_barrier_init();
    if (a.kv_static) xattn_issue(xs, bar, &tm_k, &tm_v, item, 0, tm_heads, S);
  }
  // what does not come from the preceding kernel is read ahead of the wait as well: the padding flag of this lane's
  // key in the first tile (static with the keys) and the query bias
  int pad_first = -1;
  if (a.kv_static) {
    const int kpos0 = warp * 16 + key;
    pad_first = (a.pad_mask && kpos0 < S) ? (int)a.pad_mask[(long long)b * S + kpos0] : (kpos0 < S ? 0 : 1);
  }
  float2 qb_pre = make_float2(0.f, 0.f);
  if (a.bias) qb_pre = __ldg(reinterpret_cast<const float2*>(a.bias + h * DH + lane * 2));
  LS100_TRACE(0);
  pdl_wait();
  LS100_TRACE(1);
  if (threadIdx.x == 0 && !a.kv_static) xattn_issue(xs, bar, &tm_k, &tm_v, item, 0, tm_heads, S);
  // q of this (sentence, head): warp w converts beams w and w + 4 (dims 2*lane, 2*lane+1 live in half (lane >> 4))
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int bm = warp + i * XWARPS;
    if (bm < NB) {
      float q0 = 0.f, q1 = 0.f;
      if (bm < a.beam) {
        const short qraw = *reinterpret_cast<const short*>(a.q + (long long)(b * a.beam + bm) * a.ld_q + h * DH + lane * 2);
        const float2 qb = qb_pre;
        q0 = __fadd_rn(__fmul_rn((float)(int8_t)(qraw & 0xff), a.s_q), qb.x);
        q1 = __fadd_rn(__fmul_rn((float)(int8_t)((qraw >> 8) & 0xff), a.s_q), qb.y);
      }
      float* qd = qs + bm * XQ + (lane >> 4) * 36 + ((lane * 2) & 31);
      qd[0] = __fmul_rn(q0, 0.125f);
      qd[1] = __fmul_rn(q1, 0.125f);
    }
  }
  __syncthreads();  // q and the barrier initialisation visible to every warp

  float m[NB], l[NB], acc[NB][2];
#pragma unroll
  for (int bm = 0; bm < NB; ++bm) {
    m[bm] = -INFINITY;
    l[bm] = 0.f;
    acc[bm][0] = 0.f;
    acc[bm][1] = 0.f;
  }
  bool dead = false;  // a copy never landed: keep meeting the CTA barriers, do no work
  for (int t = 0; t < tiles; ++t) {
    const int t0 = t * XT + warp * 16;       // first key of this warp in the tile
    const int ns = max(0, min(16, S - t0));  // its keys that exist
    const int kpos = t0 + key;
    const int pad_now = (t == 0 && pad_first >= 0) ? pad_first
                        : ((a.pad_mask && kpos < S) ? (int)a.pad_mask[(long long)b * S + kpos] : (kpos < S ? 0 : 1));
    LS100_TRACE(2);
    if (!dead) {
      const bool ok = mbar_wait(bar, (uint32_t)t & 1u);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) atomicExch(err, (int)LS100_ERR_TIMEOUT);
        dead = true;
      }
    }
    LS100_TRACE(3);
    const uint8_t* buf = xs;
    if (!dead && ns > 0) {
      const int j = warp * 16 + key;  // row of the tile
      const bool valid = key < ns && !pad_now;
      // scores of key `key` against every beam: this lane's half of the head dims, then the other half by shuffle
      float s[NB][4];
#pragma unroll
      for (int bm = 0; bm < NB; ++bm) s[bm][0] = s[bm][1] = s[bm][2] = s[bm][3] = 0.f;
      {
        const uint8_t* kr = buf + hf * XHALF + j * 128;
        const float* qr = qs + hf * 36;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float4 k4 = *reinterpret_cast<const float4*>(kr + ((c ^ (j & 7)) << 4));
#pragma unroll
          for (int bm = 0; bm < NB; ++bm) {  // four running sums per beam, two packed pairs
            const float4 q4 = *reinterpret_cast<const float4*>(qr + bm * XQ + c * 4);
            const float2 s01 = f2_fma(make_float2(q4.x, q4.y), make_float2(k4.x, k4.y), make_float2(s[bm][0], s[bm][1]));
            const float2 s23 = f2_fma(make_float2(q4.z, q4.w), make_float2(k4.z, k4.w), make_float2(s[bm][2], s[bm][3]));
            s[bm][0] = s01.x;
            s[bm][1] = s01.y;
            s[bm][2] = s23.x;
            s[bm][3] = s23.y;
          }
        }
      }
      float* pr = ps + warp * NB * 16;
      // partial softmax of the 16 keys for every beam, written stage by stage over the beams so that the
      // shuffle chains of different beams overlap. Lanes 16-31 mirror lanes 0-15 after the first exchange.
      float sv[NB], tmax[NB], ex[NB], es[NB];
#pragma unroll
      for (int bm = 0; bm < NB; ++bm) sv[bm] = (s[bm][0] + s[bm][1]) + (s[bm][2] + s[bm][3]);
#pragma unroll
      for (int bm = 0; bm < NB; ++bm) sv[bm] += __shfl_xor_sync(0xffffffffu, sv[bm], 16);
#pragma unroll
      for (int bm = 0; bm < NB; ++bm) tmax[bm] = sv[bm] = valid ? sv[bm] : -INFINITY;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int bm = 0; bm < NB; ++bm) tmax[bm] = fmaxf(tmax[bm], __shfl_xor_sync(0xffffffffu, tmax[bm], o));
      bool any = false;
#pragma unroll
      for (int bm = 0; bm < NB; ++bm) {
        const float m_new = fmaxf(m[bm], tmax[bm]);
        const float resc = (m[bm] == -INFINITY) ? 0.f : __expf(m[bm] - m_new);
        ex[bm] = es[bm] = (sv[bm] == -INFINITY) ? 0.f : expf(sv[bm] - m_new);
        l[bm] *= resc;
        acc[bm][0] *= resc;
        acc[bm][1] *= resc;
        m[bm] = m_new;
        any = any || (tmax[bm] != -INFINITY);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int bm = 0; bm < NB; ++bm) es[bm] += __shfl_xor_sync(0xffffffffu, es[bm], o);
#pragma unroll
      for (int bm = 0; bm < NB; ++bm) {
        l[bm] += es[bm];
        if (hf == 0) pr[bm * 16 + key] = ex[bm];
      }
      __syncwarp();
      LS100_TRACE(4);
      if (any) {  // otherwise all of this warp's keys are masked (uniform across the warp)
        // dims 2*lane, 2*lane+1: half (lane >> 4), 16-byte chunk ((lane & 15) >> 1), 8-byte offset (lane & 1)
        const uint8_t* vb = buf + (2 + (lane >> 4)) * XHALF + (lane & 1) * 8 + warp * 16 * 128;
        const int vc = (lane & 15) >> 1;
        for (int jj = 0; jj < ns; jj += 4) {  // the probabilities beyond ns are zero
          float2 v[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            v[i] = *reinterpret_cast<const float2*>(vb + (jj + i) * 128 + ((vc ^ ((jj + i) & 7)) << 4));
#pragma unroll
          for (int bm = 0; bm < NB; ++bm) {
            const float4 w4 = *reinterpret_cast<const float4*>(pr + bm * 16 + jj);
            float2 tt = make_float2(acc[bm][0], acc[bm][1]);  // the two head dims of this lane as one packed pair
            tt = f2_fma(f2_set(w4.x), v[0], tt);
            tt = f2_fma(f2_set(w4.y), v[1], tt);
            tt = f2_fma(f2_set(w4.z), v[2], tt);
            tt = f2_fma(f2_set(w4.w), v[3], tt);
            acc[bm][0] = tt.x;
            acc[bm][1] = tt.y;
          }
        }
      }
      __syncwarp();
    }
    LS100_TRACE(5);
    if (t + 1 < tiles) {  // the next tile of a long source goes into the same buffer once every warp has finished with it
      __syncthreads();
      if (threadIdx.x == 0) xattn_issue(xs, bar, &tm_k, &tm_v, item, t + 1, tm_heads, S);
    }
  }
  // merge the four key groups of each beam and write the rows
  __syncthreads();  // every warp has finished reading the last tile: its buffer becomes the merge area
#pragma unroll
  for (int bm = 0; bm < NB; ++bm) {
    float* mp = mg + (warp * NB + bm) * (DH + 2);
    mp[lane * 2] = acc[bm][0];
    mp[lane * 2 + 1] = acc[bm][1];
    if (lane == 0) {
      mp[DH] = m[bm];
      mp[DH + 1] = l[bm];
    }
  }
  __syncthreads();
  for (int bm = warp; bm < a.beam; bm += XWARPS) {
    if (dead) break;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < XWARPS; ++w) mm = fmaxf(mm, mg[(w * NB + bm) * (DH + 2) + DH]);
    float lt = 0.f, o0 = 0.f, o1 = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < XWARPS; ++w) {
        const float* mp = mg + (w * NB + bm) * (DH + 2);
        const float f = (mp[DH] == -INFINITY) ? 0.f : __expf(mp[DH] - mm);
        lt = fmaf(mp[DH + 1], f, lt);
        o0 = fmaf(mp[lane * 2], f, o0);
        o1 = fmaf(mp[lane * 2 + 1], f, o1);
      }
    }
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    const uint32_t pk = pack_i8x4(quant_s(clipf(o0 * inv, a.amax_out), s_out, rs_out),
                                  quant_s(clipf(o1 * inv, a.amax_out), s_out, rs_out), 0.f, 0.f);
    *reinterpret_cast<unsigned short*>(a.out + (long long)(b * a.beam + bm) * a.ld_out + h * DH + lane * 2) =
        (unsigned short)(pk & 0xffff);
  }
  LS100_TRACE(6);
}

// one tile (reused as the merge area) + q and probabilities + the barrier + slack to align the tile to the swizzle period
static size_t attn_cross_smem(int nb) {
  return XTILE + (size_t)(nb * XQ + XWARPS * nb * 16) * sizeof(float) + 16 + 1024;
}

}  // namespace ls100

namespace ls100 {  // attn_tc.cu
int attn_self_tc_launch(ls100_ctx* ctx, const ls100_attn_self_args* a, cudaStream_t st);
int attn_self_tc_init_device();
}  // namespace ls100

using namespace ls100;

// Opts the cross-attention kernel into its shared-memory size (two K/V tiles) on the current device
// (called once from ls100_ctx_create, never inside a stream capture).
int ls100_attn_init_device() {
  bool ok = cudaFuncSetAttribute(attn_cross_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_cross_smem(1)) == cudaSuccess;
  ok = ok && cudaFuncSetAttribute(attn_cross_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_cross_smem(2)) == cudaSuccess;
  ok = ok && cudaFuncSetAttribute(attn_cross_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_cross_smem(4)) == cudaSuccess;
  ok = ok && cudaFuncSetAttribute(attn_cross_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_cross_smem(8)) == cudaSuccess;
  ok = ok && attn_self_tc_init_device() == LS100_OK;
  return ok ? LS100_OK : LS100_ERR_CUDA;
}

extern "C" int ls100_attn_self(ls100_ctx* ctx, const ls100_attn_self_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->qkv || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->seq <= 0 || a->heads <= 0 || !(a->amax_out > 0.f) || !(a->s_qkv > 0.f)) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->qkv) & 15) || (a->ld_qkv & 15) || (((uintptr_t)a->out) & 15) || (a->ld_out & 15)) return LS100_ERR_ALIGN;
  if (a->ld_qkv < 3 * a->heads * DH || a->ld_out < a->heads * DH) return LS100_ERR_BAD_ARG;
  if ((a->k_cache != nullptr) != (a->v_cache != nullptr)) return LS100_ERR_BAD_ARG;
  if (a->k_cache && (a->bias || a->max_step < a->seq || (((uintptr_t)a->k_cache) & 15) || (((uintptr_t)a->v_cache) & 15)))
    return LS100_ERR_BAD_ARG;
  if (a->heads > 65535 || a->batch > 65535) return LS100_ERR_UNSUPPORTED;
  // tensor-core kernel: pairs of heads, sequences of at least 16 tokens
  static const bool simt_only = getenv("LS100_ATTN_SIMT") != nullptr;
  if (!simt_only && (a->heads & 1) == 0 && a->seq >= 16 && (long long)a->batch * a->seq < (1ll << 31))
    return attn_self_tc_launch(ctx, a, (cudaStream_t)stream_);
  dim3 grid((a->seq + 63) / 64, a->heads, a->batch);
  const float so = a->amax_out / 127.0f;
  return ls100_launch(attn_self_kernel, grid, dim3(64), 0, (cudaStream_t)stream_, *a, so, 1.0f / so) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_attn_dec(ls100_ctx* ctx, const ls100_attn_dec_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->qkv || !a->k_cache || !a->v_cache || !a->step_ptr || !a->out) return LS100_ERR_BAD_ARG;
  if (a->rows <= 0 || a->heads <= 0 || a->max_step <= 0 || !(a->amax_out > 0.f) || !(a->s_kv > 0.f)) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->qkv) & 15) || (a->ld_qkv & 15) || (((uintptr_t)a->out) & 15) || (a->ld_out & 15) ||
      (((uintptr_t)a->k_cache) & 15) || (((uintptr_t)a->v_cache) & 15))
    return LS100_ERR_ALIGN;
  if (a->max_step > 2048) return LS100_ERR_UNSUPPORTED;  // 4 * max_step * 4 + 16384 bytes of shared memory per CTA (48 KB at most)
  const long long warps = (long long)a->rows * a->heads;
  const float score_scale = (a->s_kv * a->s_kv) * 0.125f;
  const float so = a->amax_out / 127.0f;
  // ancestry slots of the four warps + a 4 KB key/value block per warp
  return ls100_launch(attn_dec_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 4 * a->max_step * sizeof(int) + 4 * 4096,
                      (cudaStream_t)stream_, *a, so, 1.0f / so, score_scale) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_attn_cross(ls100_ctx* ctx, const ls100_attn_cross_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->q || !a->k || !a->v || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->src_len <= 0 || a->heads <= 0 || !(a->amax_out > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->beam > 8 || a->src_len > 4096 || a->heads > 65535) return LS100_ERR_UNSUPPORTED;
  if ((((uintptr_t)a->q) & 1) || (a->ld_q & 1) || (((uintptr_t)a->k) & 15) || (((uintptr_t)a->v) & 15) || (!a->kv_head_major && (a->ld_kv & 3)) ||
      (((uintptr_t)a->out) & 1) || (a->ld_out & 1) || (a->bias && (((uintptr_t)a->bias) & 7)))
    return LS100_ERR_ALIGN;
  if (!a->kv_head_major && a->ld_kv < a->heads * DH) return LS100_ERR_BAD_ARG;
  CUtensorMap tk, tv;  // byte views of the fp32 matrices: 128-byte x 64-row boxes
  uint64_t rows = (uint64_t)a->batch * a->src_len, cols = (uint64_t)a->heads * DH * 4, pitch = (uint64_t)a->ld_kv * 4;
  if (a->kv_head_major) {
    rows *= a->heads;
    cols = pitch = DH * 4;
  }
  int rc = ls100_get_tmap_u8(ctx, a->k, rows, cols, pitch, XT, 128, &tk);
  if (rc) return rc;
  rc = ls100_get_tmap_u8(ctx, a->v, rows, cols, pitch, XT, 128, &tv);
  if (rc) return rc;
  const long long items = (long long)a->batch * a->heads;
  if (items > 0x7fffffffLL) return LS100_ERR_UNSUPPORTED;
  dim3 grid((unsigned)items);
  const float so = a->amax_out / 127.0f;
  const cudaStream_t st = (cudaStream_t)stream_;
  const dim3 block(32 * XWARPS);
  cudaError_t e;
  if (a->beam == 1) e = ls100_launch(attn_cross_kernel<1>, grid, block, attn_cross_smem(1), st, tk, tv, *a, so, 1.0f / so, ctx->d_err);
  else if (a->beam == 2) e = ls100_launch(attn_cross_kernel<2>, grid, block, attn_cross_smem(2), st, tk, tv, *a, so, 1.0f / so, ctx->d_err);
  else if (a->beam <= 4) e = ls100_launch(attn_cross_kernel<4>, grid, block, attn_cross_smem(4), st, tk, tv, *a, so, 1.0f / so, ctx->d_err);
  else e = ls100_launch(attn_cross_kernel<8>, grid, block, attn_cross_smem(8), st, tk, tv, *a, so, 1.0f / so, ctx->d_err);
  return e == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}
