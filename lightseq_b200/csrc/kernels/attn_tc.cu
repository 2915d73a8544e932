// Encoder / BERT self-attention on the tensor cores (the same contract as attn_self_kernel in attn.cu; used when the
// number of heads is even and no KV cache is written).
//
// One CTA per (sentence, PAIR of heads, block of 128 queries). Both GEMMs of attention run as tcgen05 MMAs:
//   S = Q . K^T   int8 x int8 -> int32 (kind::i8): exact. Q and K tiles come by TMA straight out of the QKV GEMM's
//                 int8 output; a tile row is 128 bytes = the 64 dims of the two heads, so the proven 128-byte-swizzle
//                 K-major layout applies and each head is a 64-byte K-range of the same tile.
//   O += P . V    bf16 x bf16 -> fp32 (kind::f16): P in [0,1] is split into two bf16 terms (remainder < 2^-17 p),
//                 V (int8) is exact in bf16. Threads write P and V^T into shared memory in the swizzled K-major layout.
// The biases never enter a GEMM: with q = s*Qi + bq, k = s*Ki + bk the score is
//   (q.k)/8 = s^2/8 * (Qi.Ki) + s/8 * (bq.Ki) + terms constant along a query's row (which softmax cancels),
// and out = s * (P.Vi)/sum(P) + bv. Softmax is exact fp32, one thread per query row (no shuffles). Two passes over
// the keys: the first finds each row's maximum (QK^T is cheap), the second accumulates O with that fixed maximum, so
// the accumulator in TMEM never needs rescaling.
// Warps: 0 = TMA + MMA issue (one elected lane), 1 = TMEM allocation, 2-9 = softmax / epilogue (head = (w-2)/4, TMEM
// lane quarter = w % 4). Phases are separated by CTA barriers; every mbarrier wait is bounded.
#include <cuda_bf16.h>

#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr int AT_BQ = 128;  // queries per CTA
constexpr int AT_BK = 64;   // keys per tile
constexpr int AT_THREADS = 320;
// shared memory map (every tile 1024-byte aligned). The raw V tile lands inside the P area: it is transposed into
// AT_VT before the softmax threads write P, and the next V load is issued only after the P.V MMAs have completed.
// 107 KB per CTA, so two CTAs share an SM (and its 512 TMEM columns).
constexpr int AT_Q = 0;                        // [128 q][128 B]  int8, two heads
constexpr int AT_K = AT_Q + AT_BQ * 128;       // [64 keys][128 B]
constexpr int AT_P = AT_K + AT_BK * 128;       // [head][hi|lo][128 q][64 keys bf16 = 128 B]
constexpr int AT_V = AT_P;                     // [64 keys][128 B] raw int8 V, alive until transposed
constexpr int AT_VT = AT_P + 4 * AT_BQ * 128;  // [head][64 dims][64 keys bf16 = 128 B]
constexpr int AT_MISC = AT_VT + 2 * 64 * 128;  // cj[2][64] f32, key mask[64], bq[128] f32, barriers
constexpr int AT_SMEM = AT_MISC + 2048 + 1024;
constexpr int AT_TMEM_COLS = 256;              // S: 2 heads x 64 columns (int32), O: 2 heads x 64 columns (fp32)

__device__ __forceinline__ uint64_t at_desc(uint32_t saddr) {  // K-major, SWIZZLE_128B, 8-row groups 1024 B apart
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// M = 128, N = 64: int8 -> int32, and bf16 -> fp32
__device__ __forceinline__ constexpr uint32_t at_idesc_i8() {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ constexpr uint32_t at_idesc_bf16() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void at_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
// byte offset of (row, byte b of the 128-byte row) in a 128-byte-swizzled tile
__device__ __forceinline__ int at_sw(int row, int b) { return row * 128 + ((((b >> 4) ^ (row & 7))) << 4) + (b & 15); }

struct AttnTcParams {
  ls100_attn_self_args a;
  float s_out, rs_out;
  int* err;
};
// Bounded wait in time rather than in polls (a failed poll may itself suspend the thread for a while): gives up
// after about 0.2 s of SM clock, and the caller then leaves the kernel with the error word set.
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (clock64() - t0 < 400000000ll) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// 16 int8 -> 16 floats through the mantissa of 2^23 (no conversion unit), as in attn.cu
__device__ __forceinline__ void at_unpack16(const int4 v, float (&f)[16]) {
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

__global__ void __launch_bounds__(AT_THREADS, 2) attn_self_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                     const __grid_constant__ CUtensorMap tm_kv,
                                                                     const AttnTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* cj = reinterpret_cast<float*>(smem + AT_MISC);        // [2][64] bias term of the scores of this key tile
  uint8_t* kmask = smem + AT_MISC + 512;                       // [64]    1 = key masked (padding or past the end)
  float* bq = reinterpret_cast<float*>(smem + AT_MISC + 640);  // [128]   query bias of the two heads
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(smem + AT_MISC + 1536);
  uint64_t* bar_mma = bar_tma + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mma + 1);

  const ls100_attn_self_args& a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = blockIdx.x * AT_BQ, hp = blockIdx.y, b = blockIdx.z;
  const int S = a.seq, H = a.heads * 64;
  const int row_base = b * S;

  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_kv);
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, AT_TMEM_COLS);
    tmem_relinquish();
  }
  if (tid >= 64 && tid < 192) bq[tid - 64] = a.bias ? __ldg(a.bias + hp * 128 + (tid - 64)) : 0.f;  // weights: before the wait
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // only now: a dependent grid's CTAs must not take the TMEM columns this CTA still needs
  pdl_wait();

  // softmax / epilogue identity (warps 2..9): one query row of one head per thread
  const int head = (warp - 2) >> 2, quarter = warp & 3;
  const int qrow = quarter * 32 + lane, q_idx = q0 + qrow;
  const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
  const float sc = __fmul_rn(__fmul_rn(a.s_qkv, a.s_qkv), 0.125f), cs = __fmul_rn(a.s_qkv, 0.125f);
  const int k_end = a.causal ? min(S, q0 + AT_BQ) : S;
  const int n_kt = (k_end + AT_BK - 1) / AT_BK;

  uint32_t ph_tma = 0, ph_mma = 0;
  if (tid == 0) {
    mbar_expect_tx(bar_tma, AT_BQ * 128);
    tma_load_2d(smem + AT_Q, &tm_q, bar_tma, hp * 128, row_base + q0);
  }
  bool ok = at_wait(bar_tma, ph_tma);
  ph_tma ^= 1;

  float m_run = -INFINITY, l_run = 0.f;
  bool alive = true;
  for (int pass = 0; pass < 2 && alive; ++pass) {
    for (int kt = 0; kt < n_kt; ++kt) {
      const int k0 = kt * AT_BK;
      // every reader of the previous tile (shared memory and the S columns of TMEM) is done
      alive = __syncthreads_and(ok);
      if (!alive) break;
      if (tid == 0) {
        mbar_expect_tx(bar_tma, pass ? 2 * AT_BK * 128 : AT_BK * 128);
        tma_load_2d(smem + AT_K, &tm_kv, bar_tma, H + hp * 128, row_base + k0);
        if (pass) tma_load_2d(smem + AT_V, &tm_kv, bar_tma, 2 * H + hp * 128, row_base + k0);
      }
      if (tid < 64) {
        const int key = k0 + tid;
        uint8_t mk = 1;
        if (key < S) mk = a.pad_mask ? a.pad_mask[(long long)b * S + key] : 0;
        kmask[tid] = mk;
      }
      ok = at_wait(bar_tma, ph_tma);
      ph_tma ^= 1;
      if (tid == 0) {  // S[head] = Q[head] . K[head]^T : 64 dims = two K = 32 MMAs per head
        tc_fence_after();
        const uint32_t qa = smem_u32(smem + AT_Q), ka = smem_u32(smem + AT_K);
        const uint64_t qd = at_desc(qa), kd = at_desc(ka);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
            tc_mma_i8(tmem_base + (uint32_t)(hh * 64), qd + (uint64_t)((hh * 2 + kk) * 2), kd + (uint64_t)((hh * 2 + kk) * 2),
                      at_idesc_i8(), kk > 0 ? 1u : 0u);
        tc_commit(bar_mma);
      }
      // meanwhile: the bias term s/8 * (bq . Ki) of this tile's scores
      if (tid >= 64 && tid < 192) {
        const int t = tid - 64, hh = t >> 6, key = t & 63;
        float acc = 0.f;
        if (a.bias) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float f[16];
            at_unpack16(*reinterpret_cast<const int4*>(smem + AT_K + at_sw(key, hh * 64 + c * 16)), f);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc = fmaf(bq[hh * 64 + c * 16 + i], f[i], acc);
          }
        }
        cj[t] = __fmul_rn(acc, cs);
      }
      // and, in the second pass, V^T in bf16: task = (key, 16-byte chunk of the two heads' 128 bytes)
      if (pass && tid >= 64) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int task = (tid - 64) + r * 256, key = task & 63, c = task >> 6;  // c in 0..7
          float f[16];
          at_unpack16(*reinterpret_cast<const int4*>(smem + AT_V + at_sw(key, c * 16)), f);
          uint8_t* vt = smem + AT_VT + (c >> 2) * (64 * 128);
          const int d0 = (c & 3) * 16;
#pragma unroll
          for (int i = 0; i < 16; ++i)  // a small integer is exact in bf16: keep the upper half of the float
            *reinterpret_cast<uint16_t*>(vt + at_sw(d0 + i, key * 2)) = (uint16_t)(__float_as_uint(f[i]) >> 16);
        }
      }
      alive = __syncthreads_and(ok);  // cj, kmask (and V^T) are written; raw V is consumed
      if (!alive) break;
      ok = at_wait(bar_mma, ph_mma);
      ph_mma ^= 1;
      tc_fence_after();

      if (warp >= 2) {
        const float* cjh = cj + head * 64;
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(t_lane + (uint32_t)(head * 64 + c0), r);
          tmem_ld_wait();
          float sv[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int kk = c0 + j;
            const bool vis = !kmask[kk] && (!a.causal || k0 + kk <= q_idx);
            // |Qi.Ki| <= 64 * 127^2 < 2^22: int -> float by adding into the mantissa of 1.5 * 2^23
            const float sf = __fsub_rn(__uint_as_float(r[j] + 0x4B400000u), 12582912.f);
            sv[j] = vis ? fmaf(sf, sc, cjh[kk]) : -INFINITY;
          }
          if (pass == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) m_run = fmaxf(m_run, sv[j]);
          } else {
            uint8_t* ph = smem + AT_P + (head * 2) * (AT_BQ * 128);
            uint8_t* pl = ph + AT_BQ * 128;
#pragma unroll
            for (int g = 0; g < 4; ++g) {  // 8 keys = one 16-byte chunk of bf16
              uint32_t hi[4], lo[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float s0 = sv[g * 8 + e * 2], s1 = sv[g * 8 + e * 2 + 1];
                const float p0 = (s0 == -INFINITY) ? 0.f : __expf(s0 - m_run);
                const float p1 = (s1 == -INFINITY) ? 0.f : __expf(s1 - m_run);
                l_run += p0 + p1;
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                const float2 hf = __bfloat1622float2(h2);
                const __nv_bfloat162 l2 = __floats2bfloat162_rn(p0 - hf.x, p1 - hf.y);
                hi[e] = *reinterpret_cast<const uint32_t*>(&h2);
                lo[e] = *reinterpret_cast<const uint32_t*>(&l2);
              }
              const int off = at_sw(qrow, (c0 + g * 8) * 2);
              *reinterpret_cast<uint4*>(ph + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
              *reinterpret_cast<uint4*>(pl + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
          }
        }
      }
      if (pass) {
        fence_proxy_async();  // P and V^T were written by threads; the MMAs read them through the async proxy
        tc_fence_before();
        alive = __syncthreads_and(ok);
        if (!alive) break;
        if (tid == 0) {  // O[head] += P_hi . V + P_lo . V : 64 keys = four K = 16 MMAs per term
          tc_fence_after();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const uint64_t vd = at_desc(smem_u32(smem + AT_VT + hh * (64 * 128)));
#pragma unroll
            for (int term = 0; term < 2; ++term) {
              const uint64_t pd = at_desc(smem_u32(smem + AT_P + (hh * 2 + term) * (AT_BQ * 128)));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                at_mma_bf16(tmem_base + (uint32_t)(128 + hh * 64), pd + (uint64_t)(kk * 2), vd + (uint64_t)(kk * 2), at_idesc_bf16(),
                            (kt > 0 || term > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(bar_mma);
        }
        ok = at_wait(bar_mma, ph_mma);  // P, V^T and the raw-V area may be overwritten after this
        ph_mma ^= 1;
      } else {
        tc_fence_before();  // the S columns are read; ordered before the next tile's MMA by the barrier at the loop top
      }
    }
  }

  // out = s * O / sum(P) + bv -> clip -> int8 (a row with every key masked gives 0, as the SIMT kernel does)
  if (alive) alive = __syncthreads_and(ok);
  if (alive && warp >= 2) {  // whole warps: the TMEM load is warp-collective, only the store is per row
    tc_fence_after();
    const float inv = (l_run > 0.f) ? __fdividef(a.s_qkv, l_run) : 0.f;
    const float bsel = (l_run > 0.f && a.bias) ? 1.f : 0.f;
    const float* bv = a.bias ? a.bias + 2 * H + hp * 128 + head * 64 : nullptr;
    int8_t* op = a.out + ((long long)row_base + q_idx) * a.ld_out + hp * 128 + head * 64;
#pragma unroll 1
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(t_lane + (uint32_t)(128 + head * 64 + c0), r);
      tmem_ld_wait();
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = __fmul_rn(__uint_as_float(r[j * 4 + e]), inv);
          if (bv) x = fmaf(bsel, __ldg(bv + c0 + j * 4 + e), x);
          v[e] = quant_s(clipf(x, a.amax_out), p.s_out, p.rs_out);
        }
        w[j] = pack_i8x4(v[0], v[1], v[2], v[3]);
      }
      if (q_idx < S) {
        *reinterpret_cast<uint4*>(op + c0) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(op + c0 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }
  if (!alive && tid == 0 && p.err) atomicExch(p.err, (int)LS100_ERR_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

int attn_self_tc_init_device() {
  return cudaFuncSetAttribute(attn_self_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM) == cudaSuccess ? LS100_OK
                                                                                                                          : LS100_ERR_CUDA;
}

// Launches the tensor-core kernel; the caller (ls100_attn_self) has validated the arguments and checked that the
// number of heads is even and that no KV cache is requested.
int attn_self_tc_launch(ls100_ctx* ctx, const ls100_attn_self_args* a, cudaStream_t st) {
  const int H = a->heads * 64;
  const uint64_t rows = (uint64_t)a->batch * (uint64_t)a->seq;
  CUtensorMap tq, tkv;  // byte views of the int8 QKV matrix: 128-byte (two heads) x 128-row and x 64-row boxes
  int rc = ls100_get_tmap_u8(ctx, a->qkv, rows, (uint64_t)3 * H, (uint64_t)a->ld_qkv, AT_BQ, 128, &tq);
  if (rc != LS100_OK) return rc;
  rc = ls100_get_tmap_u8(ctx, a->qkv, rows, (uint64_t)3 * H, (uint64_t)a->ld_qkv, AT_BK, 128, &tkv);
  if (rc != LS100_OK) return rc;
  AttnTcParams p;
  p.a = *a;
  p.s_out = a->amax_out / 127.0f;
  p.rs_out = 1.0f / p.s_out;
  p.err = ctx->d_err;
  dim3 grid((a->seq + AT_BQ - 1) / AT_BQ, a->heads / 2, a->batch);
  return ls100_launch(attn_self_tc_kernel, grid, dim3(AT_THREADS), AT_SMEM, st, tq, tkv, p) == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

}  // namespace ls100
