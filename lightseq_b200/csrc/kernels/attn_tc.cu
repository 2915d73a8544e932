// Encoder / BERT / GPT-prompt self-attention on the tensor cores (the same contract as attn_self_kernel in attn.cu,
// including the optional store of the int8 K/V cache; used when the number of heads is even and the sequence has at
// least 16 tokens).
//
// One CTA per (sentence, PAIR of heads, block of 128 queries). Both GEMMs of attention run as tcgen05 MMAs:
//   S = Q . K^T   int8 x int8 -> int32 (kind::i8): exact. Q and K tiles come by TMA straight out of the QKV GEMM's
//                 int8 output; a tile row is 128 bytes = the 64 dims of the two heads, so the proven 128-byte-swizzle
//                 K-major layout applies and each head is a 64-byte K-range of the same tile.
//   O += P . V    fp16 x fp16 -> fp32 (kind::f16): P in [0,1] is split into two fp16 terms (remainder < 2^-23 p + 2^-25),
//                 V (int8) is exact in fp16. Threads write P and V^T into shared memory in the swizzled K-major layout.
// The biases never enter a GEMM: with q = s*Qi + bq, k = s*Ki + bk the score is
//   (q.k)/8 = s^2/8 * (Qi.Ki) + s/8 * (bq.Ki) + terms constant along a query's row (which softmax cancels),
// and out = s * (P.Vi)/sum(P) + bv. Softmax is exact fp32, one thread per query row (no shuffles), in the log2
// domain (2^x is one instruction) with packed two-lane fp32 arithmetic. Two passes over the keys: the first finds
// each row's maximum (QK^T is cheap), the second accumulates O with that fixed maximum, so the accumulator in TMEM
// never needs rescaling.
// Warps: 0 = issuer (one lane: every TMA load and every MMA), 1 = TMEM allocation and the key-mask words of each
// tile, 2-9 = softmax / epilogue (head = (w-2)/4, TMEM lane quarter = w % 4), which also compute the bias term of the
// scores and convert V. The issuer and the other warps meet only through mbarriers (K landed, scores done, P.V done,
// K tile read, softmax done), warps 1-9 through one named barrier per tile; the K tile of g+1 is fetched while tile
// g's softmax runs, P.V of tile g and the scores of tile g+1 run while the threads prepare tile g+1, and V comes by
// plain 16-byte loads issued at the start of a tile's preparation. Every mbarrier wait is bounded in time.
#include <cuda_fp16.h>

#include "common.cuh"
#include "ctx.h"

// Phase timestamps for experiment builds; compiles to nothing in the library.
#ifndef AT_TRACE
#define AT_TRACE(pass, kt, slot)
#endif

namespace ls100 {

constexpr int AT_BQ = 128;  // queries per CTA
constexpr int AT_BK = 64;   // keys per tile
constexpr int AT_THREADS = 320;
constexpr int AT_SOFTMAX_WARPS = 8;  // warps 2..9
// shared memory map (every tile 1024-byte aligned): 107 KB per CTA, so two CTAs share an SM (and its 512 TMEM columns)
constexpr int AT_Q = 0;                        // [128 q][128 B]  int8, two heads
constexpr int AT_K = AT_Q + AT_BQ * 128;       // [64 keys][128 B]
constexpr int AT_P = AT_K + AT_BK * 128;       // [head][hi|lo][128 q][64 keys fp16 = 128 B]
constexpr int AT_VT = AT_P + 4 * AT_BQ * 128;  // [head][64 dims][64 keys fp16 = 128 B]
constexpr int AT_MISC = AT_VT + 2 * 64 * 128;  // bias terms, key-mask words, bq[128] f32, barriers
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
// M = 128, N = 64: int8 -> int32, and fp16 -> fp32
__device__ __forceinline__ constexpr uint32_t at_idesc_i8() {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ constexpr uint32_t at_idesc_f16() {  // A and B fp16 (format 0), D fp32
  return (1u << 4) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void at_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
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
// Bounded wait, in time rather than in polls (a failed poll may itself suspend the thread for a while): gives up
// after about 0.2 s of SM clock or as soon as another thread of the CTA has given up, and raises the CTA's abort
// flag; the caller then skips its remaining work and the kernel ends with the error word set.
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)  // the clock and the abort flag are looked at once per 32 polls
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag || clock64() - t0 > 400000000ll) {
      *abort_flag = 1;
      return false;
    }
  }
}
// named barrier of warps 1..9 (the mask warp and the softmax warps); the issuer warp never joins it
__device__ __forceinline__ void at_bar_prep() { asm volatile("bar.sync 1, 288;" ::: "memory"); }

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

// 16 int8 -> 16 fp16 (8 packed pairs): the byte plus 128 dropped into the mantissa of 1024 (0x6400), minus 1152; exact
__device__ __forceinline__ void at_unpack16_f16(const int4 v, uint32_t (&h)[8]) {
  const unsigned w[4] = {(unsigned)v.x ^ 0x80808080u, (unsigned)v.y ^ 0x80808080u, (unsigned)v.z ^ 0x80808080u,
                         (unsigned)v.w ^ 0x80808080u};
  const __half2 off = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t a = __byte_perm(w[i], 0x64646464u, 0x4140), b = __byte_perm(w[i], 0x64646464u, 0x4342);
    const __half2 ra = __hsub2(*reinterpret_cast<const __half2*>(&a), off), rb = __hsub2(*reinterpret_cast<const __half2*>(&b), off);
    h[i * 2] = *reinterpret_cast<const uint32_t*>(&ra);
    h[i * 2 + 1] = *reinterpret_cast<const uint32_t*>(&rb);
  }
}

__global__ void __launch_bounds__(AT_THREADS, 2) attn_self_tc_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                                     const __grid_constant__ CUtensorMap tm_kv,
                                                                     const AttnTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* cj = reinterpret_cast<float*>(smem + AT_MISC);                // [2 buffers][2 heads][64] bias term of a tile's scores
  uint32_t* kmw = reinterpret_cast<uint32_t*>(smem + AT_MISC + 1024);  // [2 buffers][2] bit j of word w: key 32 w + j is masked
  float* bq = reinterpret_cast<float*>(smem + AT_MISC + 1088);         // [128] query bias of the two heads
  uint64_t* bar_k = reinterpret_cast<uint64_t*>(smem + AT_MISC + 1600);  // K tile (and, once, the Q tile) has landed
  uint64_t* bar_s = bar_k + 1;                                           // the score MMAs of a tile have completed
  uint64_t* bar_pv = bar_k + 2;                                          // the P.V MMAs of a tile have completed
  uint64_t* bar_b = bar_k + 3;  // one arrival per softmax warp: it has read the K tile (bias term written)
  uint64_t* bar_c = bar_k + 4;  // one arrival per softmax warp: S is in registers, P and V^T are in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_k + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const ls100_attn_self_args& a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = blockIdx.x * AT_BQ, hp = blockIdx.y, b = blockIdx.z;
  const int S = a.seq, H = a.heads * 64;
  const int row_base = b * S;

  if (tid == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_kv);
    mbar_init(bar_k, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_pv, 1);
    mbar_init(bar_b, AT_SOFTMAX_WARPS);
    mbar_init(bar_c, AT_SOFTMAX_WARPS);
    *abort_flag = 0;
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

  const int k_end = a.causal ? min(S, q0 + AT_BQ) : S;
  const int n_kt = (k_end + AT_BK - 1) / AT_BK;
  const int n_g = 2 * n_kt;  // tile visits: pass 0 (row maxima) then pass 1 (P and O)

  if (warp == 0) {
    // ------------------------------------------------------------ issuer: every TMA load and every MMA
    if (lane == 0) {
      const uint64_t q_desc = at_desc(smem_u32(smem + AT_Q)), k_desc = at_desc(smem_u32(smem + AT_K));
      // S[head] = Q[head] . K[head]^T for the K tile in shared memory (64 dims = two K = 32 MMAs per head)
      auto issue_scores = [&]() {
        tc_fence_after();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
            tc_mma_i8(tmem_base + (uint32_t)(hh * 64), q_desc + (uint64_t)((hh * 2 + kk) * 2), k_desc + (uint64_t)((hh * 2 + kk) * 2),
                      at_idesc_i8(), kk > 0 ? 1u : 0u);
        tc_commit(bar_s);
      };
      mbar_expect_tx(bar_k, AT_BQ * 128 + AT_BK * 128);
      tma_load_2d(smem + AT_Q, &tm_q, bar_k, hp * 128, row_base + q0);
      tma_load_2d(smem + AT_K, &tm_kv, bar_k, H + hp * 128, row_base);
      bool ok = at_wait(bar_k, 0, abort_flag);
      if (ok) issue_scores();
      for (int g = 0; g < n_g && ok; ++g) {
        const int pass = g >= n_kt ? 1 : 0, kt = g - pass * n_kt;
        AT_TRACE(pass, kt, 0);
        if (g + 1 < n_g) {  // the K tile is free once its scores are done and the threads have read it: fetch the next
          ok = at_wait(bar_s, (uint32_t)g & 1u, abort_flag) && at_wait(bar_b, (uint32_t)g & 1u, abort_flag);
          if (!ok) break;
          const int kn = (g + 1 >= n_kt) ? g + 1 - n_kt : g + 1;
          mbar_expect_tx(bar_k, AT_BK * 128);
          tma_load_2d(smem + AT_K, &tm_kv, bar_k, H + hp * 128, row_base + kn * AT_BK);
        }
        AT_TRACE(pass, kt, 1);
        ok = at_wait(bar_c, (uint32_t)g & 1u, abort_flag);  // softmax of tile g is done
        if (!ok) break;
        AT_TRACE(pass, kt, 2);
        tc_fence_after();
        if (pass) {  // O[head] += P_hi . V + P_lo . V : 64 keys = four K = 16 MMAs per term
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const uint64_t vd = at_desc(smem_u32(smem + AT_VT + hh * (64 * 128)));
#pragma unroll
            for (int term = 0; term < 2; ++term) {
              const uint64_t pd = at_desc(smem_u32(smem + AT_P + (hh * 2 + term) * (AT_BQ * 128)));
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                at_mma_f16(tmem_base + (uint32_t)(128 + hh * 64), pd + (uint64_t)(kk * 2), vd + (uint64_t)(kk * 2), at_idesc_f16(),
                            (kt > 0 || term > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(bar_pv);
        }
        AT_TRACE(pass, kt, 3);
        if (g + 1 < n_g) {  // scores of the next tile (the S columns are in the threads' registers by now)
          ok = at_wait(bar_k, (uint32_t)(g + 1) & 1u, abort_flag);
          if (ok) issue_scores();
        }
        AT_TRACE(pass, kt, 4);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ key mask of each tile, as two 32-bit words
    for (int g = 0; g < n_g; ++g) {
      const int kt = g >= n_kt ? g - n_kt : g, k0 = kt * AT_BK;
      uint32_t m0 = 1, m1 = 1;
      if (k0 + lane < S) m0 = a.pad_mask ? a.pad_mask[(long long)b * S + k0 + lane] : 0;
      if (k0 + 32 + lane < S) m1 = a.pad_mask ? a.pad_mask[(long long)b * S + k0 + 32 + lane] : 0;
      const uint32_t w0 = __ballot_sync(0xffffffffu, m0 != 0), w1 = __ballot_sync(0xffffffffu, m1 != 0);
      if (lane == 0) {
        kmw[(g & 1) * 2] = w0;
        kmw[(g & 1) * 2 + 1] = w1;
      }
      at_bar_prep();  // with the softmax warps: mask and bias term of tile g are written
    }
  } else {
    // ------------------------------------------------------------ softmax warps (2..9): one query row of one head per thread
    const int idx = tid - 64;
    const int head = (warp - 2) >> 2, quarter = warp & 3;
    const int qrow = quarter * 32 + lane, q_idx = q0 + qrow;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
    // scores are kept in the log2 domain: exp(x) = 2^(x log2 e)
    const float sc = __fmul_rn(__fmul_rn(__fmul_rn(a.s_qkv, a.s_qkv), 0.125f), 1.4426950408889634f);
    const float cs = __fmul_rn(__fmul_rn(a.s_qkv, 0.125f), 1.4426950408889634f);
    if (a.k_cache != nullptr && q_idx < S) {  // GPT prompt: keep this row's int8 K and V of this head for the decode steps
      const int h = hp * 2 + head;
      const int8_t* kp = a.qkv + ((long long)row_base + q_idx) * a.ld_qkv + H + h * 64;
      const int8_t* vp = kp + H;
      const long long co = (((long long)b * a.heads + h) * a.max_step + q_idx) * 64;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<int4*>(a.k_cache + co + c * 16) = __ldg(reinterpret_cast<const int4*>(kp + c * 16));
        *reinterpret_cast<int4*>(a.v_cache + co + c * 16) = __ldg(reinterpret_cast<const int4*>(vp + c * 16));
      }
    }
    float m_run = -INFINITY;
    float2 l2 = make_float2(0.f, 0.f);
    bool ok = true;
    for (int g = 0; g < n_g; ++g) {
      const int pass = g >= n_kt ? 1 : 0, kt = g - pass * n_kt, k0 = kt * AT_BK;
      float* cjb = cj + (g & 1) * 128;
      if (g == n_kt && m_run == -INFINITY) m_run = 0.f;  // a row with every key masked: all P are 0
      AT_TRACE(pass, kt, 0);
      // ---- preparation of tile g (the tensor pipe may still be running P.V of tile g-1 and the scores of tile g)
      int4 vraw[2];
      if (pass) {  // this thread's two 16-byte pieces of the V tile: issued first, used last
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int task = idx + r * 256, key = task & 63, c = task >> 6;  // c in 0..7: 16-byte chunk of the two heads
          vraw[r] = make_int4(0, 0, 0, 0);
          if (k0 + key < S)
            vraw[r] = __ldg(reinterpret_cast<const int4*>(a.qkv + ((long long)row_base + k0 + key) * a.ld_qkv + 2 * H + hp * 128 + c * 16));
        }
      }
      ok = ok && at_wait(bar_k, (uint32_t)g & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {  // bias term s/8 * (bq . Ki): four lanes share a key, 16 dims each
        const int part = idx & 3, key = idx >> 2;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          if (a.bias) {
            float f[16];
            at_unpack16(*reinterpret_cast<const int4*>(smem + AT_K + at_sw(key, hh * 64 + part * 16)), f);
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              const float4 b4 = *reinterpret_cast<const float4*>(bq + hh * 64 + part * 16 + i);
              acc[0] = fmaf(b4.x, f[i], acc[0]);
              acc[1] = fmaf(b4.y, f[i + 1], acc[1]);
              acc[2] = fmaf(b4.z, f[i + 2], acc[2]);
              acc[3] = fmaf(b4.w, f[i + 3], acc[3]);
            }
          }
          float d = (acc[0] + acc[1]) + (acc[2] + acc[3]);
          d += __shfl_xor_sync(0xffffffffu, d, 1);
          d += __shfl_xor_sync(0xffffffffu, d, 2);
          if (part == 0) cjb[hh * 64 + key] = __fmul_rn(d, cs);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_b);  // this warp no longer reads the K tile
      AT_TRACE(pass, kt, 1);
      at_bar_prep();  // mask (warp 1) and bias term of tile g are visible to every softmax thread
      if (ok) ok = at_wait(bar_s, (uint32_t)g & 1u, abort_flag);
      // P.V of the previous tile was issued before these scores, so it has completed as well: this wait returns at once
      // and only keeps every phase of bar_pv observed in order (parities alias two phases apart)
      if (ok && pass && kt > 0) ok = at_wait(bar_pv, (uint32_t)(kt - 1) & 1u, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      AT_TRACE(pass, kt, 2);
      if (ok) {
        tc_fence_after();
        uint64_t vis = ~(((uint64_t)kmw[(g & 1) * 2 + 1] << 32) | (uint64_t)kmw[(g & 1) * 2]);
        if (a.causal) {
          const int d = q_idx - k0;  // keys 0..d of this tile are visible
          vis &= d >= 63 ? ~0ull : (d < 0 ? 0ull : ((2ull << d) - 1ull));
        }
        const float* cjh = cjb + head * 64;
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
          const uint32_t vw = c0 ? (uint32_t)(vis >> 32) : (uint32_t)vis;
          uint32_t r[32];
          tmem_ld32(t_lane + (uint32_t)(head * 64 + c0), r);
          tmem_ld_wait();
          // scores (log2 domain) of 32 keys, two per instruction; in pass 1 the row maximum is already subtracted
          float2 sv[16];
          const float2 sc2 = make_float2(sc, sc), magic2 = make_float2(12582912.f, 12582912.f);
          const float2 mm = make_float2(pass ? m_run : 0.f, pass ? m_run : 0.f);
#pragma unroll
          for (int j4 = 0; j4 < 32; j4 += 4) {
            const float4 c4 = *reinterpret_cast<const float4*>(cjh + c0 + j4);
            // |Qi.Ki| <= 64 * 127^2 < 2^22: int -> float by adding into the mantissa of 1.5 * 2^23
            const float2 fa = f2_sub(make_float2(__uint_as_float(r[j4] + 0x4B400000u), __uint_as_float(r[j4 + 1] + 0x4B400000u)), magic2);
            const float2 fb = f2_sub(make_float2(__uint_as_float(r[j4 + 2] + 0x4B400000u), __uint_as_float(r[j4 + 3] + 0x4B400000u)), magic2);
            sv[j4 / 2] = f2_fma(fa, sc2, f2_sub(make_float2(c4.x, c4.y), mm));
            sv[j4 / 2 + 1] = f2_fma(fb, sc2, f2_sub(make_float2(c4.z, c4.w), mm));
          }
          if (!__all_sync(0xffffffffu, vw == 0xffffffffu)) {  // some key of this half tile is masked for some row of the warp
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (!((vw >> (2 * j)) & 1u)) sv[j].x = -INFINITY;
              if (!((vw >> (2 * j + 1)) & 1u)) sv[j].y = -INFINITY;
            }
          }
          if (pass == 0) {
            float m0 = fmaxf(sv[0].x, sv[0].y), m1 = fmaxf(sv[1].x, sv[1].y);
#pragma unroll
            for (int j = 2; j < 16; j += 2) {
              m0 = fmaxf(m0, fmaxf(sv[j].x, sv[j].y));
              m1 = fmaxf(m1, fmaxf(sv[j + 1].x, sv[j + 1].y));
            }
            m_run = fmaxf(m_run, fmaxf(m0, m1));
          } else {
            uint8_t* ph = smem + AT_P + (head * 2) * (AT_BQ * 128);
            uint8_t* pl = ph + AT_BQ * 128;
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {  // 8 keys = one 16-byte chunk of fp16
              uint32_t hi[4], lo[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 pp = make_float2(ex2_approx(sv[gq * 4 + e].x), ex2_approx(sv[gq * 4 + e].y));  // 2^-inf = 0
                l2 = f2_add(l2, pp);
                // hi = fp16(p), lo = fp16(p - hi): |p - hi - lo| < 2^-23 p + 2^-25 (p <= 1, so lo may be subnormal)
                const __half2 h2 = __floats2half2_rn(pp.x, pp.y);
                const float2 rem = f2_sub(pp, __half22float2(h2));
                const __half2 lo2 = __floats2half2_rn(rem.x, rem.y);
                hi[e] = *reinterpret_cast<const uint32_t*>(&h2);
                lo[e] = *reinterpret_cast<const uint32_t*>(&lo2);
              }
              const int off = at_sw(qrow, (c0 + gq * 8) * 2);
              *reinterpret_cast<uint4*>(ph + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
              *reinterpret_cast<uint4*>(pl + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
          }
        }
        if (pass) {  // V^T in fp16, written in the swizzled K-major layout the MMA reads. The scores of this tile were
                     // issued after P.V of the previous tile, so their completion means V^T (and P) are no longer read.
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int task = idx + r * 256, key = task & 63, c = task >> 6;
            uint32_t h[8];
            at_unpack16_f16(vraw[r], h);
            uint8_t* vt = smem + AT_VT + (c >> 2) * (64 * 128);
            const int d0 = (c & 3) * 16;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              *reinterpret_cast<uint16_t*>(vt + at_sw(d0 + 2 * i, key * 2)) = (uint16_t)(h[i] & 0xffffu);
              *reinterpret_cast<uint16_t*>(vt + at_sw(d0 + 2 * i + 1, key * 2)) = (uint16_t)(h[i] >> 16);
            }
          }
          fence_proxy_async();  // P and V^T were written by threads; the MMAs read them through the async proxy
        }
        tc_fence_before();
      }
      AT_TRACE(pass, kt, 3);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_c);  // this warp has S in registers, its P and V^T in shared memory
    }

    const float l_run = l2.x + l2.y;
    // out = s * O / sum(P) + bv -> clip -> int8 (a row with every key masked gives 0, as the SIMT kernel does)
    if (ok) ok = at_wait(bar_pv, (uint32_t)(n_kt - 1) & 1u, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {  // whole warps: the TMEM load is warp-collective, only the store is per row
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
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && p.err) atomicExch(p.err, (int)LS100_ERR_TIMEOUT);
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
// number of heads is even.
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
