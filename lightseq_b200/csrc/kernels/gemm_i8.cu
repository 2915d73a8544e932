// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05.mma
// kind::i8), operands staged by TMA into 128-byte-swizzled shared memory,
// accumulators in TMEM, fused QuantLinear epilogue.
//
// out[M,N] = epilogue(A[M,K] . W[N,K]^T): both operands are K-major, which is
// the torch Linear weight layout, so no load-time transpose is needed.
//
// CTA = one 128 x BN output tile, 10 warps:
//   warp 0     TMA producer (one elected lane)
//   warp 1     TMEM allocator + MMA issuer (one elected lane)
//   warps 2-9  epilogue; warp w reads TMEM lanes 32*(w%4)..+31 (one row per thread), the two warps of a
//              lane quarter take alternate 16-column pieces
// Shared-memory ring of STAGES x (A 128x128 B + W BNx128 B); full/empty
// mbarriers; tcgen05.commit releases a stage when the MMAs that read it retire.
// Epilogue overlap comes from two co-resident CTAs per SM for BN <= 128.
//
// Every wait is bounded: on expiry the thread records LS100_ERR_TIMEOUT in the
// context's device error word and falls through to the common exit, where the
// allocating warp frees TMEM.
//
// Epilogue arithmetic restates QuantLinear.forward
// (lightseq/training/ops/pytorch/quantization.py:50-61) on exact int32
// accumulators; see include/ls100.h for the per-element recipe.
#include <string.h>

#include "common.cuh"
#include "ctx.h"

#ifndef LS100_PTRACE
#define LS100_PTRACE(id)
#endif
#ifndef LS100_TRACE
#define LS100_TRACE(slot)
#endif

namespace ls100 {

struct GemmEpi {
  int m, n, k;
  float s_acc, s_outq, s_req, rs_outq, rs_req;
  const int32_t* w_off;
  const float* bias;
  const float* resid;
  long long ldr;
  int act, out_kind;
  void* out;
  long long ldo;
  int* err;
  // fused LayerNorm + quantise of the fp32 output rows (cluster variant only)
  const float* ln_gamma;
  const float* ln_beta;
  float ln_amax, ln_scale, ln_rs;
  int8_t* ln_out;
  long long ln_ldq;
  // per (row, 64-column group) statistics of an int8 output: largest value and sum of exp((q - 127) * s_outq)
  const uint8_t* table;  // [ceil(n / 256) * 256][256] requantisation table, or null
  int8_t* st_max;
  float* st_sum;
  int st_groups;
  float st_c, st_c127;  // s_outq * log2(e) and -127 times that
};

// Running statistics of one thread's row over the chunks of its column group.
struct EpiStats {
  float sum0, sum1;  // two chains
  unsigned max4;     // four running maxima as packed int8
};

constexpr int BM = 128;
constexpr int BK = 128;  // bytes == int8 elements per k-block (one 128B swizzle row)
constexpr int UMMA_K = 32;

template <int BN, int STAGES, int BMT = 128>
struct GemmSmem {
  static constexpr int A_BYTES = BMT * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int VEC_OFFSET = BAR_OFFSET + 256;          // per-tile bias (fp32) and w_off (int32)
  static constexpr int PART_OFFSET = VEC_OFFSET + BN * 8;      // per row and column group: (sum, sum of squares), fused LayerNorm
  static constexpr int TOTAL = PART_OFFSET + BM * 32 + 1024;   // + alignment slack
};

// Shared-memory matrix descriptor, K-major, SWIZZLE_128B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                   // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                   // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
  return d;
}

template <int BN, int BMT = 128>
__device__ __forceinline__ constexpr uint32_t make_idesc_i8() {
  return (2u << 4)      // D format: s32
         | (1u << 7)    // A: signed 8-bit
         | (1u << 10)   // B: signed 8-bit
         | (0u << 15)   // A K-major
         | (0u << 16)   // B K-major
         | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BMT >> 4) << 24);
}

// Byte offset of 16-byte piece `piece` of row `r` in a 32-row x 64-byte staging block: the four pieces of a row are
// permuted by (r / 2) % 4, which makes both access orders of the epilogues (a lane's own row; eight rows x four
// pieces per instruction) free of bank conflicts without padding.
__device__ __forceinline__ int stage_off(int r, int piece) { return r * 64 + ((piece ^ ((r >> 1) & 3)) << 4); }

__device__ __forceinline__ void record_timeout(int* err) {
  if (err) atomicExch(err, (int)LS100_ERR_TIMEOUT);
}

// NC (32 or 16) consecutive columns of one output row. Written as a sequence of branch-free passes
// over the 32 registers, with the (warp-uniform) mode tests between the passes: a taken
// branch per element costs more than the arithmetic it guards.
template <int NC>
__device__ __forceinline__ void epilogue_acc(const GemmEpi& p, const uint32_t (&r)[NC], const int* s_off, int (&acc)[NC]) {
#pragma unroll
  for (int j = 0; j < NC; ++j) acc[j] = (int)r[j];
  if (p.w_off != nullptr) {
#pragma unroll
    for (int j = 0; j < NC; j += 4) {
      const int4 o = *reinterpret_cast<const int4*>(s_off + j);  // staged in shared memory, zero beyond N
      acc[j] += o.x;
      acc[j + 1] += o.y;
      acc[j + 2] += o.z;
      acc[j + 3] += o.w;
    }
  }
}

// The arithmetic of QuantLinear.forward on NC accumulators of one row (every output kind but raw int32): v[] receives
// the finished fp32 values, or for the int8 kinds the results of quant_biased.
// With `table` (this chunk's first column of a [column][256] table in shared memory, see ls100_gemm_i8_build_table)
// everything after the output quantiser is read instead of computed: the quantised output has 255 values, so bias,
// activation and requantisation are a function of (column, value).
template <int NC>
__device__ __forceinline__ void epilogue_arith(const GemmEpi& p, const int (&acc)[NC], int row, int col0,
                                               const float* s_bias, const float (&rr)[NC], bool rr_valid, float (&v)[NC],
                                               const uint8_t* table = nullptr) {
  const bool row_ok = row < p.m;
  const bool full = (col0 + NC <= p.n);
  // From here on the elements go through the arithmetic two at a time (packed fp32 pairs, every lane rounded as
  // the scalar instruction would): the epilogue is bound by instruction issue.
  bool quantised = false;
  {
    const float2 sa = f2_set(p.s_acc);
#pragma unroll
    for (int j = 0; j < NC; j += 2) {
      const float2 t = f2_mul(make_float2(__int2float_rn(acc[j]), __int2float_rn(acc[j + 1])), sa);
      v[j] = t.x;
      v[j + 1] = t.y;
    }
  }
  if (p.s_outq > 0.f) {
    const float2 so = f2_set(p.s_outq), rso = f2_set(p.rs_outq);
    if (p.out_kind == LS100_OUT_OUTQ_I8 || table != nullptr) {
#pragma unroll
      for (int j = 0; j < NC; j += 2) {
        const float2 t = f2_quant_biased(f2_div_rn(make_float2(v[j], v[j + 1]), so, rso));
        v[j] = t.x;
        v[j + 1] = t.y;
      }
      if (table != nullptr) {
        // the low byte of a biased result is the value as a two's-complement int8; a column's 256 entries start on
        // a 256-byte boundary, so "or" joins base and index
        const uint32_t base = smem_u32(table);
#pragma unroll
        for (int j = 0; j < NC; ++j) {
          const uint32_t addr = (__float_as_uint(v[j]) & 0xffu) | base;
          uint32_t e;
          asm volatile("ld.shared.u8 %0, [%1];" : "=r"(e) : "r"(addr + (uint32_t)(j * 256)));
          v[j] = __uint_as_float(e);
        }
        return;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; j += 2) {
        const float2 q = f2_sub(f2_quant_biased(f2_div_rn(make_float2(v[j], v[j + 1]), so, rso)), f2_set(kQuantMagic));
        const float2 t = f2_mul(q, so);
        v[j] = t.x;
        v[j + 1] = t.y;
      }
    }
  }
  if (p.out_kind != LS100_OUT_OUTQ_I8) {
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < NC; j += 4) {
        const float4 b = *reinterpret_cast<const float4*>(s_bias + j);
        const float2 t0 = f2_add(make_float2(v[j], v[j + 1]), make_float2(b.x, b.y));
        const float2 t1 = f2_add(make_float2(v[j + 2], v[j + 3]), make_float2(b.z, b.w));
        v[j] = t0.x;
        v[j + 1] = t0.y;
        v[j + 2] = t1.x;
        v[j + 3] = t1.y;
      }
    }
    if (p.act == LS100_ACT_RELU) {
#pragma unroll
      for (int j = 0; j < NC; ++j) v[j] = fmaxf(v[j], 0.f);
    } else if (p.act == LS100_ACT_GELU) {
      const bool requant = (p.out_kind == LS100_OUT_REQ_S8 || p.out_kind == LS100_OUT_REQ_U8) && p.resid == nullptr;
      if (requant) {
        // GELU and the requantiser in one pass. The fast GELU is good to ~1e-6; that can only change the int8
        // result when gelu(x)/s_req + 0.5 lands very close to an integer. Those rare elements (about one in
        // ten thousand) are redone with the float64 erf the oracle uses, in a second pass so that the common
        // path stays branch-free.
        const float sub = (p.out_kind == LS100_OUT_REQ_U8) ? 127.f : 0.f;
        float q[NC];
        unsigned redo = 0;
        const float2 sr = f2_set(p.s_req), rsr = f2_set(p.rs_req), sub2 = f2_set(sub), magic2 = f2_set(kQuantMagic);
#pragma unroll
        for (int j = 0; j < NC; j += 2) {
          const float2 x = make_float2(v[j], v[j + 1]);
          const float2 g = f2_gelu_fast(x);
          const float2 u = f2_add(f2_sub(f2_div_rn(g, sr, rsr), sub2), f2_set(0.5f));
          const float2 b = f2_add_rd(u, magic2);
          const float2 d = f2_sub(u, f2_sub(b, magic2));  // u - floor(u), in [0, 1)
          // |gelu_fast - gelu| <= 0.5|x| * 5e-7 (erf approximation + ex2/rcp error) + a few ulp of g; in
          // quantisation units that is the first two terms, the third covers the rounding of u itself.
          const float2 au = f2_abs(u);
          const float2 tol = f2_fma(f2_mul(f2_abs(x), rsr), f2_set(1e-6f), f2_fma(au, f2_set(2e-6f), f2_set(4e-6f)));
          const float2 dist = f2_abs(f2_sub(d, f2_set(0.5f)));
          const float2 lim = f2_sub(f2_set(0.5f), tol);
          const bool near0 = au.x < 200.f && dist.x > lim.x, near1 = au.y < 200.f && dist.y > lim.y;
          redo |= (near0 ? (1u << j) : 0u) | (near1 ? (2u << j) : 0u);
          q[j] = fminf(fmaxf(b.x, kQuantMagic - 127.f), kQuantMagic + 127.f);
          q[j + 1] = fminf(fmaxf(b.y, kQuantMagic - 127.f), kQuantMagic + 127.f);
        }
        if (redo) {
#pragma unroll
          for (int j = 0; j < NC; ++j)
            if (redo & (1u << j))
              q[j] = quant_biased(__fsub_rn(div_rn(gelu_erf_exact(v[j]), p.s_req, p.rs_req), sub));
        }
#pragma unroll
        for (int j = 0; j < NC; ++j) v[j] = q[j];
        quantised = true;
      } else {
#pragma unroll
        for (int j = 0; j < NC; ++j) v[j] = gelu_erf_exact(v[j]);
      }
    }
    if (p.resid != nullptr && row_ok) {
      if (rr_valid) {  // prefetched before the accumulator was ready
#pragma unroll
        for (int j = 0; j < NC; j += 2) {
          const float2 t = f2_add(make_float2(v[j], v[j + 1]), make_float2(rr[j], rr[j + 1]));
          v[j] = t.x;
          v[j + 1] = t.y;
        }
      } else {
        const float* rp = p.resid + (long long)row * p.ldr + col0;
        if (full && ((p.ldr & 3) == 0) && ((((uintptr_t)p.resid) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < NC; j += 4) {
            const float4 t = *reinterpret_cast<const float4*>(rp + j);
            const float2 t0 = f2_add(make_float2(v[j], v[j + 1]), make_float2(t.x, t.y));
            const float2 t1 = f2_add(make_float2(v[j + 2], v[j + 3]), make_float2(t.z, t.w));
            v[j] = t0.x;
            v[j + 1] = t0.y;
            v[j + 2] = t1.x;
            v[j + 3] = t1.y;
          }
        } else {
#pragma unroll
          for (int j = 0; j < NC; ++j)
            if (col0 + j < p.n) v[j] = __fadd_rn(v[j], rp[j]);
        }
      }
    }
    if (quantised) {
    } else if (p.out_kind == LS100_OUT_REQ_S8 || p.out_kind == LS100_OUT_REQ_U8) {
      const float2 sr = f2_set(p.s_req), rsr = f2_set(p.rs_req), sub2 = f2_set(p.out_kind == LS100_OUT_REQ_U8 ? 127.f : 0.f);
#pragma unroll
      for (int j = 0; j < NC; j += 2) {  // x - 0 is x: one form serves the signed and the unsigned quantiser
        const float2 t = f2_quant_biased(f2_sub(f2_div_rn(make_float2(v[j], v[j + 1]), sr, rsr), sub2));
        v[j] = t.x;
        v[j + 1] = t.y;
      }
    }
  }
}

// NC (32 or 16) consecutive columns of one output row: arithmetic, then the stores of this thread's own row.
template <int BN, int NC = 32>
__device__ __forceinline__ void epilogue_chunk(const GemmEpi& p, const uint32_t (&r)[NC], int row, int col0,
                                               const float* s_bias, const int* s_off, const float (&rr)[NC],
                                               bool rr_valid, double* row_sum = nullptr, double* row_sq = nullptr,
                                               EpiStats* stats = nullptr, const uint8_t* table = nullptr) {
  const bool row_ok = row < p.m;
  const bool full = (col0 + NC <= p.n);
  int acc[NC];
  epilogue_acc<NC>(p, r, s_off, acc);
  if (p.out_kind == LS100_OUT_I32) {
    if (!row_ok) return;
    int* op = reinterpret_cast<int*>(p.out) + (long long)row * p.ldo + col0;
    if (full && ((p.ldo & 3) == 0) && ((((uintptr_t)p.out) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < NC; j += 4) *reinterpret_cast<int4*>(op + j) = make_int4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (col0 + j < p.n) op[j] = acc[j];
    }
    return;
  }
  float v[NC];
  epilogue_arith<NC>(p, acc, row, col0, s_bias, rr, rr_valid, v, table);
  if (row_sum != nullptr) {  // statistics of the finished fp32 values for the fused LayerNorm
    double s[4] = {0.0, 0.0, 0.0, 0.0}, q[4] = {0.0, 0.0, 0.0, 0.0};  // four chains: fp64 latency, not rate, is the cost
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const double d = (col0 + j < p.n) ? (double)v[j] : 0.0;
      s[j & 3] += d;
      q[j & 3] = fma(d, d, q[j & 3]);
    }
    *row_sum += (s[0] + s[1]) + (s[2] + s[3]);
    *row_sq += (q[0] + q[1]) + (q[2] + q[3]);
  }
  if (!row_ok) return;
  if (p.out_kind == LS100_OUT_F32) {
    float* op = reinterpret_cast<float*>(p.out) + (long long)row * p.ldo + col0;
    if (full && ((p.ldo & 3) == 0) && ((((uintptr_t)p.out) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < NC; j += 4) *reinterpret_cast<float4*>(op + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (col0 + j < p.n) op[j] = v[j];
    }
  } else if (p.out_kind == LS100_OUT_F16) {
    __half* op = reinterpret_cast<__half*>(p.out) + (long long)row * p.ldo + col0;
    if (full && ((p.ldo & 7) == 0) && ((((uintptr_t)p.out) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < NC; j += 8) {
        __half2 h0 = __floats2half2_rn(v[j], v[j + 1]), h1 = __floats2half2_rn(v[j + 2], v[j + 3]);
        __half2 h2 = __floats2half2_rn(v[j + 4], v[j + 5]), h3 = __floats2half2_rn(v[j + 6], v[j + 7]);
        uint4 u;
        u.x = *reinterpret_cast<uint32_t*>(&h0);
        u.y = *reinterpret_cast<uint32_t*>(&h1);
        u.z = *reinterpret_cast<uint32_t*>(&h2);
        u.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(op + j) = u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (col0 + j < p.n) op[j] = __float2half_rn(v[j]);
    }
  } else {  // int8 outputs: v[] holds the results of quant_biased
    if (stats != nullptr) {  // this row's group statistics from the values in registers (columns beyond N do not count)
      const float2 magic2 = f2_set(kQuantMagic), c2 = f2_set(p.st_c), o2 = f2_set(p.st_c127);
#pragma unroll
      for (int j = 0; j < NC; j += 2) {
        const float2 arg = f2_fma(f2_sub(make_float2(v[j], v[j + 1]), magic2), c2, o2);  // (q - 127) * s * log2(e)
        const float e0 = (full || col0 + j < p.n) ? ex2_approx(arg.x) : 0.f;
        const float e1 = (full || col0 + j + 1 < p.n) ? ex2_approx(arg.y) : 0.f;
        stats->sum0 += e0;
        stats->sum1 += e1;
      }
#pragma unroll
      for (int j = 0; j < NC; j += 4) {
        unsigned w = pack_biased_i8x4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (!full) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (col0 + j + e >= p.n) w = (w & ~(0xffu << (8 * e))) | (0x80u << (8 * e));
        }
        stats->max4 = __vmaxs4(stats->max4, w);
      }
    }
    int8_t* op = reinterpret_cast<int8_t*>(p.out) + (long long)row * p.ldo + col0;
    if (full && ((p.ldo & 15) == 0) && ((((uintptr_t)p.out) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < NC; j += 16) {
        uint4 u;
        u.x = pack_biased_i8x4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        u.y = pack_biased_i8x4(v[j + 4], v[j + 5], v[j + 6], v[j + 7]);
        u.z = pack_biased_i8x4(v[j + 8], v[j + 9], v[j + 10], v[j + 11]);
        u.w = pack_biased_i8x4(v[j + 12], v[j + 13], v[j + 14], v[j + 15]);
        *reinterpret_cast<uint4*>(op + j) = u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        if (col0 + j < p.n) op[j] = (int8_t)(__float_as_uint(v[j]) & 0xffu);
    }
  }
}

// LNF: the CTAs of one 128-row block form a thread-block cluster (grid.x CTAs) and finish with LayerNorm + quantise
// of the fp32 rows they have just written: per-row (sum, sum of squares) in float64 are exchanged through
// distributed shared memory, every CTA adds them in rank order (so all agree to the bit), then each thread
// normalises and quantises its own columns. EVERY thread of the cluster meets both cluster barriers on every
// path, including the time-out paths.
// BMT = 64: tiles of 64 rows (an M = 64 MMA: row r of the tile lives in TMEM lane 32 * (r / 16) + r % 16, so every
// lane quarter and every epilogue warp keeps 16 active lanes). Half the activation bytes per CTA and twice the CTAs:
// for the decode-step GEMMs whose grid is otherwise 64 CTAs, what a CTA waits for after the grid dependency is its
// activation tile arriving at the per-SM L2 rate.
template <int BN, int STAGES, bool LNF = false, int BMT = 128>
__global__ void __launch_bounds__(320) gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                         const __grid_constant__ CUtensorMap tma_b,
                                                         const GemmEpi p) {
  static_assert(BMT == 128 || (BMT == 64 && !LNF), "tile heights");
  using SM = GemmSmem<BN, STAGES, BMT>;
  constexpr int ROWS_Q = BMT / 4;  // rows per TMEM lane quarter
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  float* s_bias = reinterpret_cast<float*>(smem + SM::VEC_OFFSET);
  int* s_off = reinterpret_cast<int*>(smem + SM::VEC_OFFSET + BN * 4);

  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * BMT;
  const int num_kb = (p.k + BK - 1) / BK;

  LS100_TRACE(0);
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // dependents may be scheduled only now: a dependent grid's CTAs that landed on this SM earlier could take the TMEM
  // columns this CTA still needs while they wait for this grid to finish
  pdl_launch_dependents();
  LS100_TRACE(1);

  if (warp == 0) {
    if (elect_one()) {
      // First ring fill: the weight tiles do not depend on the previous kernel, so they are requested
      // before the grid-dependency wait; the activation tiles follow it.
      const int n_pre = num_kb < STAGES ? num_kb : STAGES;
      const uint64_t keep = l2_policy_evict_last();  // weights are re-read every step; activations are not
      for (int kb = 0; kb < n_pre; ++kb) {
        uint8_t* sb = smem + kb * SM::STAGE_BYTES + SM::A_BYTES;
        mbar_expect_tx(&full_bar[kb], SM::STAGE_BYTES);
        tma_load_2d_hint(sb, &tma_b, &full_bar[kb], kb * BK, n0, keep);
      }
      pdl_wait();
      for (int kb = 0; kb < n_pre; ++kb) tma_load_2d(smem + kb * SM::STAGE_BYTES, &tma_a, &full_bar[kb], kb * BK, m0);
      uint32_t phase = (n_pre == STAGES) ? 1 : 0;
      int s = (n_pre == STAGES) ? 0 : n_pre;
      for (int kb = n_pre; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty_bar[s], phase ^ 1)) {
          record_timeout(p.err);
          break;
        }
        uint8_t* sa = smem + s * SM::STAGE_BYTES;
        uint8_t* sb = sa + SM::A_BYTES;
        mbar_expect_tx(&full_bar[s], SM::STAGE_BYTES);
        tma_load_2d(sa, &tma_a, &full_bar[s], kb * BK, m0);
        tma_load_2d_hint(sb, &tma_b, &full_bar[s], kb * BK, n0, keep);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8<BN, BMT>();
      uint32_t phase = 0;
      int s = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full_bar[s], phase)) {
          record_timeout(p.err);
          ok = false;
          break;
        }
        tc_fence_after();
        if (kb == 0) { LS100_TRACE(2); }
        const uint32_t sa = smem_u32(smem + s * SM::STAGE_BYTES);
        const uint64_t adesc = make_smem_desc(sa);
        const uint64_t bdesc = make_smem_desc(sa + SM::A_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          // advance 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units
          tc_mma_i8(tmem_base, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                    (kb > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&empty_bar[s]);
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
      if (ok) tc_commit(tmem_full_bar);
      LS100_TRACE(3);
    }
  } else {
    // Eight epilogue warps: warp w reads TMEM lanes 32*(w%4)..+31 (one row per thread); the two warps of a lane
    // quarter take alternate 16-column pieces of the tile, so that two instruction streams per SM sub-partition
    // hide each other's issue latency.
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;
    // lanes beyond the tile's rows of this quarter (BMT = 64: lanes 16..31) get a row no problem has: they compute on
    // zeros and store nothing
    const int row = lane < ROWS_Q ? m0 + quarter * ROWS_Q + lane : 0x7fffffff;
    // While the main loop runs: stage this tile's bias / weight offsets in shared memory and
    // prefetch the residual values of this thread's first piece, so that no global-load latency
    // is left between "accumulator ready" and the stores.
    {
      const int te = threadIdx.x - 64;
      for (int i = te; i < BN; i += 256) {
        const int n = n0 + i;
        s_bias[i] = (p.bias != nullptr && n < p.n) ? __ldg(p.bias + n) : 0.f;
        s_off[i] = (p.w_off != nullptr && n < p.n) ? __ldg(p.w_off + n) : 0;
      }
    }
    pdl_wait();  // the residual (and everything written below) belongs to the chain of kernels before this one
    float rr[16];
    const int c_first = grp * 16;
    const bool rr_ok = p.resid != nullptr && row < p.m && (n0 + c_first + 16 <= p.n) && ((p.ldr & 3) == 0) &&
                       ((((uintptr_t)p.resid) & 15) == 0) && p.out_kind != LS100_OUT_I32 && p.out_kind != LS100_OUT_OUTQ_I8;
    if (rr_ok) {
      const float* rp = p.resid + (long long)row * p.ldr + n0 + c_first;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 t = *reinterpret_cast<const float4*>(rp + j);
        rr[j] = t.x;
        rr[j + 1] = t.y;
        rr[j + 2] = t.z;
        rr[j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) rr[j] = 0.f;
    }
    const bool staged_out = p.out_kind == LS100_OUT_F32 && (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps only
    bool ok = mbar_wait(tmem_full_bar, 0);
    ok = __all_sync(0xffffffffu, ok);
    double ln_s = 0.0, ln_q = 0.0;
    if (!ok) {
      if (lane == 0) record_timeout(p.err);
    } else {
      tc_fence_after();
      LS100_TRACE(4);
#pragma unroll 1
      for (int c0 = c_first; c0 < BN; c0 += 32) {
        if (n0 + c0 >= p.n) break;
        uint32_t r[16];
        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        if (c0 == c_first) { LS100_TRACE(7); }
        if (!LNF && staged_out && n0 + c0 + 16 <= p.n) {
          // fp32 rows leave through a 2 KB block of the (now idle) operand ring: own row in, eight rows x 64 bytes out
          // per instruction, instead of 32 rows x 16 bytes
          int acc[16];
          float v[16];
          epilogue_acc<16>(p, r, s_off + c0, acc);
          epilogue_arith<16>(p, acc, row, n0 + c0, s_bias + c0, rr, rr_ok && c0 == c_first, v);
          uint8_t* stg = smem + (warp - 2) * 2048;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(stg + stage_off(lane, j)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          __syncwarp();
          float* op = reinterpret_cast<float*>(p.out);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int br = 8 * i + (lane >> 2), piece = lane & 3;
            const float4 t = *reinterpret_cast<const float4*>(stg + stage_off(br, piece));
            const int gr = m0 + quarter * ROWS_Q + br;
            if (br < ROWS_Q && gr < p.m) *reinterpret_cast<float4*>(op + (long long)gr * p.ldo + n0 + c0 + piece * 4) = t;
          }
          __syncwarp();
        } else {
          epilogue_chunk<BN, 16>(p, r, row, n0 + c0, s_bias + c0, s_off + c0, rr, rr_ok && c0 == c_first,
                                 LNF ? &ln_s : nullptr, LNF ? &ln_q : nullptr);
        }
        LS100_TRACE(8 + c0 / 32);
      }
    }
    if constexpr (LNF) {
      // this thread's partial sums: slot (row of the tile, column group)
      double* part = reinterpret_cast<double*>(smem + SM::PART_OFFSET) + ((quarter * 32 + lane) * 2 + grp) * 2;
      double* part_row = reinterpret_cast<double*>(smem + SM::PART_OFFSET) + (quarter * 32 + lane) * 4;
      part[0] = ln_s;
      part[1] = ln_q;
      __syncwarp();
      cluster_arrive();
      cluster_wait();
      LS100_TRACE(12);
      double ps[16], pq[16];  // all remote reads in flight together, then added in (rank, group) order in every CTA
#pragma unroll
      for (uint32_t rk = 0; rk < 8; ++rk) {
        const uint32_t src = rk < gridDim.x ? rk : 0u;  // the cluster is the whole grid row (at most 8 CTAs)
        ps[2 * rk] = dsmem_ld_f64(part_row, src);
        pq[2 * rk] = dsmem_ld_f64(part_row + 1, src);
        ps[2 * rk + 1] = dsmem_ld_f64(part_row + 2, src);
        pq[2 * rk + 1] = dsmem_ld_f64(part_row + 3, src);
      }
      double S = 0.0, Q = 0.0;
#pragma unroll
      for (uint32_t rk = 0; rk < 8; ++rk) {
        if (rk < gridDim.x) {
          S += ps[2 * rk] + ps[2 * rk + 1];
          Q += pq[2 * rk] + pq[2 * rk + 1];
        }
      }
      __syncwarp();
      cluster_arrive();  // this thread no longer reads its peers' shared memory
      LS100_TRACE(13);
      if (ok && row < p.m) {
        const double inv_n = 1.0 / (double)p.n;
        const double mean = S * inv_n;
        const double var = fmax(Q * inv_n - mean * mean, 0.0);
        const double rstd = 1.0 / sqrt(var + 1e-5);
        const float* xr = reinterpret_cast<const float*>(p.out) + (long long)row * p.ldo + n0;
        int8_t* qr = p.ln_out + (long long)row * p.ln_ldq + n0;
#pragma unroll 1
        for (int c0 = c_first; c0 < BN; c0 += 32) {  // this thread's own 16-column pieces
          if (n0 + c0 >= p.n) break;
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 x4 = *reinterpret_cast<const float4*>(xr + c0 + j);  // written by this thread above
            const float4 g4 = __ldg(reinterpret_cast<const float4*>(p.ln_gamma + n0 + c0 + j));
            const float4 b4 = __ldg(reinterpret_cast<const float4*>(p.ln_beta + n0 + c0 + j));
            const float y0 = __fadd_rn(__fmul_rn((float)(((double)x4.x - mean) * rstd), g4.x), b4.x);
            const float y1 = __fadd_rn(__fmul_rn((float)(((double)x4.y - mean) * rstd), g4.y), b4.y);
            const float y2 = __fadd_rn(__fmul_rn((float)(((double)x4.z - mean) * rstd), g4.z), b4.z);
            const float y3 = __fadd_rn(__fmul_rn((float)(((double)x4.w - mean) * rstd), g4.w), b4.w);
            pk[j >> 2] = pack_biased_i8x4(quant_s_biased(clipf(y0, p.ln_amax), p.ln_scale, p.ln_rs),
                                          quant_s_biased(clipf(y1, p.ln_amax), p.ln_scale, p.ln_rs),
                                          quant_s_biased(clipf(y2, p.ln_amax), p.ln_scale, p.ln_rs),
                                          quant_s_biased(clipf(y3, p.ln_amax), p.ln_scale, p.ln_rs));
          }
          *reinterpret_cast<uint4*>(qr + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      __syncwarp();
      LS100_TRACE(14);
      cluster_wait();  // no CTA leaves while a peer may still read its partial sums
      LS100_TRACE(15);
    }
  }
  if constexpr (LNF) {
    if (warp < 2) {  // producer and MMA warps only take part in the cluster barriers
      __syncwarp();
      cluster_arrive();
      cluster_wait();
      cluster_arrive();
      cluster_wait();
    }
  }
  LS100_TRACE(5);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  LS100_TRACE(6);
}

// ---------------------------------------------------------------------------------------------
// Persistent variant for problems of many tiles: one CTA per SM walks a static list of 128 x 256
// tiles. The accumulator is double-buffered in TMEM (2 x 256 columns), so the MMAs of tile i+1 run
// while sixteen epilogue warps (four per TMEM lane quarter, 64 of the 256 columns each) drain
// tile i; with K of a few hundred the epilogue is the longer of the two and it is no longer exposed.
//   warp 0     TMA producer, one ring of P_STAGES stages running across tile boundaries
//   warp 1     TMEM allocator + MMA issuer
//   warps 2-17 epilogue
// No barrier couples the epilogue warps to each other: each stages its own bias / offset slice.
// fp32 outputs (and their fp32 residual) go through shared memory: a thread owns one ROW of the accumulator, so its
// own loads and stores touch 32 different lines per instruction, 16 bytes of each, and the L2 sees half-filled
// sectors; instead every warp passes its 32 x 16 piece through a private staging block and moves it with
// instructions that cover eight rows x 64 contiguous bytes (the residual arrives by cp.async, so no register waits
// for it). The staging blocks take the place of the ring's fourth stage (plus a 16 KB tail), so such launches run a
// three-stage ring. Inside a block the four 16-byte pieces of a row are permuted by (row / 2) % 4: both access
// orders, a lane's own row and eight rows x four pieces, are then free of bank conflicts without padding.
constexpr int P_BN = 256;
constexpr int P_STAGES = 4;
constexpr int P_STG_BYTES = 32 * 16 * 4;  // one 32 x 16 fp32 block; every epilogue warp has one for each direction
constexpr int P_EPI_WARPS = 16;
constexpr int P_THREADS = 64 + 32 * P_EPI_WARPS;

struct PersistSmem {
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = P_BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // the fourth stage and a 16 KB tail behind it are one 64 KB area for the modes that run a three-stage ring
  static constexpr int AUX_OFFSET = (P_STAGES - 1) * STAGE_BYTES;
  static constexpr int AUX_BYTES = 65536;
  static constexpr int BAR_OFFSET = AUX_OFFSET + AUX_BYTES;
  static constexpr int VEC_OFFSET = BAR_OFFSET + 256;
  static constexpr int P_COLS = P_BN / (P_EPI_WARPS / 4);  // columns of a tile per epilogue warp: 64
  static constexpr int VEC_PER_WARP = P_COLS * 8;          // 64 fp32 bias + 64 int32 offsets
  static constexpr int TOTAL = VEC_OFFSET + P_EPI_WARPS * VEC_PER_WARP + 1024;
};
static_assert(PersistSmem::AUX_OFFSET + PersistSmem::AUX_BYTES >= P_STAGES * PersistSmem::STAGE_BYTES, "ring inside");
static_assert(PersistSmem::TOTAL <= 232448, "shared memory of one SM");

constexpr int P_PLAIN = 0, P_STAGED = 1, P_TABLE = 2, P_OUTQ = 3;

// The tiles of one CTA. Strided over the row-major tile list by default; with a requantisation table, a contiguous
// run of the column-major list, so that the 256-column slice of the table in shared memory changes once or twice
// per CTA instead of with every tile.
struct TileWalk {
  int first, step, count, tiles_m, tiles_n;
  bool by_column;
  __device__ __forceinline__ TileWalk(bool by_column_, int tiles_n_, int num_tiles) : tiles_n(tiles_n_), by_column(by_column_) {
    tiles_m = num_tiles / tiles_n_;
    if (by_column) {
      first = (int)((long long)blockIdx.x * num_tiles / gridDim.x);
      count = (int)((long long)(blockIdx.x + 1) * num_tiles / gridDim.x) - first;
      step = 1;
    } else {
      first = blockIdx.x;
      step = gridDim.x;
      count = ((int)blockIdx.x < num_tiles) ? (num_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    }
  }
  __device__ __forceinline__ int n_tile(int i) const { const int t = first + i * step; return by_column ? t / tiles_m : t % tiles_n; }
  __device__ __forceinline__ int m_tile(int i) const { const int t = first + i * step; return by_column ? t % tiles_m : t / tiles_n; }
};

template <int MODE>
__global__ void __launch_bounds__(P_THREADS, 1) gemm_i8_persist_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                        const __grid_constant__ CUtensorMap tma_b,
                                                                        const GemmEpi p, int tiles_n, int num_tiles) {
  using SM = PersistSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + P_STAGES;
  uint64_t* tmem_full_bar = empty_bar + P_STAGES;  // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.k + BK - 1) / BK;
  constexpr bool staged = MODE == P_STAGED;  // whole-line movement of fp32 outputs (the launcher checks the alignment)
  constexpr bool tabled = MODE == P_TABLE;    // requantisation table slice in shared memory
  constexpr int stages = (MODE == P_PLAIN || MODE == P_OUTQ) ? P_STAGES : P_STAGES - 1;
  const TileWalk walk(tabled, tiles_n, num_tiles);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
#pragma unroll
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], P_EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * P_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // dependents may be scheduled only now: a dependent grid's CTAs that landed on this SM earlier could take the TMEM
  // columns this CTA still needs while they wait for this grid to finish
  pdl_launch_dependents();

  if (warp == 0) {
    if (elect_one()) {
      // First ring fill: the weight tiles of the first tile do not depend on the previous kernel, so they are
      // requested before the grid-dependency wait (in a chain of launches this hides their trip from HBM); the
      // activation tiles of the same stages follow the wait.
      const int n_pre = walk.count > 0 ? (num_kb < stages ? num_kb : stages) : 0;
      for (int kb = 0; kb < n_pre; ++kb) {
        mbar_expect_tx(&full_bar[kb], SM::STAGE_BYTES);
        tma_load_2d(smem + kb * SM::STAGE_BYTES + SM::A_BYTES, &tma_b, &full_bar[kb], kb * BK, walk.n_tile(0) * P_BN);
      }
      pdl_wait();
      for (int kb = 0; kb < n_pre; ++kb)
        tma_load_2d(smem + kb * SM::STAGE_BYTES, &tma_a, &full_bar[kb], kb * BK, walk.m_tile(0) * BM);
      uint32_t phase = (n_pre == stages) ? 1 : 0;
      int s = (n_pre == stages) ? 0 : n_pre;
      bool ok = true;
      for (int it = 0; it < walk.count && ok; ++it) {
        const int n0 = walk.n_tile(it) * P_BN;
        const int m0 = walk.m_tile(it) * BM;
        for (int kb = (it == 0 ? n_pre : 0); kb < num_kb; ++kb) {
          // a stage that has never been filled reads as released (parity of the phase before the first)
          if (!mbar_wait(&empty_bar[s], phase ^ 1)) {
            record_timeout(p.err);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * SM::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], SM::STAGE_BYTES);
          tma_load_2d(sa, &tma_a, &full_bar[s], kb * BK, m0);
          tma_load_2d(sa + SM::A_BYTES, &tma_b, &full_bar[s], kb * BK, n0);
          if (++s == stages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_i8<P_BN>();
      uint32_t phase = 0;
      int s = 0;
      int local = 0;
      bool ok = true;
      for (; local < walk.count && ok; ++local) {
        const int buf = local & 1;
        if (!mbar_wait(&tmem_empty_bar[buf], ((uint32_t)(local >> 1) & 1u) ^ 1u)) {  // drained by the epilogue
          record_timeout(p.err);
          break;
        }
        tc_fence_after();
        LS100_PTRACE(24);
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * P_BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], phase)) {
            record_timeout(p.err);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * SM::STAGE_BYTES);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + SM::A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            tc_mma_i8(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc,
                      (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[s]);
          if (++s == stages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tmem_full_bar[buf]);
        LS100_PTRACE(25);
      }
    }
  } else {
    constexpr int COLS = SM::P_COLS;
    const int ew = warp - 2;
    const int quarter = warp & 3;  // the TMEM lanes a warp may read are fixed by its index modulo 4
    const int grp = ew >> 2;       // which 64 of the tile's 256 columns
    float* s_bias = reinterpret_cast<float*>(smem + SM::VEC_OFFSET + ew * SM::VEC_PER_WARP);
    int* s_off = reinterpret_cast<int*>(s_bias + COLS);
    float rr[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) rr[j] = 0.f;
    // staged mode: this warp's incoming (residual) and outgoing 32 x 16 blocks, and the (row, 16-byte piece) this
    // lane moves in each of the four instructions that cover a block: rows 8i + lane / 4, piece lane % 4
    uint8_t* stg_in = smem + SM::AUX_OFFSET + ew * P_STG_BYTES;
    uint8_t* stg_out = smem + SM::AUX_OFFSET + (P_EPI_WARPS + ew) * P_STG_BYTES;
    const int mv_row = lane >> 2, mv_piece = lane & 3;
    pdl_wait();  // the residual (and everything written below) belongs to the chain of kernels before this one
    int local = 0;
    bool dead = false;
    int table_tile = -1;  // the column tile whose table slice is in shared memory
    const uint8_t* table_c = nullptr;
    for (; local < walk.count; ++local) {
      const int buf = local & 1;
      const int n0 = walk.n_tile(local) * P_BN + grp * COLS;
      const int row0 = walk.m_tile(local) * BM + quarter * 32;
      const int row = row0 + lane;
      if constexpr (tabled) {
        // All sixteen epilogue warps walk the same tiles, so they meet here together (also the ones that gave up on
        // a wait: a warp that stayed away would leave the others at the barrier for good).
        if (walk.n_tile(local) != table_tile) {
          table_tile = walk.n_tile(local);
          asm volatile("bar.sync 1, %0;" ::"n"(32 * P_EPI_WARPS) : "memory");  // the old slice is no longer read
          const uint8_t* src = p.table + (long long)table_tile * SM::AUX_BYTES;
          for (int i = threadIdx.x - 64; i < SM::AUX_BYTES / 16; i += 32 * P_EPI_WARPS)
            cp_async_16(smem + SM::AUX_OFFSET + i * 16, src + i * 16);
          cp_async_commit();
          cp_async_wait_all();
          asm volatile("bar.sync 1, %0;" ::"n"(32 * P_EPI_WARPS) : "memory");
        }
        table_c = smem + SM::AUX_OFFSET + grp * COLS * 256;
      }
      if (!tabled || p.w_off != nullptr) {  // with a table the bias is inside it
        __syncwarp();
#pragma unroll
        for (int i = lane; i < COLS; i += 32) {
          const int n = n0 + i;
          s_bias[i] = (p.bias != nullptr && n < p.n) ? __ldg(p.bias + n) : 0.f;
          s_off[i] = (p.w_off != nullptr && n < p.n) ? __ldg(p.w_off + n) : 0;
        }
        __syncwarp();
      }
      if (dead) continue;
      LS100_PTRACE(20);
      // the residual of this warp's first piece is requested before the accumulator is waited for
      auto fetch_resid = [&](int c0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int br = 8 * i + mv_row;
          if (row0 + br < p.m)
            cp_async_16(stg_in + stage_off(br, mv_piece), p.resid + (long long)(row0 + br) * p.ldr + n0 + c0 + mv_piece * 4);
        }
        cp_async_commit();
      };
      if constexpr (staged) {
        if (p.resid != nullptr && n0 + 16 <= p.n) fetch_resid(0);
      }
      bool ok = mbar_wait(&tmem_full_bar[buf], (uint32_t)(local >> 1) & 1u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) record_timeout(p.err);
        dead = true;
        continue;
      }
      tc_fence_after();
      LS100_PTRACE(21);
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P_BN + grp * COLS);
      EpiStats stats = {0.f, 0.f, 0x80808080u};
      const bool with_stats = p.st_max != nullptr && p.out_kind == LS100_OUT_OUTQ_I8;
      auto present = [&](int c0) { return c0 < COLS && n0 + c0 < p.n; };
      if (!present(0)) {  // the whole group lies beyond N: nothing to read, release at once
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
      }
      if constexpr (MODE == P_OUTQ) {
        // Output-quantised int8 only (logits, QKV): the epilogue is short enough for a second register set, so the
        // TMEM read of the next piece is in flight during the arithmetic of this one (a read takes ~0.3 us from
        // issue to data, a third of a piece's time). In the general kernel the same loop spilled and lost 40 %.
        GemmEpi q = p;  // the fields this mode fixes, spelled out for the compiler
        q.out_kind = LS100_OUT_OUTQ_I8;
        q.bias = nullptr;
        q.resid = nullptr;
        q.act = LS100_ACT_NONE;
        q.table = nullptr;
        q.st_max = nullptr;
        if (present(0)) {
          uint32_t ra[16], rb[16];
          tmem_ld16(t_addr, ra);
#pragma unroll 1
          for (int c0 = 0; c0 < COLS; c0 += 32) {
            tmem_ld_wait();
            const bool more_b = present(c0 + 16);
            if (more_b) {
              tmem_ld16(t_addr + (uint32_t)(c0 + 16), rb);
            } else {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
            }
            epilogue_chunk<P_BN, 16>(q, ra, row, n0 + c0, s_bias + c0, s_off + c0, rr, false);
            if (!more_b) break;
            tmem_ld_wait();
            const bool more_a = present(c0 + 32);
            if (more_a) {
              tmem_ld16(t_addr + (uint32_t)(c0 + 32), ra);
            } else {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
            }
            epilogue_chunk<P_BN, 16>(q, rb, row, n0 + c0 + 16, s_bias + c0 + 16, s_off + c0 + 16, rr, false);
            if (!more_a) break;
          }
        }
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; present(c0); c0 += 16) {
        uint32_t r[16];
        tmem_ld16(t_addr + (uint32_t)c0, r);
        tmem_ld_wait();
        // `last`: the accumulator buffer goes back to the MMA warp (this warp's last read of it has completed)
        const bool last = !present(c0 + 16);
        LS100_PTRACE(22);
        if (last) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
        }
        if (staged && n0 + c0 + 16 <= p.n) {
          const bool with_resid = p.resid != nullptr;
          if (with_resid) {  // the piece requested one step ago has landed in row order
            cp_async_wait_all();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 t = *reinterpret_cast<const float4*>(stg_in + stage_off(lane, j));
              rr[4 * j] = t.x;
              rr[4 * j + 1] = t.y;
              rr[4 * j + 2] = t.z;
              rr[4 * j + 3] = t.w;
            }
            __syncwarp();
            if (!last && n0 + c0 + 32 <= p.n) fetch_resid(c0 + 16);  // in flight during this piece's arithmetic
          }
          int acc[16];
          float v[16];
          epilogue_acc<16>(p, r, s_off + c0, acc);
          epilogue_arith<16>(p, acc, row, n0 + c0, s_bias + c0, rr, with_resid, v);
          // own row in, eight rows x 64 bytes out per instruction
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(stg_out + stage_off(lane, j)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          __syncwarp();
          float* op = reinterpret_cast<float*>(p.out);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int br = 8 * i + mv_row;
            const float4 t = *reinterpret_cast<const float4*>(stg_out + stage_off(br, mv_piece));
            if (row0 + br < p.m) *reinterpret_cast<float4*>(op + (long long)(row0 + br) * p.ldo + n0 + c0 + mv_piece * 4) = t;
          }
          __syncwarp();  // the block is rewritten in the other order by the next piece
        } else {
          epilogue_chunk<P_BN, 16>(p, r, row, n0 + c0, s_bias + c0, s_off + c0, rr, false, nullptr, nullptr,
                                   with_stats ? &stats : nullptr, tabled ? table_c + c0 * 256 : nullptr);
        }
        LS100_PTRACE(23);
      
      }
      if (with_stats && row < p.m && n0 < p.n) {  // COLS == 64: this warp's column group is one statistics group
        const unsigned m2 = __vmaxs4(stats.max4, stats.max4 >> 16);
        const unsigned m1 = __vmaxs4(m2, m2 >> 8);
        const long long slot = ((long long)(row >> 7) * p.st_groups + (n0 >> 6)) * 128 + (row & 127);
        p.st_max[slot] = (int8_t)(m1 & 0xffu);
        p.st_sum[slot] = stats.sum0 + stats.sum1;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * P_BN);
  }
}

// One thread per (column, value): what the epilogue computes after the output quantiser, with the scalar forms of the
// same roundings (and the float64-erf GELU the fast path falls back to), so that reading the table and computing
// agree in every bit. Value 0x80 (-128) never leaves the quantiser; it repeats the entry of -127.
__global__ void requant_table_kernel(GemmEpi p, uint8_t* table, int cols_padded) {
  const int col = blockIdx.x;
  const int i = threadIdx.x;
  if (col >= cols_padded) return;
  uint8_t out = 0;
  if (col < p.n) {
    int q = (int)(int8_t)i;
    if (q == -128) q = -127;
    float v = __fmul_rn((float)q, p.s_outq);
    if (p.bias != nullptr) v = __fadd_rn(v, p.bias[col]);
    if (p.act == LS100_ACT_RELU)
      v = fmaxf(v, 0.f);
    else if (p.act == LS100_ACT_GELU)
      v = gelu_erf_exact(v);
    const float sub = (p.out_kind == LS100_OUT_REQ_U8) ? 127.f : 0.f;
    out = (uint8_t)(__float_as_uint(quant_biased(__fsub_rn(div_rn(v, p.s_req, p.rs_req), sub))) & 0xffu);
  }
  table[(long long)col * 256 + i] = out;
}

static GemmEpi make_epi(const ls100_ctx* ctx, const ls100_gemm_i8_args* a) {
  GemmEpi p;
  p.m = a->m;
  p.n = a->n;
  p.k = a->k;
  p.s_acc = a->s_acc;
  p.s_outq = a->s_outq;
  p.s_req = a->s_req;
  p.rs_outq = a->s_outq > 0.f ? 1.0f / a->s_outq : 0.f;
  p.rs_req = a->s_req > 0.f ? 1.0f / a->s_req : 0.f;
  p.w_off = a->w_off;
  p.bias = a->bias;
  p.resid = a->resid;
  p.ldr = a->ldr;
  p.act = a->act;
  p.out_kind = a->out_kind;
  p.out = a->out;
  p.ldo = a->ldo;
  p.err = ctx->d_err;
  p.ln_gamma = a->ln_gamma;
  p.ln_beta = a->ln_beta;
  p.ln_amax = a->ln_amax;
  p.ln_scale = a->ln_amax / 127.0f;
  p.ln_rs = a->ln_amax > 0.f ? 1.0f / p.ln_scale : 0.f;
  p.ln_out = a->ln_out;
  p.ln_ldq = a->ln_ldq;
  p.table = a->req_table;
  p.st_max = a->stat_max;
  p.st_sum = a->stat_sum;
  p.st_groups = (a->n + 63) / 64;
  p.st_c = a->s_outq * 1.4426950408889634f;
  p.st_c127 = -127.f * p.st_c;
  return p;
}

static int launch_gemm_persist(ls100_ctx* ctx, const ls100_gemm_i8_args* a, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int rc = ls100_get_tmap_u8(ctx, a->a, (uint64_t)a->m, (uint64_t)a->k, (uint64_t)a->lda, BM, BK, &ta);
  if (rc) return rc;
  rc = ls100_get_tmap_u8(ctx, a->w, (uint64_t)a->n, (uint64_t)a->k, (uint64_t)a->ldw, P_BN, BK, &tb);
  if (rc) return rc;
  const GemmEpi p = make_epi(ctx, a);
  const int tiles_n = (a->n + P_BN - 1) / P_BN;
  const long long tiles = (long long)tiles_n * ((a->m + BM - 1) / BM);
  if (tiles > 0x7fffffffLL) return LS100_ERR_BAD_ARG;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  // fp32 outputs move through shared memory in whole lines when the rows on both sides are 16-byte aligned; int8
  // outputs whose bias / activation / requantisation the caller tabulated read the table
  const bool staged = a->out_kind == LS100_OUT_F32 && (a->ldo & 3) == 0 && (((uintptr_t)a->out) & 15) == 0 &&
                      (a->resid == nullptr || ((a->ldr & 3) == 0 && (((uintptr_t)a->resid) & 15) == 0));
  const bool tabled = a->req_table != nullptr;  // validated by the caller: int8 requantised kind, output quantiser, no residual
  const bool outq = a->out_kind == LS100_OUT_OUTQ_I8 && !a->stat_max && !a->bias && !a->resid && a->act == LS100_ACT_NONE && !tabled;
  auto kern = staged ? gemm_i8_persist_kernel<P_STAGED>
              : tabled ? gemm_i8_persist_kernel<P_TABLE>
              : outq   ? gemm_i8_persist_kernel<P_OUTQ>
                       : gemm_i8_persist_kernel<P_PLAIN>;
  const cudaError_t e = ls100_launch(kern, dim3(grid), dim3(P_THREADS), PersistSmem::TOTAL, stream, ta, tb, p, tiles_n, (int)tiles);
  return e == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

template <int BN, int STAGES, bool LNF = false, int BMT = 128>
static int launch_gemm(ls100_ctx* ctx, const ls100_gemm_i8_args* a, cudaStream_t stream) {
  using SM = GemmSmem<BN, STAGES, BMT>;
  auto kern = gemm_i8_tc_kernel<BN, STAGES, LNF, BMT>;
  CUtensorMap ta, tb;
  int rc = ls100_get_tmap_u8(ctx, a->a, (uint64_t)a->m, (uint64_t)a->k, (uint64_t)a->lda, BMT, BK, &ta);
  if (rc) return rc;
  rc = ls100_get_tmap_u8(ctx, a->w, (uint64_t)a->n, (uint64_t)a->k, (uint64_t)a->ldw, BN, BK, &tb);
  if (rc) return rc;
  const GemmEpi p = make_epi(ctx, a);
  dim3 grid((a->n + BN - 1) / BN, (a->m + BMT - 1) / BMT);
  if (LNF)  // one cluster per 128-row block
    return ls100_launch_cluster(kern, grid, dim3(320), SM::TOTAL, stream, grid.x, ta, tb, p) == cudaSuccess ? LS100_OK
                                                                                                             : LS100_ERR_CUDA;
  return ls100_launch(kern, grid, dim3(320), SM::TOTAL, stream, ta, tb, p) == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

template <int BN, int STAGES, bool LNF = false, int BMT = 128>
static int set_smem_attr() {
  return cudaFuncSetAttribute(gemm_i8_tc_kernel<BN, STAGES, LNF, BMT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GemmSmem<BN, STAGES, BMT>::TOTAL) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

}  // namespace ls100

// Opts every tile variant into its dynamic shared-memory size on the current device.
// Called once from ls100_ctx_create so that no attribute call happens inside a stream capture.
int ls100_gemm_i8_init_device() {
  using namespace ls100;
  int rc = set_smem_attr<128, 3>();
  if (!rc) rc = set_smem_attr<64, 4>();
  if (!rc) rc = set_smem_attr<32, 4>();
  if (!rc) rc = set_smem_attr<32, 8>();
  if (!rc) rc = set_smem_attr<32, 4, false, 64>();
  if (!rc) rc = set_smem_attr<32, 4, true>();
  if (!rc) rc = set_smem_attr<64, 4, true>();
  if (!rc) rc = set_smem_attr<128, 3, true>();
  if (!rc && (cudaFuncSetAttribute(gemm_i8_persist_kernel<P_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PersistSmem::TOTAL) != cudaSuccess ||
              cudaFuncSetAttribute(gemm_i8_persist_kernel<P_STAGED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PersistSmem::TOTAL) != cudaSuccess ||
              cudaFuncSetAttribute(gemm_i8_persist_kernel<P_TABLE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PersistSmem::TOTAL) != cudaSuccess ||
              cudaFuncSetAttribute(gemm_i8_persist_kernel<P_OUTQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   PersistSmem::TOTAL) != cudaSuccess))
    rc = LS100_ERR_CUDA;
  return rc;
}

extern "C" int ls100_gemm_i8(ls100_ctx* ctx, const ls100_gemm_i8_args* a, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !a->a || !a->w || !a->out) return LS100_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->a) & 15) || (((uintptr_t)a->w) & 15) || (a->lda & 15) || (a->ldw & 15)) return LS100_ERR_ALIGN;
  if (a->lda < a->k || a->ldw < a->k) return LS100_ERR_BAD_ARG;
  if (a->out_kind < LS100_OUT_OUTQ_I8 || a->out_kind > LS100_OUT_I32) return LS100_ERR_BAD_ARG;
  if (a->out_kind == LS100_OUT_OUTQ_I8 && !(a->s_outq > 0.f)) return LS100_ERR_BAD_ARG;
  if ((a->out_kind == LS100_OUT_REQ_S8 || a->out_kind == LS100_OUT_REQ_U8) && !(a->s_req > 0.f))
    return LS100_ERR_BAD_ARG;
  if (a->resid && a->ldr < a->n) return LS100_ERR_BAD_ARG;
  if (a->ldo < a->n) return LS100_ERR_BAD_ARG;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (a->req_table && ((a->out_kind != LS100_OUT_REQ_S8 && a->out_kind != LS100_OUT_REQ_U8) || !(a->s_outq > 0.f) ||
                       a->resid || a->ln_out || a->stat_max || (((uintptr_t)a->req_table) & 15)))
    return LS100_ERR_BAD_ARG;
  if ((a->stat_max != nullptr) != (a->stat_sum != nullptr)) return LS100_ERR_BAD_ARG;
  if (a->stat_max) {  // only the many-tile kernel's epilogue keeps the statistics (its warps own whole 64-column groups)
    if (a->out_kind != LS100_OUT_OUTQ_I8 || a->ln_out || (((uintptr_t)a->stat_sum) & 3)) return LS100_ERR_BAD_ARG;
    return launch_gemm_persist(ctx, a, stream);
  }
  if (a->ln_out) {
    if (a->out_kind != LS100_OUT_F32 || !a->ln_gamma || !a->ln_beta || !(a->ln_amax > 0.f) || a->ln_ldq < a->n)
      return LS100_ERR_BAD_ARG;
    if ((((uintptr_t)a->ln_out) & 15) || (a->ln_ldq & 15) || (((uintptr_t)a->out) & 15) || (a->ldo & 3) ||
        (((uintptr_t)a->ln_gamma) & 15) || (((uintptr_t)a->ln_beta) & 15))
      return LS100_ERR_ALIGN;
    // cluster form: the CTAs of a 128-row block (at most 8) hold the whole row between them
    if ((a->n & 31) == 0 && a->n <= 256) return launch_gemm<32, 4, true>(ctx, a, stream);
    if ((a->n & 31) == 0 && a->n <= 512) return launch_gemm<64, 4, true>(ctx, a, stream);
    if ((a->n & 31) == 0 && a->n <= 1024) return launch_gemm<128, 3, true>(ctx, a, stream);
    // otherwise: the plain GEMM, then the stand-alone LayerNorm kernel
    ls100_gemm_i8_args g = *a;
    g.ln_out = nullptr;
    const int rc = ls100_gemm_i8(ctx, &g, stream_);
    if (rc != LS100_OK) return rc;
    ls100_ln_quant_args l;
    memset(&l, 0, sizeof(l));
    l.x = static_cast<const float*>(a->out);
    l.ldx = a->ldo;
    l.gamma = a->ln_gamma;
    l.beta = a->ln_beta;
    l.rows = a->m;
    l.hidden = a->n;
    l.amax = a->ln_amax;
    l.out_q = a->ln_out;
    l.ldq = a->ln_ldq;
    return ls100_ln_quant(ctx, &l, stream_);
  }
  const long long mt = (a->m + BM - 1) / BM;
  auto ctas = [&](int bn) { return mt * ((a->n + bn - 1) / bn); };
  const long long sms = ctx->sm_count;
  // Largest tile that still fills the machine; small problems fall to BN=32.
  if (ctas(256) >= 2 * sms) return launch_gemm_persist(ctx, a, stream);
  if (ctas(128) >= sms) return launch_gemm<128, 3>(ctx, a, stream);
  if (ctas(64) >= sms) return launch_gemm<64, 4>(ctx, a, stream);
  // one row block and fewer CTAs than SMs (decoder-only generation: a few dozen rows against large weights): the main
  // loop is bound by the latency of its tile copies, so a long K gets a deeper ring. Measured: GPT-2 medium decode
  // steps 17 % faster; with several row blocks (Transformer-base FFN2, 512 rows) the deeper ring was 1.8 us SLOWER
  // per launch, so those keep four stages.
  if (mt == 1 && a->k > 4 * BK && ctas(32) <= sms) return launch_gemm<32, 8>(ctx, a, stream);
  // several row blocks and at most half a wave of 128-row tiles: 64-row tiles halve the activation bytes a CTA waits
  // for and still fit one CTA per SM
  const long long ctas64 = ((a->m + 63) / 64) * ((a->n + 31) / 32);
  if (mt >= 2 && ctas64 <= sms) return launch_gemm<32, 4, false, 64>(ctx, a, stream);
  return launch_gemm<32, 4>(ctx, a, stream);
}

extern "C" size_t ls100_gemm_i8_table_bytes(int64_t n) { return n > 0 ? (size_t)((n + 255) / 256) * 65536 : 0; }

extern "C" int ls100_gemm_i8_build_table(ls100_ctx* ctx, const ls100_gemm_i8_args* a, uint8_t* table, ls100_stream_t stream_) {
  using namespace ls100;
  if (!ctx || !a || !table || a->n <= 0) return LS100_ERR_BAD_ARG;
  if ((a->out_kind != LS100_OUT_REQ_S8 && a->out_kind != LS100_OUT_REQ_U8) || !(a->s_outq > 0.f) || !(a->s_req > 0.f) ||
      a->resid || a->act < LS100_ACT_NONE || a->act > LS100_ACT_GELU)
    return LS100_ERR_BAD_ARG;
  if (((uintptr_t)table) & 15) return LS100_ERR_ALIGN;
  const GemmEpi p = make_epi(ctx, a);
  const int cols = (int)((a->n + 255) / 256 * 256);
  requant_table_kernel<<<cols, 256, 0, (cudaStream_t)stream_>>>(p, table, cols);
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}
