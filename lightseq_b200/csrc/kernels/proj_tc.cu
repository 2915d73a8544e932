// Cross-attention K/V projection on the tensor cores:  out_f32[M,N] = (x_f32[M,K] . Wq_i8[N,K]^T) * s_w + bias
// (QuantLinear with pre_activation="encoder_out": only the weight is fake-quantised,
// lightseq/training/ops/pytorch/quantization.py:41-46; QuantDecoder::project_encoder_output,
// lightseq/inference/model/quant_decoder.cc.cu:489-520, where it is one fp16 cuBLAS GEMM).
//
// fp32 activations do not fit a tensor-core operand, but they split exactly enough: x = hi + mid + lo with three
// bf16 numbers (8 significant bits each; the remainder is below 2^-27 |x|), and an int8 weight IS a bf16 number. So
//   x . W^T = [lo | mid | hi] . [W | W | W]^T
// is one bf16 GEMM with K' = 3K whose products are exact in fp32; only the fp32 accumulation of tcgen05.mma
// (kind::f16, fp32 accumulator in TMEM) rounds. ls100_split_bf16x3 writes the [M, 3K] operand once per request (the
// same encoder output feeds the K and the V projection of every decoder layer); the weight's three copies are never
// materialised: the TMA coordinate of the weight tile wraps around K.
//
// Kernel: persistent, one CTA per SM over 128 x 128 tiles, six-stage TMA ring of (A 128x64 bf16, W 128x64 bf16)
// tiles with 128-byte swizzle, two 128-column fp32 accumulators in TMEM (the MMAs of tile i+1 run under the
// epilogue of tile i), warps: 0 TMA producer, 1 TMEM allocator + MMA issuer, 2-9 epilogue (two per TMEM lane
// quarter, 64 columns each). Every mbarrier wait is bounded and reports through the context's error word.
#include <cuda_bf16.h>

#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr int T_BM = 128, T_BN = 128, T_BK_BYTES = 128;  // 64 bf16 per k-block
constexpr int T_STAGES = 6, T_EPI_WARPS = 8, T_THREADS = 64 + 32 * T_EPI_WARPS;
constexpr int T_A_BYTES = T_BM * T_BK_BYTES, T_B_BYTES = T_BN * T_BK_BYTES, T_STAGE_BYTES = T_A_BYTES + T_B_BYTES;
constexpr int T_BAR_OFFSET = T_STAGES * T_STAGE_BYTES;
constexpr int T_SMEM = T_BAR_OFFSET + 256 + 1024;

struct ProjTcParams {
  int m, n, k3_bytes, k_bytes;  // k3_bytes = 3K * 2, k_bytes = K * 2
  float s_w;
  const float* bias;
  float* out;
  long long ldo;
  int split_seq;
  int* err;
};

// K-major, SWIZZLE_128B, 8-row groups 1024 B apart (the same descriptor form as the int8 GEMM)
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, N = 128, M = 128
__device__ __forceinline__ constexpr uint32_t tc_idesc_bf16() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(T_BN >> 3) << 17) | ((uint32_t)(T_BM >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// x fp32 [M, K] -> bf16 [M, 3K]: columns [0,K) lo, [K,2K) mid, [2K,3K) hi. Smallest terms first: the tensor core's
// fp32 accumulation loses about 2^-24 of the running sum per MMA, so the sum should stay small for as long as possible
// (measured: 3x closer to the exact product than with the large terms first).
__global__ void __launch_bounds__(256) split_bf16x3_kernel(const float* __restrict__ x, long long ldx, int m, int k,
                                                           __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)m * (k >> 2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / (k >> 2)), c = (int)(i % (k >> 2)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + (long long)r * ldx + c);
    const float f[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat16 hi[4], mid[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hi[j] = __float2bfloat16_rn(f[j]);
      const float r1 = __fsub_rn(f[j], __bfloat162float(hi[j]));  // exact
      mid[j] = __float2bfloat16_rn(r1);
      const float r2 = __fsub_rn(r1, __bfloat162float(mid[j]));  // exact
      lo[j] = __float2bfloat16_rn(r2);
    }
    __nv_bfloat16* o = out + (long long)r * 3 * k + c;
    *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(lo);
    *reinterpret_cast<uint2*>(o + k) = *reinterpret_cast<const uint2*>(mid);
    *reinterpret_cast<uint2*>(o + 2 * k) = *reinterpret_cast<const uint2*>(hi);
  }
}

// int8 [N, K] -> bf16 [N, K] (exact)
__global__ void __launch_bounds__(256) i8_to_bf16_kernel(const int8_t* __restrict__ w, long long ldw, int n, int k,
                                                         __nv_bfloat16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)n * k;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / k), c = (int)(i % k);
    out[i] = __float2bfloat16_rn((float)w[(long long)r * ldw + c]);
  }
}

__global__ void __launch_bounds__(T_THREADS, 1) proj_tc_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                               const __grid_constant__ CUtensorMap tma_b,
                                                               const ProjTcParams p, int tiles_n, int num_tiles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + T_BAR_OFFSET);
  uint64_t* empty_bar = full_bar + T_STAGES;
  uint64_t* tmem_full_bar = empty_bar + T_STAGES;  // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = p.k3_bytes / T_BK_BYTES;  // K is a multiple of 64, checked by the launcher

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
#pragma unroll
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], T_EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * T_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // only once this CTA owns its TMEM columns (a dependent's CTAs must not take them first)

  if (warp == 0) {
    if (elect_one()) {
      pdl_wait();
      uint32_t phase = 0;
      int s = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int n0 = (tile % tiles_n) * T_BN, m0 = (tile / tiles_n) * T_BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[s], phase ^ 1)) {  // a stage never filled reads as released
            if (p.err) atomicExch(p.err, (int)LS100_ERR_TIMEOUT);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * T_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], T_STAGE_BYTES);
          tma_load_2d(sa, &tma_a, &full_bar[s], kb * T_BK_BYTES, m0);
          tma_load_2d(sa + T_A_BYTES, &tma_b, &full_bar[s], (kb * T_BK_BYTES) % p.k_bytes, n0);  // [W | W | W]
          if (++s == T_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = tc_idesc_bf16();
      uint32_t phase = 0;
      int s = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (!mbar_wait(&tmem_empty_bar[buf], ((uint32_t)(local >> 1) & 1u) ^ 1u)) {  // drained by the epilogue
          if (p.err) atomicExch(p.err, (int)LS100_ERR_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * T_BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[s], phase)) {
            if (p.err) atomicExch(p.err, (int)LS100_ERR_TIMEOUT);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * T_STAGE_BYTES);
          const uint64_t adesc = tc_smem_desc(sa), bdesc = tc_smem_desc(sa + T_A_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)  // 16 bf16 = 32 bytes per MMA: +2 in 16-byte units inside the swizzle row
            tc_mma_bf16(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&empty_bar[s]);
          if (++s == T_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tmem_full_bar[buf]);
      }
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    pdl_wait();
    int local = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int n0 = (tile % tiles_n) * T_BN + half * 64;
      const int row = (tile / tiles_n) * T_BM + quarter * 32 + lane;
      if (dead) continue;
      bool ok = mbar_wait(&tmem_full_bar[buf], (uint32_t)(local >> 1) & 1u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0 && p.err) atomicExch(p.err, (int)LS100_ERR_TIMEOUT);
        dead = true;
        continue;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * T_BN + half * 64);
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(t_addr + (uint32_t)c0, r);
        tmem_ld_wait();
        if (c0 == 32) {  // this warp's part of the buffer is in registers: hand it back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
        }
        const int col0 = n0 + c0;
        if (row < p.m && col0 < p.n) {  // N is a multiple of 64 when head-split, of 4 otherwise (launcher)
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = __fmul_rn(__uint_as_float(r[j]), p.s_w);
            if (p.bias && col0 + j < p.n) v[j] = __fadd_rn(v[j], __ldg(p.bias + col0 + j));
          }
          float* op;
          if (p.split_seq > 0) {  // [batch, heads, split_seq, 64]: a 32-column chunk lies inside one head
            const int b = row / p.split_seq, sq = row - b * p.split_seq;
            op = p.out + (((long long)b * (p.n >> 6) + (col0 >> 6)) * p.split_seq + sq) * 64 + (col0 & 63);
          } else {
            op = p.out + (long long)row * p.ldo + col0;
          }
          if (col0 + 32 <= p.n) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(op + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.n) op[j] = v[j];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * T_BN);
  }
}

}  // namespace ls100

using namespace ls100;

int ls100_proj_tc_init_device() {
  return cudaFuncSetAttribute(proj_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM) == cudaSuccess ? LS100_OK
                                                                                                                    : LS100_ERR_CUDA;
}

extern "C" int ls100_split_bf16x3(ls100_ctx* ctx, const float* x, int64_t ldx, int32_t m, int32_t k, void* out,
                                  ls100_stream_t stream_) {
  if (!ctx || !x || !out || m <= 0 || k <= 0) return LS100_ERR_BAD_ARG;
  if ((k & 3) || (ldx & 3) || (((uintptr_t)x) & 15) || (((uintptr_t)out) & 15)) return LS100_ERR_ALIGN;
  const long long total = (long long)m * (k >> 2);
  const unsigned blocks = (unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  return ls100_launch(split_bf16x3_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream_, x, (long long)ldx, (int)m, (int)k,
                      static_cast<__nv_bfloat16*>(out)) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_i8_to_bf16(ls100_ctx* ctx, const int8_t* w, int64_t ldw, int32_t n, int32_t k, void* out,
                               ls100_stream_t stream_) {
  if (!ctx || !w || !out || n <= 0 || k <= 0 || ldw < k) return LS100_ERR_BAD_ARG;
  const long long wn = (long long)n * k;
  const unsigned wb = (unsigned)((wn + 255) / 256 < 2048 ? (wn + 255) / 256 : 2048);
  return ls100_launch(i8_to_bf16_kernel, dim3(wb), dim3(256), 0, (cudaStream_t)stream_, w, (long long)ldw, (int)n, (int)k,
                      static_cast<__nv_bfloat16*>(out)) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_proj_tc(ls100_ctx* ctx, const ls100_proj_tc_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->x3 || !a->w_bf16 || !a->out) return LS100_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0 || !(a->s_w > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->k & 63) return LS100_ERR_UNSUPPORTED;  // a k-block of 64 bf16 must not straddle the hi / mid / lo sections
  if ((((uintptr_t)a->x3) & 15) || (((uintptr_t)a->w_bf16) & 15) || (((uintptr_t)a->out) & 15)) return LS100_ERR_ALIGN;
  if (a->split_seq < 0 || (a->split_seq > 0 && (a->n & 63))) return LS100_ERR_BAD_ARG;
  if (a->split_seq == 0 && ((a->ldo & 3) || a->ldo < a->n)) return LS100_ERR_BAD_ARG;
  cudaStream_t stream = (cudaStream_t)stream_;
  CUtensorMap ta, tb;  // byte views of the bf16 matrices: 128-byte x 128-row boxes
  int rc = ls100_get_tmap_u8(ctx, a->x3, (uint64_t)a->m, (uint64_t)a->k * 6, (uint64_t)a->k * 6, T_BM, T_BK_BYTES, &ta);
  if (rc) return rc;
  rc = ls100_get_tmap_u8(ctx, a->w_bf16, (uint64_t)a->n, (uint64_t)a->k * 2, (uint64_t)a->k * 2, T_BN, T_BK_BYTES, &tb);
  if (rc) return rc;
  ProjTcParams p;
  p.m = a->m;
  p.n = a->n;
  p.k3_bytes = a->k * 6;
  p.k_bytes = a->k * 2;
  p.s_w = a->s_w;
  p.bias = a->bias;
  p.out = static_cast<float*>(a->out);
  p.ldo = a->ldo;
  p.split_seq = a->split_seq;
  p.err = ctx->d_err;
  const int tiles_n = (a->n + T_BN - 1) / T_BN;
  const long long tiles = (long long)tiles_n * ((a->m + T_BM - 1) / T_BM);
  if (tiles > 0x7fffffffLL) return LS100_ERR_BAD_ARG;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  return ls100_launch(proj_tc_kernel, dim3(grid), dim3(T_THREADS), T_SMEM, stream, ta, tb, p, tiles_n, (int)tiles) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}
