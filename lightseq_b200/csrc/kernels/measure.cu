// Measurement and diagnostic kernels (not on any model's path):
//   ls100_measure_i8_mma_peak   steady-state issue rate of tcgen05.mma kind::i8 from operands resident in shared
//                               memory: the tensor-pipe ceiling the int8 GEMMs of this library are held against
//   ls100_measure_phase_floor   cost of one dependent phase three ways: kernel after kernel, kernel after kernel
//                               with programmatic dependent launch, and phases of ONE persistent kernel separated by
//                               a global-memory grid barrier. Decides whether a chain of small kernels is better
//                               replaced by one persistent kernel (on B200 it is not: the barrier costs more than
//                               the launch)
//   ls100_debug_expire_wait     one CTA waits on an mbarrier that nobody arrives at, with a short budget, records
//                               LS100_ERR_TIMEOUT in the context's error word and returns normally: exercises the
//                               error path of the bounded waits without faulting or hanging anything
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

// ------------------------------------------------------------------------------------------------ int8 MMA peak
constexpr int PK_M = 128, PK_N = 256, PK_KB = 128;  // one k-block = 128 bytes = four K=32 MMAs
constexpr int PK_SMEM = PK_M * PK_KB + PK_N * PK_KB + 64 + 1024;

__device__ __forceinline__ uint64_t pk_desc(uint32_t saddr) {  // K-major, 128-byte swizzle, 8-row groups 1024 B apart
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(128, 1) i8_mma_peak_kernel(int iters, int* err) {
  extern __shared__ uint8_t pk_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pk_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + PK_M * PK_KB + PK_N * PK_KB);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bar + 1);
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < (PK_M + PK_N) * PK_KB / 4; i += blockDim.x)  // any int8 values: small, mixed signs
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01ff02feu * (uint32_t)(i * 2654435761u >> 29);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *slot;
  if (warp == 1 && elect_one()) {
    constexpr uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PK_N >> 3) << 17) | ((uint32_t)(PK_M >> 4) << 24);
    const uint64_t ad = pk_desc(smem_u32(smem)), bd = pk_desc(smem_u32(smem + PK_M * PK_KB));
    for (int it = 0; it < iters; ++it) {
      const uint32_t d = tmem_base + (uint32_t)((it & 1) * PK_N);  // two accumulators, as the persistent GEMM uses
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) tc_mma_i8(d, ad + (uint64_t)(kk * 2), bd + (uint64_t)(kk * 2), idesc, 1u);
    }
    tc_commit(bar);
    if (!mbar_wait(bar, 0) && err) atomicExch(err, (int)LS100_ERR_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ phase floor
__device__ __forceinline__ void pf_work(const float* src, float* dst, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  dst[i] = src[(i + n / 2 + 37) % n] + 1.f;  // an element another CTA wrote in the previous phase
}
__global__ void pf_kernel(const float* src, float* dst, int n) {
  pdl_launch_dependents();
  pdl_wait();
  pf_work(src, dst, n);
}
__global__ void pf_persistent_kernel(float* a, float* b, int n, unsigned* bar, int phases, int* err) {
  float *src = a, *dst = b;
  for (int p = 0; p < phases; ++p) {
    pf_work(src, dst, n);
    __syncthreads();
    if (threadIdx.x == 0) {
      asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(bar), "r"(1u) : "memory");
      const unsigned target = gridDim.x * (unsigned)(p + 1);
      const long long t0 = clock64();
      unsigned v = 0;
      do {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar) : "memory");
      } while (v < target && clock64() - t0 < LS100_WAIT_CYCLES);
      if (v < target && err) atomicExch(err, (int)LS100_ERR_TIMEOUT);
    }
    __syncthreads();
    float* t = src;
    src = dst;
    dst = t;
  }
}

// ------------------------------------------------------------------------------------------------ expiring wait
__global__ void expire_wait_kernel(int* err, long long budget_cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait_cycles(&bar, 0, budget_cycles)) atomicExch(err, (int)LS100_ERR_TIMEOUT);
}

}  // namespace ls100

using namespace ls100;

extern "C" int ls100_measure_i8_mma_peak(ls100_ctx* ctx, int iters, ls100_stream_t stream_, double* tops_out, float* ms_out) {
  if (!ctx || iters < 1 || !tops_out) return LS100_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(i8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM) != cudaSuccess) return LS100_ERR_CUDA;
    attr = true;
  }
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return LS100_ERR_CUDA;
  i8_mma_peak_kernel<<<ctx->sm_count, 128, PK_SMEM, st>>>(iters, ctx->d_err);  // warm-up
  cudaEventRecord(e0, st);
  i8_mma_peak_kernel<<<ctx->sm_count, 128, PK_SMEM, st>>>(iters, ctx->d_err);
  cudaEventRecord(e1, st);
  const bool ok = cudaEventSynchronize(e1) == cudaSuccess;
  float ms = 0.f;
  if (ok) cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (!ok || ms <= 0.f) return LS100_ERR_CUDA;
  const double ops = 2.0 * PK_M * PK_N * 32.0 * 4.0 * (double)iters * (double)ctx->sm_count;
  *tops_out = ops / (ms * 1e-3) / 1e12;
  if (ms_out) *ms_out = ms;
  return LS100_OK;
}

extern "C" int ls100_measure_phase_floor(ls100_ctx* ctx, int phases, int grid, ls100_stream_t stream_, float* us_per_phase /* [3] */) {
  if (!ctx || phases < 1 || grid < 1 || grid > 2 * ctx->sm_count || !us_per_phase) return LS100_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  cudaStream_t own = nullptr;
  if (!st) {  // the phases are captured into a graph, which the legacy default stream cannot do
    if (cudaStreamCreateWithFlags(&own, cudaStreamNonBlocking) != cudaSuccess) return LS100_ERR_CUDA;
    st = own;
  }
  const int threads = 256, n = grid * threads;
  float *a = nullptr, *b = nullptr;
  unsigned* bar = nullptr;
  if (cudaMalloc(&a, n * 4) != cudaSuccess || cudaMalloc(&b, n * 4) != cudaSuccess || cudaMalloc(&bar, 4) != cudaSuccess) {
    if (own) cudaStreamDestroy(own);
    return LS100_ERR_CUDA;
  }
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  int rc = LS100_OK;
  for (int mode = 0; mode < 3 && rc == LS100_OK; ++mode) {
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ex = nullptr;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { rc = LS100_ERR_CUDA; break; }
    cudaMemsetAsync(a, 0, n * 4, st);
    cudaMemsetAsync(bar, 0, 4, st);
    if (mode < 2) {
      for (int i = 0; i < phases; ++i) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(threads);
        cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = mode == 1 ? 1 : 0;
        cudaLaunchKernelEx(&cfg, pf_kernel, (const float*)((i & 1) ? b : a), (i & 1) ? a : b, n);
      }
    } else {
      int* err = ctx->d_err;
      void* args[] = {&a, &b, (void*)&n, &bar, (void*)&phases, &err};
      cudaLaunchCooperativeKernel((void*)pf_persistent_kernel, dim3(grid), dim3(threads), args, 0, st);
    }
    if (cudaStreamEndCapture(st, &g) != cudaSuccess || !g || cudaGraphInstantiate(&ex, g, 0) != cudaSuccess) {
      if (g) cudaGraphDestroy(g);
      rc = LS100_ERR_CUDA;
      break;
    }
    for (int i = 0; i < 3; ++i) cudaGraphLaunch(ex, st);
    cudaEventRecord(e0, st);
    const int reps = 20;
    for (int i = 0; i < reps; ++i) cudaGraphLaunch(ex, st);
    cudaEventRecord(e1, st);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = LS100_ERR_CUDA;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    us_per_phase[mode] = ms * 1e3f / (float)(reps * phases);
    cudaGraphExecDestroy(ex);
    cudaGraphDestroy(g);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamSynchronize(st);
  cudaFree(a);
  cudaFree(b);
  cudaFree(bar);
  if (own) cudaStreamDestroy(own);
  return rc;
}

extern "C" int ls100_debug_expire_wait(ls100_ctx* ctx, ls100_stream_t stream_) {
  if (!ctx) return LS100_ERR_BAD_ARG;
  expire_wait_kernel<<<1, 32, 0, (cudaStream_t)stream_>>>(ctx->d_err, 200000ll);  // about 0.1 ms
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}
