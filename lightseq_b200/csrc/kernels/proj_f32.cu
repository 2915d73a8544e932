// out_f32[M,N] = (x_f32[M,K] . Wq_i8[N,K]^T) * s_w + bias
// The decoder's cross-attention k_proj / v_proj: activations stay fp32, only the weight
// is fake-quantised (QuantLinear with pre_activation="encoder_out",
// lightseq/training/ops/pytorch/quantization.py:41-46). Runs once per request
// (QuantDecoder::project_encoder_output, lightseq/inference/model/quant_decoder.cc.cu:489-520).
// fp32 SIMT tile kernel: 128x128 output tile, 256 threads x (8x8), K staged 16 at a time, double-buffered.
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

__global__ void __launch_bounds__(256, 2) proj_f32_kernel(const ls100_proj_f32_args a) {
  // 128 x 128 output tile, 256 threads x (8 x 8) outputs, K staged 16 at a time through two shared-memory buffers
  // (the loads of step k+1 are in registers while step k is multiplied). Each thread's 8 rows / 8 columns are
  // two groups of 4 that lie 64 apart, so that the 16-byte shared-memory reads of a warp are conflict-free.
  // Every output is still one fmaf chain over k in ascending order.
  __shared__ __align__(16) float As[2][16][128 + 4];
  __shared__ __align__(16) float Ws[2][16][128 + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int t = threadIdx.x;
  const int m0 = blockIdx.y * 128, n0 = blockIdx.x * 128;
  const int tx = t & 15, ty = t >> 4;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  // staging: thread handles row lr (and lr + 64) of the tile, k-values lc .. lc+3
  const int lr = t >> 2, lc = (t & 3) * 4;
  float4 ra[2];
  float rw[2][4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int m = m0 + lr + hh * 64;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < a.m && k0 + lc + 3 < a.k) {
        v = *reinterpret_cast<const float4*>(a.x + (long long)m * a.ldx + k0 + lc);
      } else if (m < a.m) {
        float e[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < 4; ++j)
          if (k0 + lc + j < a.k) e[j] = a.x[(long long)m * a.ldx + k0 + lc + j];
        v = make_float4(e[0], e[1], e[2], e[3]);
      }
      ra[hh] = v;
      const int n = n0 + lr + hh * 64;
#pragma unroll
      for (int j = 0; j < 4; ++j) rw[hh][j] = (n < a.n && k0 + lc + j < a.k) ? (float)a.w[(long long)n * a.ldw + k0 + lc + j] : 0.f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = lr + hh * 64;
      As[buf][lc][r] = ra[hh].x;
      As[buf][lc + 1][r] = ra[hh].y;
      As[buf][lc + 2][r] = ra[hh].z;
      As[buf][lc + 3][r] = ra[hh].w;
#pragma unroll
      for (int j = 0; j < 4; ++j) Ws[buf][lc + j][r] = rw[hh][j];
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < a.k; k0 += 16) {
    const bool more = k0 + 16 < a.k;
    if (more) fetch(k0 + 16);
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      const float4 w0 = *reinterpret_cast<const float4*>(&Ws[buf][kk][tx * 4]);
      const float4 w1 = *reinterpret_cast<const float4*>(&Ws[buf][kk][64 + tx * 4]);
      const float ar[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float wr[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    if (more) {
      stash(buf ^ 1);  // the other buffer was last read one iteration ago, before the barrier below
      __syncthreads();
      buf ^= 1;
    }
  }
  float* out = reinterpret_cast<float*>(a.out);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int m = m0 + (i >> 2) * 64 + ty * 4 + (i & 3);
    if (m >= a.m) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
      if (n >= a.n) continue;
      float v = __fmul_rn(acc[i][j], a.s_w);
      if (a.bias) v = __fadd_rn(v, __ldg(a.bias + n));
      if (a.split_seq > 0) {  // [batch, heads, split_seq, 64]
        const int b = m / a.split_seq, sq = m - b * a.split_seq;
        out[(((long long)b * (a.n >> 6) + (n >> 6)) * a.split_seq + sq) * 64 + (n & 63)] = v;
      } else {
        out[(long long)m * a.ldo + n] = v;
      }
    }
  }
}

}  // namespace ls100

extern "C" int ls100_proj_f32(ls100_ctx* ctx, const ls100_proj_f32_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->x || !a->w || !a->out) return LS100_ERR_BAD_ARG;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0 || !(a->s_w > 0.f)) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->x) & 15) || (a->ldx & 3)) return LS100_ERR_ALIGN;
  if (a->split_seq < 0 || (a->split_seq > 0 && (a->n & 63))) return LS100_ERR_BAD_ARG;
  dim3 grid((a->n + 127) / 128, (a->m + 127) / 128);
  return ls100_launch(ls100::proj_f32_kernel, grid, dim3(256), 0, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}
