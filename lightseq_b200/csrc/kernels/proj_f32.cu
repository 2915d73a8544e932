// out_f32[M,N] = (x_f32[M,K] . Wq_i8[N,K]^T) * s_w + bias
// The decoder's cross-attention k_proj / v_proj: activations stay fp32, only the weight
// is fake-quantised (QuantLinear with pre_activation="encoder_out",
// lightseq/training/ops/pytorch/quantization.py:41-46). Runs once per request
// (QuantDecoder::project_encoder_output, lightseq/inference/model/quant_decoder.cc.cu:489-520).
// fp32 SIMT tile kernel: 64x64 output tile, 256 threads x (4x4), K staged 16 at a time.
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

__global__ void __launch_bounds__(256) proj_f32_kernel(const ls100_proj_f32_args a) {
  __shared__ float As[16][64 + 4];
  __shared__ float Ws[16][64 + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int t = threadIdx.x;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = t & 15, ty = t >> 4;  // 16 x 16 threads, each 4 x 4 outputs
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int lr = t >> 2, lc = (t & 3) * 4;  // 64 rows x 4 groups of 4 k-values
  for (int k0 = 0; k0 < a.k; k0 += 16) {
    {
      const int m = m0 + lr;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < a.m && k0 + lc + 3 < a.k) v = *reinterpret_cast<const float4*>(a.x + (long long)m * a.ldx + k0 + lc);
      else if (m < a.m) {
        float e[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < 4; ++j)
          if (k0 + lc + j < a.k) e[j] = a.x[(long long)m * a.ldx + k0 + lc + j];
        v = make_float4(e[0], e[1], e[2], e[3]);
      }
      As[lc][lr] = v.x;
      As[lc + 1][lr] = v.y;
      As[lc + 2][lr] = v.z;
      As[lc + 3][lr] = v.w;
      const int n = n0 + lr;
      float e[4] = {0.f, 0.f, 0.f, 0.f};
      if (n < a.n) {
        for (int j = 0; j < 4; ++j)
          if (k0 + lc + j < a.k) e[j] = (float)a.w[(long long)n * a.ldw + k0 + lc + j];
      }
      Ws[lc][lr] = e[0];
      Ws[lc + 1][lr] = e[1];
      Ws[lc + 2][lr] = e[2];
      Ws[lc + 3][lr] = e[3];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* out = reinterpret_cast<float*>(a.out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
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
  dim3 grid((a->n + 63) / 64, (a->m + 63) / 64);
  return ls100_launch(ls100::proj_f32_kernel, grid, dim3(256), 0, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}
