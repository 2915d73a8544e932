// Bandwidth-bound row kernels: LayerNorm (+ int8 quantise), embedding lookup and the
// load-time weight quantiser. One warp per row, 16-byte vector accesses, shuffle
// reductions; LayerNorm statistics are accumulated in float64 so the result does not
// depend on the reduction order.
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ LayerNorm
constexpr int LN_MAXV = 32;  // float4 per lane -> hidden <= 32*32*4 = 4096

template <int NV>
__global__ void __launch_bounds__(256, NV <= 6 ? 3 : 1) ln_quant_kernel(const ls100_ln_quant_args a, const float scale, const float rs) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= a.rows) return;
  const float* xr = a.x + (long long)warp * a.ldx;
  float4 v[NV];
  double s = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < a.hidden) {
      v[i] = *reinterpret_cast<const float4*>(xr + c);
      s += (double)v[i].x + (double)v[i].y + (double)v[i].z + (double)v[i].w;
    }
  }
  s = warp_sum_d(s);
  const double mean = s / (double)a.hidden;
  double sq = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < a.hidden) {
      const double d0 = (double)v[i].x - mean, d1 = (double)v[i].y - mean;
      const double d2 = (double)v[i].z - mean, d3 = (double)v[i].w - mean;
      sq += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
    }
  }
  sq = warp_sum_d(sq);
  const double rstd = 1.0 / sqrt(sq / (double)a.hidden + 1e-5);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * 32 + lane) * 4;
    if (c < a.hidden) {
      const float4 g = *reinterpret_cast<const float4*>(a.gamma + c);
      const float4 b = *reinterpret_cast<const float4*>(a.beta + c);
      float4 y;
      y.x = __fadd_rn(__fmul_rn((float)(((double)v[i].x - mean) * rstd), g.x), b.x);
      y.y = __fadd_rn(__fmul_rn((float)(((double)v[i].y - mean) * rstd), g.y), b.y);
      y.z = __fadd_rn(__fmul_rn((float)(((double)v[i].z - mean) * rstd), g.z), b.z);
      y.w = __fadd_rn(__fmul_rn((float)(((double)v[i].w - mean) * rstd), g.w), b.w);
      if (a.out_f) *reinterpret_cast<float4*>(a.out_f + (long long)warp * a.ldf + c) = y;
      if (a.out_q) {
        // (clamping to +-amax first, as the learned-amax quantiser does, cannot change the result: amax / scale is 127)
        const float2 q01 = f2_quant_biased(f2_div_rn(make_float2(y.x, y.y), f2_set(scale), f2_set(rs)));
        const float2 q23 = f2_quant_biased(f2_div_rn(make_float2(y.z, y.w), f2_set(scale), f2_set(rs)));
        *reinterpret_cast<uint32_t*>(a.out_q + (long long)warp * a.ldq + c) = pack_biased_i8x4(q01.x, q01.y, q23.x, q23.y);
      }
    }
  }
}

// Few rows (decode steps: a few hundred rows of 512..1024 values): one CTA of four warps per row, so that a row is one
// 16-byte load per thread (two for 1024 values) and the float64 arithmetic per thread is a handful of operations; the
// statistics cross the warps through shared memory. Same arithmetic as the warp-per-row kernel (two-pass variance,
// float64 statistics), different summation order of the float64 partial sums.
constexpr int LN_ROW_THREADS = 128;

template <int NV>  // float4 per thread
__global__ void __launch_bounds__(LN_ROW_THREADS) ln_quant_row_kernel(const ls100_ln_quant_args a, const float scale,
                                                                      const float rs) {
  __shared__ double s_part[2][LN_ROW_THREADS / 32];
  pdl_launch_dependents();
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int row = blockIdx.x;
  // gamma / beta do not depend on the previous kernel: fetched before the grid-dependency wait
  float4 g[NV], b[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * LN_ROW_THREADS + t) * 4;
    if (c < a.hidden) {
      g[i] = __ldg(reinterpret_cast<const float4*>(a.gamma + c));
      b[i] = __ldg(reinterpret_cast<const float4*>(a.beta + c));
    }
  }
  pdl_wait();
  float4 v[NV];
  double s = 0.0;
  if (a.emb.table_q != nullptr) {
    // decode-step embedding in place of the load (the arithmetic of embed_kernel's step form); the looked-up row is
    // also written out: it is the residual stream of the layer stack
    const ls100_embed_args& e = a.emb;
    const int step = *e.step_ptr;
    int id = e.ids[(long long)row * e.ld_ids + step];
    int pos = (e.pos_mode == 1 || id != e.pad_id) ? step : 0;
    const bool is_pad = (id == e.pad_id);
    if (id < 0 || id >= e.vocab) id = (e.pad_id >= 0 && e.pad_id < e.vocab) ? e.pad_id : 0;
    if (pos >= e.n_pos) pos = e.n_pos - 1;
    const int8_t* er = e.table_q + (long long)id * a.hidden;
    const float* pr = e.pos + (long long)pos * a.hidden;
    const float m = (is_pad && e.pos_mode == 0) ? 0.f : 1.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * LN_ROW_THREADS + t) * 4;
      if (c < a.hidden) {
        const char4 q = *reinterpret_cast<const char4*>(er + c);
        const float4 p = *reinterpret_cast<const float4*>(pr + c);
        v[i].x = __fadd_rn(__fmul_rn(e.sqrt_h, __fmul_rn((float)q.x, e.s_emb)), __fmul_rn(p.x, m));
        v[i].y = __fadd_rn(__fmul_rn(e.sqrt_h, __fmul_rn((float)q.y, e.s_emb)), __fmul_rn(p.y, m));
        v[i].z = __fadd_rn(__fmul_rn(e.sqrt_h, __fmul_rn((float)q.z, e.s_emb)), __fmul_rn(p.z, m));
        v[i].w = __fadd_rn(__fmul_rn(e.sqrt_h, __fmul_rn((float)q.w, e.s_emb)), __fmul_rn(p.w, m));
        *reinterpret_cast<float4*>(e.out + (long long)row * a.hidden + c) = v[i];
        s += ((double)v[i].x + (double)v[i].y) + ((double)v[i].z + (double)v[i].w);
      }
    }
  } else {
    const float* xr = a.x + (long long)row * a.ldx;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * LN_ROW_THREADS + t) * 4;
      if (c < a.hidden) {
        v[i] = *reinterpret_cast<const float4*>(xr + c);
        s += ((double)v[i].x + (double)v[i].y) + ((double)v[i].z + (double)v[i].w);
      }
    }
  }
  s = warp_sum_d(s);
  if (lane == 0) s_part[0][warp] = s;
  __syncthreads();
  const double mean = ((s_part[0][0] + s_part[0][1]) + (s_part[0][2] + s_part[0][3])) / (double)a.hidden;
  double sq = 0.0;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * LN_ROW_THREADS + t) * 4;
    if (c < a.hidden) {
      const double d0 = (double)v[i].x - mean, d1 = (double)v[i].y - mean;
      const double d2 = (double)v[i].z - mean, d3 = (double)v[i].w - mean;
      sq += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
  }
  sq = warp_sum_d(sq);
  if (lane == 0) s_part[1][warp] = sq;
  __syncthreads();
  const double var = ((s_part[1][0] + s_part[1][1]) + (s_part[1][2] + s_part[1][3])) / (double)a.hidden;
  const double rstd = 1.0 / sqrt(var + 1e-5);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = (i * LN_ROW_THREADS + t) * 4;
    if (c < a.hidden) {
      float4 y;
      y.x = __fadd_rn(__fmul_rn((float)(((double)v[i].x - mean) * rstd), g[i].x), b[i].x);
      y.y = __fadd_rn(__fmul_rn((float)(((double)v[i].y - mean) * rstd), g[i].y), b[i].y);
      y.z = __fadd_rn(__fmul_rn((float)(((double)v[i].z - mean) * rstd), g[i].z), b[i].z);
      y.w = __fadd_rn(__fmul_rn((float)(((double)v[i].w - mean) * rstd), g[i].w), b[i].w);
      if (a.out_f) *reinterpret_cast<float4*>(a.out_f + (long long)row * a.ldf + c) = y;
      if (a.out_q) {
        // (clamping to +-amax first, as the learned-amax quantiser does, cannot change the result: amax / scale is 127)
        const float2 q01 = f2_quant_biased(f2_div_rn(make_float2(y.x, y.y), f2_set(scale), f2_set(rs)));
        const float2 q23 = f2_quant_biased(f2_div_rn(make_float2(y.z, y.w), f2_set(scale), f2_set(rs)));
        *reinterpret_cast<uint32_t*>(a.out_q + (long long)row * a.ldq + c) = pack_biased_i8x4(q01.x, q01.y, q23.x, q23.y);
      }
    }
  }
}

// ------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(256) embed_kernel(const ls100_embed_args a) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int rows = a.batch * a.seq;
  if (warp >= rows) return;
  const int b = warp / a.seq, s = warp % a.seq;
  int id, pos;
  if (a.step_ptr) {
    const int step = *a.step_ptr;
    id = a.ids[(long long)b * a.ld_ids + step];
    pos = (a.pos_mode == 1 || id != a.pad_id) ? step : 0;
  } else {
    const int32_t* row = a.ids + (long long)b * a.ld_ids;
    id = row[s];
    if (a.pos_mode == 1) {
      pos = s;
    } else {
      // position = (#non-pad ids in row[0..s]) - 1, zero for pads
      int cnt = 0;
      for (int j = lane; j <= s; j += 32) cnt += (row[j] != a.pad_id) ? 1 : 0;
      cnt = warp_sum_i(cnt);
      pos = (id != a.pad_id) ? cnt - 1 : 0;
    }
  }
  const bool is_pad = (id == a.pad_id);
  if (a.pad_mask && lane == 0) a.pad_mask[warp] = is_pad ? 1 : 0;
  // out-of-range ids read the pad row (row 0 when there is no pad id) instead of faulting
  if (id < 0 || id >= a.vocab) id = (a.pad_id >= 0 && a.pad_id < a.vocab) ? a.pad_id : 0;
  if (pos >= a.n_pos) pos = a.n_pos - 1;
  const int8_t* er = a.table_q + (long long)id * a.hidden;
  const float* pr = a.pos + (long long)pos * a.hidden;
  float* orow = a.out + (long long)warp * a.hidden;
  const float m = (is_pad && a.pos_mode == 0) ? 0.f : 1.f;
  for (int c = lane * 4; c < a.hidden; c += 128) {
    const char4 q = *reinterpret_cast<const char4*>(er + c);
    const float4 p = *reinterpret_cast<const float4*>(pr + c);
    float4 y;
    y.x = __fadd_rn(__fmul_rn(a.sqrt_h, __fmul_rn((float)q.x, a.s_emb)), __fmul_rn(p.x, m));
    y.y = __fadd_rn(__fmul_rn(a.sqrt_h, __fmul_rn((float)q.y, a.s_emb)), __fmul_rn(p.y, m));
    y.z = __fadd_rn(__fmul_rn(a.sqrt_h, __fmul_rn((float)q.z, a.s_emb)), __fmul_rn(p.z, m));
    y.w = __fadd_rn(__fmul_rn(a.sqrt_h, __fmul_rn((float)q.w, a.s_emb)), __fmul_rn(p.w, m));
    *reinterpret_cast<float4*>(orow + c) = y;
  }
}

// ------------------------------------------------------------------ weight quantiser
__global__ void __launch_bounds__(256) quantize_weight_kernel(const float* __restrict__ w, long long rows,
                                                               long long cols, float amax, float scale, float rs,
                                                               int8_t* __restrict__ out, int32_t* __restrict__ off) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const float* wr = w + warp * cols;
  int8_t* orow = out + warp * cols;
  int sum = 0;
  for (long long c = lane * 4; c < cols; c += 128) {
    const float4 x = *reinterpret_cast<const float4*>(wr + c);
    const float q0 = quant_s(clipf(x.x, amax), scale, rs), q1 = quant_s(clipf(x.y, amax), scale, rs);
    const float q2 = quant_s(clipf(x.z, amax), scale, rs), q3 = quant_s(clipf(x.w, amax), scale, rs);
    sum += (int)q0 + (int)q1 + (int)q2 + (int)q3;
    *reinterpret_cast<uint32_t*>(orow + c) = pack_i8x4(q0, q1, q2, q3);
  }
  if (off) {
    sum = warp_sum_i(sum);
    if (lane == 0) off[warp] = 127 * sum;
  }
}

// ------------------------------------------------------------------ ViT patch embedding
// CTA = 16 consecutive tokens (of the flattened [batch, 1 + patches] list) x 256 hidden channels; a thread owns one
// channel and 16 float64 accumulators. The patch pixels are staged through shared memory 256 values at a time, already
// converted to float64 (read back as broadcasts), the transposed weight is read coalesced, once per CTA.
constexpr int PE_TOK = 16, PE_KC = 256;
__global__ void __launch_bounds__(256) patch_embed_kernel(const ls100_patch_embed_args a) {
  __shared__ double xs[PE_TOK][PE_KC];  // converted once while staging: the inner loop is one broadcast load and one DFMA per token
  pdl_launch_dependents();
  pdl_wait();
  const int grid_w = a.image / a.patch, n_patch = grid_w * grid_w, seq = n_patch + 1;
  const int K = a.channels * a.patch * a.patch, pp = a.patch * a.patch;
  const long long tokens = (long long)a.batch * seq;
  const long long t0 = (long long)blockIdx.x * PE_TOK;
  const int h = blockIdx.y * 256 + threadIdx.x;
  double acc[PE_TOK];
#pragma unroll
  for (int p = 0; p < PE_TOK; ++p) acc[p] = 0.0;
  for (int k0 = 0; k0 < K; k0 += PE_KC) {
    __syncthreads();
    for (int id = threadIdx.x; id < PE_TOK * PE_KC; id += 256) {
      const int p = id / PE_KC, kk = id % PE_KC, k = k0 + kk;
      const long long tok = t0 + p;
      float v = 0.f;
      if (tok < tokens && k < K) {
        const int b = (int)(tok / seq), n = (int)(tok % seq);
        if (n > 0) {
          const int pr = (n - 1) / grid_w, pc = (n - 1) % grid_w;
          const int c = k / pp, r = (k % pp) / a.patch, q = k % a.patch;
          v = __ldg(a.pixels + (((long long)b * a.channels + c) * a.image + (pr * a.patch + r)) * a.image + pc * a.patch + q);
        }
      }
      xs[p][kk] = (double)v;
    }
    __syncthreads();
    if (h < a.hidden) {
      const int kn = min(PE_KC, K - k0);
      for (int kk = 0; kk < kn; ++kk) {
        const double w = (double)__ldg(a.conv_wt + (long long)(k0 + kk) * a.hidden + h);
#pragma unroll
        for (int p = 0; p < PE_TOK; ++p) acc[p] = fma(xs[p][kk], w, acc[p]);
      }
    }
  }
  if (h >= a.hidden) return;
  const float bias = __ldg(a.conv_bias + h), cls = __ldg(a.cls + h);
#pragma unroll
  for (int p = 0; p < PE_TOK; ++p) {
    const long long tok = t0 + p;
    if (tok >= tokens) break;
    const int n = (int)(tok % seq);
    const float pos = __ldg(a.pos + (long long)n * a.hidden + h);
    a.out[tok * a.hidden + h] = n == 0 ? __fadd_rn(cls, pos) : __fadd_rn(__fadd_rn((float)acc[p], bias), pos);
  }
}

}  // namespace ls100

using namespace ls100;

extern "C" int ls100_ln_quant(ls100_ctx* ctx, const ls100_ln_quant_args* a, ls100_stream_t stream_) {
  const bool lookup = a && a->emb.table_q != nullptr;
  if (!ctx || !a || (!a->x && !lookup) || !a->gamma || !a->beta || (!a->out_q && !a->out_f)) return LS100_ERR_BAD_ARG;
  if (lookup) {  // the decode-step form of ls100_embed feeding the LayerNorm directly
    const ls100_embed_args& e = a->emb;
    if (!e.ids || !e.pos || !e.out || !e.step_ptr || e.seq != 1 || e.batch != a->rows || e.hidden != a->hidden || e.n_pos <= 0 ||
        e.vocab <= 0 || e.pad_mask != nullptr)
      return LS100_ERR_BAD_ARG;
    if (a->rows > 2048) return LS100_ERR_UNSUPPORTED;
    if ((((uintptr_t)e.table_q) & 3) || (((uintptr_t)e.pos) & 15) || (((uintptr_t)e.out) & 15)) return LS100_ERR_ALIGN;
  }
  if (a->rows <= 0 || a->hidden <= 0) return LS100_ERR_BAD_ARG;
  if ((a->hidden & 3) || a->hidden > LN_MAXV * 128) return LS100_ERR_UNSUPPORTED;
  if (a->out_q && !(a->amax > 0.f)) return LS100_ERR_BAD_ARG;
  if ((!lookup && ((((uintptr_t)a->x) & 15) || (a->ldx & 3))) || (((uintptr_t)a->gamma) & 15) || (((uintptr_t)a->beta) & 15))
    return LS100_ERR_ALIGN;
  if (a->out_q && ((((uintptr_t)a->out_q) & 3) || (a->ldq & 3))) return LS100_ERR_ALIGN;
  if (a->out_f && ((((uintptr_t)a->out_f) & 15) || (a->ldf & 3))) return LS100_ERR_ALIGN;
  cudaStream_t stream = (cudaStream_t)stream_;
  const float scale = a->amax / 127.0f;
  const int warps_per_block = 8;
  const int blocks = (a->rows + warps_per_block - 1) / warps_per_block;
  const int nv = (a->hidden + 127) / 128;
  const float rs = 1.0f / scale;
  cudaError_t e;
  if (a->rows <= 2048) {  // decode-step sizes: a CTA per row (at 16384 rows it times the same as a warp per row)
    const int nvr = (a->hidden + 4 * LN_ROW_THREADS - 1) / (4 * LN_ROW_THREADS);
    if (nvr <= 1) e = ls100_launch(ln_quant_row_kernel<1>, dim3(a->rows), dim3(LN_ROW_THREADS), 0, stream, *a, scale, rs);
    else if (nvr <= 2) e = ls100_launch(ln_quant_row_kernel<2>, dim3(a->rows), dim3(LN_ROW_THREADS), 0, stream, *a, scale, rs);
    else if (nvr <= 4) e = ls100_launch(ln_quant_row_kernel<4>, dim3(a->rows), dim3(LN_ROW_THREADS), 0, stream, *a, scale, rs);
    else e = ls100_launch(ln_quant_row_kernel<8>, dim3(a->rows), dim3(LN_ROW_THREADS), 0, stream, *a, scale, rs);
    return e == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
  }
  if (nv <= 4) e = ls100_launch(ln_quant_kernel<4>, dim3(blocks), dim3(256), 0, stream, *a, scale, rs);
  else if (nv <= 6) e = ls100_launch(ln_quant_kernel<6>, dim3(blocks), dim3(256), 0, stream, *a, scale, rs);
  else if (nv <= 8) e = ls100_launch(ln_quant_kernel<8>, dim3(blocks), dim3(256), 0, stream, *a, scale, rs);
  else if (nv <= 16) e = ls100_launch(ln_quant_kernel<16>, dim3(blocks), dim3(256), 0, stream, *a, scale, rs);
  else e = ls100_launch(ln_quant_kernel<32>, dim3(blocks), dim3(256), 0, stream, *a, scale, rs);
  return e == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

extern "C" int ls100_embed(ls100_ctx* ctx, const ls100_embed_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->ids || !a->table_q || !a->pos || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->seq <= 0 || a->hidden <= 0 || a->n_pos <= 0 || a->vocab <= 0) return LS100_ERR_BAD_ARG;
  if (a->step_ptr && a->seq != 1) return LS100_ERR_BAD_ARG;
  if (a->hidden & 3) return LS100_ERR_UNSUPPORTED;
  if ((((uintptr_t)a->table_q) & 3) || (((uintptr_t)a->pos) & 15) || (((uintptr_t)a->out) & 15)) return LS100_ERR_ALIGN;
  const int rows = a->batch * a->seq;
  return ls100_launch(embed_kernel, dim3((rows + 7) / 8), dim3(256), 0, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_patch_embed(ls100_ctx* ctx, const ls100_patch_embed_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->pixels || !a->conv_wt || !a->conv_bias || !a->pos || !a->cls || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->channels <= 0 || a->image <= 0 || a->patch <= 0 || a->hidden <= 0) return LS100_ERR_BAD_ARG;
  if (a->image % a->patch) return LS100_ERR_BAD_ARG;
  if (a->hidden & 3) return LS100_ERR_UNSUPPORTED;
  const long long g = a->image / a->patch, tokens = (long long)a->batch * (g * g + 1);
  const long long bx = (tokens + PE_TOK - 1) / PE_TOK;
  if (bx > 0x7fffffffll) return LS100_ERR_UNSUPPORTED;
  return ls100_launch(patch_embed_kernel, dim3((unsigned)bx, (unsigned)((a->hidden + 255) / 256)), dim3(256), 0, (cudaStream_t)stream_,
                      *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_quantize_weight(ls100_ctx* ctx, const float* w, int64_t rows, int64_t cols, float amax,
                                     int8_t* out_q, int32_t* row_off, ls100_stream_t stream_) {
  if (!ctx || !w || !out_q || rows <= 0 || cols <= 0 || !(amax > 0.f)) return LS100_ERR_BAD_ARG;
  if (cols & 3) return LS100_ERR_UNSUPPORTED;
  if ((((uintptr_t)w) & 15) || (((uintptr_t)out_q) & 3)) return LS100_ERR_ALIGN;
  const float scale = amax / 127.0f;
  const long long blocks = (rows + 7) / 8;
  quantize_weight_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream_>>>(w, rows, cols, amax, scale, 1.0f / scale, out_q,
                                                                               row_off);
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}
