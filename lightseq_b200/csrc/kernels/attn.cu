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
#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr int DH = 64;

__device__ __forceinline__ void unpack16(const int4 v, float (&f)[16]) {
  const int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i * 4 + 0] = (float)(int8_t)(w[i] & 0xff);
    f[i * 4 + 1] = (float)(int8_t)((w[i] >> 8) & 0xff);
    f[i * 4 + 2] = (float)(int8_t)((w[i] >> 16) & 0xff);
    f[i * 4 + 3] = (float)(int8_t)((w[i] >> 24) & 0xff);
  }
}

// ------------------------------------------------------------------ attn_self
__global__ void __launch_bounds__(64) attn_self_kernel(const ls100_attn_self_args a, const float s_out, const float rs_out) {
  __shared__ __align__(16) float Ks[64][DH];
  __shared__ __align__(16) float Vs[64][DH];
  __shared__ uint8_t msk[64];
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
__global__ void __launch_bounds__(128) attn_dec_kernel(const ls100_attn_dec_args a, const float s_out,
                                                        const float rs_out, const float score_scale) {
  extern __shared__ float sc_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wid = blockIdx.x * 4 + warp;
  if (wid >= a.rows * a.heads) return;
  const int r = wid / a.heads, h = wid % a.heads;
  const int hidden = a.heads * DH;
  const int step = *a.step_ptr;
  const int L = step + 1;
  float* sc = sc_all + warp * a.max_step;
  const int g = lane >> 2, c = lane & 3;
  const int8_t* row = a.qkv + (long long)r * a.ld_qkv + h * DH + c * 16;
  const int4 q4 = *reinterpret_cast<const int4*>(row);
  const int4 knew = *reinterpret_cast<const int4*>(row + hidden);
  const int4 vnew = *reinterpret_cast<const int4*>(row + 2 * hidden);
  const long long own = (((long long)r * a.heads + h) * a.max_step + step) * DH + c * 16;
  if (g == 0) *reinterpret_cast<int4*>(a.k_cache + own) = knew;
  if (g == 1) *reinterpret_cast<int4*>(a.v_cache + own) = vnew;
  const int32_t* anc = a.anc ? a.anc + (long long)r * a.max_step : nullptr;

  // scores: 8 positions per pass, 4 lanes per position
  for (int p0 = 0; p0 < L; p0 += 8) {
    const int p = p0 + g;
    int dot = 0;
    if (p < L) {
      int4 k4;
      if (p == step) k4 = knew;
      else {
        const int slot = anc ? anc[p] : r;
        k4 = *reinterpret_cast<const int4*>(a.k_cache + (((long long)slot * a.heads + h) * a.max_step + p) * DH + c * 16);
      }
      dot = __dp4a(q4.x, k4.x, dot);
      dot = __dp4a(q4.y, k4.y, dot);
      dot = __dp4a(q4.z, k4.z, dot);
      dot = __dp4a(q4.w, k4.w, dot);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    if (p < L && c == 0) sc[p] = (float)dot * score_scale;
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int p = lane; p < L; p += 32) mx = fmaxf(mx, sc[p]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int p = lane; p < L; p += 32) {
    const float e = expf(sc[p] - mx);
    sc[p] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  __syncwarp();
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  for (int p0 = 0; p0 < L; p0 += 8) {
    const int p = p0 + g;
    if (p < L) {
      int4 v4;
      if (p == step) v4 = vnew;
      else {
        const int slot = anc ? anc[p] : r;
        v4 = *reinterpret_cast<const int4*>(a.v_cache + (((long long)slot * a.heads + h) * a.max_step + p) * DH + c * 16);
      }
      float f[16];
      unpack16(v4, f);
      const float w = sc[p];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = fmaf(w, f[j], acc[j]);
    }
  }
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
// One CTA per (batch, head), one warp per beam; encoder keys/values are fp32 rows of 64
// floats: 16 lanes x 16 bytes cover a row, two rows per pass.
__global__ void __launch_bounds__(256) attn_cross_kernel(const ls100_attn_cross_args a, const float s_out, const float rs_out) {
  extern __shared__ float sc_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= a.beam) return;
  const int b = blockIdx.x, h = blockIdx.y;
  const int r = b * a.beam + warp;
  const int S = a.src_len;
  float* sc = sc_all + warp * S;
  const int g = lane >> 4, c = lane & 15;
  float qf[4];
  {
    const int8_t* qp = a.q + (long long)r * a.ld_q + h * DH + c * 4;
    const int w = *reinterpret_cast<const int*>(qp);
#pragma unroll
    for (int j = 0; j < 4; ++j) qf[j] = __fmul_rn((float)(int8_t)((w >> (j * 8)) & 0xff), a.s_q);
    if (a.bias) {
      const float4 bb = __ldg(reinterpret_cast<const float4*>(a.bias + h * DH + c * 4));
      qf[0] = __fadd_rn(qf[0], bb.x);
      qf[1] = __fadd_rn(qf[1], bb.y);
      qf[2] = __fadd_rn(qf[2], bb.z);
      qf[3] = __fadd_rn(qf[3], bb.w);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) qf[j] = __fmul_rn(qf[j], 0.125f);
  }
  const float* kb = reinterpret_cast<const float*>(a.k) + (long long)b * S * a.ld_kv + h * DH + c * 4;
  const float* vb = reinterpret_cast<const float*>(a.v) + (long long)b * S * a.ld_kv + h * DH + c * 4;
  const uint8_t* pm = a.pad_mask ? a.pad_mask + (long long)b * S : nullptr;
  for (int j0 = 0; j0 < S; j0 += 2) {
    const int j = j0 + g;
    float s = 0.f;
    const bool ok = (j < S) && !(pm && pm[j]);
    if (ok) {
      const float4 k4 = *reinterpret_cast<const float4*>(kb + (long long)j * a.ld_kv);
      s = fmaf(qf[0], k4.x, s);
      s = fmaf(qf[1], k4.y, s);
      s = fmaf(qf[2], k4.z, s);
      s = fmaf(qf[3], k4.w, s);
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s += __shfl_xor_sync(0xffffffffu, s, 8);
    if (j < S && c == 0) sc[j] = ok ? s : -INFINITY;
  }
  __syncwarp();
  float mx = -INFINITY;
  for (int j = lane; j < S; j += 32) mx = fmaxf(mx, sc[j]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int j = lane; j < S; j += 32) {
    const float e = (sc[j] == -INFINITY) ? 0.f : expf(sc[j] - mx);
    sc[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  __syncwarp();
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j0 = 0; j0 < S; j0 += 2) {
    const int j = j0 + g;
    if (j < S) {
      const float w = sc[j];
      if (w != 0.f) {
        const float4 v4 = *reinterpret_cast<const float4*>(vb + (long long)j * a.ld_kv);
        acc[0] = fmaf(w, v4.x, acc[0]);
        acc[1] = fmaf(w, v4.y, acc[1]);
        acc[2] = fmaf(w, v4.z, acc[2]);
        acc[3] = fmaf(w, v4.w, acc[3]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 16);
  if (g == 0) {
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    const uint32_t u = pack_i8x4(quant_s(clipf(acc[0] * inv, a.amax_out), s_out, rs_out),
                                 quant_s(clipf(acc[1] * inv, a.amax_out), s_out, rs_out),
                                 quant_s(clipf(acc[2] * inv, a.amax_out), s_out, rs_out),
                                 quant_s(clipf(acc[3] * inv, a.amax_out), s_out, rs_out));
    *reinterpret_cast<uint32_t*>(a.out + (long long)r * a.ld_out + h * DH + c * 4) = u;
  }
}

}  // namespace ls100

using namespace ls100;

extern "C" int ls100_attn_self(ls100_ctx* ctx, const ls100_attn_self_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->qkv || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->seq <= 0 || a->heads <= 0 || !(a->amax_out > 0.f) || !(a->s_qkv > 0.f)) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->qkv) & 15) || (a->ld_qkv & 15) || (((uintptr_t)a->out) & 15) || (a->ld_out & 15)) return LS100_ERR_ALIGN;
  if (a->ld_qkv < 3 * a->heads * DH || a->ld_out < a->heads * DH) return LS100_ERR_BAD_ARG;
  if ((a->k_cache != nullptr) != (a->v_cache != nullptr)) return LS100_ERR_BAD_ARG;
  if (a->k_cache && (a->bias || a->max_step < a->seq || (((uintptr_t)a->k_cache) & 15) || (((uintptr_t)a->v_cache) & 15)))
    return LS100_ERR_BAD_ARG;
  if (a->heads > 65535 || a->batch > 65535) return LS100_ERR_UNSUPPORTED;
  dim3 grid((a->seq + 63) / 64, a->heads, a->batch);
  attn_self_kernel<<<grid, 64, 0, (cudaStream_t)stream_>>>(*a, a->amax_out / 127.0f, 1.0f / (a->amax_out / 127.0f));
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

extern "C" int ls100_attn_dec(ls100_ctx* ctx, const ls100_attn_dec_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->qkv || !a->k_cache || !a->v_cache || !a->step_ptr || !a->out) return LS100_ERR_BAD_ARG;
  if (a->rows <= 0 || a->heads <= 0 || a->max_step <= 0 || !(a->amax_out > 0.f) || !(a->s_kv > 0.f)) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->qkv) & 15) || (a->ld_qkv & 15) || (((uintptr_t)a->out) & 15) || (a->ld_out & 15) ||
      (((uintptr_t)a->k_cache) & 15) || (((uintptr_t)a->v_cache) & 15))
    return LS100_ERR_ALIGN;
  if (a->max_step > 2048) return LS100_ERR_UNSUPPORTED;
  const long long warps = (long long)a->rows * a->heads;
  const float score_scale = (a->s_kv * a->s_kv) * 0.125f;
  attn_dec_kernel<<<(unsigned)((warps + 3) / 4), 128, 4 * a->max_step * sizeof(float), (cudaStream_t)stream_>>>(
      *a, a->amax_out / 127.0f, 1.0f / (a->amax_out / 127.0f), score_scale);
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}

extern "C" int ls100_attn_cross(ls100_ctx* ctx, const ls100_attn_cross_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->q || !a->k || !a->v || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->src_len <= 0 || a->heads <= 0 || !(a->amax_out > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->beam > 8 || a->src_len > 4096 || a->heads > 65535) return LS100_ERR_UNSUPPORTED;
  if ((((uintptr_t)a->q) & 3) || (a->ld_q & 3) || (((uintptr_t)a->k) & 15) || (((uintptr_t)a->v) & 15) || (a->ld_kv & 3) ||
      (((uintptr_t)a->out) & 3) || (a->ld_out & 3))
    return LS100_ERR_ALIGN;
  dim3 grid(a->batch, a->heads);
  attn_cross_kernel<<<grid, 32 * a->beam, (size_t)a->beam * a->src_len * sizeof(float), (cudaStream_t)stream_>>>(
      *a, a->amax_out / 127.0f, 1.0f / (a->amax_out / 127.0f));
  return cudaGetLastError() == cudaSuccess ? LS100_OK : LS100_ERR_CUDA;
}
