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
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wid = blockIdx.x * 4 + warp;
  if (wid >= a.rows * a.heads) return;
  const int r = wid / a.heads, h = wid % a.heads;
  const int hidden = a.heads * DH;
  const int step = *a.step_ptr;
  const int L = step + 1;
  int* slot_s = slot_all + warp * a.max_step;
  const int g = lane >> 2, c = lane & 3;
  {
    const int32_t* anc = a.anc ? a.anc + (long long)r * a.max_step : nullptr;
    for (int p = lane; p < L; p += 32) slot_s[p] = (anc && p < step) ? anc[p] : r;
  }
  const int8_t* row = a.qkv + (long long)r * a.ld_qkv + h * DH + c * 16;
  const int4 q4 = *reinterpret_cast<const int4*>(row);
  const int4 knew = *reinterpret_cast<const int4*>(row + hidden);
  const int4 vnew = *reinterpret_cast<const int4*>(row + 2 * hidden);
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
  for (int p0 = 0; p0 < L; p0 += 32) {
    int4 k4[4], v4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int p = p0 + u * 8 + g;
      k4[u] = make_int4(0, 0, 0, 0);
      v4[u] = make_int4(0, 0, 0, 0);
      if (p < step) {
        const long long o = slot_s[p] * slot_stride + head_off + (long long)p * DH;
        k4[u] = *reinterpret_cast<const int4*>(a.k_cache + o);
        v4[u] = *reinterpret_cast<const int4*>(a.v_cache + o);
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
// One CTA per (batch, head), one warp per beam. The head's fp32 keys and values are staged in
// shared memory once per 128-key tile with coalesced 16-byte loads (all loads in flight
// together, then shared by the beams), scores use one key per lane, the PV product two head
// dims per lane; tiles are merged with an online softmax.
constexpr int XT = 128;      // keys per tile
constexpr int XKS = DH + 1;  // padded key row (conflict-free when lanes read different rows)

__global__ void __launch_bounds__(256) attn_cross_kernel(const ls100_attn_cross_args a, const float s_out, const float rs_out,
                                                          const int tr /* tile rows held in shared memory, <= XT */) {
  extern __shared__ float xs[];
  pdl_launch_dependents();
  pdl_wait();
  float* Ks = xs;                    // [tr][XKS]
  float* Vs = Ks + tr * XKS;         // [tr][DH]
  float* qs = Vs + tr * DH;          // [beam][DH]
  float* ps = qs + a.beam * DH;      // [beam][tr]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, h = blockIdx.y;
  const int r = b * a.beam + warp;
  const int S = a.src_len;
  {  // q of this beam -> shared memory, dequantised, biased, scaled
    const int8_t* qp = a.q + (long long)r * a.ld_q + h * DH + lane * 2;
    const short w = *reinterpret_cast<const short*>(qp);
    float q0 = __fmul_rn((float)(int8_t)(w & 0xff), a.s_q), q1 = __fmul_rn((float)(int8_t)((w >> 8) & 0xff), a.s_q);
    if (a.bias) {
      const float2 bb = __ldg(reinterpret_cast<const float2*>(a.bias + h * DH + lane * 2));
      q0 = __fadd_rn(q0, bb.x);
      q1 = __fadd_rn(q1, bb.y);
    }
    qs[warp * DH + lane * 2] = __fmul_rn(q0, 0.125f);
    qs[warp * DH + lane * 2 + 1] = __fmul_rn(q1, 0.125f);
  }
  const float* kb = reinterpret_cast<const float*>(a.k) + (long long)b * S * a.ld_kv + h * DH;
  const float* vb = reinterpret_cast<const float*>(a.v) + (long long)b * S * a.ld_kv + h * DH;
  const uint8_t* pm = a.pad_mask ? a.pad_mask + (long long)b * S : nullptr;
  float m = -INFINITY, l = 0.f, acc0 = 0.f, acc1 = 0.f;
  for (int t0 = 0; t0 < S; t0 += tr) {
    const int ns = min(tr, S - t0);
    __syncthreads();
    for (int i0 = threadIdx.x; i0 < ns * 16; i0 += 4 * blockDim.x) {
      float4 k4[4], v4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {  // 8 x 16-byte loads in flight per thread before any store
        const int i = i0 + u * blockDim.x;
        if (i < ns * 16) {
          const int row = i >> 4, c4 = (i & 15) * 4;
          k4[u] = *reinterpret_cast<const float4*>(kb + (long long)(t0 + row) * a.ld_kv + c4);
          v4[u] = *reinterpret_cast<const float4*>(vb + (long long)(t0 + row) * a.ld_kv + c4);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < ns * 16) {
          const int row = i >> 4, c4 = (i & 15) * 4;
          float* kd = Ks + row * XKS + c4;
          kd[0] = k4[u].x;
          kd[1] = k4[u].y;
          kd[2] = k4[u].z;
          kd[3] = k4[u].w;
          *reinterpret_cast<float4*>(Vs + row * DH + c4) = v4[u];
        }
      }
    }
    __syncthreads();
    // scores: lane handles keys lane, lane+32, ...
    float sc[XT / 32];
    float tmax = -INFINITY;
#pragma unroll
    for (int u = 0; u < XT / 32; ++u) {
      const int j = u * 32 + lane;
      float sv = -INFINITY;
      if (j < ns && !(pm && pm[t0 + j])) {
        sv = 0.f;
        const float* kr = Ks + j * XKS;
        const float* qr = qs + warp * DH;
#pragma unroll
        for (int d = 0; d < DH; d += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + d);
          sv = fmaf(q4.x, kr[d], sv);
          sv = fmaf(q4.y, kr[d + 1], sv);
          sv = fmaf(q4.z, kr[d + 2], sv);
          sv = fmaf(q4.w, kr[d + 3], sv);
        }
      }
      sc[u] = sv;
      tmax = fmaxf(tmax, sv);
    }
    tmax = warp_max(tmax);
    if (tmax == -INFINITY) continue;  // whole tile masked (uniform across the warp)
    const float m_new = fmaxf(m, tmax);
    const float resc = __expf(m - m_new);  // 0 when m = -inf
    l *= resc;
    acc0 *= resc;
    acc1 *= resc;
    m = m_new;
    float lsum = 0.f;
#pragma unroll
    for (int u = 0; u < XT / 32; ++u) {
      const int j = u * 32 + lane;
      const float e = (sc[u] == -INFINITY) ? 0.f : expf(sc[u] - m);
      if (j < tr) ps[warp * tr + j] = e;
      lsum += e;
    }
    l += warp_sum(lsum);
    __syncwarp();
    const float* pr = ps + warp * tr;
    for (int j = 0; j < ns; ++j) {
      const float w = pr[j];
      const float2 v2 = *reinterpret_cast<const float2*>(Vs + j * DH + lane * 2);
      acc0 = fmaf(w, v2.x, acc0);
      acc1 = fmaf(w, v2.y, acc1);
    }
    __syncwarp();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const float o0 = quant_s(clipf(acc0 * inv, a.amax_out), s_out, rs_out);
  const float o1 = quant_s(clipf(acc1 * inv, a.amax_out), s_out, rs_out);
  const uint32_t pk = pack_i8x4(o0, o1, 0.f, 0.f);
  *reinterpret_cast<unsigned short*>(a.out + (long long)r * a.ld_out + h * DH + lane * 2) = (unsigned short)(pk & 0xffff);
}

}  // namespace ls100

using namespace ls100;

// Opts the cross-attention kernel into its largest shared-memory tile on the current device
// (called once from ls100_ctx_create, never inside a stream capture).
int ls100_attn_init_device() {
  const size_t smem = (size_t)(XT * XKS + XT * DH + 8 * DH + 8 * XT) * sizeof(float);
  return cudaFuncSetAttribute(attn_cross_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
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
  if (a->max_step > 2048) return LS100_ERR_UNSUPPORTED;  // 4 * max_step * 4 bytes of shared memory per CTA
  const long long warps = (long long)a->rows * a->heads;
  const float score_scale = (a->s_kv * a->s_kv) * 0.125f;
  const float so = a->amax_out / 127.0f;
  return ls100_launch(attn_dec_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 4 * a->max_step * sizeof(int),
                      (cudaStream_t)stream_, *a, so, 1.0f / so, score_scale) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_attn_cross(ls100_ctx* ctx, const ls100_attn_cross_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->q || !a->k || !a->v || !a->out) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->src_len <= 0 || a->heads <= 0 || !(a->amax_out > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->beam > 8 || a->src_len > 4096 || a->heads > 65535) return LS100_ERR_UNSUPPORTED;
  if ((((uintptr_t)a->q) & 1) || (a->ld_q & 1) || (((uintptr_t)a->k) & 15) || (((uintptr_t)a->v) & 15) || (a->ld_kv & 3) ||
      (((uintptr_t)a->out) & 1) || (a->ld_out & 1) || (a->bias && (((uintptr_t)a->bias) & 7)))
    return LS100_ERR_ALIGN;
  dim3 grid(a->batch, a->heads);
  // 32-key tiles keep a CTA at ~17 KB of shared memory, so that every (sentence, head) CTA of a large batch is
  // resident at once and the tile loads of one CTA overlap the arithmetic of the others
  const int tr = 32;
  const size_t smem = (size_t)(tr * XKS + tr * DH + a->beam * DH + a->beam * tr) * sizeof(float);
  const float so = a->amax_out / 127.0f;
  return ls100_launch(attn_cross_kernel, grid, dim3(32 * a->beam), smem, (cudaStream_t)stream_, *a, so, 1.0f / so, tr) ==
                 cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}
