/*
 * ls100 — C ABI of the B200 (sm_100a) int8 Transformer inference kernels.
 *
 * Every entry point takes caller-owned DEVICE pointers (unless the name ends in
 * `_host`), plain sizes and fp32 scales by value, launches on the given stream
 * and returns 0 or a negative LS100_ERR_* code without launching. Nothing here
 * synchronises or allocates unless its comment says so. `stream` is a
 * cudaStream_t passed as void*.
 *
 * Each declaration cites the reference interface it replaces (paths are
 * relative to the bytedance/lightseq source tree).
 *
 * Quantiser convention (lightseq/training/pytorch_quantization/tensor_quant.py:349-409):
 *   scale = amax/127 (unsigned: amax/254); q = clamp(floor(x/scale + 0.5), -127, 127)
 *   (unsigned: x/scale - 127 before rounding); fake value = q*scale (unsigned: (q+127)*scale).
 */
#ifndef LS100_H_
#define LS100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LS100_OK 0
#define LS100_ERR_BAD_ARG (-1)
#define LS100_ERR_ALIGN (-2)
#define LS100_ERR_UNSUPPORTED (-3)
#define LS100_ERR_CUDA (-4)
#define LS100_ERR_TIMEOUT (-5)
#define LS100_ERR_NO_DRIVER (-6)

typedef struct ls100_ctx ls100_ctx;
typedef void* ls100_stream_t;

/* Context: device id, SM count, tensor-map cache, device error word.
 * Replaces the per-model cublasLt handle + stream set-up of
 * lightseq/inference/pywrapper/quant_transformer.cc:8-71.
 * Create/destroy allocate/free a few bytes of device memory; nothing else does. */
int ls100_ctx_create(ls100_ctx** out, int device);
void ls100_ctx_destroy(ls100_ctx* ctx);
const char* ls100_strerror(int code);
/* Synchronises `stream`, returns (and clears) the device error word: 0, or
 * LS100_ERR_TIMEOUT if a kernel's bounded wait gave up. */
int ls100_ctx_poll_error(ls100_ctx* ctx, ls100_stream_t stream);
int ls100_sm_count(const ls100_ctx* ctx);

/* ------------------------------------------------------------------ GEMM ---
 * out[M,N] = epilogue( A_i8[M,K] . W_i8[N,K]^T ), int32 accumulation in TMEM
 * (tcgen05.mma kind::i8), fused epilogue. Replaces cublaslt_gemm /
 * cublasLtMM_withAlgo_i8IO (lightseq/inference/model/cublas_helper.cc:31-483)
 * and the elementwise kernels that follow each call in
 * lightseq/inference/model/quant_encoder.cc.cu:289-460 (ker_arrange_*_qkv,
 * ker_bias_{relu,gelu}_i8I_i8O, ker_residual_bias_ln_*), restating
 * QuantLinear.forward (lightseq/training/ops/pytorch/quantization.py:50-61).
 *
 * Per element (every step a separately rounded fp32 operation):
 *   a = acc + (w_off ? w_off[n] : 0)                  int32
 *   v = float(a) * s_acc
 *   if s_outq > 0: q = quant(v, s_outq); v = q * s_outq   (output fake-quant)
 *   if bias: v += bias[n];  act: relu / erf-gelu;  if resid: v += resid[m,n]
 *   out_kind: OUTQ_I8 stores q (before bias);  F32 / F16 store v;
 *             REQ_S8 stores quant(v, s_req);  REQ_U8 stores the unsigned quantiser's q.
 */
enum {
  LS100_OUT_OUTQ_I8 = 0,
  LS100_OUT_F32 = 1,
  LS100_OUT_REQ_S8 = 2,
  LS100_OUT_REQ_U8 = 3,
  LS100_OUT_F16 = 4,
  LS100_OUT_I32 = 5 /* raw accumulators (+w_off) */
};
enum { LS100_ACT_NONE = 0, LS100_ACT_RELU = 1, LS100_ACT_GELU = 2 };

typedef struct {
  const int8_t* a; /* [M,K], K contiguous */
  int64_t lda;     /* bytes between rows, multiple of 16 */
  const int8_t* w; /* [N,K], K contiguous (torch Linear layout) */
  int64_t ldw;
  int32_t m, n, k;
  float s_acc;          /* s_in * s_w */
  const int32_t* w_off; /* optional [N] */
  float s_outq;         /* > 0 enables the output fake-quant */
  const float* bias;    /* optional [N] */
  int32_t act;
  const float* resid; /* optional [M,N] fp32 */
  int64_t ldr;        /* elements */
  int32_t out_kind;
  float s_req;
  void* out;
  int64_t ldo; /* elements */
} ls100_gemm_i8_args;

int ls100_gemm_i8(ls100_ctx* ctx, const ls100_gemm_i8_args* args, ls100_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LS100_H_ */
