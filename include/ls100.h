/*
 * ls100 — C ABI of the B200 (sm_100a) int8 Transformer inference kernels.
 *
 * Every entry point takes caller-owned DEVICE pointers (unless the name ends in
 * `_host`), plain sizes and fp32 scales by value, launches on the given stream
 * and returns 0 or a negative LS100_ERR_* code without launching. Nothing here
 * synchronises or allocates unless its comment says so. `stream` is a
 * cudaStream_t passed as void*. Zero-initialise every `*_args` struct before
 * filling it in: optional members (and members added in later versions) are
 * off when zero.
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
  const int8_t* w; /* [N,K], K contiguous (torch Linear layout). A weight: it, w_off, bias and req_table must be complete
                      before a full stream dependency that precedes this launch (they are what load-time preparation
                      wrote); the kernels fetch their first tiles of w ahead of the grid dependency on the preceding
                      kernel, which orders only a, resid and the outputs. */
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
  /* Optional fused LayerNorm + quantise of the finished rows (out_kind F32 only): when ln_out is not NULL,
   * ln_out[M,N] = quant(LayerNorm(out row; ln_gamma, ln_beta, eps 1e-5), ln_amax) as ls100_ln_quant computes it
   * (float64 statistics), in the same launch: the CTAs of a 128-row block form a thread-block cluster and exchange
   * the row sums through distributed shared memory. Replaces the LayerNorm half of ker_residual_bias_ln_i8I_i8O /
   * ker_residual_bias_ln_i32I_i8O (lightseq/inference/kernels/transformerKernels_int8.cc.cu:318-700) that follows
   * every attention-out and FFN2 GEMM. Shapes the cluster form does not cover (N > 1024 or N not a multiple
   * of 32) run as this GEMM followed by ls100_ln_quant. Measured on B200 at 512 x 512 x 512 the fused launch takes
   * 12.1 us against 4.5 + 2.9 us for the two separate kernels (the float64 row sums and the two cluster barriers
   * sit on the critical path of a 32-CTA grid), so the model drivers keep the separate kernels. */
  const float* ln_gamma; /* [N] */
  const float* ln_beta;  /* [N] */
  float ln_amax;
  int8_t* ln_out;
  int64_t ln_ldq; /* elements */
  /* Optional per-row statistics of an OUTQ_I8 output (the logits of a beam-search step), taken from the registers of
   * the epilogue so that the selection that follows need not read the [M,N] matrix again: for every row and every
   * group of 64 consecutive columns, the largest int8 value of the group (-128 for a group beyond N) and
   * sum_j exp((q_j - 127) * s_outq). Layout of both arrays: [ceil(M/128)][ceil(N/64)][128] (the 128 rows of a row
   * block contiguous). Replaces the log-sum-exp pass of select_beam_rough_topk_i8I
   * (lightseq/inference/kernels/transformerKernels_int8.cc.cu:1718-1760). Both or neither. */
  int8_t* stat_max;
  float* stat_sum;
  /* Optional table of everything after the output quantiser, for REQ_S8 / REQ_U8 outputs with the output quantiser on
   * and no residual: the quantised output takes 255 values, so bias, activation and requantisation are a function
   * of (column, value) that ls100_gemm_i8_build_table evaluates once per weight matrix. The many-tile kernel then
   * reads it from shared memory instead of computing it per element (about a third of the epilogue's instructions
   * for bias + requantise, a fifth with the erf GELU); the one-tile kernels ignore it. Results are identical either
   * way. 16-byte aligned, ls100_gemm_i8_table_bytes(n) bytes, built with the same s_outq, bias, act, out_kind, s_req. */
  const uint8_t* req_table;
} ls100_gemm_i8_args;

int ls100_gemm_i8(ls100_ctx* ctx, const ls100_gemm_i8_args* args, ls100_stream_t stream);
/* Fills `table` for the given n, s_outq, bias, act, out_kind and s_req (the other members are not read). */
size_t ls100_gemm_i8_table_bytes(int64_t n);
int ls100_gemm_i8_build_table(ls100_ctx* ctx, const ls100_gemm_i8_args* args, uint8_t* table, ls100_stream_t stream);


/* ----------------------------------------------------------------- embedding ---
 * x[r, :] = sqrt_h * (table_q[id] * s_emb) + pos[p] * (id != pad_id), p = (#non-pad ids
 * up to and including this one) - 1 + pos_offset. Replaces launch_enc_emb_i8I /
 * launch_dec_emb_i8I (lightseq/inference/kernels/embKernels_int8.cc.cu:99-212); restates
 * TransformerEmbeddingLayer.forward (torch_transformer_layers.py:1027-1036).
 * Encoder form: ids [batch, seq] (ld_ids = seq), step_ptr NULL.
 * Decoder form: seq = 1, the id of row r is ids[r*ld_ids + *step_ptr] and pos_offset = *step_ptr
 * (step read on the device so a captured CUDA graph can be replayed every step). */
typedef struct {
  const int32_t* ids;
  int64_t ld_ids;
  int32_t batch, seq, hidden;
  const int32_t* step_ptr; /* optional device int */
  const int8_t* table_q;   /* [vocab, hidden] int8 */
  float s_emb;             /* amax_emb / 127 */
  float sqrt_h;            /* embed_scale */
  const float* pos;        /* [n_pos, hidden] fp32 */
  int32_t n_pos, pad_id, vocab;
  float* out;        /* [batch*seq, hidden] fp32 */
  uint8_t* pad_mask; /* optional [batch, seq], 1 = pad */
  int32_t pos_mode;  /* 0: positions count non-pad tokens and pads get none (fairseq / Transformer);
                        1: position = column index (+ *step_ptr), added to every token (BERT, GPT-2 learned tables) */
} ls100_embed_args;
int ls100_embed(ls100_ctx* ctx, const ls100_embed_args* args, ls100_stream_t stream);

/* ------------------------------------------------------- LayerNorm + quantise ---
 * y = LayerNorm(x) over the last dim (eps 1e-5, float64 statistics), optionally
 * written as fp32 and/or quantised to int8 with the consumer's input clip-max.
 * Replaces ker_norm_layer_resual_i8O (lightseq/inference/kernels/transformerKernels_int8.cc.cu:149-316);
 * restates the LayerNorm -> QuantLinear.input_quant edge of
 * lightseq/training/ops/pytorch/torch_transformer_layers.py:642-661.
 * hidden % 4 == 0, hidden <= 4096. */
typedef struct {
  const float* x;
  int64_t ldx; /* elements */
  const float* gamma;
  const float* beta;
  int32_t rows, hidden;
  float amax;   /* clip-max of the int8 output (used when out_q != NULL) */
  int8_t* out_q; /* optional [rows, hidden] */
  int64_t ldq;
  float* out_f; /* optional fp32 LayerNorm output */
  int64_t ldf;
  /* optional (emb.table_q != NULL): the rows are not read from x but looked up, the decode-step form of
   * ls100_embed (emb.seq == 1, emb.step_ptr != NULL, emb.batch == rows, emb.hidden == hidden); emb.out receives
   * the looked-up rows (the residual stream) as ls100_embed would write them. One launch instead of two at the
   * head of every decode step; rows <= 2048. */
  ls100_embed_args emb;
} ls100_ln_quant_args;
int ls100_ln_quant(ls100_ctx* ctx, const ls100_ln_quant_args* args, ls100_stream_t stream);


/* ---------------------------------------------------------- ViT patch embedding ---
 * out[b, 0, :]     = cls + pos[0]
 * out[b, 1 + n, :] = conv(patch n of image b) + conv_bias + pos[1 + n]
 * with a convolution of kernel = stride = patch (patches in row-major order over the image, the weight index is
 * (hidden, channel, row, col)); nothing is quantised here. The dot products are accumulated in float64 and rounded
 * once to fp32, so the result does not depend on the summation order; bias and position are fp32 additions in that
 * order. Replaces launch_patch_emb (lightseq/inference/kernels/embKernels.cc.cu:547-618; one CTA per output value
 * there). conv_wt is the TRANSPOSED weight [channels*patch*patch, hidden]. hidden % 4 == 0. */
typedef struct {
  const float* pixels;   /* [batch, channels, image, image] fp32 */
  const float* conv_wt;  /* [channels*patch*patch, hidden] fp32 */
  const float* conv_bias; /* [hidden] */
  const float* pos;      /* [1 + (image/patch)^2, hidden] */
  const float* cls;      /* [hidden] */
  int32_t batch, channels, image, patch, hidden;
  float* out; /* [batch, 1 + (image/patch)^2, hidden] fp32 */
} ls100_patch_embed_args;
int ls100_patch_embed(ls100_ctx* ctx, const ls100_patch_embed_args* args, ls100_stream_t stream);

/* ------------------------------------------------- encoder-style self attention ---
 * softmax((q*dh^-0.5) k^T + mask) v per (batch, head) over a full sequence, output
 * quantised with the out-projection's input clip-max. q,k,v are read from the QKV
 * GEMM's int8 output [batch*seq, 3*hidden] as x*s_qkv (+ bias[c]). Key-padding mask
 * excludes keys; `causal` also excludes keys after the query (GPT prefill).
 * Replaces ker_arrange_encself_qkv_i8I + cublasGemmStridedBatchedEx x2 +
 * ker_correlation_softmax_encself + ker_arrange_atten_output_i8O
 * (lightseq/inference/model/quant_encoder.cc.cu:306-342); restates
 * MultiheadAttention.forward (torch_transformer_layers.py:201-376). head_dim == 64. */
typedef struct {
  const int8_t* qkv;
  int64_t ld_qkv;
  float s_qkv;
  const float* bias; /* optional [3*hidden] */
  const uint8_t* pad_mask; /* optional [batch, seq] */
  int32_t batch, seq, heads, causal;
  float amax_out;
  int8_t* out; /* [batch*seq, hidden] */
  int64_t ld_out;
  /* optional: also store k,v of every position into an int8 cache laid out
   * [batch, heads, max_step, 64] (GPT prefill); requires bias == NULL */
  int8_t* k_cache;
  int8_t* v_cache;
  int32_t max_step;
} ls100_attn_self_args;
int ls100_attn_self(ls100_ctx* ctx, const ls100_attn_self_args* args, ls100_stream_t stream);

/* --------------------------------------- decoder self attention over int8 KV cache ---
 * One new token per row. qkv [rows, 3*hidden] int8 holds attention_quant(q,k,v) (scale
 * s_kv). The new k,v are appended at position *step_ptr of the row's own cache slot;
 * history position p of row r lives in slot anc[r*max_step + p] (beam ancestry, written
 * by ls100_beam_update; pass NULL for "own slot"). Caches: [rows, heads, max_step, 64].
 * Replaces ker_arrange_decself_qkv_i8I_i8O + int8 cublasGemmStridedBatchedEx +
 * ker_fuse_softmax_new_value_i32I_i8O and the per-step ker_refresh_cache
 * (lightseq/inference/model/quant_decoder.cc.cu:662-700,1060-1074); restates the
 * incremental branch of MultiheadAttention.forward (torch_transformer_layers.py:262-300). */
typedef struct {
  const int8_t* qkv;
  int64_t ld_qkv;
  float s_kv;
  int8_t* k_cache;
  int8_t* v_cache;
  const int32_t* anc; /* optional [rows, max_step] */
  const int32_t* step_ptr;
  int32_t rows, heads, max_step;
  float amax_out;
  int8_t* out;
  int64_t ld_out;
  /* Nonzero: *step_ptr, anc and the cache positions below *step_ptr were complete before a full stream dependency
   * that precedes this launch (the decode step runs as one graph launch and they were written by earlier ones), so
   * the kernel may read them before its grid dependency on the preceding kernel resolves; only qkv then waits for
   * that kernel. Zero is always safe. */
  int32_t history_static;
} ls100_attn_dec_args;
int ls100_attn_dec(ls100_ctx* ctx, const ls100_attn_dec_args* args, ls100_stream_t stream);

/* ------------------------------------------------------------- cross attention ---
 * rows = batch*beam queries (q int8 * s_q + bias) against the fp32 encoder keys/values
 * [batch*src_len, hidden] of one decoder layer, source key-padding mask, output int8.
 * Replaces ker_arrange_encdec_q_i8I + cublasGemmStridedBatchedEx x2 +
 * ker_correlation_softmax_encdec + ker_arrange_atten_output_i8O
 * (lightseq/inference/model/quant_decoder.cc.cu:767-814). */
typedef struct {
  const int8_t* q;
  int64_t ld_q;
  float s_q;
  const float* bias; /* [hidden] */
  const void* k;     /* fp32 [batch*src_len, hidden], or head-major: see kv_head_major */
  const void* v;
  int64_t ld_kv; /* elements */
  const uint8_t* pad_mask; /* [batch, src_len] */
  int32_t batch, beam, src_len, heads;
  float amax_out;
  int8_t* out;
  int64_t ld_out;
  /* Nonzero: k, v and pad_mask were complete before a full stream dependency that precedes this launch (a graph
   * launch, a copy, a kernel launched without programmatic serialisation), so the kernel may fetch them before
   * its own grid dependency on the preceding kernel resolves. Zero is always safe. */
  int32_t kv_static;
  /* Nonzero: k and v are fp32 [batch, heads, src_len, 64] (ls100_proj_f32 with split_seq = src_len; ld_kv
   * unused): a head's keys are one contiguous run of src_len * 256 bytes. Zero: [batch * src_len, ld_kv]. */
  int32_t kv_head_major;
} ls100_attn_cross_args;
int ls100_attn_cross(ls100_ctx* ctx, const ls100_attn_cross_args* args, ls100_stream_t stream);

/* -------------------------------------------- fp32 x fake-quant weight projection ---
 * out_f32[M,N] = (x[M,K] . Wq[N,K]^T) * s_w + bias : the weight-only-quantised k_proj /
 * v_proj of the decoder's cross attention, run once per request. Replaces the fp16
 * cublasGemmEx + ker_arrange_encdec_kv of QuantDecoder::project_encoder_output
 * (lightseq/inference/model/quant_decoder.cc.cu:489-520); restates QuantLinear with
 * pre_activation="encoder_out" (quantization.py:41-46). */
typedef struct {
  const float* x;
  int64_t ldx;
  const int8_t* w;
  int64_t ldw;
  float s_w;
  const float* bias;
  int32_t m, n, k;
  void* out; /* fp32 */
  int64_t ldo;
  /* > 0: head-split output, as ker_arrange_encdec_kv does: row m = b * split_seq + s and column n = h * 64 + d
   * are stored at out[((b * (N / 64) + h) * split_seq + s) * 64 + d], i.e. fp32 [batch, heads, split_seq, 64]
   * (N a multiple of 64; ldo unused). 0: row-major [M, ldo]. */
  int32_t split_seq;
} ls100_proj_f32_args;
int ls100_proj_f32(ls100_ctx* ctx, const ls100_proj_f32_args* args, ls100_stream_t stream);

/* The same projection on the tensor cores. The fp32 activations are split once into three bf16 terms
 * (x = hi + mid + lo, remainder below 2^-27 |x|): ls100_split_bf16x3 writes x3 = [lo | mid | hi] as bf16 [M, 3K]
 * (smallest terms first, which keeps the tensor core's running fp32 sum small for two thirds of the products);
 * the int8 weight is exact in bf16 (ls100_i8_to_bf16, once at load). ls100_proj_tc then runs ONE tcgen05 kind::f16
 * GEMM with K' = 3K against [W | W | W] (never materialised) with fp32 accumulation, scales by s_w, adds the bias
 * and stores fp32 row-major or head-split like ls100_proj_f32. K must be a multiple of 64. Differs from
 * ls100_proj_f32 only in the rounding of the fp32 accumulation (both within 1e-6 relative of the exact product). */
int ls100_split_bf16x3(ls100_ctx* ctx, const float* x, int64_t ldx, int32_t m, int32_t k, void* out_bf16 /* [m, 3k] */,
                       ls100_stream_t stream);
int ls100_i8_to_bf16(ls100_ctx* ctx, const int8_t* w, int64_t ldw, int32_t n, int32_t k, void* out_bf16 /* [n, k] */,
                     ls100_stream_t stream);
typedef struct {
  const void* x3;     /* bf16 [m, 3k] from ls100_split_bf16x3 */
  const void* w_bf16; /* bf16 [n, k] from ls100_i8_to_bf16 */
  float s_w;
  const float* bias;
  int32_t m, n, k;
  void* out; /* fp32 */
  int64_t ldo;
  int32_t split_seq; /* as in ls100_proj_f32_args */
} ls100_proj_tc_args;
int ls100_proj_tc(ls100_ctx* ctx, const ls100_proj_tc_args* args, ls100_stream_t stream);

/* ------------------------------------------------------------------ beam search ---
 * Step 1 (ls100_beam_topk): per (batch, beam) row of int8 logits, log-softmax base from
 * the 255-bin histogram (exp arguments clamped at -64), exact top-`beam` by (logit desc,
 * token asc), candidate score = max((logit + prefix - logsumexp) * length_norm, -1999);
 * a finished row (last token == end_id, step > 0) emits only (seq_score, EOS).
 * Step 2 (ls100_beam_update): per batch, best `beam` of the beam*beam candidates by
 * (score desc, beam asc, token asc); rebuilds alive_seq and the KV ancestry table in
 * place, updates seq_probs / seq_score, counts finished beams, advances *step_ptr and
 * records the first step at which every beam is finished in *stop_step (init -1).
 * Replaces select_beam_rough_topk_i8I (transformerKernels_int8.cc.cu:1690-1906), the
 * thrust scan/sort + two host syncs of QuantDecoder::beam_search
 * (quant_decoder.cc.cu:987-1076), ker_refresh_result (transformerKernels.cc.cu:1398-1463)
 * and ker_refresh_cache (:1578-1681). beam <= 8. */
typedef struct {
  const int8_t* logits; /* [batch*beam, ld_logits] */
  int64_t ld_logits;
  float s_logits;
  int32_t batch, beam, vocab, max_step, end_id;
  const int32_t* step_ptr;
  const float* length_norm; /* [max_step] device table, entry s = norm of length s+1 */
  const int32_t* alive;     /* [batch, beam, max_step] */
  const float* seq_probs;   /* [batch, beam] */
  const float* seq_score;   /* [batch, beam] */
  float* cand_score;        /* out [batch*beam, beam] */
  int32_t* cand_token;      /* out [batch*beam, beam] */
  float diverse_lambda;     /* diverse beam search: the r-th best candidate of a row competes with score - lambda * (r + 1)
                               (ker_diverse_beam_search, lightseq/inference/kernels/transformerKernels.cc.cu:312-333); 0 = off */
} ls100_beam_topk_args;
int ls100_beam_topk(ls100_ctx* ctx, const ls100_beam_topk_args* args, ls100_stream_t stream);

/* Step 1 from the statistics ls100_gemm_i8 kept while it wrote the logits (stat_max / stat_sum of its arguments,
 * n_groups = ceil(vocab / 64)): the same candidates as ls100_beam_topk without reading the [rows, vocab] matrix
 * again - the log-sum-exp comes from the group sums, and only the few 64-column groups whose largest value reaches
 * the row's K-th largest group maximum are read. Scores agree with ls100_beam_topk to float rounding (the
 * exponentials are summed in a different order), tokens exactly. */
typedef struct {
  ls100_beam_topk_args topk;
  const int8_t* stat_max; /* [ceil(rows/128)][n_groups][128] */
  const float* stat_sum;  /* same layout */
  int32_t n_groups;
} ls100_beam_select_args;
int ls100_beam_select(ls100_ctx* ctx, const ls100_beam_select_args* args, ls100_stream_t stream);

typedef struct {
  const float* cand_score;
  const int32_t* cand_token;
  int32_t batch, beam, max_step, end_id;
  int32_t* step_ptr;   /* advanced by one */
  const float* length_norm;
  int32_t* alive;      /* in place */
  int32_t* anc;        /* in place, optional */
  float* seq_probs;
  float* seq_score;
  int32_t* fin_count;  /* [max_step] zeroed by the caller before the first step */
  int32_t* ticket;     /* [max_step] zeroed by the caller before the first step */
  int32_t* stop_step;  /* device int, -1 until every beam is finished */
  int32_t* stop_host;  /* optional mapped host int mirroring *stop_step */
  float diverse_lambda; /* the penalty ls100_beam_topk subtracted is added back before scores and prefixes are stored
                           (ker_refresh_result, lightseq/inference/kernels/transformerKernels.cc.cu:1430-1458) */
} ls100_beam_update_args;
int ls100_beam_update(ls100_ctx* ctx, const ls100_beam_update_args* args, ls100_stream_t stream);

/* Result of a finished generation from the beam state: `mode` 0 = beam 0 of every sentence
 * (ker_write_trg_tokenid_pos_penalty, lightseq/inference/kernels/transformerKernels.cc.cu:1722-1733), 1 = the beam
 * with the best score per non-EOS token, for a negative length penalty after an early stop
 * (ker_write_trg_tokenid_neg_penalty, :1752-1784), 2 = every beam with the last position forced to EOS
 * (ker_write_topk_result, :1803-1813). Tokens are positions 1 .. n_out of the histories. */
typedef struct {
  const int32_t* alive;    /* [batch, beam, max_step] */
  const float* seq_score;  /* [batch, beam] */
  int32_t batch, beam, max_step, end_id;
  int32_t n_out;           /* tokens per output row */
  int32_t mode;
  int32_t* out_tokens;     /* [batch, n_out] (modes 0, 1) or [batch * beam, n_out] (mode 2) */
  float* out_scores;       /* [batch] or [batch * beam] */
} ls100_beam_result_args;
int ls100_beam_write_result(ls100_ctx* ctx, const ls100_beam_result_args* args, ls100_stream_t stream);

/* Allocation-free form of ls100_beam_update. It has no counterpart in the reference.
 * For callers that cannot provide the two scratch arrays because they cannot allocate device memory at all:
 * a serving process that handed every byte of the GPU to its own arena at start-up, or a latency-critical
 * thread that must never reach cudaMalloc/cudaFree (both synchronise the device). The `fin_count` and `ticket`
 * fields of `args` are ignored; the counters live in an 8 KB array inside the library image (held by every GPU
 * that loads the library until the process exits), which bounds max_step to
 * LS100_BEAM_UPDATE_NOALLOC_MAX_STEP - larger values return LS100_ERR_UNSUPPORTED and launch nothing.
 * Everything else (inputs, outputs, results) is exactly ls100_beam_update's.
 *  - The FIRST call on each device looks up the array's device address (the context's device must be
 *    current). Make that first call outside any stream capture.
 *  - Every call clears the array on `stream` before launching, so it does not matter what the previous call
 *    left behind; but all calls share the one array: two calls that can overlap on the GPU (different streams,
 *    or different contexts on the same device) race on it. Serialise them on one stream.
 *  - No cudaMalloc, cudaFree or allocating library routine is called. */
#define LS100_BEAM_UPDATE_NOALLOC_MAX_STEP 1024
int ls100_beam_update_noalloc(ls100_ctx* ctx, const ls100_beam_update_args* args, ls100_stream_t stream);

/* ------------------------------------------------------------- top-k sampling ---
 * One new token per row from the int8 logits of its newest position: exact top-k by (logit desc, token asc),
 * softmax over those k (p_i = exp(l_i - l_0) / sum), cumulative in that order, pick the first i with
 * u <= cum_i where u in (0,1] comes from Philox4x32-10 with key (seed_lo, seed_hi) and counter
 * (position, row, 0, 0): u = ((x0 >> 8) + 1) * 2^-24. A row whose newest token is `end_id` appends `end_id`.
 * The token is written to seq[row, *cur + 1]; the last CTA advances *cur and, when every row has ended,
 * records the position in *stop (init -1). Replaces ker_topk_sample_i8I + the per-token host sync of
 * QuantGptEncoder::sample_one_token_with_cache (lightseq/inference/kernels/gptKernels_int8.cc.cu:252-430,
 * lightseq/inference/model/quant_gpt_encoder.cc.cu:441-481); the rough threshold, CUB scan and clock()-seeded
 * cuRAND state of the reference become an exact selection and a counter-based generator, so a run is
 * reproducible. k <= 8. */
typedef struct {
  const int8_t* logits; /* [rows, ld_logits] */
  int64_t ld_logits;
  float s_logits;
  int32_t rows, vocab, k, max_step, end_id;
  uint32_t seed_lo, seed_hi;
  int32_t* seq;     /* [rows, max_step], in place */
  int32_t* cur;     /* device int: index of the newest token of every row; advanced by one */
  int32_t* ticket;  /* device int, zero before the call sequence starts; reset by the kernel */
  int32_t* n_ended; /* device int, zero before the call sequence starts; reset by the kernel */
  int32_t* stop;    /* device int, -1 until every row has produced end_id */
  int32_t* stop_host; /* optional mapped host mirror of *stop */
} ls100_sample_topk_args;
int ls100_sample_topk(ls100_ctx* ctx, const ls100_sample_topk_args* args, ls100_stream_t stream);

/* ------------------------------------------------------------- top-p (nucleus) sampling ---
 * One new token per row. Int8 logits take at most 255 distinct values, so the nucleus is found exactly from a
 * histogram of the row: with tokens ordered by (logit desc, token asc), w_q = exp((q - q_max) * s_logits) and
 * n_q tokens at level q, the cumulative mass after j tokens of level q is C_q + float(j) * w_q, where C_q is the
 * float32 sum, taken level by level from q_max down, of float(n_q') * w_q' over the levels above. The nucleus is
 * the shortest prefix whose mass reaches p * total; its mass is M. With u as in ls100_sample_topk the token is
 * the first of that order whose cumulative mass reaches u * M. Bookkeeping (seq, *cur, *stop) as in
 * ls100_sample_topk. Replaces ker_topp_sample_i8I (lightseq/inference/kernels/transformerKernels_int8.cc.cu:
 * 2131-2294, gptKernels_int8.cc.cu:432-656), whose nucleus is approximate: it keeps one candidate per thread
 * (the maximum of a stride of the row), sorts those 1024 values with CUB and cuts by their cumulative sum. */
typedef struct {
  const int8_t* logits; /* [rows, ld_logits] */
  int64_t ld_logits;
  float s_logits;
  float p;          /* in (0, 1] */
  int32_t rows, vocab, max_step, end_id;
  uint32_t seed_lo, seed_hi;
  int32_t* seq;     /* [rows, max_step], in place */
  int32_t* cur;     /* device int: index of the newest token of every row; advanced by one */
  int32_t* ticket;  /* device int, zero before the call sequence starts; reset by the kernel */
  int32_t* n_ended; /* device int, zero before the call sequence starts; reset by the kernel */
  int32_t* stop;    /* device int, -1 until every row has produced end_id */
  int32_t* stop_host; /* optional mapped host mirror of *stop */
} ls100_sample_topp_args;
int ls100_sample_topp(ls100_ctx* ctx, const ls100_sample_topp_args* args, ls100_stream_t stream);

/* ------------------------------------------------------------- perplexity ---
 * ls100_token_nll: for each of `rows` consecutive (sequence, position) rows starting at flat row `row0` of a
 * [batch, seq] batch, nll = logsumexp_v(q_v * s_logits) - q_target * s_logits where the target is the NEXT token
 * of the sequence, ids[b, t + 1] (0 for the last position of a sequence, which has no target). `logits` points
 * at the int8 logits of flat row `row0`. ls100_seq_ppl then gives, per sequence, the mean of nll[b, t] over
 * t < len_b - 1, where len_b counts the tokens different from `pad_id` (pad_id < 0: every token counts); a
 * sequence of fewer than two tokens yields 0. Together they replace ker_ppl_i8I
 * (lightseq/inference/kernels/gptKernels_int8.cc.cu:108-190), whose per-token atomicAdd makes the sum depend
 * on the order in which the blocks finish; here each sequence is summed by one warp in a fixed order. */
typedef struct {
  const int8_t* logits; /* [rows, ld_logits], row 0 = flat row `row0` */
  int64_t ld_logits;
  float s_logits;
  int32_t rows, row0, vocab;
  const int32_t* ids; /* [batch, seq] */
  int32_t batch, seq;
  float* nll;         /* [batch * seq]; rows row0 .. row0 + rows - 1 are written */
} ls100_token_nll_args;
int ls100_token_nll(ls100_ctx* ctx, const ls100_token_nll_args* args, ls100_stream_t stream);
typedef struct {
  const float* nll;   /* [batch * seq] */
  const int32_t* ids; /* [batch, seq] */
  int32_t batch, seq, pad_id;
  float* ppl;         /* [batch] */
} ls100_seq_ppl_args;
int ls100_seq_ppl(ls100_ctx* ctx, const ls100_seq_ppl_args* args, ls100_stream_t stream);

/* ------------------------------------------------------------- load-time prep ---
 * fp32 -> int8 with the tensor's clip-max (quantize_weight, lightseq/inference/model/
 * cublas_helper.cc:553-593) and, optionally, off[n] = 127 * sum_k q[n,k]: the exact
 * integer form of the ReLU "colsum" correction (launch_scaled_colsum,
 * lightseq/inference/kernels/transformerKernels.cc.cu:18-80). */
int ls100_quantize_weight(ls100_ctx* ctx, const float* w, int64_t rows, int64_t cols, float amax, int8_t* out_q,
                          int32_t* row_off /* optional [rows] */, ls100_stream_t stream);

/* ------------------------------------------------------------- measurement and diagnostics ---
 * No counterparts in the reference (its tensor ceilings come from cuBLASLt's autotuner tables,
 * tests/gemm_test/configs/igemm_*.cfg). These run no model work; they allocate their own small buffers and
 * synchronise the stream.
 *
 * ls100_measure_i8_mma_peak: one CTA per SM issues `iters` x 4 tcgen05.mma kind::i8 instructions (128 x 256 x 32
 * each) back to back from operands resident in shared memory into two TMEM accumulators; *tops_out = integer
 * operations per second / 1e12 over the whole device, timed with CUDA events on `stream`. The measured ceiling of
 * the tensor pipe for int8, the denominator of the GEMM rooflines.
 *
 * ls100_measure_phase_floor: time per dependent phase (every thread reads a float another CTA wrote in the
 * previous phase) for `phases` phases of `grid` CTAs x 256 threads: us_per_phase[0] kernel after kernel,
 * [1] kernel after kernel with programmatic dependent launch, [2] phases of one persistent cooperative kernel
 * separated by a global-memory grid barrier (bounded wait).
 *
 * ls100_debug_expire_wait: launches one CTA that waits about 0.1 ms on an mbarrier nobody arrives at, gives up,
 * records LS100_ERR_TIMEOUT in the context's error word and returns normally (nothing traps, the context stays
 * usable); ls100_ctx_poll_error then reports the code once. */
int ls100_measure_i8_mma_peak(ls100_ctx* ctx, int iters, ls100_stream_t stream, double* tops_out, float* ms_out /* optional */);
int ls100_measure_phase_floor(ls100_ctx* ctx, int phases, int grid, ls100_stream_t stream, float* us_per_phase /* [3] */);
int ls100_debug_expire_wait(ls100_ctx* ctx, ls100_stream_t stream);

/* ------------------------------------------------------------- model level ---
 * The LSModel interface of lightseq/inference/pywrapper/model_base.h:59-148 as plain C:
 * create by name ("QuantTransformer", "QuantBert", "QuantGpt", "QuantVit") from a weight file and
 * max batch size, hand over caller-owned DEVICE pointers, run, read shapes back.
 * Every function returns 0 or a negative code; ls100_model_last_error() gives the
 * message of the last failure on the calling thread (what the C++ API throws as
 * std::runtime_error). A model uses the device that is current at creation. */
typedef struct ls100_model ls100_model;
int ls100_model_create(const char* model_name, const char* weight_path, int max_batch_size, ls100_model** out);
void ls100_model_destroy(ls100_model* m);
const char* ls100_model_last_error(void);
int ls100_model_set_input_ptr(ls100_model* m, int index, void* device_ptr);
int ls100_model_set_input_shape(ls100_model* m, int index, const int32_t* dims, int ndim);
int ls100_model_set_output_ptr(ls100_model* m, int index, void* device_ptr);
int ls100_model_infer(ls100_model* m);
int ls100_model_get_output_shape(ls100_model* m, int index, int32_t* dims /* >= 4 */, int* ndim);
int ls100_model_get_output_max_shape(ls100_model* m, int index, int32_t* dims /* >= 4 */, int* ndim);
int ls100_model_benchmark_mode(ls100_model* m, int on);
/* The cudaStream_t every kernel of this model is launched on (for event timing by the caller). */
int ls100_model_get_stream(ls100_model* m, ls100_stream_t* stream);

/* Host-buffer convenience = what PyQuantTransformer::infer does
 * (lightseq/inference/pywrapper/wrapper.cc:121-155): H2D copy of ids [batch, seq_len],
 * Infer(), D2H copy of tokens [batch, 1, *out_len] (written densely into out_tokens, which
 * must hold batch*max_step ints) and scores [batch]. Device staging buffers are owned by
 * the model and allocated at creation. */
int ls100_transformer_infer_host(ls100_model* m, const int32_t* ids, int batch, int seq_len, int32_t* out_tokens,
                                 float* out_scores, int* out_len);
/* The same for models that return several sequences per sentence (every beam: `output_topk`, or a sampling method;
 * QuantTransformer::Infer sets the output shapes to {batch, output_k, len}, lightseq/inference/pywrapper/
 * quant_transformer.cc:100-109): tokens [batch, *out_k, *out_len] into out_tokens (batch * beam * max_step ints),
 * scores [batch, *out_k] into out_scores (batch * beam floats). */
int ls100_transformer_infer_host_k(ls100_model* m, const int32_t* ids, int batch, int seq_len, int32_t* out_tokens,
                                   float* out_scores, int* out_k, int* out_len);
/* QuantBert: ids [batch, seq_len] -> fp32 encoder output [batch, seq_len, hidden] (PyQuantBert::infer,
 * lightseq/inference/pywrapper/wrapper.cc:276-321). */
int ls100_bert_infer_host(ls100_model* m, const int32_t* ids, int batch, int seq_len, float* out);
/* QuantVit: pixels [batch, channels, image, image] fp32 -> fp32 encoder output [batch, 1 + patches, hidden]
 * (PyQuantVit::infer, lightseq/inference/pywrapper/wrapper.cc). Host buffers. */
int ls100_vit_infer_host(ls100_model* m, const float* pixels, int batch, int channels, int image, float* out);
/* QuantGpt: prompt ids [batch, prompt_len] -> prompt + sampled tokens [batch, *out_len], written densely into
 * out_tokens (batch*max_step ints) (PyQuantGpt::sample, lightseq/inference/pywrapper/wrapper.cc:463-495). */
int ls100_gpt_sample_host(ls100_model* m, const int32_t* ids, int batch, int prompt_len, int32_t* out_tokens, int* out_len);
/* QuantGpt.ppl(int32[B,S]) -> float32[B] (PyQuantGpt::ppl, lightseq/inference/pywrapper/wrapper.cc:497-531): mean
 * negative log-likelihood of every sequence's own next tokens. Host buffers; copies inside the call. */
int ls100_gpt_ppl_host(ls100_model* m, const int32_t* ids, int batch, int seq_len, float* out_ppl);

#ifdef __cplusplus
}
#endif
#endif /* LS100_H_ */
