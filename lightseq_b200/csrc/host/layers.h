// Layers of the int8 Transformer, with the constructor / operator() / before_forward /
// forward shape of the reference's new-arch layers
// (lightseq/csrc/layers_new/includes/transformer_encoder_layer.h:17-36,
//  transformer_decoder_layer.h:33-61, generator_layer.cpp:5-110); the dataflow and the
// clip-max placement follow the PyTorch fake-quant layers
// (lightseq/training/ops/pytorch/torch_transformer_layers.py:630-679, 844-965).
#pragma once
#include "ops.h"

namespace ls100 {

struct LayerNormParams {
  float* g = nullptr;
  float* b = nullptr;
  void load(Context& ctx, const WeightsFile& wf, const std::string& name, int hidden) {
    g = upload_vec(ctx, wf, name + ".g", hidden);
    b = upload_vec(ctx, wf, name + ".b", hidden);
  }
};

// Buffers shared by every layer of a stack (sized for the maxima at construction).
struct StackBuffers {
  Variable* x = nullptr;       // fp32 residual stream [rows, H]
  Variable* a_q = nullptr;     // int8 LayerNorm output [rows, H]
  Variable* qkv_q = nullptr;   // int8 [rows, 3H]
  Variable* attn_q = nullptr;  // int8 [rows, H]
  Variable* h_q = nullptr;     // int8 [rows, F]
  Variable* q_q = nullptr;     // int8 [rows, H] (cross-attention query)
};

// ---------------------------------------------------------------------------------------
// Encoder layer (pre- or post-LN, ReLU or GELU). Also serves BERT (post-LN, GELU).
class QuantTransformerEncoderLayer : public Layer {
 public:
  QuantTransformerEncoderLayer(ContextPtr ctx, const WeightsFile& wf, const std::string& prefix, int layer_id,
                               int max_batch_tokens, int max_seq_len, int hidden, int heads, int ffn, bool is_pre_ln,
                               const std::string& activation_fn, bool mask_future = false)
      : Layer(prefix, ctx), hidden_(hidden), heads_(heads), ffn_(ffn), pre_ln_(is_pre_ln), causal_(mask_future),
        act_(activation_fn == "gelu" ? Act::Gelu : Act::Relu), max_tokens_(max_batch_tokens) {
    (void)layer_id;
    (void)max_seq_len;
    const bool relu = act_ == Act::Relu;
    qkv_.load(*ctx, wf, prefix + ".qkv", false);
    out_.load(*ctx, wf, prefix + ".out", false);
    fc1_.load(*ctx, wf, prefix + ".fc1", false);
    fc2_.load(*ctx, wf, prefix + ".fc2", relu, true, true, "", "", true, true);  // the encoder-only file formats hold no fc2.out
    ln1_.load(*ctx, wf, prefix + ".ln1", hidden);
    ln2_.load(*ctx, wf, prefix + ".ln2", hidden);
    // what follows fc1's output quantiser is a function of (column, value): tabulated once for the many-tile GEMM
    fc1_.build_table(*ctx, relu ? LS100_OUT_REQ_U8 : LS100_OUT_REQ_S8, (int)act_, true, fc2_.s_in);
  }
  // (inp, pad_mask) -> out, in place on the residual stream
  Variable* operator()(StackBuffers* bufs, Variable* pad_mask) {
    b_ = bufs;
    pad_mask_ = pad_mask;
    return bufs->x;
  }
  void before_forward(int batch, int seq) {
    batch_ = batch;
    seq_ = seq;
    if ((long long)batch * seq > max_tokens_) throw std::runtime_error("batch tokens exceed max_batch_tokens");
  }
  const QLinearParams& qkv() const { return qkv_; }
  const QLinearParams& fc1() const { return fc1_; }
  const LayerNormParams& ln1() const { return ln1_; }

  // Post-LN layers hand their output to the next layer already quantised with that layer's QKV input
  // clip-max (0 = last layer: no int8 copy is written).
  void set_next_input_amax(float amax) { next_amax_ = amax; }

  void forward() override {
    const int rows = batch_ * seq_;
    if (!pre_ln_) {
      // x is the post-LN output of the previous block and a_q = quant(x) with this layer's QKV clip-max
      gemm(b_->a_q, qkv_, rows, LS100_OUT_OUTQ_I8, b_->qkv_q, true, false, Act::None, nullptr, 0.f);
      attention(rows);
      gemm(b_->attn_q, out_, rows, LS100_OUT_F32, b_->x, true, true, Act::None, b_->x, 0.f);
      ln_quant(rows, ln1_, fc1_.amax_in, true, true);
      gemm(b_->a_q, fc1_, rows, act_ == Act::Relu ? LS100_OUT_REQ_U8 : LS100_OUT_REQ_S8, b_->h_q, true, true, act_,
           nullptr, fc2_.s_in);
      gemm(b_->h_q, fc2_, rows, LS100_OUT_F32, b_->x, true, true, Act::None, b_->x, 0.f);
      ln_quant(rows, ln2_, next_amax_, true, next_amax_ > 0.f);
      return;
    }
    ls100_ctx* k = ctx_->kernels();
    cudaStream_t s = ctx_->get_stream();
    ln_quant(rows, ln1_, qkv_.amax_in);
    gemm(b_->a_q, qkv_, rows, LS100_OUT_OUTQ_I8, b_->qkv_q, true, false, Act::None, nullptr, 0.f);
    attention(rows);
    gemm(b_->attn_q, out_, rows, LS100_OUT_F32, b_->x, true, true, Act::None, b_->x, 0.f);
    ln_quant(rows, ln2_, fc1_.amax_in);
    gemm(b_->a_q, fc1_, rows, act_ == Act::Relu ? LS100_OUT_REQ_U8 : LS100_OUT_REQ_S8, b_->h_q, true, true, act_,
         nullptr, fc2_.s_in);
    gemm(b_->h_q, fc2_, rows, LS100_OUT_F32, b_->x, true, true, Act::None, b_->x, 0.f);
    (void)k;
    (void)s;
  }

 protected:
  void ln_quant(int rows, const LayerNormParams& ln, float amax, bool write_f = false, bool write_q = true) {
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = b_->x->value<float>();
    a.ldx = hidden_;
    a.gamma = ln.g;
    a.beta = ln.b;
    a.rows = rows;
    a.hidden = hidden_;
    a.amax = amax;
    a.out_q = write_q ? b_->a_q->value<int8_t>() : nullptr;
    a.ldq = hidden_;
    a.out_f = write_f ? b_->x->value<float>() : nullptr;  // in place: a row is read completely before it is written
    a.ldf = hidden_;
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, ctx_->get_stream()));
  }
  void gemm(Variable* in, const QLinearParams& p, int rows, int out_kind, Variable* out, bool out_quant, bool add_bias,
            Act act, Variable* resid, float s_req) {
    QuantLinearOp op(ctx_, name_ + ".gemm", &p, out_kind, act, out_quant, add_bias, s_req);
    op(in, out, resid);
    op.before_forward(rows);
    op.forward();
  }
  void attention(int rows) {
    (void)rows;
    ls100_attn_self_args a;
    memset(&a, 0, sizeof(a));
    a.qkv = b_->qkv_q->value<int8_t>();
    a.ld_qkv = 3 * hidden_;
    a.s_qkv = qkv_.s_out;
    a.bias = qkv_.bias;
    a.pad_mask = pad_mask_ ? pad_mask_->value<uint8_t>() : nullptr;
    a.batch = batch_;
    a.seq = seq_;
    a.heads = heads_;
    a.causal = causal_ ? 1 : 0;
    a.amax_out = out_.amax_in;
    a.out = b_->attn_q->value<int8_t>();
    a.ld_out = hidden_;
    LS_RC(ls100_attn_self(ctx_->kernels(), &a, ctx_->get_stream()));
  }

  int hidden_, heads_, ffn_;
  bool pre_ln_, causal_;
  Act act_;
  int max_tokens_;
  QLinearParams qkv_, out_, fc1_, fc2_;
  LayerNormParams ln1_, ln2_;
  StackBuffers* b_ = nullptr;
  Variable* pad_mask_ = nullptr;
  int batch_ = 0, seq_ = 0;
  float next_amax_ = 0.f;
};

// ---------------------------------------------------------------------------------------
// Decoder layer, one token per row per call (incremental decoding with an int8 self-attention
// cache and fp32 cross-attention keys/values computed once per request).
class QuantTransformerDecoderLayer : public Layer {
 public:
  // the decode-step embedding lookup to run inside this layer's first LayerNorm launch (first layer of a stack only)
  void set_embed_source(const ls100_embed_args* e) { embed_src_ = e; }
  QuantTransformerDecoderLayer(ContextPtr ctx, const WeightsFile& wf, const std::string& prefix, int layer_id,
                               int max_batch_tokens, int max_seq_len, int hidden, int heads, int ffn, bool is_pre_ln,
                               const std::string& activation_fn, int max_batch_size, int beam_size, int max_step)
      : Layer(prefix, ctx), hidden_(hidden), heads_(heads), ffn_(ffn), act_(activation_fn == "gelu" ? Act::Gelu : Act::Relu),
        max_rows_(max_batch_size * beam_size), max_step_(max_step), max_enc_tokens_(max_batch_tokens), pre_ln_(is_pre_ln) {
    (void)layer_id;
    (void)max_seq_len;
    const bool relu = act_ == Act::Relu;
    qkv_.load(*ctx, wf, prefix + ".qkv", false);
    out_.load(*ctx, wf, prefix + ".out", false);
    xq_.load(*ctx, wf, prefix + ".xq", false);
    xk_.load(*ctx, wf, prefix + ".xk", false, false, false);
    xv_.load(*ctx, wf, prefix + ".xv", false, false, false);
    xout_.load(*ctx, wf, prefix + ".xout", false);
    fc1_.load(*ctx, wf, prefix + ".fc1", false);
    fc2_.load(*ctx, wf, prefix + ".fc2", relu);
    ln1_.load(*ctx, wf, prefix + ".ln1", hidden);
    ln2_.load(*ctx, wf, prefix + ".ln2", hidden);
    ln3_.load(*ctx, wf, prefix + ".ln3", hidden);
    amax_kv_ = wf.amax(prefix + ".kv");
    s_kv_ = amax_kv_ / 127.0f;
    const size_t cache = (size_t)max_rows_ * max_step * hidden;
    k_cache_ = ctx->alloc_n<int8_t>(cache);
    v_cache_ = ctx->alloc_n<int8_t>(cache);
    LS_CUDA(cudaMemset(k_cache_, 0, cache));
    LS_CUDA(cudaMemset(v_cache_, 0, cache));
    enc_k_ = ctx->alloc_n<float>((size_t)max_batch_tokens * hidden);
    enc_v_ = ctx->alloc_n<float>((size_t)max_batch_tokens * hidden);
  }
  void operator()(StackBuffers* bufs, Variable* src_pad_mask, const int32_t* anc, const int32_t* step_ptr) {
    b_ = bufs;
    pad_mask_ = src_pad_mask;
    anc_ = anc;
    step_ptr_ = step_ptr;
  }
  void before_forward(int batch, int beam, int src_len) {
    batch_ = batch;
    beam_ = beam;
    src_len_ = src_len;
    if (batch * beam > max_rows_) throw std::runtime_error("decoder rows exceed max_batch_size * beam_size");
    if ((long long)batch * src_len > max_enc_tokens_) throw std::runtime_error("encoder tokens exceed max_batch_tokens");
  }
  // cross-attention keys / values of this layer from the encoder output (once per request)
  // `enc_x3`: the encoder output split into three bf16 terms (ls100_split_bf16x3), or NULL for the fp32 SIMT kernel
  void project_encoder_output(const float* enc_out, const void* enc_x3) {
    for (int which = 0; which < 2; ++which) {
      const QLinearParams& p = which == 0 ? xk_ : xv_;
      if (enc_x3 && w_bf16_[which]) {  // tensor cores
        ls100_proj_tc_args a;
        memset(&a, 0, sizeof(a));
        a.x3 = enc_x3;
        a.w_bf16 = w_bf16_[which];
        a.s_w = p.s_w;
        a.bias = p.bias;
        a.m = batch_ * src_len_;
        a.n = hidden_;
        a.k = hidden_;
        a.out = which == 0 ? enc_k_ : enc_v_;
        a.ldo = hidden_;
        a.split_seq = src_len_;
        LS_RC(ls100_proj_tc(ctx_->kernels(), &a, ctx_->get_stream()));
        continue;
      }
      ls100_proj_f32_args a;
      memset(&a, 0, sizeof(a));
      a.x = enc_out;
      a.ldx = hidden_;
      a.w = p.w;
      a.ldw = p.k;
      a.s_w = p.s_w;
      a.bias = p.bias;
      a.m = batch_ * src_len_;
      a.n = hidden_;
      a.k = hidden_;
      a.out = which == 0 ? enc_k_ : enc_v_;
      a.ldo = hidden_;
      a.split_seq = src_len_;  // [batch, heads, src_len, 64]: a head's keys are contiguous for the decode steps
      LS_RC(ls100_proj_f32(ctx_->kernels(), &a, ctx_->get_stream()));
    }
  }
  // bf16 copies of the two projection weights (exact: int8 values), made once so that the projection can run on the
  // tensor cores; hidden sizes that are not a multiple of 64 keep the SIMT kernel
  void prepare_tensor_core_projection() {
    if (hidden_ % 64) return;
    for (int which = 0; which < 2; ++which) {
      const QLinearParams& p = which == 0 ? xk_ : xv_;
      w_bf16_[which] = ctx_->alloc((size_t)hidden_ * hidden_ * 2);
      LS_RC(ls100_i8_to_bf16(ctx_->kernels(), p.w, p.k, hidden_, hidden_, w_bf16_[which], ctx_->get_stream()));
    }
  }
  // Post-LN layers hand their output to the next consumer already quantised with that consumer's input clip-max
  // (the next layer's QKV projection, or the output projection after the last layer).
  void set_next_input_amax(float amax) { next_amax_ = amax; }
  float qkv_input_amax() const { return qkv_.amax_in; }
  // The decode step is replayed as one graph launch: the step counter, the ancestry table and the cache history were
  // written by earlier launches, so the self-attention kernel may read them ahead of its grid dependency.
  void set_history_static(bool on) { history_static_ = on; }

  void forward() override {
    const int rows = batch_ * beam_;
    // pre-LN: LayerNorm opens every sublayer. Post-LN (torch_transformer_layers.py:844-965 with normalize_before
    // false): x is the previous LayerNorm's output and a_q its int8 form; LayerNorm closes every sublayer, writing the
    // residual stream in place and the int8 input of the next GEMM.
    if (pre_ln_) ln_quant(rows, ln1_, qkv_.amax_in, embed_src_);
    // qkv = attention_quant(fq_out(acc) + bias): int8 with the KV-cache clip-max
    gemm(b_->a_q, qkv_, rows, LS100_OUT_REQ_S8, b_->qkv_q, Act::None, nullptr, s_kv_);
    {
      ls100_attn_dec_args a;
      memset(&a, 0, sizeof(a));
      a.qkv = b_->qkv_q->value<int8_t>();
      a.ld_qkv = 3 * hidden_;
      a.s_kv = s_kv_;
      a.k_cache = k_cache_;
      a.v_cache = v_cache_;
      a.anc = anc_;
      a.step_ptr = step_ptr_;
      a.rows = rows;
      a.heads = heads_;
      a.max_step = max_step_;
      a.amax_out = out_.amax_in;
      a.out = b_->attn_q->value<int8_t>();
      a.ld_out = hidden_;
      a.history_static = history_static_ ? 1 : 0;
      LS_RC(ls100_attn_dec(ctx_->kernels(), &a, ctx_->get_stream()));
    }
    gemm(b_->attn_q, out_, rows, LS100_OUT_F32, b_->x, Act::None, b_->x, 0.f);
    if (pre_ln_) ln_quant(rows, ln2_, xq_.amax_in);
    else ln_quant(rows, ln1_, xq_.amax_in, nullptr, true);
    gemm(b_->a_q, xq_, rows, LS100_OUT_OUTQ_I8, b_->q_q, Act::None, nullptr, 0.f, false);
    {
      ls100_attn_cross_args a;
      memset(&a, 0, sizeof(a));
      a.q = b_->q_q->value<int8_t>();
      a.ld_q = hidden_;
      a.s_q = xq_.s_out;
      a.bias = xq_.bias;
      a.k = enc_k_;
      a.v = enc_v_;
      a.ld_kv = hidden_;
      a.pad_mask = pad_mask_->value<uint8_t>();
      a.batch = batch_;
      a.beam = beam_;
      a.src_len = src_len_;
      a.heads = heads_;
      a.amax_out = xout_.amax_in;
      a.out = b_->attn_q->value<int8_t>();
      a.ld_out = hidden_;
      a.kv_head_major = 1;
      a.kv_static = 1;  // written by the projection, which copies and memsets separate from the decode kernels
      LS_RC(ls100_attn_cross(ctx_->kernels(), &a, ctx_->get_stream()));
    }
    gemm(b_->attn_q, xout_, rows, LS100_OUT_F32, b_->x, Act::None, b_->x, 0.f);
    if (pre_ln_) ln_quant(rows, ln3_, fc1_.amax_in);
    else ln_quant(rows, ln2_, fc1_.amax_in, nullptr, true);
    gemm(b_->a_q, fc1_, rows, act_ == Act::Relu ? LS100_OUT_REQ_U8 : LS100_OUT_REQ_S8, b_->h_q, act_, nullptr, fc2_.s_in);
    gemm(b_->h_q, fc2_, rows, LS100_OUT_F32, b_->x, Act::None, b_->x, 0.f);
    if (!pre_ln_) ln_quant(rows, ln3_, next_amax_, nullptr, true);
  }

 private:
  // write_f: also write the fp32 LayerNorm output over the residual stream (post-LN; a row is read before it is written)
  void ln_quant(int rows, const LayerNormParams& ln, float amax, const ls100_embed_args* lookup = nullptr, bool write_f = false) {
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = b_->x->value<float>();
    a.ldx = hidden_;
    a.gamma = ln.g;
    a.beta = ln.b;
    a.rows = rows;
    a.hidden = hidden_;
    a.amax = amax;
    a.out_q = b_->a_q->value<int8_t>();
    a.ldq = hidden_;
    if (write_f) {
      a.out_f = b_->x->value<float>();
      a.ldf = hidden_;
    }
    if (lookup) a.emb = *lookup;  // the rows come from the embedding lookup of this decode step, in the same launch
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, ctx_->get_stream()));
  }
  void gemm(Variable* in, const QLinearParams& p, int rows, int out_kind, Variable* out, Act act, Variable* resid,
            float s_req, bool add_bias = true) {
    QuantLinearOp op(ctx_, name_ + ".gemm", &p, out_kind, act, true, add_bias, s_req);
    op(in, out, resid);
    op.before_forward(rows);
    op.forward();
  }
  bool history_static_ = false;
  int hidden_, heads_, ffn_;
  Act act_;
  int max_rows_, max_step_, max_enc_tokens_;
  bool pre_ln_ = true;
  float next_amax_ = 0.f;
  QLinearParams qkv_, out_, xq_, xk_, xv_, xout_, fc1_, fc2_;
  LayerNormParams ln1_, ln2_, ln3_;
  float amax_kv_ = 0, s_kv_ = 0;
  int8_t *k_cache_ = nullptr, *v_cache_ = nullptr;
  float *enc_k_ = nullptr, *enc_v_ = nullptr;
  void* w_bf16_[2] = {nullptr, nullptr};
  StackBuffers* b_ = nullptr;
  Variable* pad_mask_ = nullptr;
  const int32_t* anc_ = nullptr;
  const int32_t* step_ptr_ = nullptr;
  const ls100_embed_args* embed_src_ = nullptr;
  int batch_ = 0, beam_ = 0, src_len_ = 0;
};

// ---------------------------------------------------------------------------------------
// Decoder-only layer (GPT-2 layout: pre-LN, causal self-attention on attention_quant(qkv), GELU FFN), with the
// prefill form (all prompt positions at once, filling the int8 KV cache) and the one-token decode form.
// Counterpart of GptLayer / GptAttentionLayer (lightseq/csrc/layers_new/includes/gpt_layer.h) and of
// QuantGptEncoder::self_attention / self_attention_with_cache (lightseq/inference/model/quant_gpt_encoder.cc.cu:485-658).
class QuantGptLayer : public Layer {
 public:
  // the decode-step embedding lookup to run inside this layer's first LayerNorm launch (first layer of a stack only)
  void set_embed_source(const ls100_embed_args* e) { embed_src_ = e; }
  QuantGptLayer(ContextPtr ctx, const WeightsFile& wf, const std::string& prefix, int layer_id, int max_batch_tokens,
                int max_seq_len, int hidden, int heads, int ffn, int max_batch_size)
      : Layer(prefix, ctx), hidden_(hidden), heads_(heads), ffn_(ffn), max_tokens_(max_batch_tokens),
        max_bs_(max_batch_size), max_step_(max_seq_len) {
    (void)layer_id;
    qkv_.load(*ctx, wf, prefix + ".qkv", false);
    out_.load(*ctx, wf, prefix + ".out", false);
    fc1_.load(*ctx, wf, prefix + ".fc1", false);
    fc2_.load(*ctx, wf, prefix + ".fc2", false, true, true, "", "", true, true);
    ln1_.load(*ctx, wf, prefix + ".ln1", hidden);
    ln2_.load(*ctx, wf, prefix + ".ln2", hidden);
    s_kv_ = wf.amax(prefix + ".kv") / 127.0f;
    fc1_.build_table(*ctx, LS100_OUT_REQ_S8, (int)Act::Gelu, true, fc2_.s_in);  // used by the prompt pass's many-tile GEMM
    const size_t cache = (size_t)max_batch_size * max_seq_len * hidden;
    k_cache_ = ctx->alloc_n<int8_t>(cache);
    v_cache_ = ctx->alloc_n<int8_t>(cache);
    LS_CUDA(cudaMemset(k_cache_, 0, cache));
    LS_CUDA(cudaMemset(v_cache_, 0, cache));
  }
  void set_history_static(bool on) { history_static_ = on; }  // see QuantTransformerDecoderLayer
  void operator()(StackBuffers* bufs, const int32_t* step_ptr) {
    b_ = bufs;
    step_ptr_ = step_ptr;
  }
  // prompt_len > 0: prefill of batch x prompt_len rows; prompt_len == 0: one token per sequence at *step_ptr
  void before_forward(int batch, int prompt_len) {
    batch_ = batch;
    prompt_ = prompt_len;
    if (batch > max_bs_) throw std::runtime_error("batch exceeds max_batch_size");
    if ((long long)batch * std::max(prompt_len, 1) > max_tokens_) throw std::runtime_error("tokens exceed max_batch_tokens");
    if (prompt_len > max_step_) throw std::runtime_error("prompt longer than max_step");
  }
  void forward() override {
    const int rows = prompt_ > 0 ? batch_ * prompt_ : batch_;
    ln_quant(rows, ln1_, qkv_.amax_in, embed_src_);
    gemm(b_->a_q, qkv_, rows, LS100_OUT_REQ_S8, b_->qkv_q, Act::None, nullptr, s_kv_);
    if (prompt_ > 0) {
      ls100_attn_self_args a;
      memset(&a, 0, sizeof(a));
      a.qkv = b_->qkv_q->value<int8_t>();
      a.ld_qkv = 3 * hidden_;
      a.s_qkv = s_kv_;
      a.batch = batch_;
      a.seq = prompt_;
      a.heads = heads_;
      a.causal = 1;
      a.amax_out = out_.amax_in;
      a.out = b_->attn_q->value<int8_t>();
      a.ld_out = hidden_;
      a.k_cache = k_cache_;
      a.v_cache = v_cache_;
      a.max_step = max_step_;
      LS_RC(ls100_attn_self(ctx_->kernels(), &a, ctx_->get_stream()));
    } else {
      ls100_attn_dec_args a;
      memset(&a, 0, sizeof(a));
      a.qkv = b_->qkv_q->value<int8_t>();
      a.ld_qkv = 3 * hidden_;
      a.s_kv = s_kv_;
      a.k_cache = k_cache_;
      a.v_cache = v_cache_;
      a.step_ptr = step_ptr_;
      a.rows = rows;
      a.heads = heads_;
      a.max_step = max_step_;
      a.amax_out = out_.amax_in;
      a.out = b_->attn_q->value<int8_t>();
      a.ld_out = hidden_;
      a.history_static = history_static_ ? 1 : 0;
      LS_RC(ls100_attn_dec(ctx_->kernels(), &a, ctx_->get_stream()));
    }
    gemm(b_->attn_q, out_, rows, LS100_OUT_F32, b_->x, Act::None, b_->x, 0.f);
    ln_quant(rows, ln2_, fc1_.amax_in);
    gemm(b_->a_q, fc1_, rows, LS100_OUT_REQ_S8, b_->h_q, Act::Gelu, nullptr, fc2_.s_in);
    gemm(b_->h_q, fc2_, rows, LS100_OUT_F32, b_->x, Act::None, b_->x, 0.f);
  }

 private:
  void ln_quant(int rows, const LayerNormParams& ln, float amax, const ls100_embed_args* lookup = nullptr) {
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = b_->x->value<float>();
    a.ldx = hidden_;
    a.gamma = ln.g;
    a.beta = ln.b;
    a.rows = rows;
    a.hidden = hidden_;
    a.amax = amax;
    a.out_q = b_->a_q->value<int8_t>();
    a.ldq = hidden_;
    if (lookup) a.emb = *lookup;  // the rows come from the embedding lookup of this decode step, in the same launch
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, ctx_->get_stream()));
  }
  void gemm(Variable* in, const QLinearParams& p, int rows, int out_kind, Variable* out, Act act, Variable* resid, float s_req) {
    QuantLinearOp op(ctx_, name_ + ".gemm", &p, out_kind, act, true, true, s_req);
    op(in, out, resid);
    op.before_forward(rows);
    op.forward();
  }
  bool history_static_ = false;
  int hidden_, heads_, ffn_, max_tokens_, max_bs_, max_step_;
  QLinearParams qkv_, out_, fc1_, fc2_;
  LayerNormParams ln1_, ln2_;
  float s_kv_ = 0.f;
  int8_t *k_cache_ = nullptr, *v_cache_ = nullptr;
  StackBuffers* b_ = nullptr;
  const int32_t* step_ptr_ = nullptr;
  const ls100_embed_args* embed_src_ = nullptr;
  int batch_ = 0, prompt_ = 0;
};

}  // namespace ls100
