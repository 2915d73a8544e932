// QuantBert: int8 BERT encoder (post-LN, GELU) behind the LSModel interface.
// Replaces lightseq/inference/pywrapper/quant_bert.cc + QuantBertEncoder
// (lightseq/inference/model/quant_bert_encoder.cc.cu:214-520); numerics follow BertEmbeddingLayer +
// post-LN TransformerEncoderLayer (lightseq/training/ops/pytorch/torch_transformer_layers.py:1177-1207, 630-679).
#include <memory>

#include "engine_model.h"
#include "layers.h"

namespace ls100 {

class QuantBert : public EngineModel {
 public:
  QuantBert(const std::string& weight_path, int max_batch_size)
      : EngineModel({"token_ids"}, {"encoder_output"}), max_bs_(max_batch_size) {
    WeightsFile wf(weight_path);
    H_ = (int)wf.conf("hidden");
    heads_ = (int)wf.conf("heads");
    F_ = (int)wf.conf("ffn");
    n_layer_ = (int)wf.conf("n_enc");
    V_ = (int)wf.conf("vocab");
    max_step_ = (int)wf.conf("max_step");
    pad_id_ = (int)wf.conf("pad_id");
    const bool gelu = wf.conf_or("act_gelu", 1.0) != 0.0;
    const bool pre_ln = wf.conf_or("pre_ln", 0.0) != 0.0;
    if (H_ != heads_ * 64) throw std::runtime_error("QuantBert: head_dim must be 64");
    if (pre_ln) throw std::runtime_error("QuantBert: expects a post-LN model");
    if (max_batch_size < 1) throw std::runtime_error("max_batch_size must be positive");
    ctx_ = Context::create(StatusType::Inference);
    Context& c = *ctx_;
    const int max_tokens = max_bs_ * max_step_;
    // embedding table = quant(word + token_type[0]) with the embedding clip-max; positions fp32
    {
      const HostTensor& we = wf.tensor("emb");
      const HostTensor& te = wf.tensor("type_emb");
      if (we.dims.size() != 2 || we.dims[0] != V_ || we.dims[1] != H_ || te.numel() < H_)
        throw std::runtime_error("QuantBert: bad embedding tensors");
      std::vector<float> sum((size_t)V_ * H_);
      for (int v = 0; v < V_; ++v)
        for (int h = 0; h < H_; ++h) sum[(size_t)v * H_ + h] = we.data[(size_t)v * H_ + h] + te.data[h];
      float* staging = nullptr;
      LS_CUDA(cudaMalloc(&staging, sum.size() * sizeof(float)));
      LS_CUDA(cudaMemcpy(staging, sum.data(), sum.size() * sizeof(float), cudaMemcpyHostToDevice));
      emb_q_ = c.alloc_n<int8_t>(sum.size());
      amax_emb_ = wf.amax("emb");
      LS_RC(ls100_quantize_weight(c.kernels(), staging, V_, H_, amax_emb_, emb_q_, nullptr, c.get_stream()));
      LS_CUDA(cudaStreamSynchronize(c.get_stream()));
      LS_CUDA(cudaFree(staging));
    }
    n_pos_ = (int)wf.tensor("pos").dims[0];
    pos_ = upload_vec(c, wf, "pos", (int64_t)n_pos_ * H_);
    emb_ln_.load(c, wf, "emb.ln", H_);
    for (int l = 0; l < n_layer_; ++l)
      layers_.emplace_back(new QuantTransformerEncoderLayer(ctx_, wf, "enc." + std::to_string(l), l, max_tokens, max_step_,
                                                            H_, heads_, F_, false, gelu ? "gelu" : "relu"));
    for (int l = 0; l < n_layer_; ++l)
      layers_[l]->set_next_input_amax(l + 1 < n_layer_ ? layers_[l + 1]->qkv().amax_in : 0.f);
    auto mk = [&](const char* n, size_t bytes) { vars_.emplace_back(new Variable(n, c, bytes)); return vars_.back().get(); };
    buf_.x = mk("x", (size_t)max_tokens * H_ * 4);
    buf_.a_q = mk("a_q", (size_t)max_tokens * H_);
    buf_.qkv_q = mk("qkv_q", (size_t)max_tokens * 3 * H_);
    buf_.attn_q = mk("attn_q", (size_t)max_tokens * H_);
    buf_.h_q = mk("h_q", (size_t)max_tokens * F_);
    pad_mask_ = mk("pad_mask", (size_t)max_tokens);
  }

  void Infer() override {
    if (input_shapes_[0].size() != 2) throw std::runtime_error("token_ids must be [batch, seq_len]");
    const int B = input_shapes_[0][0], S = input_shapes_[0][1];
    if (B > max_bs_) throw std::runtime_error("batch size of input greater than max_batch_size");
    if (S > max_step_) throw std::runtime_error("seq len of input greater than max_step");
    if (B < 1 || S < 1) throw std::runtime_error("empty input");
    if (!d_ids_ || !d_out_) throw std::runtime_error("input/output pointers not set");
    LS_CUDA(cudaSetDevice(ctx_->device()));
    cudaStream_t st = ctx_->get_stream();
    ls100_embed_args e;
    memset(&e, 0, sizeof(e));
    e.ids = d_ids_;
    e.ld_ids = S;
    e.batch = B;
    e.seq = S;
    e.hidden = H_;
    e.table_q = emb_q_;
    e.s_emb = amax_emb_ / 127.0f;
    e.sqrt_h = 1.0f;
    e.pos = pos_;
    e.n_pos = n_pos_;
    e.pad_id = pad_id_;
    e.vocab = V_;
    e.out = buf_.x->value<float>();
    e.pad_mask = pad_mask_->value<uint8_t>();
    e.pos_mode = 1;
    LS_RC(ls100_embed(ctx_->kernels(), &e, st));
    // embedding LayerNorm -> residual stream (fp32) and the int8 input of layer 0
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = buf_.x->value<float>();
    a.ldx = H_;
    a.gamma = emb_ln_.g;
    a.beta = emb_ln_.b;
    a.rows = B * S;
    a.hidden = H_;
    a.amax = layers_[0]->qkv().amax_in;
    a.out_q = buf_.a_q->value<int8_t>();
    a.ldq = H_;
    a.out_f = buf_.x->value<float>();
    a.ldf = H_;
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, st));
    tap_reset();
    tap(buf_.x->value<float>(), (size_t)B * S * H_, st);
    for (auto& l : layers_) {
      (*l)(&buf_, pad_mask_);
      l->before_forward(B, S);
      l->forward();
      tap(buf_.x->value<float>(), (size_t)B * S * H_, st);
    }
    LS_CUDA(cudaMemcpyAsync(d_out_, buf_.x->value<float>(), (size_t)B * S * H_ * 4, cudaMemcpyDeviceToDevice, st));
    LS_CUDA(cudaStreamSynchronize(st));
    const int err = ls100_ctx_poll_error(ctx_->kernels(), st);
    if (err != 0) throw std::runtime_error(std::string("device reported: ") + ls100_strerror(err));
    set_output_shape(0, {B, S, H_});
  }

  void set_input_ptr(int index, void* p) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    d_ids_ = static_cast<const int32_t*>(p);
  }
  void set_output_ptr(int index, void* p) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    d_out_ = static_cast<float*>(p);
  }
  const void* get_output_ptr(int index) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    return d_out_;
  }
  std::vector<int> get_input_max_shape(int index) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    return {max_bs_, max_step_};
  }
  std::vector<int> get_output_max_shape(int index) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    return {max_bs_, max_step_, H_};
  }
  DataType get_input_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    return kInt32;
  }
  DataType get_output_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    return kFloat32;
  }
  void benchmark_mode(bool) override {}
  ContextPtr context() const override { return ctx_; }

 private:
  int max_bs_, H_ = 0, heads_ = 0, F_ = 0, n_layer_ = 0, V_ = 0, max_step_ = 0, pad_id_ = 0, n_pos_ = 0;
  float amax_emb_ = 0.f;
  ContextPtr ctx_;
  int8_t* emb_q_ = nullptr;
  float* pos_ = nullptr;
  LayerNormParams emb_ln_;
  std::vector<std::unique_ptr<QuantTransformerEncoderLayer>> layers_;
  std::vector<std::unique_ptr<Variable>> vars_;
  StackBuffers buf_;
  Variable* pad_mask_ = nullptr;
  const int32_t* d_ids_ = nullptr;
  float* d_out_ = nullptr;
};

LSMODEL_REGISTER(QuantBert)

}  // namespace ls100
