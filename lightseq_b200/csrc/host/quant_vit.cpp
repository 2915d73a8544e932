// QuantVit: ViT encoder with int8 layers behind the LSModel interface: fp32 patch embedding (convolution with
// kernel = stride = patch, class token, learned positions), pre-LN encoder layers, final LayerNorm.
// Replaces lightseq/inference/pywrapper/quant_vit.cc + QuantVitEncoder
// (lightseq/inference/model/quant_vit_encoder.cc.cu:189-232); the layers are the same
// QuantTransformerEncoderLayer the Transformer encoder uses.
#include <memory>

#include "engine_model.h"
#include "layers.h"

namespace ls100 {

class QuantVit : public EngineModel {
 public:
  QuantVit(const std::string& weight_path, int max_batch_size)
      : EngineModel({"pixel_input"}, {"encoder_output"}), max_bs_(max_batch_size) {
    WeightsFile wf(weight_path);
    H_ = (int)wf.conf("hidden");
    heads_ = (int)wf.conf("heads");
    F_ = (int)wf.conf("ffn");
    n_layer_ = (int)wf.conf("n_enc");
    image_ = (int)wf.conf("image_size");
    patch_ = (int)wf.conf("patch_size");
    channels_ = (int)wf.conf_or("channels", 3.0);
    const bool gelu = wf.conf_or("act_gelu", 1.0) != 0.0;
    const bool pre_ln = wf.conf_or("pre_ln", 1.0) != 0.0;
    if (H_ != heads_ * 64) throw std::runtime_error("QuantVit: head_dim must be 64");
    if (!pre_ln) throw std::runtime_error("QuantVit: expects a pre-LN model");
    if (patch_ < 1 || image_ < patch_ || image_ % patch_) throw std::runtime_error("QuantVit: image_size must be a multiple of patch_size");
    if (max_batch_size < 1) throw std::runtime_error("max_batch_size must be positive");
    seq_ = 1 + (image_ / patch_) * (image_ / patch_);
    ctx_ = Context::create(StatusType::Inference);
    Context& c = *ctx_;
    const int K = channels_ * patch_ * patch_;
    {  // the convolution weight [hidden, K] is kept transposed, [K, hidden]: threads of a warp read consecutive channels
      const HostTensor& cw = wf.tensor("conv.w");
      if (cw.numel() != (int64_t)H_ * K) throw std::runtime_error("conv.w: size mismatch");
      std::vector<float> tr((size_t)K * H_);
      for (int h = 0; h < H_; ++h)
        for (int k = 0; k < K; ++k) tr[(size_t)k * H_ + h] = cw.data[(size_t)h * K + k];
      conv_wt_ = c.alloc_n<float>(tr.size());
      LS_CUDA(cudaMemcpy(conv_wt_, tr.data(), tr.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    conv_b_ = upload_vec(c, wf, "conv.b", H_);
    pos_ = upload_vec(c, wf, "pos", (int64_t)seq_ * H_);
    cls_ = upload_vec(c, wf, "cls", H_);
    final_ln_.load(c, wf, "enc.ln", H_);
    const int max_tokens = max_bs_ * seq_;
    for (int l = 0; l < n_layer_; ++l)
      layers_.emplace_back(new QuantTransformerEncoderLayer(ctx_, wf, "enc." + std::to_string(l), l, max_tokens, seq_, H_,
                                                            heads_, F_, true, gelu ? "gelu" : "relu"));
    auto mk = [&](const char* n, size_t bytes) { vars_.emplace_back(new Variable(n, c, bytes)); return vars_.back().get(); };
    buf_.x = mk("x", (size_t)max_tokens * H_ * 4);
    buf_.a_q = mk("a_q", (size_t)max_tokens * H_);
    buf_.qkv_q = mk("qkv_q", (size_t)max_tokens * 3 * H_);
    buf_.attn_q = mk("attn_q", (size_t)max_tokens * H_);
    buf_.h_q = mk("h_q", (size_t)max_tokens * F_);
  }

  void Infer() override {
    const std::vector<int>& shp = input_shapes_[0];
    if (shp.size() != 4 || shp[1] != channels_ || shp[2] != image_ || shp[3] != image_)
      throw std::runtime_error("pixel_input must be [batch, channels, image_size, image_size]");
    const int B = shp[0];
    if (B > max_bs_) throw std::runtime_error("batch size of input greater than max_batch_size");
    if (B < 1) throw std::runtime_error("empty input");
    if (!d_pixels_ || !d_out_) throw std::runtime_error("input/output pointers not set");
    LS_CUDA(cudaSetDevice(ctx_->device()));
    cudaStream_t st = ctx_->get_stream();
    ls100_patch_embed_args e;
    memset(&e, 0, sizeof(e));
    e.pixels = d_pixels_;
    e.conv_wt = conv_wt_;
    e.conv_bias = conv_b_;
    e.pos = pos_;
    e.cls = cls_;
    e.batch = B;
    e.channels = channels_;
    e.image = image_;
    e.patch = patch_;
    e.hidden = H_;
    e.out = buf_.x->value<float>();
    LS_RC(ls100_patch_embed(ctx_->kernels(), &e, st));
    for (auto& l : layers_) {
      (*l)(&buf_, nullptr);  // no token is padding
      l->before_forward(B, seq_);
      l->forward();
    }
    ls100_ln_quant_args a;  // final LayerNorm, fp32 only, straight into the caller's buffer
    memset(&a, 0, sizeof(a));
    a.x = buf_.x->value<float>();
    a.ldx = H_;
    a.gamma = final_ln_.g;
    a.beta = final_ln_.b;
    a.rows = B * seq_;
    a.hidden = H_;
    a.out_f = d_out_;
    a.ldf = H_;
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, st));
    LS_CUDA(cudaStreamSynchronize(st));
    const int err = ls100_ctx_poll_error(ctx_->kernels(), st);
    if (err != 0) throw std::runtime_error(std::string("device reported: ") + ls100_strerror(err));
    set_output_shape(0, {B, seq_, H_});
  }

  void set_input_ptr(int index, void* p) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    d_pixels_ = static_cast<const float*>(p);
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
    return {max_bs_, channels_, image_, image_};
  }
  std::vector<int> get_output_max_shape(int index) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    return {max_bs_, seq_, H_};
  }
  DataType get_input_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    return kFloat32;
  }
  DataType get_output_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    return kFloat32;
  }
  void benchmark_mode(bool) override {}
  ContextPtr context() const override { return ctx_; }

 private:
  int max_bs_, H_ = 0, heads_ = 0, F_ = 0, n_layer_ = 0, image_ = 0, patch_ = 0, channels_ = 3, seq_ = 0;
  ContextPtr ctx_;
  float *conv_wt_ = nullptr, *conv_b_ = nullptr, *pos_ = nullptr, *cls_ = nullptr;
  LayerNormParams final_ln_;
  std::vector<std::unique_ptr<QuantTransformerEncoderLayer>> layers_;
  std::vector<std::unique_ptr<Variable>> vars_;
  StackBuffers buf_;
  const float* d_pixels_ = nullptr;
  float* d_out_ = nullptr;
};

LSMODEL_REGISTER(QuantVit)

}  // namespace ls100
