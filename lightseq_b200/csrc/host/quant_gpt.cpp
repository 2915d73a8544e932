// QuantGpt: int8 GPT-2 style decoder-only generation with top-k sampling, behind the LSModel interface.
// Replaces lightseq/inference/pywrapper/quant_gpt.cc + QuantGptEncoder::run_one_sample
// (lightseq/inference/model/quant_gpt_encoder.cc.cu:300-481). As in the QuantTransformer engine, one decode
// step is a CUDA graph replayed with the position in device memory; the KV cache is appended in place (the
// reference copies the whole cache every token, gptKernels_int8.cc.cu:658-812); sampling needs no host sync.
#include <algorithm>
#include <map>
#include <cstdlib>
#include <memory>

#include "engine_model.h"
#include "layers.h"

namespace ls100 {

class QuantGpt : public EngineModel {
 public:
  QuantGpt(const std::string& weight_path, int max_batch_size)
      : EngineModel({"token_ids"}, {"gpt_out"}), max_bs_(max_batch_size) {
    WeightsFile wf(weight_path);
    H_ = (int)wf.conf("hidden");
    heads_ = (int)wf.conf("heads");
    F_ = (int)wf.conf("ffn");
    n_layer_ = (int)wf.conf("n_dec");
    V_ = (int)wf.conf("vocab");
    max_step_ = (int)wf.conf("max_step");
    end_id_ = (int)wf.conf("end_id");
    topk_ = (int)wf.conf_or("topk", 1);
    topp_ = (float)wf.conf_or("topp", 0.0);  // > 0 selects nucleus sampling, as sampling_method "topp" does in the reference
    max_new_ = (int)wf.conf_or("max_new_tokens", max_step_);
    pad_id_ = (int)wf.conf_or("pad_id", -1);
    const uint64_t seed = (uint64_t)wf.conf_or("rng_seed", 2024);
    seed_lo_ = (uint32_t)(seed & 0xffffffffu);
    seed_hi_ = (uint32_t)(seed >> 32);
    if (H_ != heads_ * 64) throw std::runtime_error("QuantGpt: head_dim must be 64");
    if (topk_ < 1 || topk_ > 8) throw std::runtime_error("QuantGpt: topk must be in [1, 8]");
    if (topp_ < 0.f || topp_ > 1.f) throw std::runtime_error("QuantGpt: topp must be in [0, 1]");
    if (max_batch_size < 1) throw std::runtime_error("max_batch_size must be positive");
    ctx_ = Context::create(StatusType::Inference);
    Context& c = *ctx_;
    const int max_tokens = max_bs_ * max_step_;
    emb_.load(c, wf, "logits", false, true, true, "emb", "emb", false);
    n_pos_ = (int)wf.tensor("pos").dims[0];
    pos_ = upload_vec(c, wf, "pos", (int64_t)n_pos_ * H_);
    for (int l = 0; l < n_layer_; ++l)
      layers_.emplace_back(new QuantGptLayer(ctx_, wf, "dec." + std::to_string(l), l, max_tokens, max_step_, H_, heads_, F_, max_bs_));
    ln_f_.load(c, wf, "dec.ln", H_);
    auto mk = [&](const char* n, size_t bytes) { vars_.emplace_back(new Variable(n, c, bytes)); return vars_.back().get(); };
    buf_.x = mk("x", (size_t)max_tokens * H_ * 4);
    buf_.a_q = mk("a_q", (size_t)max_tokens * H_);
    buf_.qkv_q = mk("qkv_q", (size_t)max_tokens * 3 * H_);
    buf_.attn_q = mk("attn_q", (size_t)max_tokens * H_);
    buf_.h_q = mk("h_q", (size_t)max_tokens * F_);
    last_q_ = mk("last_q", (size_t)max_bs_ * H_);
    ldv_ = (V_ + 15) / 16 * 16;
    logits_q_ = mk("logits_q", (size_t)max_bs_ * ldv_);
    seq_ = c.alloc_n<int32_t>((size_t)max_bs_ * max_step_);
    counters_ = c.alloc_n<int32_t>(4);  // cur, ticket, n_ended, stop
    stop_host_ = static_cast<int32_t*>(c.alloc_host_mapped(sizeof(int32_t)));
    LS_CUDA(cudaHostGetDevicePointer((void**)&stop_host_dev_, stop_host_, 0));
    h_seq_.assign((size_t)max_bs_ * max_step_, end_id_);
    LS_CUDA(cudaHostRegister(h_seq_.data(), h_seq_.size() * 4, cudaHostRegisterDefault));
    for (auto& e : ring_) LS_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    use_graph_ = getenv("LS100_NO_GRAPH") == nullptr;
    for (auto& l : layers_) l->set_history_static(use_graph_);  // a decode step is then one graph launch
  }
  ~QuantGpt() override {
    cudaSetDevice(ctx_->device());
    cudaStreamSynchronize(ctx_->get_stream());
    for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second);
    for (auto& e : ring_) cudaEventDestroy(e);
    cudaHostUnregister(h_seq_.data());
  }

  void Infer() override {
    if (input_shapes_[0].size() != 2) throw std::runtime_error("token_ids must be [batch, seq_len]");
    const int B = input_shapes_[0][0], P = input_shapes_[0][1];
    if (B > max_bs_) throw std::runtime_error("batch size of input greater than max_batch_size");
    if (P >= max_step_) throw std::runtime_error("seq len of input greater than max_step");
    if (B < 1 || P < 1) throw std::runtime_error("empty input");
    if (!d_ids_ || !d_out_) throw std::runtime_error("input/output pointers not set");
    LS_CUDA(cudaSetDevice(ctx_->device()));
    cudaStream_t st = ctx_->get_stream();
    // token history: prompt, then end_id filler
    LS_CUDA(cudaMemcpyAsync(seq_, h_seq_.data(), (size_t)B * max_step_ * 4, cudaMemcpyHostToDevice, st));
    LS_CUDA(cudaMemcpy2DAsync(seq_, (size_t)max_step_ * 4, d_ids_, (size_t)P * 4, (size_t)P * 4, B, cudaMemcpyDeviceToDevice, st));
    const int32_t init[4] = {P - 1, 0, 0, -1};
    LS_CUDA(cudaMemcpyAsync(counters_, init, sizeof(init), cudaMemcpyHostToDevice, st));
    *stop_host_ = -1;
    const int last = std::min(max_step_, P + max_new_);  // exclusive bound on positions
    if (last > P) {
      prefill(B, P);
      int launched = 1;
      cudaGraphExec_t exec = use_graph_ ? decode_graph(B) : nullptr;
      for (int pos = P; pos + 1 < last; ++pos) {  // the step at `pos` consumes token[pos] and produces token[pos + 1]
        const int s = pos - P;
        if (s >= kRing) {
          LS_CUDA(cudaEventSynchronize(ring_[s % kRing]));
          if (!benchmark_ && *((volatile int32_t*)stop_host_) >= 0) break;
        }
        if (exec) LS_CUDA(cudaGraphLaunch(exec, st));
        else decode_step(B);
        LS_CUDA(cudaEventRecord(ring_[s % kRing], st));
        ++launched;
      }
      steps_run_ = launched;
    }
    int32_t h[4];
    LS_CUDA(cudaMemcpyAsync(h, counters_, sizeof(h), cudaMemcpyDeviceToHost, st));
    LS_CUDA(cudaStreamSynchronize(st));
    const int err = ls100_ctx_poll_error(ctx_->kernels(), st);
    if (err != 0) throw std::runtime_error(std::string("device reported: ") + ls100_strerror(err));
    int n_out = h[0] + 1;                                   // tokens known = newest index + 1
    if (!benchmark_ && h[3] >= 0) n_out = std::min(n_out, h[3] + 1);  // stop at the position where every row had ended
    LS_CUDA(cudaMemcpy2DAsync(d_out_, (size_t)n_out * 4, seq_, (size_t)max_step_ * 4, (size_t)n_out * 4, B, cudaMemcpyDeviceToDevice, st));
    LS_CUDA(cudaStreamSynchronize(st));
    set_output_shape(0, {B, n_out});
  }

  void set_input_ptr(int index, void* p) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    d_ids_ = static_cast<const int32_t*>(p);
  }
  void set_output_ptr(int index, void* p) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    d_out_ = static_cast<int32_t*>(p);
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
    return {max_bs_, max_step_};
  }
  DataType get_input_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    return kInt32;
  }
  DataType get_output_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid output index");
    return kInt32;
  }
  void benchmark_mode(bool b) override { benchmark_ = b; }
  ContextPtr context() const override { return ctx_; }

  // Mean negative log-likelihood of each sequence's own next tokens (QuantGptEncoder::run_one_infer +
  // compute_ppl, lightseq/inference/model/quant_gpt_encoder.cc.cu:257-298,797-822): the prompt pass, then the
  // logits of EVERY position, kPplRows rows at a time so that the int8 logits never need more than one slab.
  void Ppl(const int32_t* d_ids, int B, int S, float* d_ppl) {
    if (B > max_bs_) throw std::runtime_error("batch size of input greater than max_batch_size");
    if (S > max_step_) throw std::runtime_error("seq len of input greater than max_step");
    if (B < 1 || S < 1) throw std::runtime_error("empty input");
    LS_CUDA(cudaSetDevice(ctx_->device()));
    cudaStream_t st = ctx_->get_stream();
    ls100_ctx* k = ctx_->kernels();
    Context& c = *ctx_;
    const int rows = B * S;
    if (!ppl_logits_) {
      ppl_logits_ = new Variable("ppl_logits", c, (size_t)kPplRows * ldv_);
      vars_.emplace_back(ppl_logits_);
      ppl_nll_ = c.alloc_n<float>((size_t)max_bs_ * max_step_);
    }
    const int32_t* saved = d_ids_;
    d_ids_ = d_ids;
    embed(B, S, false);
    d_ids_ = saved;
    for (auto& l : layers_) {
      (*l)(&buf_, counters_);
      l->before_forward(B, S);
      l->forward();
    }
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = buf_.x->value<float>();
    a.ldx = H_;
    a.gamma = ln_f_.g;
    a.beta = ln_f_.b;
    a.rows = rows;
    a.hidden = H_;
    a.amax = emb_.amax_in;
    a.out_q = buf_.a_q->value<int8_t>();
    a.ldq = H_;
    LS_RC(ls100_ln_quant(k, &a, st));
    for (int r0 = 0; r0 < rows; r0 += kPplRows) {
      const int n = std::min(kPplRows, rows - r0);
      ls100_gemm_i8_args g;
      memset(&g, 0, sizeof(g));
      g.a = buf_.a_q->value<int8_t>() + (size_t)r0 * H_;
      g.lda = H_;
      g.w = emb_.w;
      g.ldw = H_;
      g.m = n;
      g.n = V_;
      g.k = H_;
      g.s_acc = emb_.s_acc;
      g.s_outq = emb_.s_out;
      g.out_kind = LS100_OUT_OUTQ_I8;
      g.out = ppl_logits_->value<int8_t>();
      g.ldo = ldv_;
      LS_RC(ls100_gemm_i8(k, &g, st));
      ls100_token_nll_args t;
      memset(&t, 0, sizeof(t));
      t.logits = ppl_logits_->value<int8_t>();
      t.ld_logits = ldv_;
      t.s_logits = emb_.s_out;
      t.rows = n;
      t.row0 = r0;
      t.vocab = V_;
      t.ids = d_ids;
      t.batch = B;
      t.seq = S;
      t.nll = ppl_nll_;
      LS_RC(ls100_token_nll(k, &t, st));
    }
    ls100_seq_ppl_args p;
    memset(&p, 0, sizeof(p));
    p.nll = ppl_nll_;
    p.ids = d_ids;
    p.batch = B;
    p.seq = S;
    p.pad_id = pad_id_;
    p.ppl = d_ppl;
    LS_RC(ls100_seq_ppl(k, &p, st));
    LS_CUDA(cudaStreamSynchronize(st));
    const int err = ls100_ctx_poll_error(k, st);
    if (err != 0) throw std::runtime_error(std::string("device reported: ") + ls100_strerror(err));
  }
  int steps_run() const { return steps_run_; }

 private:
  static constexpr int kRing = 4;
  static constexpr int kPplRows = 4096;
  ls100_embed_args embed_args_;  // outlives embed(): the first layer reads it during its forward()

  // decode && fuse: the lookup is handed to the first layer, which runs it inside its first LayerNorm launch
  void embed(int B, int P, bool decode) {
    static const bool separate_embed = getenv("LS100_NO_EMBED_FUSE") != nullptr;
    const bool fused = decode && !separate_embed && B <= 2048 && !layers_.empty();
    ls100_embed_args& e = embed_args_;
    memset(&e, 0, sizeof(e));
    e.ids = decode ? seq_ : d_ids_;
    e.ld_ids = decode ? max_step_ : P;
    e.batch = B;
    e.seq = decode ? 1 : P;
    e.hidden = H_;
    e.step_ptr = decode ? counters_ : nullptr;
    e.table_q = emb_.w;
    e.s_emb = emb_.s_w;
    e.sqrt_h = 1.0f;
    e.pos = pos_;
    e.n_pos = n_pos_;
    e.pad_id = -1;
    e.vocab = V_;
    e.out = buf_.x->value<float>();
    e.pos_mode = 1;
    if (!layers_.empty()) layers_[0]->set_embed_source(fused ? &e : nullptr);
    if (!fused) LS_RC(ls100_embed(ctx_->kernels(), &e, ctx_->get_stream()));
  }
  // final LayerNorm of the newest position of every row -> int8 -> logits -> sample
  void head(int B, int row_stride, int row_offset) {
    ls100_ctx* k = ctx_->kernels();
    cudaStream_t st = ctx_->get_stream();
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = buf_.x->value<float>() + (size_t)row_offset * H_;
    a.ldx = (int64_t)row_stride * H_;
    a.gamma = ln_f_.g;
    a.beta = ln_f_.b;
    a.rows = B;
    a.hidden = H_;
    a.amax = emb_.amax_in;
    a.out_q = last_q_->value<int8_t>();
    a.ldq = H_;
    LS_RC(ls100_ln_quant(k, &a, st));
    QuantLinearOp logits(ctx_, "logits", &emb_, LS100_OUT_OUTQ_I8, Act::None, true, false);
    logits(last_q_, logits_q_);
    logits.before_forward(B, ldv_);
    logits.forward();
    if (topp_ > 0.f) {
      ls100_sample_topp_args s;
      memset(&s, 0, sizeof(s));
      s.logits = logits_q_->value<int8_t>();
      s.ld_logits = ldv_;
      s.s_logits = emb_.s_out;
      s.p = topp_;
      s.rows = B;
      s.vocab = V_;
      s.max_step = max_step_;
      s.end_id = end_id_;
      s.seed_lo = seed_lo_;
      s.seed_hi = seed_hi_;
      s.seq = seq_;
      s.cur = counters_;
      s.ticket = counters_ + 1;
      s.n_ended = counters_ + 2;
      s.stop = counters_ + 3;
      s.stop_host = stop_host_dev_;
      LS_RC(ls100_sample_topp(k, &s, st));
      return;
    }
    ls100_sample_topk_args s;
    memset(&s, 0, sizeof(s));
    s.logits = logits_q_->value<int8_t>();
    s.ld_logits = ldv_;
    s.s_logits = emb_.s_out;
    s.rows = B;
    s.vocab = V_;
    s.k = topk_;
    s.max_step = max_step_;
    s.end_id = end_id_;
    s.seed_lo = seed_lo_;
    s.seed_hi = seed_hi_;
    s.seq = seq_;
    s.cur = counters_;
    s.ticket = counters_ + 1;
    s.n_ended = counters_ + 2;
    s.stop = counters_ + 3;
    s.stop_host = stop_host_dev_;
    LS_RC(ls100_sample_topk(k, &s, st));
  }
  void prefill(int B, int P) {
    embed(B, P, false);
    tap_reset();
    tap(buf_.x->value<float>(), (size_t)B * P * H_, ctx_->get_stream());
    for (auto& l : layers_) {
      (*l)(&buf_, counters_);
      l->before_forward(B, P);
      l->forward();
      tap(buf_.x->value<float>(), (size_t)B * P * H_, ctx_->get_stream());
    }
    head(B, P, P - 1);
  }
  void decode_step(int B) {
    embed(B, 1, true);
    for (auto& l : layers_) {
      (*l)(&buf_, counters_);
      l->before_forward(B, 0);
      l->forward();
    }
    head(B, 1, 0);
  }
  cudaGraphExec_t decode_graph(int B) {
    auto it = graphs_.find(B);
    if (it != graphs_.end()) return it->second;
    cudaStream_t st = ctx_->get_stream();
    cudaGraph_t g = nullptr;
    LS_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    try {
      decode_step(B);
    } catch (...) {
      cudaStreamEndCapture(st, &g);
      if (g) cudaGraphDestroy(g);
      throw;
    }
    LS_CUDA(cudaStreamEndCapture(st, &g));
    cudaGraphExec_t exec = nullptr;
    LS_CUDA(cudaGraphInstantiate(&exec, g, 0));
    cudaGraphDestroy(g);
    graphs_[B] = exec;
    return exec;
  }

  int max_bs_, H_ = 0, heads_ = 0, F_ = 0, n_layer_ = 0, V_ = 0, max_step_ = 0, end_id_ = 0, topk_ = 1, max_new_ = 0;
  int n_pos_ = 0, ldv_ = 0;
  float topp_ = 0.f;
  int pad_id_ = -1;
  Variable* ppl_logits_ = nullptr;
  float* ppl_nll_ = nullptr;
  uint32_t seed_lo_ = 0, seed_hi_ = 0;
  ContextPtr ctx_;
  QLinearParams emb_;
  float* pos_ = nullptr;
  std::vector<std::unique_ptr<QuantGptLayer>> layers_;
  LayerNormParams ln_f_;
  std::vector<std::unique_ptr<Variable>> vars_;
  StackBuffers buf_;
  Variable *last_q_ = nullptr, *logits_q_ = nullptr;
  int32_t *seq_ = nullptr, *counters_ = nullptr, *stop_host_ = nullptr, *stop_host_dev_ = nullptr;
  std::vector<int32_t> h_seq_;
  cudaEvent_t ring_[kRing];
  std::map<int, cudaGraphExec_t> graphs_;
  bool use_graph_ = true, benchmark_ = false;
  const int32_t* d_ids_ = nullptr;
  int32_t* d_out_ = nullptr;
  int steps_run_ = 0;
};

LSMODEL_REGISTER(QuantGpt)

void quant_gpt_ppl(LSModel* m, const int32_t* d_ids, int batch, int seq_len, float* d_ppl) {
  auto* g = dynamic_cast<QuantGpt*>(m);
  if (!g) throw std::runtime_error("ppl: the model is not a QuantGpt");
  g->Ppl(d_ids, batch, seq_len, d_ppl);
}

}  // namespace ls100
