// QuantTransformer: int8 encoder-decoder with beam search, behind the LSModel interface.
//
// Replaces lightseq/inference/pywrapper/quant_transformer.cc + the QuantEncoder /
// QuantDecoder drivers (lightseq/inference/model/quant_encoder.cc.cu:219-460,
// quant_decoder.cc.cu:415-1098). Differences in structure, all to remove launch/sync
// latency from the decode loop:
//   * one decode step is captured once per (batch, src_len) into a CUDA graph and
//     replayed; the step index lives in device memory and is advanced by the beam kernel;
//   * no host sync inside a step (the reference does two); early stop is seen through a
//     mapped host word while a short ring of events keeps the host a few steps ahead;
//   * the self-attention KV cache is never permuted: attention follows a beam-ancestry table.
#include <math.h>
#include <stdlib.h>

#include <map>
#include <cstdlib>
#include <memory>

#include "engine_model.h"
#include "layers.h"

namespace ls100 {

class QuantTransformer : public EngineModel {
 public:
  QuantTransformer(const std::string& weight_path, int max_batch_size)
      : EngineModel({"source_ids"}, {"target_ids", "target_scores"}), max_bs_(max_batch_size) {
    WeightsFile wf(weight_path);
    H_ = (int)wf.conf("hidden");
    heads_ = (int)wf.conf("heads");
    F_ = (int)wf.conf("ffn");
    n_enc_ = (int)wf.conf("n_enc");
    n_dec_ = (int)wf.conf("n_dec");
    V_ = (int)wf.conf("vocab");
    beam_ = (int)wf.conf("beam");
    max_step_ = (int)wf.conf("max_step");
    pad_id_ = (int)wf.conf("pad_id");
    start_id_ = (int)wf.conf("start_id");
    end_id_ = (int)wf.conf("end_id");
    extra_len_ = (int)wf.conf("extra_decode_length");
    length_penalty_ = (float)wf.conf("length_penalty");
    const bool gelu = wf.conf_or("act_gelu", 0.0) != 0.0;
    const bool pre_ln = wf.conf_or("pre_ln", 1.0) != 0.0;
    // generator options (lightseq/inference/proto/quant_transformer.proto:140-149, quant_decoder.cc.cu:388-397)
    sampling_ = (int)wf.conf_or("sampling_method", 0.0);  // 0 beam_search, 1 topk, 2 topp, 3 topk_greedy
    topk_ = (int)wf.conf_or("topk", 1.0);
    topp_ = (float)wf.conf_or("topp", 0.0);
    seed_lo_ = (uint32_t)wf.conf_or("rng_seed", 0.0);
    output_topk_ = wf.conf_or("output_topk", 0.0) != 0.0 || sampling_ != 0;
    no_scale_embedding_ = wf.conf_or("no_scale_embedding", 0.0) != 0.0;
    if (sampling_ < 0 || sampling_ > 3) throw std::runtime_error("QuantTransformer: unknown sampling_method");
    diverse_lambda_ = sampling_ == 0 ? (float)wf.conf_or("diverse_lambda", 0.0) : 0.f;  // topk_greedy_search zeroes it
    if (sampling_ == 1 && (topk_ < 1 || topk_ > 8)) throw std::runtime_error("QuantTransformer: topk must be in [1, 8]");
    if (sampling_ == 2 && !(topp_ > 0.f && topp_ <= 1.f)) throw std::runtime_error("QuantTransformer: topp must be in (0, 1]");
    if (sampling_ == 1 || sampling_ == 2) beam_ = 1;  // one sampled sequence per sentence (pywrapper/quant_transformer.cc:35-37)
    if (H_ != heads_ * 64) throw std::runtime_error("QuantTransformer: head_dim must be 64");
    if (beam_ < 1 || beam_ > 8) throw std::runtime_error("QuantTransformer: beam size must be in [1, 8]");
    if (max_batch_size < 1) throw std::runtime_error("max_batch_size must be positive");
    ctx_ = Context::create(StatusType::Inference);
    Context& c = *ctx_;
    const int max_enc_tokens = max_bs_ * max_step_;
    const int max_rows = max_bs_ * beam_;

    // embedding table: int8 with the (shared) embedding clip-max; also the logits weight
    emb_.load(c, wf, "logits", false, true, true, "emb", "emb", false);
    amax_emb_ = wf.amax("emb");
    const HostTensor& pos = wf.tensor("pos");
    n_pos_ = (int)pos.dims[0];
    pos_ = upload_vec(c, wf, "pos", (int64_t)n_pos_ * H_);

    const std::string act = gelu ? "gelu" : "relu";
    for (int l = 0; l < n_enc_; ++l)
      enc_layers_.emplace_back(new QuantTransformerEncoderLayer(ctx_, wf, "enc." + std::to_string(l), l, max_enc_tokens,
                                                                max_step_, H_, heads_, F_, pre_ln, act));
    enc_ln_.load(c, wf, "enc.ln", H_);
    for (int l = 0; l < n_dec_; ++l)
      dec_layers_.emplace_back(new QuantTransformerDecoderLayer(ctx_, wf, "dec." + std::to_string(l), l, max_enc_tokens,
                                                                max_step_, H_, heads_, F_, pre_ln, act, max_bs_, beam_,
                                                                max_step_));
    dec_ln_.load(c, wf, "dec.ln", H_);
    pre_ln_ = pre_ln;
    if (!pre_ln_) {  // post-LN: every layer's closing LayerNorm quantises for the next consumer; no final LayerNorms
      for (int l = 0; l < n_enc_; ++l)
        enc_layers_[l]->set_next_input_amax(l + 1 < n_enc_ ? enc_layers_[l + 1]->qkv().amax_in : 0.f);
      for (int l = 0; l < n_dec_; ++l)
        dec_layers_[l]->set_next_input_amax(l + 1 < n_dec_ ? dec_layers_[l + 1]->qkv_input_amax() : emb_.amax_in);
    }
    if (H_ % 64 == 0 && getenv("LS100_PROJ_SIMT") == nullptr) {  // cross K/V projection on the tensor cores
      enc_x3_ = c.alloc((size_t)max_enc_tokens * 3 * H_ * 2);
      for (auto& l : dec_layers_) l->prepare_tensor_core_projection();
    }

    auto mk = [&](const char* n, size_t bytes) { vars_.emplace_back(new Variable(n, c, bytes)); return vars_.back().get(); };
    enc_.x = mk("enc.x", (size_t)max_enc_tokens * H_ * 4);
    enc_.a_q = mk("enc.a_q", (size_t)max_enc_tokens * H_);
    enc_.qkv_q = mk("enc.qkv_q", (size_t)max_enc_tokens * 3 * H_);
    enc_.attn_q = mk("enc.attn_q", (size_t)max_enc_tokens * H_);
    enc_.h_q = mk("enc.h_q", (size_t)max_enc_tokens * F_);
    enc_out_ = mk("enc.out", (size_t)max_enc_tokens * H_ * 4);
    pad_mask_ = mk("enc.pad_mask", (size_t)max_enc_tokens);
    dec_.x = mk("dec.x", (size_t)max_rows * H_ * 4);
    dec_.a_q = mk("dec.a_q", (size_t)max_rows * H_);
    dec_.qkv_q = mk("dec.qkv_q", (size_t)max_rows * 3 * H_);
    dec_.attn_q = mk("dec.attn_q", (size_t)max_rows * H_);
    dec_.h_q = mk("dec.h_q", (size_t)max_rows * F_);
    dec_.q_q = mk("dec.q_q", (size_t)max_rows * H_);
    ldv_ = (V_ + 15) / 16 * 16;
    logits_q_ = mk("dec.logits_q", (size_t)max_rows * ldv_);
    // Per (row, 64-column group) statistics of the logits, kept by the logits GEMM for the beam selection
    // (ls100_beam_select). Off unless LS100_FUSED_SELECT is set: measured on B200 at 512 rows x 32000 the statistics cost
    // the GEMM epilogue 8.4 us (18.1 -> 26.5 us: it is bound by instruction issue already) and the selection kernel,
    // 16 CTAs of dependent round trips, 46 us in place of the 23 us of ls100_beam_topk.
    n_groups_ = (V_ + 63) / 64;
    fused_select_ = getenv("LS100_FUSED_SELECT") != nullptr;
    {
      const size_t slots = (size_t)((max_rows + 127) / 128) * n_groups_ * 128;
      stat_max_ = c.alloc_n<int8_t>(slots);
      stat_sum_ = c.alloc_n<float>(slots);
    }

    alive_ = c.alloc_n<int32_t>((size_t)max_rows * max_step_);
    anc_ = c.alloc_n<int32_t>((size_t)max_rows * max_step_);
    seq_probs_ = c.alloc_n<float>(max_rows);
    seq_score_ = c.alloc_n<float>(max_rows);
    cand_score_ = c.alloc_n<float>((size_t)max_rows * beam_);
    cand_token_ = c.alloc_n<int32_t>((size_t)max_rows * beam_);
    counters_ = c.alloc_n<int32_t>(2 * max_step_ + 4);  // [step, stop, fin[max_step], ticket[max_step], 2 for sampling]
    step_ptr_ = counters_;
    stop_ptr_ = counters_ + 1;
    fin_ptr_ = counters_ + 2;
    ticket_ptr_ = counters_ + 2 + max_step_;
    sample_ticket_ = counters_ + 2 + 2 * max_step_;
    sample_ended_ = sample_ticket_ + 1;
    stop_host_ = static_cast<int32_t*>(c.alloc_host_mapped(sizeof(int32_t)));
    LS_CUDA(cudaHostGetDevicePointer((void**)&stop_host_dev_, stop_host_, 0));

    // length-norm table, entry s = norm of length s+1 (lightseq/inference/kernels/transformerKernels.h:137-140)
    std::vector<float> ln(max_step_);
    for (int i = 0; i < max_step_; ++i) {
      const int len = i + 1;
      ln[i] = length_penalty_ < 0.f ? 1.f / len : powf((5.f + len) / 6.f, -length_penalty_);
    }
    length_norm_ = c.alloc_n<float>(max_step_);
    LS_CUDA(cudaMemcpy(length_norm_, ln.data(), max_step_ * sizeof(float), cudaMemcpyHostToDevice));

    // host templates of the per-request initial state
    h_alive_.assign((size_t)max_rows * max_step_, end_id_);
    for (int r = 0; r < max_rows; ++r) h_alive_[(size_t)r * max_step_] = start_id_;
    h_probs_.assign(max_rows, -1000.f);  // min_log_probability / 2 (quant_decoder.cc.cu:57-66)
    for (int r = 0; r < max_rows; r += beam_) h_probs_[r] = 0.f;
    h_counters_.assign(2 * max_step_ + 4, 0);
    h_counters_[1] = -1;
    if (sampling_ != 0) {  // rows keep their own cache slots once they are sampled independently
      h_anc_.resize((size_t)max_rows * max_step_);
      for (int r = 0; r < max_rows; ++r)
        for (int p = 0; p < max_step_; ++p) h_anc_[(size_t)r * max_step_ + p] = r;
      LS_CUDA(cudaHostRegister(h_anc_.data(), h_anc_.size() * 4, cudaHostRegisterDefault));
    }
    LS_CUDA(cudaHostRegister(h_alive_.data(), h_alive_.size() * 4, cudaHostRegisterDefault));
    LS_CUDA(cudaHostRegister(h_probs_.data(), h_probs_.size() * 4, cudaHostRegisterDefault));
    LS_CUDA(cudaHostRegister(h_counters_.data(), h_counters_.size() * 4, cudaHostRegisterDefault));
    for (auto& e : ring_) LS_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    use_graph_ = getenv("LS100_NO_GRAPH") == nullptr;
    for (auto& l : dec_layers_) l->set_history_static(use_graph_);  // a decode step is then one graph launch
  }

  ~QuantTransformer() override {
    cudaSetDevice(ctx_->device());
    cudaStreamSynchronize(ctx_->get_stream());
    for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second);
    for (auto& e : ring_) cudaEventDestroy(e);
    cudaHostUnregister(h_alive_.data());
    cudaHostUnregister(h_probs_.data());
    cudaHostUnregister(h_counters_.data());
    if (!h_anc_.empty()) cudaHostUnregister(h_anc_.data());
  }

  void Infer() override {
    if (input_shapes_[0].size() != 2) throw std::runtime_error("source_ids must be [batch, seq_len]");
    const int B = input_shapes_[0][0], S = input_shapes_[0][1];
    if (B > max_bs_) throw std::runtime_error("batch size of input greater than max_batch_size");
    if (S > max_step_) throw std::runtime_error("seq len of input greater than max_step");
    if (B < 1 || S < 1) throw std::runtime_error("empty input");
    if (!d_src_ || !d_out_ids_ || !d_out_scores_) throw std::runtime_error("input/output pointers not set");
    LS_CUDA(cudaSetDevice(ctx_->device()));
    cudaStream_t st = ctx_->get_stream();
    run_encoder(B, S);
    if (enc_x3_)  // one split of the encoder output serves the 2 x n_dec projections
      LS_RC(ls100_split_bf16x3(ctx_->kernels(), enc_out_->value<float>(), H_, B * S, H_, enc_x3_, st));
    for (auto& l : dec_layers_) {
      l->before_forward(B, beam_, S);
      l->project_encoder_output(enc_out_->value<float>(), enc_x3_);
    }
    const int rows = B * beam_;
    LS_CUDA(cudaMemcpyAsync(alive_, h_alive_.data(), (size_t)rows * max_step_ * 4, cudaMemcpyHostToDevice, st));
    LS_CUDA(cudaMemcpyAsync(seq_probs_, h_probs_.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, st));
    LS_CUDA(cudaMemcpyAsync(counters_, h_counters_.data(), h_counters_.size() * 4, cudaMemcpyHostToDevice, st));
    LS_CUDA(cudaMemsetAsync(seq_score_, 0, (size_t)rows * 4, st));
    if (sampling_ != 0) LS_CUDA(cudaMemcpyAsync(anc_, h_anc_.data(), (size_t)rows * max_step_ * 4, cudaMemcpyHostToDevice, st));
    else LS_CUDA(cudaMemsetAsync(anc_, 0, (size_t)rows * max_step_ * 4, st));
    *stop_host_ = -1;

    // _batch_max_decode_length of the reference (quant_decoder.cc.cu:428-436): sampling runs to max_step
    const int max_decode = sampling_ != 0 ? max_step_ : std::min(max_step_, S + extra_len_) - 1;
    int n_steps = std::max(max_decode - 1, 0);
    if (debug_step_limit_ >= 0) n_steps = std::min(n_steps, debug_step_limit_);
    int launched = 0;
    for (int s = 0; s < n_steps; ++s) {
      if (s >= kRing) {
        LS_CUDA(cudaEventSynchronize(ring_[s % kRing]));
        if (!benchmark_ && *((volatile int32_t*)stop_host_) >= 0) break;
      }
      const bool beam_step = sampling_ == 0 || (sampling_ == 3 && s == 0);  // topk_greedy: a beam step, then greedy rows
      if (use_graph_) LS_CUDA(cudaGraphLaunch(decode_graph(B, S, beam_step), st));
      else decode_step(B, S, beam_step);
      LS_CUDA(cudaEventRecord(ring_[s % kRing], st));
      ++launched;
    }
    int32_t h_stop = -1;
    LS_CUDA(cudaMemcpyAsync(&h_stop, stop_ptr_, 4, cudaMemcpyDeviceToHost, st));
    LS_CUDA(cudaStreamSynchronize(st));
    const int err = ls100_ctx_poll_error(ctx_->kernels(), st);
    if (err != 0) throw std::runtime_error(std::string("device reported: ") + ls100_strerror(err));
    // the beam kernels report the step at which every beam had finished, the sampling kernels the position written then
    const bool stopped_in_sampling = sampling_ == 1 || sampling_ == 2 || (sampling_ == 3 && launched > 1);
    int cur_step;
    if (!benchmark_ && h_stop >= 0) cur_step = stopped_in_sampling ? h_stop - 1 : h_stop;
    else cur_step = std::max(max_decode - 1, 0);
    const int n_out = std::min(cur_step + 1, max_step_ - 1);
    // what the reference writes out (quant_decoder.cc.cu:456-478): every beam when the model outputs its top k or
    // samples; else beam 0, or, for a negative length penalty, the beam with the best score per token
    ls100_beam_result_args r;
    memset(&r, 0, sizeof(r));
    r.alive = alive_;
    r.seq_score = seq_score_;
    r.batch = B;
    r.beam = beam_;
    r.max_step = max_step_;
    r.end_id = end_id_;
    r.n_out = n_out;
    r.mode = output_topk_ ? 2 : (length_penalty_ < 0.f ? 1 : 0);
    r.out_tokens = d_out_ids_;
    r.out_scores = d_out_scores_;
    LS_RC(ls100_beam_write_result(ctx_->kernels(), &r, st));
    LS_CUDA(cudaStreamSynchronize(st));
    const int out_k = output_topk_ ? beam_ : 1;
    set_output_shape(0, {B, out_k, n_out});
    set_output_shape(1, {B, out_k});
    steps_run_ = launched;
  }

  void set_input_ptr(int index, void* p) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    d_src_ = static_cast<const int32_t*>(p);
  }
  void set_output_ptr(int index, void* p) override {
    if (index == 0) d_out_ids_ = static_cast<int32_t*>(p);
    else if (index == 1) d_out_scores_ = static_cast<float*>(p);
    else throw std::runtime_error("invalid output index");
  }
  const void* get_output_ptr(int index) override {
    if (index == 0) return d_out_ids_;
    if (index == 1) return d_out_scores_;
    throw std::runtime_error("invalid output index");
  }
  std::vector<int> get_input_max_shape(int index) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    return {max_bs_, max_step_};
  }
  std::vector<int> get_output_max_shape(int index) override {
    if (index == 0) return {max_bs_, beam_, max_step_};
    if (index == 1) return {max_bs_, beam_};
    throw std::runtime_error("invalid output index");
  }
  DataType get_input_dtype(int index) override {
    if (index != 0) throw std::runtime_error("invalid input index");
    return kInt32;
  }
  DataType get_output_dtype(int index) override {
    if (index == 0) return kInt32;
    if (index == 1) return kFloat32;
    throw std::runtime_error("invalid output index");
  }
  void benchmark_mode(bool b) override { benchmark_ = b; }

  // Debug taps used by the parity tests (device pointers valid until the next Infer()).
  const float* encoder_output() const { return enc_out_->value<float>(); }
  const int8_t* last_logits() const { return logits_q_->value<int8_t>(); }
  int logits_ld() const { return ldv_; }
  int steps_run() const { return steps_run_; }
  void set_debug_step_limit(int n) { debug_step_limit_ = n; }
  // beam state after the last Infer(): alive [rows, max_step], anc [rows, max_step], probs/score [rows]
  void beam_state(const int32_t** alive, const int32_t** anc, const float** probs, const float** score, int* max_step,
                  int* beam) const {
    *alive = alive_;
    *anc = anc_;
    *probs = seq_probs_;
    *score = seq_score_;
    *max_step = max_step_;
    *beam = beam_;
  }
  ContextPtr context() const override { return ctx_; }

 private:
  static constexpr int kRing = 4;

  void run_encoder(int B, int S) {
    ls100_embed_args e;
    memset(&e, 0, sizeof(e));
    e.ids = d_src_;
    e.ld_ids = S;
    e.batch = B;
    e.seq = S;
    e.hidden = H_;
    e.table_q = emb_.w;
    e.s_emb = emb_.s_w;
    e.sqrt_h = no_scale_embedding_ ? 1.0f : sqrtf((float)H_);
    e.pos = pos_;
    e.n_pos = n_pos_;
    e.pad_id = pad_id_;
    e.vocab = V_;
    e.out = enc_.x->value<float>();
    e.pad_mask = pad_mask_->value<uint8_t>();
    LS_RC(ls100_embed(ctx_->kernels(), &e, ctx_->get_stream()));
    tap_reset();
    tap(enc_.x->value<float>(), (size_t)B * S * H_, ctx_->get_stream());
    if (!pre_ln_ && !enc_layers_.empty())  // post-LN: the first layer reads the embedding already quantised
      LS_RC(ls100_quantize_weight(ctx_->kernels(), enc_.x->value<float>(), (int64_t)B * S, H_, enc_layers_[0]->qkv().amax_in,
                                  enc_.a_q->value<int8_t>(), nullptr, ctx_->get_stream()));
    for (auto& l : enc_layers_) {
      (*l)(&enc_, pad_mask_);
      l->before_forward(B, S);
      l->forward();
      tap(enc_.x->value<float>(), (size_t)B * S * H_, ctx_->get_stream());
    }
    if (!pre_ln_) {  // the last layer's own LayerNorm closed the stack
      LS_CUDA(cudaMemcpyAsync(enc_out_->value<float>(), enc_.x->value<float>(), (size_t)B * S * H_ * 4, cudaMemcpyDeviceToDevice,
                              ctx_->get_stream()));
      return;
    }
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = enc_.x->value<float>();
    a.ldx = H_;
    a.gamma = enc_ln_.g;
    a.beta = enc_ln_.b;
    a.rows = B * S;
    a.hidden = H_;
    a.out_f = enc_out_->value<float>();
    a.ldf = H_;
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, ctx_->get_stream()));
  }

  void decode_step(int B, int S, bool beam_step) {
    const int rows = B * beam_;
    ls100_ctx* k = ctx_->kernels();
    cudaStream_t st = ctx_->get_stream();
    ls100_embed_args e;
    memset(&e, 0, sizeof(e));
    e.ids = alive_;
    e.ld_ids = max_step_;
    e.batch = rows;
    e.seq = 1;
    e.hidden = H_;
    e.step_ptr = step_ptr_;
    e.table_q = emb_.w;
    e.s_emb = emb_.s_w;
    e.sqrt_h = no_scale_embedding_ ? 1.0f : sqrtf((float)H_);
    e.pos = pos_;
    e.n_pos = n_pos_;
    e.pad_id = pad_id_;
    e.vocab = V_;
    e.out = dec_.x->value<float>();
    // the lookup runs inside the first layer's LayerNorm launch (one kernel less per step) unless switched off
    static const bool separate_embed = getenv("LS100_NO_EMBED_FUSE") != nullptr;
    const bool fused = pre_ln_ && !separate_embed && rows <= 2048 && !dec_layers_.empty();
    if (!fused) LS_RC(ls100_embed(k, &e, st));
    if (!pre_ln_ && !dec_layers_.empty())  // post-LN: the first layer reads the embedding already quantised
      LS_RC(ls100_quantize_weight(k, dec_.x->value<float>(), rows, H_, dec_layers_[0]->qkv_input_amax(), dec_.a_q->value<int8_t>(),
                                  nullptr, st));
    if (!dec_layers_.empty()) dec_layers_[0]->set_embed_source(fused ? &e : nullptr);
    for (auto& l : dec_layers_) {
      (*l)(&dec_, pad_mask_, anc_, step_ptr_);
      l->before_forward(B, beam_, S);
      l->forward();
    }
    if (!dec_layers_.empty()) dec_layers_[0]->set_embed_source(nullptr);  // `e` goes out of scope with this call
    if (pre_ln_) {  // post-LN: the last layer's closing LayerNorm already wrote the int8 input of the output projection
      ls100_ln_quant_args a;
      memset(&a, 0, sizeof(a));
      a.x = dec_.x->value<float>();
      a.ldx = H_;
      a.gamma = dec_ln_.g;
      a.beta = dec_ln_.b;
      a.rows = rows;
      a.hidden = H_;
      a.amax = emb_.amax_in;
      a.out_q = dec_.a_q->value<int8_t>();
      a.ldq = H_;
      LS_RC(ls100_ln_quant(k, &a, st));
    }
    QuantLinearOp logits(ctx_, "logits", &emb_, LS100_OUT_OUTQ_I8, Act::None, true, false);
    logits(dec_.a_q, logits_q_);
    logits.before_forward(rows, ldv_);
    if (beam_step && fused_select_) logits.keep_statistics(stat_max_, stat_sum_);
    logits.forward();
    if (!beam_step) {  // QuantDecoder::sample / topk_greedy_search (quant_decoder.cc.cu:951-985, 1101-1133)
      sample_step(rows);
      return;
    }
    ls100_beam_topk_args t;
    memset(&t, 0, sizeof(t));
    t.logits = logits_q_->value<int8_t>();
    t.ld_logits = ldv_;
    t.s_logits = emb_.s_out;
    t.batch = B;
    t.beam = beam_;
    t.vocab = V_;
    t.max_step = max_step_;
    t.end_id = end_id_;
    t.step_ptr = step_ptr_;
    t.length_norm = length_norm_;
    t.alive = alive_;
    t.seq_probs = seq_probs_;
    t.seq_score = seq_score_;
    t.cand_score = cand_score_;
    t.cand_token = cand_token_;
    t.diverse_lambda = diverse_lambda_;
    if (fused_select_) {  // candidates from the statistics: the logits are not read again, except a few groups per row
      ls100_beam_select_args sel;
      memset(&sel, 0, sizeof(sel));
      sel.topk = t;
      sel.stat_max = stat_max_;
      sel.stat_sum = stat_sum_;
      sel.n_groups = n_groups_;
      LS_RC(ls100_beam_select(k, &sel, st));
    } else {
      LS_RC(ls100_beam_topk(k, &t, st));
    }
    ls100_beam_update_args u;
    memset(&u, 0, sizeof(u));
    u.cand_score = cand_score_;
    u.cand_token = cand_token_;
    u.batch = B;
    u.beam = beam_;
    u.max_step = max_step_;
    u.end_id = end_id_;
    u.step_ptr = step_ptr_;
    u.length_norm = length_norm_;
    u.alive = alive_;
    u.anc = anc_;
    u.seq_probs = seq_probs_;
    u.seq_score = seq_score_;
    u.fin_count = fin_ptr_;
    u.ticket = ticket_ptr_;
    u.stop_step = stop_ptr_;
    u.stop_host = stop_host_dev_;
    u.diverse_lambda = diverse_lambda_;
    LS_RC(ls100_beam_update(k, &u, st));
  }

  // one new token per row, each row on its own: top-k (k = 1 for topk_greedy) or nucleus sampling, Philox keyed by
  // (seed; position, row); EOS bookkeeping and the stop word stay on the device
  void sample_step(int rows) {
    ls100_ctx* k = ctx_->kernels();
    cudaStream_t st = ctx_->get_stream();
    if (sampling_ == 2) {
      ls100_sample_topp_args s;
      memset(&s, 0, sizeof(s));
      s.logits = logits_q_->value<int8_t>();
      s.ld_logits = ldv_;
      s.s_logits = emb_.s_out;
      s.p = topp_;
      s.rows = rows;
      s.vocab = V_;
      s.max_step = max_step_;
      s.end_id = end_id_;
      s.seed_lo = seed_lo_;
      s.seed_hi = 0;
      s.seq = alive_;
      s.cur = step_ptr_;
      s.ticket = sample_ticket_;
      s.n_ended = sample_ended_;
      s.stop = stop_ptr_;
      s.stop_host = stop_host_dev_;
      LS_RC(ls100_sample_topp(k, &s, st));
      return;
    }
    ls100_sample_topk_args s;
    memset(&s, 0, sizeof(s));
    s.logits = logits_q_->value<int8_t>();
    s.ld_logits = ldv_;
    s.s_logits = emb_.s_out;
    s.rows = rows;
    s.vocab = V_;
    s.k = sampling_ == 3 ? 1 : topk_;
    s.max_step = max_step_;
    s.end_id = end_id_;
    s.seed_lo = seed_lo_;
    s.seed_hi = 0;
    s.seq = alive_;
    s.cur = step_ptr_;
    s.ticket = sample_ticket_;
    s.n_ended = sample_ended_;
    s.stop = stop_ptr_;
    s.stop_host = stop_host_dev_;
    LS_RC(ls100_sample_topk(k, &s, st));
  }

  cudaGraphExec_t decode_graph(int B, int S, bool beam_step) {
    const long long key = ((long long)B * 100000 + S) * 2 + (beam_step ? 1 : 0);
    auto it = graphs_.find(key);
    if (it != graphs_.end()) return it->second;
    cudaStream_t st = ctx_->get_stream();
    cudaGraph_t g = nullptr;
    LS_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    try {
      decode_step(B, S, beam_step);
    } catch (...) {
      cudaStreamEndCapture(st, &g);
      if (g) cudaGraphDestroy(g);
      throw;
    }
    LS_CUDA(cudaStreamEndCapture(st, &g));
    cudaGraphExec_t exec = nullptr;
    LS_CUDA(cudaGraphInstantiate(&exec, g, 0));
    cudaGraphDestroy(g);
    if (graphs_.size() >= 64) {
      for (auto& kv : graphs_) cudaGraphExecDestroy(kv.second);
      graphs_.clear();
    }
    graphs_[key] = exec;
    return exec;
  }

  int max_bs_, H_ = 0, heads_ = 0, F_ = 0, n_enc_ = 0, n_dec_ = 0, V_ = 0, beam_ = 0, max_step_ = 0;
  int pad_id_ = 0, start_id_ = 0, end_id_ = 0, extra_len_ = 0, n_pos_ = 0, ldv_ = 0;
  float length_penalty_ = 0.f, amax_emb_ = 0.f;
  ContextPtr ctx_;
  QLinearParams emb_;  // table [V,H] int8 = embedding and logits weight; in/out = logits clip-max
  float* pos_ = nullptr;
  std::vector<std::unique_ptr<QuantTransformerEncoderLayer>> enc_layers_;
  std::vector<std::unique_ptr<QuantTransformerDecoderLayer>> dec_layers_;
  LayerNormParams enc_ln_, dec_ln_;
  std::vector<std::unique_ptr<Variable>> vars_;
  StackBuffers enc_, dec_;
  Variable *enc_out_ = nullptr, *pad_mask_ = nullptr, *logits_q_ = nullptr;
  int32_t *alive_ = nullptr, *anc_ = nullptr, *cand_token_ = nullptr, *counters_ = nullptr;
  int32_t *step_ptr_ = nullptr, *stop_ptr_ = nullptr, *fin_ptr_ = nullptr, *ticket_ptr_ = nullptr;
  int32_t *stop_host_ = nullptr, *stop_host_dev_ = nullptr, *sample_ticket_ = nullptr, *sample_ended_ = nullptr;
  int sampling_ = 0, topk_ = 1;
  float topp_ = 0.f, diverse_lambda_ = 0.f;
  uint32_t seed_lo_ = 0;
  bool output_topk_ = false, no_scale_embedding_ = false, pre_ln_ = true, fused_select_ = true;
  int n_groups_ = 0;
  int8_t* stat_max_ = nullptr;
  float* stat_sum_ = nullptr;
  std::vector<int32_t> h_anc_;
  float *seq_probs_ = nullptr, *seq_score_ = nullptr, *cand_score_ = nullptr, *length_norm_ = nullptr;
  std::vector<int32_t> h_alive_, h_counters_;
  std::vector<float> h_probs_;
  cudaEvent_t ring_[kRing];
  std::map<long long, cudaGraphExec_t> graphs_;
  bool use_graph_ = true, benchmark_ = false;
  void* enc_x3_ = nullptr;
  const int32_t* d_src_ = nullptr;
  int32_t* d_out_ids_ = nullptr;
  float* d_out_scores_ = nullptr;
  int steps_run_ = 0;
  int debug_step_limit_ = -1;
};

LSMODEL_REGISTER(QuantTransformer)

cudaStream_t model_stream(LSModel* m) {
  if (auto* t = dynamic_cast<EngineModel*>(m)) return t->context()->get_stream();
  return nullptr;
}

// Accessors for the test-only debug taps declared in model_abi.cpp.
const float* quant_transformer_encoder_output(LSModel* m) {
  auto* t = dynamic_cast<QuantTransformer*>(m);
  return t ? t->encoder_output() : nullptr;
}
const int8_t* quant_transformer_last_logits(LSModel* m, int* ld) {
  auto* t = dynamic_cast<QuantTransformer*>(m);
  if (!t) return nullptr;
  if (ld) *ld = t->logits_ld();
  return t->last_logits();
}
int quant_transformer_set_step_limit(LSModel* m, int n) {
  auto* t = dynamic_cast<QuantTransformer*>(m);
  if (!t) return -1;
  t->set_debug_step_limit(n);
  return 0;
}
int quant_transformer_beam_state(LSModel* m, const int32_t** alive, const int32_t** anc, const float** probs,
                                 const float** score, int* max_step, int* beam) {
  auto* t = dynamic_cast<QuantTransformer*>(m);
  if (!t) return -1;
  t->beam_state(alive, anc, probs, score, max_step, beam);
  return 0;
}
int quant_transformer_steps_run(LSModel* m) {
  auto* t = dynamic_cast<QuantTransformer*>(m);
  return t ? t->steps_run() : -1;
}

}  // namespace ls100
