// Operators of the int8 inference graph. Each mirrors the interface shape of an operator
// in the reference's lightseq/csrc/ops_new (constructor with maxima, `operator()` wiring
// Variables, `before_forward(...)` with the per-call sizes, `forward()` launching on the
// Context stream) and launches one ls100_* kernel family.
#pragma once
#include <math.h>

#include "lsflow.h"
#include "weights_file.h"

namespace ls100 {

enum class Act { None = LS100_ACT_NONE, Relu = LS100_ACT_RELU, Gelu = LS100_ACT_GELU };

// Device-resident parameters of one QuantLinear
// (lightseq/training/ops/pytorch/quantization.py:33-61): int8 weight [N,K], fp32 bias,
// clip-max of input / weight / output, and 127*rowsum(Wq) when the input quantiser is
// the unsigned post-ReLU one.
struct QLinearParams {
  int n = 0, k = 0;
  int8_t* w = nullptr;
  float* bias = nullptr;
  int32_t* w_off = nullptr;
  float amax_in = 0, amax_w = 0, amax_out = 0;
  float s_in = 0, s_w = 0, s_out = 0, s_acc = 0;
  bool unsigned_in = false;
  // Optional table of bias + activation + requantisation per (column, quantised output value), see
  // ls100_gemm_i8_args::req_table, and the epilogue it was built for
  uint8_t* req_table = nullptr;
  int tab_out_kind = -1, tab_act = -1;
  bool tab_bias = false;
  float tab_s_req = 0.f;

  void build_table(Context& ctx, int out_kind, int act, bool add_bias, float s_req) {
    if (!(s_out > 0.f) || !(s_req > 0.f)) return;
    ls100_gemm_i8_args a;
    memset(&a, 0, sizeof(a));
    a.n = n;
    a.s_outq = s_out;
    a.bias = add_bias ? bias : nullptr;
    a.act = act;
    a.out_kind = out_kind;
    a.s_req = s_req;
    req_table = ctx.alloc_n<uint8_t>(ls100_gemm_i8_table_bytes(n));
    LS_RC(ls100_gemm_i8_build_table(ctx.kernels(), &a, req_table, ctx.get_stream()));
    LS_CUDA(cudaStreamSynchronize(ctx.get_stream()));
    tab_out_kind = out_kind;
    tab_act = act;
    tab_bias = add_bias;
    tab_s_req = s_req;
  }
  const uint8_t* table_for(int out_kind, int act, bool out_quant, bool add_bias, float s_req, bool has_resid) const {
    return (req_table && out_quant && !has_resid && out_kind == tab_out_kind && act == tab_act && add_bias == tab_bias &&
            s_req == tab_s_req)
               ? req_table
               : nullptr;
  }

  // Uploads W (fp32), quantises it on the device (ls100_quantize_weight) and frees the staging copy.
  void load(Context& ctx, const WeightsFile& wf, const std::string& name, bool unsigned_in_, bool has_in = true,
            bool has_out = true, const std::string& wname = "", const std::string& w_amax = "", bool has_bias = true,
            bool out_optional = false) {
    const std::string wn = wname.empty() ? name + ".w" : wname;
    const HostTensor& W = wf.tensor(wn);
    if (W.dims.size() != 2) throw std::runtime_error(wn + ": expected a matrix");
    n = (int)W.dims[0];
    k = (int)W.dims[1];
    unsigned_in = unsigned_in_;
    amax_w = wf.amax(w_amax.empty() ? name + ".w" : w_amax);
    s_w = amax_w / 127.0f;
    if (has_in) {
      amax_in = wf.amax(name + ".in");
      s_in = unsigned_in ? amax_in / 254.0f : amax_in / 127.0f;
      s_acc = s_in * s_w;
    }
    if (has_out) {
      // out_optional: 0 = the output stays unquantised (s_out 0 switches the epilogue's output quantiser off)
      amax_out = out_optional ? wf.amax_or_unquantised(name + ".out") : wf.amax(name + ".out");
      s_out = amax_out / 127.0f;
    }
    float* staging = nullptr;
    LS_CUDA(cudaMalloc(&staging, (size_t)n * k * sizeof(float)));
    LS_CUDA(cudaMemcpyAsync(staging, W.data, (size_t)n * k * sizeof(float), cudaMemcpyHostToDevice, ctx.get_stream()));
    w = ctx.alloc_n<int8_t>((size_t)n * k);
    if (unsigned_in) w_off = ctx.alloc_n<int32_t>(n);
    LS_RC(ls100_quantize_weight(ctx.kernels(), staging, n, k, amax_w, w, w_off, ctx.get_stream()));
    LS_CUDA(cudaStreamSynchronize(ctx.get_stream()));
    LS_CUDA(cudaFree(staging));
    if (has_bias) {
      const HostTensor& B = wf.tensor(name + ".b");
      if (B.numel() != n) throw std::runtime_error(name + ".b: size mismatch");
      bias = ctx.alloc_n<float>(n);
      LS_CUDA(cudaMemcpy(bias, B.data, n * sizeof(float), cudaMemcpyHostToDevice));
    }
  }
};

inline float* upload_vec(Context& ctx, const WeightsFile& wf, const std::string& name, int64_t expect) {
  const HostTensor& t = wf.tensor(name);
  if (t.numel() != expect) throw std::runtime_error(name + ": size mismatch");
  float* d = ctx.alloc_n<float>((size_t)expect);
  LS_CUDA(cudaMemcpy(d, t.data, (size_t)expect * sizeof(float), cudaMemcpyHostToDevice));
  return d;
}

// int8 GEMM + fused epilogue. Counterpart of LinearOp (lightseq/csrc/ops_new/linear.cpp:5-45)
// for the quantised path.
class QuantLinearOp : public Operator {
 public:
  QuantLinearOp(ContextPtr ctx, std::string name, const QLinearParams* p, int out_kind, Act act = Act::None,
                bool out_quant = true, bool add_bias = true, float s_req = 0.f)
      : Operator(std::move(name), std::move(ctx)), p_(p), out_kind_(out_kind), act_(act), out_quant_(out_quant),
        add_bias_(add_bias), s_req_(s_req) {}
  Variable* operator()(Variable* inp, Variable* out, Variable* resid = nullptr) {
    in_ = inp;
    out_ = out;
    resid_ = resid;
    return out;
  }
  // LayerNorm + quantise of the finished fp32 rows in the same launch (the next sublayer's input quantiser)
  void fuse_layer_norm(const float* gamma, const float* beta, float amax, Variable* out_q) {
    ln_g_ = gamma;
    ln_b_ = beta;
    ln_amax_ = amax;
    ln_out_ = out_q;
  }
  void before_forward(int rows, int64_t ldo = 0) {
    rows_ = rows;
    ldo_ = ldo ? ldo : p_->n;
  }
  // per-row group statistics of an int8 output (see ls100_gemm_i8_args::stat_max): the logits of a beam-search step
  void keep_statistics(int8_t* stat_max, float* stat_sum) {
    stat_max_ = stat_max;
    stat_sum_ = stat_sum;
  }
  void forward() override {
    ls100_gemm_i8_args a;
    memset(&a, 0, sizeof(a));
    a.a = in_->value<int8_t>();
    a.lda = p_->k;
    a.w = p_->w;
    a.ldw = p_->k;
    a.m = rows_;
    a.n = p_->n;
    a.k = p_->k;
    a.s_acc = p_->s_acc;
    a.w_off = p_->w_off;
    a.s_outq = out_quant_ ? p_->s_out : 0.f;
    a.bias = add_bias_ ? p_->bias : nullptr;
    a.act = (int)act_;
    a.resid = resid_ ? resid_->value<float>() : nullptr;
    a.ldr = p_->n;
    a.out_kind = out_kind_;
    a.s_req = s_req_;
    a.out = out_->value<void>();
    a.ldo = ldo_;
    if (ln_out_) {
      a.ln_gamma = ln_g_;
      a.ln_beta = ln_b_;
      a.ln_amax = ln_amax_;
      a.ln_out = ln_out_->value<int8_t>();
      a.ln_ldq = p_->n;
    }
    a.stat_max = stat_max_;
    a.stat_sum = stat_sum_;
    if (!ln_out_ && !stat_max_) a.req_table = p_->table_for(out_kind_, (int)act_, out_quant_, add_bias_, s_req_, resid_ != nullptr);
    LS_RC(ls100_gemm_i8(ctx_->kernels(), &a, ctx_->get_stream()));
  }

 private:
  const QLinearParams* p_;
  int out_kind_;
  Act act_;
  bool out_quant_, add_bias_;
  float s_req_;
  Variable *in_ = nullptr, *out_ = nullptr, *resid_ = nullptr, *ln_out_ = nullptr;
  const float *ln_g_ = nullptr, *ln_b_ = nullptr;
  float ln_amax_ = 0.f;
  int8_t* stat_max_ = nullptr;
  float* stat_sum_ = nullptr;
  int rows_ = 0;
  int64_t ldo_ = 0;
};

// LayerNorm (+ quantise for the next QuantLinear). Counterpart of LayerNormalizeOp
// (lightseq/csrc/ops_new/layer_normalize.cpp).
class LayerNormQuantOp : public Operator {
 public:
  LayerNormQuantOp(ContextPtr ctx, std::string name, int hidden, const float* gamma, const float* beta, float amax)
      : Operator(std::move(name), std::move(ctx)), hidden_(hidden), gamma_(gamma), beta_(beta), amax_(amax) {}
  void operator()(Variable* inp, Variable* out_q, Variable* out_f = nullptr) {
    in_ = inp;
    out_q_ = out_q;
    out_f_ = out_f;
  }
  void before_forward(int rows) { rows_ = rows; }
  void forward() override {
    ls100_ln_quant_args a;
    memset(&a, 0, sizeof(a));
    a.x = in_->value<float>();
    a.ldx = hidden_;
    a.gamma = gamma_;
    a.beta = beta_;
    a.rows = rows_;
    a.hidden = hidden_;
    a.amax = amax_;
    a.out_q = out_q_ ? out_q_->value<int8_t>() : nullptr;
    a.ldq = hidden_;
    a.out_f = out_f_ ? out_f_->value<float>() : nullptr;
    a.ldf = hidden_;
    LS_RC(ls100_ln_quant(ctx_->kernels(), &a, ctx_->get_stream()));
  }

 private:
  int hidden_;
  const float *gamma_, *beta_;
  float amax_;
  Variable *in_ = nullptr, *out_q_ = nullptr, *out_f_ = nullptr;
  int rows_ = 0;
};

}  // namespace ls100
