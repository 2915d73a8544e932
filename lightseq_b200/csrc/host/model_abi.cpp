// C ABI over LSModel / LSModelFactory (see include/ls100.h, "model level").
#include <cuda_runtime.h>
#include <string.h>

#include <memory>
#include <string>

#include "../../../include/ls100.h"
#include "lsflow.h"
#include "engine_model.h"
#include "model_base.h"

namespace ls100 {
cudaStream_t model_stream(LSModel* m);
void quant_gpt_ppl(LSModel* m, const int32_t* d_ids, int batch, int seq_len, float* d_ppl);
const float* quant_transformer_encoder_output(LSModel* m);
const int8_t* quant_transformer_last_logits(LSModel* m, int* ld);
int quant_transformer_steps_run(LSModel* m);
int quant_transformer_set_step_limit(LSModel* m, int n);
int quant_transformer_beam_state(LSModel* m, const int32_t** alive, const int32_t** anc, const float** probs,
                                 const float** score, int* max_step, int* beam);
}  // namespace ls100

struct ls100_model {
  std::unique_ptr<ls100::LSModel> model;
  // staging buffers of the *_host entry points
  void* d_in = nullptr;
  void* d_out0 = nullptr;
  void* d_out1 = nullptr;
  size_t in_bytes = 0, out0_bytes = 0, out1_bytes = 0;
  int device = 0;
};

static thread_local std::string g_last_error;

template <typename F>
static int guarded(F&& f) {
  try {
    f();
    return LS100_OK;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return LS100_ERR_BAD_ARG;
  } catch (...) {
    g_last_error = "unknown error";
    return LS100_ERR_BAD_ARG;
  }
}

static size_t prod(const std::vector<int>& v) {
  size_t n = 1;
  for (int d : v) n *= (size_t)d;
  return n;
}

extern "C" const char* ls100_model_last_error(void) { return g_last_error.c_str(); }

extern "C" int ls100_model_create(const char* name, const char* path, int max_bs, ls100_model** out) {
  if (!name || !path || !out) return LS100_ERR_BAD_ARG;
  *out = nullptr;
  return guarded([&] {
    std::unique_ptr<ls100_model> h(new ls100_model());
    LS_CUDA(cudaGetDevice(&h->device));
    h->model.reset(ls100::LSModelFactory::GetInstance().CreateModel(name, path, max_bs));
    ls100::LSModel& m = *h->model;
    h->in_bytes = prod(m.get_input_max_shape(0)) * 4;
    LS_CUDA(cudaMalloc(&h->d_in, h->in_bytes));
    h->out0_bytes = prod(m.get_output_max_shape(0)) * 4;
    LS_CUDA(cudaMalloc(&h->d_out0, h->out0_bytes));
    if (m.get_output_size() > 1) {
      h->out1_bytes = prod(m.get_output_max_shape(1)) * 4;
      LS_CUDA(cudaMalloc(&h->d_out1, h->out1_bytes));
    }
    *out = h.release();
  });
}

extern "C" void ls100_model_destroy(ls100_model* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  m->model.reset();
  cudaFree(m->d_in);
  cudaFree(m->d_out0);
  cudaFree(m->d_out1);
  delete m;
}

extern "C" int ls100_model_set_input_ptr(ls100_model* m, int index, void* p) {
  if (!m) return LS100_ERR_BAD_ARG;
  return guarded([&] { m->model->set_input_ptr(index, p); });
}
extern "C" int ls100_model_set_input_shape(ls100_model* m, int index, const int32_t* dims, int nd) {
  if (!m || !dims || nd < 0) return LS100_ERR_BAD_ARG;
  return guarded([&] { m->model->set_input_shape(index, std::vector<int>(dims, dims + nd)); });
}
extern "C" int ls100_model_set_output_ptr(ls100_model* m, int index, void* p) {
  if (!m) return LS100_ERR_BAD_ARG;
  return guarded([&] { m->model->set_output_ptr(index, p); });
}
extern "C" int ls100_model_infer(ls100_model* m) {
  if (!m) return LS100_ERR_BAD_ARG;
  return guarded([&] { m->model->Infer(); });
}
static int copy_shape(const std::vector<int>& s, int32_t* dims, int* nd) {
  if (s.size() > 4) return LS100_ERR_UNSUPPORTED;
  for (size_t i = 0; i < s.size(); ++i) dims[i] = s[i];
  *nd = (int)s.size();
  return LS100_OK;
}
extern "C" int ls100_model_get_output_shape(ls100_model* m, int index, int32_t* dims, int* nd) {
  if (!m || !dims || !nd) return LS100_ERR_BAD_ARG;
  int rc = LS100_OK;
  int g = guarded([&] { rc = copy_shape(m->model->get_output_shape(index), dims, nd); });
  return g ? g : rc;
}
extern "C" int ls100_model_get_output_max_shape(ls100_model* m, int index, int32_t* dims, int* nd) {
  if (!m || !dims || !nd) return LS100_ERR_BAD_ARG;
  int rc = LS100_OK;
  int g = guarded([&] { rc = copy_shape(m->model->get_output_max_shape(index), dims, nd); });
  return g ? g : rc;
}
extern "C" int ls100_model_benchmark_mode(ls100_model* m, int on) {
  if (!m) return LS100_ERR_BAD_ARG;
  return guarded([&] { m->model->benchmark_mode(on != 0); });
}

extern "C" int ls100_model_get_stream(ls100_model* m, ls100_stream_t* stream) {
  if (!m || !stream) return LS100_ERR_BAD_ARG;
  cudaStream_t s = ls100::model_stream(m->model.get());
  *stream = (ls100_stream_t)s;
  return LS100_OK;
}

// H2D copy of the ids + Infer() into the model's staging buffers; k sequences of n tokens per sentence come out
static void transformer_run_host(ls100_model* m, const int32_t* ids, int batch, int seq_len, int* k, int* n) {
  const size_t nb = (size_t)batch * seq_len * 4;
  if (nb > m->in_bytes) throw std::runtime_error("input larger than max_batch_size x max_step");
  LS_CUDA(cudaSetDevice(m->device));
  LS_CUDA(cudaMemcpy(m->d_in, ids, nb, cudaMemcpyHostToDevice));
  m->model->set_input_ptr(0, m->d_in);
  m->model->set_input_shape(0, {batch, seq_len});
  m->model->set_output_ptr(0, m->d_out0);
  m->model->set_output_ptr(1, m->d_out1);
  m->model->Infer();
  const std::vector<int> shp = m->model->get_output_shape(0);
  *k = shp.at(1);
  *n = shp.at(2);
}

extern "C" int ls100_transformer_infer_host_k(ls100_model* m, const int32_t* ids, int batch, int seq_len,
                                              int32_t* out_tokens, float* out_scores, int* out_k, int* out_len) {
  if (!m || !ids || !out_tokens || !out_scores || !out_k || !out_len || batch < 1 || seq_len < 1) return LS100_ERR_BAD_ARG;
  return guarded([&] {
    int k = 0, n = 0;
    transformer_run_host(m, ids, batch, seq_len, &k, &n);
    LS_CUDA(cudaMemcpy(out_tokens, m->d_out0, (size_t)batch * k * n * 4, cudaMemcpyDeviceToHost));
    LS_CUDA(cudaMemcpy(out_scores, m->d_out1, (size_t)batch * k * 4, cudaMemcpyDeviceToHost));
    *out_k = k;
    *out_len = n;
  });
}

extern "C" int ls100_transformer_infer_host(ls100_model* m, const int32_t* ids, int batch, int seq_len,
                                            int32_t* out_tokens, float* out_scores, int* out_len) {
  if (!m || !ids || !out_tokens || !out_scores || !out_len || batch < 1 || seq_len < 1) return LS100_ERR_BAD_ARG;
  return guarded([&] {
    int k = 0, n = 0;
    transformer_run_host(m, ids, batch, seq_len, &k, &n);
    if (k != 1)  // the caller's buffers hold one sequence per sentence: nothing is copied
      throw std::runtime_error("this model returns several sequences per sentence: call ls100_transformer_infer_host_k");
    LS_CUDA(cudaMemcpy(out_tokens, m->d_out0, (size_t)batch * n * 4, cudaMemcpyDeviceToHost));
    LS_CUDA(cudaMemcpy(out_scores, m->d_out1, (size_t)batch * 4, cudaMemcpyDeviceToHost));
    *out_len = n;
  });
}

extern "C" int ls100_bert_infer_host(ls100_model* m, const int32_t* ids, int batch, int seq_len, float* out) {
  if (!m || !ids || !out || batch < 1 || seq_len < 1) return LS100_ERR_BAD_ARG;
  return guarded([&] {
    const size_t nb = (size_t)batch * seq_len * 4;
    if (nb > m->in_bytes) throw std::runtime_error("input larger than max_batch_size x max_step");
    LS_CUDA(cudaSetDevice(m->device));
    LS_CUDA(cudaMemcpy(m->d_in, ids, nb, cudaMemcpyHostToDevice));
    m->model->set_input_ptr(0, m->d_in);
    m->model->set_input_shape(0, {batch, seq_len});
    m->model->set_output_ptr(0, m->d_out0);
    m->model->Infer();
    const std::vector<int> shp = m->model->get_output_shape(0);
    LS_CUDA(cudaMemcpy(out, m->d_out0, prod(shp) * 4, cudaMemcpyDeviceToHost));
  });
}

extern "C" int ls100_vit_infer_host(ls100_model* m, const float* pixels, int batch, int channels, int image, float* out) {
  if (!m || !pixels || !out || batch < 1) return LS100_ERR_BAD_ARG;
  return guarded([&] {
    std::vector<int> in = m->model->get_input_max_shape(0);  // [max_batch, channels, image, image]
    if (in.size() != 4) throw std::runtime_error("not a QuantVit model");
    if (batch > in[0]) throw std::runtime_error("batch size of input greater than max_batch_size");
    if (channels != in[1] || image != in[2])
      throw std::runtime_error("pixel_input must be [batch, " + std::to_string(in[1]) + ", " + std::to_string(in[2]) + ", " +
                               std::to_string(in[3]) + "]");
    in[0] = batch;
    LS_CUDA(cudaSetDevice(m->device));
    LS_CUDA(cudaMemcpy(m->d_in, pixels, prod(in) * 4, cudaMemcpyHostToDevice));
    m->model->set_input_ptr(0, m->d_in);
    m->model->set_input_shape(0, in);
    m->model->set_output_ptr(0, m->d_out0);
    m->model->Infer();
    LS_CUDA(cudaMemcpy(out, m->d_out0, prod(m->model->get_output_shape(0)) * 4, cudaMemcpyDeviceToHost));
  });
}

extern "C" int ls100_gpt_sample_host(ls100_model* m, const int32_t* ids, int batch, int prompt_len, int32_t* out_tokens,
                                     int* out_len) {
  if (!m || !ids || !out_tokens || !out_len || batch < 1 || prompt_len < 1) return LS100_ERR_BAD_ARG;
  return guarded([&] {
    const size_t nb = (size_t)batch * prompt_len * 4;
    if (nb > m->in_bytes) throw std::runtime_error("input larger than max_batch_size x max_step");
    LS_CUDA(cudaSetDevice(m->device));
    LS_CUDA(cudaMemcpy(m->d_in, ids, nb, cudaMemcpyHostToDevice));
    m->model->set_input_ptr(0, m->d_in);
    m->model->set_input_shape(0, {batch, prompt_len});
    m->model->set_output_ptr(0, m->d_out0);
    m->model->Infer();
    const std::vector<int> shp = m->model->get_output_shape(0);
    LS_CUDA(cudaMemcpy(out_tokens, m->d_out0, prod(shp) * 4, cudaMemcpyDeviceToHost));
    *out_len = shp.at(1);
  });
}

extern "C" int ls100_gpt_ppl_host(ls100_model* m, const int32_t* ids, int batch, int seq_len, float* out_ppl) {
  if (!m || !ids || !out_ppl || batch < 1 || seq_len < 1) return LS100_ERR_BAD_ARG;
  return guarded([&] {
    const size_t nb = (size_t)batch * seq_len * 4;
    if (nb > m->in_bytes) throw std::runtime_error("input larger than max_batch_size x max_step");
    if ((size_t)batch * 4 > m->out0_bytes) throw std::runtime_error("batch larger than max_batch_size");
    LS_CUDA(cudaSetDevice(m->device));
    LS_CUDA(cudaMemcpy(m->d_in, ids, nb, cudaMemcpyHostToDevice));
    ls100::quant_gpt_ppl(m->model.get(), static_cast<const int32_t*>(m->d_in), batch, seq_len,
                         static_cast<float*>(m->d_out0));
    LS_CUDA(cudaMemcpy(out_ppl, m->d_out0, (size_t)batch * 4, cudaMemcpyDeviceToHost));
  });
}

// ---- test-only taps (not declared in include/ls100.h): device pointers valid until the next Infer()
extern "C" const float* ls100_debug_encoder_output(ls100_model* m) {
  return m ? ls100::quant_transformer_encoder_output(m->model.get()) : nullptr;
}
extern "C" const int8_t* ls100_debug_last_logits(ls100_model* m, int* ld) {
  return m ? ls100::quant_transformer_last_logits(m->model.get(), ld) : nullptr;
}
// every later Infer() copies the residual stream after the embedding and after each encoder layer into `device_buf`
// (NULL switches the tap off); returns the number of floats the last Infer() wrote
extern "C" long long ls100_debug_set_layer_tap(ls100_model* m, float* device_buf, long long capacity_floats) {
  auto* e = m ? dynamic_cast<ls100::EngineModel*>(m->model.get()) : nullptr;
  if (!e || capacity_floats < 0) return -1;
  const long long used = (long long)e->layer_tap_floats();
  e->set_layer_tap(device_buf, (size_t)capacity_floats);
  return used;
}
// launches the expiring wait of ls100_debug_expire_wait on the model's own context and stream: the next Infer() must
// surface LS100_ERR_TIMEOUT as an error
extern "C" int ls100_debug_model_expire_wait(ls100_model* m) {
  auto* e = m ? dynamic_cast<ls100::EngineModel*>(m->model.get()) : nullptr;
  if (!e) return LS100_ERR_BAD_ARG;
  return ls100_debug_expire_wait(e->context()->kernels(), (ls100_stream_t)e->context()->get_stream());
}
extern "C" int ls100_debug_steps_run(ls100_model* m) {
  return m ? ls100::quant_transformer_steps_run(m->model.get()) : -1;
}
extern "C" int ls100_debug_set_step_limit(ls100_model* m, int n) {
  return m ? ls100::quant_transformer_set_step_limit(m->model.get(), n) : -1;
}
extern "C" int ls100_debug_beam_state(ls100_model* m, const int32_t** alive, const int32_t** anc, const float** probs,
                                      const float** score, int* max_step, int* beam) {
  return m ? ls100::quant_transformer_beam_state(m->model.get(), alive, anc, probs, score, max_step, beam) : -1;
}
