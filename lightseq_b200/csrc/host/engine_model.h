// Base of the engine's LSModel implementations: exposes the Context (stream, kernel handle).
#pragma once
#include "lsflow.h"
#include "model_base.h"

namespace ls100 {

class EngineModel : public LSModel {
 public:
  using LSModel::LSModel;
  virtual ContextPtr context() const = 0;

  // Test tap: when a device buffer is set, every Infer() copies the fp32 residual stream into it after the embedding
  // and after each encoder layer (slices of batch x seq x hidden floats, in that order), as far as the buffer reaches.
  void set_layer_tap(float* device_buf, size_t capacity_floats) {
    tap_ = device_buf;
    tap_cap_ = capacity_floats;
    tap_used_ = 0;
  }
  size_t layer_tap_floats() const { return tap_used_; }

 protected:
  void tap_reset() { tap_used_ = 0; }
  void tap(const float* src, size_t n, cudaStream_t st) {
    if (!tap_ || tap_used_ + n > tap_cap_) return;
    cudaMemcpyAsync(tap_ + tap_used_, src, n * sizeof(float), cudaMemcpyDeviceToDevice, st);
    tap_used_ += n;
  }

 private:
  float* tap_ = nullptr;
  size_t tap_cap_ = 0, tap_used_ = 0;
};

// QuantGpt only (quant_gpt.cpp): device ids [batch, seq_len] -> device ppl [batch]; synchronises the stream.
void quant_gpt_ppl(LSModel* m, const int32_t* d_ids, int batch, int seq_len, float* d_ppl);

}  // namespace ls100
