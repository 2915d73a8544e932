// Base of the engine's LSModel implementations: exposes the Context (stream, kernel handle).
#pragma once
#include "lsflow.h"
#include "model_base.h"

namespace ls100 {

class EngineModel : public LSModel {
 public:
  using LSModel::LSModel;
  virtual ContextPtr context() const = 0;
};

// QuantGpt only (quant_gpt.cpp): device ids [batch, seq_len] -> device ppl [batch]; synchronises the stream.
void quant_gpt_ppl(LSModel* m, const int32_t* d_ids, int batch, int seq_len, float* d_ppl);

}  // namespace ls100
