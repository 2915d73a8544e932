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

}  // namespace ls100
