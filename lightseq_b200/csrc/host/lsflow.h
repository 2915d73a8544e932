// A thin re-statement of the reference's "lsflow" runtime shape
// (lightseq/csrc/lsflow: Context, Variable, Operator, Layer): a Context owns the stream,
// the kernel context and every device buffer; Variables are named device buffers;
// Operators wire Variables (`operator()`), take their per-call sizes in
// `before_forward(...)` and launch exactly one C-ABI kernel family in `forward()`;
// Layers own Operators and run them in order. There is no shape-inference dry run and
// no buffer-sharing planner: every buffer is sized for the maxima given at construction,
// which is what 180 GB of HBM makes affordable, and it keeps pointers stable so that a
// decode step can be captured once into a CUDA graph and replayed.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/ls100.h"

namespace ls100 {

inline void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
inline void check_rc(int rc, const char* what) {
  if (rc != LS100_OK) throw std::runtime_error(std::string(what) + ": " + ls100_strerror(rc));
}
#define LS_CUDA(expr) ::ls100::check_cuda((expr), #expr)
#define LS_RC(expr) ::ls100::check_rc((expr), #expr)

enum class StatusType { Inference };

class Context {
 public:
  // Mirrors Context::create_global_context(StatusType::Inference) of the reference
  // (lightseq/csrc/lsflow/context.cpp:103-130); one Context per model instance here.
  static std::shared_ptr<Context> create(StatusType, int device = -1) {
    int dev = device;
    if (dev < 0) LS_CUDA(cudaGetDevice(&dev));
    std::shared_ptr<Context> c(new Context());
    c->device_ = dev;
    LS_CUDA(cudaSetDevice(dev));
    LS_RC(ls100_ctx_create(&c->k_, dev));
    LS_CUDA(cudaStreamCreateWithFlags(&c->stream_, cudaStreamNonBlocking));
    return c;
  }
  ~Context() {
    cudaSetDevice(device_);
    for (void* p : owned_) cudaFree(p);
    for (void* p : owned_host_) cudaFreeHost(p);
    if (stream_) cudaStreamDestroy(stream_);
    if (k_) ls100_ctx_destroy(k_);
  }
  ls100_ctx* kernels() const { return k_; }
  cudaStream_t get_stream() const { return stream_; }
  int device() const { return device_; }
  void* alloc(size_t bytes) {
    void* p = nullptr;
    LS_CUDA(cudaMalloc(&p, bytes ? bytes : 16));
    owned_.push_back(p);
    bytes_ += bytes;
    return p;
  }
  template <typename T>
  T* alloc_n(size_t n) {
    return static_cast<T*>(alloc(n * sizeof(T)));
  }
  void* alloc_host_mapped(size_t bytes) {
    void* p = nullptr;
    LS_CUDA(cudaHostAlloc(&p, bytes, cudaHostAllocMapped));
    owned_host_.push_back(p);
    return p;
  }
  size_t allocated_bytes() const { return bytes_; }

 private:
  Context() = default;
  int device_ = 0;
  ls100_ctx* k_ = nullptr;
  cudaStream_t stream_ = nullptr;
  std::vector<void*> owned_, owned_host_;
  size_t bytes_ = 0;
};
using ContextPtr = std::shared_ptr<Context>;

// A named device buffer. `value()` is what the reference's Variable::value() returns.
class Variable {
 public:
  Variable(std::string name, void* ptr, size_t bytes) : name_(std::move(name)), ptr_(ptr), bytes_(bytes) {}
  Variable(std::string name, Context& ctx, size_t bytes) : name_(std::move(name)), ptr_(ctx.alloc(bytes)), bytes_(bytes) {}
  template <typename T>
  T* value() const {
    return static_cast<T*>(ptr_);
  }
  void set_value(void* p) { ptr_ = p; }
  size_t bytes() const { return bytes_; }
  const std::string& name() const { return name_; }

 private:
  std::string name_;
  void* ptr_;
  size_t bytes_;
};

class Node {
 public:
  Node(std::string name, ContextPtr ctx) : name_(std::move(name)), ctx_(std::move(ctx)) {}
  virtual ~Node() {}
  virtual void forward() = 0;
  const std::string& name() const { return name_; }

 protected:
  std::string name_;
  ContextPtr ctx_;
};

class Operator : public Node {
 public:
  using Node::Node;
};

class Layer : public Node {
 public:
  using Node::Node;
};

}  // namespace ls100
