// Model-level interface kept from the reference so that serving shells written against
// it keep working: LSModel (set_input_ptr / set_input_shape / Infer / get_output_*),
// LSModelFactory::GetInstance().CreateModel(name, weight_path, max_batch_size) and the
// LSMODEL_REGISTER(cls) macro (lightseq/inference/pywrapper/model_base.h:59-148).
// Pointers handed to set_input_ptr / set_output_ptr are caller-owned DEVICE pointers;
// Infer() returns after the model's stream has been synchronised; errors are
// std::runtime_error; an instance is not thread-safe.
#pragma once
#include <functional>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace ls100 {

enum DataType {
  kNotSupported = 0,
  kFloat32 = 1,
  kInt32 = 2,
  kInt64 = 3,
  kFloat16 = 4,
  kInt8 = 5,
  kInt16 = 6,
  kByte = 7,
  kUInt8 = 8,
  kUInt16 = 9,
  kUInt32 = 10,
  kUInt64 = 11,
  kFloat64 = 12
};

class LSModel {
 public:
  LSModel(std::vector<std::string> input_names, std::vector<std::string> output_names)
      : input_names_(std::move(input_names)), output_names_(std::move(output_names)),
        input_shapes_(input_names_.size()), output_shapes_(output_names_.size()) {}
  virtual ~LSModel() {}

  virtual void Infer() = 0;

  virtual void set_input_ptr(int index, void* input_ptr) = 0;
  void set_input_shape(int index, std::vector<int> shape) { input_shapes_.at(index) = std::move(shape); }
  virtual std::vector<int> get_input_max_shape(int index) = 0;
  virtual DataType get_input_dtype(int index) = 0;
  std::string get_input_name(int index) const { return input_names_.at(index); }
  int get_input_size() const { return (int)input_names_.size(); }

  virtual void set_output_ptr(int index, void* output_ptr) = 0;
  virtual const void* get_output_ptr(int index) = 0;
  virtual std::vector<int> get_output_max_shape(int index) = 0;
  virtual DataType get_output_dtype(int index) = 0;
  std::vector<int> get_output_shape(int index) const { return output_shapes_.at(index); }
  std::string get_output_name(int index) const { return output_names_.at(index); }
  int get_output_size() const { return (int)output_names_.size(); }

  virtual void benchmark_mode(bool is_benchmark) = 0;

 protected:
  void set_output_shape(int index, std::vector<int> shape) { output_shapes_.at(index) = std::move(shape); }
  std::vector<std::string> input_names_, output_names_;
  std::vector<std::vector<int>> input_shapes_, output_shapes_;
};

class LSModelFactory {
 public:
  using Constructor = std::function<LSModel*(const std::string&, int)>;
  static LSModelFactory& GetInstance() {
    static LSModelFactory f;
    return f;
  }
  void ModelRegister(const std::string& name, Constructor c) { ctors_[name] = std::move(c); }
  LSModel* CreateModel(const std::string& name, const std::string& weight_path, int max_batch_size) {
    auto it = ctors_.find(name);
    if (it == ctors_.end()) throw std::runtime_error("Model not supported: " + name);
    return it->second(weight_path, max_batch_size);
  }

 private:
  std::map<std::string, Constructor> ctors_;
};

struct LSModelRegistrar {
  LSModelRegistrar(const std::string& name, LSModelFactory::Constructor c) {
    LSModelFactory::GetInstance().ModelRegister(name, std::move(c));
  }
};

#define LSMODEL_REGISTER(className)                                        \
  static ::ls100::LSModelRegistrar registrar_##className(                  \
      #className, [](const std::string& path, int max_bs) -> ::ls100::LSModel* { return new className(path, max_bs); });

}  // namespace ls100
