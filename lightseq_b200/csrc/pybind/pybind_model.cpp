// pybind11 module with the class surface of the reference's `lightseq.inference`
// (lightseq/inference/pywrapper/wrapper.cc:85-156 PyQuantTransformer, :919-996 module
// definition): QuantTransformer(weight_path, max_batch_size).infer(int32[B,S]) ->
// (int32[B,1,L], float32[B,1]). Each call copies the ids host->device, runs the model and
// copies the results back, like the reference wrapper. The classes sit on the C ABI of
// libls100.so (include/ls100.h, "model level").
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "ls100.h"

namespace py = pybind11;

namespace {

void check(int rc, const char* what) {
  if (rc != LS100_OK) {
    const char* msg = ls100_model_last_error();
    throw std::runtime_error(std::string(what) + ": " + ((msg && *msg) ? msg : ls100_strerror(rc)));
  }
}

class PyQuantTransformer {
 public:
  PyQuantTransformer(const std::string& weight_path, int max_batch_size) {
    check(ls100_model_create("QuantTransformer", weight_path.c_str(), max_batch_size, &m_), "QuantTransformer");
    int32_t dims[4];
    int nd = 0;
    check(ls100_model_get_output_max_shape(m_, 0, dims, &nd), "get_output_max_shape");
    beam_ = dims[1];
    max_step_ = dims[2];
  }
  ~PyQuantTransformer() { ls100_model_destroy(m_); }
  PyQuantTransformer(const PyQuantTransformer&) = delete;
  PyQuantTransformer& operator=(const PyQuantTransformer&) = delete;

  std::tuple<py::array_t<int>, py::array_t<float>> infer(
      py::array_t<int, py::array::c_style | py::array::forcecast> input_seq) {
    if (input_seq.ndim() != 2) throw std::runtime_error("input_seq must be a 2-D int32 array [batch, seq_len]");
    const int batch = (int)input_seq.shape(0), seq = (int)input_seq.shape(1);
    std::vector<int32_t> toks((size_t)batch * beam_ * max_step_);
    std::vector<float> sc((size_t)batch * beam_);
    int n = 0, k = 0;
    {
      py::gil_scoped_release nogil;
      check(ls100_transformer_infer_host_k(m_, input_seq.data(), batch, seq, toks.data(), sc.data(), &k, &n), "infer");
    }
    py::array_t<int> tokens({batch, k, n});
    py::array_t<float> scores({batch, k});
    std::copy(toks.begin(), toks.begin() + (size_t)batch * k * n, tokens.mutable_data());
    std::copy(sc.begin(), sc.begin() + (size_t)batch * k, scores.mutable_data());
    return std::make_tuple(tokens, scores);
  }
  void benchmark_mode(bool on) { check(ls100_model_benchmark_mode(m_, on ? 1 : 0), "benchmark_mode"); }
  std::uintptr_t handle() const { return reinterpret_cast<std::uintptr_t>(m_); }

 private:
  ls100_model* m_ = nullptr;
  int beam_ = 1, max_step_ = 0;
};

// QuantBert(weight_path, max_batch_size).infer(int32[B,S]) -> float32[B,S,H]
// (PyQuantBert, lightseq/inference/pywrapper/wrapper.cc:240-321)
class PyQuantBert {
 public:
  PyQuantBert(const std::string& weight_path, int max_batch_size) {
    check(ls100_model_create("QuantBert", weight_path.c_str(), max_batch_size, &m_), "QuantBert");
    int32_t dims[4];
    int nd = 0;
    check(ls100_model_get_output_max_shape(m_, 0, dims, &nd), "get_output_max_shape");
    hidden_ = dims[2];
  }
  ~PyQuantBert() { ls100_model_destroy(m_); }
  PyQuantBert(const PyQuantBert&) = delete;
  PyQuantBert& operator=(const PyQuantBert&) = delete;
  py::array_t<float> infer(py::array_t<int, py::array::c_style | py::array::forcecast> input_seq) {
    if (input_seq.ndim() != 2) throw std::runtime_error("input_seq must be a 2-D int32 array [batch, seq_len]");
    const int batch = (int)input_seq.shape(0), seq = (int)input_seq.shape(1);
    py::array_t<float> out({batch, seq, hidden_});
    {
      py::gil_scoped_release nogil;
      check(ls100_bert_infer_host(m_, input_seq.data(), batch, seq, out.mutable_data()), "infer");
    }
    return out;
  }
  std::uintptr_t handle() const { return reinterpret_cast<std::uintptr_t>(m_); }

 private:
  ls100_model* m_ = nullptr;
  int hidden_ = 0;
};

// QuantVit(weight_path, max_batch_size).infer(float32[B,C,I,I]) -> float32[B,1+patches,H]
// (PyQuantVit, lightseq/inference/pywrapper/wrapper.cc)
class PyQuantVit {
 public:
  PyQuantVit(const std::string& weight_path, int max_batch_size) {
    check(ls100_model_create("QuantVit", weight_path.c_str(), max_batch_size, &m_), "QuantVit");
    int32_t dims[4];
    int nd = 0;
    check(ls100_model_get_output_max_shape(m_, 0, dims, &nd), "get_output_max_shape");
    seq_ = dims[1];
    hidden_ = dims[2];
  }
  ~PyQuantVit() { ls100_model_destroy(m_); }
  PyQuantVit(const PyQuantVit&) = delete;
  PyQuantVit& operator=(const PyQuantVit&) = delete;
  py::array_t<float> infer(py::array_t<float, py::array::c_style | py::array::forcecast> pixel_input) {
    if (pixel_input.ndim() != 4) throw std::runtime_error("pixel_input must be a 4-D float32 array [batch, channels, image, image]");
    if (pixel_input.shape(2) != pixel_input.shape(3)) throw std::runtime_error("pixel_input must be square images");
    const int batch = (int)pixel_input.shape(0), channels = (int)pixel_input.shape(1), image = (int)pixel_input.shape(2);
    py::array_t<float> out({batch, seq_, hidden_});
    {
      py::gil_scoped_release nogil;
      check(ls100_vit_infer_host(m_, pixel_input.data(), batch, channels, image, out.mutable_data()), "infer");
    }
    return out;
  }
  std::uintptr_t handle() const { return reinterpret_cast<std::uintptr_t>(m_); }

 private:
  ls100_model* m_ = nullptr;
  int seq_ = 0, hidden_ = 0;
};

// QuantGpt(weight_path, max_batch_size).sample(int32[B,P]) -> int32[B,L]
// (PyQuantGpt::sample, lightseq/inference/pywrapper/wrapper.cc:427-495)
class PyQuantGpt {
 public:
  PyQuantGpt(const std::string& weight_path, int max_batch_size) {
    check(ls100_model_create("QuantGpt", weight_path.c_str(), max_batch_size, &m_), "QuantGpt");
    int32_t dims[4];
    int nd = 0;
    check(ls100_model_get_output_max_shape(m_, 0, dims, &nd), "get_output_max_shape");
    max_step_ = dims[1];
  }
  ~PyQuantGpt() { ls100_model_destroy(m_); }
  PyQuantGpt(const PyQuantGpt&) = delete;
  PyQuantGpt& operator=(const PyQuantGpt&) = delete;
  py::array_t<int> sample(py::array_t<int, py::array::c_style | py::array::forcecast> input_seq) {
    if (input_seq.ndim() != 2) throw std::runtime_error("input_seq must be a 2-D int32 array [batch, seq_len]");
    const int batch = (int)input_seq.shape(0), seq = (int)input_seq.shape(1);
    std::vector<int32_t> toks((size_t)batch * max_step_);
    int n = 0;
    {
      py::gil_scoped_release nogil;
      check(ls100_gpt_sample_host(m_, input_seq.data(), batch, seq, toks.data(), &n), "sample");
    }
    py::array_t<int> out({batch, n});
    std::copy(toks.begin(), toks.begin() + (size_t)batch * n, out.mutable_data());
    return out;
  }
  // ppl(int32[B,S]) -> float32[B] (PyQuantGpt::ppl, lightseq/inference/pywrapper/wrapper.cc:497-531)
  py::array_t<float> ppl(py::array_t<int, py::array::c_style | py::array::forcecast> input_seq) {
    if (input_seq.ndim() != 2) throw std::runtime_error("input_seq must be a 2-D int32 array [batch, seq_len]");
    const int batch = (int)input_seq.shape(0), seq = (int)input_seq.shape(1);
    py::array_t<float> out({batch});
    {
      py::gil_scoped_release nogil;
      check(ls100_gpt_ppl_host(m_, input_seq.data(), batch, seq, out.mutable_data()), "ppl");
    }
    return out;
  }
  void benchmark_mode(bool on) { check(ls100_model_benchmark_mode(m_, on ? 1 : 0), "benchmark_mode"); }
  std::uintptr_t handle() const { return reinterpret_cast<std::uintptr_t>(m_); }

 private:
  ls100_model* m_ = nullptr;
  int max_step_ = 0;
};

}  // namespace

PYBIND11_MODULE(_ls100_py, m) {
  m.doc() = "B200 int8 inference engine with the lightseq.inference class surface";
  py::class_<PyQuantTransformer>(m, "QuantTransformer")
      .def(py::init<const std::string&, int>(), py::arg("weight_path"), py::arg("max_batch_size"))
      .def("infer", &PyQuantTransformer::infer, py::arg("input_seq"))
      .def("benchmark_mode", &PyQuantTransformer::benchmark_mode)
      .def_property_readonly("_handle", &PyQuantTransformer::handle);
  py::class_<PyQuantGpt>(m, "QuantGpt")
      .def(py::init<const std::string&, int>(), py::arg("weight_path"), py::arg("max_batch_size"))
      .def("sample", &PyQuantGpt::sample, py::arg("input_seq"))
      .def("ppl", &PyQuantGpt::ppl, py::arg("input_seq"))
      .def("benchmark_mode", &PyQuantGpt::benchmark_mode)
      .def_property_readonly("_handle", &PyQuantGpt::handle);
  py::class_<PyQuantBert>(m, "QuantBert")
      .def(py::init<const std::string&, int>(), py::arg("weight_path"), py::arg("max_batch_size"))
      .def("infer", &PyQuantBert::infer, py::arg("input_seq"))
      .def_property_readonly("_handle", &PyQuantBert::handle);
  py::class_<PyQuantVit>(m, "QuantVit")
      .def(py::init<const std::string&, int>(), py::arg("weight_path"), py::arg("max_batch_size"))
      .def("infer", &PyQuantVit::infer, py::arg("pixel_input"))
      .def_property_readonly("_handle", &PyQuantVit::handle);
}
