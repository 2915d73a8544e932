// Reader of the flat ".ls100" weight container (layout documented in
// lightseq_b200/weights.py). Plays the role of the reference's
// QuantTransformerWeight::initializing (lightseq/inference/proto/quant_transformer_weight.cc):
// model configuration, every clip-max and the fp32 tensors, which the engine then
// quantises on the device.
#pragma once
#include <stdint.h>
#include <string.h>

#include <fstream>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace ls100 {

struct HostTensor {
  std::vector<int64_t> dims;
  const float* data = nullptr;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
};

class WeightsFile {
 public:
  explicit WeightsFile(const std::string& path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open weight file: " + path);
    const std::streamsize n = f.tellg();
    f.seekg(0);
    buf_.resize((size_t)n);
    if (!f.read(buf_.data(), n)) throw std::runtime_error("cannot read weight file: " + path);
    static const char magic[8] = {'L', 'S', '1', '0', '0', 'W', 1, 0};
    if (n < 8 || memcmp(buf_.data(), magic, 8) != 0) throw std::runtime_error(path + ": not an .ls100 weight file");
    size_t p = 8;
    uint32_t cnt = rd<uint32_t>(p);
    for (uint32_t i = 0; i < cnt; ++i) {
      std::string k = rd_name(p);
      conf_[k] = rd<double>(p);
    }
    cnt = rd<uint32_t>(p);
    for (uint32_t i = 0; i < cnt; ++i) {
      std::string k = rd_name(p);
      strs_[k] = rd_name(p);
    }
    cnt = rd<uint32_t>(p);
    for (uint32_t i = 0; i < cnt; ++i) {
      std::string k = rd_name(p);
      amax_[k] = rd<float>(p);
    }
    cnt = rd<uint32_t>(p);
    struct Meta {
      std::string name;
      std::vector<int64_t> dims;
      uint64_t off, nbytes;
    };
    std::vector<Meta> metas;
    for (uint32_t i = 0; i < cnt; ++i) {
      Meta m;
      m.name = rd_name(p);
      const uint32_t nd = rd<uint32_t>(p);
      for (uint32_t d = 0; d < nd; ++d) m.dims.push_back((int64_t)rd<uint64_t>(p));
      m.off = rd<uint64_t>(p);
      m.nbytes = rd<uint64_t>(p);
      metas.push_back(std::move(m));
    }
    const size_t data0 = (p + 63) / 64 * 64;
    for (auto& m : metas) {
      if (data0 + m.off + m.nbytes > buf_.size()) throw std::runtime_error(path + ": truncated tensor " + m.name);
      HostTensor t;
      t.dims = m.dims;
      t.data = reinterpret_cast<const float*>(buf_.data() + data0 + m.off);
      if ((uint64_t)t.numel() * 4 != m.nbytes) throw std::runtime_error(path + ": bad size for tensor " + m.name);
      tensors_[m.name] = t;
    }
  }

  double conf(const std::string& k) const {
    auto it = conf_.find(k);
    if (it == conf_.end()) throw std::runtime_error("weight file has no config entry '" + k + "'");
    return it->second;
  }
  double conf_or(const std::string& k, double dflt) const {
    auto it = conf_.find(k);
    return it == conf_.end() ? dflt : it->second;
  }
  float amax(const std::string& k) const {
    auto it = amax_.find(k);
    if (it == amax_.end()) throw std::runtime_error("weight file has no clip-max '" + k + "'");
    if (!(it->second > 0.f)) throw std::runtime_error("clip-max '" + k + "' is not positive");
    return it->second;
  }
  // A clip-max that may be stored as 0 = "this output is not quantised" (file formats without that entry).
  float amax_or_unquantised(const std::string& k) const {
    auto it = amax_.find(k);
    if (it == amax_.end()) throw std::runtime_error("weight file has no clip-max '" + k + "'");
    if (it->second == 0.f) return 0.f;
    return amax(k);
  }
  const HostTensor& tensor(const std::string& k) const {
    auto it = tensors_.find(k);
    if (it == tensors_.end()) throw std::runtime_error("weight file has no tensor '" + k + "'");
    return it->second;
  }
  bool has_tensor(const std::string& k) const { return tensors_.count(k) != 0; }
  std::string model() const {
    auto it = strs_.find("model");
    return it == strs_.end() ? std::string() : it->second;
  }

 private:
  template <typename T>
  T rd(size_t& p) {
    if (p + sizeof(T) > buf_.size()) throw std::runtime_error("weight file header truncated");
    T v;
    memcpy(&v, buf_.data() + p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string rd_name(size_t& p) {
    const uint16_t n = rd<uint16_t>(p);
    if (p + n > buf_.size()) throw std::runtime_error("weight file header truncated");
    std::string s(buf_.data() + p, n);
    p += n;
    return s;
  }
  std::vector<char> buf_;
  std::map<std::string, double> conf_;
  std::map<std::string, std::string> strs_;
  std::map<std::string, float> amax_;
  std::map<std::string, HostTensor> tensors_;
};

}  // namespace ls100
