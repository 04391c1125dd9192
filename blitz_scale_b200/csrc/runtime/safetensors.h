// Read-only view of a .safetensors file: 8-byte little-endian header length, a JSON header mapping tensor names to
// {dtype, shape, data_offsets}, then the raw little-endian tensor bytes.  The file is mapped, not read: a tensor is a
// pointer into the mapping, and the weight converter copies each one exactly once, into the weight segment.
// Counterpart of the reference's vendored safetensors reader (src/model/safetensors.hh), which nothing there uses;
// here it feeds the Hugging Face -> weight-segment converter.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../util/minijson.h"

namespace blitz {

struct SafeTensorInfo {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // byte range inside the data section
};

inline int safetensors_dtype_size(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
  return 0;
}

class SafeTensorsFile {
 public:
  explicit SafeTensorsFile(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("safetensors: cannot open " + path);
    struct stat st;
    if (::fstat(fd_, &st) != 0 || st.st_size < 8) { ::close(fd_); throw std::runtime_error("safetensors: short file " + path); }
    size_ = static_cast<uint64_t>(st.st_size);
    map_ = static_cast<uint8_t*>(::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0));
    if (map_ == MAP_FAILED) { ::close(fd_); map_ = nullptr; throw std::runtime_error("safetensors: mmap failed"); }
    uint64_t hlen = 0;
    std::memcpy(&hlen, map_, 8);
    if (hlen > size_ - 8 || hlen > (100ull << 20)) { release(); throw std::runtime_error("safetensors: bad header length"); }
    data_ = 8 + hlen;
    try {
      const json::Value root = json::parse(std::string_view(reinterpret_cast<const char*>(map_ + 8), hlen));
      for (const auto& kv : root.obj) {
        if (kv.first == "__metadata__") {
          for (const auto& m : kv.second.obj) metadata_.emplace_back(m.first, m.second.str);
          continue;
        }
        SafeTensorInfo t;
        t.name = kv.first;
        t.dtype = kv.second.at("dtype").str;
        for (const auto& d : kv.second.at("shape").arr) t.shape.push_back(d.as_int());
        const auto& off = kv.second.at("data_offsets").arr;
        if (off.size() != 2) throw std::runtime_error("safetensors: bad data_offsets for " + t.name);
        // the offsets come from the file: compare them as the numbers they are before any conversion, so that a
        // negative, fractional or huge value cannot wrap into the mapped range
        const double avail = static_cast<double>(size_ - data_);
        if (!(off[0].num >= 0) || !(off[1].num >= off[0].num) || !(off[1].num <= avail))
          throw std::runtime_error("safetensors: tensor " + t.name + " does not fit its byte range");
        t.begin = static_cast<uint64_t>(off[0].num);
        t.end = static_cast<uint64_t>(off[1].num);
        uint64_t want = static_cast<uint64_t>(safetensors_dtype_size(t.dtype));
        for (int64_t d : t.shape) {
          if (d < 0 || (d > 0 && want > (size_ / static_cast<uint64_t>(d))))   // also bounds the product: no overflow
            throw std::runtime_error("safetensors: tensor " + t.name + " has a shape its file cannot hold");
          want *= static_cast<uint64_t>(d);
        }
        if (t.end < t.begin || t.end > size_ - data_ || (safetensors_dtype_size(t.dtype) && want != t.end - t.begin))
          throw std::runtime_error("safetensors: tensor " + t.name + " does not fit its byte range");
        tensors_.push_back(std::move(t));
      }
    } catch (...) {
      release();
      throw;
    }
  }
  ~SafeTensorsFile() { release(); }
  SafeTensorsFile(const SafeTensorsFile&) = delete;
  SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;

  const std::vector<SafeTensorInfo>& tensors() const { return tensors_; }
  const std::vector<std::pair<std::string, std::string>>& metadata() const { return metadata_; }
  const SafeTensorInfo* find(const std::string& name) const {
    for (const auto& t : tensors_) if (t.name == name) return &t;
    return nullptr;
  }
  const uint8_t* data(const SafeTensorInfo& t) const { return map_ + data_ + t.begin; }

 private:
  int fd_ = -1;
  uint8_t* map_ = nullptr;
  uint64_t size_ = 0, data_ = 0;
  std::vector<SafeTensorInfo> tensors_;
  std::vector<std::pair<std::string, std::string>> metadata_;
  void release() {
    if (map_) ::munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
    map_ = nullptr;
    fd_ = -1;
  }
};

}  // namespace blitz
