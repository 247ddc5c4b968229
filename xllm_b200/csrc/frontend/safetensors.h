// safetensors reader: mmap + header parse, zero-copy tensor views.
//
// The reference reads safetensors through a Rust FFI crate
// (xllm/core/framework/state_dict/safetensors/src/lib.rs) wrapped by StateDictFromSafeTensor; the
// format is small enough to read directly: 8-byte little-endian header length, a JSON header
// mapping names to {dtype, shape, data_offsets}, then the raw tensor bytes.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.h"

namespace xllm {

struct TensorInfo {
  std::string name, dtype;
  std::vector<int64_t> shape;
  uint64_t begin = 0, end = 0;  // byte range inside the data section
};

class SafeTensorsFile {
 public:
  explicit SafeTensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw std::runtime_error("cannot open " + path);
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 8) { ::close(fd_); throw std::runtime_error("bad safetensors file " + path); }
    size_ = (size_t)st.st_size;
    base_ = (uint8_t*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (base_ == MAP_FAILED) { ::close(fd_); throw std::runtime_error("mmap failed for " + path); }
    uint64_t hlen = 0;
    memcpy(&hlen, base_, 8);
    if (hlen > size_ - 8) { cleanup(); throw std::runtime_error("corrupt safetensors header in " + path); }
    data_ = base_ + 8 + hlen;
    data_size_ = size_ - 8 - hlen;
    Json h = Json::parse(std::string((const char*)base_ + 8, (size_t)hlen));
    for (auto& kv : h.members()) {
      if (kv.first == "__metadata__") {
        for (auto& m : kv.second.members()) metadata_.emplace_back(m.first, m.second.as_string());
        continue;
      }
      TensorInfo t;
      t.name = kv.first;
      t.dtype = kv.second["dtype"].as_string();
      for (auto& d : kv.second["shape"].items()) t.shape.push_back(d.as_int());
      const Json& off = kv.second["data_offsets"];
      t.begin = (uint64_t)off[0].as_int();
      t.end = (uint64_t)off[1].as_int();
      if (t.end < t.begin || t.end > data_size_) { cleanup(); throw std::runtime_error("tensor " + t.name + " out of bounds in " + path); }
      tensors_.push_back(std::move(t));
    }
  }
  ~SafeTensorsFile() { cleanup(); }
  SafeTensorsFile(const SafeTensorsFile&) = delete;
  SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;

  const std::vector<TensorInfo>& tensors() const { return tensors_; }
  const std::vector<std::pair<std::string, std::string>>& metadata() const { return metadata_; }
  const uint8_t* data() const { return data_; }
  size_t data_size() const { return data_size_; }
  const std::string& path() const { return path_; }

 private:
  void cleanup() {
    if (base_ && base_ != MAP_FAILED) munmap(base_, size_);
    base_ = nullptr;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }
  std::string path_;
  int fd_ = -1;
  size_t size_ = 0, data_size_ = 0;
  uint8_t* base_ = nullptr;
  const uint8_t* data_ = nullptr;
  std::vector<TensorInfo> tensors_;
  std::vector<std::pair<std::string, std::string>> metadata_;
};

}  // namespace xllm
