// Hugging Face safetensors, read-only: header parse + index over one or more shards, tensors reached
// through mmap. File layout: 8-byte little-endian header length, JSON header (name -> dtype, shape,
// data_offsets relative to the end of the header), raw data.
// Reference: crates/kern-runtime/src/weights.rs:23-252 (Blob, Safetensors, header, find, dtype names).
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../manifest/json.hpp"
#include "../manifest/types.hpp"

namespace kern {

struct MappedFile {
  int fd = -1;
  const uint8_t* data = nullptr;
  size_t size = 0;
  std::string path;
  explicit MappedFile(const std::string& p) : path(p) {
    fd = ::open(p.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("cannot open " + p);
    struct stat st;
    if (fstat(fd, &st) != 0) { ::close(fd); throw std::runtime_error("cannot stat " + p); }
    size = (size_t)st.st_size;
    if (size) {
      void* m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
      if (m == MAP_FAILED) { ::close(fd); throw std::runtime_error("cannot mmap " + p); }
      data = static_cast<const uint8_t*>(m);
    }
  }
  ~MappedFile() {
    if (data) munmap(const_cast<uint8_t*>(data), size);
    if (fd >= 0) ::close(fd);
  }
  MappedFile(const MappedFile&) = delete;
};

struct TensorInfo {
  std::string dtype;               // safetensors spelling: BF16, F16, F32, F8_E4M3, F8_E8M0, I8, U8, I32, U32, I64, U64
  std::vector<uint64_t> shape;
  const uint8_t* data = nullptr;
  uint64_t bytes = 0;
  std::string file;
};

// manifest dtype for a safetensors dtype name; false when there is no counterpart
inline bool dtype_named(const std::string& st, DType& out) {
  static const std::pair<const char*, DType> t[] = {
      {"BF16", DType::bf16}, {"F16", DType::f16}, {"F32", DType::f32}, {"F8_E4M3", DType::fp8e4m3},
      {"F8_E8M0", DType::fp8e8m0}, {"I8", DType::i8}, {"U8", DType::u8}, {"I32", DType::i32},
      {"U32", DType::u32}, {"I64", DType::i64}, {"U64", DType::u64}};
  for (auto& p : t) if (st == p.first) { out = p.second; return true; }
  return false;
}

class Safetensors {
 public:
  // `paths`: shard files; a tensor must appear in exactly one of them
  explicit Safetensors(const std::vector<std::string>& paths) {
    for (auto& p : paths) add(p);
  }
  const TensorInfo* find(const std::string& name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &it->second;
  }
  std::vector<std::string> names() const {
    std::vector<std::string> out;
    for (auto& kv : index_) out.push_back(kv.first);
    return out;
  }
  size_t size() const { return index_.size(); }

 private:
  std::vector<std::unique_ptr<MappedFile>> files_;
  std::map<std::string, TensorInfo> index_;

  void add(const std::string& path) {
    files_.push_back(std::make_unique<MappedFile>(path));
    const MappedFile& f = *files_.back();
    if (f.size < 8) throw std::runtime_error(path + ": shorter than a safetensors header");
    uint64_t hlen = 0;
    for (int i = 0; i < 8; ++i) hlen |= (uint64_t)f.data[i] << (8 * i);
    if (hlen > f.size - 8) throw std::runtime_error(path + ": header length runs past the file");
    Json h = parse_json(std::string(reinterpret_cast<const char*>(f.data + 8), (size_t)hlen));
    if (!h.is_obj()) throw std::runtime_error(path + ": header is not an object");
    const uint8_t* base = f.data + 8 + hlen;
    const uint64_t avail = f.size - 8 - hlen;
    for (auto& kv : h.obj) {
      if (kv.first == "__metadata__") continue;
      const Json* dt = kv.second.find("dtype");
      const Json* sh = kv.second.find("shape");
      const Json* off = kv.second.find("data_offsets");
      if (!dt || !dt->is_str() || !sh || !sh->is_arr() || !off || !off->is_arr() || off->arr.size() != 2 ||
          !off->arr[0].is_uint() || !off->arr[1].is_uint())
        throw std::runtime_error(path + ": tensor `" + kv.first + "` has a malformed header entry");
      TensorInfo t;
      t.dtype = dt->s;
      for (auto& d : sh->arr) {
        if (!d.is_uint()) throw std::runtime_error(path + ": tensor `" + kv.first + "` has a malformed shape");
        t.shape.push_back(d.u);
      }
      const uint64_t lo = off->arr[0].u, hi = off->arr[1].u;
      if (lo > hi || hi > avail) throw std::runtime_error(path + ": tensor `" + kv.first + "` lies outside the file");
      t.data = base + lo;
      t.bytes = hi - lo;
      t.file = path;
      if (index_.count(kv.first)) throw std::runtime_error("tensor `" + kv.first + "` appears in more than one shard");
      index_[kv.first] = std::move(t);
    }
  }
};

}  // namespace kern
