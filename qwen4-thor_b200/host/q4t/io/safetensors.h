// Read-only access to .safetensors files for the MoE loader: the subset of the engine's
// io::SafetensorsFile interface (reference include/q4t/io/safetensors.h:27-125) that the
// expert loader and its contract check use, header-only.
//
// File format: 8-byte little-endian header length, a JSON object
//   { "<tensor>": { "dtype": "U8", "shape": [..], "data_offsets": [begin, end] }, ...,
//     "__metadata__": { ... } }
// and the tensor bytes; data_offsets count from the first byte after the header.
// The file is mapped read-only; nothing is read until a tensor is asked for.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "q4t/status.h"

namespace q4t {
namespace io {

enum class Dtype { kF64, kF32, kF16, kBF16, kI64, kI32, kI16, kI8, kU8, kBool, kF8E4M3, kF8E5M2 };

inline size_t DtypeSize(Dtype d) {
  switch (d) {
    case Dtype::kF64: case Dtype::kI64: return 8;
    case Dtype::kF32: case Dtype::kI32: return 4;
    case Dtype::kF16: case Dtype::kBF16: case Dtype::kI16: return 2;
    default: return 1;
  }
}

inline bool ParseDtype(const std::string& s, Dtype* out) {
  static const std::pair<const char*, Dtype> table[] = {
      {"F64", Dtype::kF64}, {"F32", Dtype::kF32}, {"F16", Dtype::kF16}, {"BF16", Dtype::kBF16},
      {"I64", Dtype::kI64}, {"I32", Dtype::kI32}, {"I16", Dtype::kI16}, {"I8", Dtype::kI8},
      {"U8", Dtype::kU8},   {"BOOL", Dtype::kBool}, {"F8_E4M3", Dtype::kF8E4M3}, {"F8_E5M2", Dtype::kF8E5M2}};
  for (const auto& e : table)
    if (s == e.first) {
      *out = e.second;
      return true;
    }
  return false;
}

struct TensorInfo {
  std::string name;
  Dtype dtype = Dtype::kF32;
  std::vector<int64_t> shape;
  uint64_t data_start = 0;  // byte offset into the data region
  uint64_t data_end = 0;    // exclusive
  // Element count; UINT64_MAX when a dimension is negative or the product does not fit
  // (a hostile header), which no extent check can then accept.
  uint64_t numel() const {
    uint64_t n = 1;
    for (int64_t d : shape) {
      if (d < 0) return UINT64_MAX;
      const uint64_t u = static_cast<uint64_t>(d);
      if (u != 0 && n > UINT64_MAX / u) return UINT64_MAX;
      n *= u;
    }
    return n;
  }
  uint64_t byte_size() const { return data_end - data_start; }
};

namespace detail {

// A JSON reader just large enough for safetensors headers and index files: objects,
// arrays, strings (escapes decoded except \u, which is kept verbatim), integers; other
// scalars are skipped.  Values are visited through callbacks, nothing is built.
class JsonCursor {
 public:
  JsonCursor(const char* p, const char* end) : p_(p), end_(end) {}
  bool failed() const { return failed_; }
  void Fail() { failed_ = true; }
  void Skip() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool Peek(char c) {
    Skip();
    return p_ < end_ && *p_ == c;
  }
  bool Eat(char c) {
    if (!Peek(c)) return false;
    ++p_;
    return true;
  }
  bool String(std::string* out) {
    if (!Eat('"')) return fail();
    out->clear();
    while (p_ < end_ && *p_ != '"') {
      if (*p_ == '\\' && p_ + 1 < end_) {
        ++p_;
        switch (*p_) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': out->append("\\u"); break;
          default: out->push_back(*p_);
        }
        ++p_;
      } else {
        out->push_back(*p_++);
      }
    }
    if (p_ >= end_) return fail();
    ++p_;
    return true;
  }
  bool Integer(int64_t* out) {
    Skip();
    const char* s = p_;
    bool neg = false;
    if (p_ < end_ && *p_ == '-') {
      neg = true;
      ++p_;
    }
    uint64_t v = 0;
    const char* digits = p_;
    while (p_ < end_ && *p_ >= '0' && *p_ <= '9') {
      if (v > (UINT64_MAX - 9) / 10) return fail();
      v = v * 10 + static_cast<uint64_t>(*p_++ - '0');
    }
    if (p_ == digits || (p_ < end_ && (*p_ == '.' || *p_ == 'e' || *p_ == 'E'))) {
      p_ = s;
      return fail();
    }
    if (v > static_cast<uint64_t>(INT64_MAX)) return fail();
    *out = neg ? -static_cast<int64_t>(v) : static_cast<int64_t>(v);
    return true;
  }
  // Skips any value.
  bool Any(int depth = 0) {
    if (depth > 64) return fail();
    Skip();
    if (p_ >= end_) return fail();
    if (*p_ == '"') {
      std::string s;
      return String(&s);
    }
    if (*p_ == '{' || *p_ == '[') {
      const char close = *p_ == '{' ? '}' : ']';
      const bool object = *p_ == '{';
      ++p_;
      if (Eat(close)) return true;
      for (;;) {
        if (object) {
          std::string k;
          if (!String(&k) || !Eat(':')) return fail();
        }
        if (!Any(depth + 1)) return false;
        if (Eat(',')) continue;
        return Eat(close) ? true : fail();
      }
    }
    // a bare scalar ends at a separator, a closing bracket or any JSON whitespace
    while (p_ < end_ && *p_ != ',' && *p_ != '}' && *p_ != ']' && *p_ != ' ' && *p_ != '\n' && *p_ != '\t' &&
           *p_ != '\r')
      ++p_;
    return true;
  }
  // Calls f(key) for every member of the object at the cursor; f consumes the value.
  template <class F>
  bool Object(F&& f) {
    if (!Eat('{')) return fail();
    if (Eat('}')) return true;
    for (;;) {
      std::string key;
      if (!String(&key) || !Eat(':')) return fail();
      if (!f(key) || failed_) return fail();
      if (Eat(',')) continue;
      return Eat('}') ? true : fail();
    }
  }
  template <class F>
  bool Array(F&& f) {
    if (!Eat('[')) return fail();
    if (Eat(']')) return true;
    for (;;) {
      if (!f() || failed_) return fail();
      if (Eat(',')) continue;
      return Eat(']') ? true : fail();
    }
  }

 private:
  bool fail() {
    failed_ = true;
    return false;
  }
  const char* p_;
  const char* end_;
  bool failed_ = false;
};

}  // namespace detail

class SafetensorsFile {
 public:
  static Status Open(const std::string& path, SafetensorsFile** out) {
    *out = nullptr;
    std::unique_ptr<SafetensorsFile> f(new SafetensorsFile());
    f->fd_ = ::open(path.c_str(), O_RDONLY);
    if (f->fd_ < 0) return Status::Fail("cannot open " + path);
    struct stat st;
    if (fstat(f->fd_, &st) != 0 || st.st_size < 8) return Status::Fail("not a safetensors file: " + path);
    f->size_ = static_cast<uint64_t>(st.st_size);
    f->map_ = mmap(nullptr, f->size_, PROT_READ, MAP_PRIVATE, f->fd_, 0);
    if (f->map_ == MAP_FAILED) {
      f->map_ = nullptr;
      return Status::Fail("mmap failed: " + path);
    }
    const uint8_t* b = static_cast<const uint8_t*>(f->map_);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | b[i];
    if (hlen > f->size_ - 8) return Status::Fail("safetensors header length out of range: " + path);
    f->data_ = 8 + hlen;
    const uint64_t data_bytes = f->size_ - f->data_;
    detail::JsonCursor js(reinterpret_cast<const char*>(b + 8), reinterpret_cast<const char*>(b + 8 + hlen));
    std::string problem;
    const bool ok = js.Object([&](const std::string& name) {
      if (name == "__metadata__") return js.Any();
      TensorInfo t;
      t.name = name;
      bool have_dtype = false, have_offsets = false;
      if (!js.Object([&](const std::string& key) {
            if (key == "dtype") {
              std::string s;
              if (!js.String(&s)) return false;
              if (!ParseDtype(s, &t.dtype)) {
                problem = "unknown dtype " + s + " for " + name;
                return false;
              }
              have_dtype = true;
              return true;
            }
            if (key == "shape")
              return js.Array([&] {
                int64_t d;
                if (!js.Integer(&d) || d < 0) return false;
                t.shape.push_back(d);
                return true;
              });
            if (key == "data_offsets") {
              int64_t v[2] = {0, 0};
              int n = 0;
              if (!js.Array([&] { return n < 2 && js.Integer(&v[n++]); }) || n != 2 || v[0] < 0 || v[1] < v[0])
                return false;
              t.data_start = static_cast<uint64_t>(v[0]);
              t.data_end = static_cast<uint64_t>(v[1]);
              have_offsets = true;
              return true;
            }
            return js.Any();
          }))
        return false;
      if (!have_dtype || !have_offsets) {
        problem = "incomplete entry for " + name;
        return false;
      }
      const uint64_t n = t.numel(), esz = DtypeSize(t.dtype);
      if (t.data_end > data_bytes || n == UINT64_MAX || esz == 0 || t.byte_size() % esz != 0 ||
          t.byte_size() / esz != n) {
        problem = "extent of " + name + " does not match its shape or the file";
        return false;
      }
      f->index_[name] = f->tensors_.size();
      f->tensors_.push_back(std::move(t));
      return true;
    });
    if (!ok) return Status::Fail("bad safetensors header in " + path + (problem.empty() ? "" : ": " + problem));
    *out = f.release();
    return Status();
  }
  ~SafetensorsFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
  }
  SafetensorsFile(const SafetensorsFile&) = delete;
  SafetensorsFile& operator=(const SafetensorsFile&) = delete;

  const std::vector<TensorInfo>& tensors() const { return tensors_; }
  size_t num_tensors() const { return tensors_.size(); }
  uint64_t file_size() const { return size_; }
  const TensorInfo* Find(const std::string& name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &tensors_[it->second];
  }
  Status ReadTensor(const TensorInfo& t, void* dst) const { return ReadRange(t.data_start, t.byte_size(), dst); }
  Status ReadRange(uint64_t data_start, uint64_t length, void* dst) const {
    if (data_start > size_ - data_ || length > size_ - data_ - data_start) return Status::Fail("read beyond the data region");
    std::memcpy(dst, static_cast<const uint8_t*>(map_) + data_ + data_start, length);
    return Status();
  }

 private:
  SafetensorsFile() = default;
  int fd_ = -1;
  void* map_ = nullptr;
  uint64_t size_ = 0, data_ = 0;
  std::vector<TensorInfo> tensors_;
  std::map<std::string, size_t> index_;
};

}  // namespace io
}  // namespace q4t
