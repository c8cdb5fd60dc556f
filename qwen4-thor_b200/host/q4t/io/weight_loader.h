// Tensor lookup over a sharded checkpoint directory: the part of the engine's
// io::WeightIndex / io::WeightLoader interface (reference include/q4t/io/weight_loader.h:
// 33-125) that loading one MoE layer needs, header-only.
//
//   model.safetensors.index.json : { "metadata": {...}, "weight_map": { "<tensor>": "<shard file>" } }
//
// Shards are mapped on first use and kept in a small most-recently-used list; tensor
// metadata handed out by FindTensor stays valid for the loader's lifetime.
#pragma once

#include <cstdio>
#include <list>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "q4t/io/safetensors.h"
#include "q4t/status.h"

namespace q4t {
namespace io {

class WeightIndex {
 public:
  static Status Open(const std::string& path, WeightIndex** out) {
    *out = nullptr;
    std::FILE* fp = std::fopen(path.c_str(), "rb");
    if (!fp) return Status::Fail("cannot open " + path);
    std::string text;
    char buf[1 << 16];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof(buf), fp)) > 0) text.append(buf, n);
    std::fclose(fp);
    std::unique_ptr<WeightIndex> idx(new WeightIndex());
    detail::JsonCursor js(text.data(), text.data() + text.size());
    const bool ok = js.Object([&](const std::string& key) {
      if (key == "weight_map")
        return js.Object([&](const std::string& tensor) {
          std::string shard;
          if (!js.String(&shard)) return false;
          if (idx->map_.emplace(tensor, shard).second) idx->order_.push_back(tensor);
          return true;
        });
      if (key == "metadata")
        return js.Object([&](const std::string& k) {
          int64_t v;
          if (k == "total_size" && js.Integer(&v)) {
            idx->total_size_ = static_cast<uint64_t>(v);
            return true;
          }
          return js.Any();
        });
      return js.Any();
    });
    if (!ok || idx->map_.empty()) return Status::Fail("bad weight index: " + path);
    *out = idx.release();
    return Status();
  }
  // An index over one stand-alone .safetensors file (no index.json beside it).
  static Status FromSingleFile(const std::string& file_name, const SafetensorsFile& file, WeightIndex** out) {
    std::unique_ptr<WeightIndex> idx(new WeightIndex());
    for (const TensorInfo& t : file.tensors()) {
      idx->map_.emplace(t.name, file_name);
      idx->order_.push_back(t.name);
      idx->total_size_ += t.byte_size();
    }
    *out = idx.release();
    return Status();
  }
  WeightIndex(const WeightIndex&) = delete;
  WeightIndex& operator=(const WeightIndex&) = delete;

  const std::string* ShardOf(const std::string& name) const {
    auto it = map_.find(name);
    return it == map_.end() ? nullptr : &it->second;
  }
  bool Has(const std::string& name) const { return map_.count(name) != 0; }
  size_t num_tensors() const { return map_.size(); }
  size_t num_shards() const {
    std::map<std::string, int> s;
    for (const auto& kv : map_) s[kv.second] = 1;
    return s.size();
  }
  uint64_t total_size() const { return total_size_; }
  // (shard file, tensor names in that shard) pairs, shards in order of first appearance.
  std::vector<std::pair<std::string, std::vector<std::string>>> ShardGroups() const {
    std::vector<std::pair<std::string, std::vector<std::string>>> groups;
    std::map<std::string, size_t> where;
    for (const std::string& t : order_) {
      const std::string& shard = map_.at(t);
      auto it = where.find(shard);
      if (it == where.end()) {
        it = where.emplace(shard, groups.size()).first;
        groups.emplace_back(shard, std::vector<std::string>());
      }
      groups[it->second].second.push_back(t);
    }
    return groups;
  }

 private:
  WeightIndex() = default;
  std::map<std::string, std::string> map_;
  std::vector<std::string> order_;
  uint64_t total_size_ = 0;
};

class WeightLoader {
 public:
  static Status Create(const std::string& model_dir, const WeightIndex& index, size_t max_open_shards,
                       WeightLoader** out) {
    *out = new WeightLoader(model_dir, index, max_open_shards == 0 ? 1 : max_open_shards);
    return Status();
  }
  WeightLoader(const WeightLoader&) = delete;
  WeightLoader& operator=(const WeightLoader&) = delete;

  const std::string* ShardOf(const std::string& name) const { return index_.ShardOf(name); }
  // Metadata of `name`; nullptr when the index or its shard does not hold it.
  const TensorInfo* FindTensor(const std::string& name) const {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = info_.find(name);
    if (it != info_.end()) return it->second.get();
    const std::string* shard = index_.ShardOf(name);
    if (!shard) return nullptr;
    std::shared_ptr<SafetensorsFile> f = OpenLocked(*shard);
    const TensorInfo* t = f ? f->Find(name) : nullptr;
    if (!t) return nullptr;
    return info_.emplace(name, std::unique_ptr<TensorInfo>(new TensorInfo(*t))).first->second.get();
  }
  Status ReadTensor(const std::string& name, void* dst) const { return Read(name, dst, false, 0); }
  // Fixed-layout consumer: a different byte size is refused before dst is written.
  Status ReadTensor(const std::string& name, void* dst, size_t expected_bytes) const {
    return Read(name, dst, true, expected_bytes);
  }
  size_t open_shards() const {
    std::lock_guard<std::mutex> lock(mu_);
    return open_.size();
  }

 private:
  WeightLoader(std::string dir, const WeightIndex& index, size_t max_open)
      : dir_(std::move(dir)), index_(index), max_open_(max_open) {}
  Status Read(const std::string& name, void* dst, bool check, size_t expected) const {
    const std::string* shard = index_.ShardOf(name);
    if (!shard) return Status::Fail("tensor not in the index: " + name);
    std::shared_ptr<SafetensorsFile> f;
    {
      std::lock_guard<std::mutex> lock(mu_);
      f = OpenLocked(*shard);
    }
    if (!f) return Status::Fail("cannot open shard " + *shard);
    const TensorInfo* t = f->Find(name);
    if (!t) return Status::Fail("tensor missing from its shard: " + name);
    if (check && t->byte_size() != expected)
      return Status::Fail("tensor " + name + " holds " + std::to_string(t->byte_size()) + " bytes, expected " +
                          std::to_string(expected));
    return f->ReadTensor(*t, dst);  // the copy runs outside the lock; `f` keeps the mapping alive
  }
  std::shared_ptr<SafetensorsFile> OpenLocked(const std::string& shard) const {
    for (auto it = open_.begin(); it != open_.end(); ++it)
      if (it->first == shard) {
        open_.splice(open_.begin(), open_, it);
        return open_.front().second;
      }
    SafetensorsFile* raw = nullptr;
    if (!SafetensorsFile::Open(dir_ + "/" + shard, &raw).ok()) return nullptr;
    open_.emplace_front(shard, std::shared_ptr<SafetensorsFile>(raw));
    while (open_.size() > max_open_) open_.pop_back();
    return open_.front().second;
  }
  std::string dir_;
  const WeightIndex& index_;
  size_t max_open_;
  mutable std::mutex mu_;
  mutable std::list<std::pair<std::string, std::shared_ptr<SafetensorsFile>>> open_;
  mutable std::map<std::string, std::unique_ptr<TensorInfo>> info_;
};

}  // namespace io
}  // namespace q4t
