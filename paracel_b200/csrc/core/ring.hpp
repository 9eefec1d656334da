// Hashing and the consistent-hash ring that places string keys on servers.
//
// Same construction as the reference (include/ring.hpp:35-98,
// include/utils/hash.hpp:37-92): every server contributes 32 virtual nodes
// "<name>:<i>" hashed with std::hash<std::string>; a key goes to the first
// virtual node whose hash is >= the key's hash (wrapping to the first node).
// Because std::hash is the C++ library's, placements agree with a reference
// build made with the same standard library.
#pragma once
#include <algorithm>
#include <cstdint>
#include <functional>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

namespace pcl {

inline uint64_t hash_string(const std::string& s) { return (uint64_t)std::hash<std::string>()(s); }
inline uint64_t hash_u64(uint64_t x) { return (uint64_t)std::hash<uint64_t>()(x); }
inline uint64_t hash_double(double x) { return (uint64_t)std::hash<double>()(x); }

inline uint64_t hash_value_combine(uint64_t x, uint64_t y) {
  const uint64_t kMul = 0x9ddfea08eb382d69ULL;
  uint64_t a = (x ^ y) * kMul;
  a ^= (a >> 47);
  uint64_t b = (y ^ a) * kMul;
  b ^= (b >> 47);
  b *= kMul;
  return b;
}

// hash of a list: the items are streamed after the tag "vechash" and the string is hashed
inline uint64_t hash_string_list(const std::vector<std::string>& items) {
  std::string buf("vechash");
  for (auto& s : items) buf.append(s);
  return hash_string(buf);
}

inline size_t ring_bsearch(const std::vector<uint64_t>& data, uint64_t key) {
  if (data.empty()) return 0;
  if (key < data.front() || key > data.back()) return 0;
  return (size_t)(std::lower_bound(data.begin(), data.end(), key) - data.begin());
}

class Ring {
 public:
  explicit Ring(int replicas = 32) : replicas_(replicas) {}
  void add_server(const std::string& name) {
    for (int i = 0; i < replicas_; ++i) {
      uint64_t k = hash_string(name + ":" + std::to_string(i));
      owner_[k] = name;
      ring_.push_back(k);
    }
    std::sort(ring_.begin(), ring_.end());
  }
  void remove_server(const std::string& name) {
    for (int i = 0; i < replicas_; ++i) {
      uint64_t k = hash_string(name + ":" + std::to_string(i));
      owner_.erase(k);
      auto it = std::find(ring_.begin(), ring_.end(), k);
      if (it != ring_.end()) ring_.erase(it);
    }
  }
  const std::string& get_server_by_hash(uint64_t h) const {
    return owner_.at(ring_[ring_bsearch(ring_, h)]);
  }
  const std::string& get_server(const std::string& key) const {
    return get_server_by_hash(hash_string(key));
  }
  size_t size() const { return ring_.size(); }

 private:
  int replicas_;
  std::vector<uint64_t> ring_;
  std::unordered_map<uint64_t, std::string> owner_;
};

}  // namespace pcl
