// In-memory key/value table of one parameter-server shard.
//
// Operation set and return conventions follow the reference's kvs<K,V>
// (include/kv.hpp:29-173): contains, set, set_multi, get (optional / bool
// form), get_multi (strict list form throws on a missing key, dict form skips
// missing keys), incr for numbers and equal-length sequences, gets + cas with a
// content hash as the version, del, clean, getall.  Unlike the reference the
// table carries its own reader/writer lock, so concurrent pulls never observe
// a half-written value (the reference answers pulls outside its global mutex,
// include/server.hpp:237-264 vs 311).
#pragma once
#include <functional>
#include <optional>
#include <shared_mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace pcl {

template <class K, class V>
class KVS {
 public:
  bool contains(const K& k) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    return d_.count(k) != 0;
  }
  void set(const K& k, const V& v) {
    std::unique_lock<std::shared_mutex> g(mu_);
    d_[k] = v;
  }
  void set_multi(const std::vector<std::pair<K, V>>& kvs) {
    std::unique_lock<std::shared_mutex> g(mu_);
    for (auto& kv : kvs) d_[kv.first] = kv.second;
  }
  std::optional<V> get(const K& k) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    auto it = d_.find(k);
    if (it == d_.end()) return std::nullopt;
    return it->second;
  }
  bool get(const K& k, V& v) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    auto it = d_.find(k);
    if (it == d_.end()) return false;
    v = it->second;
    return true;
  }
  // strict form: every key must exist
  std::vector<V> get_multi(const std::vector<K>& keys) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    std::vector<V> out;
    out.reserve(keys.size());
    for (auto& k : keys) {
      auto it = d_.find(k);
      if (it == d_.end()) throw std::out_of_range("get_multi: missing key");
      out.push_back(it->second);
    }
    return out;
  }
  // tolerant form: only the keys that exist
  std::vector<std::pair<K, V>> get_multi_existing(const std::vector<K>& keys) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    std::vector<std::pair<K, V>> out;
    for (auto& k : keys) {
      auto it = d_.find(k);
      if (it != d_.end()) out.emplace_back(k, it->second);
    }
    return out;
  }
  // read-modify-write under the table lock; f(old_or_null) -> new
  template <class F>
  V update(const K& k, F&& f) {
    std::unique_lock<std::shared_mutex> g(mu_);
    auto it = d_.find(k);
    if (it == d_.end()) {
      V nv = f(nullptr);
      d_[k] = nv;
      return nv;
    }
    V nv = f(&it->second);
    it->second = nv;
    return nv;
  }
  std::optional<std::pair<V, size_t>> gets(const K& k) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    auto it = d_.find(k);
    if (it == d_.end()) return std::nullopt;
    return std::make_pair(it->second, std::hash<V>()(it->second));
  }
  bool cas(const K& k, const V& v, size_t uniq) {
    std::unique_lock<std::shared_mutex> g(mu_);
    auto it = d_.find(k);
    if (it == d_.end()) {
      d_[k] = v;
      return true;
    }
    if (std::hash<V>()(it->second) != uniq) return false;
    it->second = v;
    return true;
  }
  bool del(const K& k) {
    std::unique_lock<std::shared_mutex> g(mu_);
    return d_.erase(k) != 0;
  }
  void clean() {
    std::unique_lock<std::shared_mutex> g(mu_);
    d_.clear();
  }
  std::vector<std::pair<K, V>> getall() const {
    std::shared_lock<std::shared_mutex> g(mu_);
    return std::vector<std::pair<K, V>>(d_.begin(), d_.end());
  }
  template <class P>
  std::vector<std::pair<K, V>> getall_if(P&& pred) const {
    std::shared_lock<std::shared_mutex> g(mu_);
    std::vector<std::pair<K, V>> out;
    for (auto& kv : d_)
      if (pred(kv.first, kv.second)) out.push_back(kv);
    return out;
  }
  template <class P>
  size_t del_if(P&& pred) {
    std::unique_lock<std::shared_mutex> g(mu_);
    size_t n = 0;
    for (auto it = d_.begin(); it != d_.end();) {
      if (pred(it->first, it->second)) { it = d_.erase(it); ++n; }
      else ++it;
    }
    return n;
  }
  size_t size() const {
    std::shared_lock<std::shared_mutex> g(mu_);
    return d_.size();
  }

 private:
  mutable std::shared_mutex mu_;
  std::unordered_map<K, V> d_;
};

}  // namespace pcl
