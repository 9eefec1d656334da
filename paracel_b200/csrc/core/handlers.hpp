// Built-in update handlers of the host parameter server, selected by name.
//
// The reference loads user handlers from a shared object with dlopen and calls
// them through update_proxy on msgpack strings (include/server.hpp:177-191,
// include/proxy.hpp:56-73).  The handlers it ships fall into a few kinds, which
// are implemented here directly on msgpack values:
//   add        numbers, equal-shape (nested) sequences, and maps merged by
//              adding values (default_incr_*, lr/ridge theta update, mf_*,
//              cnt_updater, svd_updater, gLDA word/topic/sum updates, k-means
//              cluster sums, word-count dictionary merge)
//   max / min  scalars (max_updater)
//   concat     list append (PageRank init_updater)
//   map_concat map of lists, lists appended per key (k-means groups)
//   dict_index map word -> dense id, unseen words get the next id (gLDA dict)
//   min_pair   keep the pair with the smaller second element (decision tree)
//   replace    last writer wins
// Anything else is a Python callable or a C-ABI function from a user .so.
#pragma once
#include <algorithm>
#include <map>
#include <string>

#include "msgpack_lite.hpp"

namespace pcl {

inline Value add_values(const Value& a, const Value& b) {
  if (a.is_number() && b.is_number()) {
    if (a.is_integer() && b.is_integer()) return Value::integer(a.as_int() + b.as_int());
    return Value::real(a.as_double() + b.as_double());
  }
  if (a.t == Value::ARR && b.t == Value::ARR) {
    if (a.a.size() != b.a.size()) throw std::runtime_error("add handler: length mismatch");
    Value r = Value::array();
    r.a.reserve(a.a.size());
    for (size_t i = 0; i < a.a.size(); ++i) r.a.push_back(add_values(a.a[i], b.a[i]));
    return r;
  }
  if (a.t == Value::MAP && b.t == Value::MAP) {
    Value r = a;
    for (auto& kv : b.m) {
      std::string kb = pack_value(kv.first);
      bool found = false;
      for (auto& rk : r.m) {
        if (pack_value(rk.first) == kb) { rk.second = add_values(rk.second, kv.second); found = true; break; }
      }
      if (!found) r.m.push_back(kv);
    }
    return r;
  }
  throw std::runtime_error("add handler: unsupported value types");
}

// map merge with hashing (large dictionaries: word count)
inline Value add_maps_fast(const Value& a, const Value& b) {
  std::unordered_map<std::string, size_t> idx;
  Value r = a;
  idx.reserve(r.m.size() + b.m.size());
  for (size_t i = 0; i < r.m.size(); ++i) idx[pack_value(r.m[i].first)] = i;
  for (auto& kv : b.m) {
    std::string kb = pack_value(kv.first);
    auto it = idx.find(kb);
    if (it == idx.end()) { idx[kb] = r.m.size(); r.m.push_back(kv); }
    else r.m[it->second].second = add_values(r.m[it->second].second, kv.second);
  }
  return r;
}

enum class HandlerKind { ADD, MAX, MIN, CONCAT, MAP_CONCAT, DICT_INDEX, MIN_PAIR, REPLACE, UNKNOWN };

inline HandlerKind handler_kind(const std::string& name) {
  static const std::map<std::string, HandlerKind> table = {
      {"add", HandlerKind::ADD}, {"default_incr_i", HandlerKind::ADD},
      {"default_incr_f", HandlerKind::ADD}, {"default_incr_d", HandlerKind::ADD},
      {"default_incr_li", HandlerKind::ADD}, {"default_incr_lf", HandlerKind::ADD},
      {"default_incr_ld", HandlerKind::ADD}, {"lr_theta_update", HandlerKind::ADD},
      {"ridge_theta_update", HandlerKind::ADD}, {"cnt_updater", HandlerKind::ADD},
      {"mf_fac_updater", HandlerKind::ADD}, {"mf_bias_updater", HandlerKind::ADD},
      {"svd_updater", HandlerKind::ADD}, {"gLDA_topic_update", HandlerKind::ADD},
      {"gLDA_word_update", HandlerKind::ADD}, {"gLDA_sum_topic_update", HandlerKind::ADD},
      {"local_update_kmeans_clusters", HandlerKind::ADD}, {"wc_updater", HandlerKind::ADD},
      {"wc_updater_slow", HandlerKind::ADD}, {"local_update", HandlerKind::ADD},
      {"max", HandlerKind::MAX}, {"max_updater", HandlerKind::MAX}, {"min", HandlerKind::MIN},
      {"concat", HandlerKind::CONCAT}, {"init_updater", HandlerKind::CONCAT},
      {"map_concat", HandlerKind::MAP_CONCAT},
      {"local_update_kmeans_groups", HandlerKind::MAP_CONCAT},
      {"dict_index", HandlerKind::DICT_INDEX}, {"gLDA_dict_update", HandlerKind::DICT_INDEX},
      {"min_pair", HandlerKind::MIN_PAIR}, {"smallest_error_updater", HandlerKind::MIN_PAIR},
      {"replace", HandlerKind::REPLACE},
  };
  auto it = table.find(name);
  return it == table.end() ? HandlerKind::UNKNOWN : it->second;
}

inline std::string apply_builtin(HandlerKind k, const std::string& old_packed,
                                 const std::string& delta_packed) {
  if (k == HandlerKind::REPLACE) return delta_packed;
  Value a = unpack_value(old_packed), b = unpack_value(delta_packed);
  switch (k) {
    case HandlerKind::ADD:
      if (a.t == Value::MAP && b.t == Value::MAP) return pack_value(add_maps_fast(a, b));
      return pack_value(add_values(a, b));
    case HandlerKind::MAX:
      return a.as_double() >= b.as_double() ? old_packed : delta_packed;
    case HandlerKind::MIN:
      return a.as_double() <= b.as_double() ? old_packed : delta_packed;
    case HandlerKind::CONCAT: {
      if (a.t != Value::ARR || b.t != Value::ARR) throw std::runtime_error("concat: not lists");
      a.a.insert(a.a.end(), b.a.begin(), b.a.end());
      return pack_value(a);
    }
    case HandlerKind::MAP_CONCAT: {
      if (a.t != Value::MAP || b.t != Value::MAP) throw std::runtime_error("map_concat: not maps");
      for (auto& kv : b.m) {
        std::string kb = pack_value(kv.first);
        bool found = false;
        for (auto& rk : a.m) {
          if (pack_value(rk.first) == kb) {
            rk.second.a.insert(rk.second.a.end(), kv.second.a.begin(), kv.second.a.end());
            found = true;
            break;
          }
        }
        if (!found) a.m.push_back(kv);
      }
      return pack_value(a);
    }
    case HandlerKind::DICT_INDEX: {
      if (a.t != Value::MAP || b.t != Value::MAP) throw std::runtime_error("dict_index: not maps");
      std::unordered_map<std::string, bool> seen;
      for (auto& kv : a.m) seen[pack_value(kv.first)] = true;
      int64_t next = (int64_t)a.m.size();
      for (auto& kv : b.m) {
        std::string kb = pack_value(kv.first);
        if (!seen.count(kb)) {
          seen[kb] = true;
          a.m.emplace_back(kv.first, Value::integer(next++));
        }
      }
      return pack_value(a);
    }
    case HandlerKind::MIN_PAIR: {
      if (a.t != Value::ARR || b.t != Value::ARR || a.a.size() < 2 || b.a.size() < 2)
        throw std::runtime_error("min_pair: not pairs");
      return a.a[1].as_double() <= b.a[1].as_double() ? old_packed : delta_packed;
    }
    default: throw std::runtime_error("unknown builtin handler");
  }
}

}  // namespace pcl
