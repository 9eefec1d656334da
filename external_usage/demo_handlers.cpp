// Native version of demo_handlers.py.  A server loads this library when the job config names
// "libdemo_handlers.so" as update_file / filter_file and resolves the functions by name.
//
// ABI (paracel_b200/csrc/core/ps_server.hpp): values travel as msgpack byte strings;
//   int update(old, old_n, delta, delta_n, &out, &out_n)   returns 0 and a malloc'ed result
//   int filter(key, key_n, val, val_n)                      returns non-zero to keep the entry
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>

#include "msgpack_lite.hpp"

extern "C" int add_counts(const char* old_p, size_t old_n, const char* delta_p, size_t delta_n,
                          char** out_p, size_t* out_n) {
  try {
    pcl::Value a = pcl::unpack_value(std::string(old_p, old_n));
    pcl::Value b = pcl::unpack_value(std::string(delta_p, delta_n));
    const std::string r = pcl::pack_value(pcl::Value::integer(a.as_int() + b.as_int()));
    *out_p = (char*)std::malloc(r.size());
    std::memcpy(*out_p, r.data(), r.size());
    *out_n = r.size();
    return 0;
  } catch (...) {
    return 1;
  }
}

extern "C" int length_keys(const char* key_p, size_t key_n, const char*, size_t) {
  return key_n >= 4 && std::memcmp(key_p, "len_", 4) == 0;
}
