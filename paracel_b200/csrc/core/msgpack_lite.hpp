// Minimal msgpack codec used by the host-side parameter server.
//
// Values on the CPU parameter server are opaque msgpack byte strings, exactly
// as in the reference (include/packer.hpp:39-75 packs every value with
// msgpack-c; include/kv_def.hpp:24 stores string -> string).  The server only
// has to look inside a value when a built-in update handler combines an old
// value with a delta, so this codec covers the msgpack subset that handlers
// need: nil, bool, integers, float32/64, str, bin, array and map.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace pcl {

struct Value {
  enum Type { NIL, BOOL, INT, UINT, FLOAT, STR, BIN, ARR, MAP };
  Type t = NIL;
  bool b = false;
  int64_t i = 0;
  uint64_t u = 0;
  double f = 0.0;
  std::string s;
  std::vector<Value> a;
  std::vector<std::pair<Value, Value>> m;

  static Value nil() { return Value(); }
  static Value boolean(bool x) { Value v; v.t = BOOL; v.b = x; return v; }
  static Value integer(int64_t x) { Value v; v.t = INT; v.i = x; return v; }
  static Value uinteger(uint64_t x) { Value v; v.t = UINT; v.u = x; return v; }
  static Value real(double x) { Value v; v.t = FLOAT; v.f = x; return v; }
  static Value str(std::string x) { Value v; v.t = STR; v.s = std::move(x); return v; }
  static Value bin(std::string x) { Value v; v.t = BIN; v.s = std::move(x); return v; }
  static Value array() { Value v; v.t = ARR; return v; }
  static Value map() { Value v; v.t = MAP; return v; }

  bool is_number() const { return t == INT || t == UINT || t == FLOAT; }
  bool is_integer() const { return t == INT || t == UINT; }
  double as_double() const {
    switch (t) {
      case INT: return (double)i;
      case UINT: return (double)u;
      case FLOAT: return f;
      case BOOL: return b ? 1.0 : 0.0;
      default: throw std::runtime_error("msgpack value is not a number");
    }
  }
  int64_t as_int() const {
    switch (t) {
      case INT: return i;
      case UINT: return (int64_t)u;
      case FLOAT: return (int64_t)f;
      case BOOL: return b ? 1 : 0;
      default: throw std::runtime_error("msgpack value is not an integer");
    }
  }
};

class Packer {
 public:
  std::string out;

  void pack(const Value& v) {
    switch (v.t) {
      case Value::NIL: put8(0xc0); break;
      case Value::BOOL: put8(v.b ? 0xc3 : 0xc2); break;
      case Value::INT: pack_int(v.i); break;
      case Value::UINT: pack_uint(v.u); break;
      case Value::FLOAT: pack_double(v.f); break;
      case Value::STR: pack_str(v.s); break;
      case Value::BIN: pack_bin(v.s); break;
      case Value::ARR:
        pack_array_header(v.a.size());
        for (auto& x : v.a) pack(x);
        break;
      case Value::MAP:
        pack_map_header(v.m.size());
        for (auto& kv : v.m) { pack(kv.first); pack(kv.second); }
        break;
    }
  }
  void pack_nil() { put8(0xc0); }
  void pack_bool(bool b) { put8(b ? 0xc3 : 0xc2); }
  void pack_uint(uint64_t u) {
    if (u < 128) put8((uint8_t)u);
    else if (u <= 0xff) { put8(0xcc); put8((uint8_t)u); }
    else if (u <= 0xffff) { put8(0xcd); put_be<uint16_t>((uint16_t)u); }
    else if (u <= 0xffffffffULL) { put8(0xce); put_be<uint32_t>((uint32_t)u); }
    else { put8(0xcf); put_be<uint64_t>(u); }
  }
  void pack_int(int64_t i) {
    if (i >= 0) { pack_uint((uint64_t)i); return; }
    if (i >= -32) put8((uint8_t)(int8_t)i);
    else if (i >= -128) { put8(0xd0); put8((uint8_t)(int8_t)i); }
    else if (i >= -32768) { put8(0xd1); put_be<uint16_t>((uint16_t)(int16_t)i); }
    else if (i >= -2147483648LL) { put8(0xd2); put_be<uint32_t>((uint32_t)(int32_t)i); }
    else { put8(0xd3); put_be<uint64_t>((uint64_t)i); }
  }
  void pack_double(double d) {
    uint64_t bits;
    std::memcpy(&bits, &d, 8);
    put8(0xcb);
    put_be<uint64_t>(bits);
  }
  void pack_str(const std::string& s) {
    size_t n = s.size();
    if (n < 32) put8((uint8_t)(0xa0 | n));
    else if (n <= 0xff) { put8(0xd9); put8((uint8_t)n); }
    else if (n <= 0xffff) { put8(0xda); put_be<uint16_t>((uint16_t)n); }
    else { put8(0xdb); put_be<uint32_t>((uint32_t)n); }
    out.append(s);
  }
  void pack_bin(const std::string& s) {
    size_t n = s.size();
    if (n <= 0xff) { put8(0xc4); put8((uint8_t)n); }
    else if (n <= 0xffff) { put8(0xc5); put_be<uint16_t>((uint16_t)n); }
    else { put8(0xc6); put_be<uint32_t>((uint32_t)n); }
    out.append(s);
  }
  void pack_array_header(size_t n) {
    if (n < 16) put8((uint8_t)(0x90 | n));
    else if (n <= 0xffff) { put8(0xdc); put_be<uint16_t>((uint16_t)n); }
    else { put8(0xdd); put_be<uint32_t>((uint32_t)n); }
  }
  void pack_map_header(size_t n) {
    if (n < 16) put8((uint8_t)(0x80 | n));
    else if (n <= 0xffff) { put8(0xde); put_be<uint16_t>((uint16_t)n); }
    else { put8(0xdf); put_be<uint32_t>((uint32_t)n); }
  }

 private:
  void put8(uint8_t x) { out.push_back((char)x); }
  template <class T>
  void put_be(T x) {
    for (int k = (int)sizeof(T) - 1; k >= 0; --k) out.push_back((char)((x >> (8 * k)) & 0xff));
  }
};

class Unpacker {
 public:
  Unpacker(const char* p, size_t n) : p_((const uint8_t*)p), end_((const uint8_t*)p + n) {}
  explicit Unpacker(const std::string& s) : Unpacker(s.data(), s.size()) {}

  bool done() const { return p_ >= end_; }

  Value next() {
    uint8_t c = get8();
    if (c < 0x80) return Value::integer(c);
    if (c >= 0xe0) return Value::integer((int8_t)c);
    if (c >= 0xa0 && c <= 0xbf) return Value::str(take(c & 0x1f));
    if (c >= 0x90 && c <= 0x9f) return arr(c & 0x0f);
    if (c >= 0x80 && c <= 0x8f) return map(c & 0x0f);
    switch (c) {
      case 0xc0: return Value::nil();
      case 0xc2: return Value::boolean(false);
      case 0xc3: return Value::boolean(true);
      case 0xc4: return Value::bin(take(get8()));
      case 0xc5: return Value::bin(take(be<uint16_t>()));
      case 0xc6: return Value::bin(take(be<uint32_t>()));
      case 0xca: { uint32_t b = be<uint32_t>(); float f; std::memcpy(&f, &b, 4); return Value::real(f); }
      case 0xcb: { uint64_t b = be<uint64_t>(); double d; std::memcpy(&d, &b, 8); return Value::real(d); }
      case 0xcc: return Value::integer(get8());
      case 0xcd: return Value::integer(be<uint16_t>());
      case 0xce: return Value::integer(be<uint32_t>());
      case 0xcf: {
        uint64_t u = be<uint64_t>();
        if (u > 0x7fffffffffffffffULL) return Value::uinteger(u);
        return Value::integer((int64_t)u);
      }
      case 0xd0: return Value::integer((int8_t)get8());
      case 0xd1: return Value::integer((int16_t)be<uint16_t>());
      case 0xd2: return Value::integer((int32_t)be<uint32_t>());
      case 0xd3: return Value::integer((int64_t)be<uint64_t>());
      case 0xd9: return Value::str(take(get8()));
      case 0xda: return Value::str(take(be<uint16_t>()));
      case 0xdb: return Value::str(take(be<uint32_t>()));
      case 0xdc: return arr(be<uint16_t>());
      case 0xdd: return arr(be<uint32_t>());
      case 0xde: return map(be<uint16_t>());
      case 0xdf: return map(be<uint32_t>());
      default: throw std::runtime_error("unsupported msgpack type byte");
    }
  }

 private:
  const uint8_t* p_;
  const uint8_t* end_;
  uint8_t get8() {
    if (p_ >= end_) throw std::runtime_error("msgpack: truncated input");
    return *p_++;
  }
  template <class T>
  T be() {
    if ((size_t)(end_ - p_) < sizeof(T)) throw std::runtime_error("msgpack: truncated input");
    T x = 0;
    for (size_t k = 0; k < sizeof(T); ++k) x = (T)((x << 8) | *p_++);
    return x;
  }
  std::string take(size_t n) {
    if ((size_t)(end_ - p_) < n) throw std::runtime_error("msgpack: truncated input");
    std::string s((const char*)p_, n);
    p_ += n;
    return s;
  }
  Value arr(size_t n) {
    Value v = Value::array();
    v.a.reserve(n);
    for (size_t k = 0; k < n; ++k) v.a.push_back(next());
    return v;
  }
  Value map(size_t n) {
    Value v = Value::map();
    v.m.reserve(n);
    for (size_t k = 0; k < n; ++k) {
      Value key = next();
      Value val = next();
      v.m.emplace_back(std::move(key), std::move(val));
    }
    return v;
  }
};

inline std::string pack_value(const Value& v) {
  Packer p;
  p.pack(v);
  return std::move(p.out);
}

inline Value unpack_value(const std::string& s) {
  Unpacker u(s);
  return u.next();
}

}  // namespace pcl
