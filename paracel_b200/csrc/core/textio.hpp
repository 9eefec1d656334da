// File partitioning and line parsing for the distributed loaders.
//
// Behaviour kept from the reference (include/load/partition.hpp:57-229): the
// corpus is the concatenation of all input files, it is cut into np * blk_sz
// byte ranges of equal size (the last one takes the remainder), and a line
// belongs to the range that holds its first byte, so no line is lost or read
// twice whatever np is.  The implementation is new: ranges are resolved per
// file with pread-style buffered reads, lines crossing a range end are
// finished by the range that started them, and a file boundary always ends a
// line (the reference stops at the first empty line when it crosses files).
#pragma once
#include <sys/stat.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

namespace pcl {

inline long file_size(const std::string& name) {
  struct stat st;
  if (stat(name.c_str(), &st) != 0) throw std::runtime_error("cannot stat " + name);
  return (long)st.st_size;
}

struct FilePartition {
  std::vector<std::string> names;
  std::vector<long> displs;  // cumulative sizes, names.size() + 1 entries
  std::vector<long> starts, ends;

  FilePartition(const std::vector<std::string>& n, int np, int blk_sz) : names(n) {
    displs.assign(names.size() + 1, 0);
    for (size_t i = 0; i < names.size(); ++i) displs[i + 1] = displs[i] + file_size(names[i]);
    long sz = displs.back();
    long nbk = (long)np * blk_sz;
    if (nbk <= 0) throw std::runtime_error("partition: np * blk_sz must be positive");
    long bk = sz / nbk;
    for (long i = 0; i < nbk; ++i) {
      long s = i * bk;
      long e = (i == nbk - 1) ? sz : (i + 1) * bk;
      starts.push_back(s);
      ends.push_back(e);
    }
  }

  // lines whose first byte lies in [st, en) of the concatenated corpus
  template <class F>
  void for_each_line(long st, long en, F&& func) const {
    if (st >= en) return;
    for (size_t fi = 0; fi < names.size(); ++fi) {
      long f0 = displs[fi], f1 = displs[fi + 1];
      if (f1 <= st || f0 >= en || f1 == f0) continue;
      long lo = (st > f0 ? st : f0) - f0;  // local offsets
      long hi = (en < f1 ? en : f1) - f0;
      read_range(names[fi], lo, hi, f1 - f0, func);
    }
  }

 private:
  template <class F>
  static void read_range(const std::string& name, long lo, long hi, long fsz, F&& func) {
    FILE* f = std::fopen(name.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + name);
    std::vector<char> buf(1 << 20);
    long pos = lo;
    bool skipping = false;
    if (lo > 0) {
      // the line that contains byte lo-1 belongs to an earlier range unless lo-1 is '\n'
      std::fseek(f, lo - 1, SEEK_SET);
      int c = std::fgetc(f);
      skipping = (c != '\n');
    } else {
      std::fseek(f, 0, SEEK_SET);
    }
    std::string cur;
    bool in_line = false;  // cur holds a line that started inside [lo, hi)
    bool done = false;
    while (!done && pos < fsz) {
      size_t want = (size_t)std::min<long>((long)buf.size(), fsz - pos);
      size_t got = std::fread(buf.data(), 1, want, f);
      if (got == 0) break;
      for (size_t k = 0; k < got; ++k) {
        char c = buf[k];
        long at = pos + (long)k;
        if (skipping) {
          if (c == '\n') skipping = false;
          continue;
        }
        if (!in_line) {
          if (at >= hi) { done = true; break; }
          in_line = true;
          cur.clear();
        }
        if (c == '\n') {
          if (!cur.empty() && cur.back() == '\r') cur.pop_back();
          func(cur);
          in_line = false;
        } else {
          cur.push_back(c);
        }
      }
      pos += (long)got;
    }
    if (in_line) {  // last line of the file without a trailing newline
      if (!cur.empty() && cur.back() == '\r') cur.pop_back();
      func(cur);
    }
    std::fclose(f);
  }
};

inline std::vector<std::string> split_char(const std::string& s, char sep) {
  // consecutive separators do not produce empty fields (paracel::str_split semantics)
  std::vector<std::string> out;
  size_t i = 0, n = s.size();
  while (i < n) {
    while (i < n && s[i] == sep) ++i;
    size_t j = i;
    while (j < n && s[j] != sep) ++j;
    if (j > i) out.emplace_back(s, i, j - i);
    i = j;
  }
  return out;
}

inline std::vector<std::string> split_any(const std::string& s, const std::string& seps) {
  std::vector<std::string> out;
  size_t i = 0, n = s.size();
  while (i < n) {
    while (i < n && seps.find(s[i]) != std::string::npos) ++i;
    size_t j = i;
    while (j < n && seps.find(s[j]) == std::string::npos) ++j;
    if (j > i) out.emplace_back(s, i, j - i);
    i = j;
  }
  return out;
}

struct Triples {
  std::vector<uint64_t> a, b;
  std::vector<double> w;
  std::vector<int32_t> slot;
};

// Numeric fast path of the loader's line organiser (include/load/scheduler.hpp:107-156):
// 2 fields "a b" or "a b:0.2"; with mix, an adjacency list "a b c" / "a b|0.2 c|0.4";
// otherwise exactly 3 fields "a b w".  Destination slot = (a % npx) * npy + b % npy,
// which is what the reference's hash gives for integer ids.
inline void organize_numeric(const std::vector<std::string>& fields, bool mix, int npx, int npy,
                             Triples& out) {
  auto emit = [&](uint64_t a, uint64_t b, double w) {
    out.a.push_back(a);
    out.b.push_back(b);
    out.w.push_back(w);
    out.slot.push_back((int32_t)((a % (uint64_t)npx) * (uint64_t)npy + b % (uint64_t)npy));
  };
  auto item = [&](uint64_t a, const std::string& it) {
    auto tmp = split_any(it, ":| ");
    if (tmp.size() == 1) emit(a, std::strtoull(tmp[0].c_str(), nullptr, 10), 1.0);
    else if (tmp.size() >= 2)
      emit(a, std::strtoull(tmp[0].c_str(), nullptr, 10), std::strtod(tmp[1].c_str(), nullptr));
  };
  if (fields.size() < 2) return;
  uint64_t a = std::strtoull(fields[0].c_str(), nullptr, 10);
  if (fields.size() == 2) {
    item(a, fields[1]);
  } else if (mix) {
    for (size_t i = 1; i < fields.size(); ++i) item(a, fields[i]);
  } else {
    if (fields.size() != 3) throw std::runtime_error("lines_organize: unsupported line format");
    emit(a, std::strtoull(fields[1].c_str(), nullptr, 10), std::strtod(fields[2].c_str(), nullptr));
  }
}

}  // namespace pcl
