// Host-side parameter server daemon and its client connection.
//
// Role: the CPU backend of the framework (the plumbing configuration "2 workers
// + 1 parameter server on CPU", the oracle for the GPU tables, and the home of
// values that are not fixed-width rows: dictionaries, lists of pairs, graphs).
// It keeps the reference's operation table (include/server.hpp:232-397: contains,
// pull, pull_multi, pull_multi_check, pullall, pullall_special, register_*,
// push, push_multi, update, bupdate, bupdate_multi, remove, remove_special,
// clear, and push_int / incr_int / pull_int on the SSP table) and its rule that
// an update of a missing key stores the delta (server.hpp:88-100).
//
// What is different by design: one TCP listener and a length-prefixed msgpack
// array per request instead of five ZeroMQ REP sockets and "_PARACEL_"-joined
// fields; every request gets a reply (the reference never answers
// register_update, server.hpp:299-303); handlers are resolved once per
// (file, function) pair instead of a dlopen per request (server.hpp:336-339);
// the SSP clock counts each commit exactly once (the reference counts it twice,
// server.hpp:136-151) and advances when every still-running worker has
// committed that clock.
#pragma once
#include <arpa/inet.h>
#include <dlfcn.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <thread>

#include "handlers.hpp"
#include "kv.hpp"

namespace pcl {

inline bool send_all(int fd, const char* p, size_t n) {
  while (n > 0) {
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k <= 0) return false;
    p += k;
    n -= (size_t)k;
  }
  return true;
}

inline bool recv_all(int fd, char* p, size_t n) {
  while (n > 0) {
    ssize_t k = ::recv(fd, p, n, 0);
    if (k <= 0) return false;
    p += k;
    n -= (size_t)k;
  }
  return true;
}

inline bool send_frame(int fd, const std::string& body) {
  uint64_t n = body.size();
  char hdr[8];
  for (int i = 0; i < 8; ++i) hdr[i] = (char)((n >> (8 * i)) & 0xff);
  return send_all(fd, hdr, 8) && send_all(fd, body.data(), body.size());
}

inline bool recv_frame(int fd, std::string& body) {
  char hdr[8];
  if (!recv_all(fd, hdr, 8)) return false;
  uint64_t n = 0;
  for (int i = 0; i < 8; ++i) n |= ((uint64_t)(uint8_t)hdr[i]) << (8 * i);
  if (n > (1ULL << 36)) return false;
  body.resize(n);
  return n == 0 || recv_all(fd, &body[0], n);
}

// C ABI of a user handler in a shared object: returns 0 on success and a
// malloc'ed result that the server frees.
typedef int (*c_update_fn)(const char* old_p, size_t old_n, const char* delta_p, size_t delta_n,
                           char** out_p, size_t* out_n);
typedef int (*c_filter_fn)(const char* key_p, size_t key_n, const char* val_p, size_t val_n);

using py_update_cb = std::function<std::string(const std::string& file, const std::string& func,
                                               const std::string& old_v, const std::string& delta)>;
using py_filter_cb = std::function<bool(const std::string& file, const std::string& func,
                                        const std::string& key, const std::string& val)>;

enum Status { ST_OK = 0, ST_NOKEY = 1, ST_ERROR = 2 };

class PsServer {
 public:
  PsServer() {}
  ~PsServer() { stop(); }

  py_update_cb py_update;
  py_filter_cb py_filter;

  int start(const std::string& host, int port) {
    listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (listen_fd_ < 0) throw std::runtime_error("socket() failed");
    int one = 1;
    setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    if (host.empty() || host == "*" || host == "0.0.0.0") addr.sin_addr.s_addr = INADDR_ANY;
    else if (inet_pton(AF_INET, host.c_str(), &addr.sin_addr) != 1)
      throw std::runtime_error("bad listen address " + host);
    if (::bind(listen_fd_, (sockaddr*)&addr, sizeof(addr)) != 0)
      throw std::runtime_error("bind() failed");
    if (::listen(listen_fd_, 256) != 0) throw std::runtime_error("listen() failed");
    socklen_t len = sizeof(addr);
    getsockname(listen_fd_, (sockaddr*)&addr, &len);
    port_ = ntohs(addr.sin_port);
    running_ = true;
    acceptor_ = std::thread([this] { accept_loop(); });
    return port_;
  }

  int port() const { return port_; }
  bool running() const { return running_; }

  void stop() {
    bool was = running_.exchange(false);
    if (!was) return;
    ::shutdown(listen_fd_, SHUT_RDWR);
    ::close(listen_fd_);
    if (acceptor_.joinable()) acceptor_.join();
    std::vector<std::thread> ths;
    {
      std::lock_guard<std::mutex> g(conn_mu_);
      for (int fd : conn_fds_) ::shutdown(fd, SHUT_RDWR);
      ths.swap(conn_threads_);
    }
    for (auto& t : ths)
      if (t.joinable()) t.join();
    done_cv_.notify_all();
  }

  // blocks until a client sends "shutdown" or stop() is called
  void wait() {
    std::unique_lock<std::mutex> g(done_mu_);
    done_cv_.wait(g, [this] { return !running_ || shutdown_requested_; });
  }
  bool wait_for(double seconds) {
    std::unique_lock<std::mutex> g(done_mu_);
    return done_cv_.wait_for(g, std::chrono::duration<double>(seconds),
                             [this] { return !running_ || shutdown_requested_; });
  }

  size_t size() const { return store_.size(); }
  KVS<std::string, std::string>& store() { return store_; }

  // ---- request execution (also callable in-process, without sockets)
  std::string execute(const std::string& req) {
    Packer out;
    try {
      Unpacker u(req);
      Value r = u.next();
      if (r.t != Value::ARR || r.a.empty() || r.a[0].t != Value::STR)
        throw std::runtime_error("malformed request");
      dispatch(r, out);
    } catch (const std::exception& e) {
      Packer err;
      err.pack_array_header(2);
      err.pack_int(ST_ERROR);
      err.pack_str(e.what());
      return std::move(err.out);
    }
    return std::move(out.out);
  }

 private:
  struct Resolved {
    HandlerKind kind = HandlerKind::UNKNOWN;
    c_update_fn cfn = nullptr;
    std::string file, func;
  };

  void accept_loop() {
    while (running_) {
      int fd = ::accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) {
        if (!running_) break;
        continue;
      }
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::lock_guard<std::mutex> g(conn_mu_);
      conn_fds_.push_back(fd);
      conn_threads_.emplace_back([this, fd] { serve(fd); });
    }
  }

  void serve(int fd) {
    std::string req;
    while (running_ && recv_frame(fd, req)) {
      std::string rep = execute(req);
      if (!send_frame(fd, rep)) break;
    }
    ::close(fd);
    std::lock_guard<std::mutex> g(conn_mu_);
    conn_fds_.erase(std::remove(conn_fds_.begin(), conn_fds_.end(), fd), conn_fds_.end());
  }

  static void ok_header(Packer& out) { out.pack_array_header(2); out.pack_int(ST_OK); }

  Resolved resolve_update(const Value& r, size_t file_idx) {
    std::string file, func;
    if (r.a.size() > file_idx + 1) { file = r.a[file_idx].s; func = r.a[file_idx + 1].s; }
    if (func.empty()) {
      std::lock_guard<std::mutex> g(reg_mu_);
      file = reg_update_file_;
      func = reg_update_func_;
    }
    if (func.empty()) func = "default_incr_i";  // same fallback family as server.hpp:341-344 (add)
    std::string key = file + "\n" + func;
    {
      std::lock_guard<std::mutex> g(reg_mu_);
      auto it = resolved_.find(key);
      if (it != resolved_.end()) return it->second;
    }
    Resolved res;
    res.file = file;
    res.func = func;
    res.kind = handler_kind(func);
    bool is_so = file.size() > 3 && file.compare(file.size() - 3, 3, ".so") == 0;
    if (is_so) {
      void* h = dlopen(file.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (h != nullptr) {
        void* sym = dlsym(h, func.c_str());
        if (sym != nullptr) {
          res.cfn = (c_update_fn)sym;
          res.kind = HandlerKind::UNKNOWN;
        }
      }
      if (res.cfn == nullptr && res.kind == HandlerKind::UNKNOWN)
        throw std::runtime_error("cannot load handler " + func + " from " + file);
    }
    std::lock_guard<std::mutex> g(reg_mu_);
    resolved_[key] = res;
    return res;
  }

  std::string apply_update(const Resolved& h, const std::string& old_v, const std::string& delta) {
    if (h.cfn != nullptr) {
      char* out_p = nullptr;
      size_t out_n = 0;
      int rc = h.cfn(old_v.data(), old_v.size(), delta.data(), delta.size(), &out_p, &out_n);
      if (rc != 0) throw std::runtime_error("user handler returned an error");
      std::string r(out_p, out_n);
      free(out_p);
      return r;
    }
    if (h.kind != HandlerKind::UNKNOWN) return apply_builtin(h.kind, old_v, delta);
    if (py_update) return py_update(h.file, h.func, old_v, delta);
    throw std::runtime_error("no handler named " + h.func);
  }

  std::string kv_update(const std::string& key, const std::string& delta, const Resolved& h) {
    return store_.update(key, [&](const std::string* old_v) {
      if (old_v == nullptr) return delta;  // first update of a missing key stores the delta
      return apply_update(h, *old_v, delta);
    });
  }

  bool run_filter(const std::string& file, const std::string& func, const std::string& k,
                  const std::string& v) {
    // "prefix:xyz" / "suffix:xyz" / "contains:xyz" and the filters shipped with the reference
    static const std::map<std::string, std::pair<int, std::string>> named = {
        {"mf_ubias_filter", {0, "usr_bias_"}}, {"mf_ibias_filter", {0, "item_bias_"}},
        {"mf_W_filter", {0, "W_"}}, {"mf_H_filter", {0, "H_"}},
        {"mf_cntx_filter", {1, "_u_cnt"}}, {"mf_cnty_filter", {1, "_i_cnt"}},
        {"pr_filter", {1, "_pr"}}, {"wc_filter", {0, "key_"}}, {"gLDA_dump_filter", {0, "key_"}},
    };
    int mode = -1;
    std::string pat;
    auto it = named.find(func);
    if (it != named.end()) { mode = it->second.first; pat = it->second.second; }
    else if (func.rfind("prefix:", 0) == 0) { mode = 0; pat = func.substr(7); }
    else if (func.rfind("suffix:", 0) == 0) { mode = 1; pat = func.substr(7); }
    else if (func.rfind("contains:", 0) == 0) { mode = 2; pat = func.substr(9); }
    if (mode == 0) return k.compare(0, pat.size(), pat) == 0;
    if (mode == 1) return k.size() >= pat.size() && k.compare(k.size() - pat.size(), pat.size(), pat) == 0;
    if (mode == 2) return k.find(pat) != std::string::npos;
    bool is_so = file.size() > 3 && file.compare(file.size() - 3, 3, ".so") == 0;
    if (is_so) {
      void* h = dlopen(file.c_str(), RTLD_NOW | RTLD_LOCAL);
      void* sym = h ? dlsym(h, func.c_str()) : nullptr;
      if (sym) return ((c_filter_fn)sym)(k.data(), k.size(), v.data(), v.size()) != 0;
      throw std::runtime_error("cannot load filter " + func + " from " + file);
    }
    if (py_filter) return py_filter(file, func, k, v);
    throw std::runtime_error("no filter named " + func);
  }

  static void pack_kv_map(Packer& out, const std::vector<std::pair<std::string, std::string>>& kvs) {
    out.pack_map_header(kvs.size());
    for (auto& kv : kvs) { out.pack_str(kv.first); out.pack_bin(kv.second); }
  }

  void ssp_advance_locked() {
    while (worker_sz_ > 0) {
      auto it = commits_.find(server_clock_);
      if (it == commits_.end() || it->second < worker_sz_) break;
      commits_.erase(it);
      ++server_clock_;
    }
  }

  void dispatch(const Value& r, Packer& out) {
    const std::string& op = r.a[0].s;
    auto need = [&](size_t n) {
      if (r.a.size() < n + 1) throw std::runtime_error("op " + op + ": missing arguments");
    };
    if (op == "contains") {
      need(1);
      ok_header(out);
      out.pack_bool(store_.contains(r.a[1].s));
    } else if (op == "pull") {
      need(1);
      std::string v;
      if (!store_.get(r.a[1].s, v)) {
        out.pack_array_header(2); out.pack_int(ST_NOKEY); out.pack_nil();
      } else {
        ok_header(out);
        out.pack_bin(v);
      }
    } else if (op == "pull_multi") {
      need(1);
      std::vector<std::string> keys;
      for (auto& k : r.a[1].a) keys.push_back(k.s);
      std::vector<std::string> vals;
      try {
        vals = store_.get_multi(keys);
      } catch (const std::out_of_range&) {
        out.pack_array_header(2); out.pack_int(ST_NOKEY); out.pack_nil();
        return;
      }
      ok_header(out);
      out.pack_array_header(vals.size());
      for (auto& v : vals) out.pack_bin(v);
    } else if (op == "pull_multi_check") {
      need(1);
      std::vector<std::string> keys;
      for (auto& k : r.a[1].a) keys.push_back(k.s);
      auto kvs = store_.get_multi_existing(keys);
      ok_header(out);
      pack_kv_map(out, kvs);
    } else if (op == "pullall") {
      ok_header(out);
      pack_kv_map(out, store_.getall());
    } else if (op == "pullall_special") {
      std::string file, func;
      if (r.a.size() >= 3) { file = r.a[1].s; func = r.a[2].s; }
      else { std::lock_guard<std::mutex> g(reg_mu_); file = reg_pullall_file_; func = reg_pullall_func_; }
      auto kvs = store_.getall();
      std::vector<std::pair<std::string, std::string>> sel;
      for (auto& kv : kvs)
        if (run_filter(file, func, kv.first, kv.second)) sel.push_back(kv);
      ok_header(out);
      pack_kv_map(out, sel);
    } else if (op == "register_pullall_special" || op == "register_remove_special" ||
               op == "register_update" || op == "register_bupdate") {
      need(2);
      std::lock_guard<std::mutex> g(reg_mu_);
      if (op == "register_pullall_special") { reg_pullall_file_ = r.a[1].s; reg_pullall_func_ = r.a[2].s; }
      else if (op == "register_remove_special") { reg_remove_file_ = r.a[1].s; reg_remove_func_ = r.a[2].s; }
      else { reg_update_file_ = r.a[1].s; reg_update_func_ = r.a[2].s; }
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "push") {
      need(2);
      store_.set(r.a[1].s, r.a[2].s);
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "push_multi") {
      need(2);
      if (r.a[1].a.size() != r.a[2].a.size()) throw std::runtime_error("push_multi: size mismatch");
      std::vector<std::pair<std::string, std::string>> kvs;
      for (size_t i = 0; i < r.a[1].a.size(); ++i) kvs.emplace_back(r.a[1].a[i].s, r.a[2].a[i].s);
      store_.set_multi(kvs);
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "update" || op == "bupdate") {
      need(2);
      Resolved h = resolve_update(r, 3);
      std::string nv = kv_update(r.a[1].s, r.a[2].s, h);
      ok_header(out);
      out.pack_bin(nv);
    } else if (op == "bupdate_multi") {
      need(2);
      if (r.a[1].a.size() != r.a[2].a.size()) throw std::runtime_error("bupdate_multi: size mismatch");
      Resolved h = resolve_update(r, 3);
      std::vector<std::string> nvs;
      for (size_t i = 0; i < r.a[1].a.size(); ++i)
        nvs.push_back(kv_update(r.a[1].a[i].s, r.a[2].a[i].s, h));
      ok_header(out);
      out.pack_array_header(nvs.size());
      for (auto& v : nvs) out.pack_bin(v);
    } else if (op == "remove") {
      need(1);
      ok_header(out);
      out.pack_bool(store_.del(r.a[1].s));
    } else if (op == "remove_special") {
      std::string file, func;
      if (r.a.size() >= 3) { file = r.a[1].s; func = r.a[2].s; }
      else { std::lock_guard<std::mutex> g(reg_mu_); file = reg_remove_file_; func = reg_remove_func_; }
      auto kvs = store_.getall();
      for (auto& kv : kvs)
        if (run_filter(file, func, kv.first, kv.second)) store_.del(kv.first);
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "clear") {
      store_.clean();
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "size") {
      ok_header(out);
      out.pack_int((int64_t)store_.size());
    } else if (op == "push_int") {
      need(2);
      std::lock_guard<std::mutex> g(ssp_mu_);
      ints_[r.a[1].s] = r.a[2].as_int();
      if (r.a[1].s == "worker_sz") { worker_sz_ = r.a[2].as_int(); ssp_advance_locked(); }
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "incr_int") {
      need(2);
      std::lock_guard<std::mutex> g(ssp_mu_);
      ints_[r.a[1].s] += r.a[2].as_int();
      if (r.a[1].s == "worker_sz") { worker_sz_ = ints_[r.a[1].s]; ssp_advance_locked(); }
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "pull_int") {
      need(1);
      std::lock_guard<std::mutex> g(ssp_mu_);
      if (r.a[1].s == "server_clock") { ok_header(out); out.pack_int(server_clock_); return; }
      auto it = ints_.find(r.a[1].s);
      if (it == ints_.end()) { out.pack_array_header(2); out.pack_int(ST_NOKEY); out.pack_nil(); }
      else { ok_header(out); out.pack_int(it->second); }
    } else if (op == "ssp_commit") {  // [clock that the worker has just finished]
      need(1);
      std::lock_guard<std::mutex> g(ssp_mu_);
      ++commits_[r.a[1].as_int()];
      ssp_advance_locked();
      ok_header(out);
      out.pack_int(server_clock_);
    } else if (op == "ssp_depart") {
      std::lock_guard<std::mutex> g(ssp_mu_);
      if (worker_sz_ > 0) --worker_sz_;
      ints_["worker_sz"] = worker_sz_;
      ssp_advance_locked();
      ok_header(out);
      out.pack_int(server_clock_);
    } else if (op == "ssp_reset") {
      std::lock_guard<std::mutex> g(ssp_mu_);
      commits_.clear();
      server_clock_ = 0;
      if (r.a.size() > 1) { worker_sz_ = r.a[1].as_int(); ints_["worker_sz"] = worker_sz_; }
      ok_header(out);
      out.pack_bool(true);
    } else if (op == "ping") {
      ok_header(out);
      out.pack_str("pong");
    } else if (op == "shutdown") {
      {
        std::lock_guard<std::mutex> g(done_mu_);
        shutdown_requested_ = true;
      }
      done_cv_.notify_all();
      ok_header(out);
      out.pack_bool(true);
    } else {
      throw std::runtime_error("unknown op " + op);
    }
  }

  KVS<std::string, std::string> store_;
  int listen_fd_ = -1;
  int port_ = 0;
  std::atomic<bool> running_{false};
  std::thread acceptor_;
  std::mutex conn_mu_;
  std::vector<int> conn_fds_;
  std::vector<std::thread> conn_threads_;
  std::mutex reg_mu_;
  std::string reg_update_file_, reg_update_func_, reg_pullall_file_, reg_pullall_func_,
      reg_remove_file_, reg_remove_func_;
  std::map<std::string, Resolved> resolved_;
  std::mutex ssp_mu_;
  std::map<std::string, int64_t> ints_;
  std::map<int64_t, int64_t> commits_;
  int64_t worker_sz_ = 0;
  int64_t server_clock_ = 0;
  std::mutex done_mu_;
  std::condition_variable done_cv_;
  bool shutdown_requested_ = false;
};

// Rendezvous of the launcher with freshly started servers (the role of the reference's
// paracelrun_cpp_proxy, src/paracelrun_cpp_proxy.cpp:23-35 and include/utils.hpp:58-77):
// listen on `port`, accept `n` connections, read one "host:port" line from each, answer
// "done", and return the lines.  Gives up after `timeout_s`.
inline std::vector<std::string> collect_endpoints(const std::string& host, int port, int n,
                                                  double timeout_s, int* bound_port = nullptr,
                                                  std::function<void(int)> on_listening = nullptr) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) throw std::runtime_error("socket() failed");
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_port = htons((uint16_t)port);
  if (host.empty() || host == "*") addr.sin_addr.s_addr = INADDR_ANY;
  else inet_pton(AF_INET, host.c_str(), &addr.sin_addr);
  if (::bind(fd, (sockaddr*)&addr, sizeof(addr)) != 0 || ::listen(fd, 64) != 0) {
    ::close(fd);
    throw std::runtime_error("rendezvous: cannot listen on port " + std::to_string(port));
  }
  socklen_t len = sizeof(addr);
  getsockname(fd, (sockaddr*)&addr, &len);
  if (bound_port) *bound_port = ntohs(addr.sin_port);
  if (on_listening) on_listening(ntohs(addr.sin_port));
  timeval tv;
  tv.tv_sec = (long)timeout_s;
  tv.tv_usec = (long)((timeout_s - (long)timeout_s) * 1e6);
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  std::vector<std::string> out;
  for (int i = 0; i < n; ++i) {
    int c = ::accept(fd, nullptr, nullptr);
    if (c < 0) {
      ::close(fd);
      throw std::runtime_error("rendezvous: only " + std::to_string(i) + " of " + std::to_string(n) +
                               " servers reported in time");
    }
    setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    std::string line;
    char ch;
    while (::recv(c, &ch, 1, 0) == 1 && ch != '\n') line.push_back(ch);
    send_all(c, "done", 4);
    ::close(c);
    out.push_back(line);
  }
  ::close(fd);
  return out;
}

// Blocking request/reply connection to one server.
class PsConnection {
 public:
  PsConnection(const std::string& host, int port, double timeout_s = 0.0) {
    fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) throw std::runtime_error("socket() failed");
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons((uint16_t)port);
    std::string h = (host == "localhost" || host.empty()) ? "127.0.0.1" : host;
    if (inet_pton(AF_INET, h.c_str(), &addr.sin_addr) != 1) {
      ::close(fd_);
      throw std::runtime_error("bad server address " + host);
    }
    if (timeout_s > 0) {
      timeval tv;
      tv.tv_sec = (long)timeout_s;
      tv.tv_usec = (long)((timeout_s - (long)timeout_s) * 1e6);
      setsockopt(fd_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
      setsockopt(fd_, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    }
    if (::connect(fd_, (sockaddr*)&addr, sizeof(addr)) != 0) {
      ::close(fd_);
      fd_ = -1;
      throw std::runtime_error("connect() to " + h + ":" + std::to_string(port) + " failed");
    }
    int one = 1;
    setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  }
  ~PsConnection() { close(); }
  void close() {
    if (fd_ >= 0) { ::close(fd_); fd_ = -1; }
  }
  std::string request(const std::string& req) {
    std::lock_guard<std::mutex> g(mu_);
    if (fd_ < 0) throw std::runtime_error("connection closed");
    if (!send_frame(fd_, req)) throw std::runtime_error("send to parameter server failed");
    std::string rep;
    if (!recv_frame(fd_, rep)) throw std::runtime_error("no reply from parameter server (timeout or closed)");
    return rep;
  }

 private:
  int fd_ = -1;
  std::mutex mu_;
};

}  // namespace pcl
