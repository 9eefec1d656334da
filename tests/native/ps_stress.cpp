// Concurrency stress of the host parameter server and its store, meant to be built with
// -fsanitize=thread or -fsanitize=address (tests/test_cpu_sanitizers.py does both).
// Eight client threads hammer one TCP server with bupdate (add handler), push, pull,
// contains and SSP clock requests on overlapping keys; the main thread checks the sums.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include "ps_server.hpp"

using namespace pcl;

static std::string req(const std::string& op, const std::vector<Value>& args) {
  Packer p;
  p.pack_array_header(1 + args.size());
  p.pack_str(op);
  for (auto& a : args) p.pack(a);
  return p.out;
}

static Value reply_body(const std::string& rep) {
  Unpacker u(rep);
  Value r = u.next();
  if (r.t != Value::ARR || r.a.size() != 2) { std::fprintf(stderr, "bad reply\n"); std::exit(2); }
  if (r.a[0].as_int() == ST_ERROR) { std::fprintf(stderr, "server error: %s\n", r.a[1].s.c_str()); std::exit(2); }
  return r.a[1];
}

int main() {
  const int kThreads = 8, kIters = 400, kKeys = 16;
  PsServer srv;
  const int port = srv.start("127.0.0.1", 0);
  if (port <= 0) { std::fprintf(stderr, "cannot start server\n"); return 2; }
  {
    PsConnection c("127.0.0.1", port, 10.0);
    reply_body(c.request(req("ssp_reset", {Value::integer(kThreads)})));
  }
  std::vector<std::thread> ths;
  for (int t = 0; t < kThreads; ++t) {
    ths.emplace_back([&, t] {
      PsConnection c("127.0.0.1", port, 10.0);
      for (int it = 0; it < kIters; ++it) {
        const std::string key = "k" + std::to_string((t + it) % kKeys);
        // bupdate with the built-in integer add handler; a missing key behaves as a write
        reply_body(c.request(req("bupdate", {Value::str(key), Value::bin(pack_value(Value::integer(1))),
                                             Value::str(""), Value::str("default_incr_i")})));
        reply_body(c.request(req("push", {Value::str("own" + std::to_string(t)),
                                          Value::bin(pack_value(Value::integer(it)))})));
        reply_body(c.request(req("contains", {Value::str(key)})));
        c.request(req("pull", {Value::str("k" + std::to_string(it % kKeys))}));
        if (it % 50 == 49) reply_body(c.request(req("ssp_commit", {Value::integer(it / 50)})));
      }
    });
  }
  for (auto& th : ths) th.join();
  long total = 0;
  {
    PsConnection c("127.0.0.1", port, 10.0);
    for (int k = 0; k < kKeys; ++k) {
      Value v = reply_body(c.request(req("pull", {Value::str("k" + std::to_string(k))})));
      total += (long)unpack_value(v.s).as_int();
    }
    Value clk = reply_body(c.request(req("pull_int", {Value::str("server_clock")})));
    if (clk.as_int() != kIters / 50) { std::fprintf(stderr, "server_clock %ld\n", (long)clk.as_int()); return 3; }
  }
  srv.stop();
  if (total != (long)kThreads * kIters) { std::fprintf(stderr, "lost updates: %ld\n", total); return 3; }
  std::printf("ok %ld\n", total);
  return 0;
}
