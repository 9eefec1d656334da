// pybind11 module `_pcl_core`: host runtime of paracel_b200.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "balltree.hpp"
#include "cpu_algos.hpp"
#include "handlers.hpp"
#include "kv.hpp"
#include "msgpack_lite.hpp"
#include "ps_server.hpp"
#include "ring.hpp"
#include "textio.hpp"

namespace py = pybind11;
using namespace pcl;

namespace {

template <class T>
py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a((py::ssize_t)v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

using StrKV = KVS<std::string, std::string>;

}  // namespace

PYBIND11_MODULE(_pcl_core, m) {
  m.doc() = "paracel_b200 host runtime: KV store, parameter server, ring, loaders, ball tree";

  // ---- hashing / ring
  m.def("hash_string", [](const std::string& s) { return hash_string(s); });
  m.def("hash_bytes", [](py::bytes b) { return hash_string(std::string(b)); });
  m.def("hash_u64", &hash_u64);
  m.def("hash_double", &hash_double);
  m.def("hash_value_combine", &hash_value_combine);
  m.def("hash_string_list", &hash_string_list);
  m.def("ring_bsearch", &ring_bsearch);
  py::class_<Ring>(m, "Ring")
      .def(py::init<int>(), py::arg("replicas") = 32)
      .def("add_server", &Ring::add_server)
      .def("remove_server", &Ring::remove_server)
      .def("get_server", &Ring::get_server)
      .def("get_server_by_hash", &Ring::get_server_by_hash)
      .def("__len__", &Ring::size);

  // ---- KV store (bytes -> bytes)
  py::class_<StrKV>(m, "KVStore")
      .def(py::init<>())
      .def("contains", [](StrKV& s, const std::string& k) { return s.contains(k); })
      .def("set", [](StrKV& s, const std::string& k, py::bytes v) { s.set(k, std::string(v)); })
      .def("set_multi", [](StrKV& s, const std::map<std::string, py::bytes>& d) {
        std::vector<std::pair<std::string, std::string>> kvs;
        for (auto& kv : d) kvs.emplace_back(kv.first, std::string(kv.second));
        s.set_multi(kvs);
      })
      .def("get", [](StrKV& s, const std::string& k) -> py::object {
        auto v = s.get(k);
        if (!v) return py::none();
        return py::bytes(*v);
      })
      .def("get_multi", [](StrKV& s, const std::vector<std::string>& keys) {
        py::list out;
        for (auto& v : s.get_multi(keys)) out.append(py::bytes(v));
        return out;
      })
      .def("get_multi_existing", [](StrKV& s, const std::vector<std::string>& keys) {
        py::dict out;
        for (auto& kv : s.get_multi_existing(keys)) out[py::str(kv.first)] = py::bytes(kv.second);
        return out;
      })
      .def("incr", [](StrKV& s, const std::string& k, py::bytes delta) {
        // numbers and equal-length sequences; false when the key is missing or shapes differ
        if (!s.contains(k)) return false;
        std::string d(delta);
        try {
          s.update(k, [&](const std::string* old_v) { return apply_builtin(HandlerKind::ADD, *old_v, d); });
        } catch (const std::exception&) {
          return false;
        }
        return true;
      })
      .def("gets", [](StrKV& s, const std::string& k) -> py::object {
        auto r = s.gets(k);
        if (!r) return py::none();
        return py::make_tuple(py::bytes(r->first), r->second);
      })
      .def("cas", [](StrKV& s, const std::string& k, py::bytes v, size_t uniq) {
        return s.cas(k, std::string(v), uniq);
      })
      .def("delete", [](StrKV& s, const std::string& k) { return s.del(k); })
      .def("clean", &StrKV::clean)
      .def("getall", [](StrKV& s) {
        py::dict out;
        for (auto& kv : s.getall()) out[py::str(kv.first)] = py::bytes(kv.second);
        return out;
      })
      .def("__len__", &StrKV::size);

  // ---- built-in handlers on packed values
  m.def("handler_is_builtin", [](const std::string& name) {
    return handler_kind(name) != HandlerKind::UNKNOWN;
  });
  m.def("apply_builtin_handler", [](const std::string& name, py::bytes old_v, py::bytes delta) {
    HandlerKind k = handler_kind(name);
    if (k == HandlerKind::UNKNOWN) throw std::runtime_error("no built-in handler named " + name);
    return py::bytes(apply_builtin(k, std::string(old_v), std::string(delta)));
  });

  // ---- parameter server daemon
  py::class_<PsServer>(m, "PsServer")
      .def(py::init<>())
      .def("start", &PsServer::start, py::arg("host") = "127.0.0.1", py::arg("port") = 0)
      .def("stop", &PsServer::stop, py::call_guard<py::gil_scoped_release>())
      .def("wait", &PsServer::wait, py::call_guard<py::gil_scoped_release>())
      .def("wait_for", &PsServer::wait_for, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("port", &PsServer::port)
      .def_property_readonly("running", &PsServer::running)
      .def("__len__", &PsServer::size)
      .def("execute", [](PsServer& s, py::bytes req) {
        std::string r(req), out;
        {
          py::gil_scoped_release rel;
          out = s.execute(r);
        }
        return py::bytes(out);
      })
      .def("set_python_update", [](PsServer& s, py::function f) {
        auto fp = std::make_shared<py::function>(std::move(f));
        s.py_update = [fp](const std::string& file, const std::string& func,
                           const std::string& old_v, const std::string& delta) {
          py::gil_scoped_acquire g;
          py::object r = (*fp)(file, func, py::bytes(old_v), py::bytes(delta));
          return std::string(py::bytes(r));
        };
      })
      .def("set_python_filter", [](PsServer& s, py::function f) {
        auto fp = std::make_shared<py::function>(std::move(f));
        s.py_filter = [fp](const std::string& file, const std::string& func,
                           const std::string& k, const std::string& v) {
          py::gil_scoped_acquire g;
          return (*fp)(file, func, k, py::bytes(v)).cast<bool>();
        };
      });

  m.def("collect_endpoints", [](const std::string& host, int port, int n, double timeout_s,
                                py::object on_listening) {
    std::function<void(int)> cb = nullptr;
    if (!on_listening.is_none()) {
      auto fp = std::make_shared<py::object>(on_listening);
      cb = [fp](int p) { py::gil_scoped_acquire g; (*fp)(p); };
    }
    std::vector<std::string> out;
    {
      py::gil_scoped_release rel;
      out = collect_endpoints(host, port, n, timeout_s, nullptr, cb);
    }
    return out;
  }, py::arg("host"), py::arg("port"), py::arg("n"), py::arg("timeout_s") = 60.0,
     py::arg("on_listening") = py::none());

  py::class_<PsConnection>(m, "PsConnection")
      .def(py::init<const std::string&, int, double>(), py::arg("host"), py::arg("port"),
           py::arg("timeout_s") = 0.0)
      .def("close", &PsConnection::close)
      .def("request", [](PsConnection& c, py::bytes req) {
        std::string r(req), out;
        {
          py::gil_scoped_release rel;
          out = c.request(r);
        }
        return py::bytes(out);
      });

  // ---- file partition / parsing
  py::class_<FilePartition>(m, "FilePartition")
      .def(py::init<const std::vector<std::string>&, int, int>(), py::arg("names"), py::arg("np"),
           py::arg("blk_sz") = 1)
      .def_readonly("starts", &FilePartition::starts)
      .def_readonly("ends", &FilePartition::ends)
      .def_readonly("displs", &FilePartition::displs)
      .def("load_lines", [](const FilePartition& p, long st, long en) {
        std::vector<std::string> lines;
        {
          py::gil_scoped_release rel;
          p.for_each_line(st, en, [&](const std::string& l) { lines.push_back(l); });
        }
        return lines;
      })
      .def("load_blocks", [](const FilePartition& p, int first_blk, int last_blk) {
        std::vector<std::string> lines;
        {
          py::gil_scoped_release rel;
          for (int b = first_blk; b < last_blk; ++b)
            p.for_each_line(p.starts[b], p.ends[b], [&](const std::string& l) { lines.push_back(l); });
        }
        return lines;
      })
      // numeric triples straight from the byte ranges: (a, b, w, slot) arrays
      .def("load_triples", [](const FilePartition& p, int first_blk, int last_blk, const std::string& seps,
                              bool mix, int npx, int npy, std::vector<int> drop_fields) {
        Triples t;
        {
          py::gil_scoped_release rel;
          for (int b = first_blk; b < last_blk; ++b)
            p.for_each_line(p.starts[b], p.ends[b], [&](const std::string& l) {
              if (l.empty()) return;
              auto f = split_any(l, seps);
              if (!drop_fields.empty()) {
                std::vector<std::string> g;
                for (size_t i = 0; i < f.size(); ++i)
                  if (std::find(drop_fields.begin(), drop_fields.end(), (int)i) == drop_fields.end())
                    g.push_back(f[i]);
                f.swap(g);
              }
              organize_numeric(f, mix, npx, npy, t);
            });
        }
        return py::make_tuple(to_array(t.a), to_array(t.b), to_array(t.w), to_array(t.slot));
      }, py::arg("first_blk"), py::arg("last_blk"), py::arg("seps") = " ", py::arg("mix") = false,
         py::arg("npx") = 1, py::arg("npy") = 1, py::arg("drop_fields") = std::vector<int>());
  m.def("split_char", &split_char);
  m.def("split_any", &split_any);
  m.def("organize_numeric", [](const std::vector<std::vector<std::string>>& rows, bool mix, int npx, int npy) {
    Triples t;
    for (auto& f : rows) organize_numeric(f, mix, npx, npy, t);
    return py::make_tuple(to_array(t.a), to_array(t.b), to_array(t.w), to_array(t.slot));
  });
  // dense rows "f1,f2,...,fk" -> (n, k) float64 array
  m.def("parse_dense_rows", [](const std::vector<std::string>& lines, const std::string& seps) {
    std::vector<double> vals;
    long n = 0, k = -1;
    for (auto& l : lines) {
      if (l.empty()) continue;
      auto f = split_any(l, seps);
      if (k < 0) k = (long)f.size();
      if ((long)f.size() != k) throw std::runtime_error("parse_dense_rows: ragged rows");
      for (auto& s : f) vals.push_back(std::strtod(s.c_str(), nullptr));
      ++n;
    }
    if (k < 0) k = 0;
    py::array_t<double> a({(py::ssize_t)n, (py::ssize_t)k});
    if (!vals.empty()) std::memcpy(a.mutable_data(), vals.data(), vals.size() * sizeof(double));
    return a;
  });

  // ---- sequential CPU kernels
  using darr = py::array_t<double, py::array::c_style>;
  using iarr = py::array_t<int64_t, py::array::c_style>;
  using i32arr = py::array_t<int32_t, py::array::c_style>;
  m.def("linear_sgd_pass", [](darr X, darr y, iarr idx, darr theta, darr delta, double alpha,
                              double beta, bool logistic, bool accumulate) {
    long dim = (long)X.shape(1), n = (long)idx.size();
    if ((long)theta.size() != dim || (long)delta.size() != dim) throw std::runtime_error("bad theta size");
    const double *Xp = X.data(), *yp = y.data();
    const int64_t* ip = idx.data();
    double *tp = theta.mutable_data(), *dp = delta.mutable_data();
    py::gil_scoped_release rel;
    linear_sgd_pass(Xp, yp, dim, ip, n, tp, dp, alpha, beta, logistic, accumulate);
  });
  m.def("logloss_sum", [](darr X, darr y, darr theta) {
    return logloss_sum(X.data(), y.data(), (long)X.shape(1), (long)X.shape(0), theta.data());
  });
  m.def("mf_sgd_pass", [](iarr u, iarr it, darr r, darr W, darr H, darr bu, darr bi, double mu,
                          double alpha, double beta) {
    const int64_t *up = u.data(), *ip = it.data();
    const double* rp = r.data();
    long nnz = (long)u.size(), k = (long)W.shape(1);
    double *Wp = W.mutable_data(), *Hp = H.mutable_data(), *bup = bu.mutable_data(),
           *bip = bi.mutable_data();
    py::gil_scoped_release rel;
    mf_sgd_pass(up, ip, rp, nnz, k, Wp, Hp, bup, bip, mu, alpha, beta);
  });
  m.def("lda_gibbs_sweep", [](iarr doc_ptr, i32arr words, i32arr z, i32arr doc_topic,
                              i32arr word_topic, i32arr topic_sum, i32arr doc_len, long K, long V,
                              double alpha, double beta, uint64_t seed) {
    const int64_t* dp = doc_ptr.data();
    long nd = (long)doc_ptr.size() - 1;
    const int32_t *wp = words.data(), *dl = doc_len.data();
    int32_t *zp = z.mutable_data(), *dt = doc_topic.mutable_data(), *wt = word_topic.mutable_data(),
            *ts = topic_sum.mutable_data();
    py::gil_scoped_release rel;
    lda_gibbs_sweep(dp, nd, wp, zp, dt, wt, ts, dl, K, V, alpha, beta, seed);
  });
  m.def("shooting_steps", [](py::array_t<double, py::array::f_style> Xc, darr y, darr W, darr z,
                             double lambda, long steps, bool logistic, uint64_t seed) {
    const double *xp = Xc.data(), *yp = y.data();
    long n = (long)Xc.shape(0), k = (long)Xc.shape(1);
    double *wp = W.mutable_data(), *zp = z.mutable_data();
    py::gil_scoped_release rel;
    shooting_steps(xp, yp, n, k, wp, zp, lambda, steps, logistic, seed);
  });

  // ---- ball tree
  py::class_<BallTree>(m, "BallTree")
      .def(py::init([](py::array_t<double, py::array::c_style | py::array::forcecast> items, int limit) {
        if (items.ndim() != 2) throw std::runtime_error("BallTree: items must be 2-D");
        std::vector<double> d(items.data(), items.data() + items.size());
        return new BallTree(std::move(d), (long)items.shape(0), (int)items.shape(1), limit);
      }), py::arg("items"), py::arg("limit") = 20)
      .def("build", &BallTree::build, py::call_guard<py::gil_scoped_release>())
      .def("pickle", &BallTree::pickle)
      .def("unpickle", &BallTree::unpickle)
      .def("build_from_file", &BallTree::unpickle)
      .def_property_readonly("node_count", &BallTree::node_count)
      .def_property_readonly("last_visited", &BallTree::last_visited)
      .def("search", [](const BallTree& t, const std::vector<double>& q, int k,
                        const std::unordered_set<long>& black, const std::unordered_set<long>& white) {
        std::vector<std::pair<long, double>> out;
        for (auto& h : t.search(q, k, black, white)) out.emplace_back(h.id, h.score);
        return out;
      }, py::arg("q"), py::arg("k") = 1, py::arg("black_list") = std::unordered_set<long>(),
         py::arg("white_list") = std::unordered_set<long>())
      .def("brute_force", [](const BallTree& t, const std::vector<double>& q, int k,
                             const std::unordered_set<long>& black, const std::unordered_set<long>& white) {
        std::vector<std::pair<long, double>> out;
        for (auto& h : t.brute_force(q, k, black, white)) out.emplace_back(h.id, h.score);
        return out;
      }, py::arg("q"), py::arg("k") = 1, py::arg("black_list") = std::unordered_set<long>(),
         py::arg("white_list") = std::unordered_set<long>())
      .def("export_arrays", [](const BallTree& t) {
        // flat arrays for the GPU search: centres (nodes x dim), radius, children, ranges, order
        const auto& nd = t.nodes();
        std::vector<double> mu, rad;
        std::vector<int32_t> child;
        std::vector<int64_t> range, order(t.order().begin(), t.order().end());
        for (auto& n : nd) {
          mu.insert(mu.end(), n.mu.begin(), n.mu.end());
          rad.push_back(n.radius);
          child.push_back(n.left);
          child.push_back(n.right);
          range.push_back(n.begin);
          range.push_back(n.end);
        }
        return py::make_tuple(to_array(mu), to_array(rad), to_array(child), to_array(range), to_array(order));
      });
}
