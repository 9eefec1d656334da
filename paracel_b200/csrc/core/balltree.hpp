// Ball tree for maximum-inner-product search (MIPS).
//
// Feature parity with the reference tool (tool/balltree/balltree.hpp:179-650):
// build with a leaf limit (default 20) by splitting on the two mutually
// farthest points, text pickle / unpickle, top-k search by branch and bound
// with the bound  q.mu + |q| * radius  (balltree.hpp:405-409), optional black
// and white lists of item ids, and a brute-force search for checking.
// The node pool is a flat vector (indices instead of pointers) so the tree can
// be copied to a GPU as three arrays.
#pragma once
#include <algorithm>
#include <cmath>
#include <fstream>
#include <limits>
#include <numeric>
#include <queue>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_set>
#include <vector>

namespace pcl {

struct BallNode {
  int left = -1, right = -1;   // children, -1 for a leaf
  long begin = 0, end = 0;     // range in `order` (leaf items)
  double radius = 0.0;
  std::vector<double> mu;
};

class BallTree {
 public:
  BallTree(std::vector<double> data, long n, int dim, int limit = 20)
      : x_(std::move(data)), n_(n), dim_(dim), limit_(limit) {
    if ((long)x_.size() != n * dim) throw std::runtime_error("balltree: bad data size");
  }

  void build() {
    nodes_.clear();
    order_.resize(n_);
    std::iota(order_.begin(), order_.end(), 0L);
    if (n_ > 0) build_rec(0, n_);
  }

  long size() const { return n_; }
  int dim() const { return dim_; }
  size_t node_count() const { return nodes_.size(); }
  const std::vector<BallNode>& nodes() const { return nodes_; }
  const std::vector<long>& order() const { return order_; }
  const std::vector<double>& data() const { return x_; }

  struct Hit { long id; double score; };

  // top-k by inner product; returns hits sorted by decreasing score
  std::vector<Hit> search(const std::vector<double>& q, int k,
                          const std::unordered_set<long>& black = {},
                          const std::unordered_set<long>& white = {}) const {
    if ((int)q.size() != dim_) throw std::runtime_error("balltree: bad query size");
    Heap heap;
    visited_ = 0;
    if (!nodes_.empty() && k > 0) {
      double qn = norm(q.data());
      search_rec(0, q.data(), qn, k, black, white, heap);
    }
    return drain(heap);
  }

  std::vector<Hit> brute_force(const std::vector<double>& q, int k,
                               const std::unordered_set<long>& black = {},
                               const std::unordered_set<long>& white = {}) const {
    Heap heap;
    for (long i = 0; i < n_; ++i) consider(i, q.data(), k, black, white, heap);
    return drain(heap);
  }

  long last_visited() const { return visited_; }

  // text pickle: header line, then one node per line in pre-order
  void pickle(const std::string& fn) const {
    std::ofstream os(fn);
    os.precision(17);
    os << n_ << ' ' << dim_ << ' ' << limit_ << ' ' << nodes_.size() << '\n';
    for (auto& nd : nodes_) {
      os << nd.left << ' ' << nd.right << ' ' << nd.begin << ' ' << nd.end << ' ' << nd.radius;
      for (double v : nd.mu) os << ' ' << v;
      os << '\n';
    }
    for (long i = 0; i < n_; ++i) os << order_[i] << (i + 1 == n_ ? '\n' : ' ');
  }

  void unpickle(const std::string& fn) {
    std::ifstream is(fn);
    if (!is) throw std::runtime_error("balltree: cannot open " + fn);
    long n; int dim, limit; size_t nn;
    is >> n >> dim >> limit >> nn;
    if (n != n_ || dim != dim_) throw std::runtime_error("balltree: pickle does not match the items");
    limit_ = limit;
    nodes_.assign(nn, BallNode());
    for (auto& nd : nodes_) {
      is >> nd.left >> nd.right >> nd.begin >> nd.end >> nd.radius;
      nd.mu.resize(dim_);
      for (auto& v : nd.mu) is >> v;
    }
    order_.resize(n_);
    for (auto& o : order_) is >> o;
  }

 private:
  struct Cmp { bool operator()(const Hit& a, const Hit& b) const { return a.score > b.score; } };
  using Heap = std::priority_queue<Hit, std::vector<Hit>, Cmp>;  // min-heap on score

  const double* row(long i) const { return x_.data() + i * dim_; }
  double norm(const double* a) const {
    double s = 0;
    for (int d = 0; d < dim_; ++d) s += a[d] * a[d];
    return std::sqrt(s);
  }
  double dot(const double* a, const double* b) const {
    double s = 0;
    for (int d = 0; d < dim_; ++d) s += a[d] * b[d];
    return s;
  }
  double dist(const double* a, const double* b) const {
    double s = 0;
    for (int d = 0; d < dim_; ++d) { double t = a[d] - b[d]; s += t * t; }
    return std::sqrt(s);
  }
  long farthest(const double* from, long b, long e) const {
    long best = order_[b];
    double bd = -1;
    for (long k = b; k < e; ++k) {
      double d = dist(from, row(order_[k]));
      if (d > bd) { bd = d; best = order_[k]; }
    }
    return best;
  }

  int build_rec(long b, long e) {
    int id = (int)nodes_.size();
    nodes_.emplace_back();
    {
      BallNode& nd = nodes_[id];
      nd.begin = b; nd.end = e;
      nd.mu.assign(dim_, 0.0);
      for (long k = b; k < e; ++k) {
        const double* r = row(order_[k]);
        for (int d = 0; d < dim_; ++d) nd.mu[d] += r[d];
      }
      for (int d = 0; d < dim_; ++d) nd.mu[d] /= (double)(e - b);
      for (long k = b; k < e; ++k) nd.radius = std::max(nd.radius, dist(nd.mu.data(), row(order_[k])));
    }
    if (e - b <= limit_) return id;
    // pivots: A = farthest from an arbitrary point, B = farthest from A
    long a = farthest(row(order_[b]), b, e);
    long bb = farthest(row(a), b, e);
    const double* pa = row(a);
    const double* pb = row(bb);
    auto mid = std::partition(order_.begin() + b, order_.begin() + e, [&](long i) {
      return dist(row(i), pa) <= dist(row(i), pb);
    });
    long m = (long)(mid - order_.begin());
    if (m == b || m == e) return id;  // all points coincide: keep as a (large) leaf
    int l = build_rec(b, m);
    int r = build_rec(m, e);
    nodes_[id].left = l;
    nodes_[id].right = r;
    return id;
  }

  void consider(long i, const double* q, int k, const std::unordered_set<long>& black,
                const std::unordered_set<long>& white, Heap& heap) const {
    if (!white.empty() && !white.count(i)) return;
    if (black.count(i)) return;
    double s = dot(q, row(i));
    if ((int)heap.size() < k) heap.push({i, s});
    else if (s > heap.top().score) { heap.pop(); heap.push({i, s}); }
  }

  void search_rec(int id, const double* q, double qn, int k, const std::unordered_set<long>& black,
                  const std::unordered_set<long>& white, Heap& heap) const {
    const BallNode& nd = nodes_[id];
    double bound = dot(q, nd.mu.data()) + qn * nd.radius;
    if ((int)heap.size() >= k && bound <= heap.top().score) return;
    ++visited_;
    if (nd.left < 0) {
      for (long t = nd.begin; t < nd.end; ++t) consider(order_[t], q, k, black, white, heap);
      return;
    }
    const BallNode& L = nodes_[nd.left];
    const BallNode& R = nodes_[nd.right];
    double bl = dot(q, L.mu.data()) + qn * L.radius;
    double br = dot(q, R.mu.data()) + qn * R.radius;
    if (bl >= br) {
      search_rec(nd.left, q, qn, k, black, white, heap);
      search_rec(nd.right, q, qn, k, black, white, heap);
    } else {
      search_rec(nd.right, q, qn, k, black, white, heap);
      search_rec(nd.left, q, qn, k, black, white, heap);
    }
  }

  static std::vector<Hit> drain(Heap& heap) {
    std::vector<Hit> out;
    while (!heap.empty()) { out.push_back(heap.top()); heap.pop(); }
    std::reverse(out.begin(), out.end());
    return out;
  }

  std::vector<double> x_;
  long n_;
  int dim_;
  int limit_;
  std::vector<BallNode> nodes_;
  std::vector<long> order_;
  mutable long visited_ = 0;
};

}  // namespace pcl
