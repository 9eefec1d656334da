// Sequential CPU kernels used by the host backend and as oracles for the GPU
// kernels: SGD passes of logistic / ridge regression, the MF rating pass, the
// collapsed-Gibbs LDA sweep, the shooting (coordinate) steps of Lasso / L1-LR.
// Arithmetic is fp64 like the reference.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <random>
#include <vector>

namespace pcl {

inline double sigmoid(double z) { return 1.0 / (1.0 + std::exp(-z)); }

// One pass over samples idx[0..n) of a row-major matrix X (n_rows x dim):
//   theta_i += alpha * (y - h(x)) * x_i - 2 * alpha * beta * theta_i
// with h = sigmoid(theta.x) (logistic) or theta.x (ridge).  When `accumulate` is set the
// step is added to `delta` with theta frozen (the reference's "dgd" variant,
// alg/classification/logistic_regression/lr.cpp:119-145); otherwise theta moves after
// every sample ("ipm", lr.cpp:165-193; ridge.hpp:73-96).
inline void linear_sgd_pass(const double* X, const double* y, long dim, const int64_t* idx, long n,
                            double* theta, double* delta, double alpha, double beta,
                            bool logistic, bool accumulate) {
  const double coff2 = 2.0 * beta * alpha;
  for (long k = 0; k < n; ++k) {
    const double* x = X + idx[k] * dim;
    double dp = 0.0;
    for (long i = 0; i < dim; ++i) dp += x[i] * theta[i];
    const double h = logistic ? sigmoid(dp) : dp;
    const double coff1 = alpha * (y[idx[k]] - h);
    if (accumulate) {
      for (long i = 0; i < dim; ++i) delta[i] += coff1 * x[i] - coff2 * theta[i];
    } else {
      for (long i = 0; i < dim; ++i) theta[i] += coff1 * x[i] - coff2 * theta[i];
    }
  }
}

inline double logloss_sum(const double* X, const double* y, long dim, long n, const double* theta) {
  double loss = 0.0;
  for (long k = 0; k < n; ++k) {
    double dp = 0.0;
    for (long i = 0; i < dim; ++i) dp += X[k * dim + i] * theta[i];
    const double h = sigmoid(dp);
    loss += (y[k] == 1.0) ? -std::log(h) : -std::log(1.0 - h);
  }
  return loss;
}

// Sequential biased-MF pass (alg/recommendation/matrix_factorization/mf.hpp:266-280).
inline void mf_sgd_pass(const int64_t* u, const int64_t* it, const double* r, long nnz, long k,
                        double* W, double* H, double* bu, double* bi, double mu, double alpha,
                        double beta) {
  std::vector<double> dW(k), dH(k);
  for (long e = 0; e < nnz; ++e) {
    double* w = W + u[e] * k;
    double* h = H + it[e] * k;
    double pred = mu + bu[u[e]] + bi[it[e]];
    for (long d = 0; d < k; ++d) pred += w[d] * h[d];
    pred = std::min(5.0, std::max(1.0, pred));
    const double err = r[e] - pred;
    for (long d = 0; d < k; ++d) {
      dW[d] = alpha * (2 * err * h[d] - beta * w[d]);
      dH[d] = alpha * (2 * err * w[d] - beta * h[d]);
    }
    for (long d = 0; d < k; ++d) { w[d] += dW[d]; h[d] += dH[d]; }
    bu[u[e]] += alpha * (2 * err - beta * bu[u[e]]);
    bi[it[e]] += alpha * (2 * err - beta * bi[it[e]]);
  }
}

// One collapsed-Gibbs sweep over all tokens (alg/topic_model/gLDA.hpp:408-426):
// remove the token, p(k) ~ (n_dk + alpha) / (n_d + K alpha) * (n_wk + beta) / (n_k + V beta),
// cumulative sums in place, sample with the first k whose cumulative sum exceeds u * total.
inline void lda_gibbs_sweep(const int64_t* doc_ptr, long n_docs, const int32_t* words, int32_t* z,
                            int32_t* doc_topic, int32_t* word_topic, int32_t* topic_sum,
                            const int32_t* doc_len, long K, long V, double alpha, double beta,
                            uint64_t seed) {
  std::mt19937_64 gen(seed);
  std::uniform_real_distribution<double> uni(0.0, 1.0);
  std::vector<double> p(K);
  for (long d = 0; d < n_docs; ++d) {
    int32_t* nd = doc_topic + d * K;
    for (int64_t t = doc_ptr[d]; t < doc_ptr[d + 1]; ++t) {
      const int32_t w = words[t];
      int32_t* nw = word_topic + (long)w * K;
      int32_t k_old = z[t];
      nd[k_old] -= 1; nw[k_old] -= 1; topic_sum[k_old] -= 1;
      const double denom_d = (doc_len[d] - 1) + K * alpha;
      double acc = 0.0;
      for (long k = 0; k < K; ++k) {
        acc += (nd[k] + alpha) / denom_d * (nw[k] + beta) / (topic_sum[k] + V * beta);
        p[k] = acc;
      }
      const double x = uni(gen) * acc;
      long k_new = K - 1;
      for (long k = 0; k < K; ++k) {
        if (p[k] > x) { k_new = k; break; }
      }
      z[t] = (int32_t)k_new;
      nd[k_new] += 1; nw[k_new] += 1; topic_sum[k_new] += 1;
    }
  }
}

// Stochastic coordinate descent ("shooting") on the duplicated non-negative features
// W in R^{2k} (tool/lasso_serial.cpp:46-76, tool/lr_l1_serial.cpp:46-73).  X is column
// major (n x k); z is the current prediction X w (lasso) or margin (L1-LR, labels +-1).
inline void shooting_steps(const double* Xc, const double* y, long n, long k, double* W, double* z,
                           double lambda, long steps, bool logistic, uint64_t seed) {
  std::mt19937_64 gen(seed);
  std::uniform_int_distribution<long> pick(0, 2 * k - 1);
  for (long s = 0; s < steps; ++s) {
    const long j = pick(gen);
    const long col = j % k;
    const double sign = j < k ? 1.0 : -1.0;
    const double* x = Xc + col * n;
    double g = 0.0;
    if (logistic) {
      for (long i = 0; i < n; ++i) g += (-y[i] / (1.0 + std::exp(z[i] * y[i]))) * sign * x[i];
    } else {
      for (long i = 0; i < n; ++i) g += (z[i] - y[i]) * sign * x[i];
    }
    double delta = (lambda + g) / (double)n;
    if (logistic) delta *= 4.0;
    const double eta = std::max(-W[j], -delta);
    W[j] += eta;
    for (long i = 0; i < n; ++i) z[i] += eta * sign * x[i];
  }
}

}  // namespace pcl
