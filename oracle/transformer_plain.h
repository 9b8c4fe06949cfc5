// TEST INFRASTRUCTURE: float64 restatement of one transformer encoder layer,
// used only as the checker of the encrypted layer in tests. Parity unpinned by
// the reference: the reference has no transformer code (CMakeLists.txt:63-75
// lists every extension source), so there is nothing of its own to compare
// with; this file states the layer in natural units from the textbook
// definition (Vaswani et al. 2017; BERT: post-LayerNorm, GELU), once with the
// exact non-linear functions and once with each of them replaced by a
// Chebyshev series handed in by the caller (the series the encrypted layer
// evaluates). The token offsets of the attention run cyclically over the
// whole sequence (every token attends to every token: no mask). Pinned on the
// CPU against PyTorch's float64 softmax / GELU / layer_norm
// (tests/test_plain_layer_cpu.py).
#pragma once
#include <cmath>
#include <vector>

namespace plain_transformer {

struct Spec {
  int seq_len, hidden, heads, head_dim, ffn;
  double score_range, sum_lo, sum_hi, var_lo, var_hi, gelu_range, ln_eps;
  std::vector<double> exp_c, inv_c, rsqrt_c, gelu_c;  // Chebyshev coefficients (T_0 first)
  bool exact;  // true: exp / reciprocal / rsqrt / GELU themselves
};

struct Weights {
  const double *wq, *wk, *wv, *wo, *w1, *w2;  // [in][out]
  const double *bq, *bk, *bv, *bo, *b1, *b2, *gamma1, *beta1, *gamma2, *beta2;
};

inline double Clenshaw(const std::vector<double> &c, double x) {
  double b1 = 0, b2 = 0;
  for (int k = (int)c.size() - 1; k >= 1; k--) {
    const double b0 = c[k] + 2 * x * b1 - b2;
    b2 = b1;
    b1 = b0;
  }
  return c[0] + x * b1 - b2;
}

inline void Linear(std::vector<double> &y, const std::vector<double> &x, const double *w, const double *b, int rows,
                   int n_in, int n_out) {
  y.assign((size_t)rows * n_out, 0.0);
  for (int t = 0; t < rows; t++)
    for (int k = 0; k < n_in; k++) {
      const double xv = x[(size_t)t * n_in + k];
      const double *wr = w + (size_t)k * n_out;
      double *yr = &y[(size_t)t * n_out];
      for (int j = 0; j < n_out; j++) yr[j] += xv * wr[j];
    }
  for (int t = 0; t < rows; t++)
    for (int j = 0; j < n_out; j++) y[(size_t)t * n_out + j] += b[j];
}

inline void LayerNorm(std::vector<double> &h, const Spec &s, const double *gamma, const double *beta, double *var_min,
                      double *var_max) {
  const int T = s.seq_len, H = s.hidden;
  for (int t = 0; t < T; t++) {
    double *r = &h[(size_t)t * H];
    double mean = 0, var = 0;
    for (int j = 0; j < H; j++) mean += r[j];
    mean /= H;
    for (int j = 0; j < H; j++) var += (r[j] - mean) * (r[j] - mean);
    var /= H;
    if (var_min && var < *var_min) *var_min = var;
    if (var_max && var > *var_max) *var_max = var;
    double inv;
    if (s.exact)
      inv = 1.0 / std::sqrt(var + s.ln_eps);
    else
      inv = 2.0 * Clenshaw(s.rsqrt_c, (2.0 * var - (s.var_hi + s.var_lo)) / (s.var_hi - s.var_lo));
    for (int j = 0; j < H; j++) r[j] = gamma[j] * (r[j] - mean) * inv + beta[j];
  }
}

// Ranges met on the way (to check that every series stays on its interval).
struct Ranges {
  double score_abs = 0, sum_min = 1e300, sum_max = 0, var_min = 1e300, var_max = 0, pre_abs = 0, out_abs = 0;
};

// Intermediate results, [seq_len][width] each, in natural units.
struct Trace {
  std::vector<double> q, k, v, attention, sum1, norm1, pre, gelu, sum2;  // sum1, sum2: residual sums before LayerNorm
};

// x, out: [seq_len][hidden]
inline void Layer(std::vector<double> &out, const std::vector<double> &x, const Spec &s, const Weights &w,
                  Ranges *ranges = nullptr, Trace *trace = nullptr) {
  const int T = s.seq_len, H = s.hidden, D = s.head_dim, F = s.ffn;
  Ranges local;
  Ranges &rg = ranges ? *ranges : local;
  std::vector<double> q, k, v, o((size_t)T * H, 0.0), e(T);
  Linear(q, x, w.wq, w.bq, T, H, H);
  Linear(k, x, w.wk, w.bk, T, H, H);
  Linear(v, x, w.wv, w.bv, T, H, H);
  for (int h = 0; h < s.heads; h++)
    for (int t = 0; t < T; t++) {
      double sum = 0;
      for (int r = 0; r < T; r++) {
        const int u = (t + r) % T;
        double sc = 0;
        for (int d = 0; d < D; d++) sc += q[(size_t)t * H + h * D + d] * k[(size_t)u * H + h * D + d];
        sc /= std::sqrt((double)D);
        rg.score_abs = std::fmax(rg.score_abs, std::fabs(sc));
        e[r] = s.exact ? std::exp(sc - s.score_range) : Clenshaw(s.exp_c, sc / s.score_range);
        sum += e[r];
      }
      const double mean = sum / T;
      rg.sum_min = std::fmin(rg.sum_min, mean);
      rg.sum_max = std::fmax(rg.sum_max, mean);
      const double inv = s.exact ? 1.0 / sum
                                 : Clenshaw(s.inv_c, (2.0 * mean - (s.sum_hi + s.sum_lo)) / (s.sum_hi - s.sum_lo));
      for (int d = 0; d < D; d++) {
        double acc = 0;
        for (int r = 0; r < T; r++) acc += e[r] * v[(size_t)((t + r) % T) * H + h * D + d];
        o[(size_t)t * H + h * D + d] = acc * inv;
      }
    }
  std::vector<double> h1, a, h2;
  Linear(h1, o, w.wo, w.bo, T, H, H);
  for (size_t i = 0; i < h1.size(); i++) h1[i] += x[i];
  if (trace) {
    trace->q = q;
    trace->k = k;
    trace->v = v;
    trace->attention = o;
    trace->sum1 = h1;
  }
  LayerNorm(h1, s, w.gamma1, w.beta1, &rg.var_min, &rg.var_max);
  Linear(a, h1, w.w1, w.b1, T, H, F);
  if (trace) {
    trace->norm1 = h1;
    trace->pre = a;
  }
  for (auto &p : a) {
    rg.pre_abs = std::fmax(rg.pre_abs, std::fabs(p));
    if (s.exact)
      p = 0.5 * p * (1.0 + std::erf(p / std::sqrt(2.0)));
    else
      p = s.gelu_range * Clenshaw(s.gelu_c, p / s.gelu_range);
  }
  if (trace) trace->gelu = a;
  Linear(h2, a, w.w2, w.b2, T, F, H);
  for (size_t i = 0; i < h2.size(); i++) h2[i] += h1[i];
  if (trace) trace->sum2 = h2;
  LayerNorm(h2, s, w.gamma2, w.beta2, &rg.var_min, &rg.var_max);
  for (double p : h2) rg.out_abs = std::fmax(rg.out_abs, std::fabs(p));
  out = std::move(h2);
}

}  // namespace plain_transformer
