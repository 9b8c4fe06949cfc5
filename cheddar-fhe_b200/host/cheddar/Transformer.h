// One encrypted transformer encoder layer (BERT shape: multi-head self
// attention, residual + LayerNorm, GELU feed-forward, residual + LayerNorm)
// composed from the operators of this library: the tensor-core ciphertext x
// plaintext contraction (cfhe_ctpt_gemm), hoisted rotations, HMult, Chebyshev
// polynomial evaluation (EvalPoly) and bootstrapping (BootContext::Boot).
//
// The reference has no transformer code (its extension directory holds
// BootContext, EvalMod, EvalPoly, EvalSpecialFFT, Hoist, LinearTransform and
// StripedMatrix only, CMakeLists.txt:63-75); this file composes the layer from
// the counterparts of those pieces (src/extension/EvalPoly.cpp:408-661,
// src/extension/BootContext.cpp:299-365, src/extension/Hoist.cu:578-691).
//
// Packing. One ciphertext per feature. Slot t * B + b of feature ciphertext j
// holds x[b][t][j] / act_div: token t of sequence b of a batch of
// B = num_slots / seq_len sequences (256 for 128 tokens at N = 2^16). With
// that layout
//   * a projection y_j = sum_k W[k][j] x_k is a contraction ACROSS ciphertexts
//     by plaintext scalars: an exact integer GEMM over the RNS limbs, run on
//     the tensor cores;
//   * a rotation by r * B slots moves token t + r onto token t in every
//     sequence at once, so score offset r of a head is
//     sum_d Q_d * rot_r(K_d): rotations come in baby steps (hoisted, one ModUp
//     per ciphertext) and giant steps;
//   * the softmax denominator and the LayerNorm statistics are sums across
//     ciphertexts, no rotation at all, and live in ONE ciphertext per head or
//     per LayerNorm: those are the ciphertexts whose reciprocal / reciprocal
//     square root is evaluated (bootstrapped first, so that the expensive
//     polynomial costs levels of one ciphertext, not of hundreds).
//
// Every non-linear function is a Chebyshev series on [-1, 1] (TransformerPolys);
// the float64 layer used as the checker in the tests evaluates the same series.
//
// Host threads. Below level 13 a ciphertext operator is a few small kernels,
// and a degree-31 series is about 400 launches: one host thread cannot enqueue
// them as fast as the GPU runs them, and one stream leaves SMs idle. Stages
// that are independent per ciphertext (series, rotations, rescales, products)
// therefore run as a parallel loop over `workers` host threads, each with its
// own engine context (stream, workspace, allocation pool); the streams are
// ordered after the main stream when the loop starts and the main stream after
// them when it ends. Inside such a loop an item frees only what it allocated
// itself, so no block changes pool while another stream may still read it.
//
// Several GPUs (one process each, RankGroup). One layer call is sharded by
// heads and by blocks of ciphertexts: a rank projects Q, K, V for its heads
// only and runs their attention; the attention outputs are all-gathered; from
// there on a rank owns a block of the residual ciphertexts (its columns of the
// output projection and of the second feed-forward projection, its share of
// the residual sums, the LayerNorm products and the bootstraps) and a block of
// the feed-forward features, with an all-gather where the next stage needs
// every ciphertext; a LayerNorm's sum of squares gathers one partial sum per
// rank, and the statistic's bootstrap and series run on every rank alike.
// Every rank starts from the same ciphertexts and keys and all arithmetic is
// exact, so the sharded result is bit-identical to the one-GPU result.
#pragma once
#include <chrono>
#include <atomic>
#include <random>
#include <thread>
#include <tuple>

#include "cheddar/Boot.h"
#include "cheddar/RankGroup.h"

namespace cheddar {

struct TransformerConfig {
  int seq_len = 128, hidden = 768, heads = 12, head_dim = 64, ffn = 3072;
  int baby = 16;             // baby steps of the token rotations (divides seq_len)
  double act_div = 8.0;      // ciphertexts of the residual stream hold value / act_div
  double score_range = 2.0;  // bound on |q . k| / sqrt(head_dim)
  double sum_lo = 0.04, sum_hi = 0.8;  // bounds on mean_r exp(s_r - score_range)
  double var_lo = 0.3, var_hi = 6.5;   // bounds on the LayerNorm variance
  double gelu_range = 4.0;             // bound on the feed-forward pre-activation
  double ln_eps = 1e-5;
  int exp_degree = 15, inv_degree = 63, rsqrt_degree = 63, gelu_degree = 31;
  bool pair_boot = true;  // bootstrap two real ciphertexts as one complex one
  int workers = 4;        // host threads (and streams) of the per-ciphertext stages
  static TransformerConfig BertBase() { return TransformerConfig{}; }
  static TransformerConfig Small() {
    TransformerConfig c;
    c.seq_len = 16;
    c.hidden = 32;
    c.heads = 2;
    c.head_dim = 16;
    c.ffn = 64;
    c.baby = 4;
    c.var_lo = 0.15;  // the variance of 32 features spreads wider than that of 768
    return c;
  }
};

// Row-major [in][out] matrices, as a framework stores nn.Linear weights transposed.
struct TransformerWeights {
  std::vector<double> wq, wk, wv, wo, w1, w2;
  std::vector<double> bq, bk, bv, bo, b1, b2;
  std::vector<double> gamma1, beta1, gamma2, beta2;
  static TransformerWeights Random(const TransformerConfig &c, uint64_t seed, double stddev) {
    std::mt19937_64 gen(seed);
    std::normal_distribution<double> nd(0.0, stddev);
    auto fill = [&](std::vector<double> &v, size_t n, double centre) {
      v.resize(n);
      for (auto &x : v) x = centre + nd(gen);
    };
    TransformerWeights w;
    const size_t H = c.hidden, F = c.ffn;
    fill(w.wq, H * H, 0);
    fill(w.wk, H * H, 0);
    fill(w.wv, H * H, 0);
    fill(w.wo, H * H, 0);
    fill(w.w1, H * F, 0);
    fill(w.w2, F * H, 0);
    fill(w.bq, H, 0);
    fill(w.bk, H, 0);
    fill(w.bv, H, 0);
    fill(w.bo, H, 0);
    fill(w.b1, F, 0);
    fill(w.b2, H, 0);
    fill(w.gamma1, H, 1);
    fill(w.beta1, H, 0);
    fill(w.gamma2, H, 1);
    fill(w.beta2, H, 0);
    return w;
  }
};

// The four Chebyshev series of the layer, each on its own affine image of [-1, 1].
struct TransformerPolys {
  std::vector<double> exp_c;    // u in [-1,1] -> exp(R (u - 1)),               u = s / R
  std::vector<double> inv_c;    // w -> 1 / (T m),  m = ((hi-lo) w + hi+lo)/2 the mean of the exponentials
  std::vector<double> rsqrt_c;  // w -> 1 / (2 sqrt(v + eps)), v = ((hi-lo) w + hi+lo)/2 the variance
  std::vector<double> gelu_c;   // t -> GELU(G t) / G,          t = a / G
  // GELU(x) = x / 2 + E(x) with E even, so the series above is t / 2 plus a
  // series in T_2(t) = 2 t^2 - 1 (T_2k(t) = T_k(T_2(t))): its even coefficients
  std::vector<double> gelu_even_c;
  explicit TransformerPolys(const TransformerConfig &c) {
    using P = EvalPoly<uint32_t>;
    const double R = c.score_range, T = c.seq_len, G = c.gelu_range;
    exp_c = P::ChebyshevCoefficients([=](double u) { return std::exp(R * (u - 1.0)); }, c.exp_degree);
    inv_c = P::ChebyshevCoefficients(
        [=](double w) { return 1.0 / (T * 0.5 * ((c.sum_hi - c.sum_lo) * w + c.sum_hi + c.sum_lo)); },
        c.inv_degree);
    rsqrt_c = P::ChebyshevCoefficients(
        [=](double w) {
          return 0.5 / std::sqrt(0.5 * ((c.var_hi - c.var_lo) * w + c.var_hi + c.var_lo) + c.ln_eps);
        },
        c.rsqrt_degree);
    gelu_c = P::ChebyshevCoefficients(
        [=](double t) {
          const double a = G * t;
          return 0.5 * a * (1.0 + std::erf(a / std::sqrt(2.0))) / G;
        },
        c.gelu_degree);
    for (size_t k = 0; k < gelu_c.size(); k += 2) gelu_even_c.push_back(gelu_c[k]);
  }
};

// A plaintext matrix encoded on the limbs of one level and packed for the
// tensor-core contraction.
template <typename word>
class PlainMatrix {
  using Ct = Ciphertext<word>;

 public:
  // w: [n_in][n_out] real weights, encoded as round(w * scale) mod every prime of `level`
  PlainMatrix(const Context<word> &ctx, const std::vector<double> &w, int n_in, int n_out, int level,
              double scale)
      : n_in_{n_in}, n_out_{n_out}, level_{level}, scale_{scale} {
    AssertTrue((size_t)n_in * n_out == w.size(), "PlainMatrix: wrong weight count");
    const NPInfo np = ctx.param_.LevelToNP(level);
    g_ = ctx.param_.GetLimbIndices(np);
    const auto primes = ctx.param_.GetPrimeVector(np);
    const size_t per = (size_t)n_in * n_out;
    std::vector<uint32_t> host(per * primes.size());
    for (size_t i = 0; i < per; i++) {
      const double scaled = std::nearbyint(w[i] * scale);
      AssertTrue(std::abs(scaled) < 9.0e18, "PlainMatrix: weight too large for the scale");
      const int64_t v = (int64_t)scaled;
      for (size_t l = 0; l < primes.size(); l++) {
        int64_t r = v % (int64_t)primes[l];
        if (r < 0) r += primes[l];
        host[l * per + i] = detail::ToMontgomery((word)r, primes[l]);
      }
    }
    const size_t bytes = cfhe_gemm_weight_bytes(n_in, n_out, (int)g_.size());
    packed_.resize((int)((bytes + sizeof(word) - 1) / sizeof(word)));
    CheckAbi(cfhe_gemm_pack_weights(ctx.h_, packed_.data(), host.data(), n_in, n_out, g_.data(), (int)g_.size()));
    ctx.Synchronize();
  }
  int level() const { return level_; }
  double scale() const { return scale_; }
  // y[j] = sum_k w[k][j] x[k] on both polynomials, at the level of x, scale
  // x.scale * scale, not rescaled
  void Apply(const Context<word> &ctx, std::vector<Ct> &y, const std::vector<const Ct *> &x) const {
    AssertTrue((int)x.size() == n_in_, "PlainMatrix: wrong input count");
    const NPInfo np = ctx.param_.LevelToNP(level_);
    std::vector<const word *> xb(n_in_), xa(n_in_);
    for (int k = 0; k < n_in_; k++) {
      AssertTrue(x[k]->GetNP() == np && !x[k]->HasRx(), "PlainMatrix: input at the wrong level");
      xb[k] = x[k]->bx_.data();
      xa[k] = x[k]->ax_.data();
    }
    y.clear();
    y.reserve(n_out_);
    std::vector<word *> yb(n_out_), ya(n_out_);
    for (int j = 0; j < n_out_; j++) {
      y.emplace_back(np);
      y[j].SetScale(x[0]->GetScale() * scale_);
      y[j].SetNumSlots(x[0]->GetNumSlots());
      yb[j] = y[j].bx_.data();
      ya[j] = y[j].ax_.data();
    }
    CheckAbi(cfhe_ctpt_gemm(ctx.h_, yb.data(), xb.data(), packed_.data(), n_in_, n_out_, g_.data(), (int)g_.size()));
    CheckAbi(cfhe_ctpt_gemm(ctx.h_, ya.data(), xa.data(), packed_.data(), n_in_, n_out_, g_.data(), (int)g_.size()));
  }
  // 8-bit multiply-accumulates of one Apply (both polynomials, all limbs)
  double Int8Macs(int degree) const { return 2.0 * g_.size() * 16.0 * n_in_ * (double)n_out_ * degree; }

 private:
  int n_in_, n_out_, level_;
  double scale_;
  std::vector<int> g_;
  DeviceVector<word> packed_;
};

template <typename word>
class EncryptedTransformerLayer {
  using Ct = Ciphertext<word>;
  using Const = Constant<word>;
  using Evk = EvaluationKey<word>;
  using Boot = BootContext<word>;

 public:
  EncryptedTransformerLayer(std::shared_ptr<Boot> ctx, const TransformerConfig &cfg, const TransformerWeights &w,
                            std::shared_ptr<RankGroup> group = nullptr)
      : ctx_{std::move(ctx)}, cfg_{cfg}, w_{w}, polys_{cfg}, group_{std::move(group)} {
    if (!group_) group_ = std::make_shared<RankGroup>();
    AssertTrue(group_->world() <= cfg.heads, "Transformer: more ranks than heads");
    AssertTrue(cfg.heads * cfg.head_dim == cfg.hidden, "Transformer: heads * head_dim != hidden");
    AssertTrue(cfg.seq_len % cfg.baby == 0, "Transformer: baby must divide seq_len");
    slots_ = ctx_->param_.degree_ / 2;
    AssertTrue(slots_ % cfg.seq_len == 0, "Transformer: seq_len must divide the slot count");
    lane_ = slots_ / cfg.seq_len;
    main_ = ctx_;
    cfhe_context *current = detail::CurrentHandle();
    for (int k = 1; k < cfg.workers; k++) workers_.push_back(Context<word>::Create(ctx_->param_));
    detail::CurrentHandle() = current;
  }
  int BatchSize() const { return lane_; }
  // Called after every stage with its name, the ciphertexts it produced and the
  // factor that turns their slot values into the layer's natural units (for
  // tests that decrypt intermediate results).
  using Probe = std::function<void(const std::string &, const std::vector<Ct> &, double)>;
  void SetProbe(Probe p) { probe_ = std::move(p); }
  const TransformerPolys &polys() const { return polys_; }

  // rotation keys of the token shifts (the bootstrapping keys are requested by the BootContext)
  void AddRequiredRotations(EvkRequest &req) const {
    const int level = ctx_->param_.max_level_;
    for (int b = 1; b < cfg_.baby; b++) req.AddRequest(b * lane_, level);
    for (int g = 1; g < cfg_.seq_len / cfg_.baby; g++) req.AddRequest(g * cfg_.baby * lane_, level);
  }

  // x: `hidden` ciphertexts at the level bootstrapping ends on, slot t * B + b
  // holding x[b][t][j] / act_div. out: the same layout and level.
  void Forward(std::vector<Ct> &out, const std::vector<Ct> &x, const EvkMap<word> &evk) {
    const int H = cfg_.hidden, heads = cfg_.heads, D = cfg_.head_dim, F = cfg_.ffn;
    const double A = cfg_.act_div;
    AssertTrue((int)x.size() == H, "Transformer: wrong number of input ciphertexts");
    const Evk &mult = evk.GetMultiplicationKey();
    const int rank = group_->rank(), world = group_->world();
    const auto [head0, head1] = Block(heads, rank);   // this rank's heads
    const auto [res0, res1] = Block(H, rank);         // its block of the residual ciphertexts
    const auto [ffn0, ffn1] = Block(F, rank);         // its block of the feed-forward features
    stage_s_.clear();
    gemm_s_ = 0;
    pack_s_ = 0;
    gemm_macs_ = 0;
    boots_ = 0;
    ctx_->Synchronize();
    last_ = std::chrono::steady_clock::now();

    // ---- attention
    std::vector<Ct> qkv;
    {
      // Q is pre-divided by sqrt(head_dim) * score_range: the score ciphertexts hold s / score_range
      const double qs = 1.0 / (std::sqrt((double)D) * cfg_.score_range);
      // columns of this rank's heads only: Q, K and V of head h are features h D .. (h+1) D - 1
      std::vector<int> cols;
      for (int part = 0; part < 3; part++)
        for (int j = head0 * D; j < head1 * D; j++) cols.push_back(part * H + j);
      const int nc = cols.size();
      if (!m_qkv_) {
        std::vector<double> wm((size_t)H * nc);
        for (int k = 0; k < H; k++)
          for (int c = 0; c < nc; c++) {
            const int part = cols[c] / H, j = cols[c] % H;
            const double v = part == 0 ? w_.wq[(size_t)k * H + j] * A * qs
                                       : part == 1 ? w_.wk[(size_t)k * H + j] * A : w_.wv[(size_t)k * H + j] * A;
            wm[(size_t)k * nc + c] = v;
          }
        m_qkv_ = MakeMatrix(wm, H, nc, x[0]);
      }
      std::vector<double> bias(nc);
      for (int c = 0; c < nc; c++) {
        const int part = cols[c] / H, j = cols[c] % H;
        bias[c] = part == 0 ? w_.bq[j] * qs : part == 1 ? w_.bk[j] : w_.bv[j];
      }
      qkv.resize(3 * H);
      Project(qkv, *m_qkv_, Pointers(x), bias, cols);
    }
    Mark("QKV projection");
    if (probe_) probe_("qkv", qkv, 1.0);
    std::vector<Ct> o_un(H), stat(head1 - head0);
    for (int h = head0; h < head1; h++) AttentionHead(h, qkv, o_un, stat[h - head0], evk);
    qkv.clear();
    Mark("scores, exponentials, weighted values");
    std::vector<Ct> o(H);
    {
      BootAll(stat, evk, true);
      for (int h = head0; h < head1; h++) {
        Ct p;
        Poly(main_, p, stat[h - head0], polys_.inv_c, mult);
        LevelTo(main_, p, Level(o_un[h * D]));
        AssertTrue(Level(p) == Level(o_un[h * D]), "Transformer: the normaliser ended below the weighted values");
        ParallelFor(D, [&](const ConstContextPtr<word> &c, int d) {
          c->HMult(o[h * D + d], o_un[h * D + d], p, mult);
        });
      }
      o_un.clear();
    }
    Mark("softmax normaliser");
    if (world > 1) {
      AllGather(o, [&](int j) { return BlockOwner(heads, j / D); });
      Mark("all-gather: attention outputs");
    }
    if (probe_) probe_("attention", o, 1.0);
    std::vector<Ct> y1;
    {
      // the mean over the features is removed here: C = I - 11^T / H commutes
      // with the residual sum, so C is folded into the weights and the bias
      std::vector<int> cols;
      for (int j = res0; j < res1; j++) cols.push_back(j);
      if (!m_wo_) m_wo_ = MakeMatrix(Columns(Centred(w_.wo, H, H, 1.0 / A), H, H, cols), H, cols.size(), o[0]);
      y1.resize(H);
      Project(y1, *m_wo_, Pointers(o), Select(CentredBias(w_.bo, 1.0 / A), cols), cols);
      o.clear();
      AddCentredResidual(y1, x, res0, res1);
    }
    Mark("output projection, residual");
    if (probe_) probe_("centred sum 1", y1, A);
    std::vector<Ct> z;
    LayerNorm(z, y1, w_.gamma1, w_.beta1, evk, res0, res1);
    y1.clear();
    Mark("LayerNorm 1");
    if (probe_) probe_("LayerNorm 1", z, A);
    BootBlock(z, res0, res1, evk);
    Mark("bootstrap (before the feed-forward block)");
    if (world > 1) {
      AllGather(z, [&](int j) { return BlockOwner(H, j); });
      Mark("all-gather: refreshed LayerNorm outputs");
    }
    if (probe_) probe_("LayerNorm 1, refreshed", z, A);

    // ---- feed-forward
    std::vector<Ct> act;
    {
      const double G = cfg_.gelu_range;
      std::vector<int> cols;
      for (int j = ffn0; j < ffn1; j++) cols.push_back(j);
      const int nc = cols.size();
      if (!m_w1_) {
        std::vector<double> wm((size_t)H * nc);
        for (int k = 0; k < H; k++)
          for (int c = 0; c < nc; c++) wm[(size_t)k * nc + c] = w_.w1[(size_t)k * F + cols[c]] * A / G;
        m_w1_ = MakeMatrix(wm, H, nc, z[0]);
      }
      std::vector<double> bias(nc);
      for (int c = 0; c < nc; c++) bias[c] = w_.b1[cols[c]] / G;
      std::vector<Ct> pre(F);
      Project(pre, *m_w1_, Pointers(z), bias, cols);
      Mark("feed-forward projection 1");
      if (probe_) probe_("pre-activation", pre, cfg_.gelu_range);
      act.resize(F);
      // only the even part E of GELU(a) = a / 2 + E(a) is evaluated, as a series of
      // half the degree in 2 t^2 - 1; the linear part a / 2 = (W1^T z + b1) / 2 goes
      // through the second projection as a linear map of z and joins the residual
      ParallelFor(nc, [&](const ConstContextPtr<word> &c, int i) {
        Ct y;
        EvalPoly<word>::Node(c, y, pre[ffn0 + i], pre[ffn0 + i], nullptr, 1.0, mult);
        Poly(c, act[ffn0 + i], y, polys_.gelu_even_c, mult);
      });
      pre.clear();
      Mark("GELU");
      if (world > 1) {
        AllGather(act, [&](int j) { return BlockOwner(F, j); });
        Mark("all-gather: feed-forward activations");
      }
      if (probe_) probe_("GELU", act, cfg_.gelu_range);
    }
    std::vector<Ct> y2(H);
    {
      std::vector<int> cols;
      for (int j = res0; j < res1; j++) cols.push_back(j);
      if (!m_w2_)
        m_w2_ = MakeMatrix(Columns(Centred(w_.w2, F, H, cfg_.gelu_range / A), F, H, cols), F, cols.size(), act[0]);
      // bias: b2 / A plus the constant of the linear part, W2^T b1 / (2 A), centred
      std::vector<double> bias(H, 0.0);
      for (int f = 0; f < F; f++)
        for (int j = 0; j < H; j++) bias[j] += 0.5 * w_.b1[f] * w_.w2[(size_t)f * H + j];
      for (int j = 0; j < H; j++) bias[j] += w_.b2[j];
      Project(y2, *m_w2_, Pointers(act), Select(CentredBias(bias, 1.0 / A), cols), cols);
      act.clear();
      // residual and linear part of the GELU in one projection of z: (I + W1 W2 / 2)^T z, centred
      if (!m_res_) {
        const auto t0 = std::chrono::steady_clock::now();
        std::vector<double> m((size_t)H * H, 0.0);
        for (int k = 0; k < H; k++) {
          double *row = &m[(size_t)k * H];
          for (int f = 0; f < F; f++) {
            const double a = 0.5 * w_.w1[(size_t)k * F + f];
            const double *w2 = &w_.w2[(size_t)f * H];
            for (int j = 0; j < H; j++) row[j] += a * w2[j];
          }
          row[k] += 1.0;
        }
        const auto d = std::chrono::steady_clock::now() - t0;
        last_ += d;
        pack_s_ += std::chrono::duration<double>(d).count();
        m_res_ = MakeMatrix(Columns(Centred(m, H, H, 1.0), H, H, cols), H, cols.size(), z[0]);
      }
      std::vector<Ct> lin(H);
      Project(lin, *m_res_, Pointers(z), std::vector<double>(cols.size(), 0.0), cols);
      const int ly = Level(y2[res0]);
      ParallelFor(res1 - res0, [&](const ConstContextPtr<word> &cx, int i) {
        const int j = res0 + i;
        Ct low;  // lin[j] belongs to another item's pool: it is read here and freed after the loop
        cx->LevelDown(low, lin[j], ly);
        cx->Add(y2[j], y2[j], low);
      });
    }
    z.clear();
    Mark("feed-forward projection 2, residual");
    if (probe_) probe_("centred sum 2", y2, A);
    LayerNorm(out, y2, w_.gamma2, w_.beta2, evk, res0, res1);
    y2.clear();
    Mark("LayerNorm 2");
    if (probe_) probe_("LayerNorm 2", out, A);
    BootBlock(out, res0, res1, evk);
    Mark("bootstrap (end of the layer)");
    if (world > 1) {
      AllGather(out, [&](int j) { return BlockOwner(H, j); });
      Mark("all-gather: layer outputs");
    }
  }

  // seconds per stage of the last Forward (the host synchronises between stages)
  const std::vector<std::pair<std::string, double>> &StageSeconds() const { return stage_s_; }
  double GemmSeconds() const { return gemm_s_; }
  double PackSeconds() const { return pack_s_; }  // encoding and packing the weights (first Forward only)
  double GemmInt8Macs() const { return gemm_macs_; }
  int Bootstraps() const { return boots_; }

 private:
  int Level(const Ct &c) const { return ctx_->param_.NPToLevel(c.GetNP()); }
  double Canon(int level) const { return ctx_->param_.GetScale(level); }
  static std::vector<const Ct *> Pointers(const std::vector<Ct> &v) {
    std::vector<const Ct *> p(v.size());
    for (size_t i = 0; i < v.size(); i++) p[i] = &v[i];
    return p;
  }
  void Mark(const char *name) {
    ctx_->Synchronize();
    const auto now = std::chrono::steady_clock::now();
    stage_s_.emplace_back(name, std::chrono::duration<double>(now - last_).count());
    last_ = now;
  }
  // fn(context, i) for every i in [0, n), shared out over the worker threads
  template <typename F>
  void ParallelFor(int n, F &&fn) {
    if (workers_.empty() || n < 2) {
      for (int i = 0; i < n; i++) fn(main_, i);
      return;
    }
    for (auto &w : workers_) CheckAbi(cfhe_order_after(w->h_, ctx_->h_));
    std::atomic<int> next{0};
    auto run = [&](const ConstContextPtr<word> &c) {
      ScopedCurrentHandle scope(c->h_);
      for (int i; (i = next.fetch_add(1)) < n;) fn(c, i);
    };
    std::vector<std::thread> threads;
    for (auto &w : workers_) threads.emplace_back(run, w);
    run(main_);
    for (auto &t : threads) t.join();
    for (auto &w : workers_) CheckAbi(cfhe_order_after(ctx_->h_, w->h_));
  }
  // c must be a ciphertext the calling item owns
  void LevelTo(const ConstContextPtr<word> &cx, Ct &c, int level) const {
    if (Level(c) <= level) return;
    Ct t;
    cx->LevelDown(t, c, level);
    c = std::move(t);
  }
  // res = value * a one level below a, at the canonical scale of that level
  void MultConstRescale(const ConstContextPtr<word> &cx, Ct &res, const Ct &a, double value) const {
    const int l = Level(a);
    Const k;
    cx->encoder().EncodeConstant(k, l, Canon(l - 1) * cx->param_.GetRescalePrimeProd(l) / a.GetScale(), value);
    Ct t;
    cx->Mult(t, a, k);
    cx->Rescale(res, t);
  }
  void AddConst(const ConstContextPtr<word> &cx, Ct &c, double value) const {
    if (value == 0.0) return;
    Const k;
    cx->encoder().EncodeConstant(k, Level(c), c.GetScale(), value);
    cx->Add(c, c, k);
  }
  void Poly(const ConstContextPtr<word> &cx, Ct &res, const Ct &x, const std::vector<double> &coeffs,
            const Evk &mult) const {
    int k = 1;
    while ((size_t(1) << k) < coeffs.size()) k++;
    EvalPoly<word>::EvaluateChebyshev(cx, res, x, coeffs, mult, Canon(Level(x) - k));
  }
  // Encoding and packing a matrix happens once, on the first Forward, and is
  // kept out of the stage times (reported by PackSeconds).
  std::unique_ptr<PlainMatrix<word>> MakeMatrix(const std::vector<double> &wm, int n_in, int n_out,
                                                const Ct &sample) {
    ctx_->Synchronize();
    const auto t0 = std::chrono::steady_clock::now();
    const int l = Level(sample);
    const double s = Canon(l - 1) * ctx_->param_.GetRescalePrimeProd(l) / sample.GetScale();
    auto m = std::make_unique<PlainMatrix<word>>(*ctx_, wm, n_in, n_out, l, s);
    const auto d = std::chrono::steady_clock::now() - t0;
    last_ += d;
    pack_s_ += std::chrono::duration<double>(d).count();
    return m;
  }
  // y = rescale(W x) + bias, one level below x at the canonical scale
  // out_index (optional): result c is stored in y[out_index[c]] (y keeps its size)
  void Project(std::vector<Ct> &y, const PlainMatrix<word> &m, const std::vector<const Ct *> &x,
               const std::vector<double> &bias, const std::vector<int> &out_index = {}) {
    AssertTrue(Level(*x[0]) == m.level(), "Transformer: the matrix was prepared for another level");
    ctx_->AssertSameScale(x[0]->GetScale() * m.scale(),
                          Canon(m.level() - 1) * ctx_->param_.GetRescalePrimeProd(m.level()));
    std::vector<Ct> raw;
    ctx_->Synchronize();
    const auto t0 = std::chrono::steady_clock::now();
    m.Apply(*ctx_, raw, x);
    ctx_->Synchronize();
    gemm_s_ += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    gemm_macs_ += m.Int8Macs(ctx_->param_.degree_);
    if (out_index.empty()) {
      y.clear();
      y.resize(raw.size());
    }
    ParallelFor((int)raw.size(), [&](const ConstContextPtr<word> &c, int j) {
      Ct &dst = y[out_index.empty() ? j : out_index[j]];
      c->Rescale(dst, raw[j]);
      AddConst(c, dst, bias[j]);
    });
  }

  // ---- ranks: contiguous blocks, the first n % world ranks hold one more
  std::pair<int, int> Block(int n, int rank) const { return BlockOfRank(n, group_->world(), rank); }
  int BlockOwner(int n, int i) const { return RankOfItem(n, group_->world(), i); }
  // Every rank ends with all of v: element i travels from owner(i). Elements
  // a rank does not own are allocated like the ones it owns (same level,
  // scale and slot count on every rank).
  void AllGather(std::vector<Ct> &v, const std::function<int(int)> &owner) {
    const int rank = group_->rank(), n = v.size();
    const Ct *like = nullptr;
    for (int i = 0; i < n && !like; i++)
      if (owner(i) == rank) like = &v[i];
    AssertTrue(like != nullptr, "Transformer: a rank owns nothing of a gathered vector");
    const NPInfo np = like->GetNP();
    const bool rx = like->HasRx();
    const size_t bytes = (size_t)np.GetNumTotal() * ctx_->param_.degree_ * sizeof(word);
    void *stream = cfhe_get_stream(ctx_->h_);
    constexpr int kPerGroup = 256;
    for (int i0 = 0; i0 < n; i0 += kPerGroup) {
      const int i1 = Min(n, i0 + kPerGroup);
      for (int i = i0; i < i1; i++)
        if (owner(i) != rank) {
          Ct fresh(np, rx);
          fresh.SetScale(like->GetScale());
          fresh.SetNumSlots(like->GetNumSlots());
          v[i] = std::move(fresh);
        }
      group_->Start();
      for (int i = i0; i < i1; i++) {
        group_->Broadcast(v[i].bx_.data(), bytes, owner(i), stream);
        group_->Broadcast(v[i].ax_.data(), bytes, owner(i), stream);
        if (rx) group_->Broadcast(v[i].rx_.data(), bytes, owner(i), stream);
      }
      group_->End();
    }
  }
  // BootAll on v[lo, hi)
  void BootBlock(std::vector<Ct> &v, int lo, int hi, const EvkMap<word> &evk) {
    std::vector<Ct> mine;
    for (int i = lo; i < hi; i++) mine.push_back(std::move(v[i]));
    BootAll(mine, evk);
    for (int i = lo; i < hi; i++) v[i] = std::move(mine[i - lo]);
  }
  // W (I - 11^T / n_out) * factor: every row loses its mean
  static std::vector<double> Centred(const std::vector<double> &w, int n_in, int n_out, double factor) {
    std::vector<double> r(w.size());
    for (int k = 0; k < n_in; k++) {
      double mean = 0;
      for (int j = 0; j < n_out; j++) mean += w[(size_t)k * n_out + j];
      mean /= n_out;
      for (int j = 0; j < n_out; j++) r[(size_t)k * n_out + j] = (w[(size_t)k * n_out + j] - mean) * factor;
    }
    return r;
  }
  // the listed columns of a row-major [n_in][n_out] matrix
  static std::vector<double> Columns(const std::vector<double> &w, int n_in, int n_out, const std::vector<int> &cols) {
    const int nc = cols.size();
    std::vector<double> r((size_t)n_in * nc);
    for (int k = 0; k < n_in; k++)
      for (int c = 0; c < nc; c++) r[(size_t)k * nc + c] = w[(size_t)k * n_out + cols[c]];
    return r;
  }
  static std::vector<double> Select(const std::vector<double> &v, const std::vector<int> &idx) {
    std::vector<double> r(idx.size());
    for (size_t c = 0; c < idx.size(); c++) r[c] = v[idx[c]];
    return r;
  }
  static std::vector<double> CentredBias(const std::vector<double> &b, double factor) {
    double mean = 0;
    for (double v : b) mean += v;
    mean /= b.size();
    std::vector<double> r(b.size());
    for (size_t j = 0; j < b.size(); j++) r[j] = (b[j] - mean) * factor;
    return r;
  }
  // y[j] += x[j] - mean_j x[j] for j in [lo, hi), x brought down to the level of y
  void AddCentredResidual(std::vector<Ct> &y, const std::vector<Ct> &x, int lo, int hi) {
    const int H = x.size(), lx = Level(x[0]), ly = Level(y[lo]);
    AssertTrue(lx > ly, "Transformer: the residual must sit above the block's output");
    Ct sum;
    ctx_->Copy(sum, x[0]);
    for (int j = 1; j < H; j++) ctx_->Add(sum, sum, x[j]);
    const double s = Canon(lx - 1) * ctx_->param_.GetRescalePrimeProd(lx) / x[0].GetScale();
    Const one, inv;
    ctx_->encoder().EncodeConstant(one, lx, s, 1.0);
    ctx_->encoder().EncodeConstant(inv, lx, s, 1.0 / H);
    Ct mean;
    ctx_->Mult(mean, sum, inv);
    ParallelFor(hi - lo, [&](const ConstContextPtr<word> &cx, int i) {
      const int j = lo + i;
      Ct t, c;
      cx->Mult(t, x[j], one);
      cx->Sub(t, t, mean);
      cx->Rescale(c, t);
      LevelTo(cx, c, ly);
      cx->Add(y[j], y[j], c);  // in place: y[j] keeps its buffers
    });
  }

  // out[0] = a, out[b] = a rotated by b tokens, b < baby (one ModUp for all of them)
  void BabyRotations(const ConstContextPtr<word> &cx, std::vector<Ct> &out, const Ct &a,
                     const EvkMap<word> &evk) const {
    std::vector<int> dists;
    std::vector<const Evk *> keys;
    for (int b = 1; b < cfg_.baby; b++) {
      dists.push_back(b * lane_);
      keys.push_back(&evk.GetRotationKey(b * lane_));
    }
    std::vector<Ct> rot;
    if (!dists.empty()) cx->HoistedRotate(rot, a, dists, keys);
    out.clear();
    out.resize(cfg_.baby);
    cx->Copy(out[0], a);
    for (int b = 1; b < cfg_.baby; b++) out[b] = std::move(rot[b - 1]);
  }
  void RotateTokens(const ConstContextPtr<word> &cx, Ct &res, const Ct &a, int tokens,
                    const EvkMap<word> &evk) const {
    const int dist = ((tokens % cfg_.seq_len) + cfg_.seq_len) % cfg_.seq_len * lane_;
    cx->HRot(res, a, evk.GetRotationKey(dist), dist);
  }

  // Head h: e_r = exp(s_r - R) for the 'seq_len' offsets r, stat = their mean
  // mapped to [-1, 1], o_un[d] = sum_r e_r * rot_r(V_d) (not yet normalised).
  void AttentionHead(int h, const std::vector<Ct> &qkv, std::vector<Ct> &o_un, Ct &stat,
                     const EvkMap<word> &evk) {
    const int H = cfg_.hidden, D = cfg_.head_dim, T = cfg_.seq_len, nb = cfg_.baby, ng = T / nb;
    const Evk &mult = evk.GetMultiplicationKey();
    auto Q = [&](int d) -> const Ct & { return qkv[h * D + d]; };
    auto K = [&](int d) -> const Ct & { return qkv[H + h * D + d]; };
    auto V = [&](int d) -> const Ct & { return qkv[2 * H + h * D + d]; };
    using Cx = ConstContextPtr<word>;
    std::vector<Ct> e(T);
    {
      // s_{g nb + b}[t] = sum_d Q_d[t] K_d[t + g nb + b]
      //                 = rot_{g nb}( sum_d rot_{-g nb}(Q_d) * rot_b(K_d) )[t]
      std::vector<std::vector<Ct>> kb(D), qg(ng);
      ParallelFor(D, [&](const Cx &c, int d) { BabyRotations(c, kb[d], K(d), evk); });
      for (int g = 1; g < ng; g++) qg[g].resize(D);
      ParallelFor((ng - 1) * D, [&](const Cx &c, int i) {
        const int g = 1 + i / D, d = i % D;
        RotateTokens(c, qg[g][d], Q(d), -g * nb, evk);
      });
      ParallelFor(T, [&](const Cx &c, int r) {
        const int g = r / nb, b = r % nb;
        Ct acc, u;
        std::vector<const Ct *> left(D), right(D);
        for (int d = 0; d < D; d++) {
          left[d] = g ? &qg[g][d] : &Q(d);
          right[d] = &kb[d][b];
        }
        c->MultSumUnsafe(acc, left, right);
        c->RelinearizeRescale(u, acc, mult);
        if (g) {
          Ct rot;
          RotateTokens(c, rot, u, g * nb, evk);
          u = std::move(rot);
        }
        Poly(c, e[r], u, polys_.exp_c, mult);
      });
    }
    {
      Ct sum;
      ctx_->Copy(sum, e[0]);
      for (int r = 1; r < T; r++) ctx_->Add(sum, sum, e[r]);
      const double span = cfg_.sum_hi - cfg_.sum_lo;
      MaskedAffine(stat, sum, 2.0 / (T * span), -(cfg_.sum_hi + cfg_.sum_lo) / span);
    }
    // o_d[t] = sum_g rot_{g nb}( sum_b rot_{-g nb}(e_{g nb + b}) * rot_b(V_d) )[t]
    const int le = Level(e[0]);
    std::vector<std::vector<Ct>> vb(D), eg(ng), part(ng);
    ParallelFor(D, [&](const Cx &c, int d) {
      Ct low;
      c->LevelDown(low, V(d), le);
      BabyRotations(c, vb[d], low, evk);
    });
    for (int g = 1; g < ng; g++) eg[g].resize(nb);
    ParallelFor((ng - 1) * nb, [&](const Cx &c, int i) {
      const int g = 1 + i / nb, b = i % nb;
      RotateTokens(c, eg[g][b], e[g * nb + b], -g * nb, evk);
    });
    for (int g = 0; g < ng; g++) part[g].resize(D);
    ParallelFor(ng * D, [&](const Cx &c, int i) {
      const int g = i / D, d = i % D;
      Ct acc, t;
      std::vector<const Ct *> left(nb), right(nb);
      for (int b = 0; b < nb; b++) {
        left[b] = g ? &eg[g][b] : &e[b];
        right[b] = &vb[d][b];
      }
      c->MultSumUnsafe(acc, left, right);
      c->RelinearizeRescale(t, acc, mult);
      if (g)
        RotateTokens(c, part[g][d], t, g * nb, evk);
      else
        part[0][d] = std::move(t);
    });
    ParallelFor(D, [&](const Cx &c, int d) {
      Ct &dst = o_un[h * D + d];
      c->Copy(dst, part[0][d]);
      for (int g = 1; g < ng; g++) c->Add(dst, dst, part[g][d]);
    });
  }

  // z[j] = gamma_j y[j] / sqrt(var + eps) + beta_j / act_div for centred y
  // (mean already removed), var = (act_div^2 / H) sum_j y[j]^2
  // This rank holds y[lo, hi) and produces z[lo, hi); the sum of squares
  // collects the ranks' partial sums (exact modular sums: any grouping gives
  // the same words), the statistic's bootstrap and series run on every rank.
  void LayerNorm(std::vector<Ct> &z, const std::vector<Ct> &y, const std::vector<double> &gamma,
                 const std::vector<double> &beta, const EvkMap<word> &evk, int lo, int hi) {
    const int H = y.size();
    const double A = cfg_.act_div, span = cfg_.var_hi - cfg_.var_lo;
    const Evk &mult = evk.GetMultiplicationKey();
    Ct acc, ss, w;
    {
      std::vector<const Ct *> mine;
      for (int j = lo; j < hi; j++) mine.push_back(&y[j]);
      ctx_->MultSumUnsafe(acc, mine, mine);
    }
    if (group_->world() > 1) {
      std::vector<Ct> parts(group_->world());
      parts[group_->rank()] = std::move(acc);
      AllGather(parts, [](int r) { return r; });
      acc = std::move(parts[0]);
      for (int r = 1; r < group_->world(); r++) ctx_->Add(acc, acc, parts[r]);
    }
    ctx_->RelinearizeRescale(ss, acc, mult);
    MaskedAffine(w, ss, 2.0 * A * A / (H * span), -(cfg_.var_hi + cfg_.var_lo) / span);
    std::vector<Ct> one(1);
    one[0] = std::move(w);
    BootAll(one, evk, true);
    Ct f;
    Poly(main_, f, one[0], polys_.rsqrt_c, mult);  // 1 / (2 sqrt(var + eps))
    const int target = Min(Level(f), Level(y[lo]) - 1);
    LevelTo(main_, f, target);
    z.clear();
    z.resize(H);
    ParallelFor(hi - lo, [&](const ConstContextPtr<word> &c, int i) {
      const int j = lo + i;
      Ct t;
      MultConstRescale(c, t, y[j], 2.0 * gamma[j]);
      LevelTo(c, t, target);
      c->HMult(z[j], t, f, mult);
      AddConst(c, z[j], beta[j] / A);
    });
  }

  // A statistic (softmax denominator, LayerNorm variance) is nearly the same
  // number in every slot, so its plaintext polynomial is one large coefficient,
  // and the sine that bootstrapping evaluates coefficient by coefficient is
  // only accurate to (2 pi c / q0)^2 / 6 relative on a coefficient c: half a
  // percent for a constant 0.8. Multiplying the slots by a fixed public pattern
  // of +-1 spreads the plaintext over all coefficients (each of size about
  // |value| / sqrt(n), as for random data); the same pattern takes it off after
  // the bootstrap. Both multiplications ride on constants that are needed anyway.
  const Plaintext<word> &Mask(int level, double scale, double factor) {
    const auto key = std::make_tuple(level, scale, factor);
    auto it = masks_.find(key);
    if (it == masks_.end()) {
      if (mask_signs_.empty()) {
        std::mt19937_64 gen(0x5EEDull);
        mask_signs_.resize(slots_);
        for (auto &v : mask_signs_) v = (gen() & 1) ? 1.0 : -1.0;
      }
      std::vector<Complex> msg(slots_);
      for (int i = 0; i < slots_; i++) msg[i] = Complex(mask_signs_[i] * factor, 0.0);
      Plaintext<word> pt;
      ctx_->encoder().Encode(pt, level, scale, msg, 0);
      it = masks_.emplace(key, std::move(pt)).first;
    }
    return it->second;
  }
  // res = mask * (mul * a + add), one level below a at the canonical scale
  void MaskedAffine(Ct &res, const Ct &a, double mul, double add) {
    const int l = Level(a);
    Ct t;
    ctx_->Mult(t, a, Mask(l, Canon(l - 1) * ctx_->param_.GetRescalePrimeProd(l) / a.GetScale(), mul));
    ctx_->Rescale(res, t);
    ctx_->Add(res, res, Mask(l - 1, res.GetScale(), add));
  }
  void MultMaskRescale(Ct &res, const Ct &a, double factor) {
    const int l = Level(a);
    Ct t;
    ctx_->Mult(t, a, Mask(l, Canon(l - 1) * ctx_->param_.GetRescalePrimeProd(l) / a.GetScale(), factor));
    ctx_->Rescale(res, t);
  }

  // Refreshes every ciphertext. Slot values are real, so two ciphertexts ride
  // through one bootstrap as a + i b and are separated by the conjugate
  // afterwards: a = (c + conj c) / 2, b = (c - conj c) / 2i. The halving is
  // one constant product with a rescale, so a pair-bootstrapped ciphertext
  // ends one level lower. masked: the inputs carry the +-1 pattern of Mask,
  // taken off by the same product.
  void BootAll(std::vector<Ct> &v, const EvkMap<word> &evk, bool masked = false) {
    const size_t n = v.size();
    auto finish = [&](Ct &dst, Ct &src, double factor, bool needed) {
      if (masked) {
        MultMaskRescale(dst, src, factor);
      } else if (needed) {
        MultConstRescale(main_, dst, src, factor);
      } else {
        dst = std::move(src);
      }
    };
    // statistics go through one by one: they are few, and which heads share a
    // bootstrap would otherwise depend on how many ranks the heads are spread over
    const bool pairs = cfg_.pair_boot && n > 1 && !masked;
    const Evk &conj = evk.GetConjugationKey();
    for (size_t i = 0; i < n; i += 2) {
      if (!pairs || i + 1 == n) {
        for (size_t j = i; j < Min(i + 2, n); j++) {
          Ct fresh;
          ctx_->Boot(fresh, v[j], evk);
          boots_++;
          finish(v[j], fresh, 1.0, pairs);  // in a paired run every output ends on one level
        }
        continue;
      }
      Ct im, both, fresh, cj, re2, im2;
      ctx_->MultImaginaryUnit(im, v[i + 1]);
      ctx_->Add(both, v[i], im);
      ctx_->Boot(fresh, both, evk);
      boots_++;
      ctx_->HConj(cj, fresh, conj);
      ctx_->Add(re2, fresh, cj);  // 2 a
      ctx_->Sub(im2, cj, fresh);  // -2 i b
      ctx_->MultImaginaryUnit(im2, im2);  // 2 b
      finish(v[i], re2, 0.5, true);
      finish(v[i + 1], im2, 0.5, true);
    }
  }

  std::shared_ptr<Boot> ctx_;
  ConstContextPtr<word> main_;                 // ctx_ as the type the operators take
  std::vector<ContextPtr<word>> workers_;      // one more engine context per extra host thread
  TransformerConfig cfg_;
  TransformerWeights w_;
  TransformerPolys polys_;
  std::shared_ptr<RankGroup> group_;
  int slots_ = 0, lane_ = 0;
  std::unique_ptr<PlainMatrix<word>> m_qkv_, m_wo_, m_w1_, m_w2_, m_res_;
  Probe probe_;
  std::map<std::tuple<int, double, double>, Plaintext<word>> masks_;
  std::vector<double> mask_signs_;
  std::vector<std::pair<std::string, double>> stage_s_;
  std::chrono::steady_clock::time_point last_;
  double gemm_s_ = 0, gemm_macs_ = 0, pack_s_ = 0;
  int boots_ = 0;
};

}  // namespace cheddar
