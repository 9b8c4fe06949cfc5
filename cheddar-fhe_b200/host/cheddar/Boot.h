// Bootstrapping on top of the operator API (host-side planning in C++; every
// GPU step is a C-ABI call made through Context).
//
// Class names follow the reference's extension (include/extension/
// StripedMatrix.h, LinearTransform.h, EvalPoly.h, EvalMod.h, EvalSpecialFFT.h,
// BootParameter.h, BootContext.h); the pipeline is the same mathematics
//   scale up -> ModUpToMax (with sparse-secret encapsulation) -> CoeffToSlot
//   -> EvalMod on the real and imaginary parts -> SlotToCoeff
// (reference src/extension/BootContext.cpp:299-365) with its own planning:
//  * linear transforms are diagonal (striped) matrices evaluated by
//    baby-step/giant-step, the baby rotations sharing one ModUp (hoisting);
//  * CoeffToSlot and SlotToCoeff are merged groups of radix-2 stages of the
//    encoder's special (I)FFT (reference src/core/Encode.cpp:85-133), one
//    group per level the BootParameter grants them;
//  * polynomials are evaluated in the Chebyshev basis by recursive splitting
//    p = q * T_m + r (depth ceil(log2(degree + 1))) with exact scale tracking:
//    every sum is formed at one agreed scale before a single rescale, the
//    constants carrying whatever factor that takes, so rational rescaling
//    (levels whose prime products differ) costs no precision and no level;
//  * EvalMod is an even Chebyshev series of degree 30 for
//    (1/2pi)^(1/8) cos(2pi(K t - 1/4)/8), evaluated as a degree-15 series in
//    T_2(t) (five levels), followed by three double-angle steps (reference
//    src/extension/EvalMod.cpp:8-61 uses the same function with K = 16 and
//    the same eight levels).
// Any power-of-two slot count up to 2^(logN-1): fewer slots go through Trace
// onto the subring and transforms with periodic diagonals.
#pragma once
#include <chrono>
#include <functional>
#include <set>

#include "cheddar/Cheddar.h"

namespace cheddar {

// ------------------------------------------------------------ StripedMatrix
// (M v)[p] = sum_k diag[k][p] * v[(p + k) mod n]
struct StripedMatrix {
  int n = 0;
  std::map<int, std::vector<Complex>> diag;

  explicit StripedMatrix(int size = 0) : n(size) {}
  // the reference's form (include/extension/StripedMatrix.h:11-31): a map from
  // diagonal offset to diagonal, square matrices only here
  StripedMatrix(int height, int width) : n(height) {
    AssertTrue(height == width, "StripedMatrix: square matrices only");
  }
  int GetHeight() const { return n; }
  int GetWidth() const { return n; }
  int GetNumDiag() const { return (int)diag.size(); }
  auto begin() const { return diag.begin(); }
  auto end() const { return diag.end(); }
  auto find(int k) const { return diag.find(k); }
  std::vector<Complex> &operator[](int k) { return At(k); }
  static StripedMatrix Mult(const StripedMatrix &A, const Complex b) {
    StripedMatrix C = A;
    C.Scale(b);
    return C;
  }
  std::vector<Complex> &At(int k) {
    k = ((k % n) + n) % n;
    auto it = diag.find(k);
    if (it == diag.end()) it = diag.emplace(k, std::vector<Complex>(n, Complex(0, 0))).first;
    return it->second;
  }
  // A * B (B is applied first)
  static StripedMatrix Mult(const StripedMatrix &A, const StripedMatrix &B) {
    StripedMatrix C(A.n);
    for (auto &[k, a] : A.diag)
      for (auto &[l, b] : B.diag) {
        auto &c = C.At(k + l);
        for (int p = 0; p < A.n; p++) c[p] += a[p] * b[(p + k) % A.n];
      }
    return C;
  }
  void Scale(Complex s) {
    for (auto &[k, d] : diag)
      for (auto &x : d) x *= s;
  }
  std::vector<Complex> Apply(const std::vector<Complex> &v) const {
    std::vector<Complex> r(n, Complex(0, 0));
    for (auto &[k, d] : diag)
      for (int p = 0; p < n; p++) r[p] += d[p] * v[(p + k) % n];
    return r;
  }
};

// ------------------------------------------------------------ LinearTransform
// res = Rescale( sum_k diag_k (*) rot_k(in) ) by baby-step/giant-step, run by
// one engine call (cfhe_linear_transform) that hoists both the baby and the
// giant steps.
template <typename word>
class LinearTransform {
  using Ct = Ciphertext<word>;
  using Pt = Plaintext<word>;

 public:
  // The plaintext diagonals are encoded at `level`, on the auxiliary primes as
  // well, with the scale that makes the output scale scale_out for an input of
  // scale scale_in. baby_steps <= 16.
  LinearTransform(const ConstContextPtr<word> &ctx, const StripedMatrix &m, int level, double scale_in,
                  double scale_out, int baby_steps = 16)
      : level_(level), bs_(baby_steps), n_(m.n), scale_out_(scale_out) {
    const auto &param = ctx->param_;
    AssertTrue(level > 0, "LinearTransform needs a level that can be rescaled");
    AssertTrue(bs_ >= 1 && bs_ <= 16, "LinearTransform: 1 to 16 baby steps");
    const double pt_scale = param.GetRescalePrimeProd(level) * (scale_out / scale_in);
    // stride g = gcd of the offsets and n; signed multiples t in (-n/2g, n/2g]
    int g = n_;
    for (auto &[k, d] : m.diag)
      if (k) g = std::gcd(g, k);
    const int period = n_ / g;
    int tmin = 0, tmax = 0;
    std::map<int, const std::vector<Complex> *> by_t;
    for (auto &[k, d] : m.diag) {
      int t = k / g;
      if (t > period / 2) t -= period;
      by_t[t] = &d;
      tmin = std::min(tmin, t);
      tmax = std::max(tmax, t);
    }
    // giant offsets are multiples of bs, so one of them is zero whenever the
    // range of t includes it (one key switch fewer)
    const int t0 = (int)std::floor((double)tmin / bs_) * bs_;
    g_ = g % n_;
    giant_stride_ = Mod((long long)g * bs_);
    giant_first_ = Mod((long long)g * t0);
    // giant steps form the progression giant_first_ + jj * giant_stride_ (mod n);
    // offsets wrap modulo n, so different multiples can be the same rotation
    const int wrap = giant_stride_ ? n_ / std::gcd(giant_stride_, n_) : 1;
    std::map<int, int> jj_of;              // giant rotation -> position in the progression
    std::map<int, std::map<int, Pt>> pts;  // [giant rotation][baby index]
    std::set<int> babies{0};
    for (auto &[t, d] : by_t) {
      const int j = (t - t0) / bs_, i = (t - t0) % bs_;
      const int G = Mod((long long)g * (t0 + bs_ * j));
      jj_of[G] = j % wrap;
      // the giant rotation is applied after the product: pre-rotate by -G
      std::vector<Complex> v(n_);
      for (int p = 0; p < n_; p++) v[p] = (*d)[Mod((long long)p - G)];
      AssertTrue(!pts[G].count(i), "LinearTransform: two diagonals share a slot");
      ctx->encoder().Encode(pts[G][i], level, pt_scale, v, param.alpha_);
      babies.insert(i);
    }
    std::map<int, int> baby_slot;
    for (int i : babies) {
      baby_slot[i] = baby_rot_.size();
      baby_rot_.push_back(Mod((long long)g * i));
      baby_idx_.push_back(i);
    }
    for (auto &[G, row] : pts) {
      giant_rot_.push_back(G);
      giant_jj_.push_back(jj_of.at(G));
      std::vector<Pt> dense(baby_rot_.size());
      std::vector<bool> have(baby_rot_.size(), false);
      for (auto &[i, pt] : row) {
        dense[baby_slot.at(i)] = std::move(pt);
        have[baby_slot.at(i)] = true;
      }
      for (size_t k = 0; k < dense.size(); k++) {
        pts_.push_back(std::move(dense[k]));
        present_.push_back(have[k]);
      }
    }
    AssertTrue(giant_rot_.size() <= 16, "LinearTransform: more than 16 giant steps");
  }

  // The reference's constructor (include/extension/LinearTransform.h:43-46,
  // src/extension/LinearTransform.cpp:8-93): plaintexts at pt_level with scale
  // pt_scale, the output scale follows from the input's
  // (in.scale * pt_scale / rescaling ratio of pt_level). Diagonal i acts on the
  // input rotated by i - pre_rotation, and every plaintext is additionally
  // turned by additional_pt_rot slots:
  //   out[p] = sum_i diag_i[p + additional_pt_rot] * in[p + i - pre_rotation].
  // bs * gs must cover the diagonals as in the reference; the giant steps are
  // then planned by this class (gs is an upper bound, not a layout).
  LinearTransform(const ConstContextPtr<word> &ctx, const StripedMatrix &matrix, int pt_level, double pt_scale,
                  int bs, int gs = 1, int pre_rotation = 0, int additional_pt_rot = 0)
      : LinearTransform(ctx, Shifted(matrix, bs, gs, pre_rotation, additional_pt_rot), pt_level, 1.0,
                        pt_scale / ctx->param_.GetRescalePrimeProd(pt_level), bs > 16 ? 16 : bs) {
    relative_scale_ = true;
    ref_bs_ = bs;
    ref_gs_ = gs;
    pre_rotation_ = pre_rotation;
  }
  bool IsUsingBSGS() const { return ref_bs_ > 1 && ref_gs_ > 1; }
  int GetBS() const { return ref_bs_; }
  int GetGS() const { return ref_gs_; }
  int GetPreRotationAmount() const { return pre_rotation_; }
  void AddRequiredRotations(EvkRequest &req, bool min_ks = false) const {
    std::set<int> rots;
    AddRequiredRotations(rots, min_ks);
    for (int r : rots) req.AddRequest(r, level_);
  }

  // min_ks: the plan that needs at most three keys per transform (the baby
  // stride, the giant stride and the first giant offset), at the price of
  // sequential, unhoisted rotations (the reference's minimum key-switching
  // mode, src/extension/Hoist.cu:979-985).
  void AddRequiredRotations(std::set<int> &rots, bool min_ks = false) const {
    if (min_ks) {
      if (baby_idx_.back() > 0) rots.insert(g_);
      int jmax = 0;
      for (int jj : giant_jj_) jmax = Max(jmax, jj);
      if (jmax > 0 && giant_stride_) rots.insert(giant_stride_);
      if (giant_first_) rots.insert(giant_first_);
      return;
    }
    for (int r : baby_rot_)
      if (r) rots.insert(r);
    for (int r : giant_rot_)
      if (r) rots.insert(r);
  }

  void Evaluate(const ConstContextPtr<word> &ctx, Ct &res, const Ct &in, const EvkMap<word> &keys,
                bool min_ks = false) const {
    if (min_ks) {
      EvaluateMinKS(ctx, res, in, keys);
      return;
    }
    const auto &param = ctx->param_;
    AssertTrue(param.NPToLevel(in.GetNP()) == level_, "LinearTransform: wrong input level");
    AssertFalse(in.HasRx(), "LinearTransform: relinearize first");
    const int beta = cfhe_beta(ctx->h_, level_);
    int key_main = -1;
    auto gather = [&](const std::vector<int> &rots, std::vector<const word *> &kb,
                      std::vector<const word *> &ka) {
      for (int r : rots)
        for (int d = 0; d < beta; d++) {
          if (!r) {
            kb.push_back(nullptr);
            ka.push_back(nullptr);
            continue;
          }
          const auto &key = keys.GetRotationKey(r);
          AssertTrue(key.GetBeta() >= beta, "Beta mismatch");
          AssertTrue(key_main < 0 || key_main == key.GetNP().num_main_, "LinearTransform: key shapes differ");
          key_main = key.GetNP().num_main_;
          kb.push_back(key.bx_[d].data());
          ka.push_back(key.ax_[d].data());
        }
    };
    std::vector<const word *> bkb, bka, gkb, gka, pt;
    gather(baby_rot_, bkb, bka);
    gather(giant_rot_, gkb, gka);
    for (size_t k = 0; k < pts_.size(); k++) pt.push_back(present_[k] ? pts_[k].mx_.data() : nullptr);
    Ct out(param.LevelToNP(level_ - 1));
    CheckAbi(cfhe_linear_transform(ctx->h_, level_, 1, out.bx_.data(), out.ax_.data(), in.bx_.data(),
                                   in.ax_.data(), baby_rot_.size(), baby_rot_.data(), bkb.data(), bka.data(),
                                   giant_rot_.size(), giant_rot_.data(), gkb.data(), gka.data(), pt.data(),
                                   Max(key_main, 0)));
    out.SetScale(relative_scale_ ? in.GetScale() * scale_out_ : scale_out_);
    out.SetNumSlots(in.GetNumSlots());
    res = std::move(out);
  }

  // Baby rotations one after the other with the key of the baby stride, the
  // giant sums folded Horner-wise with the key of the giant stride:
  //   out = rot_first( acc_0 + rot_S( acc_1 + rot_S( acc_2 + ... ) ) )
  void EvaluateMinKS(const ConstContextPtr<word> &ctx, Ct &res, const Ct &in, const EvkMap<word> &keys) const {
    const auto &param = ctx->param_;
    AssertTrue(param.NPToLevel(in.GetNP()) == level_, "LinearTransform: wrong input level");
    AssertFalse(in.HasRx(), "LinearTransform: relinearize first");
    const int nb = baby_rot_.size(), top = baby_idx_.back();
    std::vector<Ct> store(top + 1);
    std::vector<const Ct *> rot(top + 1, nullptr);
    rot[0] = &in;
    for (int i = 1; i <= top; i++) {
      ctx->HRot(store[i], *rot[i - 1], keys.GetRotationKey(g_), g_);
      rot[i] = &store[i];
    }
    int jmax = 0;
    for (int jj : giant_jj_) jmax = Max(jmax, jj);
    std::vector<Ct> acc(jmax + 1);
    std::vector<bool> have(jmax + 1, false);
    Ct term;
    for (size_t gi = 0; gi < giant_rot_.size(); gi++) {
      const int jj = giant_jj_[gi];
      for (int k = 0; k < nb; k++) {
        if (!present_[gi * nb + k]) continue;
        const Ct &r = *rot[baby_idx_[k]];
        if (!have[jj]) {
          ctx->MultUnsafe(acc[jj], r, pts_[gi * nb + k], level_);  // the Q limbs of the extended plaintext
          have[jj] = true;
        } else {
          ctx->MultUnsafe(term, r, pts_[gi * nb + k], level_);
          ctx->Add(acc[jj], acc[jj], term);
        }
      }
    }
    Ct sum, turned;
    bool started = false;
    for (int jj = jmax; jj >= 0; jj--) {
      if (started && giant_stride_) {
        if (have[jj]) {
          ctx->HRotAdd(turned, sum, acc[jj], keys.GetRotationKey(giant_stride_), giant_stride_);
        } else {
          ctx->HRot(turned, sum, keys.GetRotationKey(giant_stride_), giant_stride_);
        }
        sum = std::move(turned);
      } else if (have[jj]) {
        if (started) {
          ctx->Add(sum, sum, acc[jj]);
        } else {
          sum = std::move(acc[jj]);
          started = true;
        }
      }
    }
    AssertTrue(started, "LinearTransform: empty matrix");
    if (giant_first_) {
      ctx->HRot(turned, sum, keys.GetRotationKey(giant_first_), giant_first_);
      sum = std::move(turned);
    }
    ctx->Rescale(res, sum);
    res.SetScale(relative_scale_ ? in.GetScale() * scale_out_ : scale_out_);
  }

  int level() const { return level_; }
  double OutputScaleFactor() const { return scale_out_; }  // output scale for an input of scale 1
  int NumBabySteps() const { return baby_rot_.size(); }
  int NumGiantSteps() const { return giant_rot_.size(); }

 private:
  // the reference constructor's matrix in this class's convention
  static StripedMatrix Shifted(const StripedMatrix &m, int bs, int gs, int pre_rotation, int additional_pt_rot) {
    const int n = m.GetWidth();
    AssertTrue(n > 0 && (n & (n - 1)) == 0, "LinearTransform requires power-of-two width");
    AssertTrue(m.GetNumDiag() > 1, "LinearTransform requires at least 2 plaintexts");
    StripedMatrix out(n);
    int g = 0, max_rot = 0;
    for (const auto &[i, d] : m) {
      const int rot = (((i - pre_rotation) % n) + n) % n;
      g = std::gcd(g, rot);
      max_rot = std::max(max_rot, rot);
      auto &o = out.At(rot);
      for (int p = 0; p < n; p++) o[p] = d[(((p + additional_pt_rot) % n) + n) % n];
    }
    AssertTrue(g > 0, "Something went wrong during LinearTransform setup");
    AssertTrue(max_rot <= (bs * gs - 1) * g,
               "Incompatible matrix and LinearTransform parameters: bs (" + std::to_string(bs) + "), gs (" +
                   std::to_string(gs) + "), pre_rotation (" + std::to_string(pre_rotation) + ")");
    return out;
  }
  int Mod(long long x) const { return (int)(((x % n_) + n_) % n_); }
  int level_, bs_, n_;
  double scale_out_;
  bool relative_scale_ = false;  // scale_out_ multiplies the input's scale (reference-shaped constructor)
  int ref_bs_ = 0, ref_gs_ = 0, pre_rotation_ = 0;
  int g_ = 0, giant_stride_ = 0, giant_first_ = 0;  // slot distances of the min_ks plan
  std::vector<int> baby_idx_, giant_jj_;            // baby multiple / giant position per entry
  std::vector<int> baby_rot_, giant_rot_;  // slot distances; baby_rot_[0] == 0
  std::vector<Pt> pts_;                    // [giant][baby], dense
  std::vector<bool> present_;
};

// ------------------------------------------------------------ HoistHandler
// The reference's baby-step/giant-step evaluator (include/extension/Hoist.h:28-104):
//   res = Rescale( sum_gs rot_gs( sum_bs hoist_map[gs][bs] (*) rot_bs(input) ) ).
// Here it is an adapter: the map is turned back into the striped matrix it
// came from (plaintext gs/bs holds diagonal gs + bs turned by gs slots) and
// handed to LinearTransform, whose single engine call hoists both kinds of step.
using Message = std::vector<Complex>;
using PlainHoistMap = std::map<int, std::map<int, Message>>;

template <typename word>
class HoistHandler {
  using Ct = Ciphertext<word>;

 public:
  HoistHandler(const ConstContextPtr<word> &context, const PlainHoistMap &hoist_map, int pt_level, double pt_scale,
               bool suppress_bs_swap = false)
      : lt_(context, ToMatrix(hoist_map), pt_level, 1.0,
            pt_scale / context->param_.GetRescalePrimeProd(pt_level), BabySteps(hoist_map)),
        pt_level_(pt_level) {
    (void)suppress_bs_swap;  // a layout choice of the reference's kernels
  }
  HoistHandler(const HoistHandler &) = delete;
  HoistHandler &operator=(const HoistHandler &) = delete;
  HoistHandler(HoistHandler &&) = default;

  void AddRequiredRotations(EvkRequest &req, bool min_ks = false) const {
    std::set<int> rots;
    lt_.AddRequiredRotations(rots, min_ks);
    for (int r : rots) req.AddRequest(r, pt_level_);
  }
  void Evaluate(const ConstContextPtr<word> &context, Ct &res, const Ct &input, const EvkMap<word> &evk_map,
                bool min_ks = false) const {
    const double in_scale = input.GetScale();
    lt_.Evaluate(context, res, input, evk_map, min_ks);
    res.SetScale(in_scale * lt_.OutputScaleFactor());
  }

 private:
  static StripedMatrix ToMatrix(const PlainHoistMap &map) {
    AssertTrue(!map.empty() && !map.begin()->second.empty(), "HoistHandler: empty map");
    const int n = (int)map.begin()->second.begin()->second.size();
    StripedMatrix m(n);
    for (const auto &[gs, row] : map)
      for (const auto &[bs, pt] : row) {
        AssertTrue((int)pt.size() == n, "HoistHandler: plaintexts of different sizes");
        auto &d = m.At(gs + bs);
        for (int p = 0; p < n; p++) d[p] = pt[(((p + gs) % n) + n) % n];
      }
    return m;
  }
  static int BabySteps(const PlainHoistMap &map) {
    std::set<int> bs;
    for (const auto &[gs, row] : map)
      for (const auto &[b, pt] : row) bs.insert(b);
    int k = 1;
    while (k < (int)bs.size()) k <<= 1;
    return std::min(k, 16);
  }
  LinearTransform<word> lt_;
  int pt_level_;
};

// ------------------------------------------------------------ EvalPoly
// Chebyshev-basis polynomial evaluation with exact scale tracking.
template <typename word>
class EvalPoly {
  using Ct = Ciphertext<word>;
  using Evk = EvaluationKey<word>;

 public:
  // ---- the reference's object interface (include/extension/EvalPoly.h:203-223) ----
  // coefficients[k] multiplies x^k, or T_k(x) when `chebyshev` is set. The
  // result sits ceil(log2(#coefficients)) levels below input_level at scale
  // target_scale. Evaluation always runs in the Chebyshev basis (the power
  // basis is converted exactly, as a polynomial identity), with the
  // recursive splitting of EvaluateChebyshev below.
  EvalPoly(const std::vector<double> &coefficients, int input_level, double input_scale, double target_scale,
           bool chebyshev = false)
      : coefficients_(coefficients),
        chebyshev_(chebyshev),
        input_level_(input_level),
        input_scale_(input_scale),
        target_scale_(target_scale) {
    AssertTrue(!coefficients_.empty(), "EvalPoly: no coefficients");
  }
  EvalPoly(const EvalPoly &) = delete;
  EvalPoly &operator=(const EvalPoly &) = delete;
  EvalPoly(EvalPoly &&) = default;

  int GetPolyDegree() const {
    int d = (int)coefficients_.size() - 1;
    while (d > 0 && coefficients_[d] == 0.0) d--;
    return d;
  }
  void ConvertToChebyshevBasis() {
    if (chebyshev_) return;
    coefficients_ = PowerToChebyshev(coefficients_);
    chebyshev_ = true;
  }
  void ConvertToNormalBasis() {
    if (!chebyshev_) return;
    coefficients_ = ChebyshevToPower(coefficients_);
    chebyshev_ = false;
  }
  // Fixes the evaluation plan: the Chebyshev coefficients and the level budget.
  void Compile(const ConstContextPtr<word> &context) {
    compiled_ = chebyshev_ ? coefficients_ : PowerToChebyshev(coefficients_);
    int k = 1;
    while ((size_t(1) << k) < compiled_.size()) k++;
    AssertTrue(input_level_ - k >= 0 && input_level_ <= context->param_.max_level_,
               "EvalPoly: not enough levels below the input level");
  }
  void Evaluate(const ConstContextPtr<word> &context, Ct &res, const Ct &input, const Evk &mult_key) const {
    AssertTrue(!compiled_.empty(), "EvalPoly: Compile first");
    AssertTrue(context->param_.NPToLevel(input.GetNP()) == input_level_, "EvalPoly: wrong input level");
    context->AssertSameScale(input.GetScale(), input_scale_);
    EvaluateChebyshev(context, res, input, compiled_, mult_key, target_scale_);
  }
  double PlainEvaluate(double x) const {
    if (!chebyshev_) {
      double r = 0;
      for (int k = (int)coefficients_.size() - 1; k >= 0; k--) r = r * x + coefficients_[k];
      return r;
    }
    double b1 = 0, b2 = 0;  // Clenshaw
    for (int k = (int)coefficients_.size() - 1; k >= 1; k--) {
      const double b0 = coefficients_[k] + 2 * x * b1 - b2;
      b2 = b1;
      b1 = b0;
    }
    return coefficients_[0] + x * b1 - b2;
  }
  // x^k as a combination of T_0..T_k and back (long double, exact to rounding)
  static std::vector<double> PowerToChebyshev(const std::vector<double> &a) {
    const int n = a.size();
    std::vector<long double> c(n, 0.0L), xk(n, 0.0L), next(n);
    xk[0] = 1.0L;  // x^0 = T_0
    for (int k = 0; k < n; k++) {
      for (int j = 0; j <= k; j++) c[j] += (long double)a[k] * xk[j];
      // x * T_j = (T_{j+1} + T_{|j-1|}) / 2
      std::fill(next.begin(), next.end(), 0.0L);
      for (int j = 0; j <= k && k + 1 < n; j++) {
        if (j == 0) {
          next[1] += xk[0];
        } else {
          next[j + 1] += xk[j] / 2;
          next[j - 1] += xk[j] / 2;
        }
      }
      xk = next;
    }
    return std::vector<double>(c.begin(), c.end());
  }
  static std::vector<double> ChebyshevToPower(const std::vector<double> &c) {
    const int n = c.size();
    std::vector<long double> a(n, 0.0L), t0(n, 0.0L), t1(n, 0.0L), t2(n);
    t0[0] = 1.0L;
    if (n > 1) t1[1] = 1.0L;
    for (int k = 0; k < n; k++) {
      const auto &tk = k == 0 ? t0 : t1;
      for (int j = 0; j <= k; j++) a[j] += (long double)c[k] * tk[j];
      if (k >= 1) {  // T_{k+1} = 2 x T_k - T_{k-1}
        std::fill(t2.begin(), t2.end(), 0.0L);
        for (int j = 0; j <= k && j + 1 < n; j++) t2[j + 1] += 2 * t1[j];
        for (int j = 0; j < k; j++) t2[j] -= t0[j];
        t0 = t1;
        t1 = t2;
      }
    }
    return std::vector<double>(a.begin(), a.end());
  }

 private:
  std::vector<double> coefficients_, compiled_;
  bool chebyshev_ = true;
  int input_level_ = 0;
  double input_scale_ = 0, target_scale_ = 0;

 public:
  // ---- the static form used by EvalMod ----
  // res = 2*A*B - C (C may be null: 2*A*B - c0 with the real constant c0),
  // one level below min(level A, level B). Everything is subtracted from the
  // unrelinearised product, so the node costs one RelinearizeRescale.
  static void Node(const ConstContextPtr<word> &ctx, Ct &res, const Ct &A, const Ct &B, const Ct *C,
                   double c0, const Evk &mult_key) {
    const auto &param = ctx->param_;
    const int la = param.NPToLevel(A.GetNP()), lb = param.NPToLevel(B.GetNP());
    const int l = Min(la, lb);
    Ct prod, lowered;
    const NPInfo np = param.LevelToNP(l);
    if (np.IsSubsetOf(A.GetNP()) && np.IsSubsetOf(B.GetNP())) {
      ctx->MultUnsafe(prod, A, B, l);  // operands of a higher level are read in place
    } else {
      // levels that do not nest (rational rescaling): bring the higher operand down
      ctx->LevelDown(lowered, la > lb ? A : B, l);
      ctx->MultUnsafe(prod, la > lb ? lowered : A, la > lb ? B : lowered, l);
    }
    ctx->Add(prod, prod, prod);
    const double s = prod.GetScale();
    if (C) {
      Ct cs, c_low;
      const Ct *c_at = C;
      if (!np.IsSubsetOf(C->GetNP())) {
        ctx->LevelDown(c_low, *C, l);
        c_at = &c_low;
      }
      Constant<word> one;
      ctx->encoder().EncodeConstant(one, l, s / c_at->GetScale(), 1.0, 0);
      ctx->MultUnsafe(cs, *c_at, one, l);
      cs.SetScale(s);
      ctx->Sub(prod, prod, cs);
    } else if (c0 != 0.0) {
      Constant<word> k;
      ctx->encoder().EncodeConstant(k, l, s, c0, 0);
      ctx->Sub(prod, prod, k);
    }
    ctx->RelinearizeRescale(res, prod, mult_key);
  }

  // Rescale of a sum that may still carry unrelinearised products
  static void Finish(const ConstContextPtr<word> &ctx, Ct &res, const Ct &sum, const Evk &mult_key) {
    if (sum.HasRx())
      ctx->RelinearizeRescale(res, sum, mult_key);
    else
      ctx->Rescale(res, sum);
  }

  // res = sum_k coeffs[k] T_k(x), x with slot values in [-1, 1]. The result
  // sits ceil(log2(#coeffs)) levels below x, at scale target_scale.
  static void EvaluateChebyshev(const ConstContextPtr<word> &ctx, Ct &res, const Ct &x,
                                const std::vector<double> &coeffs, const Evk &mult_key,
                                double target_scale) {
    const auto &param = ctx->param_;
    std::vector<double> c = coeffs;
    while (c.size() > 2 && c.back() == 0.0) c.pop_back();
    int k = 1;
    while ((size_t(1) << k) < c.size()) k++;
    // T_1, T_2, T_4, ... each one level below the previous
    Basis T;
    ctx->Copy(T.top[1], x);
    for (int j = 1; j < k; j++)
      Node(ctx, T.top[1 << j], T.top.at(1 << (j - 1)), T.top.at(1 << (j - 1)), nullptr, 1.0, mult_key);
    const int top = param.NPToLevel(x.GetNP()) - (k - 1);
    AssertTrue(top > 0, "EvaluateChebyshev: not enough levels");
    Ct sum;
    Sum(ctx, sum, c, target_scale * param.GetRescalePrimeProd(top), top, T, mult_key);
    Finish(ctx, res, sum, mult_key);
  }

 private:
  // res = sum_k c[k] T_k at level `level`, at scale W, not yet rescaled and
  // with its products not yet relinearised (all products formed at one level
  // share the relinearisation that Finish performs).
  // T_{m+j} = 2 T_m T_j - T_{m-j} turns p into q * T_m + r with
  //   q_0 = c_m, q_j = 2 c_{m+j};  r_0 = c_0, r_k = c_k - c_{2m-k}.
  // T_1, T_2, T_4, ... as computed, and their copies on lower levels for the
  // parameter sets whose levels do not nest (a product reads the limbs of its
  // own level in place out of a higher operand only when they are all there;
  // otherwise the operand is brought down with LevelDown, once per level, as
  // the reference does with its MultiLevelCiphertext, src/extension/EvalPoly.cpp:408-661)
  struct Basis {
    std::map<int, Ct> top;
    std::map<std::pair<int, int>, Ct> low;
    const Ct &At(const ConstContextPtr<word> &ctx, int m, int level) {
      const Ct &t = top.at(m);
      if (ctx->param_.LevelToNP(level).IsSubsetOf(t.GetNP())) return t;
      auto it = low.find({m, level});
      if (it == low.end()) {
        // start from the lowest copy above `level` that exists already
        const Ct *from = &t;
        auto above = low.upper_bound({m, level});
        if (above != low.end() && above->first.first == m) from = &above->second;
        Ct down;
        ctx->LevelDown(down, *from, level);
        it = low.emplace(std::make_pair(m, level), std::move(down)).first;
      }
      return it->second;
    }
  };
  static void Sum(const ConstContextPtr<word> &ctx, Ct &res, const std::vector<double> &c, double W,
                  int level, Basis &T, const Evk &mult_key) {
    const auto &param = ctx->param_;
    const int len = c.size();
    auto add_const = [&](Ct &ct, double v) {
      if (v == 0.0) return;
      Constant<word> k0;
      ctx->encoder().EncodeConstant(k0, level, W, v, 0);
      ctx->Add(ct, ct, k0);
    };
    auto scaled = [&](Ct &out, const Ct &basis, double v) {  // v * basis at scale W
      Constant<word> k1;
      ctx->encoder().EncodeConstant(k1, level, W / basis.GetScale(), v, 0);
      ctx->MultUnsafe(out, basis, k1, level);
      out.SetScale(W);
    };
    if (len <= 2) {
      scaled(res, T.At(ctx, 1, level), len == 2 ? c[1] : 0.0);
      add_const(res, c[0]);
      return;
    }
    int m = 1;
    while (2 * m < len) m *= 2;
    std::vector<double> q(len - m), r(m);
    q[0] = c[m];
    for (int j = 1; j < len - m; j++) q[j] = 2.0 * c[m + j];
    for (int i = 0; i < m; i++) r[i] = c[i] - (i > 0 && 2 * m - i < len ? c[2 * m - i] : 0.0);
    Ct high;
    if (q.size() == 1) {
      scaled(high, T.At(ctx, m, level), q[0]);
    } else {
      Ct qsum, qv;
      const Ct &tm = T.At(ctx, m, level);
      Sum(ctx, qsum, q, (W / tm.GetScale()) * param.GetRescalePrimeProd(level + 1), level + 1, T, mult_key);
      Finish(ctx, qv, qsum, mult_key);
      ctx->MultUnsafe(high, qv, tm, level);
      high.SetScale(W);
    }
    bool r_zero = true;
    for (double v : r) r_zero = r_zero && v == 0.0;
    if (r_zero) {
      res = std::move(high);
      return;
    }
    while (r.size() > 1 && r.back() == 0.0) r.pop_back();
    if (r.size() == 1) {
      res = std::move(high);
      add_const(res, r[0]);
      return;
    }
    Ct low;
    Sum(ctx, low, r, W, level, T, mult_key);
    ctx->Add(res, high, low);
  }

 public:
  // Chebyshev coefficients of f on [-1,1] (interpolation at `points` nodes)
  static std::vector<double> ChebyshevCoefficients(const std::function<double(double)> &f, int degree,
                                                   int points = 256) {
    std::vector<double> c(degree + 1, 0.0);
    for (int k = 0; k <= degree; k++) {
      long double s = 0;
      for (int j = 0; j < points; j++) {
        const long double th = M_PIl * (j + 0.5L) / points;
        s += (long double)f((double)std::cos(th)) * std::cos(k * th);
      }
      c[k] = (double)(s * (k == 0 ? 1.0L : 2.0L) / points);
    }
    return c;
  }
};

// ------------------------------------------------------------ BootParameter
struct BootParameter {
  BootParameter(int max_level, int num_cts_levels, int num_stc_levels, int log_message_ratio = 5)
      : max_level_{max_level},
        num_cts_levels_{num_cts_levels},
        num_stc_levels_{num_stc_levels},
        log_message_ratio_{log_message_ratio} {}
  const int max_level_, num_cts_levels_, num_stc_levels_, log_message_ratio_;
  const int num_double_angle_ = 3;
  const int K_ = 16;           // u = m/q0 + I is divided by K before EvalMod
  const int max_integer_part_ = 12;  // |I| the sine approximation is fitted for (7 sigma at h = 32)
  const int poly_degree_ = 30;  // even series in t, degree 15 in T_2(t)
  // levels: 1 (T_2(t)) + 4 (series of 16 terms in T_2(t)) + double angles
  int GetNumEvalModLevels() const { return 5 + num_double_angle_; }
  int GetMaxLevel() const { return max_level_; }
  int GetStartLevel() const { return max_level_; }
  int GetCtSStartLevel() const { return max_level_; }
  int GetEvalModStartLevel() const { return max_level_ - num_cts_levels_; }
  int GetStCStartLevel() const { return GetEvalModStartLevel() - GetNumEvalModLevels(); }
  int GetEndLevel() const { return GetStCStartLevel() - num_stc_levels_; }
};

// ------------------------------------------------------------ EvalMod
// res ~ (1/2pi) sin(2pi u) for an input holding u/K (real slot values).
template <typename word>
class EvalMod {
  using Ct = Ciphertext<word>;

 public:
  explicit EvalMod(const BootParameter &bp) : bp_(bp) { in_s_ = FitNearIntegers(bp); }

  // Coefficients c_k of sum_k c_k T_k(s), s = T_2(t), for
  //   f(t) = (1/2pi)^(1/2^r) cos(2 pi K t / 2^r),  t = (u - 1/4) / K,
  // fitted by least squares only where it is evaluated: u within
  // 2^-log_message_ratio of an integer of magnitude <= max_integer_part_.
  // Restricting the fit to those intervals buys several digits over the
  // Chebyshev series on all of [-1, 1] at the same degree. Householder QR in
  // long double; the sample points are Chebyshev nodes of each interval.
  static std::vector<double> FitNearIntegers(const BootParameter &bp) {
    using ld = long double;
    const int deg = bp.poly_degree_ / 2, per = 33, I_max = bp.max_integer_part_;
    const ld K = bp.K_, radius = std::ldexp(1.0L, -bp.log_message_ratio_);
    const ld amp = std::pow((ld)0.5 / M_PIl, (ld)1 / (1 << bp.num_double_angle_));
    const ld ang = 2 * M_PIl * K / (1 << bp.num_double_angle_);
    const int rows = (2 * I_max + 1) * per, cols = deg + 1;
    std::vector<ld> A((size_t)rows * cols), b(rows);
    int row = 0;
    for (int I = -I_max; I <= I_max; I++)
      for (int k = 0; k < per; k++, row++) {
        const ld u = I + radius * std::cos(M_PIl * (k + 0.5L) / per);
        const ld t = (u - 0.25L) / K, x = 2 * t * t - 1;
        b[row] = amp * std::cos(ang * t);
        ld t0 = 1, t1 = x;
        A[(size_t)row * cols] = 1;
        if (cols > 1) A[(size_t)row * cols + 1] = x;
        for (int j = 2; j < cols; j++) {
          const ld t2 = 2 * x * t1 - t0;
          A[(size_t)row * cols + j] = t2;
          t0 = t1;
          t1 = t2;
        }
      }
    for (int j = 0; j < cols; j++) {  // Householder reflections, applied to A and b
      ld norm = 0;
      for (int i = j; i < rows; i++) norm += A[(size_t)i * cols + j] * A[(size_t)i * cols + j];
      norm = std::sqrt(norm);
      if (A[(size_t)j * cols + j] > 0) norm = -norm;
      std::vector<ld> v(rows - j);
      for (int i = j; i < rows; i++) v[i - j] = A[(size_t)i * cols + j];
      v[0] -= norm;
      ld vv = 0;
      for (ld x : v) vv += x * x;
      if (vv == 0) continue;
      for (int c = j; c < cols; c++) {
        ld dot = 0;
        for (int i = j; i < rows; i++) dot += v[i - j] * A[(size_t)i * cols + c];
        dot *= 2 / vv;
        for (int i = j; i < rows; i++) A[(size_t)i * cols + c] -= dot * v[i - j];
      }
      ld dot = 0;
      for (int i = j; i < rows; i++) dot += v[i - j] * b[i];
      dot *= 2 / vv;
      for (int i = j; i < rows; i++) b[i] -= dot * v[i - j];
    }
    std::vector<ld> c(cols);
    for (int j = cols - 1; j >= 0; j--) {
      ld acc = b[j];
      for (int k = j + 1; k < cols; k++) acc -= A[(size_t)j * cols + k] * c[k];
      c[j] = acc / A[(size_t)j * cols + j];
    }
    return std::vector<double>(c.begin(), c.end());
  }

  void Evaluate(const ConstContextPtr<word> &ctx, Ct &res, const Ct &input,
                const EvaluationKey<word> &mult_key) const {
    const auto &param = ctx->param_;
    const int level = param.NPToLevel(input.GetNP());
    // t = u/K - 1/(4K)
    Constant<word> shift;
    ctx->encoder().EncodeConstant(shift, level, input.GetScale(), 0.25 / bp_.K_, 0);
    Ct t, s, y;
    ctx->Sub(t, input, shift);
    EvalPoly<word>::Node(ctx, s, t, t, nullptr, 1.0, mult_key);  // s = 2 t^2 - 1
    EvalPoly<word>::EvaluateChebyshev(ctx, y, s, in_s_, mult_key, s.GetScale());
    // y_i = (1/2pi)^(2^i / 2^r) cos(2^i theta): y <- 2 y^2 - (1/2pi)^(2^(i+1) / 2^r)
    double c = std::pow(0.5 / M_PI, 1.0 / (1 << bp_.num_double_angle_));
    for (int i = 0; i < bp_.num_double_angle_; i++) {
      c *= c;
      Ct next;
      EvalPoly<word>::Node(ctx, next, y, y, nullptr, c, mult_key);
      y = std::move(next);
    }
    res = std::move(y);
  }

 private:
  BootParameter bp_;
  std::vector<double> in_s_;
};

// ------------------------------------------------------------ EvalSpecialFFT
// Stage matrices of the encoder's special FFT / IFFT without the bit-reversal
// permutation, merged in groups.
template <typename word>
class EvalSpecialFFT {
 public:
  // one radix-2 stage of SpecialIFFT (reference src/core/Encode.cpp:85-109)
  static StripedMatrix IfftStage(const Parameter<word> &param, int n, int stride) {
    StripedMatrix m(n);
    const int M = 2 * param.degree_, st8 = stride << 3, gap = M / st8;
    auto &d0 = m.At(0), &dp = m.At(stride), &dm = m.At(-stride);
    for (int i = 0; i < n; i += 2 * stride)
      for (int j = 0; j < stride; j++) {
        const int idx = ((st8 - (param.GetGaloisFactor(j) % st8)) * gap) % M;
        const Complex tw = std::polar(1.0, 2.0 * M_PI * idx / M);
        d0[i + j] += 1.0;
        dp[i + j] += 1.0;
        d0[i + j + stride] += -tw;
        dm[i + j + stride] += tw;
      }
    return m;
  }
  // one radix-2 stage of SpecialFFT (reference src/core/Encode.cpp:111-133)
  static StripedMatrix FftStage(const Parameter<word> &param, int n, int stride) {
    StripedMatrix m(n);
    const int M = 2 * param.degree_, st8 = stride << 3, gap = M / st8;
    auto &d0 = m.At(0), &dp = m.At(stride), &dm = m.At(-stride);
    for (int i = 0; i < n; i += 2 * stride)
      for (int j = 0; j < stride; j++) {
        const int idx = ((param.GetGaloisFactor(j) % st8) * gap) % M;
        const Complex tw = std::polar(1.0, 2.0 * M_PI * idx / M);
        d0[i + j] += 1.0;
        dp[i + j] += tw;
        d0[i + j + stride] += -tw;
        dm[i + j + stride] += 1.0;
      }
    return m;
  }
  // Groups of merged stages, in application order. CtS: IFFT stages from the
  // largest stride down; StC: FFT stages from stride 1 up. `total_const` is
  // spread evenly over the groups.
  static std::vector<StripedMatrix> Groups(const Parameter<word> &param, int n, bool cts, int groups,
                                           double total_const) {
    std::vector<int> strides;
    if (cts)
      for (int s = n / 2; s >= 1; s /= 2) strides.push_back(s);
    else
      for (int s = 1; s < n; s *= 2) strides.push_back(s);
    const double each = std::pow(total_const, 1.0 / groups);
    std::vector<StripedMatrix> out;
    const int per = strides.empty() ? 1 : ((int)strides.size() + groups - 1) / groups;
    for (size_t at = 0; at < strides.size(); at += per) {
      StripedMatrix g = cts ? IfftStage(param, n, strides[at]) : FftStage(param, n, strides[at]);
      for (size_t k = at + 1; k < std::min(strides.size(), at + per); k++) {
        StripedMatrix next = cts ? IfftStage(param, n, strides[k]) : FftStage(param, n, strides[k]);
        g = StripedMatrix::Mult(next, g);
      }
      g.Scale(each);
      out.push_back(std::move(g));
    }
    // fewer stages than levels (few slots): the remaining levels carry the constant only
    while ((int)out.size() < groups) {
      StripedMatrix id(n);
      auto &d = id.At(0);
      for (auto &x : d) x = each;
      out.push_back(std::move(id));
    }
    return out;
  }
};

// How Boot finishes (reference include/extension/BootContext.h:16-20).
enum class BootVariant {
  kNormal,             // complex bootstrapping
  kImaginaryRemoving,  // SlotToCoeff carries a factor 1/2 and Boot ends with res + conj(res)
  kMergeTwoReal        // SlotToCoeff carries the factor 1/2; the caller combines two results
};

// ------------------------------------------------------------ BootContext
// A Context that can also refresh a ciphertext (reference
// include/extension/BootContext.h, src/extension/BootContext.cpp).
template <typename word>
class BootContext : public Context<word> {
  using Base = Context<word>;
  using Ct = Ciphertext<word>;
  using Evk = EvaluationKey<word>;
  using Dv = DeviceVector<word>;

 public:
  static std::shared_ptr<BootContext<word>> Create(const Parameter<word> &param,
                                                   const BootParameter &boot_param) {
    return std::shared_ptr<BootContext<word>>(new BootContext<word>(param, boot_param));
  }
  ConstContextPtr<word> GetContext() const { return this->shared_from_this(); }

  const BootParameter boot_param_;

  void PrepareEvalMod() {
    if (eval_mod_) {
      Warn("EvalMod already prepared");
      return;
    }
    eval_mod_ = std::make_unique<EvalMod<word>>(boot_param_);
    // A second engine context (own stream, workspace and allocation cache) for
    // the imaginary part: below the top levels one EvalMod leaves most of the
    // GPU idle, two side by side do not. UseSideStream(false) keeps one stream.
    cfhe_context *current = detail::CurrentHandle();
    side_ = Context<word>::Create(this->param_);
    detail::CurrentHandle() = current;
  }
  // false: both EvalMods run on this context's stream (what per-stage device
  // profiling needs, since it sees one context)
  void UseSideStream(bool on) { use_side_ = on; }
  // true: Boot's phase report also says how long the host took to enqueue each phase
  void ReportPhaseEnqueue(bool on) { report_enqueue_ = on; }

  // Linear transforms for ciphertexts with num_slots slots (a power of two up to
  // degree / 2). Fewer slots mean a plaintext in the subring of X^(degree/2/num_slots):
  // the transforms have num_slots-periodic diagonals, and Boot projects the
  // raised ciphertext onto the subring first (Trace).
  void PrepareEvalSpecialFFT(int num_slots, BootVariant variant = BootVariant::kNormal) {
    const auto &param = this->param_;
    const int half = param.degree_ / 2;
    AssertTrue(num_slots >= 2 && num_slots <= half && (num_slots & (num_slots - 1)) == 0,
               "Only power-of-two slots are supported");
    if (eval_fft_.count(num_slots)) {
      Warn("EvalSpecialFFT already prepared");
      return;
    }
    FftPlan &plan = eval_fft_[num_slots];
    plan.variant = variant;
    const int n = num_slots;
    // CoeffToSlot: the raised (and traced) ciphertext holds (half / n) * q0 * u(Y),
    // Y = X^(half/n); read at scale q0 its n distinct slots are
    // (half/n) * SpecialFFT_n(u_j + i u_{j+n}). The groups apply the inverse
    // transform, its 1/n, the 1/(half/n) of the trace and 1/(2K), so that the
    // real and imaginary parts taken afterwards (each a sum of two terms) are
    // u / K: the constant is 1 / (half * 2K) whatever n is.
    auto cts = EvalSpecialFFT<word>::Groups(param, n, true, boot_param_.num_cts_levels_,
                                            1.0 / ((double)half * 2.0 * boot_param_.K_));
    // With fewer than degree / 2 slots there is room for the real and the
    // imaginary parts side by side: the last CoeffToSlot group M is replaced by
    //   U = A x + B conj(x),  A = diag(D1) M,  B = diag(D2) conj(M)
    // on 2n slots, D1 = (1 | -i), D2 = (1 | i) on the two halves, so that
    // U = (2 Re(M x) | 2 Im(M x)) and a single EvalMod serves both parts; the
    // first SlotToCoeff group S absorbs the way back, S (V + i rot_n(V)).
    plan.merged = n < half;
    const Complex I(0, 1);
    double s_in = q0_prod_;
    int level = boot_param_.GetCtSStartLevel();
    for (size_t gi = 0; gi < cts.size(); gi++) {
      const StripedMatrix &g = cts[gi];
      if (plan.merged && gi + 1 == cts.size()) {
        StripedMatrix A(2 * n), B(2 * n);
        for (auto &[k, d] : g.diag) {
          const int ks = k > n / 2 ? k - n : k;  // the same rotation of an n-periodic vector, nearer zero
          auto &da = A.At(ks), &db = B.At(ks);
          for (int p = 0; p < 2 * n; p++) {
            const Complex m = d[p % n];
            da[p] = (p < n ? Complex(1, 0) : -I) * m;
            db[p] = (p < n ? Complex(1, 0) : I) * std::conj(m);
          }
        }
        plan.cts_last.emplace_back(GetContext(), A, level, s_in, eval_mod_scale_, kBabySteps);
        plan.cts_last.emplace_back(GetContext(), B, level, s_in, eval_mod_scale_, kBabySteps);
      } else {
        plan.cts.emplace_back(GetContext(), g, level, s_in, eval_mod_scale_, kBabySteps);
      }
      s_in = eval_mod_scale_;
      level--;
    }
    // SlotToCoeff: the slots hold (p_j + i p_{j+n}) / q0 for the refreshed
    // plaintext p = scale0' * m; the forward transform and q0 / scale0' give m.
    // The scale drops from EvalMod's to the end level's in equal steps, which
    // keeps every diagonal plaintext well above the rounding of its encoding.
    auto stc = EvalSpecialFFT<word>::Groups(
        param, n, false, boot_param_.num_stc_levels_,
        (q0_prod_ / boot_input_scale_) * (variant == BootVariant::kNormal ? 1.0 : 0.5));
    if (plan.merged) {
      StripedMatrix tiled(2 * n), back(2 * n);
      for (auto &[k, d] : stc[0].diag) {
        auto &t = tiled.At(k > n / 2 ? k - n : k);
        for (int p = 0; p < 2 * n; p++) t[p] = d[p % n];
      }
      auto &c0 = back.At(0), &c1 = back.At(n);
      for (int p = 0; p < 2 * n; p++) {
        c0[p] = p < n ? Complex(1, 0) : I;
        c1[p] = p < n ? I : Complex(1, 0);
      }
      stc[0] = StripedMatrix::Mult(tiled, back);
    }
    level = boot_param_.GetStCStartLevel();
    s_in = eval_mod_end_scale_;
    const double s_end = param.GetScale(boot_param_.GetEndLevel());
    const int ng = stc.size();
    for (int i = 0; i < ng; i++) {
      const double s_out = i + 1 == ng ? s_end : s_in * std::pow(s_end / s_in, 1.0 / (ng - i));
      plan.stc.emplace_back(GetContext(), stc[i], level, s_in, s_out, kBabySteps);
      s_in = s_out;
      level--;
    }
  }

  bool IsBootPrepared(int num_slots) const { return eval_mod_ && eval_fft_.count(num_slots); }

  // Rotation keys Boot needs for this slot count: those of the linear
  // transforms and the trace's num_slots * 2^i (reference AddRequiredRotations,
  // src/extension/BootContext.cpp:174-184).
  void AddRequiredRotations(EvkRequest &req, int num_slots, bool min_ks = false) const {
    AssertTrue(IsBootPrepared(num_slots), "Bootstrapping is not prepared for this slot count");
    const FftPlan &plan = eval_fft_.at(num_slots);
    std::set<int> rots;
    for (auto &lt : plan.cts) lt.AddRequiredRotations(rots, min_ks);
    for (auto &lt : plan.cts_last) lt.AddRequiredRotations(rots, min_ks);
    for (auto &lt : plan.stc) lt.AddRequiredRotations(rots, min_ks);
    for (int ns = num_slots; ns < this->param_.degree_ / 2; ns *= 2) rots.insert(ns);
    for (int r : rots) req.AddRequest(r, boot_param_.GetMaxLevel());
  }

  // res = sum_{j < num_accum} rot_{j * start_rot_dist}(input), num_accum a
  // power of two (reference Trace, src/extension/BootContext.cpp:367-402).
  void Trace(Ct &res, int start_rot_dist, int num_accum, const Ct &input, const EvkMap<word> &evk_map) const {
    AssertTrue(num_accum >= 1 && (num_accum & (num_accum - 1)) == 0, "Num accum must be power of 2");
    AssertTrue(input.GetNP().num_aux_ == 0, "Trace: Aux primes are not allowed");
    if (num_accum == 1) {
      this->Copy(res, input);
      return;
    }
    const int num_slots = input.GetNumSlots();
    Ct acc, next;
    const Ct *cur = &input;
    for (int step = 1; step < num_accum; step *= 2) {
      int rot = (int)(((long long)start_rot_dist * step) % num_slots);
      if (rot < 0) rot += num_slots;
      this->HRotAdd(next, *cur, *cur, evk_map.GetRotationKey(rot), rot);
      acc = std::move(next);
      cur = &acc;
    }
    res = std::move(acc);
  }

  // Raises a ciphertext on the lowest level's primes to the highest level:
  // exact centred lift of both parts (reference ModUpToMax,
  // src/extension/BootContext.cpp:188-277). With sparse-secret encapsulation
  // the lift is wrapped in a switch to the sparse secret and back; the lifted
  // a part is produced on the auxiliary primes as well, so that the switch
  // back is one product with a single-digit key and one ModDown.
  void ModUpToMax(Ct &res, const Ct &input, const EvkMap<word> &evk_map) const {
    const auto &param = this->param_;
    const int n = param.degree_, L = param.L_, alpha = param.alpha_;
    NPInfo low = param.LevelToNP(-1), top = param.LevelToNP(param.max_level_);
    AssertTrue(input.GetNP() == low, "ModUpToMax: input NP mismatch");
    AssertFalse(input.HasRx(), "ModUpToMax: input has Rx");
    AssertTrue(top.GetNumQ() == L, "ModUpToMax: the top level must hold every prime");
    const bool sse = param.IsUsingSparseSecretEncapsulation();
    Ct switched;
    const Ct *work = &input;
    if (sse) {
      this->MultKey(switched, input, evk_map.GetDenseToSparseKey());
      work = &switched;
    }
    auto g_low = param.GetLimbIndices(low);
    auto g_top = param.GetLimbIndices(top);
    auto g_all = param.GetLimbIndices(param.LevelToNP(param.max_level_, alpha));
    const int nl = g_low.size();
    AssertTrue(nl <= 2, "ModUpToMax: at most two base primes");
    // (N * product of the other base primes)^-1 on each base prime
    std::vector<word> icrt(nl);
    auto primes = param.GetPrimeVector(low);
    for (int i = 0; i < nl; i++) {
      word prod = (word)(n % primes[i]);
      for (int j = 0; j < nl; j++)
        if (j != i) prod = detail::MulMod(prod, primes[j] % primes[i], primes[i]);
      icrt[i] = detail::InvMod(prod, primes[i]);
    }
    auto raise = [&](Dv &dst, const Dv &src, const std::vector<int> &g_dst) {
      Dv coef((size_t)nl * n);
      CheckAbi(cfhe_intt(this->h_, coef.data(), src.data(), g_low.data(), nl, 1, 0, 0, icrt.data(), 0, 0));
      dst.resize(g_dst.size() * n);
      CheckAbi(cfhe_modup_to_max(this->h_, dst.data(), coef.data(), g_low.data(), nl, g_dst.data(),
                                 g_dst.size()));
      CheckAbi(cfhe_ntt(this->h_, dst.data(), dst.data(), g_dst.data(), g_dst.size(), 1, 0, 0, 1));
    };
    Ct out(top);
    if (!sse) {
      raise(out.bx_, work->bx_, g_top);
      raise(out.ax_, work->ax_, g_top);
    } else {
      const Evk &key = evk_map.GetSparseToDenseKey();
      AssertTrue(key.GetNP() == param.LevelToNP(param.max_level_, alpha), "Invalid sparse-to-dense key");
      Dv b_up, a_up;
      raise(b_up, work->bx_, g_top);
      raise(a_up, work->ax_, g_all);
      const size_t ext = (size_t)(L + alpha) * n;
      Dv acc(2 * ext);
      // acc_b = a * key_b + P * b on the Q limbs; acc_a = a * key_a
      CheckAbi(cfhe_binary(this->h_, 3, acc.data(), a_up.data(), key.bx_[0].data(), g_all.data(), g_all.size()));
      CheckAbi(cfhe_binary(this->h_, 3, acc.data() + ext, a_up.data(), key.ax_[0].data(), g_all.data(),
                           g_all.size()));
      std::vector<word> p_prod(L);
      for (int i = 0; i < L; i++) {
        const word q = cfhe_prime(this->h_, g_top[i]);
        word pp = 1;
        for (int j = 0; j < alpha; j++) pp = detail::MulMod(pp, param.aux_primes_[j] % q, q);
        p_prod[i] = detail::ToMontgomery(pp, q);
      }
      CheckAbi(cfhe_const_op(this->h_, 4, acc.data(), b_up.data(), acc.data(), p_prod.data(), g_top.data(), L));
      Dv both((size_t)2 * L * n);
      CheckAbi(cfhe_moddown(this->h_, param.max_level_, 0, both.data(), acc.data(), 2, (long long)L * n,
                            (long long)ext));
      std::vector<word> zero(L, 0);
      this->ConstKernel(0, out.bx_.data(), both.data(), nullptr, zero, top);
      this->ConstKernel(0, out.ax_.data(), both.data() + (size_t)L * n, nullptr, zero, top);
    }
    out.SetScale(input.GetScale());
    out.SetNumSlots(input.GetNumSlots());
    res = std::move(out);
  }

  // With fewer than degree / 2 slots the result has twice the input's slots:
  // real parts of the coefficients' slots in the first half, imaginary parts
  // in the second (see PrepareEvalSpecialFFT); SlotToCoeff takes that form back.
  void CoeffToSlot(Ct &res, const Ct &input, const EvkMap<word> &evk_map, bool min_ks = false) const {
    const FftPlan &plan = PlanFor(input.GetNumSlots());
    if (!plan.merged) {
      RunGroups(res, input, plan.cts, evk_map, min_ks);
      return;
    }
    Ct x, xc, ua, ub;
    const Ct *in = &input;
    if (!plan.cts.empty()) {
      RunGroups(x, input, plan.cts, evk_map, min_ks);
      in = &x;
    }
    this->HConj(xc, *in, evk_map.GetConjugationKey());
    plan.cts_last[0].Evaluate(GetContext(), ua, *in, evk_map, min_ks);
    plan.cts_last[1].Evaluate(GetContext(), ub, xc, evk_map, min_ks);
    this->Add(res, ua, ub);
    res.SetNumSlots(2 * input.GetNumSlots());
  }
  void SlotToCoeff(Ct &res, const Ct &input, const EvkMap<word> &evk_map, bool min_ks = false) const {
    const int half = this->param_.degree_ / 2;
    // a merged input carries twice the plan's slot count
    auto it = eval_fft_.find(input.GetNumSlots());
    const bool direct = it != eval_fft_.end() && !it->second.merged;
    const int num_slots = direct ? input.GetNumSlots() : input.GetNumSlots() / 2;
    AssertTrue(num_slots <= half, "SlotToCoeff: too many slots");
    RunGroups(res, input, PlanFor(num_slots).stc, evk_map, min_ks);
    res.SetNumSlots(num_slots);
  }
  void EvaluateMod(Ct &res, const Ct &input, const Evk &mult_key) const {
    AssertTrue(eval_mod_ != nullptr, "EvalMod not prepared");
    this->AssertSameScale(input.GetScale(), eval_mod_scale_);
    eval_mod_->Evaluate(GetContext(), res, input, mult_key);
    this->AssertSameScale(res.GetScale(), eval_mod_end_scale_);
  }

  // Refreshes a level-0 ciphertext with slot values in [-1, 1]^2 to
  // boot_param_.GetEndLevel() (reference Boot, src/extension/BootContext.cpp:299-365).
  // phase_ms (optional): the host synchronises after every phase and appends
  // its name and wall-clock milliseconds.
  // min_ks: linear transforms with at most three rotation keys each.
  void Boot(Ct &res, const Ct &input, const EvkMap<word> &evk_map, bool min_ks = false,
            std::vector<std::pair<std::string, double>> *phase_ms = nullptr) const {
    const auto &param = this->param_;
    auto last = std::chrono::steady_clock::now();
    auto phase = [&](const char *name) {
      if (!phase_ms) return;
      if (report_enqueue_)
        phase_ms->emplace_back(std::string(name) + " (enqueue)",
                               std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - last).count());
      this->Synchronize();
      auto now = std::chrono::steady_clock::now();
      phase_ms->emplace_back(name, std::chrono::duration<double, std::milli>(now - last).count());
      last = now;
    };
    AssertTrue(IsBootPrepared(input.GetNumSlots()), "Boot: not prepared for this slot count");
    AssertFalse(input.HasRx(), "Boot: relinearize first");
    if (param.NPToLevel(input.GetNP()) > 0) {
      Ct low;
      this->LevelDown(low, input, 0);
      Boot(res, low, evk_map, min_ks, phase_ms);
      return;
    }
    this->AssertSameScale(input.GetScale() * (double)(UINT64_C(1) << log_scaleup_), boot_input_scale_);
    // 0. integer scale-up: the plaintext fills q0 / 2^log_message_ratio
    Ct main;
    {
      NPInfo low = input.GetNP();
      main.ModifyNP(low);
      auto primes = param.GetPrimeVector(low);
      std::vector<word> k(primes.size());
      for (size_t i = 0; i < primes.size(); i++)
        k[i] = detail::ToMontgomery((word)((UINT64_C(1) << log_scaleup_) % primes[i]), primes[i]);
      this->ConstKernel(3, main.bx_.data(), input.bx_.data(), nullptr, k, low);
      this->ConstKernel(3, main.ax_.data(), input.ax_.data(), nullptr, k, low);
      main.SetNumSlots(input.GetNumSlots());
      main.SetScale(boot_input_scale_);
    }
    // 1. to the top level
    Ct raised;
    ModUpToMax(raised, main, evk_map);
    raised.SetScale(q0_prod_);
    const int half = param.degree_ / 2, num_slots = input.GetNumSlots();
    if (num_slots < half) {
      // fewer slots: keep only the subring part of the raised polynomial
      Ct traced;
      raised.SetNumSlots(half);
      Trace(traced, num_slots, half / num_slots, raised, evk_map);
      raised = std::move(traced);
      raised.SetNumSlots(num_slots);
    }
    phase("ModUpToMax");
    // 2. coefficients to slots
    Ct slots;
    CoeffToSlot(slots, raised, evk_map, min_ks);
    phase("CoeffToSlot");
    // 3. real and imaginary parts through EvalMod: side by side in one
    // ciphertext when there is room, else one after the other
    Ct re_mod;
    if (PlanFor(num_slots).merged) {
      EvaluateMod(re_mod, slots, evk_map.GetMultiplicationKey());
      phase("EvalMod");
    } else {
      Ct conj, re, im, im_mod;
      this->HConj(conj, slots, evk_map.GetConjugationKey());
      this->Add(re, slots, conj);
      this->Sub(im, conj, slots);
      this->MultImaginaryUnit(im, im);
      phase("conjugate split");
      if (side_ && use_side_) {
        // im was produced on this stream and is read on the side stream; im_mod
        // is produced there and read here: one ordering call each way. im_mod
        // and every temporary of the side evaluation come from the side
        // context's allocation cache, whose reuse is ordered on the side stream.
        CheckAbi(cfhe_order_after(side_->h_, this->h_));
        {
          ScopedCurrentHandle on_side(side_->h_);
          eval_mod_->Evaluate(side_, im_mod, im, evk_map.GetMultiplicationKey());
          side_->MultImaginaryUnit(im_mod, im_mod);
        }
        EvaluateMod(re_mod, re, evk_map.GetMultiplicationKey());
        CheckAbi(cfhe_order_after(this->h_, side_->h_));
      } else {
        EvaluateMod(re_mod, re, evk_map.GetMultiplicationKey());
        EvaluateMod(im_mod, im, evk_map.GetMultiplicationKey());
        this->MultImaginaryUnit(im_mod, im_mod);
      }
      this->Add(re_mod, re_mod, im_mod);
      phase("EvalMod x2");
    }
    // 4. slots to coefficients
    SlotToCoeff(res, re_mod, evk_map, min_ks);
    if (PlanFor(num_slots).variant == BootVariant::kImaginaryRemoving)
      this->HConjAdd(res, res, res, evk_map.GetConjugationKey());  // res + conj(res): the real part, twice the half
    res.SetNumSlots(input.GetNumSlots());
    phase("SlotToCoeff");
  }

  int GetLogScaleUp() const { return log_scaleup_; }

 private:
  static constexpr int kBabySteps = 16;

  BootContext(const Parameter<word> &param, const BootParameter &bp) : Base(param), boot_param_{bp} {
    AssertTrue(param.max_level_ == bp.max_level_ && param.default_encryption_level_ == bp.GetStCStartLevel(),
               "Parameter mismatch for BootContext");
    auto round_log2 = [](double x) { return (int)std::floor(std::log2(x) + 0.5); };
    q0_prod_ = 1.0;
    for (word q : param.GetPrimeVector(param.LevelToNP(-1))) q0_prod_ *= (double)q;
    // level-0 scale times 2^log_scaleup ~ q0 / 2^log_message_ratio
    // (reference src/extension/BootContext.cpp:47-66)
    log_scaleup_ = round_log2(q0_prod_) - round_log2(param.base_scale_) - bp.log_message_ratio_;
    AssertTrue(log_scaleup_ >= 0, "Invalid level zero scaleup");
    boot_input_scale_ = param.base_scale_ * (double)(UINT64_C(1) << log_scaleup_);
    const int em = bp.GetEvalModStartLevel();
    eval_mod_scale_ = std::ldexp(1.0, round_log2(param.GetRescalePrimeProd(em)));
    // EvalMod: T_2(t) squares the scale once, the series keeps it, every
    // double-angle step squares it again
    eval_mod_end_scale_ = eval_mod_scale_ * eval_mod_scale_ / param.GetRescalePrimeProd(em);
    for (int i = 0; i < bp.num_double_angle_; i++)
      eval_mod_end_scale_ = eval_mod_end_scale_ * eval_mod_end_scale_ /
                            param.GetRescalePrimeProd(em - bp.GetNumEvalModLevels() + bp.num_double_angle_ - i);
  }

  void RunGroups(Ct &res, const Ct &input, const std::vector<LinearTransform<word>> &groups,
                 const EvkMap<word> &evk_map, bool min_ks) const {
    AssertFalse(groups.empty(), "EvalSpecialFFT not prepared");
    Ct cur, next;
    const Ct *in = &input;
    for (auto &lt : groups) {
      lt.Evaluate(GetContext(), next, *in, evk_map, min_ks);
      cur = std::move(next);
      in = &cur;
    }
    res = std::move(cur);
  }

  double q0_prod_ = 1.0, boot_input_scale_ = 1.0, eval_mod_scale_ = 1.0, eval_mod_end_scale_ = 1.0;
  int log_scaleup_ = 0;
  std::unique_ptr<EvalMod<word>> eval_mod_;
  ContextPtr<word> side_;
  bool use_side_ = true;
  bool report_enqueue_ = false;
  struct FftPlan {
    bool merged = false;  // fewer than degree / 2 slots: one EvalMod for both parts
    BootVariant variant = BootVariant::kNormal;
    std::vector<LinearTransform<word>> cts, cts_last, stc;
  };
  const FftPlan &PlanFor(int num_slots) const {
    auto it = eval_fft_.find(num_slots);
    AssertTrue(it != eval_fft_.end(), "BootContext not prepared for num slots: " + std::to_string(num_slots));
    return it->second;
  }
  std::map<int, FftPlan> eval_fft_;
};

}  // namespace cheddar
