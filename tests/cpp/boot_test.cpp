// Tests of the bootstrapping building blocks and of full bootstrapping on the
// C++ mirror of the reference API (the reference's boot_test checks Boot on
// 2^15 random complex slots in [-1,1]^2, unittest/Bootstrapping.cpp:10-41).
//
//   boot_test <parameter.json> [--only linear,poly,evalmod,fft,boot,minks,sparse]
#include <algorithm>
#include <chrono>
#include <cstring>
#include <iomanip>

#include "cheddar/Boot.h"

using namespace cheddar;
using word = uint32_t;
using Ct = Ciphertext<word>;
using Pt = Plaintext<word>;
using Msg = std::vector<Complex>;

static int failures = 0;

static void Report(const std::string &what, const Msg &expected, const Msg &got, double tol) {
  double worst = 0, sum = 0;
  for (size_t i = 0; i < expected.size(); i++) {
    const double d = std::abs(expected[i] - got[i]);
    worst = std::max(worst, d);
    sum += d;
  }
  const bool ok = worst <= tol;
  std::cout << (ok ? "[ OK ] " : "[FAIL] ") << what << "  max|diff| " << std::scientific
            << std::setprecision(3) << worst << "  precision " << std::fixed << std::setprecision(2)
            << -std::log2(sum / expected.size()) << " bits" << std::endl;
  if (!ok) failures++;
}

int main(int argc, char **argv) {
  if (argc < 2) {
    std::cerr << "usage: boot_test <parameter.json> [--only a,b]\n";
    return 2;
  }
  std::set<std::string> only;
  for (int i = 2; i < argc; i++)
    if (!strcmp(argv[i], "--only") && i + 1 < argc) {
      std::stringstream ss(argv[++i]);
      std::string t;
      while (std::getline(ss, t, ',')) only.insert(t);
    }
  auto want = [&](const char *n) { return only.empty() || only.count(n); };
  Random::Seed(0xC0FFEE04);
  ParameterJson json = LoadParameterJson(argv[1]);
  auto param = MakeParameter<word>(json);
  AssertTrue(json.boot, "the parameter file does not enable bootstrapping");
  BootParameter boot_param(param->max_level_, json.num_cts_levels, json.num_stc_levels);
  auto boot_ctx = BootContext<word>::Create(*param, boot_param);
  ContextPtr<word> ctx = boot_ctx;
  UserInterface<word> ui(ctx);
  const int n = param->degree_ / 2;
  auto scale_of = [&](int level) {
    return level <= param->default_encryption_level_ ? param->GetScale(level)
                                                     : param->GetRescalePrimeProd(level);
  };
  auto encrypt = [&](Ct &ct, const Msg &m, int level, double scale) {
    Pt pt;
    ctx->encoder().Encode(pt, level, scale, m, 0);
    ui.Encrypt(ct, pt);
  };
  auto decrypt = [&](Msg &m, const Ct &ct) {
    Pt pt;
    ui.Decrypt(pt, ct);
    ctx->encoder().Decode(m, pt);
  };
  auto random_msg = [&](Msg &m, double lo, double hi, bool complex) {
    m.assign(n, Complex(0, 0));
    Random::SampleUniformComplex(m.data(), n, lo, hi);
    if (!complex)
      for (auto &x : m) x = Complex(x.real(), 0);
  };

  if (want("linear")) {
    // striped matrix with offsets that are multiples of 16, t in [-10, 20]
    const int level = 20;
    StripedMatrix M(n);
    for (int t : {-10, -3, -1, 0, 1, 2, 7, 8, 9, 15, 16, 20}) {
      auto &d = M.At(16 * t);
      Random::SampleUniformComplex(d.data(), n, -1.0, 1.0);
    }
    Msg z, got;
    random_msg(z, -1, 1, true);
    Ct ct, out;
    const double s = scale_of(level);
    encrypt(ct, z, level, s);
    LinearTransform<word> lt(ctx, M, level, s, s, 8);
    std::set<int> rots;
    lt.AddRequiredRotations(rots);
    for (int r : rots) ui.PrepareRotationKey(r, param->max_level_);
    lt.Evaluate(ctx, out, ct, ui.GetEvkMap());
    decrypt(got, out);
    Report("LinearTransform (12 diagonals, baby steps of 8, level 20)", M.Apply(z), got, 1e-4);
    std::cout << "       rotations used: " << rots.size() << std::endl;
  }

  if (want("poly")) {
    const int level = 24;
    std::vector<double> c(16);
    for (auto &x : c) {
      Complex t;
      Random::SampleUniformComplex(&t, 1, -1.0, 1.0);
      x = t.real();
    }
    Msg x, got, expect;
    random_msg(x, -1, 1, false);
    for (auto &v : x) {
      // Clenshaw in double
      double b1 = 0, b2 = 0, t = v.real();
      for (int k = 15; k >= 1; k--) {
        double b0 = c[k] + 2 * t * b1 - b2;
        b2 = b1;
        b1 = b0;
      }
      expect.push_back(Complex(c[0] + t * b1 - b2, 0));
    }
    Ct ct, out;
    const double s = (double)(UINT64_C(1) << (int)std::lround(std::log2(scale_of(level))));
    encrypt(ct, x, level, s);
    EvalPoly<word>::EvaluateChebyshev(ctx, out, ct, c, ui.GetMultiplicationKey(), s);
    decrypt(got, out);
    std::cout << "       output level " << param->NPToLevel(out.GetNP()) << std::endl;
    Report("EvalPoly Chebyshev degree 15 (level 24)", expect, got, 1e-5);
  }

  if (want("adapters")) {
    // The reference's extension interfaces (include/extension/{EvalPoly,LinearTransform,Hoist}.h)
    // as callers of the reference write them.
    {
      // EvalPoly object: power-basis coefficients, Compile, Evaluate, PlainEvaluate
      const int level = 20;
      std::vector<double> c = {0.3, -0.7, 0.11, 0.5, -0.25, 0.06, 0.02, -0.13};
      const double s = (double)(UINT64_C(1) << (int)std::lround(std::log2(scale_of(level))));
      EvalPoly<word> poly(c, level, s, s, false);
      if (poly.GetPolyDegree() != 7) {
        std::cout << "[FAIL] EvalPoly::GetPolyDegree" << std::endl;
        failures++;
      }
      poly.Compile(ctx);
      Msg x, got, expect;
      random_msg(x, -1, 1, false);
      for (auto &v : x) expect.push_back(Complex(poly.PlainEvaluate(v.real()), 0));
      Ct ct, out;
      encrypt(ct, x, level, s);
      poly.Evaluate(ctx, out, ct, ui.GetMultiplicationKey());
      decrypt(got, out);
      Report("EvalPoly(coefficients, level, scale, target).Compile/Evaluate, power basis degree 7", expect, got, 1e-5);
      // basis conversion is an identity on the function
      EvalPoly<word> twin(c, level, s, s, false);
      twin.ConvertToChebyshevBasis();
      double worst = 0;
      for (double t : {-1.0, -0.3, 0.0, 0.77, 1.0}) worst = std::max(worst, std::abs(twin.PlainEvaluate(t) - poly.PlainEvaluate(t)));
      twin.ConvertToNormalBasis();
      for (double t : {-1.0, 0.4, 1.0}) worst = std::max(worst, std::abs(twin.PlainEvaluate(t) - poly.PlainEvaluate(t)));
      std::cout << (worst < 1e-12 ? "[ OK ] " : "[FAIL] ") << "EvalPoly basis conversions, max difference " << worst << std::endl;
      if (!(worst < 1e-12)) failures++;
    }
    {
      // LinearTransform(context, matrix, pt_level, pt_scale, bs, gs, pre_rotation, additional_pt_rot)
      const int level = 18, pre = 3, extra = 5;
      StripedMatrix M(n, n);
      for (int i : {3, 4, 5, 7, 11, 19, 35}) {  // offsets i - pre are 0, 1, 2, 4, 8, 16, 32
        auto &d = M[i];
        Random::SampleUniformComplex(d.data(), n, -1.0, 1.0);
      }
      Msg z, got, expect(n, Complex(0, 0));
      random_msg(z, -1, 1, true);
      for (const auto &[i, d] : M)
        for (int p = 0; p < n; p++) expect[p] += d[(p + extra) % n] * z[((p + i - pre) % n + n) % n];
      const double s = scale_of(level), pt_scale = param->GetRescalePrimeProd(level);
      Ct ct, out;
      encrypt(ct, z, level, s);
      LinearTransform<word> lt(ctx, M, level, pt_scale, 8, 8, pre, extra);
      EvkRequest req;
      lt.AddRequiredRotations(req);
      // one key shape for all rotations of a transform (some exist already at the top level)
      for (auto &[rot, lvl] : req)
        if (ui.GetEvkMap().find(rot) == ui.GetEvkMap().end()) ui.PrepareRotationKey(rot, param->max_level_);
      lt.Evaluate(ctx, out, ct, ui.GetEvkMap());
      ctx->AssertSameScale(out.GetScale(), s);
      decrypt(got, out);
      Report("LinearTransform reference constructor (bs 8, gs 8, pre_rotation 3, additional_pt_rot 5)", expect, got, 1e-4);
      if (!lt.IsUsingBSGS() || lt.GetBS() != 8 || lt.GetGS() != 8 || lt.GetPreRotationAmount() != pre) {
        std::cout << "[FAIL] LinearTransform accessors" << std::endl;
        failures++;
      }
    }
    {
      // HoistHandler(context, hoist_map, pt_level, pt_scale): plaintext [gs][bs] multiplies
      // rot_bs(input) and the sum over bs is rotated by gs
      const int level = 16;
      PlainHoistMap map;
      Msg z, got, expect(n, Complex(0, 0));
      random_msg(z, -1, 1, true);
      for (int gs : {0, 8, 16})
        for (int bs : {0, 1, 2, 5}) {
          Msg pt(n);
          Random::SampleUniformComplex(pt.data(), n, -1.0, 1.0);
          for (int p = 0; p < n; p++) expect[p] += pt[(p + gs) % n] * z[(p + gs + bs) % n];
          map[gs][bs] = std::move(pt);
        }
      const double s = scale_of(level), pt_scale = param->GetRescalePrimeProd(level);
      Ct ct, out;
      encrypt(ct, z, level, s);
      HoistHandler<word> hoist(ctx, map, level, pt_scale);
      EvkRequest req;
      hoist.AddRequiredRotations(req);
      for (auto &[rot, lvl] : req)
        if (ui.GetEvkMap().find(rot) == ui.GetEvkMap().end()) ui.PrepareRotationKey(rot, param->max_level_);
      hoist.Evaluate(ctx, out, ct, ui.GetEvkMap());
      decrypt(got, out);
      Report("HoistHandler (3 giant x 4 baby plaintexts)", expect, got, 1e-4);
    }
  }

  if (want("evalmod")) {
    const BootParameter &bp = boot_param;
    const int level = bp.GetEvalModStartLevel();
    EvalMod<word> em(bp);
    Msg u, got, expect;
    random_msg(u, -1, 1, false);
    // u = I + eps with |I| <= 12 and |eps| <= 2^-8
    for (auto &v : u) {
      const double I = std::floor(v.real() * 12.0 + 0.5);
      Complex e;
      Random::SampleUniformComplex(&e, 1, -1.0, 1.0);
      const double eps = e.real() / 256.0;
      expect.push_back(Complex(std::sin(2 * M_PI * eps) / (2 * M_PI), 0));
      v = Complex((I + eps) / bp.K_, 0);
    }
    Ct ct, out;
    const double s = (double)(UINT64_C(1) << (int)std::lround(std::log2(scale_of(level))));
    encrypt(ct, u, level, s);
    em.Evaluate(ctx, out, ct, ui.GetMultiplicationKey());
    decrypt(got, out);
    std::cout << "       levels " << level << " -> " << param->NPToLevel(out.GetNP()) << std::endl;
    Report("EvalMod (K = 16) against sin(2 pi u) / 2 pi", expect, got, 1e-9);
  }

  if (want("fft")) {
    // host-side consistency of the merged stage matrices: StC o CtS = n * identity
    auto cts = EvalSpecialFFT<word>::Groups(*param, n, true, boot_param.num_cts_levels_, 1.0);
    auto stc = EvalSpecialFFT<word>::Groups(*param, n, false, boot_param.num_stc_levels_, 1.0);
    Msg z;
    random_msg(z, -1, 1, true);
    Msg v = z;
    for (auto &g : cts) v = g.Apply(v);
    for (auto &g : stc) v = g.Apply(v);
    for (auto &x : v) x /= n;
    size_t diags = 0;
    for (auto &g : cts) diags += g.diag.size();
    for (auto &g : stc) diags += g.diag.size();
    std::cout << "       diagonals in the six groups: " << diags << std::endl;
    Report("special FFT groups: StC(CtS(z)) / n == z (host)", z, v, 1e-9);
  }

  if (want("boot")) {
    auto t0 = std::chrono::steady_clock::now();
    boot_ctx->PrepareEvalMod();
    boot_ctx->PrepareEvalSpecialFFT(n);
    EvkRequest req;
    boot_ctx->AddRequiredRotations(req, n);
    ui.PrepareRotationKey(req);
    auto t1 = std::chrono::steady_clock::now();
    std::cout << "       prepared " << req.size() << " rotation keys and the diagonals in "
              << std::chrono::duration<double>(t1 - t0).count() << " s" << std::endl;
    Msg m, got;
    random_msg(m, -1, 1, true);
    Ct ct, out;
    encrypt(ct, m, 0, param->GetScale(0));
    double best = 1e30;
    for (int it = 0; it < 4; it++) {
      ctx->Synchronize();
      auto a = std::chrono::steady_clock::now();
      boot_ctx->Boot(out, ct, ui.GetEvkMap());
      ctx->Synchronize();
      auto b = std::chrono::steady_clock::now();
      best = std::min(best, std::chrono::duration<double, std::milli>(b - a).count());
    }
    std::vector<std::pair<std::string, double>> phases;
    boot_ctx->Boot(out, ct, ui.GetEvkMap(), false, &phases);
    std::cout << "       phases (ms, host-synchronised):";
    for (auto &[name, ms] : phases) std::cout << "  " << name << " " << std::fixed << std::setprecision(2) << ms;
    std::cout << std::endl;
    if (only.count("profile")) {
      // device time per pipeline stage (CUDA events after every stage), summed by name
      boot_ctx->UseSideStream(false);
      CheckAbi(cfhe_profile_begin(ctx->h_));
      boot_ctx->Boot(out, ct, ui.GetEvkMap());
      std::vector<char> names(1 << 20);
      std::vector<float> ms(1 << 16);
      const int cnt = cfhe_profile_end(ctx->h_, names.data(), names.size(), ms.data(), ms.size());
      std::map<std::string, std::pair<double, int>> by_name;
      std::stringstream ss(names.data());
      std::string nm;
      double total = 0;
      for (int i = 0; i < cnt && std::getline(ss, nm, ';'); i++) {
        by_name[nm].first += ms[i];
        by_name[nm].second++;
        total += ms[i];
      }
      std::cout << "       device time by stage (" << cnt << " stages, " << total << " ms):" << std::endl;
      for (auto &[k, v] : by_name)
        std::cout << "         " << std::setw(16) << k << "  " << std::setw(5) << v.second << " x  " << std::fixed
                  << std::setprecision(3) << v.first << " ms" << std::endl;
    }
    decrypt(got, out);
    std::cout << "       Boot: level 0 -> " << param->NPToLevel(out.GetNP()) << ", best of 4: " << best << " ms"
              << std::endl;
    // the reference's acceptance bound (unittest/Testbed.h:93)
    Report("Boot, 2^15 complex slots in [-1,1]^2", m, got, 1e-3);
    // an input above level 0 is first brought down (reference BootContext.cpp:308-313)
    Ct high;
    encrypt(high, m, 3, param->GetScale(3));
    boot_ctx->Boot(out, high, ui.GetEvkMap());
    decrypt(got, out);
    Report("Boot of a level-3 input", m, got, 1e-3);
  }

  if (want("minks")) {
    // the plan with at most three rotation keys per linear transform
    // (the reference's Boot(..., min_ks = true), unittest/Bootstrapping.cpp:34-40)
    boot_ctx->PrepareEvalMod();
    boot_ctx->PrepareEvalSpecialFFT(n);
    EvkRequest req;
    boot_ctx->AddRequiredRotations(req, n, true);
    ui.PrepareRotationKey(req);
    Msg m, got;
    random_msg(m, -1, 1, true);
    Ct ct, out;
    encrypt(ct, m, 0, param->GetScale(0));
    double best = 1e30;
    for (int it = 0; it < 3; it++) {
      ctx->Synchronize();
      auto a = std::chrono::steady_clock::now();
      boot_ctx->Boot(out, ct, ui.GetEvkMap(), true);
      ctx->Synchronize();
      best = std::min(best, std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - a).count());
    }
    decrypt(got, out);
    std::cout << "       min_ks: " << req.size() << " rotation keys, best of 3: " << best << " ms" << std::endl;
    Report("Boot with minimum key switching", m, got, 1e-3);
  }

  if (want("sparse")) {
    // fewer slots than degree / 2: subring plaintexts, Trace after the lift
    boot_ctx->PrepareEvalMod();
    for (int ns : {1 << 10, 1 << 3}) {
      boot_ctx->PrepareEvalSpecialFFT(ns);
      EvkRequest req;
      boot_ctx->AddRequiredRotations(req, ns);
      ui.PrepareRotationKey(req);
      Msg m(ns), got;
      Random::SampleUniformComplex(m.data(), ns, -1.0, 1.0);
      Pt pt;
      Ct ct, out;
      ctx->encoder().Encode(pt, 0, param->GetScale(0), m, 0);
      ui.Encrypt(ct, pt);
      double ms = 1e30;
      for (int it = 0; it < 3; it++) {  // the first call also grows the workspace
        ctx->Synchronize();
        auto a = std::chrono::steady_clock::now();
        boot_ctx->Boot(out, ct, ui.GetEvkMap());
        ctx->Synchronize();
        ms = std::min(ms, std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - a).count());
      }
      Pt dec;
      ui.Decrypt(dec, out);
      ctx->encoder().Decode(got, dec);
      std::cout << "       " << ns << " slots: " << req.size() << " rotation keys requested, best of 3: " << ms
                << " ms, level " << param->NPToLevel(out.GetNP()) << std::endl;
      // With few slots the plaintext coefficients are large (about 1/sqrt(slots)),
      // and the cubic term of sin(2 pi x)/2 pi, 6.6 * (coefficient / 35)^3 * 35 per
      // coefficient at this message ratio, is no longer below 1e-3 on the slots.
      Report("Boot with " + std::to_string(ns) + " slots", m, got, ns >= 64 ? 1e-3 : 5e-3);
    }
    {
      // imaginary-removing variant on a real message (256 slots)
      const int ns = 1 << 8;
      boot_ctx->PrepareEvalSpecialFFT(ns, BootVariant::kImaginaryRemoving);
      EvkRequest req;
      boot_ctx->AddRequiredRotations(req, ns);
      ui.PrepareRotationKey(req);
      Msg m(ns), got;
      Random::SampleUniformComplex(m.data(), ns, -1.0, 1.0);
      for (auto &x : m) x = Complex(x.real(), 0);
      Pt pt, dec;
      Ct ct, out;
      ctx->encoder().Encode(pt, 0, param->GetScale(0), m, 0);
      ui.Encrypt(ct, pt);
      boot_ctx->Boot(out, ct, ui.GetEvkMap());
      ui.Decrypt(dec, out);
      ctx->encoder().Decode(got, dec);
      Report("Boot, imaginary-removing variant, 256 real slots", m, got, 1e-3);
    }
  }

  if (only.count("stages")) {
    // error introduced by each stage of Boot, against the same stage computed
    // in double precision from the decrypted input of that stage
    boot_ctx->PrepareEvalMod();
    boot_ctx->PrepareEvalSpecialFFT(n);
    EvkRequest req;
    boot_ctx->AddRequiredRotations(req, n);
    ui.PrepareRotationKey(req);
    const auto &evk = ui.GetEvkMap();
    Msg m;
    random_msg(m, -1, 1, true);
    Ct ct, up, raised, slots, conj, re, im, re_mod, im_mod, sum, out;
    encrypt(ct, m, 0, param->GetScale(0));
    const int lsu = boot_ctx->GetLogScaleUp();
    {
      Constant<word> k;
      ctx->encoder().EncodeConstant(k, 0, 1.0, (double)(1 << lsu), 0);
      ctx->Mult(up, ct, k);
      up.SetScale(ct.GetScale() * (1 << lsu));
    }
    boot_ctx->ModUpToMax(raised, up, evk);
    double q0 = 1;
    for (word q : param->GetPrimeVector(param->LevelToNP(-1))) q0 *= q;
    raised.SetScale(q0);
    Msg z0, z1, got;
    decrypt(z0, raised);
    {
      double big = 0;
      for (auto &x : z0) big = std::max(big, std::abs(x));
      std::cout << "       raised: max |slot| at scale q0 = " << big << std::endl;
    }
    auto cts = EvalSpecialFFT<word>::Groups(*param, n, true, boot_param.num_cts_levels_,
                                            1.0 / ((double)n * 2.0 * boot_param.K_));
    z1 = z0;
    for (auto &g : cts) z1 = g.Apply(z1);
    {
      double big = 0;
      for (auto &x : z1) big = std::max(big, std::max(std::abs(x.real()), std::abs(x.imag())));
      std::cout << "       after CtS: max |u|/(2K) = " << big << "  (max |u| = " << big * 2 * boot_param.K_ << ")" << std::endl;
    }
    boot_ctx->CoeffToSlot(slots, raised, evk);
    decrypt(got, slots);
    Report("stage CoeffToSlot", z1, got, 1e-9);
    ctx->HConj(conj, slots, evk.GetConjugationKey());
    ctx->Add(re, slots, conj);
    ctx->Sub(im, conj, slots);
    ctx->MultImaginaryUnit(im, im);
    Msg re_in, im_in, expect;
    decrypt(re_in, re);
    decrypt(im_in, im);
    boot_ctx->EvaluateMod(re_mod, re, evk.GetMultiplicationKey());
    boot_ctx->EvaluateMod(im_mod, im, evk.GetMultiplicationKey());
    auto sine = [&](const Msg &in) {
      Msg o;
      for (auto &x : in) o.push_back(Complex(std::sin(2 * M_PI * boot_param.K_ * x.real()) / (2 * M_PI), 0));
      return o;
    };
    decrypt(got, re_mod);
    Report("stage EvalMod (real part)", sine(re_in), got, 1e-8);
    Msg re_out = got;
    decrypt(got, im_mod);
    Report("stage EvalMod (imaginary part)", sine(im_in), got, 1e-8);
    ctx->MultImaginaryUnit(im_mod, im_mod);
    ctx->Add(sum, re_mod, im_mod);
    Msg z2;
    decrypt(z2, sum);
    auto stc = EvalSpecialFFT<word>::Groups(*param, n, false, boot_param.num_stc_levels_,
                                            q0 / (param->GetScale(0) * (1 << lsu)));
    Msg z3 = z2;
    for (auto &g : stc) z3 = g.Apply(z3);
    boot_ctx->SlotToCoeff(out, sum, evk);
    decrypt(got, out);
    Report("stage SlotToCoeff", z3, got, 1e-5);
    Report("whole Boot", m, got, 1e-3);
    // where the largest errors sit
    std::vector<std::pair<double, int>> worst;
    for (int i = 0; i < n; i++) worst.emplace_back(std::abs(m[i] - got[i]), i);
    std::sort(worst.rbegin(), worst.rend());
    std::cout << "       largest errors (slot: error):";
    for (int i = 0; i < 8; i++) std::cout << "  " << worst[i].second << ": " << std::scientific << worst[i].first;
    std::cout << std::endl;
  }

  std::cout << (failures ? "FAILED " : "PASSED ") << "(" << failures << " failures)" << std::endl;
  return failures ? 1 : 0;
}
