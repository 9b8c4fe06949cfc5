// One encrypted transformer encoder layer against the float64 layer that
// evaluates the same Chebyshev series (oracle/transformer_plain.h). Parity
// unpinned by the reference: the reference has no transformer code, so the
// checker is the textbook layer in double precision.
//
//   transformer_test <parameter.json> [--stddev s] [--seed n] [--no-pair] [--workers T]
//
// Reduced dimensions (16 tokens, hidden 32, 2 heads of 16, feed-forward 64,
// batch 2048 sequences per ciphertext); every stage of the full-size layer runs:
// tensor-core projections, baby/giant token rotations, the four polynomial
// stages, single and paired bootstraps.
#include <cstring>
#include <iomanip>

#include "../../oracle/transformer_plain.h"
#include "cheddar/Transformer.h"

using namespace cheddar;
using word = uint32_t;

int main(int argc, char **argv) {
  if (argc < 2) {
    std::cerr << "usage: transformer_test <parameter.json> [--stddev s] [--seed n] [--no-pair] [--workers T]\n";
    return 2;
  }
  double stddev = 0.08;
  uint64_t seed = 2024;
  bool trace = false;  // decrypt after every stage and compare sequence 0 with the float64 layer
  int lanes = 0;       // sequences checked against the float64 layer (0 = all of them)
  TransformerConfig cfg = TransformerConfig::Small();
  for (int i = 2; i < argc; i++) {
    if (!strcmp(argv[i], "--stddev") && i + 1 < argc) stddev = atof(argv[++i]);
    else if (!strcmp(argv[i], "--seed") && i + 1 < argc) seed = strtoull(argv[++i], nullptr, 10);
    else if (!strcmp(argv[i], "--no-pair")) cfg.pair_boot = false;
    else if (!strcmp(argv[i], "--trace")) trace = true;
    else if (!strcmp(argv[i], "--base")) {
      // BERT-base shape; the float64 layer is evaluated for the first `lanes` sequences only
      const bool pair = cfg.pair_boot;
      const int workers = cfg.workers;
      cfg = TransformerConfig::BertBase();
      cfg.pair_boot = pair;
      cfg.workers = workers;
      stddev = 0.02;
      lanes = 2;
    } else if (!strcmp(argv[i], "--lanes") && i + 1 < argc) lanes = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--workers") && i + 1 < argc) cfg.workers = std::max(1, atoi(argv[++i]));
  }
  Random::Seed(0xBE27 + seed);
  ParameterJson json = LoadParameterJson(argv[1]);
  AssertTrue(json.boot, "the parameter file does not enable bootstrapping");
  auto param = MakeParameter<word>(json);
  BootParameter boot_param(param->max_level_, json.num_cts_levels, json.num_stc_levels);
  auto ctx = BootContext<word>::Create(*param, boot_param);
  UserInterface<word> ui(ctx);
  ui.UseDeviceSampling(true);
  const int slots = param->degree_ / 2;
  ctx->PrepareEvalMod();
  ctx->PrepareEvalSpecialFFT(slots);
  TransformerWeights w = TransformerWeights::Random(cfg, seed, stddev);
  EncryptedTransformerLayer<word> layer(ctx, cfg, w);
  EvkRequest req;
  ctx->AddRequiredRotations(req, slots);
  layer.AddRequiredRotations(req);
  ui.PrepareRotationKey(req);

  const int T = cfg.seq_len, H = cfg.hidden, B = layer.BatchSize();
  // activations N(0, 1): x[b][t][j]
  std::vector<double> x((size_t)B * T * H);
  {
    std::mt19937_64 gen(seed * 7919 + 1);
    std::normal_distribution<double> nd(0.0, 1.0);
    for (auto &v : x) v = nd(gen);
  }
  const int level = boot_param.GetEndLevel() - (cfg.pair_boot ? 1 : 0);
  std::vector<Ciphertext<word>> in(H), out;
  for (int j = 0; j < H; j++) {
    std::vector<Complex> msg(slots);
    for (int t = 0; t < T; t++)
      for (int b = 0; b < B; b++) msg[(size_t)t * B + b] = Complex(x[((size_t)b * T + t) * H + j] / cfg.act_div, 0.0);
    Plaintext<word> pt;
    ctx->encoder().Encode(pt, level, param->GetScale(level), msg, 0);
    ui.Encrypt(in[j], pt);
  }
  plain_transformer::Spec spec{T, H, cfg.heads, cfg.head_dim, cfg.ffn, cfg.score_range, cfg.sum_lo, cfg.sum_hi,
                               cfg.var_lo, cfg.var_hi, cfg.gelu_range, cfg.ln_eps, layer.polys().exp_c,
                               layer.polys().inv_c, layer.polys().rsqrt_c, layer.polys().gelu_c, false};
  plain_transformer::Weights pw{w.wq.data(), w.wk.data(), w.wv.data(), w.wo.data(), w.w1.data(), w.w2.data(),
                                w.bq.data(), w.bk.data(), w.bv.data(), w.bo.data(), w.b1.data(), w.b2.data(),
                                w.gamma1.data(), w.beta1.data(), w.gamma2.data(), w.beta2.data()};
  if (trace) {
    auto tr = std::make_shared<plain_transformer::Trace>();
    auto final_out = std::make_shared<std::vector<double>>();
    std::vector<double> x0(x.begin(), x.begin() + (size_t)T * H);
    plain_transformer::Layer(*final_out, x0, spec, pw, nullptr, tr.get());
    auto centre = [](std::vector<double> v, int width) {
      for (size_t t = 0; t < v.size() / width; t++) {
        double m = 0;
        for (int j = 0; j < width; j++) m += v[t * width + j];
        m /= width;
        for (int j = 0; j < width; j++) v[t * width + j] -= m;
      }
      return v;
    };
    layer.SetProbe([=, &ui, &ctx](const std::string &name, const std::vector<Ciphertext<word>> &cts, double unit) {
      std::vector<double> want;
      const int width = cts.size();
      if (name == "qkv") {
        want.resize((size_t)T * 3 * H);
        for (int t = 0; t < T; t++)
          for (int j = 0; j < H; j++) {
            want[(size_t)t * 3 * H + j] = tr->q[(size_t)t * H + j] / (std::sqrt((double)cfg.head_dim) * cfg.score_range);
            want[(size_t)t * 3 * H + H + j] = tr->k[(size_t)t * H + j];
            want[(size_t)t * 3 * H + 2 * H + j] = tr->v[(size_t)t * H + j];
          }
      } else if (name == "attention") want = tr->attention;
      else if (name == "centred sum 1") want = centre(tr->sum1, H);
      else if (name == "LayerNorm 1" || name == "LayerNorm 1, refreshed") want = tr->norm1;
      else if (name == "pre-activation") want = tr->pre;
      else if (name == "GELU") {  // the layer evaluates the even part: GELU(a) - a / 2
        want = tr->gelu;
        for (size_t i = 0; i < want.size(); i++) want[i] -= 0.5 * tr->pre[i];
      }
      else if (name == "centred sum 2") want = centre(tr->sum2, H);
      else if (name == "LayerNorm 2") want = *final_out;
      else return;
      double worst = 0, mag = 0;
      for (int j = 0; j < width; j++) {
        Plaintext<word> dec;
        std::vector<Complex> msg;
        ui.Decrypt(dec, cts[j]);
        ctx->encoder().Decode(msg, dec);
        for (int t = 0; t < T; t++) {
          const double g = msg[(size_t)t * B].real() * unit, wv = want[(size_t)t * width + j];
          worst = std::max(worst, std::abs(g - wv));
          mag = std::max(mag, std::abs(wv));
        }
      }
      std::cout << "trace " << name << ": level " << ctx->param_.NPToLevel(cts[0].GetNP()) << ", max |value| " << mag
                << ", max error " << worst << " (" << -std::log2(worst / unit) << " bits on the slot values)\n";
    });
  }
  layer.Forward(out, in, ui.GetEvkMap());
  std::cout << "stages:";
  for (auto &[name, s] : layer.StageSeconds()) std::cout << " [" << name << " " << std::fixed << std::setprecision(3) << s << " s]";
  std::cout << "\nbootstraps " << layer.Bootstraps() << ", output level " << param->NPToLevel(out[0].GetNP()) << "\n";

  // decrypt: got[b][t][j]
  std::vector<double> got((size_t)B * T * H);
  double imag_max = 0;
  for (int j = 0; j < H; j++) {
    Plaintext<word> dec;
    std::vector<Complex> msg;
    ui.Decrypt(dec, out[j]);
    ctx->encoder().Decode(msg, dec);
    for (int t = 0; t < T; t++)
      for (int b = 0; b < B; b++) {
        got[((size_t)b * T + t) * H + j] = msg[(size_t)t * B + b].real() * cfg.act_div;
        imag_max = std::max(imag_max, std::abs(msg[(size_t)t * B + b].imag()) * cfg.act_div);
      }
  }

  plain_transformer::Ranges ranges;
  double err_series = 0, err_exact = 0, approx_gap = 0, sum_sq = 0;
  const int checked = lanes > 0 ? std::min(lanes, B) : B;
  for (int b = 0; b < checked; b++) {
    std::vector<double> xb(x.begin() + (size_t)b * T * H, x.begin() + (size_t)(b + 1) * T * H), series, exact;
    spec.exact = false;
    plain_transformer::Layer(series, xb, spec, pw, &ranges);
    spec.exact = true;
    plain_transformer::Layer(exact, xb, spec, pw);
    for (size_t i = 0; i < series.size(); i++) {
      const double g = got[(size_t)b * T * H + i];
      err_series = std::max(err_series, std::abs(g - series[i]));
      err_exact = std::max(err_exact, std::abs(g - exact[i]));
      approx_gap = std::max(approx_gap, std::abs(series[i] - exact[i]));
      sum_sq += (g - series[i]) * (g - series[i]);
    }
  }
  const double rms = std::sqrt(sum_sq / ((double)checked * T * H));
  std::cout << "sequences checked against the float64 layer: " << checked << " of " << B << "\n";
  std::cout << std::scientific << std::setprecision(3);
  std::cout << "ranges: |score| " << ranges.score_abs << " of " << cfg.score_range << ", exp mean [" << ranges.sum_min
            << ", " << ranges.sum_max << "] of [" << cfg.sum_lo << ", " << cfg.sum_hi << "], variance ["
            << ranges.var_min << ", " << ranges.var_max << "] of [" << cfg.var_lo << ", " << cfg.var_hi
            << "], |pre-activation| " << ranges.pre_abs << " of " << cfg.gelu_range << ", |output| "
            << ranges.out_abs << "\n";
  std::cout << "max |encrypted - float64 layer with the same series| " << err_series << " (rms " << rms << ")\n";
  std::cout << "max |float64 series layer - float64 exact layer| " << approx_gap << "\n";
  std::cout << "max |encrypted - float64 exact layer| " << err_exact << "\n";
  std::cout << "max |imaginary part| " << imag_max << "\n";
  std::cout << std::fixed << std::setprecision(2);
  std::cout << "precision_bits " << -std::log2(err_series) << "\n";
  const bool in_range = ranges.score_abs < cfg.score_range && ranges.sum_min > cfg.sum_lo &&
                        ranges.sum_max < cfg.sum_hi && ranges.var_min > cfg.var_lo && ranges.var_max < cfg.var_hi &&
                        ranges.pre_abs < cfg.gelu_range && ranges.out_abs < cfg.act_div;
  if (!in_range) {
    std::cout << "FAIL: an input left the interval its series was fitted on\n";
    return 1;
  }
  // 12 bits on outputs of magnitude up to ~4: every slot correct to 2.4e-4
  if (!(err_series < std::ldexp(1.0, -12))) {
    std::cout << "FAIL: precision below 12 bits\n";
    return 1;
  }
  std::cout << "PASS\n";
  return 0;
}
