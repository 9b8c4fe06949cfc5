// Seconds per encrypted transformer encoder layer on one GPU, printed as one
// JSON line. Default shape: BERT-base (128 tokens, hidden 768, 12 heads of 64,
// feed-forward 3072) with weights N(0, 0.02) and activations N(0, 1), one
// ciphertext per feature, 256 sequences per ciphertext at N = 2^16. The
// reference has no transformer code (CMakeLists.txt:63-75), so there is no
// reference figure for this workload.
//
//   bert_bench <parameter.json> [--passes K] [--warmup W] [--workers T] [--small] [--no-pair]
//              [--rank r --world G --rendezvous path]
//
// With --world G > 1, G processes (one per GPU, each given its rank and the same
// rendezvous path) run ONE layer call together, sharded by heads and blocks of
// ciphertexts with NCCL all-gathers between the stages; every rank builds the
// same keys and inputs from the same seeds, rank 0 prints the line. The
// output_digest (a hash of three output ciphertexts) is the same for every G.
//
// W warm-up passes (default 1) come before the K timed ones (default 1); the
// first pass also encodes and packs the weight matrices (pack_weights_s, kept
// out of every pass's time). Each pass feeds the previous pass's output back
// in, as stacked layers would.
#include <cstring>
#include <iomanip>

#include "cheddar/Transformer.h"

// FNV-1a over the words of a ciphertext, continued from h
static uint64_t Digest(uint64_t h, const cheddar::Ciphertext<uint32_t> &ct) {
  std::vector<uint32_t> w;
  for (const auto *poly : {&ct.bx_, &ct.ax_}) {
    cheddar::CopyDeviceToHost(w, *poly);
    cheddar::CheckAbi(cfhe_synchronize(cheddar::detail::CurrentHandle()));
    for (uint32_t x : w) {
      h ^= x;
      h *= 1099511628211ull;
    }
  }
  return h;
}

using namespace cheddar;
using word = uint32_t;

int main(int argc, char **argv) {
  if (argc < 2) {
    std::cerr << "usage: bert_bench <parameter.json> [--passes K] [--warmup W] [--workers T] [--small] [--no-pair]\n";
    return 2;
  }
  int passes = 1, warmup = 1, workers = 4, rank = 0, world = 1;
  std::string rendezvous;
  TransformerConfig cfg = TransformerConfig::BertBase();
  double stddev = 0.02;
  for (int i = 2; i < argc; i++) {
    if (!strcmp(argv[i], "--passes") && i + 1 < argc) passes = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = std::max(0, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--small")) {
      const bool pair = cfg.pair_boot;
      cfg = TransformerConfig::Small();
      cfg.pair_boot = pair;
      stddev = 0.08;
    } else if (!strcmp(argv[i], "--no-pair")) cfg.pair_boot = false;
    else if (!strcmp(argv[i], "--workers") && i + 1 < argc) workers = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--rank") && i + 1 < argc) rank = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--world") && i + 1 < argc) world = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--rendezvous") && i + 1 < argc) rendezvous = argv[++i];
  }
  cfg.workers = workers;
  Random::Seed(20241125);
  auto clock = [] { return std::chrono::steady_clock::now(); };
  auto since = [&](std::chrono::steady_clock::time_point t) {
    return std::chrono::duration<double>(clock() - t).count();
  };
  const auto t_setup = clock();
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
  TransformerWeights w = TransformerWeights::Random(cfg, 1, stddev);
  std::shared_ptr<RankGroup> group;
  if (world > 1) {
#ifdef CHEDDAR_WITH_NCCL
    AssertTrue(!rendezvous.empty() && rank >= 0 && rank < world, "bert_bench: --rank, --world and --rendezvous go together");
    group = std::make_shared<NcclRankGroup>(rank, world, rendezvous);
#else
    Fail("bert_bench: built without NCCL");
#endif
  }
  EncryptedTransformerLayer<word> layer(ctx, cfg, w, group);
  EvkRequest req;
  ctx->AddRequiredRotations(req, slots);
  layer.AddRequiredRotations(req);
  ui.PrepareRotationKey(req);
  ctx->Synchronize();
  const double keys_s = since(t_setup);

  const auto t_enc = clock();
  const int T = cfg.seq_len, H = cfg.hidden, B = layer.BatchSize();
  const int level = boot_param.GetEndLevel() - (cfg.pair_boot ? 1 : 0);
  std::vector<Ciphertext<word>> cur(H), next;
  {
    std::mt19937_64 gen(99);
    std::normal_distribution<double> nd(0.0, 1.0);
    std::vector<Complex> msg(slots);
    for (int j = 0; j < H; j++) {
      for (auto &v : msg) v = Complex(nd(gen) / cfg.act_div, 0.0);
      Plaintext<word> pt;
      ctx->encoder().Encode(pt, level, param->GetScale(level), msg, 0);
      ui.Encrypt(cur[j], pt);
    }
  }
  const double encrypt_s = since(t_enc);

  // seconds per layer = the sum of the stage times of a pass, averaged over the
  // timed passes; the warm-up passes (the first one also encodes and packs the
  // weight matrices and grows the device memory pool) are reported beside it
  double timed_s = 0, gemm_s = 0, gemm_macs = 0, pack_s = 0, warm_s = 0;
  std::vector<std::pair<std::string, double>> stages;
  for (int p = 0; p < warmup + passes; p++) {
    layer.Forward(next, cur, ui.GetEvkMap());
    ctx->Synchronize();
    pack_s += layer.PackSeconds();
    double total = 0;
    for (auto &st : layer.StageSeconds()) total += st.second;
    if (p < warmup) {
      warm_s += total;
    } else {
      timed_s += total;
      gemm_s += layer.GemmSeconds();
      gemm_macs += layer.GemmInt8Macs();
      if (stages.empty()) stages = layer.StageSeconds();
      else
        for (size_t i = 0; i < stages.size(); i++) stages[i].second += layer.StageSeconds()[i].second;
    }
    std::swap(cur, next);
    next.clear();
  }
  const int timed = passes;
  // the output must still be a LayerNorm output: per token, features of mean
  // about mean(beta) and variance about 1 (sequence 0 decrypted)
  double worst_mean = 0, var_lo = 1e9, var_hi = 0;
  {
    std::vector<double> lane((size_t)T * H);
    for (int j = 0; j < H; j++) {
      Plaintext<word> dec;
      std::vector<Complex> msg;
      ui.Decrypt(dec, cur[j]);
      ctx->encoder().Decode(msg, dec);
      for (int t = 0; t < T; t++) lane[(size_t)t * H + j] = msg[(size_t)t * B].real() * cfg.act_div;
    }
    for (int t = 0; t < T; t++) {
      double m = 0, v = 0;
      for (int j = 0; j < H; j++) m += lane[(size_t)t * H + j];
      m /= H;
      for (int j = 0; j < H; j++) v += (lane[(size_t)t * H + j] - m) * (lane[(size_t)t * H + j] - m);
      v /= H;
      worst_mean = std::max(worst_mean, std::abs(m));
      var_lo = std::min(var_lo, v);
      var_hi = std::max(var_hi, v);
    }
  }
  uint64_t digest = 14695981039346656037ull;
  for (int j : {0, H / 2, H - 1}) digest = Digest(digest, cur[j]);
  if (rank != 0) return 0;
  std::cout << std::setprecision(6);
  std::cout << "{\"seconds_per_layer\": " << timed_s / timed << ", \"sequences_per_layer_call\": " << B
            << ", \"seconds_per_sequence\": " << timed_s / timed / B << ", \"passes_timed\": " << timed
             << ", \"warmup_passes\": " << warmup << ", \"warmup_s\": " << warm_s << ", \"pack_weights_s\": " << pack_s << ", \"keys_s\": " << keys_s << ", \"encrypt_s\": " << encrypt_s
            << ", \"shape\": {\"seq_len\": " << T << ", \"hidden\": " << H << ", \"heads\": " << cfg.heads
            << ", \"head_dim\": " << cfg.head_dim << ", \"ffn\": " << cfg.ffn << "}"
             << ", \"gpus\": " << world << ", \"output_digest\": \"" << std::hex << digest << std::dec << "\", \"host_threads\": " << cfg.workers << ", \"bootstraps_per_layer\": " << layer.Bootstraps() << ", \"paired_bootstraps\": "
            << (cfg.pair_boot ? "true" : "false") << ", \"level_in_out\": " << level
            << ", \"gemm_seconds_per_layer\": " << gemm_s / timed << ", \"gemm_int8_TOPS\": "
            << 2.0 * gemm_macs / gemm_s * 1e-12 << ", \"output_token_mean_abs_max\": " << worst_mean
            << ", \"output_token_variance\": [" << var_lo << ", " << var_hi << "], \"stages_s\": {";
  for (size_t i = 0; i < stages.size(); i++)
    std::cout << (i ? ", " : "") << "\"" << stages[i].first << "\": " << stages[i].second / timed;
  std::cout << "}}" << std::endl;
  return 0;
}
