// Bootstrapping latency and precision on one GPU, printed as one JSON line:
// the workload of the reference's boot_test (unittest/Bootstrapping.cpp:10-41):
// a level-0 encryption of 2^(logN-1) random complex slots in [-1,1]^2 is
// refreshed `iters` times after `warmup` untimed calls; the host clock
// brackets a device synchronisation on both sides, as the reference's
// profiling macro does (unittest/Testbed.h:24-47).
//
//   boot_bench <parameter.json> [--iters K] [--warmup W]
#include <chrono>
#include <cstring>
#include <iomanip>

#include "cheddar/Boot.h"

using namespace cheddar;
using word = uint32_t;

int main(int argc, char **argv) {
  if (argc < 2) {
    std::cerr << "usage: boot_bench <parameter.json> [--iters K] [--warmup W] [--one-stream]\n";
    return 2;
  }
  int iters = 10, warmup = 3;
  bool one_stream = false;  // both EvalMods on the main context's stream
  for (int i = 2; i < argc; i++) {
    if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = std::max(0, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--one-stream")) one_stream = true;
  }
  Random::Seed(20240607);
  ParameterJson json = LoadParameterJson(argv[1]);
  AssertTrue(json.boot, "the parameter file does not enable bootstrapping");
  auto param = MakeParameter<word>(json);
  BootParameter boot_param(param->max_level_, json.num_cts_levels, json.num_stc_levels);
  auto t0 = std::chrono::steady_clock::now();
  auto ctx = BootContext<word>::Create(*param, boot_param);
  UserInterface<word> ui(ctx);
  const int n = param->degree_ / 2;
  ctx->PrepareEvalMod();
  if (one_stream) ctx->UseSideStream(false);
  ctx->PrepareEvalSpecialFFT(n);
  EvkRequest req;
  ctx->AddRequiredRotations(req, n);
  ui.PrepareRotationKey(req);
  ctx->Synchronize();
  const double prepare_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();

  std::vector<Complex> msg(n), got;
  Random::SampleUniformComplex(msg.data(), n, -1.0, 1.0);
  Plaintext<word> pt, dec;
  Ciphertext<word> ct, out;
  ctx->encoder().Encode(pt, 0, param->GetScale(0), msg, 0);
  ui.Encrypt(ct, pt);
  for (int i = 0; i < warmup; i++) ctx->Boot(out, ct, ui.GetEvkMap());
  ctx->Synchronize();
  double total = 0, best = 1e30, enqueue = 0;
  for (int i = 0; i < iters; i++) {
    auto a = std::chrono::steady_clock::now();
    ctx->Boot(out, ct, ui.GetEvkMap());
    enqueue += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - a).count();
    ctx->Synchronize();
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - a).count();
    total += ms;
    best = std::min(best, ms);
  }
  // throughput: `iters` bootstraps enqueued back to back, one synchronisation
  // at the end (the host runs ahead of the GPU, so no launch gap is exposed)
  double back_to_back = 0;
  {
    Ciphertext<word> out2;
    auto a = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; i++) ctx->Boot(i & 1 ? out2 : out, ct, ui.GetEvkMap());
    ctx->Synchronize();
    back_to_back = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - a).count() / iters;
  }
  std::vector<std::pair<std::string, double>> phases;
  ctx->Boot(out, ct, ui.GetEvkMap(), false, &phases);
  ui.Decrypt(dec, out);
  ctx->encoder().Decode(got, dec);
  double worst = 0, sum = 0;
  for (int i = 0; i < n; i++) {
    worst = std::max({worst, std::abs(msg[i].real() - got[i].real()), std::abs(msg[i].imag() - got[i].imag())});
    sum += std::abs(msg[i] - got[i]);
  }
  std::cout << std::setprecision(6) << "{\"boot_ms\": " << total / iters << ", \"boot_ms_best\": " << best
            << ", \"boot_ms_back_to_back\": " << back_to_back << ", \"host_enqueue_ms\": " << enqueue / iters << ", \"iters\": " << iters << ", \"warmup\": " << warmup << ", \"slots\": " << n
            << ", \"end_level\": " << param->NPToLevel(out.GetNP()) << ", \"max_err\": " << worst
            << ", \"mean_err\": " << sum / n << ", \"precision_bits\": " << -std::log2(sum / n)
            << ", \"prepare_s\": " << prepare_s << ", \"rotation_keys\": " << req.size() << ", \"phases_ms\": {";
  for (size_t i = 0; i < phases.size(); i++)
    std::cout << (i ? ", " : "") << "\"" << phases[i].first << "\": " << phases[i].second;
  std::cout << "}}" << std::endl;
  return 0;
}
