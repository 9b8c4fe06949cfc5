// Thin extern "C" driver over the UNMODIFIED reference library, built by
// oracle/Makefile into oracle/_ref/libcheddar_ref.so from the sources where
// they lie (test infrastructure; nothing in the product links it).
//
// It lets the GPU tests run the reference's own kernels on the same device
// buffers as this repository's engine and compare the words, and lets the
// benchmark time the reference's HMult / NTT on the same B200. Only public
// members of the reference's classes are used (Context::ntt_handler_,
// mod_switch_handlers_, the containers' bx_/ax_ vectors).
#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include <chrono>
#include <cmath>
#include <complex>

#include "Random.h"
#include "UserInterface.h"
#include "core/Context.h"
#include "core/EvkMap.h"
#include "extension/BootContext.h"
#include "extension/Hoist.h"

using word = uint32_t;
using namespace cheddar;

struct RefHandle {
  std::unique_ptr<Parameter<word>> param;
  std::shared_ptr<Context<word>> ctx;
};

namespace {
void d2d(word *dst, const word *src, size_t words) {
  cudaMemcpyAsync(dst, src, words * sizeof(word), cudaMemcpyDeviceToDevice, cudaStreamLegacy);
}

void fill_ct(RefHandle *h, Ciphertext<word> &ct, int level, const word *b, const word *a) {
  NPInfo np = h->param->LevelToNP(level);
  ct.ModifyNP(np);
  size_t words = (size_t)np.GetNumTotal() * h->param->degree_;
  d2d(ct.bx_.data(), b, words);
  d2d(ct.ax_.data(), a, words);
  ct.SetScale(1.0);
}

void fill_key(RefHandle *h, EvaluationKey<word> &key, int key_main, const word *const *kb,
              const word *const *ka, int beta) {
  NPInfo np(key_main, h->param->GetMaxNumTer(), h->param->alpha_);
  key = EvaluationKey<word>(np, beta);
  size_t words = (size_t)np.GetNumTotal() * h->param->degree_;
  for (int j = 0; j < beta; j++) {
    d2d(key.bx_[j].data(), kb[j], words);
    d2d(key.ax_[j].data(), ka[j], words);
  }
}
}  // namespace

extern "C" {

RefHandle *ref_create(int log_degree, double base_scale, int default_level, const word *main_p,
                      int n_main, const word *ter_p, int n_ter, const word *aux_p, int n_aux,
                      const int *level_config, int n_levels) {
  auto *h = new RefHandle();
  std::vector<std::pair<int, int>> lc;
  for (int i = 0; i < n_levels; i++) lc.emplace_back(level_config[2 * i], level_config[2 * i + 1]);
  h->param = std::make_unique<Parameter<word>>(
      log_degree, base_scale, default_level, lc, std::vector<word>(main_p, main_p + n_main),
      std::vector<word>(aux_p, aux_p + n_aux), std::vector<word>(ter_p, ter_p + n_ter));
  h->ctx = Context<word>::Create(*h->param);
  cudaDeviceSynchronize();
  return h;
}

void ref_destroy(RefHandle *h) {
  if (!h) return;
  h->ctx.reset();
  h->param.reset();
  delete h;
}

// NTTHandler::NTT / INTT on a polynomial with (num_main, num_ter, num_aux) limbs
int ref_ntt(RefHandle *h, word *dst, const word *src, int num_main, int num_ter, int num_aux,
            int inverse, int mont_conv) {
  NPInfo np(num_main, num_ter, num_aux);
  int n = h->param->degree_;
  int total = np.GetNumTotal() * n, aux = num_aux * n;
  DvView<word> d(dst, total, aux);
  DvConstView<word> s(src, total, aux);
  if (inverse)
    h->ctx->ntt_handler_.INTT(d, np, s, mont_conv != 0);
  else
    h->ctx->ntt_handler_.NTT(d, np, s, mont_conv != 0);
  return (int)cudaDeviceSynchronize();
}

// ModSwitchHandler::ModUp: dst = beta buffers of (nq+alpha) limbs back to back
int ref_modup(RefHandle *h, int level, word *dst, const word *src) {
  NPInfo np = h->param->LevelToNP(level);
  int n = h->param->degree_, alpha = h->param->alpha_;
  int nq = np.GetNumQ();
  const auto &ms = h->ctx->mod_switch_handlers_.at(level);
  int beta = (np.num_main_ + h->param->GetMaxNumTer() + alpha - 1) / alpha;
  std::vector<DvView<word>> views;
  for (int i = 0; i < beta; i++)
    views.emplace_back(dst + (size_t)i * (nq + alpha) * n, (nq + alpha) * n, alpha * n);
  ms.ModUp(views, DvConstView<word>(src, nq * n, 0));
  return (int)cudaDeviceSynchronize();
}

// type 0 ModDown, 1 Rescale, 2 ModDownAndRescale
int ref_moddown(RefHandle *h, int level, int type, word *dst, const word *src) {
  int n = h->param->degree_, alpha = h->param->alpha_;
  NPInfo np = h->param->LevelToNP(level);
  int nq = np.GetNumQ();
  int nd = type == 0 ? nq : h->param->LevelToNP(level - 1).GetNumQ();
  const auto &ms = h->ctx->mod_switch_handlers_.at(level);
  DvView<word> d(dst, nd * n, 0);
  if (type == 0)
    ms.ModDown(d, DvConstView<word>(src, (nq + alpha) * n, alpha * n));
  else if (type == 1)
    ms.Rescale(d, DvConstView<word>(src, nq * n, 0));
  else
    ms.ModDownAndRescale(d, DvConstView<word>(src, (nq + alpha) * n, alpha * n));
  return (int)cudaDeviceSynchronize();
}

// Context::HMult; evaluation key digits given as device pointers laid out over
// (all terminal, key_main main, alpha aux) limbs. iters > 1 repeats the call
// for timing and returns the mean device time of one call in microseconds
// through *usec (CUDA events on the legacy stream, 5 warm-up calls first).
int ref_hmult(RefHandle *h, int level, word *out_b, word *out_a, const word *b1, const word *a1,
              const word *b2, const word *a2, const word *const *kb, const word *const *ka,
              int key_main, int beta, int rescale, int iters, float *usec) {
  Ciphertext<word> x, y, res;
  fill_ct(h, x, level, b1, a1);
  fill_ct(h, y, level, b2, a2);
  EvaluationKey<word> key;
  fill_key(h, key, key_main, kb, ka, beta);
  h->ctx->HMult(res, x, y, key, rescale != 0);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  size_t words = (size_t)res.GetNP().GetNumTotal() * h->param->degree_;
  d2d(out_b, res.bx_.data(), words);
  d2d(out_a, res.ax_.data(), words);
  if (iters > 1 && usec) {
    for (int i = 0; i < 5; i++) h->ctx->HMult(res, x, y, key, rescale != 0);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, cudaStreamLegacy);
    for (int i = 0; i < iters; i++) h->ctx->HMult(res, x, y, key, rescale != 0);
    cudaEventRecord(e1, cudaStreamLegacy);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    *usec = ms * 1000.0f / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  return (int)cudaDeviceSynchronize();
}

// Forward + inverse NTT of `polys` polynomials (as the reference would run
// config 1: one call per polynomial); mean device time per fwd+inv pass of
// the whole batch in microseconds.
int ref_ntt_batch_time(RefHandle *h, word *buf_a, word *buf_b, int polys, int num_main,
                       int num_ter, int iters, float *usec) {
  NPInfo np(num_main, num_ter, 0);
  int n = h->param->degree_;
  size_t pw = (size_t)np.GetNumTotal() * n;
  auto pass = [&]() {
    for (int p = 0; p < polys; p++) {
      DvView<word> d(buf_b + p * pw, (int)pw, 0);
      h->ctx->ntt_handler_.NTT(d, np, DvConstView<word>(buf_a + p * pw, (int)pw, 0), false);
    }
    for (int p = 0; p < polys; p++) {
      DvView<word> d(buf_a + p * pw, (int)pw, 0);
      h->ctx->ntt_handler_.INTT(d, np, DvConstView<word>(buf_b + p * pw, (int)pw, 0), false);
    }
  };
  for (int i = 0; i < 3; i++) pass();
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0, cudaStreamLegacy);
  for (int i = 0; i < iters; i++) pass();
  cudaEventRecord(e1, cudaStreamLegacy);
  cudaEventSynchronize(e1);
  float ms = 0;
  cudaEventElapsedTime(&ms, e0, e1);
  *usec = ms * 1000.0f / iters;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return (int)cudaDeviceSynchronize();
}

// Config 3 on the reference: n_rot rotations of one ciphertext at `level`.
//   usec[0]: n_rot calls of Context::HRot (src/core/Context.cpp:776-791), one
//            full key switch per rotation;
//   usec[1]: HoistHandler::EvaluateBabyStep (src/extension/Hoist.cu:578-691),
//            the reference's hoisted form: one ModUp shared by all rotations.
// The same key digits are installed for every distance (timing does not depend
// on key values). Mean device time of one sweep in microseconds, CUDA events
// on the legacy stream after warm-up sweeps.
int ref_rotations_time(RefHandle *h, int level, const word *b, const word *a, const word *const *kb,
                       const word *const *ka, int key_main, int beta, int n_rot, const int *rots,
                       int iters, float *usec) {
  Ciphertext<word> x, res;
  fill_ct(h, x, level, b, a);
  const int num_slots = h->param->degree_ / 2;
  x.SetNumSlots(num_slots);
  EvkMap<word> keys;
  for (int i = 0; i < n_rot; i++) {
    EvaluationKey<word> key;
    fill_key(h, key, key_main, kb, ka, beta);
    keys.emplace(rots[i], std::move(key));
  }
  auto timed = [&](auto &&sweep, float *out) {
    for (int i = 0; i < 2; i++) sweep();
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, cudaStreamLegacy);
    for (int i = 0; i < iters; i++) sweep();
    cudaEventRecord(e1, cudaStreamLegacy);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    *out = ms * 1000.0f / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  };
  timed([&]() {
    for (int i = 0; i < n_rot; i++) h->ctx->HRot(res, x, keys.GetRotationKey(rots[i]), rots[i]);
  }, &usec[0]);
  if (cudaDeviceSynchronize() != cudaSuccess) return (int)cudaGetLastError();
  // hoisted baby step: a hoist map with one (unit) plaintext per rotation in giant step 0
  PlainHoistMap map;
  for (int i = 0; i < n_rot; i++) map[0].try_emplace(rots[i], num_slots, Complex(1.0, 0.0));
  {
    HoistHandler<word> hoist(h->ctx, map, level, 1.0, true);
    timed([&]() {
      std::map<int, Ciphertext<word>> bs;
      hoist.EvaluateBabyStep(h->ctx, bs, x, keys, false);
    }, &usec[1]);
  }
  return (int)cudaDeviceSynchronize();
}

// The reference's bootstrapping test (unittest/Bootstrapping.cpp:10-41) without
// gtest: BootContext + UserInterface on the given parameter set, Boot of a
// level-0 encryption of 2^(logN-1) random complex slots in [-1,1]^2, five
// warm-up calls, then `iters` timed calls (host clock around a device
// synchronisation, as the reference's profiling macro measures).
// out[0] = mean ms per Boot, out[1] = max |diff| per component, out[2] = mean
// |diff|, out[3] = seconds spent preparing keys and plaintexts, out[4] =
// number of rotation keys, out[5] = output level. min_ks selects the
// reference's minimum-key-switching variant.
int ref_boot(int log_degree, double base_scale, int default_level, const word *main_p, int n_main,
             const word *ter_p, int n_ter, const word *aux_p, int n_aux, const int *level_config,
             int n_levels, int dense_h, int sparse_h, int num_cts, int num_stc, int min_ks, int iters,
             double *out) {
  std::vector<std::pair<int, int>> lc;
  for (int i = 0; i < n_levels; i++) lc.emplace_back(level_config[2 * i], level_config[2 * i + 1]);
  Parameter<word> param(log_degree, base_scale, default_level, lc,
                        std::vector<word>(main_p, main_p + n_main),
                        std::vector<word>(aux_p, aux_p + n_aux),
                        std::vector<word>(ter_p, ter_p + n_ter));
  if (dense_h > 0) param.SetDenseHammingWeight(dense_h);
  if (sparse_h > 0) param.SetSparseHammingWeight(sparse_h);
  const int num_slots = param.degree_ / 2;
  auto t0 = std::chrono::steady_clock::now();
  std::shared_ptr<BootContext<word>> boot =
      BootContext<word>::Create(param, BootParameter(param.max_level_, num_cts, num_stc));
  {
    UserInterface<word> ui(boot);
    boot->PrepareEvalMod();
    boot->PrepareEvalSpecialFFT(num_slots);
    EvkRequest req;
    boot->AddRequiredRotations(req, num_slots, min_ks != 0);
    ui.PrepareRotationKey(req);
    cudaDeviceSynchronize();
    auto t1 = std::chrono::steady_clock::now();
    out[3] = std::chrono::duration<double>(t1 - t0).count();
    out[4] = (double)req.size();

    std::vector<Complex> msg(num_slots), got;
    Random::SampleUniformComplex(msg.data(), num_slots, -1.0, 1.0);
    Plaintext<word> pt;
    Ciphertext<word> ct, res;
    boot->encoder_.Encode(pt, 0, param.GetScale(0), msg);
    ui.Encrypt(ct, pt);
    for (int i = 0; i < 5; i++) boot->Boot(res, ct, ui.GetEvkMap(), min_ks != 0);
    cudaDeviceSynchronize();
    auto a = std::chrono::steady_clock::now();
    for (int i = 0; i < iters; i++) boot->Boot(res, ct, ui.GetEvkMap(), min_ks != 0);
    cudaError_t e = cudaDeviceSynchronize();
    auto b = std::chrono::steady_clock::now();
    if (e != cudaSuccess) return (int)e;
    out[0] = std::chrono::duration<double, std::milli>(b - a).count() / iters;
    Plaintext<word> dec;
    ui.Decrypt(dec, res);
    boot->encoder_.Decode(got, dec);
    double worst = 0, sum = 0;
    for (int i = 0; i < num_slots; i++) {
      worst = std::max(worst, std::max(std::abs(msg[i].real() - got[i].real()),
                                       std::abs(msg[i].imag() - got[i].imag())));
      sum += std::abs(msg[i] - got[i]);
    }
    out[1] = worst;
    out[2] = sum / num_slots;
    out[5] = (double)param.NPToLevel(res.GetNP());
  }
  boot.reset();
  return (int)cudaDeviceSynchronize();
}

}  // extern "C"
