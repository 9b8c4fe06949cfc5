// Host emulation of the cluster NTT/INTT kernels (test infrastructure).
// Runs the per-thread phase functions of csrc/ntt_core.cuh for every
// (CTA, thread) of one 8-CTA cluster, phase by phase, with plain arrays
// standing in for shared memory and for the other CTAs' receive buffers.
// This checks the index arithmetic and the lazy-range butterflies on the
// CPU; it does not replace the GPU parity tests.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "host_math.h"
#include "ntt_core.cuh"

using namespace cfhe;

namespace {
struct Cluster {
  std::vector<uint32_t> xbuf[kClusterSize], rbuf[kClusterSize];
  explicit Cluster(bool inverse) {
    for (int c = 0; c < kClusterSize; c++) {
      xbuf[c].assign(inverse ? kRowBufWords : kStripBufWords, 0xdeadbeefu);
      rbuf[c].assign(inverse ? kStripBufWords : kRowBufWords, 0xdeadbeefu);
    }
  }
};

template <bool FAST>
void fwd(const Tw *tw, uint32_t q, const uint32_t *src, uint32_t *dst,
         int premul, Tw kc) {
  Cluster cl(false);
  const uint32_t q2 = 2 * q;
  auto remote = [&](int rank) { return cl.rbuf[rank].data(); };
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++) {
      const int x = tid & 31, r0 = tid >> 5;
      uint32_t v[16];
      for (int k = 0; k < 16; k++) {
        v[k] = src[(r0 + 16 * k) * kRowWords + kStripCols * c + x];
        if (premul) v[k] = shoup_mul(v[k], kc, q);
      }
      fwd_rows_a<FAST>(v, tid, cl.xbuf[c].data(), tw, q, q2);
    }
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++)
      fwd_rows_b<FAST>(c, tid, cl.xbuf[c].data(), remote, tw, q, q2);
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++)
      fwd_cols_a<FAST>(c, tid, cl.rbuf[c].data(), cl.rbuf[c].data(), tw, q, q2);
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++) {
      uint32_t v[16];
      fwd_cols_b<FAST>(v, c, tid, cl.rbuf[c].data(), tw, q, q2);
      const int rho = tid >> 4, g = tid & 15, R = kOwnRows * c + rho;
      for (int k = 0; k < 16; k++) dst[R * kRowWords + 16 * g + k] = v[k];
    }
}

template <bool FAST>
void inv(const Tw *itw, uint32_t q, const uint32_t *src, uint32_t *dst, Tw kc,
         int centred) {
  Cluster cl(true);
  const uint32_t q2 = 2 * q;
  auto remote = [&](int rank) { return cl.rbuf[rank].data(); };
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++) {
      const int rho = tid >> 4, g = tid & 15, R = kOwnRows * c + rho;
      uint32_t v[16];
      for (int k = 0; k < 16; k++) v[k] = src[R * kRowWords + 16 * g + k];
      inv_cols_a<FAST>(v, c, tid, cl.xbuf[c].data(), itw, q, q2);
    }
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++)
      inv_cols_b<FAST>(c, tid, cl.xbuf[c].data(), remote, itw, q, q2);
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++)
      inv_rows_a<FAST>(tid, cl.rbuf[c].data(), cl.xbuf[c].data(), itw, q, q2);
  for (int c = 0; c < kClusterSize; c++)
    for (int tid = 0; tid < kNttThreads; tid++) {
      uint32_t v[16];
      inv_rows_b<FAST>(v, tid, cl.xbuf[c].data(), itw, kc, centred != 0, q, q2);
      const int x = tid & 31, r0 = tid >> 5;
      for (int k = 0; k < 16; k++)
        dst[(r0 + 16 * k) * kRowWords + kStripCols * c + x] = v[k];
    }
}
}  // namespace

extern "C" {
// mode 0: lazy path chosen by prime size as the kernels do; 1: force the
// [0,2q) path (valid for every prime).
void emu_ntt_fwd(uint32_t q, const uint32_t *src, uint32_t *dst, int mont_conv,
                 int force_slow) {
  std::vector<Tw> f(kN), i(kN);
  build_twiddles(q, kLogN, f.data(), i.data(), nullptr);
  Tw kc = make_tw(r_mod(q), q);
  if (q < (1u << 30) && !force_slow)
    fwd<true>(f.data(), q, src, dst, mont_conv, kc);
  else
    fwd<false>(f.data(), q, src, dst, mont_conv, kc);
}

// out = raw * k * 2^-32 mod q (k as the reference's Montgomery constant)
void emu_ntt_inv(uint32_t q, const uint32_t *src, uint32_t *dst, uint32_t k,
                 int centred, int force_slow) {
  std::vector<Tw> f(kN), i(kN);
  build_twiddles(q, kLogN, f.data(), i.data(), nullptr);
  Tw kc = make_tw(mulmod(k % q, rinv_mod(q), q), q);
  if (q < (1u << 30) && !force_slow)
    inv<true>(i.data(), q, src, dst, kc, centred);
  else
    inv<false>(i.data(), q, src, dst, kc, centred);
}
}
