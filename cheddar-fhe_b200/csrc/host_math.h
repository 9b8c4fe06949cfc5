// Host-side number theory and table construction (no CUDA dependency).
//
// The choices that change results bit for bit follow the reference:
//   - psi = g^((q-1)/2N) with g the smallest primitive root
//     (reference include/common/PrimeUtils.h:135-196);
//   - forward table entry j is psi^bitrev(j), inverse table psi^-bitrev(j)
//     (reference src/core/NTT.cu:1254-1290).
// Unlike the reference the tables hold plain residues with a Shoup quotient,
// not Montgomery forms; the transforms they produce are the same mod q.
#pragma once
#include <stdint.h>

#include <vector>

#include "ntt_core.cuh"

namespace cfhe {

inline uint32_t mulmod(uint32_t a, uint32_t b, uint32_t q) {
  return (uint32_t)(((uint64_t)a * b) % q);
}

inline uint32_t powmod(uint32_t a, uint64_t e, uint32_t q) {
  uint32_t r = 1;
  a %= q;
  for (; e; e >>= 1) {
    if (e & 1) r = mulmod(r, a, q);
    a = mulmod(a, a, q);
  }
  return r;
}

inline uint32_t invmod(uint32_t a, uint32_t q) { return powmod(a, (uint64_t)q - 2, q); }

inline uint32_t smallest_generator(uint32_t q) {
  std::vector<uint32_t> f;
  uint32_t t = q - 1;
  for (uint32_t i = 2; (uint64_t)i * i <= t; i++)
    if (t % i == 0) {
      f.push_back(i);
      while (t % i == 0) t /= i;
    }
  if (t > 1) f.push_back(t);
  for (uint32_t r = 2; r < q; r++) {
    bool ok = true;
    for (uint32_t p : f)
      if (powmod(r, (q - 1) / p, q) == 1) {
        ok = false;
        break;
      }
    if (ok) return r;
  }
  return 0;
}

inline uint32_t bitrev(uint32_t v, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++) r |= ((v >> i) & 1u) << (bits - 1 - i);
  return r;
}

inline Tw make_tw(uint32_t w, uint32_t q) {
  return Tw{w, (uint32_t)((((uint64_t)w) << 32) / q)};
}

inline uint32_t r_mod(uint32_t q) { return (uint32_t)((1ULL << 32) % q); }
inline uint32_t rinv_mod(uint32_t q) { return invmod(r_mod(q), q); }
inline uint32_t to_mont(uint32_t a, uint32_t q) {
  return (uint32_t)((((uint64_t)a) << 32) % q);
}

// fwd[j] = psi^bitrev(j), inv[j] = psi^-bitrev(j), j in [0, N)
inline void build_twiddles(uint32_t q, int logn, Tw *fwd, Tw *inv,
                           uint32_t *psi_out) {
  const int n = 1 << logn;
  uint32_t g = smallest_generator(q);
  uint32_t psi = powmod(g, (q - 1) / (2u * n), q);
  uint32_t ipsi = invmod(psi, q);
  if (psi_out) *psi_out = psi;
  std::vector<uint32_t> pw(n);
  pw[0] = 1;
  for (int j = 1; j < n; j++) pw[j] = mulmod(pw[j - 1], psi, q);
  for (int j = 0; j < n; j++) fwd[j] = make_tw(pw[bitrev(j, logn)], q);
  pw[0] = 1;
  for (int j = 1; j < n; j++) pw[j] = mulmod(pw[j - 1], ipsi, q);
  for (int j = 0; j < n; j++) inv[j] = make_tw(pw[bitrev(j, logn)], q);
}

}  // namespace cfhe
