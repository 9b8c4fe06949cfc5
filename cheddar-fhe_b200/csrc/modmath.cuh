// Device-side Montgomery arithmetic for the element-wise and base-conversion
// kernels. R = 2^32; nqinv = -q^-1 mod 2^32; all residues canonical [0,q),
// q odd below 2^31. The values produced are the canonical representatives of
// a*b*R^-1 mod q, i.e. the same words the reference's signed lazy reduction
// yields after its final fold (reference include/common/Basic.cuh:72-157).
#pragma once
#include <stdint.h>

namespace cfhe {

__device__ __forceinline__ uint32_t fold_q(uint32_t r, uint32_t q) {
  return min(r, r - q);  // r in [0,2q)
}

// t < q * 2^32  ->  t * R^-1 mod q in [0,q)
__device__ __forceinline__ uint32_t mont_reduce(uint64_t t, uint32_t q,
                                                uint32_t nqinv) {
  const uint32_t m = (uint32_t)t * nqinv;
  const uint64_t u = t + (uint64_t)m * q;  // low word cancels
  return fold_q((uint32_t)(u >> 32), q);
}

__device__ __forceinline__ uint32_t mont_mul(uint32_t a, uint32_t b, uint32_t q,
                                             uint32_t nqinv) {
  return mont_reduce((uint64_t)a * b, q, nqinv);
}

__device__ __forceinline__ uint32_t add_mod(uint32_t a, uint32_t b, uint32_t q) {
  return fold_q(a + b, q);
}

__device__ __forceinline__ uint32_t sub_mod(uint32_t a, uint32_t b, uint32_t q) {
  const uint32_t d = a - b;
  return a < b ? d + q : d;
}

// acc < q*2^32 on entry and exit; adds a*b (a, b < q).
__device__ __forceinline__ void mac_fold(uint64_t &acc, uint32_t a, uint32_t b,
                                         uint64_t q32) {
  acc += (uint64_t)a * b;
  if (acc >= q32) acc -= q32;
}

// signed t in [-q*2^31, q*2^31)  ->  t * R^-1 mod q in [0,q)
__device__ __forceinline__ uint32_t mont_reduce_signed(int64_t t, uint32_t q,
                                                       uint32_t qinv) {
  const int32_t lo = (int32_t)(uint32_t)t;
  const int32_t hi = (int32_t)(t >> 32);
  const int32_t m = lo * (int32_t)qinv;
  int32_t r = hi - __mulhi(m, (int32_t)q);
  if (r < 0) r += (int32_t)q;
  return (uint32_t)r;
}

}  // namespace cfhe
