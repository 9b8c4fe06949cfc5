// Fused baby steps of the baby-step/giant-step linear transform.
//
// The unfused form runs one key inner product per baby rotation, stores the
// rotated ciphertext on the extended basis (2 x (nq+alpha) limbs), and a
// second kernel reads all of them back to form the giant-step sums
//   acc_j = sum_i pt[j][i] (*) rot_i.
// Here one thread owns one output word y of one limb and walks the baby
// rotations: the automorphism of rotation i sends source index x_i(y) to y, so
// the rotated word at y is the key inner product at x_i(y); it is reduced and
// multiplied into the running sums of all giant steps. The rotated
// ciphertexts never exist in memory: per rotation 2 x (nq+alpha) limbs are
// neither written nor read back. In the bit-reversed evaluation order an
// automorphism maps every aligned block of 128 indices onto an aligned block
// of 128, so the gathers of a 128-thread block stay inside one 512-byte window
// of each operand (staging those windows through shared memory with coalesced
// loads was measured slower than letting L1 serve the gathers).
// Word for word the same results as the unfused kernels: the rotated word is
// reduced to its canonical residue before it enters the giant-step sums.
#include <string.h>

#include "context.h"
#include "kernels.h"
#include "modmath.cuh"

namespace cfhe {
namespace {

constexpr int kLtThreads = 128;

// source index of output index y under the automorphism with Galois element g:
// exponent 2*brev(y)+1 is multiplied by g (mod 2N) and mapped back
__device__ __forceinline__ uint32_t source_index(uint32_t y, uint32_t g) {
  const uint32_t e = (__brev(y) >> (31 - kLogN)) + 1;
  return __brev((e * g - 1) << (31 - kLogN)) & (kN - 1);
}

template <int G>
__global__ void __launch_bounds__(kLtThreads)
    lt_baby_kernel(const __grid_constant__ LtBabyArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y;
  const uint32_t y = blockIdx.x * kLtThreads + threadIdx.x;
  const uint32_t q = a.q[l], nq = a.nqinv[l], pm = a.pm[l];
  const uint64_t q32 = (uint64_t)q << 32;
  const size_t limb = (size_t)l * kN, poly = (size_t)a.ntot * kN;
  const size_t koff = (size_t)a.kpos[l] * kN;
  const bool on_q = l < a.nq;
  uint64_t sb[G], sa[G];
#pragma unroll
  for (int j = 0; j < G; j++) sb[j] = sa[j] = 0;
  // ModUp (or own-limb) rows of this limb, one per active digit
  const uint32_t *xrow[kMaxDigits];
#pragma unroll
  for (int d = 0; d < kMaxDigits; d++)
    xrow[d] = a.own_digit[l] == d ? a.in_a + limb : a.mu + ((size_t)a.mu_slot[d] * a.ntot + l) * kN;
#pragma unroll 1
  for (int i = 0; i < a.n_baby; i++) {
    uint32_t rb = 0, ra = 0;
    if (i == 0) {
      // the unrotated input joins as P * (b, a)
      if (on_q) {
        rb = mont_mul(a.in_b[limb + y], pm, q, nq);
        ra = mont_mul(a.in_a[limb + y], pm, q, nq);
      }
    } else {
      const uint32_t x = source_index(y, a.galois[i]);
      uint64_t tb = 0, ta = 0;
      // two products per fold: 2 q^2 <= q * 2^32 for q < 2^31
#pragma unroll
      for (int d = 0; d < kMaxDigits; d += 2)
        if (d < a.n_digits) {
          const bool two = d + 1 < a.n_digits;
          const uint32_t x0 = xrow[d][x], x1 = two ? xrow[d + 1][x] : 0u;
          const uint32_t b0 = __ldcs(a.kb[i * kMaxDigits + d] + koff + x);
          const uint32_t a0 = __ldcs(a.ka[i * kMaxDigits + d] + koff + x);
          const uint32_t b1 = two ? __ldcs(a.kb[i * kMaxDigits + d + 1] + koff + x) : 0u;
          const uint32_t a1 = two ? __ldcs(a.ka[i * kMaxDigits + d + 1] + koff + x) : 0u;
          tb += (uint64_t)x0 * b0 + (uint64_t)x1 * b1;
          ta += (uint64_t)x0 * a0 + (uint64_t)x1 * a1;
          if (tb >= q32) tb -= q32;
          if (ta >= q32) ta -= q32;
        }
      if (on_q) mac_fold(tb, a.in_b[limb + x], pm, q32);
      rb = mont_reduce(tb, q, nq);
      ra = mont_reduce(ta, q, nq);
    }
#pragma unroll
    for (int j = 0; j < G; j++)
      if (j < a.n_giant) {
        const uint32_t *p = a.pt[j * kMaxBaby + i];
        if (p) {
          const uint32_t w = __ldcs(p + limb + y);
          mac_fold(sb[j], rb, w, q32);
          mac_fold(sa[j], ra, w, q32);
        }
      }
  }
#pragma unroll
  for (int j = 0; j < G; j++)
    if (j < a.n_giant) {
      a.acc[(size_t)(2 * j) * poly + limb + y] = mont_reduce(sb[j], q, nq);
      a.acc[(size_t)(2 * j + 1) * poly + limb + y] = mont_reduce(sa[j], q, nq);
    }
}

}  // namespace

int launch_lt_baby(const Context &ctx, const LtBabyArgs &a) {
  const dim3 grid(kN / kLtThreads, a.ntot), block(kLtThreads);
  cudaError_t e;
  if (a.n_giant <= 2)
    e = launch_kernel(ctx.use_pdl, lt_baby_kernel<2>, grid, block, 0, ctx.stream, a);
  else if (a.n_giant <= 4)
    e = launch_kernel(ctx.use_pdl, lt_baby_kernel<4>, grid, block, 0, ctx.stream, a);
  else if (a.n_giant <= 8)
    e = launch_kernel(ctx.use_pdl, lt_baby_kernel<8>, grid, block, 0, ctx.stream, a);
  else
    e = launch_kernel(ctx.use_pdl, lt_baby_kernel<16>, grid, block, 0, ctx.stream, a);
  CFHE_CUDA(e);
  return 0;
}

}  // namespace cfhe
