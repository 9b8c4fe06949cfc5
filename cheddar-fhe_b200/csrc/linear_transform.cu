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

// A thread owns the output pair (y, y + 1), y even. Flipping the lowest index
// bit adds N to the exponent, and (e + N) g = e g + N (mod 2N) for odd g, so
// the two sources are also a pair (x, x ^ 1): every operand is fetched as one
// aligned 8-byte word, the two inner products are formed in source order and
// swapped into output order when x is odd.
template <int G>
__global__ void __launch_bounds__(kLtThreads)
    lt_baby_kernel(const __grid_constant__ LtBabyArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y;
  const uint32_t y = 2 * (blockIdx.x * kLtThreads + threadIdx.x);
  const uint32_t q = a.q[l], nq = a.nqinv[l], pm = a.pm[l];
  const uint64_t q32 = (uint64_t)q << 32;
  const size_t limb = (size_t)l * kN, poly = (size_t)a.ntot * kN;
  const size_t koff = (size_t)a.kpos[l] * kN;
  const bool on_q = l < a.nq;
  uint64_t sb[G][2], sa[G][2];
#pragma unroll
  for (int j = 0; j < G; j++) sb[j][0] = sb[j][1] = sa[j][0] = sa[j][1] = 0;
  // ModUp (or own-limb) rows of this limb, one per active digit
  const uint32_t *xrow[kMaxDigits];
#pragma unroll
  for (int d = 0; d < kMaxDigits; d++)
    xrow[d] = a.own_digit[l] == d ? a.in_a + limb : a.mu + ((size_t)a.mu_slot[d] * a.ntot + l) * kN;
  auto ld2 = [](const uint32_t *p) { return *reinterpret_cast<const uint2 *>(p); };
  auto ld2cs = [](const uint32_t *p) { return __ldcs(reinterpret_cast<const uint2 *>(p)); };
#pragma unroll 1
  for (int i = 0; i < a.n_baby; i++) {
    uint32_t rb0 = 0, rb1 = 0, ra0 = 0, ra1 = 0;  // rotated words at y and y + 1
    if (i + 2 < a.n_baby) {
      // The key and plaintext words of the rotation after next start their
      // way from DRAM to L2 now (distance 2 measured best; 1, 3 and 4 lose
      // 1 % each): a thread's rotations are serial, so without this every
      // iteration pays the full DRAM latency before its arithmetic. Written
      // in line: as a lambda the same code cost 44 more registers.
      const uint32_t xn = source_index(y, a.galois[i + 2]) & ~1u;
#pragma unroll
      for (int d = 0; d < kMaxDigits; d++)
        if (d < a.n_digits) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a.kb[(i + 2) * kMaxDigits + d] + koff + xn));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(a.ka[(i + 2) * kMaxDigits + d] + koff + xn));
        }
#pragma unroll
      for (int j = 0; j < G; j++)
        if (j < a.n_giant) {
          const uint32_t *p = a.pt[j * kMaxBaby + i + 2];
          if (p) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + limb + y));
        }
    }
    if (i == 0) {
      // the unrotated input joins as P * (b, a)
      if (on_q) {
        const uint2 b = ld2(a.in_b + limb + y), c = ld2(a.in_a + limb + y);
        rb0 = mont_mul(b.x, pm, q, nq);
        rb1 = mont_mul(b.y, pm, q, nq);
        ra0 = mont_mul(c.x, pm, q, nq);
        ra1 = mont_mul(c.y, pm, q, nq);
      }
    } else {
      const uint32_t x = source_index(y, a.galois[i]);
      const uint32_t xe = x & ~1u;
      uint64_t tb0 = 0, tb1 = 0, ta0 = 0, ta1 = 0;
      // two products per fold: 2 q^2 <= q * 2^32 for q < 2^31
#pragma unroll
      for (int d = 0; d < kMaxDigits; d += 2)
        if (d < a.n_digits) {
          const bool two = d + 1 < a.n_digits;
          const uint2 z = make_uint2(0u, 0u);
          const uint2 x0 = ld2(xrow[d] + xe), x1 = two ? ld2(xrow[d + 1] + xe) : z;
          const uint2 b0 = ld2cs(a.kb[i * kMaxDigits + d] + koff + xe);
          const uint2 a0 = ld2cs(a.ka[i * kMaxDigits + d] + koff + xe);
          const uint2 b1 = two ? ld2cs(a.kb[i * kMaxDigits + d + 1] + koff + xe) : z;
          const uint2 a1 = two ? ld2cs(a.ka[i * kMaxDigits + d + 1] + koff + xe) : z;
          tb0 += (uint64_t)x0.x * b0.x + (uint64_t)x1.x * b1.x;
          tb1 += (uint64_t)x0.y * b0.y + (uint64_t)x1.y * b1.y;
          ta0 += (uint64_t)x0.x * a0.x + (uint64_t)x1.x * a1.x;
          ta1 += (uint64_t)x0.y * a0.y + (uint64_t)x1.y * a1.y;
          if (tb0 >= q32) tb0 -= q32;
          if (tb1 >= q32) tb1 -= q32;
          if (ta0 >= q32) ta0 -= q32;
          if (ta1 >= q32) ta1 -= q32;
        }
      if (on_q) {
        const uint2 c0 = ld2(a.in_b + limb + xe);
        mac_fold(tb0, c0.x, pm, q32);
        mac_fold(tb1, c0.y, pm, q32);
      }
      const uint32_t eb0 = mont_reduce(tb0, q, nq), eb1 = mont_reduce(tb1, q, nq);
      const uint32_t ea0 = mont_reduce(ta0, q, nq), ea1 = mont_reduce(ta1, q, nq);
      const bool swap = x & 1u;  // y comes from the odd source
      rb0 = swap ? eb1 : eb0;
      rb1 = swap ? eb0 : eb1;
      ra0 = swap ? ea1 : ea0;
      ra1 = swap ? ea0 : ea1;
    }
#pragma unroll
    for (int j = 0; j < G; j++)
      if (j < a.n_giant) {
        const uint32_t *p = a.pt[j * kMaxBaby + i];
        if (p) {
          const uint2 w = ld2cs(p + limb + y);
          mac_fold(sb[j][0], rb0, w.x, q32);
          mac_fold(sb[j][1], rb1, w.y, q32);
          mac_fold(sa[j][0], ra0, w.x, q32);
          mac_fold(sa[j][1], ra1, w.y, q32);
        }
      }
  }
#pragma unroll
  for (int j = 0; j < G; j++)
    if (j < a.n_giant) {
      *reinterpret_cast<uint2 *>(a.acc + (size_t)(2 * j) * poly + limb + y) =
          make_uint2(mont_reduce(sb[j][0], q, nq), mont_reduce(sb[j][1], q, nq));
      *reinterpret_cast<uint2 *>(a.acc + (size_t)(2 * j + 1) * poly + limb + y) =
          make_uint2(mont_reduce(sa[j][0], q, nq), mont_reduce(sa[j][1], q, nq));
    }
}

}  // namespace

int launch_lt_baby(const Context &ctx, const LtBabyArgs &a) {
  const dim3 grid(kN / 2 / kLtThreads, a.ntot), block(kLtThreads);
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
