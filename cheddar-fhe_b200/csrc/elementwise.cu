// Element-wise limb kernels: 128-bit accesses, one launch per operator over a
// table of rows (a row = one limb of one polynomial). These are pure
// streaming kernels; the values they produce are the canonical residues the
// reference's kernels produce (reference src/core/ElementWise.cu:32-658).
#include "context.h"
#include "kernels.h"
#include "modmath.cuh"

namespace cfhe {
namespace {

constexpr int kEwThreads = 256;
constexpr int kVecPerLimb = kN / 4;                    // uint4 per limb
constexpr int kEwBlocksX = kVecPerLimb / kEwThreads;   // 64

template <typename F>
__device__ __forceinline__ uint4 map4(uint4 a, uint4 b, F f) {
  return make_uint4(f(a.x, b.x), f(a.y, b.y), f(a.z, b.z), f(a.w, b.w));
}

template <int OP>
__global__ void __launch_bounds__(kEwThreads)
    ew_kernel(const __grid_constant__ EwArgs args) {
  pdl_launch_dependents();
  pdl_wait();
  const EwRow &r = args.rows[blockIdx.y];
  const int v = blockIdx.x * kEwThreads + threadIdx.x;
  const uint32_t q = r.q, nq = r.nqinv, k = r.k;
  uint4 a = reinterpret_cast<const uint4 *>(r.a)[v];
  uint4 b = make_uint4(0, 0, 0, 0);
  if constexpr (OP == EW_ADD || OP == EW_SUB || OP == EW_MUL || OP == EW_MULC_ADD)
    b = reinterpret_cast<const uint4 *>(r.b)[v];
  uint4 o;
  if constexpr (OP == EW_ADD)
    o = map4(a, b, [=](uint32_t x, uint32_t y) { return add_mod(x, y, q); });
  else if constexpr (OP == EW_SUB)
    o = map4(a, b, [=](uint32_t x, uint32_t y) { return sub_mod(x, y, q); });
  else if constexpr (OP == EW_NEG)
    o = map4(a, b, [=](uint32_t x, uint32_t) { return x ? q - x : 0u; });
  else if constexpr (OP == EW_MUL)
    o = map4(a, b, [=](uint32_t x, uint32_t y) { return mont_mul(x, y, q, nq); });
  else if constexpr (OP == EW_ADDC)
    o = map4(a, b, [=](uint32_t x, uint32_t) { return add_mod(x, k, q); });
  else if constexpr (OP == EW_SUBC)
    o = map4(a, b, [=](uint32_t x, uint32_t) { return sub_mod(x, k, q); });
  else if constexpr (OP == EW_RSUBC)
    o = map4(a, b, [=](uint32_t x, uint32_t) { return sub_mod(k, x, q); });
  else if constexpr (OP == EW_MULC)
    o = map4(a, b, [=](uint32_t x, uint32_t) { return mont_mul(x, k, q, nq); });
  else if constexpr (OP == EW_MULC_ADD)
    o = map4(a, b, [=](uint32_t x, uint32_t y) {
      return add_mod(mont_mul(x, k, q, nq), y, q);
    });
  else if constexpr (OP == EW_IMAG) {
    // multiply by X^(N/2): +u on the first half of the evaluation points,
    // -u on the second (u = psi^(N/2) in M-form)
    const uint32_t u = (4 * v < kN / 2) ? k : q - k;
    o = map4(a, b, [=](uint32_t x, uint32_t) { return mont_mul(x, u, q, nq); });
  } else
    o = a;
  reinterpret_cast<uint4 *>(r.dst)[v] = o;
}

__global__ void __launch_bounds__(kEwThreads)
    tensor_kernel(const __grid_constant__ TensorArgs args) {
  pdl_launch_dependents();
  pdl_wait();
  const TensorRow &r = args.rows[blockIdx.y];
  const int v = blockIdx.x * kEwThreads + threadIdx.x;
  const uint32_t q = r.q, nq = r.nqinv;
  const uint4 b1 = reinterpret_cast<const uint4 *>(r.b1)[v];
  const uint4 a1 = reinterpret_cast<const uint4 *>(r.a1)[v];
  const uint4 b2 = reinterpret_cast<const uint4 *>(r.b2)[v];
  const uint4 a2 = reinterpret_cast<const uint4 *>(r.a2)[v];
  const uint64_t q32 = (uint64_t)q << 32;
  auto cross = [=](uint32_t x1, uint32_t y1, uint32_t x2, uint32_t y2) {
    uint64_t acc = (uint64_t)x1 * y2;  // b1*a2 + a1*b2, one reduction
    mac_fold(acc, y1, x2, q32);
    return mont_reduce(acc, q, nq);
  };
  auto mm = [=](uint32_t x, uint32_t y) { return mont_mul(x, y, q, nq); };
  reinterpret_cast<uint4 *>(r.d0)[v] = map4(b1, b2, mm);
  reinterpret_cast<uint4 *>(r.d2)[v] = map4(a1, a2, mm);
  reinterpret_cast<uint4 *>(r.d1)[v] =
      make_uint4(cross(b1.x, a1.x, b2.x, a2.x), cross(b1.y, a1.y, b2.y, a2.y),
                 cross(b1.z, a1.z, b2.z, a2.z), cross(b1.w, a1.w, b2.w, a2.w));
}

// dst[i] = (add ? add[i] : 0) + src[pi(i)], pi the index map of the Galois
// automorphism on bit-reversed evaluation order. Aligned blocks of 2^k
// outputs read aligned blocks of 2^k inputs, so a warp's scattered 4-byte
// loads stay inside one 512-byte block.
__global__ void __launch_bounds__(kEwThreads)
    permute_kernel(const __grid_constant__ EwArgs args, uint32_t galois) {
  pdl_launch_dependents();
  pdl_wait();
  const EwRow &r = args.rows[blockIdx.y];
  const int v = blockIdx.x * kEwThreads + threadIdx.x;
  const uint32_t q = r.q;
  uint32_t o[4];
#pragma unroll
  for (int e = 0; e < 4; e++) {
    const uint32_t i = 4 * v + e;
    const uint32_t ex = (__brev(i) >> (31 - kLogN)) + 1;  // 2*brev16(i)+1
    const uint32_t s = __brev((ex * galois - 1) << (31 - kLogN));
    o[e] = r.a[s & (kN - 1)];
  }
  uint4 out = make_uint4(o[0], o[1], o[2], o[3]);
  if (r.b) {
    const uint4 b = reinterpret_cast<const uint4 *>(r.b)[v];
    out = map4(out, b, [=](uint32_t x, uint32_t y) { return add_mod(x, y, q); });
  }
  reinterpret_cast<uint4 *>(r.dst)[v] = out;
}

// Fused n-ary sums (see NaryArgs). One thread owns four consecutive words of
// one limb of every polynomial; each term costs one 128-bit load per
// polynomial (four gathered words in the permuting mode), products are
// accumulated in 64 bits with one Montgomery reduction per output word.
template <int MODE>
__global__ void __launch_bounds__(kEwThreads)
    nary_kernel(const __grid_constant__ NaryArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y, v = blockIdx.x * kEwThreads + threadIdx.x;
  const size_t off = (size_t)l * kN;
  const uint32_t q = a.q[l], nq = a.nqinv[l];
  const uint64_t q32 = (uint64_t)q << 32;
  uint32_t perm[4];
  for (int p = 0; p < a.n_polys; p++) {
    uint32_t out[4];
    if constexpr (MODE == NARY_CONST || MODE == NARY_PLAIN) {
      uint64_t acc[4] = {0, 0, 0, 0};
      for (int t = 0; t < a.n_terms; t++) {
        const uint4 x = reinterpret_cast<const uint4 *>(a.src[t][p] + off)[v];
        uint4 k;
        if constexpr (MODE == NARY_CONST) {
          const uint32_t c = a.c[t][l];
          k = make_uint4(c, c, c, c);
        } else {
          k = reinterpret_cast<const uint4 *>(a.pt[t] + off)[v];
        }
        mac_fold(acc[0], x.x, k.x, q32);
        mac_fold(acc[1], x.y, k.y, q32);
        mac_fold(acc[2], x.z, k.z, q32);
        mac_fold(acc[3], x.w, k.w, q32);
      }
#pragma unroll
      for (int e = 0; e < 4; e++) out[e] = mont_reduce(acc[e], q, nq);
    } else {
#pragma unroll
      for (int e = 0; e < 4; e++) out[e] = 0;
      for (int t = 0; t < a.n_terms; t++) {
        uint4 x;
        if constexpr (MODE == NARY_PERMUTE) {
          const uint32_t galois = a.galois[t];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const uint32_t i = 4 * v + e;
            const uint32_t ex = (__brev(i) >> (31 - kLogN)) + 1;
            perm[e] = __brev((ex * galois - 1) << (31 - kLogN)) & (kN - 1);
          }
          const uint32_t *s = a.src[t][p] + off;
          x = make_uint4(s[perm[0]], s[perm[1]], s[perm[2]], s[perm[3]]);
        } else {
          x = reinterpret_cast<const uint4 *>(a.src[t][p] + off)[v];
        }
        out[0] = add_mod(out[0], x.x, q);
        out[1] = add_mod(out[1], x.y, q);
        out[2] = add_mod(out[2], x.z, q);
        out[3] = add_mod(out[3], x.w, q);
      }
    }
    uint4 o = make_uint4(out[0], out[1], out[2], out[3]);
    if (a.add[p]) {
      const uint4 b = reinterpret_cast<const uint4 *>(a.add[p] + off)[v];
      o = map4(o, b, [=](uint32_t x, uint32_t y) { return add_mod(x, y, q); });
    }
    reinterpret_cast<uint4 *>(a.dst[p] + off)[v] = o;
  }
}

// Sum of tensor products, each of the three outputs accumulated in 64 bits
// (folded below q * 2^32 after every product) with one Montgomery reduction
// per output word: the inner sums of an encrypted matrix product, where the
// reference would run Tensor (src/core/ElementWise.cu:504-546) and Add once per
// term. With `accumulate` the previous contents of the outputs are added.
__global__ void __launch_bounds__(kEwThreads)
    tensor_accum_kernel(const __grid_constant__ TensorAccArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y, v = blockIdx.x * kEwThreads + threadIdx.x;
  const size_t off = (size_t)l * (kN / 4) + v;
  const uint32_t q = a.q[l], nq = a.nqinv[l];
  const uint64_t q32 = (uint64_t)q << 32;
  uint64_t s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0}, s2[4] = {0, 0, 0, 0};
  for (int t = 0; t < a.n_terms; t++) {
    const uint4 b1 = reinterpret_cast<const uint4 *>(a.b1[t])[off];
    const uint4 a1 = reinterpret_cast<const uint4 *>(a.a1[t])[off];
    const uint4 b2 = reinterpret_cast<const uint4 *>(a.b2[t])[off];
    const uint4 a2 = reinterpret_cast<const uint4 *>(a.a2[t])[off];
    const uint32_t xb1[4] = {b1.x, b1.y, b1.z, b1.w}, xa1[4] = {a1.x, a1.y, a1.z, a1.w};
    const uint32_t xb2[4] = {b2.x, b2.y, b2.z, b2.w}, xa2[4] = {a2.x, a2.y, a2.z, a2.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
      mac_fold(s0[e], xb1[e], xb2[e], q32);
      mac_fold(s1[e], xb1[e], xa2[e], q32);
      mac_fold(s1[e], xa1[e], xb2[e], q32);
      mac_fold(s2[e], xa1[e], xa2[e], q32);
    }
  }
  uint64_t *const sums[3] = {s0, s1, s2};
#pragma unroll
  for (int p = 0; p < 3; p++) {
    uint4 o = make_uint4(mont_reduce(sums[p][0], q, nq), mont_reduce(sums[p][1], q, nq),
                         mont_reduce(sums[p][2], q, nq), mont_reduce(sums[p][3], q, nq));
    uint4 *dst = reinterpret_cast<uint4 *>(a.d[p]) + off;
    if (a.accumulate) {
      const uint4 old = *dst;
      o = map4(o, old, [=](uint32_t x, uint32_t y) { return add_mod(x, y, q); });
    }
    *dst = o;
  }
}

// Key-switch inner product: for every limb l of the extended basis
//   acc_b[l] = sum_i x_i[l] * kb_i[l] (+ P * c0[l] on Q limbs), same for a.
// x_i[l] is the digit's own limb read in place from `d` when limb l belongs
// to digit i, else the ModUp output. One Montgomery reduction per output.
__global__ void __launch_bounds__(kEwThreads)
    inner_kernel(const __grid_constant__ InnerArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y;
  const int v = blockIdx.x * kEwThreads + threadIdx.x;
  const uint32_t q = a.q[l], nq = a.nqinv[l];
  const uint64_t q32 = (uint64_t)q << 32;
  uint64_t sb[4] = {0, 0, 0, 0}, sa[4] = {0, 0, 0, 0};
  const size_t koff = (size_t)a.kpos[l] * kN;
#pragma unroll 1
  for (int i = 0; i < a.n_digits; i++) {
    const uint32_t *xp = (a.own_digit[l] == i && a.d)
                             ? a.d + (size_t)l * kN
                             : a.mu + ((size_t)a.mu_slot[i] * a.ntot + l) * kN;
    const uint4 x = reinterpret_cast<const uint4 *>(xp)[v];
    const uint4 kb = __ldcs(reinterpret_cast<const uint4 *>(a.kb[i] + koff) + v);
    const uint4 ka = __ldcs(reinterpret_cast<const uint4 *>(a.ka[i] + koff) + v);
    mac_fold(sb[0], x.x, kb.x, q32);
    mac_fold(sb[1], x.y, kb.y, q32);
    mac_fold(sb[2], x.z, kb.z, q32);
    mac_fold(sb[3], x.w, kb.w, q32);
    mac_fold(sa[0], x.x, ka.x, q32);
    mac_fold(sa[1], x.y, ka.y, q32);
    mac_fold(sa[2], x.z, ka.z, q32);
    mac_fold(sa[3], x.w, ka.w, q32);
  }
  if (l < a.nq) {
    const uint32_t pm = a.pm[l];
    if (a.c0) {
      const uint4 c = reinterpret_cast<const uint4 *>(a.c0 + (size_t)l * kN)[v];
      mac_fold(sb[0], c.x, pm, q32);
      mac_fold(sb[1], c.y, pm, q32);
      mac_fold(sb[2], c.z, pm, q32);
      mac_fold(sb[3], c.w, pm, q32);
    }
    if (a.c1) {
      const uint4 c = reinterpret_cast<const uint4 *>(a.c1 + (size_t)l * kN)[v];
      mac_fold(sa[0], c.x, pm, q32);
      mac_fold(sa[1], c.y, pm, q32);
      mac_fold(sa[2], c.z, pm, q32);
      mac_fold(sa[3], c.w, pm, q32);
    }
  }
  if (a.scatter_galois == 0) {
    uint4 rb = make_uint4(mont_reduce(sb[0], q, nq), mont_reduce(sb[1], q, nq),
                          mont_reduce(sb[2], q, nq), mont_reduce(sb[3], q, nq));
    uint4 ra = make_uint4(mont_reduce(sa[0], q, nq), mont_reduce(sa[1], q, nq),
                          mont_reduce(sa[2], q, nq), mont_reduce(sa[3], q, nq));
    uint4 *pb = reinterpret_cast<uint4 *>(a.acc_b + (size_t)l * kN) + v;
    uint4 *pa = reinterpret_cast<uint4 *>(a.acc_a + (size_t)l * kN) + v;
    if (a.accumulate) {
      const uint4 ob = *pb, oa = *pa;
      rb = make_uint4(add_mod(rb.x, ob.x, q), add_mod(rb.y, ob.y, q), add_mod(rb.z, ob.z, q),
                      add_mod(rb.w, ob.w, q));
      ra = make_uint4(add_mod(ra.x, oa.x, q), add_mod(ra.y, oa.y, q), add_mod(ra.z, oa.z, q),
                      add_mod(ra.w, oa.w, q));
    }
    *pb = rb;
    *pa = ra;
  } else {
    // fused automorphism: the key and the ModUp buffers are read in order and
    // the product lands where the rotation sends it (the reference's fused
    // baby-step kernel does the same, src/extension/Hoist.cu:20-78); an
    // aligned block of 128 results stays inside one aligned block of 128
    uint32_t *ob = a.acc_b + (size_t)l * kN, *oa = a.acc_a + (size_t)l * kN;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const uint32_t i = 4 * v + e;
      const uint32_t ex = (__brev(i) >> (31 - kLogN)) + 1;
      const uint32_t d = __brev((ex * a.scatter_galois - 1) << (31 - kLogN)) & (kN - 1);
      uint32_t rb = mont_reduce(sb[e], q, nq), ra = mont_reduce(sa[e], q, nq);
      if (a.accumulate) {  // every destination word belongs to exactly one thread
        rb = add_mod(rb, ob[d], q);
        ra = add_mod(ra, oa[d], q);
      }
      ob[d] = rb;
      oa[d] = ra;
    }
  }
}

// acc_j = sum_i pt[j][i] (*) rot_i on one limb, one coefficient per thread.
// The rotations are held in registers across the giant steps, so every
// plaintext word and every rotation word is read once (the reference's
// GSFusedPAccum kernel keeps the same operands in registers,
// src/extension/Hoist.cu:80-120). Products are summed in 64 bits, folded below
// q*2^32 after every second one (2 q^2 <= q*2^32 for q < 2^31), with one
// Montgomery reduction per output. About 100 registers per thread keep two
// blocks of 256 threads on an SM.
constexpr int kPtThreads = 256;
__global__ void __launch_bounds__(kPtThreads, 2)
    pt_accum_kernel(const __grid_constant__ PtAccumArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y;
  const int v = blockIdx.x * kPtThreads + threadIdx.x;
  const uint32_t q = a.q[l], nq = a.nqinv[l];
  const uint64_t q32 = (uint64_t)q << 32;
  const size_t limb = (size_t)l * kN + v, poly = (size_t)a.ntot * kN;
  uint32_t rb[kMaxBaby], ra[kMaxBaby];
#pragma unroll
  for (int i = 0; i < kMaxBaby; i++)
    if (i < a.n_baby) {
      rb[i] = a.rot[(size_t)(2 * i) * poly + limb];
      ra[i] = a.rot[(size_t)(2 * i + 1) * poly + limb];
    }
#pragma unroll 1
  for (int j = 0; j < a.n_giant; j++) {
    uint32_t w[kMaxBaby];
#pragma unroll
    for (int i = 0; i < kMaxBaby; i++) {
      const uint32_t *p = i < a.n_baby ? a.pt[j * kMaxBaby + i] : nullptr;
      w[i] = p ? __ldcs(p + limb) : 0u;
    }
    uint64_t sb = 0, sa = 0;
#pragma unroll
    for (int i = 0; i < kMaxBaby; i += 2) {
      sb += (uint64_t)rb[i] * w[i] + (uint64_t)rb[i + 1] * w[i + 1];
      sa += (uint64_t)ra[i] * w[i] + (uint64_t)ra[i + 1] * w[i + 1];
      if (sb >= q32) sb -= q32;
      if (sa >= q32) sa -= q32;
    }
    a.acc[(size_t)(2 * j) * poly + limb] = mont_reduce(sb, q, nq);
    a.acc[(size_t)(2 * j + 1) * poly + limb] = mont_reduce(sa, q, nq);
  }
}

// Exact lift of a value known modulo q0*q1 (two limbs, already multiplied by
// the inverse of the other prime) to other primes: x = centred(y0*q1 + y1*q0
// mod q0*q1), out = x mod p (reference kernel ModUpToMax2,
// src/core/ElementWise.cu:593-623; one-limb case :579-591).
__global__ void __launch_bounds__(kEwThreads)
    lift_kernel(const __grid_constant__ EwArgs args, const uint32_t *src, uint32_t q0, uint32_t q1) {
  pdl_launch_dependents();
  pdl_wait();
  const EwRow &r = args.rows[blockIdx.y];
  const int i = blockIdx.x * kEwThreads + threadIdx.x;  // one word per thread
  const uint32_t p = r.q;
  if (q1 == 0) {
    r.dst[i] = src[i] % p;
    return;
  }
  const int64_t prod = (int64_t)((uint64_t)q0 * q1);
  int64_t v = (int64_t)((uint64_t)src[i] * q1 + (uint64_t)src[i + kN] * q0);
  if (v >= prod) v -= prod;
  if (v > (prod >> 1)) v -= prod;
  int64_t m = v % (int64_t)p;
  if (m < 0) m += p;
  r.dst[i] = (uint32_t)m;
}

}  // namespace

int launch_lift(const Context &ctx, const EwArgs &args, const uint32_t *src, uint32_t q0, uint32_t q1) {
  if (args.n_rows <= 0) return 0;
  dim3 grid(kN / kEwThreads, args.n_rows), block(kEwThreads);
  CFHE_CUDA(launch_kernel(ctx.use_pdl, lift_kernel, grid, block, 0, ctx.stream, args, src, q0, q1));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_ew(const Context &ctx, int op, const EwArgs &args) {
  if (args.n_rows <= 0) return 0;
  dim3 grid(kEwBlocksX, args.n_rows), block(kEwThreads);
  switch (op) {
#define CASE(OP)                                            \
  case OP:                                                  \
    CFHE_CUDA(launch_kernel(ctx.use_pdl, ew_kernel<OP>, grid, block, 0, ctx.stream, args)); \
    break;
    CASE(EW_ADD)
    CASE(EW_SUB)
    CASE(EW_NEG)
    CASE(EW_MUL)
    CASE(EW_ADDC)
    CASE(EW_SUBC)
    CASE(EW_RSUBC)
    CASE(EW_MULC)
    CASE(EW_MULC_ADD)
    CASE(EW_IMAG)
    CASE(EW_COPY)
#undef CASE
    default:
      set_error("unknown element-wise op");
      return -1;
  }
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_tensor(const Context &ctx, const TensorArgs &args) {
  if (args.n_rows <= 0) return 0;
  dim3 grid(kEwBlocksX, args.n_rows), block(kEwThreads);
  CFHE_CUDA(launch_kernel(ctx.use_pdl, tensor_kernel, grid, block, 0, ctx.stream, args));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_permute(const Context &ctx, const EwArgs &args, uint32_t galois) {
  if (args.n_rows <= 0) return 0;
  dim3 grid(kEwBlocksX, args.n_rows), block(kEwThreads);
  CFHE_CUDA(launch_kernel(ctx.use_pdl, permute_kernel, grid, block, 0, ctx.stream, args, galois));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_nary(const Context &ctx, const NaryArgs &args) {
  if (args.n_limbs <= 0 || args.n_polys <= 0) return 0;
  dim3 grid(kEwBlocksX, args.n_limbs), block(kEwThreads);
  switch (args.mode) {
    case NARY_SUM:
      CFHE_CUDA(launch_kernel(ctx.use_pdl, nary_kernel<NARY_SUM>, grid, block, 0, ctx.stream, args));
      break;
    case NARY_CONST:
      CFHE_CUDA(launch_kernel(ctx.use_pdl, nary_kernel<NARY_CONST>, grid, block, 0, ctx.stream, args));
      break;
    case NARY_PLAIN:
      CFHE_CUDA(launch_kernel(ctx.use_pdl, nary_kernel<NARY_PLAIN>, grid, block, 0, ctx.stream, args));
      break;
    case NARY_PERMUTE:
      CFHE_CUDA(launch_kernel(ctx.use_pdl, nary_kernel<NARY_PERMUTE>, grid, block, 0, ctx.stream, args));
      break;
    default:
      set_error("unknown n-ary mode");
      return -1;
  }
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_tensor_accum(const Context &ctx, const TensorAccArgs &args) {
  if (args.n_limbs <= 0) return 0;
  dim3 grid(kEwBlocksX, args.n_limbs), block(kEwThreads);
  CFHE_CUDA(launch_kernel(ctx.use_pdl, tensor_accum_kernel, grid, block, 0, ctx.stream, args));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_pt_accum(const Context &ctx, const PtAccumArgs &args) {
  dim3 grid(kN / kPtThreads, args.ntot), block(kPtThreads);
  CFHE_CUDA(launch_kernel(ctx.use_pdl, pt_accum_kernel, grid, block, 0, ctx.stream, args));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_inner(const Context &ctx, const InnerArgs &args) {
  dim3 grid(kEwBlocksX, args.ntot), block(kEwThreads);
  CFHE_CUDA(launch_kernel(ctx.use_pdl, inner_kernel, grid, block, 0, ctx.stream, args));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
