// Client-side sampling and encryption kernels.
//
// The reference samples on the host and uploads (src/UserInterface.cu:223-276,
// 366-458: uniform ring elements for the `a` part of ciphertexts and key
// digits, rounded Gaussian errors) and combines the samples with three small
// kernels (Encrypt, EncryptZero, AddEvkPart, src/UserInterface.cu:17-108). A
// rotation key at N = 2^16 is 118 MiB of uniform words, bootstrapping needs
// eighty of them: here the words are generated where they are used.
//
// Generator: Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy
// as 1, 2, 3", SC'11), a counter-based generator: word i of limb l of draw
// (seed, stream) is a pure function of those numbers, so the output does not
// depend on the launch geometry and can be reproduced on the host (the tests
// do). Uniform residues use the multiply-and-reject map, which is exactly
// uniform; errors use a cumulative table of the rounded normal distribution
// built on the host in double precision, so the device does no floating point
// and the samples are reproducible bit for bit.
#include <math.h>

#include "context.h"
#include "kernels.h"
#include "modmath.cuh"

namespace cfhe {
namespace {

constexpr int kSampleThreads = 256;

struct Philox {
  uint32_t c[4];
};

// ten rounds of Philox-4x32 on counter c with key (k0, k1)
__host__ __device__ inline Philox philox4x32(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                             uint32_t k1) {
  Philox r{{c0, c1, c2, c3}};
#pragma unroll
  for (int round = 0; round < 10; round++) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * r.c[0], p1 = (uint64_t)0xCD9E8D57u * r.c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ r.c[1] ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ r.c[3] ^ k1, n3 = (uint32_t)p0;
    r.c[0] = n0;
    r.c[1] = n1;
    r.c[2] = n2;
    r.c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return r;
}

constexpr int kMaxRedraws = 16;

// Four uniform residues below q for words 4v .. 4v+3 of limb l. Lane e of
// draw d is accepted when the low half of r * q is at least 2^32 mod q; a
// rejected lane is redrawn with d + 1 (at most kMaxRedraws times, after which
// the last draw is taken: probability below 2^-16 even for the smallest prime).
__host__ __device__ inline void uniform4(uint32_t *out, uint32_t v, uint32_t l, uint32_t stream, uint64_t seed,
                                         uint32_t q) {
  const uint32_t reject_below = (0u - q) % q;
  bool done[4] = {false, false, false, false};
  for (int d = 0; d < kMaxRedraws; d++) {
    const Philox r = philox4x32(v, l, (uint32_t)d, stream, (uint32_t)seed, (uint32_t)(seed >> 32));
    bool all = true;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      if (done[e]) continue;
      const uint64_t m = (uint64_t)r.c[e] * q;
      out[e] = (uint32_t)(m >> 32);
      done[e] = (uint32_t)m >= reject_below || d == kMaxRedraws - 1;
      all = all && done[e];
    }
    if (all) break;
  }
}

struct SampleArgs {
  uint32_t *dst;
  int n_limbs;
  uint64_t seed;
  uint32_t stream;
  uint32_t q[kMaxLimbs];
  uint8_t g[kMaxLimbs];  // global prime index: the limb coordinate of the counter
};

__global__ void __launch_bounds__(kSampleThreads) sample_uniform_kernel(const __grid_constant__ SampleArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y, v = blockIdx.x * kSampleThreads + threadIdx.x;
  uint32_t w[4];
  uniform4(w, (uint32_t)v, a.g[l], a.stream, a.seed, a.q[l]);
  reinterpret_cast<uint4 *>(a.dst + (size_t)l * kN)[v] = make_uint4(w[0], w[1], w[2], w[3]);
}

// Rounded normal samples: cdf[k] = floor(2^64 * P(X <= k - kErrTail)), X =
// round(N(0, sigma^2)); the sample is the first k with u < cdf[k], u 64 random
// bits. One value per coefficient, written mod every prime of the list.
constexpr int kErrTail = 48;
constexpr int kErrTable = 2 * kErrTail + 1;
struct ErrorArgs {
  SampleArgs s;
  uint64_t cdf[kErrTable];
};

__host__ __device__ inline int error_from_bits(uint64_t u, const uint64_t *cdf) {
  int lo = 0, hi = kErrTable - 1;  // first index with u < cdf[index]; cdf[last] = 2^64 - 1
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (u < cdf[mid])
      hi = mid;
    else
      lo = mid + 1;
  }
  return lo - kErrTail;
}

__global__ void __launch_bounds__(kSampleThreads) sample_error_kernel(const __grid_constant__ ErrorArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int v = blockIdx.x * kSampleThreads + threadIdx.x;  // coefficients 2v, 2v + 1
  const Philox r = philox4x32((uint32_t)v, 0xE0E0E0E0u, 0u, a.s.stream, (uint32_t)a.s.seed,
                              (uint32_t)(a.s.seed >> 32));
  const int e0 = error_from_bits(((uint64_t)r.c[1] << 32) | r.c[0], a.cdf);
  const int e1 = error_from_bits(((uint64_t)r.c[3] << 32) | r.c[2], a.cdf);
  for (int l = 0; l < a.s.n_limbs; l++) {
    const uint32_t q = a.s.q[l];
    const uint32_t w0 = e0 < 0 ? q - (uint32_t)(-e0) : (uint32_t)e0;
    const uint32_t w1 = e1 < 0 ? q - (uint32_t)(-e1) : (uint32_t)e1;
    reinterpret_cast<uint2 *>(a.s.dst + (size_t)l * kN)[v] = make_uint2(w0, w1);
  }
}

// b = m + e - a * s (reference Encrypt, src/UserInterface.cu:17-53; without m:
// EncryptZero, :55-80), all operands in the NTT domain, a * s a Montgomery
// product (s in M-form).
struct EncArgs {
  uint32_t *b;
  const uint32_t *a, *s, *e, *m;  // m may be null
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs];
};

__global__ void __launch_bounds__(kSampleThreads) encrypt_kernel(const __grid_constant__ EncArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y, v = blockIdx.x * kSampleThreads + threadIdx.x;
  const size_t off = (size_t)l * (kN / 4) + v;
  const uint32_t q = a.q[l], nq = a.nqinv[l];
  const uint4 x = reinterpret_cast<const uint4 *>(a.a)[off], s = reinterpret_cast<const uint4 *>(a.s)[off];
  const uint4 e = reinterpret_cast<const uint4 *>(a.e)[off];
  auto f = [=](uint32_t xa, uint32_t xs, uint32_t xe) { return sub_mod(xe, mont_mul(xa, xs, q, nq), q); };
  uint4 r = make_uint4(f(x.x, s.x, e.x), f(x.y, s.y, e.y), f(x.z, s.z, e.z), f(x.w, s.w, e.w));
  if (a.m) {
    const uint4 m = reinterpret_cast<const uint4 *>(a.m)[off];
    r = make_uint4(add_mod(r.x, m.x, q), add_mod(r.y, m.y, q), add_mod(r.z, m.z, q), add_mod(r.w, m.w, q));
  }
  reinterpret_cast<uint4 *>(a.b)[off] = r;
}

// Encoding, device half: residues of trunc(v[i]) modulo every listed prime, v
// the plaintext polynomial's coefficients times the scale as doubles
// (reference Encoder::Encode, src/core/Encode.cpp:136-248, converts each
// coefficient to a big integer and reduces it prime by prime on the host). A
// double of magnitude below 2^63 converts exactly to a 64-bit integer; a
// larger one is m * 2^e with a 53-bit integer m and e > 0, so its residue is
// (m mod q) * (2^e mod q): no big integers either way.
struct SplitArgs {
  uint32_t *dst;
  const double *v;
  uint32_t q[kMaxLimbs];
};

__global__ void __launch_bounds__(kSampleThreads) rns_split_kernel(const __grid_constant__ SplitArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int l = blockIdx.y, i = blockIdx.x * kSampleThreads + threadIdx.x;
  const uint32_t q = a.q[l];
  const double v = a.v[i];
  const double mag = fabs(v);
  uint32_t r;
  if (mag < 9223372036854775808.0) {  // 2^63
    r = (uint32_t)((unsigned long long)mag % q);  // conversion truncates toward zero
  } else {
    int e;
    const double f = frexp(mag, &e);                              // mag = f * 2^e, f in [0.5, 1)
    const unsigned long long m = (unsigned long long)ldexp(f, 53);  // exact 53-bit integer
    int shift = e - 53;                                           // > 0 here
    uint32_t p2 = 1u % q, base = 2u % q;
    while (shift > 0) {  // 2^shift mod q by square and multiply
      if (shift & 1) p2 = (uint32_t)((uint64_t)p2 * base % q);
      base = (uint32_t)((uint64_t)base * base % q);
      shift >>= 1;
    }
    r = (uint32_t)((m % q) * p2 % q);
  }
  if (v < 0.0 && r != 0) r = q - r;
  a.dst[(size_t)l * kN + i] = r;
}

// Decoding, device half: the centred integer behind the residues of one
// coefficient (reference Encoder::Decode, src/core/Encode.cpp:250-275, lifts
// with big integers on the host). With r_j = x * (Q/q_j)^-1 mod q_j the
// integer is x = sum_j r_j (Q/q_j) - k Q, k = round(sum_j r_j / q_j): the sum
// of fractions is within 2^-40 of an integer for any decodable value (|x| is
// far below Q), so doubles find k; x itself is then computed modulo 2^128,
// exactly, because |x| < 2^127.
struct LiftArgs {
  double *out;
  const uint32_t *res;  // [n_limbs][N]
  int n_limbs;
  uint32_t q[kMaxLimbs];
  uint32_t hat[kMaxLimbs][4];  // (Q / q_j) mod 2^128, little endian words
  uint32_t q_low[4];           // Q mod 2^128
};

__global__ void __launch_bounds__(kSampleThreads) crt_lift_kernel(const __grid_constant__ LiftArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * kSampleThreads + threadIdx.x;
  unsigned __int128 acc = 0;
  double frac = 0.0;
  for (int j = 0; j < a.n_limbs; j++) {
    const uint32_t r = a.res[(size_t)j * kN + i];
    const unsigned __int128 h = ((unsigned __int128)(((uint64_t)a.hat[j][3] << 32) | a.hat[j][2]) << 64) |
                                (((uint64_t)a.hat[j][1] << 32) | a.hat[j][0]);
    acc += h * r;
    frac += (double)r / (double)a.q[j];
  }
  const unsigned __int128 ql = ((unsigned __int128)(((uint64_t)a.q_low[3] << 32) | a.q_low[2]) << 64) |
                               (((uint64_t)a.q_low[1] << 32) | a.q_low[0]);
  const long long k = llrint(frac);
  acc -= ql * (unsigned __int128)(unsigned long long)k;
  // to double through the magnitude (a negative value written as hi * 2^64 + lo
  // with hi = -1 would cancel two numbers near 2^64)
  const __int128 x = (__int128)acc;
  const bool negative = x < 0;
  const unsigned __int128 mag = negative ? (unsigned __int128)(-x) : (unsigned __int128)x;
  const double v = (double)(unsigned long long)(mag >> 64) * 18446744073709551616.0 +
                   (double)(unsigned long long)mag;
  a.out[i] = negative ? -v : v;
}

int fill_sample(const Context &c, SampleArgs &s, uint32_t *dst, const int *gidx, int n_limbs, uint64_t seed,
                uint32_t stream) {
  if (!dst || !gidx) {
    set_error("null argument");
    return -1;
  }
  if (n_limbs < 1 || n_limbs > kMaxLimbs) {
    set_error("too many limbs");
    return -1;
  }
  s.dst = dst;
  s.n_limbs = n_limbs;
  s.seed = seed;
  s.stream = stream;
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) {
      set_error("prime index out of range");
      return -1;
    }
    s.q[l] = c.q[gidx[l]];
    s.g[l] = (uint8_t)gidx[l];
  }
  return 0;
}

}  // namespace

void error_cdf_table(double sigma, uint64_t *cdf) {
  // P(X <= k) for X = round(N(0, sigma^2)) is Phi((k + 1/2) / sigma)
  for (int i = 0; i < kErrTable; i++) {
    const double k = (double)(i - kErrTail) + 0.5;
    const long double p = 0.5L * erfcl(-(long double)k / ((long double)sigma * sqrtl(2.0L)));
    const long double scaled = p * 18446744073709551616.0L;  // 2^64
    cdf[i] = scaled >= 18446744073709551615.0L ? UINT64_MAX : (uint64_t)scaled;
  }
  cdf[kErrTable - 1] = UINT64_MAX;
}

int launch_sample_uniform(const Context &c, uint32_t *dst, const int *gidx, int n_limbs, uint64_t seed,
                          uint32_t stream) {
  SampleArgs s;
  if (int r = fill_sample(c, s, dst, gidx, n_limbs, seed, stream)) return r;
  CFHE_CUDA(launch_kernel(c.use_pdl, sample_uniform_kernel, dim3(kN / 4 / kSampleThreads, n_limbs),
                          dim3(kSampleThreads), 0, c.stream, s));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_sample_error(const Context &c, uint32_t *dst, const int *gidx, int n_limbs, double sigma,
                        uint64_t seed, uint32_t stream) {
  if (!(sigma > 0.0) || sigma > 8.0) {
    set_error("error sampling: standard deviation must be in (0, 8]");
    return -1;
  }
  ErrorArgs e;
  if (int r = fill_sample(c, e.s, dst, gidx, n_limbs, seed, stream)) return r;
  error_cdf_table(sigma, e.cdf);
  CFHE_CUDA(launch_kernel(c.use_pdl, sample_error_kernel, dim3(kN / 2 / kSampleThreads), dim3(kSampleThreads), 0,
                          c.stream, e));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_rns_split(const Context &c, uint32_t *dst, const double *v, const int *gidx, int n_limbs) {
  if (!dst || !v || !gidx) {
    set_error("null argument");
    return -1;
  }
  if (n_limbs < 1 || n_limbs > kMaxLimbs) {
    set_error("too many limbs");
    return -1;
  }
  SplitArgs x;
  x.dst = dst;
  x.v = v;
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) {
      set_error("prime index out of range");
      return -1;
    }
    x.q[l] = c.q[gidx[l]];
  }
  CFHE_CUDA(launch_kernel(c.use_pdl, rns_split_kernel, dim3(kN / kSampleThreads, n_limbs), dim3(kSampleThreads), 0,
                          c.stream, x));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_crt_lift(const Context &c, double *out, const uint32_t *res, const int *gidx, int n_limbs,
                    const uint32_t *hat, const uint32_t *q_low) {
  if (!out || !res || !gidx || !hat || !q_low) {
    set_error("null argument");
    return -1;
  }
  if (n_limbs < 1 || n_limbs > kMaxLimbs) {
    set_error("too many limbs");
    return -1;
  }
  LiftArgs x;
  x.out = out;
  x.res = res;
  x.n_limbs = n_limbs;
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) {
      set_error("prime index out of range");
      return -1;
    }
    x.q[l] = c.q[gidx[l]];
    for (int w = 0; w < 4; w++) x.hat[l][w] = hat[4 * l + w];
  }
  for (int w = 0; w < 4; w++) x.q_low[w] = q_low[w];
  CFHE_CUDA(launch_kernel(c.use_pdl, crt_lift_kernel, dim3(kN / kSampleThreads), dim3(kSampleThreads), 0, c.stream, x));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

int launch_encrypt(const Context &c, uint32_t *b, const uint32_t *a, const uint32_t *s, const uint32_t *e,
                   const uint32_t *m, const int *gidx, int n_limbs) {
  if (!b || !a || !s || !e || !gidx) {
    set_error("null argument");
    return -1;
  }
  if (n_limbs < 1 || n_limbs > kMaxLimbs) {
    set_error("too many limbs");
    return -1;
  }
  EncArgs x;
  x.b = b;
  x.a = a;
  x.s = s;
  x.e = e;
  x.m = m;
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) {
      set_error("prime index out of range");
      return -1;
    }
    x.q[l] = c.q[gidx[l]];
    x.nqinv[l] = c.nqinv[gidx[l]];
  }
  CFHE_CUDA(launch_kernel(c.use_pdl, encrypt_kernel, dim3(kN / 4 / kSampleThreads, n_limbs), dim3(kSampleThreads),
                          0, c.stream, x));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
