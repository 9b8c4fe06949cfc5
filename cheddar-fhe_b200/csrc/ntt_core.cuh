// Negacyclic NTT / INTT for N = 2^16: the arithmetic (Shoup twiddles, lazy
// butterflies, radix-16 register phases) shared by the two-pass kernels
// (ntt_twopass.cu, the default) and the single-launch cluster kernels (ntt.cu),
// and the per-thread phase functions of the latter, written so that the same
// index and arithmetic code also runs inside a host emulation used by the CPU
// tests. The decomposition described next is the cluster kernels'.
//
// Decomposition: a limb is a 256 x 256 matrix (row-major, row = index >> 8).
// A thread-block cluster of 8 CTAs owns one limb of one polynomial.
//   forward  (Cooley-Tukey, natural in, bit-reversed out):
//     F1/F2  CTA c holds columns [32c, 32c+32) of every row and runs the 8
//            stages whose butterflies pair rows (strides 128..1 rows);
//     F2     then scatters its results through distributed shared memory so
//            that CTA c' holds rows [32c', 32c'+32) complete;
//     F3/F4  the 8 stages inside rows (strides 128..1 words), final fold to
//            [0,q), 128-bit stores.
//   inverse  (Gentleman-Sande, bit-reversed in, natural out) is the mirror
//            image: I1/I2 inside rows, exchange, I3/I4 across rows, then the
//            per-limb constant (1/N and whatever the caller folded in).
// Each phase is four radix-2 stages on 16 register-resident values.
//
// Arithmetic: twiddles are stored as plain residues w together with
// ws = floor(w * 2^32 / q) (Shoup); a product costs one high and two low
// 32-bit multiplies and lands in [0, 2q). Limbs whose prime is below 2^30 use
// the lazy [0,4q) butterfly (FAST); larger primes (the auxiliary primes reach
// 2^31) keep every value in [0,2q) and fold the butterfly's inputs to [0,q).
// Results are folded to the canonical [0,q) range, so they are bit-identical
// to any other correct evaluation of the same transform.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define CFHE_HD __host__ __device__ __forceinline__
#else
#define CFHE_HD inline
#endif

namespace cfhe {

struct alignas(8) Tw {
  uint32_t w;   // residue
  uint32_t ws;  // floor(w * 2^32 / q)
};

constexpr int kLogN = 16;
constexpr int kN = 1 << kLogN;
constexpr int kClusterSize = 8;
constexpr int kNttThreads = 512;
constexpr int kRowWords = 256;
constexpr int kStripCols = 32;  // columns per CTA in the row-pairing phases
constexpr int kOwnRows = 32;    // rows per CTA in the in-row phases
// In-row buffers pad 4 words after every 16 and 16 more per row so that both
// the strided (x0 + 16k) and the contiguous (16g + k) access patterns of a
// warp touch 32 distinct banks.
constexpr int kRowStride = 336;
constexpr int kRowBufWords = kOwnRows * kRowStride;    // in-row layout: 43008 B
constexpr int kStripBufWords = kRowWords * kStripCols;  // strip layout: 32768 B
// One strip-layout and one in-row-layout buffer per CTA (75 776 B), so three
// CTAs fit in the 228 KB of one SM.
constexpr int kNttSmemBytes = (kRowBufWords + kStripBufWords) * 4;

CFHE_HD uint32_t umulhi32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return (uint32_t)(((uint64_t)a * b) >> 32);
#endif
}

CFHE_HD uint32_t umin32(uint32_t a, uint32_t b) { return a < b ? a : b; }

// a * w mod q in [0, 2q) for any 32-bit a, w < q < 2^31.
CFHE_HD uint32_t shoup_mul(uint32_t a, Tw t, uint32_t q) {
  return a * t.w - umulhi32(a, t.ws) * q;
}

CFHE_HD Tw ld_tw(const Tw *p) {
#if defined(__CUDA_ARCH__)
  uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
  return Tw{v.x, v.y};
#else
  return *p;
#endif
}

template <int CNT>
CFHE_HD void ld_tws(const Tw *p, Tw *out) {
  if constexpr (CNT == 1) {
    out[0] = ld_tw(p);
  } else {
#if defined(__CUDA_ARCH__)
#pragma unroll
    for (int i = 0; i < CNT / 2; i++) {
      uint4 v = __ldg(reinterpret_cast<const uint4 *>(p) + i);
      out[2 * i] = Tw{v.x, v.y};
      out[2 * i + 1] = Tw{v.z, v.w};
    }
#else
    for (int i = 0; i < CNT; i++) out[i] = p[i];
#endif
  }
}

// (X, Y) <- (X + w Y, X - w Y). FAST: in/out [0,4q); else in/out [0,2q) with
// X and the product folded to [0,q) first, so no sum leaves 32 bits.
template <bool FAST>
CFHE_HD void ct_bfly(uint32_t &X, uint32_t &Y, Tw t, uint32_t q, uint32_t q2) {
  if constexpr (FAST) {
    uint32_t x = umin32(X, X - q2);
    uint32_t p = shoup_mul(Y, t, q);
    X = x + p;
    Y = x - p + q2;
  } else {
    uint32_t x = umin32(X, X - q);
    uint32_t p = shoup_mul(Y, t, q);
    p = umin32(p, p - q);
    X = x + p;
    Y = x - p + q;
  }
}

// Canonical [0,q) from the range the forward butterflies leave.
template <bool FAST>
CFHE_HD uint32_t ct_fold(uint32_t u, uint32_t q, uint32_t q2) {
  if constexpr (FAST) u = umin32(u, u - q2);
  return umin32(u, u - q);
}

// (X, Y) <- (X + Y, (X - Y) w), everything in [0,2q).
template <bool FAST>
CFHE_HD void gs_bfly(uint32_t &X, uint32_t &Y, Tw t, uint32_t q, uint32_t q2) {
  if constexpr (FAST) {
    uint32_t s = X + Y;
    uint32_t d = X - Y + q2;
    X = umin32(s, s - q2);
    Y = shoup_mul(d, t, q);
  } else {
    uint32_t x = umin32(X, X - q);
    uint32_t y = umin32(Y, Y - q);
    X = x + y;
    Y = shoup_mul(x - y + q, t, q);
  }
}

// Four Cooley-Tukey stages on 16 values; stage s (0..3) pairs k with
// k + (8 >> s) and takes twiddle tw[(i0 << s) + j] for its j-th block.
template <bool FAST>
CFHE_HD void ct_radix16(uint32_t *v, const Tw *tw, int i0, uint32_t q,
                        uint32_t q2) {
  {
    Tw t = ld_tw(tw + i0);
#pragma unroll
    for (int e = 0; e < 8; e++) ct_bfly<FAST>(v[e], v[e + 8], t, q, q2);
  }
  {
    Tw t[2];
    ld_tws<2>(tw + (i0 << 1), t);
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++)
        ct_bfly<FAST>(v[8 * j + e], v[8 * j + e + 4], t[j], q, q2);
  }
  {
    Tw t[4];
    ld_tws<4>(tw + (i0 << 2), t);
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int e = 0; e < 2; e++)
        ct_bfly<FAST>(v[4 * j + e], v[4 * j + e + 2], t[j], q, q2);
  }
  {
    Tw t[8];
    ld_tws<8>(tw + (i0 << 3), t);
#pragma unroll
    for (int j = 0; j < 8; j++)
      ct_bfly<FAST>(v[2 * j], v[2 * j + 1], t[j], q, q2);
  }
}

// Four Gentleman-Sande stages, the mirror image of ct_radix16.
template <bool FAST>
CFHE_HD void gs_radix16(uint32_t *v, const Tw *tw, int i0, uint32_t q,
                        uint32_t q2) {
  {
    Tw t[8];
    ld_tws<8>(tw + (i0 << 3), t);
#pragma unroll
    for (int j = 0; j < 8; j++)
      gs_bfly<FAST>(v[2 * j], v[2 * j + 1], t[j], q, q2);
  }
  {
    Tw t[4];
    ld_tws<4>(tw + (i0 << 2), t);
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int e = 0; e < 2; e++)
        gs_bfly<FAST>(v[4 * j + e], v[4 * j + e + 2], t[j], q, q2);
  }
  {
    Tw t[2];
    ld_tws<2>(tw + (i0 << 1), t);
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++)
        gs_bfly<FAST>(v[8 * j + e], v[8 * j + e + 4], t[j], q, q2);
  }
  {
    Tw t = ld_tw(tw + i0);
#pragma unroll
    for (int e = 0; e < 8; e++) gs_bfly<FAST>(v[e], v[e + 8], t, q, q2);
  }
}

// The same four stages with all 15 twiddles fetched up front, so that their
// load latency overlaps whatever the caller does between the fetch and the
// butterflies. t: [0] stage 0, [1..2] stage 1, [3..6] stage 2, [7..14] stage 3.
CFHE_HD void ld_tw16(const Tw *tw, int i0, Tw *t) {
  t[0] = ld_tw(tw + i0);
  ld_tws<2>(tw + (i0 << 1), t + 1);
  ld_tws<4>(tw + (i0 << 2), t + 3);
  ld_tws<8>(tw + (i0 << 3), t + 7);
}

template <bool FAST>
CFHE_HD void ct_radix16_pre(uint32_t *v, const Tw *t, uint32_t q, uint32_t q2) {
#pragma unroll
  for (int e = 0; e < 8; e++) ct_bfly<FAST>(v[e], v[e + 8], t[0], q, q2);
#pragma unroll
  for (int j = 0; j < 2; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) ct_bfly<FAST>(v[8 * j + e], v[8 * j + e + 4], t[1 + j], q, q2);
#pragma unroll
  for (int j = 0; j < 4; j++)
#pragma unroll
    for (int e = 0; e < 2; e++) ct_bfly<FAST>(v[4 * j + e], v[4 * j + e + 2], t[3 + j], q, q2);
#pragma unroll
  for (int j = 0; j < 8; j++) ct_bfly<FAST>(v[2 * j], v[2 * j + 1], t[7 + j], q, q2);
}

template <bool FAST>
CFHE_HD void gs_radix16_pre(uint32_t *v, const Tw *t, uint32_t q, uint32_t q2) {
#pragma unroll
  for (int j = 0; j < 8; j++) gs_bfly<FAST>(v[2 * j], v[2 * j + 1], t[7 + j], q, q2);
#pragma unroll
  for (int j = 0; j < 4; j++)
#pragma unroll
    for (int e = 0; e < 2; e++) gs_bfly<FAST>(v[4 * j + e], v[4 * j + e + 2], t[3 + j], q, q2);
#pragma unroll
  for (int j = 0; j < 2; j++)
#pragma unroll
    for (int e = 0; e < 4; e++) gs_bfly<FAST>(v[8 * j + e], v[8 * j + e + 4], t[1 + j], q, q2);
#pragma unroll
  for (int e = 0; e < 8; e++) gs_bfly<FAST>(v[e], v[e + 8], t[0], q, q2);
}

// word offset of column x inside a padded in-row buffer row
CFHE_HD int pad_col(int x) { return x + 4 * (x >> 4); }

// ---------------------------------------------------------------------------
// Forward phases. `c` = CTA rank in the cluster, `tid` = thread in the CTA.
// ---------------------------------------------------------------------------

// Stages 1-4 across rows; the 16 loaded values arrive in v (any value below
// 2q; the caller applies an optional pre-multiplication before this call).
template <bool FAST>
CFHE_HD void fwd_rows_a(uint32_t *v, int tid, uint32_t *xbuf, const Tw *tw,
                        uint32_t q, uint32_t q2) {
  const int x = tid & 31, r0 = tid >> 5;
  ct_radix16<FAST>(v, tw, 1, q, q2);
#pragma unroll
  for (int k = 0; k < 16; k++) xbuf[(r0 + 16 * k) * kStripCols + x] = v[k];
}

// Stages 5-8 across rows, then hand each value to the CTA that owns its row.
// remote(rank) returns the receive buffer of CTA `rank`.
template <bool FAST, typename Remote>
CFHE_HD void fwd_rows_b(int c, int tid, const uint32_t *xbuf, Remote remote,
                        const Tw *tw, uint32_t q, uint32_t q2) {
  const int x = tid & 31, g = tid >> 5;
  uint32_t v[16];
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = xbuf[(16 * g + k) * kStripCols + x];
  ct_radix16<FAST>(v, tw, 16 + g, q, q2);
  uint32_t *dst = remote(g >> 1);
  const int col = kStripCols * c + x;
  const int base = (16 * (g & 1)) * kRowStride + pad_col(col);
#pragma unroll
  for (int k = 0; k < 16; k++) dst[base + k * kRowStride] = v[k];
}

// Stages 9-12 inside rows. rbuf and xbuf may be the same buffer: a row is
// read and written by one half-warp only.
template <bool FAST>
CFHE_HD void fwd_cols_a(int c, int tid, const uint32_t *rbuf, uint32_t *xbuf,
                        const Tw *tw, uint32_t q, uint32_t q2) {
  const int rho = tid >> 4, x0 = tid & 15;
  const int R = kOwnRows * c + rho;
  uint32_t v[16];
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = rbuf[rho * kRowStride + x0 + 20 * k];
  ct_radix16<FAST>(v, tw, 256 + R, q, q2);
#pragma unroll
  for (int k = 0; k < 16; k++) xbuf[rho * kRowStride + x0 + 20 * k] = v[k];
}

// Stages 13-16 inside rows; leaves the 16 consecutive outputs of word offset
// R*256 + 16g in v, folded to [0,q).
template <bool FAST>
CFHE_HD void fwd_cols_b(uint32_t *v, int c, int tid, const uint32_t *xbuf,
                        const Tw *tw, uint32_t q, uint32_t q2) {
  const int rho = tid >> 4, g = tid & 15;
  const int R = kOwnRows * c + rho;
  const uint32_t *p = xbuf + rho * kRowStride + 20 * g;
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int i = 0; i < 4; i++) {
    uint4 t = reinterpret_cast<const uint4 *>(p)[i];
    v[4 * i] = t.x;
    v[4 * i + 1] = t.y;
    v[4 * i + 2] = t.z;
    v[4 * i + 3] = t.w;
  }
#else
  for (int k = 0; k < 16; k++) v[k] = p[k];
#endif
  ct_radix16<FAST>(v, tw, 4096 + 16 * R + g, q, q2);
#pragma unroll
  for (int k = 0; k < 16; k++) {
    v[k] = ct_fold<FAST>(v[k], q, q2);
  }
}

// ---------------------------------------------------------------------------
// Inverse phases.
// ---------------------------------------------------------------------------

// Stages with strides 1,2,4,8 words on the 16 consecutive inputs in v
// (canonical), then into the padded in-row buffer.
template <bool FAST>
CFHE_HD void inv_cols_a(uint32_t *v, int c, int tid, uint32_t *xbuf,
                        const Tw *itw, uint32_t q, uint32_t q2) {
  const int rho = tid >> 4, g = tid & 15;
  const int R = kOwnRows * c + rho;
  gs_radix16<FAST>(v, itw, 4096 + 16 * R + g, q, q2);
  uint32_t *p = xbuf + rho * kRowStride + 20 * g;
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int i = 0; i < 4; i++)
    reinterpret_cast<uint4 *>(p)[i] =
        make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
#else
  for (int k = 0; k < 16; k++) p[k] = v[k];
#endif
}

// Strides 16..128 words, then hand each value to the CTA owning its column.
template <bool FAST, typename Remote>
CFHE_HD void inv_cols_b(int c, int tid, const uint32_t *xbuf, Remote remote,
                        const Tw *itw, uint32_t q, uint32_t q2) {
  const int rho = tid >> 4, x0 = tid & 15;
  const int R = kOwnRows * c + rho;
  uint32_t v[16];
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = xbuf[rho * kRowStride + x0 + 20 * k];
  gs_radix16<FAST>(v, itw, 256 + R, q, q2);
#pragma unroll
  for (int k = 0; k < 16; k++) {
    const int col_l = x0 + 16 * (k & 1);
    // rows alternate a 16-word rotation so a warp (two rows x 16 columns)
    // lands on 32 distinct banks
    remote(k >> 1)[R * kStripCols + ((col_l + 16 * (R & 1)) & 31)] = v[k];
  }
}

// Strides 1..8 rows.
template <bool FAST>
CFHE_HD void inv_rows_a(int tid, const uint32_t *rbuf, uint32_t *xbuf,
                        const Tw *itw, uint32_t q, uint32_t q2) {
  const int x = tid & 31, g = tid >> 5;
  uint32_t v[16];
#pragma unroll
  for (int k = 0; k < 16; k++) {
    const int r = 16 * g + k;
    v[k] = rbuf[r * kStripCols + ((x + 16 * (r & 1)) & 31)];
  }
  gs_radix16<FAST>(v, itw, 16 + g, q, q2);
#pragma unroll
  for (int k = 0; k < 16; k++) xbuf[(16 * g + k) * kStripCols + x] = v[k];
}

// Strides 16..128 rows, then the per-limb constant; leaves rows r0 + 16k of
// column 32c + x in v, canonical or centred.
template <bool FAST>
CFHE_HD void inv_rows_b(uint32_t *v, int tid, const uint32_t *xbuf,
                        const Tw *itw, Tw kc, bool centred, uint32_t q,
                        uint32_t q2) {
  const int x = tid & 31, r0 = tid >> 5;
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = xbuf[(r0 + 16 * k) * kStripCols + x];
  gs_radix16<FAST>(v, itw, 1, q, q2);
  const uint32_t half = q >> 1;
#pragma unroll
  for (int k = 0; k < 16; k++) {
    uint32_t a = shoup_mul(v[k], kc, q);
    a = umin32(a, a - q);
    if (centred && a > half) a -= q;
    v[k] = a;
  }
}

}  // namespace cfhe
