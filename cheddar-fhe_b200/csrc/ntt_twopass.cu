// Two-pass NTT / INTT kernels for sm_100a that meet in the L2 cache.
//
// A limb is a 256 x 256 matrix (row-major). The forward transform runs the
// eight stages that pair rows in a column pass (one CTA per tile of 16
// columns: 64-byte row segments, transposition through shared memory) and the
// eight stages inside rows in a row pass (one CTA per 16 rows, one half-warp
// per row, exchange with __syncwarp only). The inverse transform is the mirror
// image. Both passes are plain grids of independent 256-thread CTAs: no
// cluster, no cross-CTA wait, at least four CTAs per SM.
//
// What makes two passes cost one trip to HBM: the host launches them over
// chunks of at most kChunkJobs limbs (48 MiB), the second pass works in place
// on what the first just wrote, and a chunk is well below the 126 MB L2. The
// first pass reads HBM and writes L2; the second reads and rewrites the same
// lines in L2; they reach HBM once, when they are evicted.
//
// The per-thread arithmetic (radix-16 register phases, Shoup twiddles, lazy
// [0,4q) butterflies for primes below 2^30) is shared with the cluster
// kernels (ntt_core.cuh); the two implementations produce the same words.
#include "context.h"

namespace cfhe {
namespace {

constexpr int kTpThreads = 256;
constexpr int kColTile = 16;   // columns per CTA in the column pass
constexpr int kRowTile = 16;   // rows per CTA in the row pass
constexpr int kChunkJobs = 192;
// column-pass buffer: word (r, x) at r*16 + x + 16*(r >> 4): both the
// (r0 + 16k) and the (16g + k) access of a warp touch 32 distinct banks
constexpr int kColBufWords = 256 * kColTile + 256;
constexpr int kRowBufTileWords = kRowTile * kRowStride;

struct Job {
  int p, l;
  uint32_t q;
  const Tw *tw;
  const uint32_t *src;
  uint32_t *dst;
};

__device__ __forceinline__ Job get_job(const NttArgs &a, int t) {
  Job j;
  j.p = t / a.n_limbs;
  j.l = t - j.p * a.n_limbs;
  j.q = a.q[j.l];
  j.tw = a.table + (size_t)a.g[j.l] * kN;
  j.src = a.src + (size_t)j.p * a.src_poly_stride + (size_t)a.src_limb[j.l] * kN;
  j.dst = a.dst + (size_t)j.p * a.dst_poly_stride + (size_t)a.dst_limb[j.l] * kN;
  return j;
}

__device__ __forceinline__ int col_word(int r, int x) { return r * kColTile + x + 16 * (r >> 4); }

// ---- forward, pass 1: stages 1-8 (rows paired), src -> dst, values lazy ----
template <bool FAST>
__device__ __forceinline__ void fwd_cols(const NttArgs &a, const Job &j, int tile, int tid,
                                         uint32_t *xbuf) {
  const uint32_t q = j.q, q2 = 2 * q;
  const int x = tid & 15, r0 = tid >> 4;
  uint32_t v[16];
  Tw t[15];
  const uint32_t *s = j.src + r0 * kRowWords + kColTile * tile + x;
  ld_tw16(j.tw, 1, t);  // the tables are never written by a kernel: fetched before the wait
  pdl_wait();
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = s[k * 16 * kRowWords];
  if (a.premul) {
    const Tw kc = a.kc[j.l];
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = shoup_mul(v[k], kc, q);
  }
  ct_radix16_pre<FAST>(v, t, q, q2);
  const int g = r0;
  ld_tw16(j.tw, 16 + g, t);  // in flight across the transposition
#pragma unroll
  for (int k = 0; k < 16; k++) xbuf[col_word(r0 + 16 * k, x)] = v[k];
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = xbuf[col_word(16 * g + k, x)];
  ct_radix16_pre<FAST>(v, t, q, q2);
  uint32_t *o = j.dst + (16 * g) * kRowWords + kColTile * tile + x;
#pragma unroll
  for (int k = 0; k < 16; k++) o[k * kRowWords] = v[k];
}

// ---- forward, pass 2: stages 9-16 (inside rows), in place on dst ----
template <bool FAST>
__device__ __forceinline__ void fwd_rows(const NttArgs &a, const Job &j, int blk, int tid,
                                         uint32_t *xbuf) {
  const uint32_t q = j.q, q2 = 2 * q;
  const int rho = tid >> 4, x0 = tid & 15, g = x0;
  const int R = kRowTile * blk + rho;
  uint32_t v[16];
  Tw t[15];
  const uint32_t *s = j.dst + R * kRowWords + x0;
  ld_tw16(j.tw, 256 + R, t);
  pdl_wait();
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = s[16 * k];
  ct_radix16_pre<FAST>(v, t, q, q2);
  ld_tw16(j.tw, 4096 + 16 * R + g, t);  // in flight across the exchange
  uint32_t *row = xbuf + rho * kRowStride;
#pragma unroll
  for (int k = 0; k < 16; k++) row[x0 + 20 * k] = v[k];
  __syncwarp();  // a row lives in one half-warp
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint4 t = reinterpret_cast<const uint4 *>(row + 20 * g)[i];
    v[4 * i] = t.x;
    v[4 * i + 1] = t.y;
    v[4 * i + 2] = t.z;
    v[4 * i + 3] = t.w;
  }
  ct_radix16_pre<FAST>(v, t, q, q2);
  const int off = R * kRowWords + 16 * g;
  if (a.ep_mode) {
    // ModDown-family epilogue: (pad * x - ntt) * scale, canonical. The
    // transform's values enter as the last stage left them (below 4q, or 2q
    // for the large primes): a Shoup product takes any 32-bit word.
    const int l = j.l;
    const Tw scale = a.ep_scale[l];
    uint32_t x[16];
    if (a.ep_limb[l] != 255) {
      const uint4 *xp = reinterpret_cast<const uint4 *>(
          a.ep_src + (size_t)j.p * a.ep_poly_stride + (size_t)a.ep_limb[l] * kN + off);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 u = xp[i];
        x[4 * i] = u.x;
        x[4 * i + 1] = u.y;
        x[4 * i + 2] = u.z;
        x[4 * i + 3] = u.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 16; k++) x[k] = 0;
    }
    if (a.ep_mode == 2) {
      // pad*scale*x - scale*ntt: two independent products
      const Tw ps = a.ep_ps[l];
#pragma unroll
      for (int k = 0; k < 16; k++) {
        uint32_t t1 = shoup_mul(x[k], ps, q), t2 = shoup_mul(v[k], scale, q);  // both below 2q
        if constexpr (FAST) {
          const uint32_t r = t1 - t2 + q2;  // (0, 4q)
          v[k] = ct_fold<true>(r, q, q2);
        } else {
          t1 = umin32(t1, t1 - q);
          t2 = umin32(t2, t2 - q);
          const uint32_t r = t1 - t2 + q;  // (0, 2q)
          v[k] = umin32(r, r - q);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 16; k++) {
        uint32_t d;
        if constexpr (FAST) {
          const uint32_t y = umin32(v[k], v[k] - q2);  // below 2q
          d = x[k] - y + q2;                            // (0, 3q)
        } else {
          const uint32_t y = umin32(v[k], v[k] - q);    // below q
          d = x[k] - y + q;                             // (0, 2q)
        }
        d = shoup_mul(d, scale, q);
        v[k] = umin32(d, d - q);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = ct_fold<FAST>(v[k], q, q2);
  }
  uint4 *o = reinterpret_cast<uint4 *>(j.dst + off);
#pragma unroll
  for (int i = 0; i < 4; i++)
    o[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

// ---- inverse, pass 1: strides 1..128 words (inside rows), src -> dst ----
template <bool FAST>
__device__ __forceinline__ void inv_rows(const NttArgs &, const Job &j, int blk, int tid,
                                         uint32_t *xbuf) {
  const uint32_t q = j.q, q2 = 2 * q;
  const int rho = tid >> 4, g = tid & 15, x0 = g;
  const int R = kRowTile * blk + rho;
  uint32_t v[16];
  Tw t[15];
  ld_tw16(j.tw, 4096 + 16 * R + g, t);
  pdl_wait();
  const uint4 *s = reinterpret_cast<const uint4 *>(j.src + R * kRowWords + 16 * g);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint4 u = s[i];
    v[4 * i] = u.x;
    v[4 * i + 1] = u.y;
    v[4 * i + 2] = u.z;
    v[4 * i + 3] = u.w;
  }
  gs_radix16_pre<FAST>(v, t, q, q2);
  ld_tw16(j.tw, 256 + R, t);  // in flight across the exchange
  uint32_t *row = xbuf + rho * kRowStride;
#pragma unroll
  for (int i = 0; i < 4; i++)
    reinterpret_cast<uint4 *>(row + 20 * g)[i] =
        make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = row[x0 + 20 * k];
  gs_radix16_pre<FAST>(v, t, q, q2);
  uint32_t *o = j.dst + R * kRowWords + x0;
#pragma unroll
  for (int k = 0; k < 16; k++) o[16 * k] = v[k];
}

// ---- inverse, pass 2: strides 1..128 rows, per-limb constant, in place ----
template <bool FAST>
__device__ __forceinline__ void inv_cols(const NttArgs &a, const Job &j, int tile, int tid,
                                         uint32_t *xbuf) {
  const uint32_t q = j.q, q2 = 2 * q;
  const int x = tid & 15, g = tid >> 4;
  uint32_t v[16];
  uint32_t *base = j.dst + kColTile * tile + x;
  Tw t[15];
  ld_tw16(j.tw, 16 + g, t);
  pdl_wait();
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = base[(16 * g + k) * kRowWords];
  gs_radix16_pre<FAST>(v, t, q, q2);
  ld_tw16(j.tw, 1, t);  // in flight across the transposition
#pragma unroll
  for (int k = 0; k < 16; k++) xbuf[col_word(16 * g + k, x)] = v[k];
  __syncthreads();
  const int r0 = g;
#pragma unroll
  for (int k = 0; k < 16; k++) v[k] = xbuf[col_word(r0 + 16 * k, x)];
  gs_radix16_pre<FAST>(v, t, q, q2);
  const Tw kc = a.kc[j.l];
  const uint32_t half = q >> 1;
  const bool centred = a.centred != 0;
#pragma unroll
  for (int k = 0; k < 16; k++) {
    uint32_t t = shoup_mul(v[k], kc, q);
    t = umin32(t, t - q);
    if (centred && t > half) t -= q;
    base[(r0 + 16 * k) * kRowWords] = t;
  }
}

// PASS 0: column pass, PASS 1: row pass. Forward runs 0 then 1; inverse 1 then 0.
template <bool INV, int PASS>
__global__ void __launch_bounds__(kTpThreads, 4)
    ntt_twopass_kernel(const __grid_constant__ NttArgs a, int job0) {
  __shared__ __align__(16) uint32_t xbuf[PASS == 0 ? kColBufWords : kRowBufTileWords];
  pdl_launch_dependents();
  const Job j = get_job(a, job0 + blockIdx.y);  // each pass calls pdl_wait() after its first twiddle fetch
  const int tid = threadIdx.x, part = blockIdx.x;
  const bool fast = j.q < (1u << 30);
  if constexpr (!INV && PASS == 0) {
    if (fast) fwd_cols<true>(a, j, part, tid, xbuf); else fwd_cols<false>(a, j, part, tid, xbuf);
  } else if constexpr (!INV && PASS == 1) {
    if (fast) fwd_rows<true>(a, j, part, tid, xbuf); else fwd_rows<false>(a, j, part, tid, xbuf);
  } else if constexpr (INV && PASS == 1) {
    if (fast) inv_rows<true>(a, j, part, tid, xbuf); else inv_rows<false>(a, j, part, tid, xbuf);
  } else {
    if (fast) inv_cols<true>(a, j, part, tid, xbuf); else inv_cols<false>(a, j, part, tid, xbuf);
  }
}

}  // namespace

int launch_ntt_twopass(const Context &ctx, const NttArgs &args, bool inverse) {
  const int total = args.n_limbs * args.n_polys;
  if (total <= 0) return 0;
  const dim3 block(kTpThreads);
  for (int job0 = 0; job0 < total; job0 += kChunkJobs) {
    const int cnt = total - job0 < kChunkJobs ? total - job0 : kChunkJobs;
    const dim3 cols(kRowWords / kColTile, cnt), rows(kRowWords / kRowTile, cnt);
    if (inverse) {
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_twopass_kernel<true, 1>, rows, block, 0, ctx.stream, args, job0));
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_twopass_kernel<true, 0>, cols, block, 0, ctx.stream, args, job0));
    } else {
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_twopass_kernel<false, 0>, cols, block, 0, ctx.stream, args, job0));
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_twopass_kernel<false, 1>, rows, block, 0, ctx.stream, args, job0));
    }
  }
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
