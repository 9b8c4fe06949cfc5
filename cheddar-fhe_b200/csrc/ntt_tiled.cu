// Pipelined two-pass NTT / INTT for sm_100a: TMA in, twiddles resident,
// several polynomials of one prime per CTA.
//
// A limb is a 256 x 256 matrix (row-major). As in ntt_twopass.cu the forward
// transform runs the eight stages that pair rows in a column pass (a CTA owns
// 16 columns) and the eight stages inside rows in a row pass (a CTA owns 16
// rows), the inverse transform the mirror image, and the two passes of a chunk
// of limbs meet in the L2 cache. What is different here:
//
//   * Limb transforms that share a prime are processed by the same CTA, one
//     after the other (a "unit": a few polynomials of one limb, or the copies
//     of one prime in the digits of a ModUp). The twiddles of a pass are
//     fetched once per unit instead of once per limb: the column pass keeps
//     the 255 twiddles of its stages in shared memory, the row pass the 240
//     twiddles of its first phase in shared memory and the 15 thread-owned
//     twiddles of its last phase in registers. Half of the bytes a row pass
//     used to pull from L2 were twiddles.
//   * Data arrive through the asynchronous copy engine: one tiled TMA load of
//     the box {16 columns, 256 rows} per column tile, sixteen 1 KiB bulk copies
//     per row tile, double buffered, so that the next polynomial's tile is on
//     its way while the current one is computed. The column pass also leaves
//     through a tiled TMA store.
//   * The inverse transform's per-limb constant is folded into its last stage.
//
// The arithmetic (Shoup twiddles, lazy butterflies, radix-16 register phases)
// is that of ntt_core.cuh; results are canonical and therefore the same words
// as the other implementations produce.
//
// Every wait on an mbarrier is bounded: a wait that runs out raises the
// context's error flag, and the CTA goes on without leaving its barrier
// pattern.
#include <cuda.h>

#include "context.h"
#include "host_math.h"

namespace cfhe {
namespace {

constexpr int kThreads = 256;
constexpr int kTile = 16;                      // columns (column pass) or rows (row pass) per CTA
constexpr int kBoxWords = kRowWords * kTile;   // one tile
constexpr int kRowPitch = 272;                 // words between two rows of a row tile: the two rows of a warp fall on different banks
constexpr int kRowBufWords = kTile * kRowPitch;
constexpr int kExWords = kTile * kRowStride;   // padded exchange buffer of the row pass (ntt_core.cuh layout)
constexpr int kMaxUnits = 256;
constexpr uint32_t kWaitHintNs = 2000;
constexpr uint32_t kSpinLimit = 1u << 20;

// Work list of one launch: unit u covers cnt[u] limb transforms starting at
// (limb l[u], polynomial p0[u]) and advancing the polynomial first, then the
// limb (the limbs a unit walks over share one prime).
struct UnitArgs {
  int n_units;
  int *error_flag;
  uint16_t l[kMaxUnits];
  uint16_t p0[kMaxUnits];
  uint8_t cnt[kMaxUnits];
  Tw kcw[kMaxLimbs];  // inverse: per-limb constant times the last stage's twiddle
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)
      : "memory");
  return ok != 0;
}
// Bounded wait. When it runs out the error flag is raised and the caller goes
// on with whatever the buffer holds, so that no thread leaves the CTA's
// barrier pattern.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int *error_flag) {
  for (uint32_t i = 0; i < kSpinLimit; i++)
    if (mbar_try_wait(bar, parity)) return;
  atomicExch(error_flag, 1);
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// generic-proxy accesses to shared memory before an asynchronous copy touches it
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap *tm, int c0, int c1, int c2,
                                             int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_box(const CUtensorMap *tm, int c0, int c1, int c2, int c3,
                                              uint32_t src) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group"
      " [%0, {%1, %2, %3, %4}], [%5];" ::"l"(tm),
      "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(src)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Data written through the generic proxy (ordinary stores of an earlier
// kernel) are read here by the asynchronous proxy (TMA and bulk loads). The
// grid-dependency wait orders the grids; this fence, executed by the thread
// that issues the copies after that wait, orders the two proxies.
__device__ __forceinline__ void fence_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the committed stores have finished reading shared memory
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ---- radix-16 phases whose twiddles sit in shared memory ---------------------
// lv[s] points at the 2^s twiddles of stage s for the caller's group.
struct TwLevels {
  const Tw *lv[4];
};
__device__ __forceinline__ Tw lds_tw(const Tw *p) {
  const uint2 v = *reinterpret_cast<const uint2 *>(p);
  return Tw{v.x, v.y};
}
template <int CNT>
__device__ __forceinline__ void lds_tws(const Tw *p, Tw *out) {
  if constexpr (CNT == 1) {
    out[0] = lds_tw(p);
  } else {
#pragma unroll
    for (int i = 0; i < CNT / 2; i++) {
      const uint4 v = reinterpret_cast<const uint4 *>(p)[i];
      out[2 * i] = Tw{v.x, v.y};
      out[2 * i + 1] = Tw{v.z, v.w};
    }
  }
}
template <bool FAST>
__device__ __forceinline__ void ct_radix16_s(uint32_t *v, const TwLevels &t, uint32_t q, uint32_t q2) {
  {
    const Tw w = lds_tw(t.lv[0]);
#pragma unroll
    for (int e = 0; e < 8; e++) ct_bfly<FAST>(v[e], v[e + 8], w, q, q2);
  }
  {
    Tw w[2];
    lds_tws<2>(t.lv[1], w);
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) ct_bfly<FAST>(v[8 * j + e], v[8 * j + e + 4], w[j], q, q2);
  }
  {
    Tw w[4];
    lds_tws<4>(t.lv[2], w);
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int e = 0; e < 2; e++) ct_bfly<FAST>(v[4 * j + e], v[4 * j + e + 2], w[j], q, q2);
  }
  {
    Tw w[8];
    lds_tws<8>(t.lv[3], w);
#pragma unroll
    for (int j = 0; j < 8; j++) ct_bfly<FAST>(v[2 * j], v[2 * j + 1], w[j], q, q2);
  }
}
// LAST false: the final stage is left to the caller (the inverse transform
// folds its per-limb constant into it)
template <bool FAST, bool LAST>
__device__ __forceinline__ void gs_radix16_s(uint32_t *v, const TwLevels &t, uint32_t q, uint32_t q2) {
  {
    Tw w[8];
    lds_tws<8>(t.lv[3], w);
#pragma unroll
    for (int j = 0; j < 8; j++) gs_bfly<FAST>(v[2 * j], v[2 * j + 1], w[j], q, q2);
  }
  {
    Tw w[4];
    lds_tws<4>(t.lv[2], w);
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int e = 0; e < 2; e++) gs_bfly<FAST>(v[4 * j + e], v[4 * j + e + 2], w[j], q, q2);
  }
  {
    Tw w[2];
    lds_tws<2>(t.lv[1], w);
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) gs_bfly<FAST>(v[8 * j + e], v[8 * j + e + 4], w[j], q, q2);
  }
  if constexpr (LAST) {
    const Tw w = lds_tw(t.lv[0]);
#pragma unroll
    for (int e = 0; e < 8; e++) gs_bfly<FAST>(v[e], v[e + 8], w, q, q2);
  }
}

// word (r, x) of a column tile: 16 words per row, dense (the layout a tiled
// TMA copy reads and writes)
__device__ __forceinline__ int box_word(int r, int x) { return r * kTile + x; }

struct Member {
  int l, p;
};
__device__ __forceinline__ void next_member(Member &m, int n_polys) {
  if (++m.p == n_polys) {
    m.p = 0;
    m.l++;
  }
}

// ---------------------------------------------------------------------------
// column pass: forward stages 1-8 (src -> dst), inverse stages 9-16 (in place)
// ---------------------------------------------------------------------------
template <bool INV, bool FAST>
__device__ __forceinline__ void cols_body(const NttArgs &a, const UnitArgs &u, int l, uint32_t q, int hi, int x,
                                          uint32_t *box, const Tw *tw_s) {
  const uint32_t q2 = 2 * q;
  uint32_t v[16];
  // twiddle groups: the strided phase (rows hi + 16k) uses group 1, the block
  // phase (rows 16hi + k) group 16 + hi
  TwLevels strided, block;
#pragma unroll
  for (int s = 0; s < 4; s++) {
    strided.lv[s] = tw_s + (1 << s);
    block.lv[s] = tw_s + ((16 + hi) << s);
  }
  if constexpr (!INV) {
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = box[box_word(hi + 16 * k, x)];
    if (a.premul) {
      const Tw kc = a.kc[l];
#pragma unroll
      for (int k = 0; k < 16; k++) v[k] = shoup_mul(v[k], kc, q);
    }
    ct_radix16_s<FAST>(v, strided, q, q2);
#pragma unroll
    for (int k = 0; k < 16; k++) box[box_word(hi + 16 * k, x)] = v[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = box[box_word(16 * hi + k, x)];
    ct_radix16_s<FAST>(v, block, q, q2);
#pragma unroll
    for (int k = 0; k < 16; k++) box[box_word(16 * hi + k, x)] = v[k];
  } else {
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = box[box_word(16 * hi + k, x)];
    gs_radix16_s<FAST, true>(v, block, q, q2);
#pragma unroll
    for (int k = 0; k < 16; k++) box[box_word(16 * hi + k, x)] = v[k];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = box[box_word(hi + 16 * k, x)];
    gs_radix16_s<FAST, false>(v, strided, q, q2);
    // last stage with the per-limb constant folded in:
    // (X, Y) <- ((X + Y) kc, (X - Y) w kc), canonical or centred
    const Tw kc = a.kc[l], kcw = u.kcw[l];
    const uint32_t half = q >> 1;
    const bool centred = a.centred != 0;
#pragma unroll
    for (int e = 0; e < 8; e++) {
      uint32_t s, d;
      if constexpr (FAST) {
        s = v[e] + v[e + 8];
        d = v[e] - v[e + 8] + q2;
      } else {
        const uint32_t xx = umin32(v[e], v[e] - q), yy = umin32(v[e + 8], v[e + 8] - q);
        s = xx + yy;
        d = xx - yy + q;
      }
      s = shoup_mul(s, kc, q);
      d = shoup_mul(d, kcw, q);
      s = umin32(s, s - q);
      d = umin32(d, d - q);
      if (centred) {
        if (s > half) s -= q;
        if (d > half) d -= q;
      }
      v[e] = s;
      v[e + 8] = d;
    }
#pragma unroll
    for (int k = 0; k < 16; k++) box[box_word(hi + 16 * k, x)] = v[k];
  }
}

template <bool INV>
__global__ void __launch_bounds__(kThreads, 4)
    ntt_cols_kernel(const __grid_constant__ NttArgs a, const __grid_constant__ UnitArgs u,
                    const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out) {
  __shared__ __align__(128) uint32_t box[2][kBoxWords];
  __shared__ __align__(16) Tw tw_s[256];
  __shared__ __align__(8) uint64_t full[2];
  const int tid = threadIdx.x, x = tid & 15, hi = tid >> 4;
  const int tile = blockIdx.x, unit = blockIdx.y;
  const int cnt = u.cnt[unit];
  Member m{u.l[unit], u.p0[unit]};
  const uint32_t q = a.q[m.l];
  const Tw *tw = a.table + (size_t)a.g[m.l] * kN;
  pdl_launch_dependents();
  if (tid == 0) {
    mbar_init(smem_u32(&full[0]), 1);
    mbar_init(smem_u32(&full[1]), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (tid == 0) {
    // the first 256 table entries hold every twiddle of the eight row-pairing
    // stages; tables are never written by a kernel, so this copy may start
    // before the grid dependency is resolved
    mbar_expect_tx(smem_u32(&full[0]), kBoxWords * 4 + 256 * sizeof(Tw));
    bulk_load(smem_u32(tw_s), tw, 256 * sizeof(Tw), smem_u32(&full[0]));
  }
  pdl_wait();
#ifndef CFHE_NO_PROXY_FENCE
  fence_async_all();
#endif
  if (tid == 0) {
    Member f = m;
    tma_load_box(smem_u32(box[0]), &tm_in, kTile * tile, 0, INV ? a.dst_limb[f.l] : a.src_limb[f.l], f.p,
                 smem_u32(&full[0]));
    if (cnt > 1) {
      next_member(f, a.n_polys);
      mbar_expect_tx(smem_u32(&full[1]), kBoxWords * 4);
      tma_load_box(smem_u32(box[1]), &tm_in, kTile * tile, 0, INV ? a.dst_limb[f.l] : a.src_limb[f.l], f.p,
                   smem_u32(&full[1]));
    }
  }
  Member ahead = m;  // runs two members ahead of m, for the refill
  next_member(ahead, a.n_polys);
  const bool fast = q < (1u << 30);
#pragma unroll 1
  for (int i = 0; i < cnt; i++) {
    const int b = i & 1;
    next_member(ahead, a.n_polys);
    mbar_wait(smem_u32(&full[b]), (i >> 1) & 1, u.error_flag);
    if (fast)
      cols_body<INV, true>(a, u, m.l, q, hi, x, box[b], tw_s);
    else
      cols_body<INV, false>(a, u, m.l, q, hi, x, box[b], tw_s);
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      tma_store_box(&tm_out, kTile * tile, 0, a.dst_limb[m.l], m.p, smem_u32(box[b]));
      bulk_commit();
      if (i + 2 < cnt) {
        bulk_wait_read();  // the store has read the buffer: it may be refilled
        mbar_expect_tx(smem_u32(&full[b]), kBoxWords * 4);
        tma_load_box(smem_u32(box[b]), &tm_in, kTile * tile, 0,
                     INV ? a.dst_limb[ahead.l] : a.src_limb[ahead.l], ahead.p, smem_u32(&full[b]));
      }
    }
    next_member(m, a.n_polys);
  }
  if (tid == 0) bulk_wait_read();
}

// ---------------------------------------------------------------------------
// row pass: forward stages 9-16 (in place on dst), inverse stages 1-8 (src -> dst)
// ---------------------------------------------------------------------------
template <bool FAST>
__device__ __forceinline__ void fwd_rows_finish(const NttArgs &a, const Member &m, uint32_t q, int off, uint32_t *v) {
  const uint32_t q2 = 2 * q;
  if (a.ep_mode) {
    // ModDown-family epilogue: (pad * x - ntt) * scale, canonical; the
    // transform's values enter as the last stage left them
    const int l = m.l;
    const Tw scale = a.ep_scale[l];
    uint32_t xin[16];
    if (a.ep_limb[l] != 255) {
      const uint4 *xp = reinterpret_cast<const uint4 *>(a.ep_src + (size_t)m.p * a.ep_poly_stride +
                                                        (size_t)a.ep_limb[l] * kN + off);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint4 w = xp[i];
        xin[4 * i] = w.x;
        xin[4 * i + 1] = w.y;
        xin[4 * i + 2] = w.z;
        xin[4 * i + 3] = w.w;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 16; k++) xin[k] = 0;
    }
    if (a.ep_mode == 2) {
      const Tw ps = a.ep_ps[l];
#pragma unroll
      for (int k = 0; k < 16; k++) {
        uint32_t t1 = shoup_mul(xin[k], ps, q), t2 = shoup_mul(v[k], scale, q);
        if constexpr (FAST) {
          v[k] = ct_fold<true>(t1 - t2 + q2, q, q2);
        } else {
          t1 = umin32(t1, t1 - q);
          t2 = umin32(t2, t2 - q);
          const uint32_t r = t1 - t2 + q;
          v[k] = umin32(r, r - q);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 16; k++) {
        uint32_t d;
        if constexpr (FAST) {
          const uint32_t y = umin32(v[k], v[k] - q2);
          d = xin[k] - y + q2;
        } else {
          const uint32_t y = umin32(v[k], v[k] - q);
          d = xin[k] - y + q;
        }
        d = shoup_mul(d, scale, q);
        v[k] = umin32(d, d - q);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = ct_fold<FAST>(v[k], q, q2);
  }
}

// v holds the member's words as the caller took them out of the row buffer:
// forward the strided set (g + 16k), inverse the block (16g .. 16g+15).
// `release` hands the row buffer back for refilling. It runs after the first
// phase, whose butterflies have consumed every loaded word: the shared-memory
// loads have then completed, not merely been issued, before the asynchronous
// copy engine (which does not queue behind them) may overwrite the buffer.
template <bool INV, bool FAST, typename Release>
__device__ __forceinline__ void rows_body(const NttArgs &a, const Member &m, uint32_t q, int R, int rho, int g,
                                          uint32_t *ex, const TwLevels &strided, const Tw *tb, uint32_t *v,
                                          Release release) {
  const uint32_t q2 = 2 * q;
  uint32_t *row = ex + rho * kRowStride;
  if constexpr (!INV) {
    ct_radix16_s<FAST>(v, strided, q, q2);
    release();
#pragma unroll
    for (int k = 0; k < 16; k++) row[g + 20 * k] = v[k];
    __syncwarp();  // a row lives in one half-warp
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 w = reinterpret_cast<const uint4 *>(row + 20 * g)[i];
      v[4 * i] = w.x;
      v[4 * i + 1] = w.y;
      v[4 * i + 2] = w.z;
      v[4 * i + 3] = w.w;
    }
    __syncwarp();  // the next member overwrites the row
    ct_radix16_pre<FAST>(v, tb, q, q2);
    const int off = R * kRowWords + 16 * g;
    fwd_rows_finish<FAST>(a, m, q, off, v);
    uint4 *o = reinterpret_cast<uint4 *>(a.dst + (size_t)m.p * a.dst_poly_stride +
                                         (size_t)a.dst_limb[m.l] * kN + off);
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    gs_radix16_pre<FAST>(v, tb, q, q2);
    release();
#pragma unroll
    for (int i = 0; i < 4; i++)
      reinterpret_cast<uint4 *>(row + 20 * g)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = row[g + 20 * k];
    __syncwarp();
    gs_radix16_s<FAST, true>(v, strided, q, q2);
    uint32_t *o = a.dst + (size_t)m.p * a.dst_poly_stride + (size_t)a.dst_limb[m.l] * kN + R * kRowWords + g;
#pragma unroll
    for (int k = 0; k < 16; k++) o[16 * k] = v[k];
  }
}

constexpr size_t kRowsSmem = (size_t)(2 * kRowBufWords + kExWords) * 4 + 240 * sizeof(Tw) + 16;

template <bool INV>
__global__ void __launch_bounds__(kThreads, 3)
    ntt_rows_kernel(const __grid_constant__ NttArgs a, const __grid_constant__ UnitArgs u) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint32_t *rowbuf = reinterpret_cast<uint32_t *>(smem_raw);  // [2][16][kRowPitch]
  uint32_t *ex = rowbuf + 2 * kRowBufWords;                     // [16][kRowStride]
  Tw *tw_s = reinterpret_cast<Tw *>(ex + kExWords);             // levels of 16, 32, 64, 128 twiddles
  uint64_t *full = reinterpret_cast<uint64_t *>(tw_s + 240);
  const int tid = threadIdx.x, rho = tid >> 4, g = tid & 15;
  const int tile = blockIdx.x, unit = blockIdx.y;
  const int R = kTile * tile + rho;
  const int cnt = u.cnt[unit];
  Member m{u.l[unit], u.p0[unit]};
  const uint32_t q = a.q[m.l];
  const Tw *tw = a.table + (size_t)a.g[m.l] * kN;
  pdl_launch_dependents();
  if (tid == 0) {
    mbar_init(smem_u32(&full[0]), 1);
    mbar_init(smem_u32(&full[1]), 1);
    fence_barrier_init();
  }
  __syncthreads();
  // Twiddles do not depend on earlier kernels. The strided phase's 16 groups
  // (256 + R for the tile's rows) go to shared memory, level s as one copy of
  // 16 << s entries; the block phase's 15 thread-owned twiddles to registers.
  if (tid == 0) {
    mbar_expect_tx(smem_u32(&full[0]), kTile * kRowWords * 4 + 240 * sizeof(Tw));
    int off = 0;
#pragma unroll
    for (int s = 0; s < 4; s++) {
      bulk_load(smem_u32(tw_s + off), tw + ((256 + kTile * tile) << s), (uint32_t)((16 << s) * sizeof(Tw)),
                smem_u32(&full[0]));
      off += 16 << s;
    }
  }
  Tw tb[15];
  ld_tw16(tw, 4096 + 16 * R + g, tb);
  TwLevels strided;
  strided.lv[0] = tw_s + rho;
  strided.lv[1] = tw_s + 16 + 2 * rho;
  strided.lv[2] = tw_s + 48 + 4 * rho;
  strided.lv[3] = tw_s + 112 + 8 * rho;
  pdl_wait();
#ifndef CFHE_NO_PROXY_FENCE
  fence_async_all();
#endif
  // a member's tile: the forward pass works in place on dst, the inverse reads src
  auto tile_src = [&](const Member &f) {
    return (INV ? a.src + (size_t)f.p * a.src_poly_stride + (size_t)a.src_limb[f.l] * kN
                : a.dst + (size_t)f.p * a.dst_poly_stride + (size_t)a.dst_limb[f.l] * kN) +
           (size_t)kTile * tile * kRowWords;
  };
  if (tid < 32) {
    Member f = m;
    __syncwarp();  // thread 0's expect_tx above precedes the copies
    if (tid < kTile)
      bulk_load(smem_u32(rowbuf + tid * kRowPitch), tile_src(f) + tid * kRowWords, kRowWords * 4,
                smem_u32(&full[0]));
    if (cnt > 1) {
      next_member(f, a.n_polys);
      if (tid == 0) mbar_expect_tx(smem_u32(&full[1]), kTile * kRowWords * 4);
      __syncwarp();
      if (tid < kTile)
        bulk_load(smem_u32(rowbuf + kRowBufWords + tid * kRowPitch), tile_src(f) + tid * kRowWords,
                  kRowWords * 4, smem_u32(&full[1]));
    }
  }
  Member ahead = m;
  next_member(ahead, a.n_polys);
  const bool fast = q < (1u << 30);
#pragma unroll 1
  for (int i = 0; i < cnt; i++) {
    const int b = i & 1;
    next_member(ahead, a.n_polys);
    mbar_wait(smem_u32(&full[b]), (i >> 1) & 1, u.error_flag);
    const uint32_t *rb = rowbuf + b * kRowBufWords + rho * kRowPitch;
    uint32_t v[16];
    if constexpr (!INV) {
#pragma unroll
      for (int k = 0; k < 16; k++) v[k] = rb[g + 16 * k];
    } else {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const uint4 w = reinterpret_cast<const uint4 *>(rb + 16 * g)[c];
        v[4 * c] = w.x;
        v[4 * c + 1] = w.y;
        v[4 * c + 2] = w.z;
        v[4 * c + 3] = w.w;
      }
    }
    auto release = [&]() {
      if (i + 2 < cnt) {
        fence_async_smem();
        __syncthreads();  // every thread has consumed its words of the buffer
        if (tid < 32) {
          if (tid == 0) mbar_expect_tx(smem_u32(&full[b]), kTile * kRowWords * 4);
          __syncwarp();
          if (tid < kTile)
            bulk_load(smem_u32(rowbuf + b * kRowBufWords + tid * kRowPitch), tile_src(ahead) + tid * kRowWords,
                      kRowWords * 4, smem_u32(&full[b]));
        }
      }
    };
    if (fast)
      rows_body<INV, true>(a, m, q, R, rho, g, ex, strided, tb, v, release);
    else
      rows_body<INV, false>(a, m, q, R, rho, g, ex, strided, tb, v, release);
    next_member(m, a.n_polys);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Tensor map over limbs laid out as [poly][limb][256][256] words, box {16, 256, 1, 1}.
int make_map(CUtensorMap *tm, const uint32_t *base, int n_limb_pos, int n_polys, long long poly_stride) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return -2;
  }
  const cuuint64_t limb_bytes = (cuuint64_t)kN * 4;
  cuuint64_t pstride = (cuuint64_t)poly_stride * 4;
  if (n_polys <= 1 || poly_stride <= 0) {
    n_polys = 1;
    pstride = limb_bytes * (cuuint64_t)n_limb_pos;
  }
  const cuuint64_t dims[4] = {(cuuint64_t)kRowWords, (cuuint64_t)kRowWords, (cuuint64_t)n_limb_pos,
                              (cuuint64_t)n_polys};
  const cuuint64_t strides[3] = {(cuuint64_t)kRowWords * 4, limb_bytes, pstride};
  const cuuint32_t box[4] = {(cuuint32_t)kTile, (cuuint32_t)kRowWords, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, const_cast<uint32_t *>(base), dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return -2;
  }
  return 0;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// false: the call has to take the plain two-pass kernels (operands the
// asynchronous copies cannot address)
bool ntt_tiled_usable(const Context &ctx, const NttArgs &args) {
  // Measured on B200: the pipelined kernels win once a prime's twiddles serve
  // four or more limb transforms and the call is large enough to fill the GPU
  // several times over (16 polynomials x 40 limbs: 158 / 151 us against 195 /
  // 208 us); on the single-ciphertext shapes of HMult (one to three copies of
  // a prime per call) the plain two-pass kernels are 5 to 15 % faster.
  if (ctx.ntt_policy == 1 && (args.n_polys < 4 || args.n_limbs * args.n_polys < 256)) return false;
  if (!aligned16(args.src) || !aligned16(args.dst)) return false;
  if (args.n_polys > 1 && ((args.src_poly_stride & 3) || (args.dst_poly_stride & 3))) return false;
  if (args.n_polys > 1 && (args.src_poly_stride <= 0 || args.dst_poly_stride <= 0)) return false;
  if (args.n_polys > 65535 || args.n_limbs * args.n_polys > 65535) return false;
  if (args.ep_mode && !aligned16(args.ep_src)) return false;
  return true;
}

int launch_ntt_tiled(const Context &ctx, const NttArgs &args, bool inverse) {
  const int total = args.n_limbs * args.n_polys;
  if (total <= 0) return 0;
  static PerDeviceOnce once;
  if (int r = once.run(ctx.device, [] {
        CFHE_CUDA(cudaFuncSetAttribute(ntt_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kRowsSmem));
        CFHE_CUDA(cudaFuncSetAttribute(ntt_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kRowsSmem));
        return 0;
      }))
    return r;
  int max_src = 0, max_dst = 0;
  for (int l = 0; l < args.n_limbs; l++) {
    max_src = args.src_limb[l] > max_src ? args.src_limb[l] : max_src;
    max_dst = args.dst_limb[l] > max_dst ? args.dst_limb[l] : max_dst;
  }
  CUtensorMap tm_src, tm_dst;
  if (int r = make_map(&tm_dst, args.dst, max_dst + 1, args.n_polys, args.dst_poly_stride)) return r;
  if (inverse)
    tm_src = tm_dst;  // the inverse column pass works in place on dst
  else if (int r = make_map(&tm_src, args.src, max_src + 1, args.n_polys, args.src_poly_stride))
    return r;

  // Units: runs of limbs with one prime (adjacent in the list), cut into
  // pieces of at most max_unit limb transforms.
  const int max_unit = ctx.ntt_unit > 0 ? ctx.ntt_unit : 4;
  UnitArgs u;
  u.error_flag = ctx.d_error_flag;
  if (inverse) {
    if (args.n_limbs > kMaxLimbs) {
      set_error("inverse transform: per-limb constants exist for at most 64 limbs");
      return -1;
    }
    for (int l = 0; l < args.n_limbs; l++) {
      const uint32_t q = args.q[l];
      u.kcw[l] = make_tw(mulmod(args.kc[l].w, ctx.inv_w1[args.g[l]], q), q);
    }
  }
  const dim3 block(kThreads);
  int l = 0;
  while (l < args.n_limbs) {
    // one chunk: units until about ntt_chunk limb transforms are collected
    u.n_units = 0;
    int members = 0;
    while (l < args.n_limbs && members < ctx.ntt_chunk) {
      int run = 1;
      if (args.n_polys == 1)  // polynomials of one limb share the prime anyway
        while (l + run < args.n_limbs && args.g[l + run] == args.g[l]) run++;
      const int n = run * args.n_polys;
      const int pieces = (n + max_unit - 1) / max_unit;
      if (u.n_units + pieces > kMaxUnits) {
        if (u.n_units == 0) {
          set_error("ntt: a single prime's limb transforms exceed the unit table");
          return -1;
        }
        break;
      }
      for (int k = 0; k < pieces; k++) {
        const int first = k * max_unit;
        const int c = n - first < max_unit ? n - first : max_unit;
        u.l[u.n_units] = (uint16_t)(l + first / args.n_polys);
        u.p0[u.n_units] = (uint16_t)(first % args.n_polys);
        u.cnt[u.n_units] = (uint8_t)c;
        u.n_units++;
      }
      members += n;
      l += run;
    }
    const dim3 grid(kRowWords / kTile, u.n_units);
    if (inverse) {
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_rows_kernel<true>, grid, block, kRowsSmem, ctx.stream, args, u));
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_cols_kernel<true>, grid, block, 0, ctx.stream, args, u, tm_src,
                              tm_dst));
    } else {
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_cols_kernel<false>, grid, block, 0, ctx.stream, args, u, tm_src,
                              tm_dst));
      CFHE_CUDA(launch_kernel(ctx.use_pdl, ntt_rows_kernel<false>, grid, block, kRowsSmem, ctx.stream, args, u));
    }
  }
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
