// Base conversion on the 5th-generation tensor cores (tcgen05, kind::i8),
// exact, for sm_100a.
//
// The conversion  out[m][c] = ( sum_k y_c[k][c] * T[m][k] ) * 2^-32 mod p_m
// (reference src/core/ModSwitch.cu:23-171) is a dense contraction over the
// source limbs k. It is evaluated as one unsigned 8-bit GEMM per tile of 128
// coefficients:
//
//   D[c][4m+j] = sum_{k,i} byte_i(y[k][c]) * byte_j( T[m][k] * 2^(8i) mod p_m )
//
//   A (128 x K, K = 4*(ns+1) bytes): one pseudo source "number of residues
//      above s_k/2" in word 0, then the canonical residues y[k][c] in [0,s_k)
//      exactly as they sit in memory (little-endian words are their own byte
//      planes). Words past the last source are zero, and so are their
//      table rows;
//   B (N x K, N = 4*nd): byte planes of the table entries pre-multiplied by
//      2^(8i), and for the pseudo source the byte planes of -(prod s)*2^64
//      mod p_m, which turns the canonical residues back into the centred
//      ones the reference convention prescribes;
//   D (int32, in tensor memory): every sum has at most 84 terms of at most
//      255*255, so it is exact.
//
// The epilogue reads a thread's row of D from tensor memory, recombines the
// four planes V = D0 + D1*2^8 + D2*2^16 + D3*2^24 (V < 2^47, congruent to the
// centred sum mod p_m) and applies one Montgomery reduction, which returns the
// same canonical word as the reference's signed reduction of the centred sum.
//
// Waits on the MMA completion barrier are bounded; on a timeout the kernel
// raises a flag in global memory, frees its tensor memory and returns.
#include <stdlib.h>
#include <string.h>

#include "context.h"
#include "host_math.h"
#include "kernels.h"
#include "modmath.cuh"

namespace cfhe {
namespace {

constexpr int kTcThreads = 128;  // one thread per coefficient of the tile
// A CTA is kTcGroups independent groups of 128 threads, one CTA per SM: each
// group owns an operand tile, a table slice, a completion barrier and 64
// columns of the CTA's tensor memory and walks its own tiles. (Measured: an SM
// admits a new CTA of the one-group form of this kernel only about every 2 us,
// so a grid of a thousand small CTAs spent two thirds of its time ramping up.)
constexpr int kTcGroups = 7;
constexpr int kTcCtaThreads = kTcThreads * kTcGroups;
constexpr int kTcTile = 128;
constexpr int kTcMaxK = 96;      // bytes of K per tile row: 4 * (20 + 1) padded to 32
constexpr int kTcSliceN = 64;    // accumulator columns per CTA: 16 destination limbs
constexpr int kTmemCols = 64;        // per group
constexpr int kTmemAlloc = 512;      // per CTA: power of two >= kTcGroups * kTmemCols
// A waiting warp sleeps in the barrier unit for up to kWaitHintNs per attempt
// instead of spending issue slots on polling; kSpinLimit attempts bound the wait.
constexpr uint32_t kWaitHintNs = 2000;
constexpr uint32_t kSpinLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// K-major, no swizzle: 8-row x 16-byte core matrices; lbo = bytes between the
// two 16-byte K chunks of one MMA, sbo = bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  return d;
}

// barrier among the 128 threads of one group (id 0 is __syncthreads)
__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(kTcThreads) : "memory");
}

// the same barrier, returning whether any of the 128 threads passed a true predicate
__device__ __forceinline__ bool group_sync_or(int group, bool pred) {
  uint32_t any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any)
      : "r"(group + 1), "n"(kTcThreads), "r"((uint32_t)pred)
      : "memory");
  return any != 0;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// KCH = 16-byte chunks of K per operand row (K = 16 * KCH bytes, 4 * KCH words:
// the pseudo source and up to 4 * KCH - 1 residues). One group walks its tiles;
// for every tile the operand rows are built once and every slice of 16
// destination limbs is then converted in turn on the group's 64 accumulator
// columns.
template <int KCH>
__device__ __forceinline__ void tc_tiles(const BconvTcArgs &a, const BconvTcJob &j, uint8_t *sA,
                                         const uint8_t *sB, uint64_t *bar, const uint4 *s_lim,
                                         uint32_t tmem, int group, int first_tile, int tile_step) {
  constexpr int kWords = 4 * KCH;
  const int tid = threadIdx.x & (kTcThreads - 1), warp = tid >> 5;
  // instruction descriptor: D = s32, A = B = u8, both K-major, M = 128, N = 64
  const uint32_t idesc =
      (2u << 4) | ((uint32_t)(kTcSliceN >> 3) << 17) | ((uint32_t)(kTcTile >> 4) << 24);
  constexpr uint32_t a_lbo = (kTcTile / 8) * 128;
  const uint32_t b_lbo = (uint32_t)(j.npad / 8) * 128;  // the table keeps all its slices
  const int n_slices = j.npad / kTcSliceN;
  uint32_t parity = 0;
  bool failed = false;

  // Residues of one coefficient. The loads of the next tile are issued before
  // the wait on the tensor core and the epilogue of the current one and are
  // not touched until the next iteration, so their latency hides behind that
  // work. Words past the last source stay zero (their table rows are zero).
  uint32_t yn[kWords - 1];
  const uint32_t *src = j.src + tid;
  // everything above (table, constants, tensor memory) did not depend on
  // earlier kernels; the residues do
  pdl_wait();
  auto load_tile = [&](int tile) {
    const uint32_t *p = src + tile * kTcTile;
#pragma unroll
    for (int k = 0; k < kWords - 1; k++) yn[k] = k < j.ns ? __ldg(p + (size_t)k * kN) : 0u;
  };
  if (first_tile < kN / kTcTile) load_tile(first_tile);

  for (int tile = first_tile; tile < kN / kTcTile && !failed; tile += tile_step) {
    const int col = tile * kTcTile + tid;
    // 1. operand row: [count of residues above half their prime, residues...]
    uint32_t w[kWords];
    uint32_t nneg = 0;
#pragma unroll
    for (int k = 0; k < kWords - 1; k++) {
      w[k + 1] = yn[k];
      nneg += yn[k] > j.half[k];  // half[k >= ns] = 2^32 - 1
    }
    w[0] = nneg;
#pragma unroll
    for (int t = 0; t < KCH; t++)
      *reinterpret_cast<uint4 *>(sA + t * a_lbo + (tid >> 3) * 128 + (tid & 7) * 16) =
          make_uint4(w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    group_sync(group);
    for (int slice = 0; slice < n_slices && !failed; slice++) {
      // 2. one thread issues the MMAs of this slice and commits them to the barrier
      if (tid == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int ks = 0; ks < KCH / 2; ks++) {
          const uint64_t da = smem_desc(smem_u32(sA) + ks * 2 * a_lbo, a_lbo, 128);
          const uint64_t db = smem_desc(
              smem_u32(sB) + ks * 2 * b_lbo + (uint32_t)slice * (kTcSliceN / 8) * 128, b_lbo, 128);
          const uint32_t acc = ks > 0;
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "setp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
              ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc)
              : "memory");
        }
        asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                smem_u32(bar))
            : "memory");
      }
      // the next tile's residues travel while the tensor core and the epilogues run
      if (slice == 0 && tile + tile_step < kN / kTcTile) load_tile(tile + tile_step);
      // 3. wait for the accumulators (bounded)
      uint32_t spins = 0;
      while (!mbar_try_wait(smem_u32(bar), parity)) {
        if (++spins > kSpinLimit) {
          failed = true;
          break;
        }
      }
      parity ^= 1;
      if (__any_sync(0xffffffffu, failed)) {
        failed = true;  // this warp skips the epilogue of the slice
        if (a.error_flag && (tid & 31) == 0) atomicExch(a.error_flag, 1);
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // 4. epilogue: 8 destination limbs (32 accumulator columns) per load
      if (!failed) {
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        const int m_count = min(j.nd - slice * (kTcSliceN / 4), kTcSliceN / 4);
        const uint4 *lims = s_lim + slice * (kTcSliceN / 4);
        uint32_t *out = j.dst + col;
#pragma unroll
        for (int m0 = 0; m0 < kTcSliceN / 4; m0 += 8) {
          if (m0 < m_count) {
            uint32_t d[32];
            tmem_ld32(lane_base + 4 * m0, d);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 8; e++) {
              const uint4 lim = lims[m0 + e];
              // V = d0 + d1*2^8 + d2*2^16 + d3*2^24; every d < 2^23, so the two
              // 16-bit-apart halves fit 32 bits and one wide multiply-add joins them
              const uint32_t lo = d[4 * e + 1] * 256u + d[4 * e];
              const uint32_t hi = d[4 * e + 3] * 256u + d[4 * e + 2];
              const uint64_t v = (uint64_t)hi * 65536u + lo;
              const uint32_t r = mont_reduce(v, lim.x, lim.y);
              if (lim.w) out[lim.z] = r;
            }
          }
        }
      }
      // the accumulators (and, after the last slice, the operand tile) are reused
      // A wait that ran out is a decision of the whole group: the barrier that
      // ends the slice also ORs the warps' flags, so all four warps leave the
      // loops together (a warp leaving alone would starve the next barrier).
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      failed = group_sync_or(group, failed);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
  }
}

constexpr int kTcMaxSlices = 4;  // 64 destination limbs
// shared memory: the whole table of the CTA's job (all slices), the per-limb
// constants, then per group an operand tile (12 KB) and a completion barrier
constexpr int kTcTableBytes = kTcMaxK * kTcSliceN * kTcMaxSlices;        // 24 KB
constexpr int kTcLimBytes = 16 * (kTcSliceN / 4) * kTcMaxSlices;          // 1 KB
constexpr int kTcGroupSmem = kTcMaxK * kTcTile + 128;
// Asked for: more than half of an SM's shared memory, so two of these CTAs
// never share an SM and the tensor-memory allocation below cannot wait on
// another CTA.
constexpr int kTcUsedSmem = kTcTableBytes + kTcLimBytes + kTcGroups * kTcGroupSmem + 16;
constexpr int kTcSmemBytes = kTcUsedSmem > 120 * 1024 ? kTcUsedSmem : 120 * 1024;
static_assert(kTcSmemBytes > 116 * 1024, "one CTA per SM is what keeps the allocation from blocking");
static_assert(kTcGroups * kTmemCols <= kTmemAlloc, "tensor memory columns");

__global__ void __launch_bounds__(kTcCtaThreads, 1)
    bconv_tc_kernel(const __grid_constant__ BconvTcArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  const int group = threadIdx.x / kTcThreads;
  // a.per_unit CTAs share the tiles of one job; every group of a CTA takes its own tiles
  const int job = blockIdx.x / a.per_unit, cta_in_job = blockIdx.x - job * a.per_unit;
  const BconvTcJob &j = a.jobs[job];
  const int first_tile = cta_in_job * kTcGroups + group, tile_step = a.per_unit * kTcGroups;
  uint8_t *sB = smem;  // [K/16][npad/8][8][16]: the job's table as it lies in memory
  // per destination limb: {q, -q^-1, word offset of the limb, in range}
  uint4 *s_lim = reinterpret_cast<uint4 *>(smem + kTcTableBytes);
  uint8_t *gs = smem + kTcTableBytes + kTcLimBytes + group * kTcGroupSmem;
  uint8_t *sA = gs;    // [K/16][16][8][16]
  uint64_t *bar = reinterpret_cast<uint64_t *>(gs + kTcMaxK * kTcTile);
  uint32_t *tmem_slot =
      reinterpret_cast<uint32_t *>(smem + kTcTableBytes + kTcLimBytes + kTcGroups * kTcGroupSmem);
  const int kbytes = j.kpad;

  for (int i = threadIdx.x; i < kbytes * j.npad / 16; i += kTcCtaThreads)
    reinterpret_cast<uint4 *>(sB)[i] = reinterpret_cast<const uint4 *>(j.btile)[i];
  if ((int)threadIdx.x < j.npad / 4) {
    const int m = threadIdx.x;
    s_lim[m] = m < j.nd ? make_uint4(j.q[m], j.nqinv[m], (uint32_t)j.dst_limb[m] * kN, 1u)
                        : make_uint4(3u, 1u, 0u, 0u);
  }
  if ((threadIdx.x & (kTcThreads - 1)) == 0) mbar_init(smem_u32(bar), 1);
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemAlloc)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_cta = *tmem_slot;
  const uint32_t tmem = tmem_cta + (uint32_t)(group * kTmemCols);

  if (kbytes == 32)
    tc_tiles<2>(a, j, sA, sB, bar, s_lim, tmem, group, first_tile, tile_step);
  else if (kbytes == 64)
    tc_tiles<4>(a, j, sA, sB, bar, s_lim, tmem, group, first_tile, tile_step);
  else
    tc_tiles<6>(a, j, sA, sB, bar, s_lim, tmem, group, first_tile, tile_step);

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_cta),
                 "r"(kTmemAlloc)
                 : "memory");
}

}  // namespace

// Builds the B operand of one conversion in shared-memory operand layout.
int build_tc_table(const Context &c, ConvPlan &cv) {
  const int ns = (int)cv.src_g.size(), nd = (int)cv.dst_g.size();
  if (ns > kMaxBconvSrc) return 0;  // handled by the SIMT kernel only
  const int kpad = ((4 * (ns + 1) + 31) / 32) * 32;
  const int npad = ((4 * nd + kTcSliceN - 1) / kTcSliceN) * kTcSliceN;
  if (kpad > kTcMaxK) return 0;
  std::vector<uint8_t> tile((size_t)kpad * npad, 0);
  const uint32_t b_lbo = (uint32_t)(npad / 8) * 128;
  auto put = [&](int n, int kappa, uint8_t v) {
    tile[(size_t)(kappa >> 4) * b_lbo + (n >> 3) * 128 + (n & 7) * 16 + (kappa & 15)] = v;
  };
  for (int m = 0; m < nd; m++) {
    const uint32_t p = c.q[cv.dst_g[m]];
    uint32_t s_all = 1;
    for (int k = 0; k < ns; k++) s_all = mulmod(s_all, c.q[cv.src_g[k]] % p, p);
    for (int k = 0; k <= ns; k++) {
      uint32_t t;
      if (k < ns) {
        t = 1;
        for (int i = 0; i < ns; i++)
          if (i != k) t = mulmod(t, c.q[cv.src_g[i]] % p, p);
      } else {
        t = s_all ? p - s_all : 0;  // -(prod s) mod p for the pseudo source
      }
      t = to_mont(to_mont(t, p), p);
      // K layout: word 0 = pseudo source, word k + 1 = source k
      const int word = k < ns ? k + 1 : 0;
      for (int i = 0; i < (k < ns ? 4 : 1); i++) {
        const uint32_t ti = mulmod(t, (uint32_t)((1ull << (8 * i)) % p), p);
        for (int jj = 0; jj < 4; jj++) put(4 * m + jj, 4 * word + i, (uint8_t)(ti >> (8 * jj)));
      }
    }
  }
  CFHE_CUDA(cudaMalloc(&cv.d_tc_table, tile.size()));
  CFHE_CUDA(cudaMemcpy(cv.d_tc_table, tile.data(), tile.size(), cudaMemcpyHostToDevice));
  cv.tc_kpad = kpad;
  cv.tc_npad = npad;
  return 0;
}


int launch_bconv_tc(const Context &ctx, const BconvTcArgs &a) {
  static PerDeviceOnce once;
  if (int r = once.run(ctx.device, [] {
        CFHE_CUDA(cudaFuncSetAttribute(bconv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kTcSmemBytes));
        return 0;
      }))
    return r;
  if (a.n_jobs <= 0) return 0;
  for (int i = 0; i < a.n_jobs; i++)
    if (a.jobs[i].npad > kTcSliceN * kTcMaxSlices || a.jobs[i].kpad > kTcMaxK) {
      set_error("bconv: conversion too wide for the tensor-core kernel");
      return -1;
    }
  // one CTA per SM; the CTAs are shared out evenly over the jobs, and the
  // kTcGroups groups of a CTA interleave over its job's tiles
  BconvTcArgs b = a;
  int per_job = ctx.num_sms / a.n_jobs;
  const int enough = (kN / kTcTile + kTcGroups - 1) / kTcGroups;
  if (per_job < 1) per_job = 1;
  if (per_job > enough) per_job = enough;
  b.per_unit = per_job;
  CFHE_CUDA(launch_kernel(ctx.use_pdl, bconv_tc_kernel, dim3(per_job * a.n_jobs), dim3(kTcCtaThreads),
                          kTcSmemBytes, ctx.stream, b));
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
