// Ciphertext x plaintext RNS GEMM on the 5th-generation tensor cores
// (tcgen05, kind::i8), exact, for sm_100a.
//
//   y_j[l][c] = sum_k W_l[k][j] * x_k[l][c] * 2^-32  mod q_l
//
// for n_in input polynomials x_k, n_out output polynomials y_j, every limb l
// and coefficient c: a projection of encrypted activations (one ciphertext
// polynomial per input feature) by a plaintext weight matrix whose entries
// W_l[k][j] are words in M-form. The result words equal those of a chain of
// Montgomery products and modular additions (cfhe_caccum), which the reference
// would use for it (ElementWiseHandler::CAccum, src/core/ElementWise.cu:1355-1394);
// the reference has no dedicated kernel for this contraction.
//
// Per limb this is a dense GEMM with M = N_poly coefficients, K = n_in and
// N = n_out over Z_q. It is evaluated exactly as an unsigned 8-bit GEMM with
// 32-bit accumulators, the same byte-plane decomposition the base conversion
// uses (bconv_tc.cu):
//
//   D[c][4j+p] = sum_{k,i} byte_i(x_k[c]) * byte_p( W[k][j] * 2^(8i) mod q )
//   V = D0 + D1 2^8 + D2 2^16 + D3 2^24  is congruent to sum_k x_k W[k][j] and
//   below q 2^32 (at most 4 n_in terms of 255 * 255 per accumulator: n_in up
//   to 8192), so one Montgomery reduction finishes an output word.
//
// Operands are packed once per call into the shared-memory operand layout
// (K-major, 8-row x 16-byte core matrices, no swizzle), so that a pipeline
// stage is two contiguous bulk copies:
//   A: activations of one limb, [tile of 128 coefficients][16-byte K chunk][16][8][16]
//      (gemm_pack_kernel, from the limb buffers of the inputs);
//   B: weight byte planes of one limb, [tile of 64 outputs][K step of 64 bytes][4][32][8][16]
//      (built on the host by cfhe_gemm_pack_weights).
// A CTA owns one 128 x 256 accumulator tile in tensor memory (64 outputs of
// 128 coefficients) and walks K in steps of 64 bytes (16 inputs) through a
// four-stage ring: one thread issues the bulk copies, one thread issues the
// MMAs and commits them to the stage's "empty" barrier, four warps run the
// epilogue. Two CTAs share an SM (2 x 256 tensor-memory columns).
//
// Every barrier wait is bounded; a wait that runs out raises the context's
// error flag and the CTA winds down without touching the accumulators.
#include <vector>

#include "context.h"
#include "host_math.h"
#include "kernels.h"
#include "modmath.cuh"

namespace cfhe {
namespace {

constexpr int kGmTile = 128;        // coefficients per CTA (accumulator rows)
constexpr int kGmOutTile = 64;      // outputs per CTA
constexpr int kGmCols = 4 * kGmOutTile;  // accumulator columns
constexpr int kGmStepBytes = 64;    // K bytes per pipeline stage: 16 inputs
constexpr int kGmStages = 4;
constexpr int kGmAStage = kGmTile * kGmStepBytes;   // 8 KiB
constexpr int kGmBStage = kGmCols * kGmStepBytes;   // 16 KiB
constexpr int kGmThreads = 192;     // warps 0-3 epilogue, warp 4 copies, warp 5 MMA
constexpr int kGmSmem = kGmStages * (kGmAStage + kGmBStage) + 128;
constexpr uint32_t kWaitHintNs = 2000;
constexpr uint32_t kSpinLimit = 1u << 20;

struct GemmArgs {
  const uint8_t *xp;          // packed activations of this limb: [N/128][K/16][2048]
  const uint8_t *wp;          // packed weights of this limb: [n_out/64][K/64][16384]
  uint32_t *const *y;         // n_out output polynomials (device table), limb l at y[j] + limb_off
  size_t limb_off;            // word offset of the limb inside an output polynomial
  int k_steps;                // K / 64
  int n_out;                  // outputs that exist (the last tile may be padded)
  uint32_t q, nqinv;
  int *error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;
  return d;
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
// false: the wait ran out
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; i++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
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

__global__ void __launch_bounds__(kGmThreads, 2) gemm_tc_kernel(const __grid_constant__ GemmArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *sA = smem;                               // [stage][4][16][8][16]
  uint8_t *sB = smem + kGmStages * kGmAStage;       // [stage][4][32][8][16]
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kGmStages * (kGmAStage + kGmBStage));
  uint64_t *full = bars, *empty = bars + kGmStages, *accum = bars + 2 * kGmStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kGmStages + 1);
  __shared__ int s_failed;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y;
  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < kGmStages; s++) {
      mbar_init(smem_u32(full + s), 1);
      mbar_init(smem_u32(empty + s), 1);
    }
    mbar_init(smem_u32(accum), 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(kGmCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  pdl_wait();

  if (tid == 4 * 32) {
    // ---- copies: stage s receives K step ks when the MMAs of step ks - kGmStages have left it
    const uint8_t *ap = a.xp + (size_t)m_tile * a.k_steps * kGmAStage;
    const uint8_t *bp = a.wp + (size_t)n_tile * a.k_steps * kGmBStage;
    for (int ks = 0; ks < a.k_steps; ks++) {
      const int s = ks % kGmStages, round = ks / kGmStages;
      if (round > 0 && !mbar_wait(smem_u32(empty + s), (round - 1) & 1)) {
        atomicExch(a.error_flag, 1);
        atomicExch(&s_failed, 1);
        break;
      }
      mbar_expect_tx(smem_u32(full + s), kGmAStage + kGmBStage);
      bulk_load(smem_u32(sA + s * kGmAStage), ap + (size_t)ks * kGmAStage, kGmAStage, smem_u32(full + s));
      bulk_load(smem_u32(sB + s * kGmBStage), bp + (size_t)ks * kGmBStage, kGmBStage, smem_u32(full + s));
    }
  } else if (tid == 5 * 32) {
    // ---- MMAs: D (128 x 256, s32) += A (128 x 64 u8) * B (64 x 256 u8) per stage, as two K = 32 instructions
    const uint32_t idesc = (2u << 4) | ((uint32_t)(kGmCols >> 3) << 17) | ((uint32_t)(kGmTile >> 4) << 24);
    constexpr uint32_t a_lbo = (kGmTile / 8) * 128, b_lbo = (kGmCols / 8) * 128;
    bool ok = true;
    for (int ks = 0; ks < a.k_steps && ok; ks++) {
      const int s = ks % kGmStages, round = ks / kGmStages;
      if (!mbar_wait(smem_u32(full + s), round & 1)) {
        atomicExch(a.error_flag, 1);
        atomicExch(&s_failed, 1);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const uint64_t da = smem_desc(smem_u32(sA + s * kGmAStage) + h * 2 * a_lbo, a_lbo, 128);
        const uint64_t db = smem_desc(smem_u32(sB + s * kGmBStage) + h * 2 * b_lbo, b_lbo, 128);
        const uint32_t acc = (ks > 0 || h > 0) ? 1u : 0u;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem),
            "l"(da), "l"(db), "r"(idesc), "r"(acc)
            : "memory");
      }
      // the stage is free again once these MMAs have read it
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                       smem_u32(empty + s))
                   : "memory");
    }
    // accumulators complete (also on failure, so that the epilogue warps wake up)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(accum))
                 : "memory");
  } else if (warp < 4) {
    // ---- epilogue: thread = coefficient, 8 outputs (32 columns) per tensor-memory load
    const bool arrived = mbar_wait(smem_u32(accum), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!arrived) atomicExch(a.error_flag, 1);
    if (arrived && !*(volatile int *)&s_failed) {
      const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
      const size_t col = a.limb_off + (size_t)m_tile * kGmTile + tid;
      const uint32_t q = a.q, nq = a.nqinv;
#pragma unroll 1
      for (int j0 = 0; j0 < kGmOutTile; j0 += 8) {
        uint32_t d[32];
        tmem_ld32(lane_base + 4 * j0, d);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const int j = n_tile * kGmOutTile + j0 + e;
          if (j < a.n_out) {
            // V = d0 + d1 2^8 + d2 2^16 + d3 2^24, every d below 2^31
            const uint64_t v = (uint64_t)d[4 * e] + ((uint64_t)d[4 * e + 1] << 8) +
                               ((uint64_t)d[4 * e + 2] << 16) + ((uint64_t)d[4 * e + 3] << 24);
            a.y[j][col] = mont_reduce(v, q, nq);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGmCols) : "memory");
}

// Packs the limb `limb_off` of n_in input polynomials into the A operand
// layout: thread = (coefficient, 16-byte K chunk of four inputs). Inputs past
// n_in are zero.
__global__ void __launch_bounds__(256) gemm_pack_kernel(uint8_t *xp, const uint32_t *const *x, size_t limb_off,
                                                        int n_in, int k_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int k = 4 * t + i;
    w[i] = k < n_in ? x[k][limb_off + c] : 0u;
  }
  uint8_t *tile = xp + ((size_t)(c >> 7) * k_chunks + t) * (kGmTile * 16);
  *reinterpret_cast<uint4 *>(tile + ((c & 127) >> 3) * 128 + (c & 7) * 16) = make_uint4(w[0], w[1], w[2], w[3]);
}

}  // namespace

size_t gemm_packed_weight_bytes(int n_in, int n_out) {
  const int k_steps = (4 * n_in + kGmStepBytes - 1) / kGmStepBytes;
  const int n_tiles = (n_out + kGmOutTile - 1) / kGmOutTile;
  return (size_t)n_tiles * k_steps * kGmBStage;
}

// Byte planes of one limb's weights in the B operand layout. w: [n_in][n_out]
// words in M-form (below q).
void gemm_pack_weights_limb(uint8_t *out, const uint32_t *w, int n_in, int n_out, uint32_t q) {
  const int k_steps = (4 * n_in + kGmStepBytes - 1) / kGmStepBytes;
  const size_t total = gemm_packed_weight_bytes(n_in, n_out);
  memset(out, 0, total);
  uint32_t shift[4];
  for (int i = 0; i < 4; i++) shift[i] = (uint32_t)((1ull << (8 * i)) % q);
  for (int k = 0; k < n_in; k++)
    for (int j = 0; j < n_out; j++) {
      const uint32_t base = w[(size_t)k * n_out + j] % q;
      const int n_tile = j / kGmOutTile, jn = j % kGmOutTile;
      for (int i = 0; i < 4; i++) {
        const uint32_t v = mulmod(base, shift[i], q);
        const int kappa = 4 * k + i;  // K byte index
        const int ks = kappa / kGmStepBytes, kk = kappa % kGmStepBytes;
        uint8_t *stage = out + ((size_t)n_tile * k_steps + ks) * kGmBStage;
        for (int p = 0; p < 4; p++) {
          const int n = 4 * jn + p;  // accumulator column
          stage[(size_t)(kk >> 4) * (kGmCols / 8) * 128 + (n >> 3) * 128 + (n & 7) * 16 + (kk & 15)] =
              (uint8_t)(v >> (8 * p));
        }
      }
    }
}

// x, y: device tables of n_in / n_out polynomial pointers ([n_limbs][N] words
// each); wp: packed weights, limb after limb; scratch: one limb of packed
// activations (gemm_scratch_bytes).
size_t gemm_scratch_bytes(int n_in) {
  const int k_steps = (4 * n_in + kGmStepBytes - 1) / kGmStepBytes;
  return (size_t)(kN / kGmTile) * k_steps * kGmAStage;
}

int launch_ctpt_gemm(const Context &c, uint32_t *const *y, const uint32_t *const *x, const uint8_t *wp,
                     uint8_t *scratch, int n_in, int n_out, const int *gidx, int n_limbs) {
  static PerDeviceOnce once;
  if (int r = once.run(c.device, [] {
        CFHE_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGmSmem));
        return 0;
      }))
    return r;
  if (n_in < 1 || n_in > 8192 || n_out < 1) {
    set_error("ct-pt GEMM: 1 to 8192 inputs, at least one output");
    return -1;
  }
  const int k_steps = (4 * n_in + kGmStepBytes - 1) / kGmStepBytes;
  const int n_tiles = (n_out + kGmOutTile - 1) / kGmOutTile;
  const size_t w_limb = gemm_packed_weight_bytes(n_in, n_out);
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) {
      set_error("prime index out of range");
      return -1;
    }
    const size_t limb_off = (size_t)l * kN;
    CFHE_CUDA(launch_kernel(c.use_pdl, gemm_pack_kernel, dim3(kN / 256, 4 * k_steps), dim3(256), 0, c.stream,
                            scratch, x, limb_off, n_in, 4 * k_steps));
    GemmArgs a;
    a.xp = scratch;
    a.wp = wp + (size_t)l * w_limb;
    a.y = y;
    a.limb_off = limb_off;
    a.k_steps = k_steps;
    a.n_out = n_out;
    a.q = c.q[gidx[l]];
    a.nqinv = c.nqinv[gidx[l]];
    a.error_flag = c.d_error_flag;
    CFHE_CUDA(launch_kernel(c.use_pdl, gemm_tc_kernel, dim3(n_tiles, kN / kGmTile), dim3(kGmThreads), kGmSmem,
                            c.stream, a));
  }
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
