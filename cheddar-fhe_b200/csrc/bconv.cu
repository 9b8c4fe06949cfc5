// Base conversion (fast basis extension) as an exact integer contraction:
//   out[m][c] = ( sum_k y[k][c] * T[m][k] ) * 2^-32  mod d_m,
// y centred residues of the source basis, T the centred table
// ((prod_{j!=k} s_j) * 2^64 mod d_m), so the result is the M-form of the
// lifted coefficient (reference src/core/ModSwitch.cu:23-171, 320-370).
// The sum is exact in 64 bits with a range fold every four terms; the single
// signed Montgomery reduction at the end returns the canonical residue.
#include "context.h"
#include "kernels.h"
#include "modmath.cuh"

namespace cfhe {
namespace {

constexpr int kBcThreads = 256;
constexpr int kBcLimbsPerBlock = 6;

template <int NS>
__device__ __forceinline__ void bconv_body(const BconvJob &j, int m0, int v) {
  int4 y[NS];
#pragma unroll
  for (int k = 0; k < NS; k++)
    y[k] = reinterpret_cast<const int4 *>(j.src + (size_t)k * kN)[v];
  const int m1 = min(m0 + kBcLimbsPerBlock, j.nd);
  for (int m = m0; m < m1; m++) {
    const uint32_t q = j.q[m], qinv = j.qinv[m];
    const int64_t q32 = (int64_t)((uint64_t)q << 32);
    const int32_t *t = j.table + m * NS;
    int64_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
#pragma unroll
    for (int k = 0; k < NS; k++) {
      const int32_t w = __ldg(t + k);
      a0 += (int64_t)y[k].x * w;
      a1 += (int64_t)y[k].y * w;
      a2 += (int64_t)y[k].z * w;
      a3 += (int64_t)y[k].w * w;
      if ((k & 3) == 3 && k + 1 < NS) {
        // keep |acc| below q*2^31 so four more products cannot overflow
        auto fold = [=](int64_t x) {
          if (x < 0) x += q32;
          if (x >= (q32 >> 1)) x -= q32;
          return x;
        };
        a0 = fold(a0);
        a1 = fold(a1);
        a2 = fold(a2);
        a3 = fold(a3);
      }
    }
    auto fin = [=](int64_t x) {
      if (NS > 2) {  // up to four unfolded products: bring into range
        if (x < 0) x += q32;
        if (x >= (q32 >> 1)) x -= q32;
      }
      return mont_reduce_signed(x, q, qinv);
    };
    reinterpret_cast<uint4 *>(j.dst + (size_t)j.dst_limb[m] * kN)[v] =
        make_uint4(fin(a0), fin(a1), fin(a2), fin(a3));
  }
}

template <int NS>
__global__ void __launch_bounds__(kBcThreads)
    bconv_kernel(const __grid_constant__ BconvArgs a) {
  const BconvJob &j = a.jobs[blockIdx.z];
  if (j.ns != NS) return;
  const int m0 = blockIdx.y * kBcLimbsPerBlock;
  if (m0 >= j.nd) return;
  bconv_body<NS>(j, m0, blockIdx.x * kBcThreads + threadIdx.x);
}

template <int NS>
void launch_ns(const Context &ctx, const BconvArgs &a, int max_nd) {
  dim3 grid(kN / 4 / kBcThreads, (max_nd + kBcLimbsPerBlock - 1) / kBcLimbsPerBlock,
            a.n_jobs);
  bconv_kernel<NS><<<grid, kBcThreads, 0, ctx.stream>>>(a);
}

}  // namespace

int launch_bconv(const Context &ctx, const BconvArgs &a) {
  if (a.n_jobs <= 0) return 0;
  // One launch per distinct source length; blocks of other jobs exit at once.
  bool done[kMaxBconvSrc + 1] = {false};
  for (int i = 0; i < a.n_jobs; i++) {
    const int ns = a.jobs[i].ns;
    if (ns < 1 || ns > kMaxBconvSrc) {
      set_error("bconv: source length must be 1..20");
      return -1;
    }
    if (done[ns]) continue;
    done[ns] = true;
    int max_nd = 0;
    for (int k = 0; k < a.n_jobs; k++)
      if (a.jobs[k].ns == ns && a.jobs[k].nd > max_nd) max_nd = a.jobs[k].nd;
    switch (ns) {
#define CASE(X)                       \
  case X:                             \
    launch_ns<X>(ctx, a, max_nd);     \
    break;
      CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8)
      CASE(9) CASE(10) CASE(11) CASE(12) CASE(13) CASE(14) CASE(15) CASE(16)
      CASE(17) CASE(18) CASE(19) CASE(20)
#undef CASE
    }
    CFHE_CUDA(cudaGetLastError());
  }
  return 0;
}

}  // namespace cfhe
