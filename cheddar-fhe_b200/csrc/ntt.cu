// Cluster NTT / INTT kernels for sm_100a: one 8-CTA thread-block cluster per
// limb, one HBM read and one HBM write per word; the 256x256 transposition
// between the row-pairing and the in-row stages goes through distributed
// shared memory. The per-thread phases live in ntt_core.cuh.
#include <cooperative_groups.h>

#include "context.h"

namespace cg = cooperative_groups;

namespace cfhe {
namespace {

// Split cluster barrier: every CTA arrives as soon as it starts and waits only
// right before its first store into a peer's shared memory, which is all the
// residency guarantee needs; the second phase orders those stores before the
// peers read them.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

struct RemoteBuf {
  cg::cluster_group cluster;
  uint32_t *local;
  __device__ __forceinline__ uint32_t *operator()(int rank) const {
    return cluster.map_shared_rank(local, rank);
  }
};

template <bool FAST>
__device__ __forceinline__ void forward_body(const NttArgs &a, int c, int tid,
                                             int p, int l, const uint32_t *src,
                                             uint32_t *dst, const Tw *tw,
                                             uint32_t q, uint32_t *xbuf,
                                             uint32_t *rbuf) {
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t q2 = 2 * q;
  uint32_t v[16];
  {
    const int x = tid & 31, r0 = tid >> 5;
    const uint32_t *p = src + r0 * kRowWords + kStripCols * c + x;
#pragma unroll
    for (int k = 0; k < 16; k++) v[k] = p[k * 16 * kRowWords];
    if (a.premul) {
      const Tw kc = a.kc[l];
#pragma unroll
      for (int k = 0; k < 16; k++) v[k] = shoup_mul(v[k], kc, q);
    }
  }
  fwd_rows_a<FAST>(v, tid, xbuf, tw, q, q2);
  __syncthreads();
  cluster_wait_acquire();  // peers are resident (arrival at kernel entry)
  fwd_rows_b<FAST>(c, tid, xbuf, RemoteBuf{cluster, rbuf}, tw, q, q2);
  cluster_arrive_release();
  cluster_wait_acquire();
  fwd_cols_a<FAST>(c, tid, rbuf, rbuf, tw, q, q2);
  // a row's 16 column groups live in one half-warp: in-place, warp-level exchange
  __syncwarp();
  fwd_cols_b<FAST>(v, c, tid, rbuf, tw, q, q2);
  {
    const int rho = tid >> 4, g = tid & 15, R = kOwnRows * c + rho;
    const int off = R * kRowWords + 16 * g;
    if (a.ep_mode) {
      // ModDown-family epilogue: ((pad * x) - ntt) * scale, canonical
      const Tw scale = a.ep_scale[l];
      uint32_t x[16];
      if (a.ep_limb[l] != 255) {
        const uint4 *xp = reinterpret_cast<const uint4 *>(
            a.ep_src + (size_t)p * a.ep_poly_stride +
            (size_t)a.ep_limb[l] * kN + off);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const uint4 t = xp[i];
          x[4 * i] = t.x;
          x[4 * i + 1] = t.y;
          x[4 * i + 2] = t.z;
          x[4 * i + 3] = t.w;
        }
        if (a.ep_mode == 2) {
          const Tw pad = a.ep_pad[l];
#pragma unroll
          for (int k = 0; k < 16; k++) {
            const uint32_t t = shoup_mul(x[k], pad, q);
            x[k] = umin32(t, t - q);
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < 16; k++) x[k] = 0;
      }
#pragma unroll
      for (int k = 0; k < 16; k++) {
        uint32_t d = x[k] - v[k];
        if (x[k] < v[k]) d += q;
        d = shoup_mul(d, scale, q);
        v[k] = umin32(d, d - q);
      }
    }
    uint4 *o = reinterpret_cast<uint4 *>(dst + off);
#pragma unroll
    for (int i = 0; i < 4; i++)
      o[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
}

template <bool FAST>
__device__ __forceinline__ void inverse_body(const NttArgs &a, int c, int tid,
                                             int l, const uint32_t *src,
                                             uint32_t *dst, const Tw *itw,
                                             uint32_t q, uint32_t *xbuf,
                                             uint32_t *rbuf) {
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t q2 = 2 * q;
  uint32_t v[16];
  {
    const int rho = tid >> 4, g = tid & 15, R = kOwnRows * c + rho;
    const uint4 *p =
        reinterpret_cast<const uint4 *>(src + R * kRowWords + 16 * g);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint4 t = p[i];
      v[4 * i] = t.x;
      v[4 * i + 1] = t.y;
      v[4 * i + 2] = t.z;
      v[4 * i + 3] = t.w;
    }
  }
  inv_cols_a<FAST>(v, c, tid, xbuf, itw, q, q2);
  __syncwarp();
  cluster_wait_acquire();  // peers are resident (arrival at kernel entry)
  inv_cols_b<FAST>(c, tid, xbuf, RemoteBuf{cluster, rbuf}, itw, q, q2);
  cluster_arrive_release();
  cluster_wait_acquire();
  inv_rows_a<FAST>(tid, rbuf, xbuf, itw, q, q2);
  __syncthreads();
  inv_rows_b<FAST>(v, tid, xbuf, itw, a.kc[l], a.centred != 0, q, q2);
  {
    const int x = tid & 31, r0 = tid >> 5;
    uint32_t *o = dst + r0 * kRowWords + kStripCols * c + x;
#pragma unroll
    for (int k = 0; k < 16; k++) o[k * 16 * kRowWords] = v[k];
  }
}

template <bool INV>
__global__ void __cluster_dims__(kClusterSize, 1, 1)
    __launch_bounds__(kNttThreads, 3)
        ntt_cluster_kernel(const __grid_constant__ NttArgs a) {
  extern __shared__ __align__(16) uint32_t smem[];
  // forward: xbuf strip layout, rbuf in-row layout; inverse: xbuf holds the
  // in-row layout first and the strip layout later, rbuf the strip layout
  uint32_t *xbuf = smem;
  uint32_t *rbuf = smem + (INV ? kRowBufWords : kStripBufWords);
  cluster_arrive_relaxed();
  const int c = blockIdx.x;  // rank inside the cluster (gridDim.x == 8)
  const int tid = threadIdx.x;
  const int t = blockIdx.y;
  const int p = t / a.n_limbs;
  const int l = t - p * a.n_limbs;
  const uint32_t q = a.q[l];
  const Tw *tw = a.table + (size_t)a.g[l] * kN;
  const uint32_t *src =
      a.src + (size_t)p * a.src_poly_stride + (size_t)a.src_limb[l] * kN;
  uint32_t *dst =
      a.dst + (size_t)p * a.dst_poly_stride + (size_t)a.dst_limb[l] * kN;
  if (q < (1u << 30)) {
    if constexpr (INV)
      inverse_body<true>(a, c, tid, l, src, dst, tw, q, xbuf, rbuf);
    else
      forward_body<true>(a, c, tid, p, l, src, dst, tw, q, xbuf, rbuf);
  } else {
    if constexpr (INV)
      inverse_body<false>(a, c, tid, l, src, dst, tw, q, xbuf, rbuf);
    else
      forward_body<false>(a, c, tid, p, l, src, dst, tw, q, xbuf, rbuf);
  }
}

}  // namespace

int launch_ntt(const Context &ctx, const NttArgs &args, bool inverse) {
  if (ctx.ntt_policy && ntt_tiled_usable(ctx, args)) return launch_ntt_tiled(ctx, args, inverse);
  if (ctx.use_twopass_ntt) return launch_ntt_twopass(ctx, args, inverse);
  static PerDeviceOnce once;
  if (int r = once.run(ctx.device, [] {
        CFHE_CUDA(cudaFuncSetAttribute(ntt_cluster_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kNttSmemBytes));
        CFHE_CUDA(cudaFuncSetAttribute(ntt_cluster_kernel<true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kNttSmemBytes));
        return 0;
      }))
    return r;
  const int total = args.n_limbs * args.n_polys;
  if (total <= 0) return 0;
  if (total > 65535) {
    set_error("ntt: more than 65535 limb transforms in one call");
    return -1;
  }
  dim3 grid(kClusterSize, total), block(kNttThreads);
  if (inverse)
    ntt_cluster_kernel<true><<<grid, block, kNttSmemBytes, ctx.stream>>>(args);
  else
    ntt_cluster_kernel<false><<<grid, block, kNttSmemBytes, ctx.stream>>>(args);
  CFHE_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace cfhe
