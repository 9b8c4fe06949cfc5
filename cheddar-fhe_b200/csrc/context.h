// Engine context: parameter set, per-prime device tables, stream, workspace.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>
#include <vector>

#include "ntt_core.cuh"

namespace cfhe {

constexpr int kMaxLimbs = 64;

// One batched transform launch: limb l of polynomial p lives at
// base + p * poly_stride + limb_pos[l] * N (strides in 32-bit words).
struct NttArgs {
  uint32_t *dst;
  const uint32_t *src;
  const Tw *table;  // forward or inverse twiddles, [num_primes][N]
  long long dst_poly_stride, src_poly_stride;
  int n_limbs, n_polys;
  int premul;   // forward: multiply the input by kc[l] first
  int centred;  // inverse: centred output
  uint8_t g[kMaxLimbs];         // global prime index
  uint8_t src_limb[kMaxLimbs];  // limb position inside the source polynomial
  uint8_t dst_limb[kMaxLimbs];
  uint32_t q[kMaxLimbs];
  Tw kc[kMaxLimbs];  // per-limb constant (Shoup pair)
};

struct Context {
  int device = 0;
  int logn = 0, n = 0;
  std::vector<uint32_t> main_primes, ter_primes, aux_primes;
  std::vector<std::pair<int, int>> level_config;  // (num_main, num_ter)
  int add_main = 0, add_ter = 0;
  int T = 0, M = 0, A = 0, L = 0, NP = 0;
  std::vector<uint32_t> q;    // global order: terminal reversed, main, aux
  std::vector<uint32_t> psi;  // primitive 2N-th roots in that order

  Tw *d_tw = nullptr, *d_itw = nullptr;  // [NP][N]
  cudaStream_t stream = nullptr;
  bool own_stream = false;
};

void set_error(const std::string &msg);
const std::string &get_error();

#define CFHE_CUDA(expr)                                                      \
  do {                                                                       \
    cudaError_t _e = (expr);                                                 \
    if (_e != cudaSuccess) {                                                 \
      cfhe::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e));   \
      return -2;                                                             \
    }                                                                        \
  } while (0)

int launch_ntt(const Context &ctx, const NttArgs &args, bool inverse);

}  // namespace cfhe
