// Engine context: parameter set, per-prime device tables, stream, workspace.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <string>
#include <utility>
#include <map>
#include <unordered_map>
#include <vector>

#include "ntt_core.cuh"

namespace cfhe {

constexpr int kMaxLimbs = 64;

constexpr int kMaxJobs = 256;

// One batched transform launch: limb l of polynomial p lives at
// base + p * poly_stride + limb_pos[l] * N (strides in 32-bit words). A launch
// may list up to kMaxJobs limbs (ModUp flattens every digit into one list);
// per-limb constants and the epilogue are available for lists of at most
// kMaxLimbs limbs.
struct NttArgs {
  uint32_t *dst;
  const uint32_t *src;
  const Tw *table;  // forward or inverse twiddles, [num_primes][N]
  long long dst_poly_stride, src_poly_stride;
  int n_limbs, n_polys;
  int premul;   // forward: multiply the input by kc[l] first
  int centred;  // inverse: centred output
  // forward epilogue (ModDown family): out = ((pad*x) - ntt) * scale, x read
  // from ep_src limb ep_limb[l] (255: no such limb, x = 0)
  int ep_mode;  // 0 none, 1 without padding constant, 2 with
  const uint32_t *ep_src;
  long long ep_poly_stride;
  uint8_t g[kMaxJobs];          // global prime index
  uint16_t src_limb[kMaxJobs];  // limb position inside the source polynomial
  uint16_t dst_limb[kMaxJobs];
  uint32_t q[kMaxJobs];
  Tw kc[kMaxLimbs];  // per-limb constant (Shoup pair)
  uint8_t ep_limb[kMaxLimbs];
  Tw ep_pad[kMaxLimbs], ep_scale[kMaxLimbs];
  Tw ep_ps[kMaxLimbs];  // pad * scale, so that the epilogue is pad*scale*x - scale*ntt
};

// One base conversion S -> D with everything its three kernels need.
struct ConvPlan {
  std::vector<int> src_g, dst_g;    // global prime indices
  std::vector<int> src_pos;         // limb positions of S inside the source
  std::vector<uint32_t> pre;        // per source limb: (S_hat_k * N)^-1 (* restored)
  int32_t *d_table = nullptr;       // [nd][ns] centred, device
  uint8_t *d_tc_table = nullptr;    // byte planes in tensor-core operand layout, or null
  int tc_kpad = 0, tc_npad = 0;
  // ModDown-family epilogue, per destination limb
  std::vector<int> ep_pos;          // position of the surviving limb in the source, -1 if restored
  std::vector<uint32_t> ep_pad;     // product of restored primes mod d (plain)
  std::vector<uint32_t> ep_scale;   // (prod S)^-1 mod d (plain)
  bool has_pad = false;
  // the same constants as Shoup pairs, ready for the kernels' argument blocks
  std::vector<Tw> pre_tw;           // pre * 2^-32 (the inverse transform's per-limb constant)
  std::vector<Tw> ep_pad_tw, ep_scale_tw, ep_ps_tw;  // ep_ps = ep_pad * ep_scale
};

struct DigitPlan {
  int index = 0;    // absolute digit number (slot of its ModUp buffer)
  int s0 = 0, s1 = 0;  // limb range inside the level's Q limbs
  ConvPlan conv;    // dst limb positions are those of the (nq+alpha) layout
  std::vector<int> dst_pos;
};

struct LevelPlan {
  int level = 0, num_main = 0, num_ter = 0, alpha = 0, nq = 0, ntot = 0, beta = 0;
  std::vector<int> q_g, full_g;     // global indices of Q limbs / Q+aux limbs
  std::vector<DigitPlan> digits;    // active digits only
  std::vector<int> own_digit;       // per Q limb: index into `digits`
  std::vector<uint32_t> p_mont;     // per Q limb: (P mod q) * 2^32 mod q
  ConvPlan down[3];                 // ModDown, Rescale, ModDownAndRescale
  bool has_rescale = false;
};

struct Context {
  int device = 0;
  int num_sms = 148;  // of `device`, read at context creation
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

  std::vector<uint32_t> nqinv;      // -q^-1 mod 2^32, global order
  bool use_tc_bconv = true;         // base conversion on tcgen05 (CFHE_BCONV=simt disables)
  bool use_fused_lt = true;         // baby steps and plaintext accumulation in one kernel (CFHE_LT=unfused disables)
  bool use_pdl = true;              // programmatic dependent launch between the kernels of a stream (CFHE_PDL=0 disables)
  bool use_twopass_ntt = true;      // two-pass NTT meeting in L2 (CFHE_NTT=cluster selects the cluster kernels)
  // Pipelined NTT (ntt_tiled.cu): 0 never, 1 when the call batches enough limb
  // transforms per prime to amortise its set-up (the default), 2 always
  int ntt_policy = 1;
  int ntt_chunk = 0;                // limb transforms per launch pair, so that the passes meet in L2 (CFHE_NTT_CHUNK)
  int ntt_unit = 0;                 // limb transforms of one prime per CTA (CFHE_NTT_UNIT)
  std::vector<uint32_t> inv_w1;     // per prime: entry 1 of the inverse twiddle table (the last inverse stage's twiddle)
  int *d_error_flag = nullptr;      // raised by a kernel whose bounded wait ran out
  cudaEvent_t order_event = nullptr;  // recorded by cfhe_order_after when this context is the earlier one
  std::vector<LevelPlan> levels;    // index level + 1 (slot 0 = short base)
  // workspace arena for pipeline temporaries (grown on demand)
  uint32_t *ws = nullptr;
  size_t ws_words = 0;

  // Device allocator behind cfhe_malloc / cfhe_free. Requests of 1 MiB and
  // more (polynomials) are carved, best fit, out of slabs of 1 GiB taken from
  // the driver, in units of 256 KiB (one limb at N = 2^16); freed ranges merge
  // with their free neighbours inside a slab. Smaller requests keep a cache
  // of blocks per 4 KiB size class. Either way a freed block goes to a later
  // request without a driver call (cudaMalloc synchronises the device), and
  // since every kernel of this context runs on one stream, the next user's
  // work is ordered after the previous user's. Slabs that are wholly free go
  // back to the driver when an allocation fails and on a stream change;
  // everything does on destroy.
  // cfhe_malloc / cfhe_free may be called from several host threads (a
  // container is freed by whichever thread drops it); the maps are guarded.
  std::mutex pool_mutex;
  std::multimap<size_t, void *> pool_free;            // small classes: size -> block
  std::unordered_map<void *, size_t> pool_live;       // every block handed out -> its rounded size
  std::multimap<size_t, char *> slab_free_by_size;    // free ranges inside slabs
  std::map<char *, size_t> slab_free_by_addr;
  std::map<char *, size_t> slabs;                     // slab start -> bytes
  size_t pool_cached_bytes = 0;

  // optional stage timing: one CUDA event after each pipeline stage
  mutable bool profiling = false;
  mutable std::vector<cudaEvent_t> prof_events;
  mutable std::vector<const char *> prof_names;
  mutable size_t prof_used = 0;
  void mark(const char *stage) const;

  const LevelPlan *plan(int level) const {
    if (level < -1 || level + 1 >= (int)levels.size()) return nullptr;
    return &levels[level + 1];
  }
};

// Kernel attributes (the opt-in to more than 48 KB of dynamic shared memory)
// are per device: a launcher raises them the first time it runs on a device,
// which is the current device of the calling thread at that moment.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  std::mutex mu;
  bool done[kMaxDevices] = {};
  // runs fn() unless it already succeeded on `device`; returns fn's code
  template <typename F>
  int run(int device, F fn) {
    if (device < 0 || device >= kMaxDevices) return -1;
    std::lock_guard<std::mutex> lock(mu);
    if (done[device]) return 0;
    const int r = fn();
    if (r == 0) done[device] = true;
    return r;
  }
};

int build_plans(Context &ctx);
int noalloc_prepare(int device);  // noalloc.cu: materialise the built-in scratch array on the current device
void free_plans(Context &ctx);
int ensure_workspace(Context &ctx, size_t words);

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


// ---- programmatic dependent launch ------------------------------------------
// Kernels of one stream are launched with the programmatic-serialisation
// attribute: a kernel may be scheduled while the previous one drains, runs
// whatever does not depend on earlier kernels (parameter decoding, table
// loads, tensor-memory allocation) and calls pdl_wait() before it reads or
// writes anything an earlier kernel touches. pdl_launch_dependents() at the
// top of a kernel lets its own successor in as soon as all of its CTAs have
// started. Both are no-ops in a kernel launched the ordinary way.
// kernels launched by this library in this process (cfhe_kernel_launch_count)
extern std::atomic<unsigned long long> g_kernel_launches;

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

int launch_ntt(const Context &ctx, const NttArgs &args, bool inverse);
int launch_ntt_twopass(const Context &ctx, const NttArgs &args, bool inverse);
int launch_ntt_tiled(const Context &ctx, const NttArgs &args, bool inverse);
bool ntt_tiled_usable(const Context &ctx, const NttArgs &args);

}  // namespace cfhe
