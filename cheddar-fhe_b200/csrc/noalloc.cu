// ModDown / Rescale / ModDownAndRescale of ONE polynomial with no device
// allocation anywhere on the call path.
//
// Who needs this: host programs that have handed all device memory to an
// allocator of their own (a serving process whose framework reserves the whole
// GPU at start-up leaves nothing for a library's cudaMalloc to find), and
// latency-sensitive loops that cannot accept the device-wide synchronisation a
// cudaMalloc / cudaFree implies. The regular cfhe_moddown() keeps its
// inverse-transform output in the context's workspace arena, which is grown
// with cudaMalloc when a call needs more than any earlier one did. This
// variant keeps that intermediate in a fixed array that is part of the
// library image instead, so nothing is ever allocated or freed.
//
// Cost and limits: the array is kNoAllocMaxSrcLimbs limbs of 2^16 words
// (16 x 256 KiB = 4 MiB). Every GPU on which the library's kernels are loaded
// holds its own copy of it until the process exits, used or not. Conversions
// that drop more than kNoAllocMaxSrcLimbs limbs are refused.
//
// Sharing: all calls on a device use the same array. It keeps whatever the
// previous call left there; that is harmless here because the inverse
// transform overwrites every word the base conversion later reads, so nothing
// has to be cleared. Two calls that are in flight on the GPU at the same time
// (different streams, different contexts, different host threads) would
// overwrite each other's intermediate: callers must order them.
#include <mutex>

#include "../../include/cheddar_b200.h"
#include "handle.h"
#include "pipeline.h"

namespace {

constexpr int kNoAllocMaxSrcLimbs = 16;
using cfhe::kMaxDevices;

// Lives in the module image of every device that loads this library. In host
// code this name is only a handle for the runtime's symbol lookup, never an
// address a kernel could use.
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocMaxSrcLimbs * cfhe::kN];

std::mutex g_setup_mutex;
uint32_t *g_scratch_addr[kMaxDevices] = {nullptr};

// Looks up the device address of the array for `device`, which must be the
// current device. Done once per device; later calls return the cached value.
// With lazy module loading this first lookup is also the moment the array
// comes into existence on that device, so cfhe_context_create() performs it
// (through cfhe::noalloc_prepare) while it is allocating anyway; a host that
// creates its contexts before it reserves the GPU's memory never sees the
// entry point below allocate.
int scratch_address(int device, uint32_t **out) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[device]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) {
      cfhe::set_error(std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
      return -2;
    }
    g_scratch_addr[device] = static_cast<uint32_t *>(p);
  }
  *out = g_scratch_addr[device];
  return 0;
}

}  // namespace

namespace cfhe {
int noalloc_prepare(int device) {
  if (device < 0 || device >= kMaxDevices) return 0;  // the entry point refuses such a device itself
  uint32_t *unused = nullptr;
  return scratch_address(device, &unused);
}
}  // namespace cfhe

extern "C" int cfhe_moddown_noalloc(cfhe_context *h, int level, int type,
                                    uint32_t *dst, const uint32_t *src) {
  using namespace cfhe;
  if (!h || !dst || !src) {
    set_error("null argument");
    return -1;
  }
  Context &c = h->c;
  const LevelPlan *lp = c.plan(level);
  if (!lp) {
    set_error("invalid level");
    return -1;
  }
  if (type < 0 || type > 2) {
    set_error("unknown ModDown type");
    return -1;
  }
  if (type != 0 && !lp->has_rescale) {
    set_error("level cannot be rescaled");
    return -1;
  }
  const ConvPlan &cv = lp->down[type];
  if ((int)cv.src_g.size() > kNoAllocMaxSrcLimbs) {
    set_error("cfhe_moddown_noalloc: the conversion drops " +
              std::to_string(cv.src_g.size()) + " limbs, the built-in scratch holds " +
              std::to_string(kNoAllocMaxSrcLimbs));
    return -1;
  }
  int current = -1;
  CFHE_CUDA(cudaGetDevice(&current));
  if (current != c.device || current < 0 || current >= kMaxDevices) {
    set_error("cfhe_moddown_noalloc: make the context's device current before the call");
    return -1;
  }
  uint32_t *scratch = nullptr;
  if (int r = scratch_address(current, &scratch)) return r;
  return run_moddown(c, cv, dst, src, 1, 0, 0, scratch);
}
