// extern "C" boundary of libcheddar_b200.so (see include/cheddar_b200.h).
#include "../../include/cheddar_b200.h"

#include <string.h>

#include <new>

#include "context.h"
#include "host_math.h"
#include "kernels.h"
#include "pipeline.h"

#include "handle.h"

namespace cfhe {
std::atomic<unsigned long long> g_kernel_launches{0};
static thread_local std::string g_error;
void set_error(const std::string &msg) { g_error = msg; }
const std::string &get_error() { return g_error; }

static int fail(const std::string &msg) {
  set_error(msg);
  return -1;
}

// Every entry point runs with the context's device current, whatever device
// the calling thread had selected, and puts the caller's choice back on return
// (kernel attributes, allocations and launches all bind to the current device).
struct DeviceScope {
  int prev = -1;
  bool switched = false;
  cudaError_t err;
  explicit DeviceScope(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      switched = err == cudaSuccess;
    }
  }
  ~DeviceScope() {
    if (switched) cudaSetDevice(prev);
  }
  DeviceScope(const DeviceScope &) = delete;
  DeviceScope &operator=(const DeviceScope &) = delete;
};
#define CFHE_ENTER(handle)                                                    \
  if (!(handle)) return fail("null context");                                 \
  DeviceScope device_scope_((handle)->c.device);                              \
  if (device_scope_.err != cudaSuccess)                                       \
    return fail(std::string("cannot select the context's device: ") + cudaGetErrorString(device_scope_.err))

// Global prime indices of (num_main, num_ter, num_aux): terminal limbs come
// from the tail of the reversed terminal block, main limbs from the head of
// the main block.
static int np_limbs(const Context &c, int nm, int nt, int na, int *gidx) {
  int k = 0;
  for (int g = c.T - nt; g < c.T + nm; g++) gidx[k++] = g;
  for (int a = 0; a < na; a++) gidx[k++] = c.L + a;
  return k;
}

static bool level_np(const Context &c, int level, int *nm, int *nt) {
  if (level == -1) {
    *nm = c.level_config[0].first - c.add_main;
    *nt = c.level_config[0].second - c.add_ter;
    return true;
  }
  if (level < 0 || level >= (int)c.level_config.size()) return false;
  *nm = c.level_config[level].first;
  *nt = c.level_config[level].second;
  return true;
}

static int fill_limbs(const Context &c, NttArgs &a, const int *gidx,
                      int n_limbs) {
  if (n_limbs < 0 || n_limbs > kMaxLimbs) return fail("too many limbs");
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) return fail("prime index out of range");
    a.g[l] = (uint8_t)gidx[l];
    a.q[l] = c.q[gidx[l]];
    a.src_limb[l] = a.dst_limb[l] = (uint16_t)l;
  }
  a.n_limbs = n_limbs;
  return 0;
}
}  // namespace cfhe

using namespace cfhe;

extern "C" {

const char *cfhe_last_error(void) { return get_error().c_str(); }

unsigned long long cfhe_kernel_launch_count(void) {
  return g_kernel_launches.load(std::memory_order_relaxed);
}

int cfhe_context_create(cfhe_context **out, int device, int log_degree,
                        const uint32_t *main_primes, int num_main,
                        const uint32_t *ter_primes, int num_ter,
                        const uint32_t *aux_primes, int num_aux,
                        const int *level_config, int num_levels, int add_main,
                        int add_ter) {
  if (!out) return fail("null output handle");
  *out = nullptr;
  if (log_degree != kLogN)
    return fail("only log_degree 16 is supported");
  if (num_main < 0 || num_ter < 0 || num_aux <= 0 ||
      num_main + num_ter + num_aux > kMaxLimbs || num_levels <= 0)
    return fail("invalid prime counts");
  cfhe_context *h = new (std::nothrow) cfhe_context();
  if (!h) return fail("out of host memory");
  Context &c = h->c;
  c.device = device;
  c.logn = log_degree;
  c.n = 1 << log_degree;
  c.main_primes.assign(main_primes, main_primes + num_main);
  c.ter_primes.assign(ter_primes, ter_primes + num_ter);
  c.aux_primes.assign(aux_primes, aux_primes + num_aux);
  for (int i = 0; i < num_levels; i++)
    c.level_config.emplace_back(level_config[2 * i], level_config[2 * i + 1]);
  c.add_main = add_main;
  c.add_ter = add_ter;
  c.T = num_ter;
  c.M = num_main;
  c.A = num_aux;
  c.L = num_main + num_ter;
  c.NP = c.L + num_aux;
  for (int i = 0; i < num_ter; i++) c.q.push_back(ter_primes[num_ter - 1 - i]);
  for (int i = 0; i < num_main; i++) c.q.push_back(main_primes[i]);
  for (int i = 0; i < num_aux; i++) c.q.push_back(aux_primes[i]);
  for (uint32_t q : c.q) {
    // same validity rules as the reference's Parameter constructor
    // (src/core/Parameter.cu:43-62): below 2^31 and 1 mod 2N
    if (q >= (1u << 31) || q % (2u * c.n) != 1) {
      delete h;
      return fail("prime is not below 2^31 or not 1 mod 2N");
    }
  }
  auto cleanup_fail = [&](const std::string &m) {
    cfhe_context_destroy(h);
    return fail(m);
  };
  DeviceScope device_scope_(device);  // the caller's device is current again on return
  cudaError_t e = device_scope_.err;
  if (e != cudaSuccess) return cleanup_fail(cudaGetErrorString(e));
  if (cudaDeviceGetAttribute(&c.num_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || c.num_sms < 1)
    c.num_sms = 148;
  e = cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return cleanup_fail(cudaGetErrorString(e));
  c.own_stream = true;
  const size_t tsz = (size_t)c.NP * c.n;
  std::vector<Tw> fwd(tsz), inv(tsz);
  c.psi.resize(c.NP);
  c.inv_w1.resize(c.NP);
  for (int g = 0; g < c.NP; g++) {
    build_twiddles(c.q[g], c.logn, fwd.data() + (size_t)g * c.n,
                   inv.data() + (size_t)g * c.n, &c.psi[g]);
    c.inv_w1[g] = inv[(size_t)g * c.n + 1].w;
  }
  e = cudaMalloc(&c.d_tw, tsz * sizeof(Tw));
  if (e == cudaSuccess) e = cudaMalloc(&c.d_itw, tsz * sizeof(Tw));
  if (e == cudaSuccess)
    e = cudaMemcpy(c.d_tw, fwd.data(), tsz * sizeof(Tw), cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaMemcpy(c.d_itw, inv.data(), tsz * sizeof(Tw), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return cleanup_fail(cudaGetErrorString(e));
  if (build_plans(c) != 0 || noalloc_prepare(device) != 0) {
    std::string m = get_error();
    return cleanup_fail(m);
  }
  *out = h;
  return 0;
}

static void pool_release_cached(Context &c);
static void pool_destroy(Context &c);

void cfhe_context_destroy(cfhe_context *h) {
  if (!h) return;
  Context &c = h->c;
  DeviceScope device_scope_(c.device);
  pool_destroy(c);
  free_plans(c);
  if (c.d_tw) cudaFree(c.d_tw);
  if (c.d_itw) cudaFree(c.d_itw);
  if (c.own_stream && c.stream) cudaStreamDestroy(c.stream);
  delete h;
}

static void drop_own_stream(Context &c) {
  if (c.own_stream && c.stream) {
    cudaStreamSynchronize(c.stream);
    cudaStreamDestroy(c.stream);
  }
  c.stream = nullptr;
  c.own_stream = false;
}

int cfhe_set_stream(cfhe_context *h, void *cuda_stream) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  Context &c = h->c;
  if ((cudaStream_t)cuda_stream == c.stream && !c.own_stream) return 0;
  // Work already enqueued on the old stream may still use the workspace and
  // cached blocks the new stream's work will touch: wait for it here (a stream
  // change is a set-up step, not a hot-path call).
  CFHE_CUDA(cudaStreamSynchronize(c.stream));
  {
    std::lock_guard<std::mutex> pool_lock(c.pool_mutex);
    pool_release_cached(c);
  }
  drop_own_stream(c);
  c.stream = (cudaStream_t)cuda_stream;
  return 0;
}

int cfhe_use_own_stream(cfhe_context *h) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  Context &c = h->c;
  if (c.own_stream) return 0;
  CFHE_CUDA(cudaStreamSynchronize(c.stream));
  {
    std::lock_guard<std::mutex> pool_lock(c.pool_mutex);
    pool_release_cached(c);
  }
  CFHE_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
  c.own_stream = true;
  return 0;
}

void *cfhe_get_stream(cfhe_context *h) { return h ? (void *)h->c.stream : nullptr; }

int cfhe_synchronize(cfhe_context *h) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  CFHE_CUDA(cudaStreamSynchronize(h->c.stream));
  int flag = 0;
  CFHE_CUDA(cudaMemcpy(&flag, h->c.d_error_flag, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag) {
    cudaMemset(h->c.d_error_flag, 0, sizeof(int));
    return fail("a kernel gave up a bounded wait (tensor-core completion barrier)");
  }
  return 0;
}

int cfhe_degree(const cfhe_context *h) { return h ? h->c.n : 0; }
int cfhe_num_primes(const cfhe_context *h) { return h ? h->c.NP : 0; }
uint32_t cfhe_prime(const cfhe_context *h, int g) {
  return (h && g >= 0 && g < h->c.NP) ? h->c.q[g] : 0;
}

int cfhe_level_limbs(const cfhe_context *h, int level, int num_aux, int *gidx) {
  if (!h || !gidx) return fail("null argument");
  int nm, nt;
  if (!level_np(h->c, level, &nm, &nt)) return fail("invalid level");
  if (num_aux < 0 || num_aux > h->c.A) return fail("invalid num_aux");
  return np_limbs(h->c, nm, nt, num_aux, gidx);
}

constexpr size_t kSlabGranule = 256u << 10;
constexpr size_t kSlabBytes = size_t(1) << 30;
constexpr size_t kSmallLimit = 1u << 20;

static void slab_insert_free(Context &c, char *p, size_t bytes) {
  c.slab_free_by_addr.emplace(p, bytes);
  c.slab_free_by_size.emplace(bytes, p);
}

static void slab_erase_free(Context &c, char *p, size_t bytes) {
  c.slab_free_by_addr.erase(p);
  auto range = c.slab_free_by_size.equal_range(bytes);
  for (auto it = range.first; it != range.second; ++it)
    if (it->second == p) {
      c.slab_free_by_size.erase(it);
      return;
    }
}

// Gives back to the driver what nobody uses: cached small blocks and slabs
// that are free from end to end.
static void pool_release_cached(Context &c) {
  if (c.pool_free.empty() && c.slab_free_by_addr.empty()) return;
  cudaStreamSynchronize(c.stream);
  for (auto &kv : c.pool_free) cudaFree(kv.second);
  c.pool_free.clear();
  for (auto it = c.slabs.begin(); it != c.slabs.end();) {
    auto f = c.slab_free_by_addr.find(it->first);
    if (f != c.slab_free_by_addr.end() && f->second == it->second) {
      slab_erase_free(c, it->first, it->second);
      cudaFree(it->first);
      it = c.slabs.erase(it);
    } else {
      ++it;
    }
  }
  c.pool_cached_bytes = 0;
  for (auto &kv : c.slab_free_by_addr) c.pool_cached_bytes += kv.second;
}

static void pool_destroy(Context &c) {
  cudaStreamSynchronize(c.stream);
  for (auto &kv : c.pool_free) cudaFree(kv.second);
  for (auto &kv : c.pool_live)
    if (kv.second < kSmallLimit) cudaFree(kv.first);
  for (auto &kv : c.slabs) cudaFree(kv.first);
  c.pool_free.clear();
  c.pool_live.clear();
  c.slabs.clear();
  c.slab_free_by_addr.clear();
  c.slab_free_by_size.clear();
  c.pool_cached_bytes = 0;
}

static cudaError_t malloc_retry(Context &c, void **ptr, size_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    pool_release_cached(c);
    e = cudaMalloc(ptr, bytes);
  }
  return e;
}

int cfhe_malloc(cfhe_context *h, void **ptr, size_t bytes) {
  CFHE_ENTER(h);
  if (!h || !ptr) return fail("null argument");
  Context &c = h->c;
  std::lock_guard<std::mutex> pool_lock(c.pool_mutex);
  if (bytes < kSmallLimit) {
    // size classes of 4 KiB; a cached block is reused only for its exact class
    const size_t rounded = bytes ? (bytes + 4095) / 4096 * 4096 : 4096;
    auto it = c.pool_free.find(rounded);
    if (it != c.pool_free.end()) {
      *ptr = it->second;
      c.pool_free.erase(it);
      c.pool_cached_bytes -= rounded;
      c.pool_live[*ptr] = rounded;
      return 0;
    }
    cudaError_t e = malloc_retry(c, ptr, rounded);
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    c.pool_live[*ptr] = rounded;
    return 0;
  }
  const size_t rounded = (bytes + kSlabGranule - 1) / kSlabGranule * kSlabGranule;
  auto it = c.slab_free_by_size.lower_bound(rounded);
  if (it == c.slab_free_by_size.end()) {
    // a new slab; when the device cannot give a whole one, just the request
    void *slab = nullptr;
    size_t slab_bytes = rounded > kSlabBytes ? rounded : kSlabBytes;
    cudaError_t e = cudaMalloc(&slab, slab_bytes);
    if (e == cudaErrorMemoryAllocation && slab_bytes > rounded) {
      cudaGetLastError();
      slab_bytes = rounded;
      e = malloc_retry(c, &slab, slab_bytes);
    } else if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();
      e = malloc_retry(c, &slab, slab_bytes);
    }
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    c.slabs.emplace((char *)slab, slab_bytes);
    slab_insert_free(c, (char *)slab, slab_bytes);
    c.pool_cached_bytes += slab_bytes;
    it = c.slab_free_by_size.lower_bound(rounded);
  }
  char *p = it->second;
  const size_t have = it->first;
  slab_erase_free(c, p, have);
  if (have > rounded) slab_insert_free(c, p + rounded, have - rounded);
  c.pool_cached_bytes -= rounded;
  c.pool_live[p] = rounded;
  *ptr = p;
  return 0;
}

int cfhe_free(cfhe_context *h, void *ptr) {
  if (!h) return fail("null context");
  if (!ptr) return 0;
  Context &c = h->c;
  std::lock_guard<std::mutex> pool_lock(c.pool_mutex);
  auto it = c.pool_live.find(ptr);
  if (it == c.pool_live.end()) return fail("cfhe_free: pointer was not returned by cfhe_malloc");
  size_t bytes = it->second;
  c.pool_live.erase(it);
  c.pool_cached_bytes += bytes;
  if (bytes < kSmallLimit) {
    c.pool_free.emplace(bytes, ptr);
    return 0;
  }
  // merge with the free neighbours of the same slab (a slab start is never merged into)
  char *p = (char *)ptr;
  auto next = c.slab_free_by_addr.lower_bound(p);
  if (next != c.slab_free_by_addr.end() && next->first == p + bytes && !c.slabs.count(next->first)) {
    const size_t nb = next->second;
    slab_erase_free(c, next->first, nb);
    bytes += nb;
  }
  auto after = c.slab_free_by_addr.lower_bound(p);
  if (after != c.slab_free_by_addr.begin() && !c.slabs.count(p)) {
    auto prev = std::prev(after);
    if (prev->first + prev->second == p) {
      char *pp = prev->first;
      const size_t pb = prev->second;
      slab_erase_free(c, pp, pb);
      p = pp;
      bytes += pb;
    }
  }
  slab_insert_free(c, p, bytes);
  return 0;
}

int cfhe_order_after(cfhe_context *later, cfhe_context *earlier) {
  if (!later || !earlier) return fail("null context");
  DeviceScope device_scope_(earlier->c.device);
  if (later == earlier || later->c.stream == earlier->c.stream) return 0;
  Context &e = earlier->c;
  if (!e.order_event) CFHE_CUDA(cudaEventCreateWithFlags(&e.order_event, cudaEventDisableTiming));
  CFHE_CUDA(cudaEventRecord(e.order_event, e.stream));
  CFHE_CUDA(cudaStreamWaitEvent(later->c.stream, e.order_event, 0));
  return 0;
}

int cfhe_copy_h2d(cfhe_context *h, void *dst, const void *src, size_t bytes) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  CFHE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, h->c.stream));
  return 0;
}

int cfhe_copy_d2h(cfhe_context *h, void *dst, const void *src, size_t bytes) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  CFHE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, h->c.stream));
  CFHE_CUDA(cudaStreamSynchronize(h->c.stream));
  return 0;
}

int cfhe_ntt(cfhe_context *h, uint32_t *dst, const uint32_t *src,
             const int *gidx, int n_limbs, int n_polys,
             long long dst_poly_stride, long long src_poly_stride,
             int mont_conv) {
  CFHE_ENTER(h);
  if (!h || !dst || !src || !gidx) return fail("null argument");
  const Context &c = h->c;
  NttArgs a;
  memset(&a, 0, sizeof(a));
  if (int r = fill_limbs(c, a, gidx, n_limbs)) return r;
  a.dst = dst;
  a.src = src;
  a.table = c.d_tw;
  a.dst_poly_stride = dst_poly_stride;
  a.src_poly_stride = src_poly_stride;
  a.n_polys = n_polys;
  a.premul = mont_conv != 0;
  if (a.premul)
    for (int l = 0; l < n_limbs; l++) a.kc[l] = make_tw(r_mod(a.q[l]), a.q[l]);
  { int r_ = launch_ntt(c, a, false); c.mark("ntt"); return r_; }
}

int cfhe_intt(cfhe_context *h, uint32_t *dst, const uint32_t *src,
              const int *gidx, int n_limbs, int n_polys,
              long long dst_poly_stride, long long src_poly_stride,
              const uint32_t *consts, int mont_keep, int centred) {
  CFHE_ENTER(h);
  if (!h || !dst || !src || !gidx) return fail("null argument");
  const Context &c = h->c;
  NttArgs a;
  memset(&a, 0, sizeof(a));
  if (int r = fill_limbs(c, a, gidx, n_limbs)) return r;
  a.dst = dst;
  a.src = src;
  a.table = c.d_itw;
  a.dst_poly_stride = dst_poly_stride;
  a.src_poly_stride = src_poly_stride;
  a.n_polys = n_polys;
  a.centred = centred != 0;
  for (int l = 0; l < n_limbs; l++) {
    const uint32_t q = a.q[l];
    uint32_t k;
    if (consts) {
      k = mulmod(consts[l] % q, rinv_mod(q), q);
    } else {
      const uint32_t ninv = invmod((uint32_t)c.n % q, q);
      k = mont_keep ? ninv : mulmod(ninv, rinv_mod(q), q);
    }
    a.kc[l] = make_tw(k, q);
  }
  { int r_ = launch_ntt(c, a, true); c.mark("intt"); return r_; }
}

// ---------------------------------------------------------------------------
// element-wise
// ---------------------------------------------------------------------------
static int fill_rows(const Context &c, EwArgs &e, uint32_t *dst,
                     const uint32_t *a, const uint32_t *b,
                     const uint32_t *consts, const int *gidx, int n_limbs) {
  if (!dst || !a || !gidx) return fail("null argument");
  if (n_limbs < 0 || n_limbs > kMaxRows) return fail("too many limbs");
  e.n_rows = n_limbs;
  for (int l = 0; l < n_limbs; l++) {
    const int g = gidx[l];
    if (g < 0 || g >= c.NP) return fail("prime index out of range");
    const size_t o = (size_t)l * kN;
    e.rows[l] = EwRow{dst + o, a + o, b ? b + o : nullptr, c.q[g], c.nqinv[g],
                      consts ? consts[l] % c.q[g] : 0u, 0u};
  }
  return 0;
}

int cfhe_binary(cfhe_context *h, int op, uint32_t *dst, const uint32_t *a,
                const uint32_t *b, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  static const int map[4] = {EW_ADD, EW_SUB, EW_NEG, EW_MUL};
  if (op < 0 || op > 3) return fail("unknown binary op");
  if (op != 2 && !b) return fail("null argument");
  EwArgs e;
  if (int r = fill_rows(h->c, e, dst, a, b, nullptr, gidx, n_limbs)) return r;
  { int r_ = launch_ew(h->c, map[op], e); h->c.mark("elementwise"); return r_; }
}

int cfhe_const_op(cfhe_context *h, int op, uint32_t *dst, const uint32_t *a,
                  const uint32_t *b, const uint32_t *consts, const int *gidx,
                  int n_limbs) {
  CFHE_ENTER(h);
  if (!h || !consts) return fail("null argument");
  static const int map[5] = {EW_ADDC, EW_SUBC, EW_RSUBC, EW_MULC, EW_MULC_ADD};
  if (op < 0 || op > 4) return fail("unknown const op");
  if (op == 4 && !b) return fail("null argument");
  EwArgs e;
  if (int r = fill_rows(h->c, e, dst, a, b, consts, gidx, n_limbs)) return r;
  { int r_ = launch_ew(h->c, map[op], e); h->c.mark("elementwise"); return r_; }
}

int cfhe_elementwise_multi(cfhe_context *h, int with_const, int op, int n_polys,
                           uint32_t *const *dst, const uint32_t *const *a,
                           const uint32_t *const *b, const uint32_t *consts,
                           const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!h || !dst || !a || !gidx) return fail("null argument");
  static const int bin[4] = {EW_ADD, EW_SUB, EW_NEG, EW_MUL};
  static const int con[5] = {EW_ADDC, EW_SUBC, EW_RSUBC, EW_MULC, EW_MULC_ADD};
  if (op < 0 || op > (with_const ? 4 : 3)) return fail("unknown element-wise op");
  if (with_const && !consts) return fail("null argument");
  const bool needs_b = with_const ? op == 4 : op != 2;
  if (n_polys < 1 || n_limbs < 0 || n_polys * n_limbs > kMaxRows) return fail("too many limbs");
  const Context &c = h->c;
  EwArgs e;
  e.n_rows = 0;
  for (int p = 0; p < n_polys; p++) {
    if (!dst[p] || !a[p] || (needs_b && (!b || !b[p]))) return fail("null argument");
    for (int l = 0; l < n_limbs; l++) {
      const int g = gidx[l];
      if (g < 0 || g >= c.NP) return fail("prime index out of range");
      const size_t o = (size_t)l * kN;
      e.rows[e.n_rows++] = EwRow{dst[p] + o, a[p] + o, (b && b[p]) ? b[p] + o : nullptr, c.q[g],
                                 c.nqinv[g], with_const ? consts[l] % c.q[g] : 0u, 0u};
    }
  }
  { int r_ = launch_ew(c, with_const ? con[op] : bin[op], e); c.mark("elementwise"); return r_; }
}

int cfhe_tensor(cfhe_context *h, uint32_t *d0, uint32_t *d1, uint32_t *d2,
                const uint32_t *b1, const uint32_t *a1, const uint32_t *b2,
                const uint32_t *a2, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!h || !d0 || !d1 || !d2 || !b1 || !a1 || !b2 || !a2 || !gidx)
    return fail("null argument");
  if (n_limbs < 0 || n_limbs > kMaxLimbs) return fail("too many limbs");
  const Context &c = h->c;
  TensorArgs t;
  t.n_rows = n_limbs;
  for (int l = 0; l < n_limbs; l++) {
    const int g = gidx[l];
    if (g < 0 || g >= c.NP) return fail("prime index out of range");
    const size_t o = (size_t)l * kN;
    t.rows[l] = TensorRow{d0 + o, d1 + o, d2 + o, b1 + o, a1 + o,
                          b2 + o, a2 + o, c.q[g], c.nqinv[g]};
  }
  { int r_ = launch_tensor(c, t); c.mark("tensor"); return r_; }
}

int cfhe_permute(cfhe_context *h, uint32_t *dst, const uint32_t *src,
                 const uint32_t *add, uint32_t galois, const int *gidx,
                 int n_limbs) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  if (dst == src) return fail("permute cannot run in place");
  if ((galois & 1u) == 0 || galois >= 2u * kN) return fail("invalid Galois element");
  EwArgs e;
  if (int r = fill_rows(h->c, e, dst, src, add, nullptr, gidx, n_limbs)) return r;
  { int r_ = launch_permute(h->c, e, galois); h->c.mark("permute"); return r_; }
}

// Shared argument checks of the four n-ary entry points; src is
// [term * n_polys + poly].
static int fill_nary(const Context &c, NaryArgs &a, int mode, int n_polys, uint32_t *const *dst,
                     int n_terms, const uint32_t *const *src, const uint32_t *const *addend,
                     const int *gidx, int n_limbs) {
  if (!dst || !src || !gidx) return fail("null argument");
  if (n_polys < 1 || n_polys > kMaxNaryPolys) return fail("n-ary sum: one to three polynomials");
  if (n_terms < 1 || n_terms > kMaxTerms) return fail("n-ary sum: one to eight terms");
  if (n_limbs < 0 || n_limbs > kMaxLimbs) return fail("too many limbs");
  memset(&a, 0, sizeof(a));
  a.mode = mode;
  a.n_terms = n_terms;
  a.n_polys = n_polys;
  a.n_limbs = n_limbs;
  for (int p = 0; p < n_polys; p++) {
    if (!dst[p]) return fail("null argument");
    a.dst[p] = dst[p];
    a.add[p] = addend ? addend[p] : nullptr;
    for (int t = 0; t < n_terms; t++) {
      if (!src[t * n_polys + p]) return fail("null argument");
      a.src[t][p] = src[t * n_polys + p];
    }
  }
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) return fail("prime index out of range");
    a.q[l] = c.q[gidx[l]];
    a.nqinv[l] = c.nqinv[gidx[l]];
  }
  return 0;
}

int cfhe_accum(cfhe_context *h, int n_polys, uint32_t *const *dst, int n_terms,
               const uint32_t *const *src, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  NaryArgs a;
  if (int r = fill_nary(h->c, a, NARY_SUM, n_polys, dst, n_terms, src, nullptr, gidx, n_limbs)) return r;
  { int r_ = launch_nary(h->c, a); h->c.mark("elementwise"); return r_; }
}

int cfhe_caccum(cfhe_context *h, int n_polys, uint32_t *const *dst, int n_terms,
                const uint32_t *const *src, const uint32_t *consts,
                const uint32_t *const *addend, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!consts) return fail("null argument");
  NaryArgs a;
  if (int r = fill_nary(h->c, a, NARY_CONST, n_polys, dst, n_terms, src, addend, gidx, n_limbs)) return r;
  for (int t = 0; t < n_terms; t++)
    for (int l = 0; l < n_limbs; l++) a.c[t][l] = consts[t * n_limbs + l] % a.q[l];
  { int r_ = launch_nary(h->c, a); h->c.mark("elementwise"); return r_; }
}

int cfhe_paccum(cfhe_context *h, int n_polys, uint32_t *const *dst, int n_terms,
                const uint32_t *const *src, const uint32_t *const *pt,
                const uint32_t *const *addend, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!pt) return fail("null argument");
  NaryArgs a;
  if (int r = fill_nary(h->c, a, NARY_PLAIN, n_polys, dst, n_terms, src, addend, gidx, n_limbs)) return r;
  for (int t = 0; t < n_terms; t++) {
    if (!pt[t]) return fail("null argument");
    a.pt[t] = pt[t];
  }
  { int r_ = launch_nary(h->c, a); h->c.mark("elementwise"); return r_; }
}

int cfhe_permute_accum(cfhe_context *h, int n_polys, uint32_t *const *dst, int n_terms,
                       const uint32_t *const *src, const uint32_t *galois,
                       const uint32_t *const *addend, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!galois) return fail("null argument");
  NaryArgs a;
  if (int r = fill_nary(h->c, a, NARY_PERMUTE, n_polys, dst, n_terms, src, addend, gidx, n_limbs)) return r;
  for (int t = 0; t < n_terms; t++) {
    if ((galois[t] & 1u) == 0 || galois[t] >= 2u * kN) return fail("invalid Galois element");
    a.galois[t] = galois[t];
    for (int p = 0; p < n_polys; p++)
      if (a.src[t][p] == a.dst[p]) return fail("permute cannot run in place");
  }
  { int r_ = launch_nary(h->c, a); h->c.mark("permute"); return r_; }
}

int cfhe_tensor_accum(cfhe_context *h, uint32_t *d0, uint32_t *d1, uint32_t *d2, int n_terms,
                      const uint32_t *const *b1, const uint32_t *const *a1, const uint32_t *const *b2,
                      const uint32_t *const *a2, int accumulate, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!d0 || !d1 || !d2 || !b1 || !a1 || !b2 || !a2 || !gidx) return fail("null argument");
  if (n_terms < 1 || n_terms > kMaxTensorTerms) return fail("tensor accumulate: one to sixteen terms");
  if (n_limbs < 0 || n_limbs > kMaxLimbs) return fail("too many limbs");
  TensorAccArgs a;
  memset(&a, 0, sizeof(a));
  a.n_terms = n_terms;
  a.n_limbs = n_limbs;
  a.accumulate = accumulate != 0;
  a.d[0] = d0;
  a.d[1] = d1;
  a.d[2] = d2;
  for (int t = 0; t < n_terms; t++) {
    if (!b1[t] || !a1[t] || !b2[t] || !a2[t]) return fail("null argument");
    a.b1[t] = b1[t];
    a.a1[t] = a1[t];
    a.b2[t] = b2[t];
    a.a2[t] = a2[t];
  }
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= h->c.NP) return fail("prime index out of range");
    a.q[l] = h->c.q[gidx[l]];
    a.nqinv[l] = h->c.nqinv[gidx[l]];
  }
  { int r_ = launch_tensor_accum(h->c, a); h->c.mark("elementwise"); return r_; }
}

int cfhe_giantstep_paccum(cfhe_context *h, uint32_t *acc, const uint32_t *rot, int n_baby, int n_giant,
                          const uint32_t *const *pt, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!acc || !rot || !pt || !gidx) return fail("null argument");
  if (n_baby < 1 || n_baby > kMaxBaby || n_giant < 1 || n_giant > kMaxGiant)
    return fail("giant-step accumulate: 1 to 16 baby and giant steps");
  if (n_limbs < 1 || n_limbs > kMaxLimbs) return fail("too many limbs");
  PtAccumArgs a;
  memset(&a, 0, sizeof(a));
  a.rot = rot;
  a.acc = acc;
  a.n_baby = n_baby;
  a.n_giant = n_giant;
  a.ntot = n_limbs;
  for (int j = 0; j < n_giant; j++)
    for (int i = 0; i < n_baby; i++) a.pt[j * kMaxBaby + i] = pt[j * n_baby + i];
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= h->c.NP) return fail("prime index out of range");
    a.q[l] = h->c.q[gidx[l]];
    a.nqinv[l] = h->c.nqinv[gidx[l]];
  }
  { int r_ = launch_pt_accum(h->c, a); h->c.mark("elementwise"); return r_; }
}

size_t cfhe_gemm_weight_bytes(int n_in, int n_out, int n_limbs) {
  if (n_in < 1 || n_out < 1 || n_limbs < 1) return 0;
  return gemm_packed_weight_bytes(n_in, n_out) * (size_t)n_limbs;
}

int cfhe_gemm_pack_weights(cfhe_context *h, void *packed, const uint32_t *weights, int n_in, int n_out,
                           const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!packed || !weights || !gidx) return fail("null argument");
  if (n_in < 1 || n_in > 8192 || n_out < 1 || n_limbs < 1 || n_limbs > kMaxLimbs)
    return fail("ct-pt GEMM: unsupported shape");
  const Context &c = h->c;
  const size_t per_limb = gemm_packed_weight_bytes(n_in, n_out);
  std::vector<uint8_t> host(per_limb);
  for (int l = 0; l < n_limbs; l++) {
    if (gidx[l] < 0 || gidx[l] >= c.NP) return fail("prime index out of range");
    gemm_pack_weights_limb(host.data(), weights + (size_t)l * n_in * n_out, n_in, n_out, c.q[gidx[l]]);
    CFHE_CUDA(cudaMemcpyAsync((uint8_t *)packed + (size_t)l * per_limb, host.data(), per_limb,
                              cudaMemcpyHostToDevice, c.stream));
    CFHE_CUDA(cudaStreamSynchronize(c.stream));  // the staging buffer is reused
  }
  return 0;
}

int cfhe_ctpt_gemm(cfhe_context *h, uint32_t *const *y, const uint32_t *const *x, const void *packed,
                   int n_in, int n_out, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!y || !x || !packed || !gidx) return fail("null argument");
  if (n_in < 1 || n_in > 8192 || n_out < 1 || n_out > 8192 || n_limbs < 1 || n_limbs > kMaxLimbs)
    return fail("ct-pt GEMM: unsupported shape");
  Context &c = h->c;
  // workspace: packed activations of one limb, then the two pointer tables
  const size_t scratch = (gemm_scratch_bytes(n_in) + 255) / 256 * 256;
  const size_t tables = (size_t)(n_in + n_out) * sizeof(void *);
  if (int r = ensure_workspace(c, (scratch + tables + 3) / 4)) return r;
  uint8_t *base = reinterpret_cast<uint8_t *>(c.ws);
  const uint32_t **dx = reinterpret_cast<const uint32_t **>(base + scratch);
  uint32_t **dy = reinterpret_cast<uint32_t **>(base + scratch + (size_t)n_in * sizeof(void *));
  for (int k = 0; k < n_in; k++)
    if (!x[k]) return fail("null argument");
  for (int j = 0; j < n_out; j++)
    if (!y[j]) return fail("null argument");
  CFHE_CUDA(cudaMemcpyAsync(dx, x, (size_t)n_in * sizeof(void *), cudaMemcpyHostToDevice, c.stream));
  CFHE_CUDA(cudaMemcpyAsync(dy, y, (size_t)n_out * sizeof(void *), cudaMemcpyHostToDevice, c.stream));
  CFHE_CUDA(cudaStreamSynchronize(c.stream));  // the host tables may go away after the call
  { int r_ = launch_ctpt_gemm(c, dy, dx, (const uint8_t *)packed, base, n_in, n_out, gidx, n_limbs); c.mark("gemm"); return r_; }
}

int cfhe_sample_uniform(cfhe_context *h, uint32_t *dst, const int *gidx, int n_limbs,
                        unsigned long long seed, unsigned int stream) {
  CFHE_ENTER(h);
  { int r_ = launch_sample_uniform(h->c, dst, gidx, n_limbs, seed, stream); h->c.mark("sample"); return r_; }
}

int cfhe_sample_error(cfhe_context *h, uint32_t *dst, const int *gidx, int n_limbs, double sigma,
                      unsigned long long seed, unsigned int stream) {
  CFHE_ENTER(h);
  { int r_ = launch_sample_error(h->c, dst, gidx, n_limbs, sigma, seed, stream); h->c.mark("sample"); return r_; }
}

int cfhe_error_cdf(double sigma, unsigned long long *cdf, int entries) {
  if (!cdf || entries != kErrorCdfEntries) return fail("cfhe_error_cdf: the table has 97 entries");
  if (!(sigma > 0.0) || sigma > 8.0) return fail("error sampling: standard deviation must be in (0, 8]");
  static_assert(sizeof(unsigned long long) == sizeof(uint64_t), "64-bit table entries");
  error_cdf_table(sigma, reinterpret_cast<uint64_t *>(cdf));
  return 0;
}

int cfhe_encrypt(cfhe_context *h, uint32_t *b, const uint32_t *a, const uint32_t *s, const uint32_t *e,
                 const uint32_t *m, const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  { int r_ = launch_encrypt(h->c, b, a, s, e, m, gidx, n_limbs); h->c.mark("encrypt"); return r_; }
}

int cfhe_encode_coeffs(cfhe_context *h, uint32_t *dst, const double *coeffs, const int *gidx, int n_limbs) {
  if (!h || !dst || !coeffs || !gidx) return fail("null argument");
  void *staging = nullptr;
  if (int r = cfhe_malloc(h, &staging, (size_t)kN * sizeof(double))) return r;
  int rc;
  {
    CFHE_ENTER(h);
    cudaError_t e = cudaMemcpyAsync(staging, coeffs, (size_t)kN * sizeof(double), cudaMemcpyHostToDevice, h->c.stream);
    rc = e == cudaSuccess ? 0 : fail(cudaGetErrorString(e));
    if (!rc) rc = launch_rns_split(h->c, dst, (const double *)staging, gidx, n_limbs);
    h->c.mark("encode");
  }
  cfhe_free(h, staging);  // reused in stream order, after the kernel above
  if (rc) return rc;
  return cfhe_ntt(h, dst, dst, gidx, n_limbs, 1, 0, 0, 1);
}

int cfhe_decode_coeffs(cfhe_context *h, double *coeffs, const uint32_t *src, const int *gidx, int n_limbs,
                       const uint32_t *icrt, const uint32_t *hat, const uint32_t *q_low) {
  if (!h || !coeffs || !src || !gidx || !icrt || !hat || !q_low) return fail("null argument");
  if (n_limbs < 1 || n_limbs > kMaxLimbs) return fail("too many limbs");
  void *res = nullptr, *out = nullptr;
  if (int r = cfhe_malloc(h, &res, (size_t)n_limbs * kN * sizeof(uint32_t))) return r;
  if (int r = cfhe_malloc(h, &out, (size_t)kN * sizeof(double))) {
    cfhe_free(h, res);
    return r;
  }
  int rc = cfhe_intt(h, (uint32_t *)res, src, gidx, n_limbs, 1, 0, 0, icrt, 0, 0);
  if (!rc) {
    CFHE_ENTER(h);
    rc = launch_crt_lift(h->c, (double *)out, (const uint32_t *)res, gidx, n_limbs, hat, q_low);
    h->c.mark("decode");
    if (!rc) {
      cudaError_t e = cudaMemcpyAsync(coeffs, out, (size_t)kN * sizeof(double), cudaMemcpyDeviceToHost, h->c.stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(h->c.stream);
      if (e != cudaSuccess) rc = fail(cudaGetErrorString(e));
    }
  }
  cfhe_free(h, out);
  cfhe_free(h, res);
  return rc;
}

int cfhe_add_evk_part(cfhe_context *h, uint32_t *bx, const uint32_t *s_target, const uint32_t *p_prod,
                      const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!p_prod) return fail("null argument");
  EwArgs e;
  if (int r = fill_rows(h->c, e, bx, s_target, bx, p_prod, gidx, n_limbs)) return r;
  { int r_ = launch_ew(h->c, EW_MULC_ADD, e); h->c.mark("elementwise"); return r_; }
}

int cfhe_copy_d2d(cfhe_context *h, void *dst, const void *src, size_t bytes) {
  CFHE_ENTER(h);
  if (!dst || !src) return fail("null argument");
  CFHE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, h->c.stream));
  return 0;
}

int cfhe_memset(cfhe_context *h, void *dst, int value, size_t bytes) {
  CFHE_ENTER(h);
  if (!dst) return fail("null argument");
  CFHE_CUDA(cudaMemsetAsync(dst, value, bytes, h->c.stream));
  return 0;
}

uint32_t cfhe_galois_for_rotation(const cfhe_context *h, int rot) {
  if (!h) return 0;
  const uint32_t m = 2u * h->c.n;
  if (rot < 0) return m - 1;
  uint32_t g = 1;
  for (int i = 0; i < rot; i++) g = (uint32_t)(((uint64_t)g * 5u) % m);
  return g;
}

int cfhe_mul_imag_unit(cfhe_context *h, uint32_t *dst, const uint32_t *src,
                       const int *gidx, int n_limbs) {
  CFHE_ENTER(h);
  if (!h || !gidx) return fail("null argument");
  const Context &c = h->c;
  if (n_limbs < 0 || n_limbs > kMaxRows) return fail("too many limbs");
  std::vector<uint32_t> u(n_limbs);
  for (int l = 0; l < n_limbs; l++) {
    const int g = gidx[l];
    if (g < 0 || g >= c.NP) return fail("prime index out of range");
    // psi^(N/2) in M-form (the reference reuses twiddle entry 1,
    // src/core/NTT.cu:1301-1310)
    u[l] = to_mont(powmod(c.psi[g], (uint64_t)c.n / 2, c.q[g]), c.q[g]);
  }
  EwArgs e;
  if (int r = fill_rows(c, e, dst, src, nullptr, u.data(), gidx, n_limbs)) return r;
  { int r_ = launch_ew(c, EW_IMAG, e); c.mark("elementwise"); return r_; }
}

int cfhe_modup_to_max(cfhe_context *h, uint32_t *dst, const uint32_t *src,
                      const int *src_gidx, int n_src, const int *dst_gidx,
                      int n_dst) {
  CFHE_ENTER(h);
  if (!h || !dst || !src || !src_gidx || !dst_gidx) return fail("null argument");
  const Context &c = h->c;
  if (n_src < 1 || n_src > 2) return fail("modup_to_max: one or two source limbs");
  if (n_dst < 1 || n_dst > kMaxRows) return fail("too many limbs");
  for (int i = 0; i < n_src; i++)
    if (src_gidx[i] < 0 || src_gidx[i] >= c.NP) return fail("prime index out of range");
  EwArgs e;
  e.n_rows = n_dst;
  for (int l = 0; l < n_dst; l++) {
    const int g = dst_gidx[l];
    if (g < 0 || g >= c.NP) return fail("prime index out of range");
    e.rows[l] = EwRow{dst + (size_t)l * kN, nullptr, nullptr, c.q[g], c.nqinv[g], 0u, 0u};
  }
  { int r_ = launch_lift(c, e, src, c.q[src_gidx[0]], n_src == 2 ? c.q[src_gidx[1]] : 0u); c.mark("lift"); return r_; }
}

// ---------------------------------------------------------------------------
// mod-switch
// ---------------------------------------------------------------------------
int cfhe_bconv(cfhe_context *h, uint32_t *dst, const int32_t *y,
               const int *src_gidx, int n_src, const int *dst_gidx, int n_dst) {
  CFHE_ENTER(h);
  if (!h || !dst || !y || !src_gidx || !dst_gidx) return fail("null argument");
  Context &c = h->c;
  if (n_src < 1 || n_src > kMaxBconvSrc || n_dst < 1 || n_dst > kMaxLimbs)
    return fail("bconv: unsupported shape");
  std::vector<int32_t> t((size_t)n_src * n_dst);
  BconvArgs b;
  memset(&b, 0, sizeof(b));
  BconvJob &j = b.jobs[0];
  for (int m = 0; m < n_dst; m++) {
    const int gd = dst_gidx[m];
    if (gd < 0 || gd >= c.NP) return fail("prime index out of range");
    const uint32_t p = c.q[gd];
    for (int k = 0; k < n_src; k++) {
      uint32_t acc = 1;
      for (int i = 0; i < n_src; i++) {
        if (src_gidx[i] < 0 || src_gidx[i] >= c.NP)
          return fail("prime index out of range");
        if (i != k) acc = mulmod(acc, c.q[src_gidx[i]] % p, p);
      }
      acc = to_mont(to_mont(acc, p), p);
      t[(size_t)m * n_src + k] = acc > (p >> 1) ? (int32_t)(acc - p) : (int32_t)acc;
    }
    j.dst_limb[m] = (uint8_t)m;
    j.q[m] = p;
    j.qinv[m] = 0u - c.nqinv[gd];
  }
  int32_t *d_t = nullptr;
  CFHE_CUDA(cudaMalloc(&d_t, t.size() * sizeof(int32_t)));
  if (cudaError_t ce = cudaMemcpyAsync(d_t, t.data(), t.size() * sizeof(int32_t), cudaMemcpyHostToDevice,
                                       c.stream);
      ce != cudaSuccess) {
    cudaFree(d_t);
    return fail(cudaGetErrorString(ce));
  }
  j.src = y;
  j.dst = dst;
  j.table = d_t;
  j.ns = n_src;
  j.nd = n_dst;
  b.n_jobs = 1;
  int r = launch_bconv(c, b);
  cudaStreamSynchronize(c.stream);
  cudaFree(d_t);
  return r;
}

static const LevelPlan *get_plan(cfhe_context *h, int level) {
  if (!h) {
    fail("null context");
    return nullptr;
  }
  const LevelPlan *lp = h->c.plan(level);
  if (!lp) fail("invalid level");
  return lp;
}

int cfhe_beta(const cfhe_context *h, int level) {
  if (!h) return fail("null context");
  const LevelPlan *lp = h->c.plan(level);
  if (!lp) return fail("invalid level");
  return lp->beta;
}

int cfhe_pseudo_modup(cfhe_context *h, int level, uint32_t *dst, const uint32_t *src) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!dst || !src) return fail("null argument");
  EwArgs e;
  if (int r = fill_rows(h->c, e, dst, src, nullptr, lp->p_mont.data(), lp->q_g.data(), lp->nq)) return r;
  { int r_ = launch_ew(h->c, EW_MULC, e); h->c.mark("elementwise"); return r_; }
}

int cfhe_modup(cfhe_context *h, int level, uint32_t *dst, const uint32_t *src) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!dst || !src) return fail("null argument");
  if (int r = ensure_workspace(h->c, modup_scratch_words(*lp))) return r;
  return run_modup(h->c, *lp, dst, src, true, h->c.ws);
}

int cfhe_moddown(cfhe_context *h, int level, int type, uint32_t *dst,
                 const uint32_t *src, int n_polys, long long dst_poly_stride,
                 long long src_poly_stride) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!dst || !src) return fail("null argument");
  if (type < 0 || type > 2) return fail("unknown ModDown type");
  if (type != 0 && !lp->has_rescale) return fail("level cannot be rescaled");
  if (n_polys < 1 || n_polys > kMaxBconvJobs) return fail("invalid n_polys");
  const ConvPlan &cv = lp->down[type];
  if (int r = ensure_workspace(h->c, moddown_scratch_words(cv, n_polys))) return r;
  return run_moddown(h->c, cv, dst, src, n_polys, dst_poly_stride,
                     src_poly_stride, h->c.ws);
}

// the three stages of cfhe_moddown as separate calls
static const ConvPlan *moddown_plan(cfhe_context *h, int level, int type, int n_polys) {
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return nullptr;
  if (type < 0 || type > 2) { fail("unknown ModDown type"); return nullptr; }
  if (type != 0 && !lp->has_rescale) { fail("level cannot be rescaled"); return nullptr; }
  if (n_polys < 1 || n_polys > kMaxBconvJobs) { fail("invalid n_polys"); return nullptr; }
  return &lp->down[type];
}

int cfhe_moddown_source_limbs(cfhe_context *h, int level, int type) {
  if (!h) return fail("null context");
  const ConvPlan *cv = moddown_plan(h, level, type, 1);
  return cv ? (int)cv->src_g.size() : -1;
}

int cfhe_intt_for_moddown(cfhe_context *h, int level, int type, uint32_t *y, const uint32_t *src, int n_polys,
                          long long src_poly_stride) {
  CFHE_ENTER(h);
  if (!y || !src) return fail("null argument");
  const ConvPlan *cv = moddown_plan(h, level, type, n_polys);
  if (!cv) return -1;
  return run_moddown_intt(h->c, *cv, y, src, n_polys, src_poly_stride);
}

int cfhe_bconv_for_moddown(cfhe_context *h, int level, int type, uint32_t *dst, uint32_t *y, int n_polys,
                           long long dst_poly_stride) {
  CFHE_ENTER(h);
  if (!dst || !y) return fail("null argument");
  const ConvPlan *cv = moddown_plan(h, level, type, n_polys);
  if (!cv) return -1;
  return run_moddown_bconv(h->c, *cv, dst, y, n_polys, dst_poly_stride);
}

int cfhe_ntt_for_moddown(cfhe_context *h, int level, int type, uint32_t *dst, const uint32_t *src, int n_polys,
                         long long dst_poly_stride, long long src_poly_stride) {
  CFHE_ENTER(h);
  if (!dst || !src) return fail("null argument");
  const ConvPlan *cv = moddown_plan(h, level, type, n_polys);
  if (!cv) return -1;
  return run_moddown_ntt(h->c, *cv, dst, src, n_polys, dst_poly_stride, src_poly_stride);
}

int cfhe_evk_inner(cfhe_context *h, int level, uint32_t *acc_b, uint32_t *acc_a,
                   const uint32_t *modup, const uint32_t *c0, const uint32_t *c1,
                   const uint32_t *const *evk_b, const uint32_t *const *evk_a,
                   int key_main) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!acc_b || !acc_a || !modup || !evk_b || !evk_a) return fail("null argument");
  return run_inner(h->c, *lp, acc_b, acc_a, modup, nullptr, c0, c1, evk_b,
                   evk_a, key_main);
}

int cfhe_keyswitch(cfhe_context *h, int level, uint32_t *out_b, uint32_t *out_a,
                   const uint32_t *d, const uint32_t *bx,
                   const uint32_t *const *evk_b, const uint32_t *const *evk_a,
                   int key_main) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!out_b || !out_a || !d || !evk_b || !evk_a) return fail("null argument");
  if (int r = ensure_workspace(h->c, keyswitch_scratch_words(*lp, 0))) return r;
  return run_keyswitch(h->c, *lp, 0, out_b, out_a, d, bx, nullptr, evk_b, evk_a,
                       key_main, h->c.ws);
}

int cfhe_hoisted_rotations(cfhe_context *h, int level, uint32_t *out,
                           const uint32_t *bx, const uint32_t *ax, int n_rot,
                           const int *rot, const uint32_t *const *evk_b,
                           const uint32_t *const *evk_a, int key_main) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!out || !bx || !ax || !rot || !evk_b || !evk_a) return fail("null argument");
  if (n_rot < 1) return fail("invalid rotation count");
  std::vector<uint32_t> galois(n_rot);
  for (int i = 0; i < n_rot; i++) {
    if (rot[i] == 0 || rot[i] >= h->c.n / 2) return fail("rotation distance out of range");
    galois[i] = cfhe_galois_for_rotation(h, rot[i]);
  }
  if (int r = ensure_workspace(h->c, hoisted_scratch_words(*lp))) return r;
  return run_hoisted_rotations(h->c, *lp, out, bx, ax, n_rot, galois.data(), evk_b,
                               evk_a, key_main, h->c.ws);
}

int cfhe_linear_transform(cfhe_context *h, int level, int rescale, uint32_t *out_b,
                          uint32_t *out_a, const uint32_t *in_b, const uint32_t *in_a,
                          int n_baby, const int *baby_rot,
                          const uint32_t *const *baby_evk_b, const uint32_t *const *baby_evk_a,
                          int n_giant, const int *giant_rot,
                          const uint32_t *const *giant_evk_b, const uint32_t *const *giant_evk_a,
                          const uint32_t *const *pt, int key_main) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!out_b || !out_a || !in_b || !in_a || !baby_rot || !giant_rot || !pt)
    return fail("null argument");
  if (n_baby < 1 || n_baby > kMaxBaby || n_giant < 1 || n_giant > kMaxGiant)
    return fail("linear transform: at most 16 baby and 16 giant steps");
  if (baby_rot[0] != 0) return fail("linear transform: the first baby step must be the identity");
  const int half = h->c.n / 2;
  std::vector<uint32_t> bg(n_baby), gg(n_giant);
  bool need_baby_keys = false, need_giant_keys = false;
  for (int i = 0; i < n_baby; i++) {
    if (baby_rot[i] < 0 || baby_rot[i] >= half || (i > 0 && baby_rot[i] == 0))
      return fail("rotation distance out of range");
    bg[i] = baby_rot[i] ? cfhe_galois_for_rotation(h, baby_rot[i]) : 1u;
    need_baby_keys = need_baby_keys || baby_rot[i] != 0;
  }
  for (int j = 0; j < n_giant; j++) {
    if (giant_rot[j] < 0 || giant_rot[j] >= half) return fail("rotation distance out of range");
    gg[j] = giant_rot[j] ? cfhe_galois_for_rotation(h, giant_rot[j]) : 1u;
    need_giant_keys = need_giant_keys || giant_rot[j] != 0;
  }
  if ((need_baby_keys && (!baby_evk_b || !baby_evk_a)) ||
      (need_giant_keys && (!giant_evk_b || !giant_evk_a)))
    return fail("null argument");
  if (int r = ensure_workspace(h->c, linear_transform_scratch_words(*lp, n_baby, n_giant, rescale != 0,
                                                              !h->c.use_fused_lt)))
    return r;
  return run_linear_transform(h->c, *lp, rescale != 0, out_b, out_a, in_b, in_a, n_baby, bg.data(),
                              baby_evk_b, baby_evk_a, n_giant, gg.data(), giant_evk_b,
                              giant_evk_a, pt, key_main, h->c.ws);
}

int cfhe_hmult(cfhe_context *h, int level, uint32_t *out_b, uint32_t *out_a,
               const uint32_t *b1, const uint32_t *a1, const uint32_t *b2,
               const uint32_t *a2, const uint32_t *const *evk_b,
               const uint32_t *const *evk_a, int key_main, int rescale) {
  CFHE_ENTER(h);
  const LevelPlan *lp = get_plan(h, level);
  if (!lp) return -1;
  if (!out_b || !out_a || !b1 || !a1 || !b2 || !a2 || !evk_b || !evk_a)
    return fail("null argument");
  const int type = rescale ? 2 : 0;
  if (rescale && !lp->has_rescale) return fail("level cannot be rescaled");
  const size_t tw = (size_t)lp->nq * kN;
  if (int r = ensure_workspace(h->c, 3 * tw + keyswitch_scratch_words(*lp, type)))
    return r;
  uint32_t *d0 = h->c.ws, *d1 = d0 + tw, *d2 = d1 + tw, *scratch = d2 + tw;
  if (int r = run_tensor(h->c, *lp, d0, d1, d2, b1, a1, b2, a2)) return r;
  return run_keyswitch(h->c, *lp, type, out_b, out_a, d2, d0, d1, evk_b, evk_a,
                       key_main, scratch);
}

// ---------------------------------------------------------------------------
// stage timing
// ---------------------------------------------------------------------------
int cfhe_profile_begin(cfhe_context *h) {
  if (!h) return fail("null context");
  h->c.profiling = true;
  h->c.prof_used = 0;
  h->c.mark("begin");
  return 0;
}

int cfhe_profile_end(cfhe_context *h, char *names, size_t names_cap, float *ms,
                     int cap) {
  CFHE_ENTER(h);
  if (!h) return fail("null context");
  Context &c = h->c;
  c.profiling = false;
  CFHE_CUDA(cudaStreamSynchronize(c.stream));
  int n = 0;
  size_t off = 0;
  if (names && names_cap) names[0] = 0;
  for (size_t i = 1; i < c.prof_used && n < cap; i++, n++) {
    CFHE_CUDA(cudaEventElapsedTime(&ms[n], c.prof_events[i - 1], c.prof_events[i]));
    const size_t len = strlen(c.prof_names[i]);
    if (names && off + len + 2 <= names_cap) {
      memcpy(names + off, c.prof_names[i], len);
      names[off + len] = ';';
      names[off + len + 1] = 0;
      off += len + 1;
    }
  }
  return n;
}

}  // extern "C"
