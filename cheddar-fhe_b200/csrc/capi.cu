// extern "C" boundary of libcheddar_b200.so (see include/cheddar_b200.h).
#include "../../include/cheddar_b200.h"

#include <string.h>

#include <new>

#include "context.h"
#include "host_math.h"

struct cfhe_context {
  cfhe::Context c;
};

namespace cfhe {
static thread_local std::string g_error;
void set_error(const std::string &msg) { g_error = msg; }
const std::string &get_error() { return g_error; }

static int fail(const std::string &msg) {
  set_error(msg);
  return -1;
}

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
    a.src_limb[l] = a.dst_limb[l] = (uint8_t)l;
  }
  a.n_limbs = n_limbs;
  return 0;
}
}  // namespace cfhe

using namespace cfhe;

extern "C" {

const char *cfhe_last_error(void) { return get_error().c_str(); }

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
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return cleanup_fail(cudaGetErrorString(e));
  e = cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return cleanup_fail(cudaGetErrorString(e));
  c.own_stream = true;
  const size_t tsz = (size_t)c.NP * c.n;
  std::vector<Tw> fwd(tsz), inv(tsz);
  c.psi.resize(c.NP);
  for (int g = 0; g < c.NP; g++)
    build_twiddles(c.q[g], c.logn, fwd.data() + (size_t)g * c.n,
                   inv.data() + (size_t)g * c.n, &c.psi[g]);
  e = cudaMalloc(&c.d_tw, tsz * sizeof(Tw));
  if (e == cudaSuccess) e = cudaMalloc(&c.d_itw, tsz * sizeof(Tw));
  if (e == cudaSuccess)
    e = cudaMemcpy(c.d_tw, fwd.data(), tsz * sizeof(Tw), cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaMemcpy(c.d_itw, inv.data(), tsz * sizeof(Tw), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return cleanup_fail(cudaGetErrorString(e));
  *out = h;
  return 0;
}

void cfhe_context_destroy(cfhe_context *h) {
  if (!h) return;
  Context &c = h->c;
  if (c.d_tw) cudaFree(c.d_tw);
  if (c.d_itw) cudaFree(c.d_itw);
  if (c.own_stream && c.stream) cudaStreamDestroy(c.stream);
  delete h;
}

int cfhe_set_stream(cfhe_context *h, void *cuda_stream) {
  if (!h) return fail("null context");
  Context &c = h->c;
  if (c.own_stream && c.stream) {
    cudaStreamSynchronize(c.stream);
    cudaStreamDestroy(c.stream);
    c.stream = nullptr;
    c.own_stream = false;
  }
  if (cuda_stream) {
    c.stream = (cudaStream_t)cuda_stream;
  } else {
    CFHE_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    c.own_stream = true;
  }
  return 0;
}

int cfhe_synchronize(cfhe_context *h) {
  if (!h) return fail("null context");
  CFHE_CUDA(cudaStreamSynchronize(h->c.stream));
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

int cfhe_malloc(cfhe_context *h, void **ptr, size_t bytes) {
  if (!h || !ptr) return fail("null argument");
  CFHE_CUDA(cudaMalloc(ptr, bytes));
  return 0;
}

int cfhe_free(cfhe_context *h, void *ptr) {
  if (!h) return fail("null context");
  CFHE_CUDA(cudaFree(ptr));
  return 0;
}

int cfhe_copy_h2d(cfhe_context *h, void *dst, const void *src, size_t bytes) {
  if (!h) return fail("null context");
  CFHE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, h->c.stream));
  return 0;
}

int cfhe_copy_d2h(cfhe_context *h, void *dst, const void *src, size_t bytes) {
  if (!h) return fail("null context");
  CFHE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, h->c.stream));
  CFHE_CUDA(cudaStreamSynchronize(h->c.stream));
  return 0;
}

int cfhe_ntt(cfhe_context *h, uint32_t *dst, const uint32_t *src,
             const int *gidx, int n_limbs, int n_polys,
             long long dst_poly_stride, long long src_poly_stride,
             int mont_conv) {
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
  return launch_ntt(c, a, false);
}

int cfhe_intt(cfhe_context *h, uint32_t *dst, const uint32_t *src,
              const int *gidx, int n_limbs, int n_polys,
              long long dst_poly_stride, long long src_poly_stride,
              const uint32_t *consts, int mont_keep, int centred) {
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
  return launch_ntt(c, a, true);
}

}  // extern "C"
