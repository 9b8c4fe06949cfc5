/*
 * Scalar CPU golden model of the CKKS RNS hot path. TEST INFRASTRUCTURE ONLY
 * (see cfhe_oracle.h). Every function names the reference code it restates.
 * The reference ships no golden vectors for this path; parity is pinned by the
 * reference itself: its CUDA sources, built unmodified, are fed the same device
 * buffers on a GPU and agree word for word with these functions, and the
 * SHA-256 digests of 27 of its outputs (tests/golden/reference_digests.json)
 * are checked against this file on the CPU.
 */
#include "cfhe_oracle.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef unsigned __int128 u128;
typedef __int128 i128;

struct orc_ctx {
  int logn, n;
  int num_main, num_ter, num_aux; /* maxima */
  int L;                          /* num_main + num_ter */
  int np;                         /* L + num_aux */
  int num_levels;
  int *level_main, *level_ter;
  int short_main, short_ter; /* level -1 base */
  uint32_t *q;               /* [np] global order */
  uint32_t *psi;             /* [np] */
  uint32_t *tw, *itw;        /* [np][n] plain psi^brev(j), psi^-brev(j) */
};

/* ------------------------------------------------------------------ */
/* number theory: include/common/PrimeUtils.h:57-248                   */
/* ------------------------------------------------------------------ */
uint32_t orc_mulmod(uint32_t a, uint32_t b, uint32_t q) {
  return (uint32_t)(((uint64_t)a * b) % q);
}

uint32_t orc_powmod(uint32_t a, uint64_t e, uint32_t q) {
  uint32_t r = 1 % q;
  a %= q;
  while (e) {
    if (e & 1) r = orc_mulmod(r, a, q);
    a = orc_mulmod(a, a, q);
    e >>= 1;
  }
  return r;
}

uint32_t orc_invmod(uint32_t a, uint32_t q) {
  /* q prime: a^(q-2); same value as the extended-Euclid result of
   * PrimeUtils.h:72-84 because the inverse mod a prime is unique. */
  return orc_powmod(a, (uint64_t)q - 2, q);
}

/* Smallest primitive root: PrimeUtils.h:135-174. */
uint32_t orc_find_generator(uint32_t q) {
  uint32_t phi = q - 1, fac[32], temp = phi;
  int nf = 0;
  for (uint32_t i = 2; (uint64_t)i * i <= temp; i++) {
    if (temp % i == 0) {
      fac[nf++] = i;
      while (temp % i == 0) temp /= i;
    }
  }
  if (temp > 1) fac[nf++] = temp;
  for (uint32_t r = 2; r <= phi; r++) {
    int ok = 1;
    for (int k = 0; k < nf; k++)
      if (orc_powmod(r, phi / fac[k], q) == 1) {
        ok = 0;
        break;
      }
    if (ok) return r;
  }
  return 0;
}

/* a * 2^32 mod q: PrimeUtils.h:242-248. */
uint32_t orc_to_mont(uint32_t a, uint32_t q) {
  return (uint32_t)((((uint64_t)a) << 32) % q);
}

static uint32_t rinv_mod(uint32_t q) { /* 2^-32 mod q */
  return orc_invmod((uint32_t)((1ULL << 32) % q), q);
}

/* a*b*2^-32 mod q in [0,q): include/common/Basic.cuh:251-260 reduces the
 * same quantity with a signed lazy Montgomery step then folds to [0,q). */
uint32_t orc_mont_mul(uint32_t a, uint32_t b, uint32_t q) {
  return orc_mulmod(orc_mulmod(a % q, b % q, q), rinv_mod(q), q);
}

/* signed x -> x * 2^-32 mod q in [0,q): Basic.cuh:150-157 */
static uint32_t mont_reduce_signed(i128 x, uint32_t q, uint32_t rinv) {
  i128 r = x % (i128)q;
  if (r < 0) r += q;
  return orc_mulmod((uint32_t)r, rinv, q);
}

/* q^-1 mod 2^32 as a signed word: PrimeUtils.h:205-232 */
static int32_t qinv_2_32(uint32_t q) {
  uint32_t x = q; /* Newton: correct to 3 bits, doubles each step */
  for (int i = 0; i < 5; i++) x *= 2u - q * x;
  return (int32_t)x;
}

static uint32_t brev(uint32_t v, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++) r |= ((v >> i) & 1u) << (bits - 1 - i);
  return r;
}

/* ------------------------------------------------------------------ */
/* context: src/core/Parameter.cu:20-136, src/core/NTT.cu:1233-1299    */
/* ------------------------------------------------------------------ */
orc_ctx *orc_create(int log_degree, const uint32_t *main_primes, int num_main,
                    const uint32_t *ter_primes, int num_ter,
                    const uint32_t *aux_primes, int num_aux,
                    const int *level_config, int num_levels, int add_main,
                    int add_ter) {
  orc_ctx *c = (orc_ctx *)calloc(1, sizeof(orc_ctx));
  c->logn = log_degree;
  c->n = 1 << log_degree;
  c->num_main = num_main;
  c->num_ter = num_ter;
  c->num_aux = num_aux;
  c->L = num_main + num_ter;
  c->np = c->L + num_aux;
  c->num_levels = num_levels;
  c->level_main = (int *)malloc(sizeof(int) * num_levels);
  c->level_ter = (int *)malloc(sizeof(int) * num_levels);
  for (int i = 0; i < num_levels; i++) {
    c->level_main[i] = level_config[2 * i];
    c->level_ter[i] = level_config[2 * i + 1];
  }
  /* Parameter.cu:133-142 */
  c->short_main = c->level_main[0] - add_main;
  c->short_ter = c->level_ter[0] - add_ter;
  c->q = (uint32_t *)malloc(sizeof(uint32_t) * c->np);
  c->psi = (uint32_t *)malloc(sizeof(uint32_t) * c->np);
  /* Parameter.cu:104-105: terminal primes reversed, then main; aux last */
  for (int i = 0; i < num_ter; i++) c->q[i] = ter_primes[num_ter - 1 - i];
  for (int i = 0; i < num_main; i++) c->q[num_ter + i] = main_primes[i];
  for (int i = 0; i < num_aux; i++) c->q[c->L + i] = aux_primes[i];
  size_t tsz = (size_t)c->np * c->n;
  c->tw = (uint32_t *)malloc(sizeof(uint32_t) * tsz);
  c->itw = (uint32_t *)malloc(sizeof(uint32_t) * tsz);
  uint32_t *pw = (uint32_t *)malloc(sizeof(uint32_t) * c->n);
  for (int g = 0; g < c->np; g++) {
    uint32_t q = c->q[g];
    /* PrimeUtils.h:184-196: psi = g^((q-1)/2N) for the smallest generator */
    uint32_t gen = orc_find_generator(q);
    uint32_t psi = orc_powmod(gen, (q - 1) / (2u * c->n), q);
    uint32_t ipsi = orc_invmod(psi, q);
    c->psi[g] = psi;
    /* NTT.cu:1264-1271: successive powers, then bit-reversal permutation */
    pw[0] = 1;
    for (int j = 1; j < c->n; j++) pw[j] = orc_mulmod(pw[j - 1], psi, q);
    for (int j = 0; j < c->n; j++)
      c->tw[(size_t)g * c->n + j] = pw[brev(j, c->logn)];
    pw[0] = 1;
    for (int j = 1; j < c->n; j++) pw[j] = orc_mulmod(pw[j - 1], ipsi, q);
    for (int j = 0; j < c->n; j++)
      c->itw[(size_t)g * c->n + j] = pw[brev(j, c->logn)];
  }
  free(pw);
  return c;
}

void orc_destroy(orc_ctx *c) {
  if (!c) return;
  free(c->level_main);
  free(c->level_ter);
  free(c->q);
  free(c->psi);
  free(c->tw);
  free(c->itw);
  free(c);
}

int orc_degree(const orc_ctx *c) { return c->n; }
int orc_num_primes(const orc_ctx *c) { return c->np; }
uint32_t orc_prime(const orc_ctx *c, int g) { return c->q[g]; }
uint32_t orc_psi(const orc_ctx *c, int g) { return c->psi[g]; }
int32_t orc_qinv(const orc_ctx *c, int g) { return qinv_2_32(c->q[g]); }

static void level_np(const orc_ctx *c, int level, int *nm, int *nt) {
  if (level == -1) { /* Parameter.cu:283-289 */
    *nm = c->short_main;
    *nt = c->short_ter;
  } else {
    *nm = c->level_main[level];
    *nt = c->level_ter[level];
  }
}

/* Parameter.cu:318-325 (GetPrimeVector) */
static int np_limbs(const orc_ctx *c, int nm, int nt, int na, int *gidx) {
  int k = 0;
  for (int g = c->num_ter - nt; g < c->num_ter + nm; g++) gidx[k++] = g;
  for (int a = 0; a < na; a++) gidx[k++] = c->L + a;
  return k;
}

int orc_level_limbs(const orc_ctx *c, int level, int num_aux, int *gidx) {
  int nm, nt;
  level_np(c, level, &nm, &nt);
  return np_limbs(c, nm, nt, num_aux, gidx);
}

static int level_alpha(const orc_ctx *c, int level) {
  /* ModSwitch.cu:180: the short base uses its own limb count as alpha */
  return level == -1 ? c->short_main + c->short_ter : c->num_aux;
}

int orc_beta(const orc_ctx *c, int level) {
  /* ModSwitch.cu:181-185 */
  if (level == -1) return 1;
  int a = c->num_aux;
  return (c->level_main[level] + c->num_ter + a - 1) / a;
}

/* ------------------------------------------------------------------ */
/* transforms: src/core/NTT.cu:606-813, include/core/NTTUtils.cuh:19-60 */
/* ------------------------------------------------------------------ */
static void ntt_limb(const orc_ctx *c, uint32_t *a, int g) {
  uint32_t q = c->q[g];
  const uint32_t *tw = c->tw + (size_t)g * c->n;
  int n = c->n;
  for (int m = 1, t = n >> 1; m < n; m <<= 1, t >>= 1) {
    for (int i = 0; i < m; i++) {
      uint32_t w = tw[m + i];
      uint32_t *x = a + 2 * i * t;
      for (int j = 0; j < t; j++) {
        uint32_t u = x[j], v = orc_mulmod(x[j + t], w, q);
        uint32_t s = u + v;
        if (s >= q) s -= q;
        uint32_t d = u >= v ? u - v : u + q - v;
        x[j] = s;
        x[j + t] = d;
      }
    }
  }
}

static void intt_limb_raw(const orc_ctx *c, uint32_t *a, int g) {
  uint32_t q = c->q[g];
  const uint32_t *tw = c->itw + (size_t)g * c->n;
  int n = c->n;
  for (int m = n >> 1, t = 1; m >= 1; m >>= 1, t <<= 1) {
    for (int i = 0; i < m; i++) {
      uint32_t w = tw[m + i];
      uint32_t *x = a + 2 * i * t;
      for (int j = 0; j < t; j++) {
        uint32_t u = x[j], v = x[j + t];
        uint32_t s = u + v;
        if (s >= q) s -= q;
        uint32_t d = u >= v ? u - v : u + q - v;
        x[j] = s;
        x[j + t] = orc_mulmod(d, w, q);
      }
    }
  }
}

void orc_ntt(const orc_ctx *c, uint32_t *dst, const uint32_t *src,
             const int *gidx, int nlimbs, int mont_conv) {
  int n = c->n;
  for (int l = 0; l < nlimbs; l++) {
    int g = gidx[l];
    uint32_t q = c->q[g];
    uint32_t *d = dst + (size_t)l * n;
    const uint32_t *s = src + (size_t)l * n;
    if (mont_conv) {
      /* NTT.cu:286-293 with montgomery_converter_ = 2^64 mod q
       * (NTT.cu:1258-1259): Mont(x, R^2) = x*R */
      for (int j = 0; j < n; j++) d[j] = orc_to_mont(s[j] % q, q);
    } else {
      for (int j = 0; j < n; j++) d[j] = s[j] % q;
    }
    ntt_limb(c, d, g);
  }
}

void orc_intt(const orc_ctx *c, uint32_t *dst, const uint32_t *src,
              const int *gidx, int nlimbs, const uint32_t *consts,
              int mode_mont_keep, int centred) {
  int n = c->n;
  for (int l = 0; l < nlimbs; l++) {
    int g = gidx[l];
    uint32_t q = c->q[g];
    uint32_t *d = dst + (size_t)l * n;
    if (d != src + (size_t)l * n) memcpy(d, src + (size_t)l * n, 4u * n);
    intt_limb_raw(c, d, g);
    uint32_t k;
    if (consts) {
      k = consts[l];
    } else {
      /* NTT.cu:703-709, 1256-1257 */
      uint32_t ninv = orc_invmod((uint32_t)n % q, q);
      k = mode_mont_keep ? orc_to_mont(ninv, q) : ninv;
    }
    for (int j = 0; j < n; j++) {
      uint32_t v = orc_mont_mul(d[j], k, q);
      /* NTTUtils.cuh:382-391 */
      if (centred && v > (q >> 1)) v -= q;
      d[j] = v;
    }
  }
}

/* ------------------------------------------------------------------ */
/* element-wise: src/core/ElementWise.cu:32-658                        */
/* ------------------------------------------------------------------ */
#define LIMB_LOOP                                \
  int n = c->n;                                  \
  for (int l = 0; l < nlimbs; l++) {             \
    uint32_t q = c->q[gidx[l]];                  \
    size_t o = (size_t)l * n;                    \
    for (int j = 0; j < n; j++) {                \
      size_t i = o + j;
#define LIMB_END \
  }              \
  }

void orc_add(const orc_ctx *c, uint32_t *d, const uint32_t *a,
             const uint32_t *b, const int *gidx, int nlimbs) {
  LIMB_LOOP
  uint32_t s = a[i] + b[i];
  d[i] = s >= q ? s - q : s;
  LIMB_END
}

void orc_sub(const orc_ctx *c, uint32_t *d, const uint32_t *a,
             const uint32_t *b, const int *gidx, int nlimbs) {
  LIMB_LOOP
  d[i] = a[i] >= b[i] ? a[i] - b[i] : a[i] + q - b[i];
  LIMB_END
}

void orc_neg(const orc_ctx *c, uint32_t *d, const uint32_t *a, const int *gidx,
             int nlimbs) {
  LIMB_LOOP
  d[i] = a[i] ? q - a[i] : 0;
  LIMB_END
}

void orc_mul(const orc_ctx *c, uint32_t *d, const uint32_t *a,
             const uint32_t *b, const int *gidx, int nlimbs) {
  int n = c->n;
  for (int l = 0; l < nlimbs; l++) {
    uint32_t q = c->q[gidx[l]], ri = rinv_mod(q);
    size_t o = (size_t)l * n;
    for (int j = 0; j < n; j++)
      d[o + j] = orc_mulmod(orc_mulmod(a[o + j], b[o + j], q), ri, q);
  }
}

/* ElementWise.cu:146-221 (const add/sub), :225-287 with one constant term */
void orc_const_op(const orc_ctx *c, uint32_t *d, const uint32_t *a,
                  const uint32_t *k, const int *gidx, int nlimbs, int op) {
  int n = c->n;
  for (int l = 0; l < nlimbs; l++) {
    uint32_t q = c->q[gidx[l]], ri = rinv_mod(q), kk = k[l];
    size_t o = (size_t)l * n;
    for (int j = 0; j < n; j++) {
      uint32_t x = a[o + j], r;
      switch (op) {
        case 0:
          r = x + kk;
          if (r >= q) r -= q;
          break;
        case 1:
          r = x >= kk ? x - kk : x + q - kk;
          break;
        case 2:
          r = kk >= x ? kk - x : kk + q - x;
          break;
        default:
          r = orc_mulmod(orc_mulmod(x, kk, q), ri, q);
      }
      d[o + j] = r;
    }
  }
}

/* ElementWise.cu:504-546: (b1b2, b1a2+a1b2, a1a2), all Montgomery products */
void orc_tensor(const orc_ctx *c, uint32_t *d0, uint32_t *d1, uint32_t *d2,
                const uint32_t *b1, const uint32_t *a1, const uint32_t *b2,
                const uint32_t *a2, const int *gidx, int nlimbs) {
  int n = c->n;
  for (int l = 0; l < nlimbs; l++) {
    uint32_t q = c->q[gidx[l]], ri = rinv_mod(q);
    size_t o = (size_t)l * n;
    for (int j = 0; j < n; j++) {
      size_t i = o + j;
      uint32_t bb = orc_mulmod(orc_mulmod(b1[i], b2[i], q), ri, q);
      uint32_t aa = orc_mulmod(orc_mulmod(a1[i], a2[i], q), ri, q);
      uint32_t ba = orc_mulmod(orc_mulmod(b1[i], a2[i], q), ri, q);
      uint32_t ab = orc_mulmod(orc_mulmod(a1[i], b2[i], q), ri, q);
      uint32_t s = ba + ab;
      if (s >= q) s -= q;
      d0[i] = bb;
      d1[i] = s;
      d2[i] = aa;
    }
  }
}

/* Parameter.cu:93-101 (5^r mod 2N); ElementWise.cu:955-964 (-1 -> 2N-1) */
uint32_t orc_galois_for_rotation(const orc_ctx *c, int rot) {
  uint32_t m = 2u * c->n;
  if (rot < 0) return m - 1;
  uint32_t g = 1;
  for (int i = 0; i < rot; i++) g = (uint32_t)(((uint64_t)g * 5u) % m);
  return g;
}

/* ElementWise.cu:370-391 */
void orc_permute(const orc_ctx *c, uint32_t *d, const uint32_t *a,
                 uint32_t galois, int nlimbs) {
  int n = c->n, lb = c->logn + 1;
  uint32_t mask = 2u * n - 1;
  for (int l = 0; l < nlimbs; l++) {
    size_t o = (size_t)l * n;
    for (int j = 0; j < n; j++) {
      uint32_t e = brev((uint32_t)j, lb) + 1;
      uint32_t s = brev((e * galois - 1) & mask, lb);
      d[o + j] = a[o + s];
    }
  }
}

/* ElementWise.cu:625-658; the unit is tw[1] = psi^(N/2) (NTT.cu:1301-1310) */
void orc_mul_imag_unit(const orc_ctx *c, uint32_t *d, const uint32_t *a,
                       const int *gidx, int nlimbs) {
  int n = c->n;
  for (int l = 0; l < nlimbs; l++) {
    int g = gidx[l];
    uint32_t q = c->q[g];
    uint32_t u = c->tw[(size_t)g * n + 1];
    size_t o = (size_t)l * n;
    for (int j = 0; j < n; j++) {
      uint32_t w = (j & (n >> 1)) ? q - u : u;
      d[o + j] = orc_mulmod(a[o + j], w, q);
    }
  }
}

/* ------------------------------------------------------------------ */
/* base conversion: src/core/ModSwitch.cu:23-171, 320-370              */
/* ------------------------------------------------------------------ */
static int32_t centre(uint32_t a, uint32_t q) { /* Basic.cuh:231-239 */
  return a > (q >> 1) ? (int32_t)(a - q) : (int32_t)a;
}

/* T[m][k] = centred( (prod_{j!=k} s_j mod d_m) * 2^64 mod d_m ) */
static void bconv_table(const orc_ctx *c, int32_t *T, const int *sg, int ns,
                        const int *dg, int nd) {
  for (int m = 0; m < nd; m++) {
    uint32_t p = c->q[dg[m]];
    for (int k = 0; k < ns; k++) {
      uint32_t acc = 1;
      for (int j = 0; j < ns; j++)
        if (j != k) acc = orc_mulmod(acc, c->q[sg[j]] % p, p);
      acc = orc_to_mont(orc_to_mont(acc, p), p);
      T[m * ns + k] = centre(acc, p);
    }
  }
}

void orc_bconv(const orc_ctx *c, uint32_t *dst, const int32_t *y,
               const int *src_gidx, int n_src, const int *dst_gidx,
               int n_dst) {
  int n = c->n;
  int32_t *T = (int32_t *)malloc(sizeof(int32_t) * n_src * n_dst);
  bconv_table(c, T, src_gidx, n_src, dst_gidx, n_dst);
  for (int m = 0; m < n_dst; m++) {
    uint32_t p = c->q[dst_gidx[m]], ri = rinv_mod(p);
    for (int j = 0; j < n; j++) {
      i128 acc = 0;
      for (int k = 0; k < n_src; k++)
        acc += (i128)y[(size_t)k * n + j] * T[m * n_src + k];
      dst[(size_t)m * n + j] = mont_reduce_signed(acc, p, ri);
    }
  }
  free(T);
}

/* c1[k] = ((prod_{j!=k} s_j) * N)^-1 * prod(restored) mod s_k, plain:
 * ModSwitch.cu:331-352 */
static void bconv_pre_consts(const orc_ctx *c, uint32_t *c1, const int *sg,
                             int ns, const int *restored, int nr) {
  for (int k = 0; k < ns; k++) {
    uint32_t s = c->q[sg[k]], acc = 1;
    for (int j = 0; j < ns; j++)
      if (j != k) acc = orc_mulmod(acc, c->q[sg[j]] % s, s);
    acc = orc_mulmod(acc, (uint32_t)c->n % s, s);
    acc = orc_invmod(acc, s);
    for (int j = 0; j < nr; j++)
      acc = orc_mulmod(acc, c->q[restored[j]] % s, s);
    c1[k] = acc;
  }
}

/* ------------------------------------------------------------------ */
/* ModUp: src/core/ModSwitch.cu:429-509 (+ constants :204-236)          */
/* ------------------------------------------------------------------ */
void orc_modup(const orc_ctx *c, int level, uint32_t *dst,
               const uint32_t *src) {
  int n = c->n, nm, nt;
  level_np(c, level, &nm, &nt);
  int alpha = level_alpha(c, level);
  int beta = orc_beta(c, level);
  int lim[128], nq = np_limbs(c, nm, nt, 0, lim);
  int full[128], ntot = np_limbs(c, nm, nt, alpha, full);
  int off = level == -1 ? 0 : c->num_ter - nt;
  int padded = nq + off;
  int32_t *y = (int32_t *)malloc(sizeof(int32_t) * (size_t)alpha * n);
  for (int i = 0; i < beta; i++) {
    int s0 = i * alpha, s1 = (i + 1) * alpha;
    if (s1 > padded) s1 = padded;
    if (s1 <= off) continue;
    s0 = s0 - off < 0 ? 0 : s0 - off;
    s1 -= off;
    int ns = s1 - s0;
    uint32_t *out = dst + (size_t)i * ntot * n;
    /* own limbs are copied: ModSwitch.cu:466-470 */
    memcpy(out + (size_t)s0 * n, src + (size_t)s0 * n, 4u * (size_t)ns * n);
    uint32_t c1[64];
    bconv_pre_consts(c, c1, lim + s0, ns, NULL, 0);
    /* INTTAndMultConst(normalize=true): ModSwitch.cu:442-445 */
    orc_intt(c, (uint32_t *)y, src + (size_t)s0 * n, lim + s0, ns, c1, 0, 1);
    int dg[128], nd = 0;
    for (int k = 0; k < ntot; k++)
      if (k < s0 || k >= s1) dg[nd++] = full[k];
    uint32_t *tmp = (uint32_t *)malloc(4u * (size_t)nd * n);
    orc_bconv(c, tmp, y, lim + s0, ns, dg, nd);
    /* NTTForModUp: no conversion, the table carries 2^64 (NTT.cu:858-869) */
    orc_ntt(c, tmp, tmp, dg, nd, 0);
    int r = 0;
    for (int k = 0; k < ntot; k++)
      if (k < s0 || k >= s1)
        memcpy(out + (size_t)k * n, tmp + (size_t)(r++) * n, 4u * n);
    free(tmp);
  }
  free(y);
}

/* ------------------------------------------------------------------ */
/* ModDown / Rescale / ModDownAndRescale:                              */
/* src/core/ModSwitch.cu:242-303, 372-411, 566-684; NTT.cu:562-600      */
/* ------------------------------------------------------------------ */
void orc_moddown(const orc_ctx *c, int level, int type, uint32_t *dst,
                 const uint32_t *src) {
  int n = c->n;
  int sm, st, dm, dt;
  int alpha = level_alpha(c, level);
  level_np(c, level, &sm, &st);
  level_np(c, type == 0 ? level : level - 1, &dm, &dt);
  int src_aux = type == 1 ? 0 : alpha;
  int km = sm < dm ? sm : dm, kt = st < dt ? st : dt; /* kept ("non-INTT") */
  int sl[128], ns_tot = np_limbs(c, sm, st, src_aux, sl);
  int dl[128], nd = np_limbs(c, dm, dt, 0, dl);
  /* source limbs of the conversion = limbs of src that do not survive */
  int sg[64], spos[64], ns = 0;
  for (int k = 0; k < ns_tot; k++) {
    int g = sl[k];
    int survives = g < c->L && g >= c->num_ter - kt && g < c->num_ter + km;
    if (!survives) {
      sg[ns] = g;
      spos[ns++] = k;
    }
  }
  /* restored limbs = limbs of dst absent from src */
  int rg[64], nr = 0;
  for (int k = 0; k < nd; k++) {
    int g = dl[k];
    int in_src = g >= c->num_ter - st && g < c->num_ter + sm;
    if (!in_src) rg[nr++] = g;
  }
  uint32_t c1[64];
  bconv_pre_consts(c, c1, sg, ns, rg, nr);
  int32_t *y = (int32_t *)malloc(4u * (size_t)ns * n);
  for (int k = 0; k < ns; k++)
    orc_intt(c, (uint32_t *)y + (size_t)k * n, src + (size_t)spos[k] * n,
             sg + k, 1, c1 + k, 0, 1);
  uint32_t *t = (uint32_t *)malloc(4u * (size_t)nd * n);
  orc_bconv(c, t, y, sg, ns, dl, nd);
  orc_ntt(c, t, t, dl, nd, 0);
  for (int m = 0; m < nd; m++) {
    int g = dl[m];
    uint32_t p = c->q[g];
    /* (prod S)^-1 mod p: ModSwitch.cu:381-391 */
    uint32_t ps = 1;
    for (int k = 0; k < ns; k++) ps = orc_mulmod(ps, c->q[sg[k]] % p, p);
    uint32_t ips = orc_invmod(ps, p);
    /* padding = prod of restored primes: ModSwitch.cu:397-410 */
    uint32_t pad = 1;
    for (int k = 0; k < nr; k++) pad = orc_mulmod(pad, c->q[rg[k]] % p, p);
    int spos_m = -1;
    for (int k = 0; k < ns_tot; k++)
      if (sl[k] == g) spos_m = k;
    for (int j = 0; j < n; j++) {
      uint32_t x = 0;
      if (spos_m >= 0) x = orc_mulmod(src[(size_t)spos_m * n + j], pad, p);
      uint32_t v = t[(size_t)m * n + j];
      uint32_t d = x >= v ? x - v : x + p - v;
      dst[(size_t)m * n + j] = orc_mulmod(d, ips, p);
    }
  }
  free(t);
  free(y);
}

/* ------------------------------------------------------------------ */
/* key switching: src/core/Context.cpp:609-712;                        */
/* inner product kernel src/core/ElementWise.cu:225-287                 */
/* ------------------------------------------------------------------ */
void orc_evk_inner(const orc_ctx *c, int level, uint32_t *acc_b,
                   uint32_t *acc_a, const uint32_t *modup,
                   const uint32_t *const *evk_b, const uint32_t *const *evk_a,
                   int key_main) {
  int n = c->n, nm, nt;
  level_np(c, level, &nm, &nt);
  int alpha = level_alpha(c, level);
  int beta = orc_beta(c, level);
  int full[128], ntot = np_limbs(c, nm, nt, alpha, full);
  int off = level == -1 ? 0 : c->num_ter - nt;
  int padded = nm + nt + off;
  /* key limb position of global prime g: the key holds every terminal limb
   * (or, on the short base, exactly the base's limbs), key_main main limbs
   * and alpha aux limbs. */
  int key_ter = level == -1 ? nt : c->num_ter;
  memset(acc_b, 0, 4u * (size_t)ntot * n);
  memset(acc_a, 0, 4u * (size_t)ntot * n);
  for (int i = 0; i < beta; i++) {
    int s1 = (i + 1) * alpha;
    if (s1 > padded) s1 = padded;
    if (s1 <= off) continue; /* Context.cpp:640-645 */
    const uint32_t *mu = modup + (size_t)i * ntot * n;
    for (int l = 0; l < ntot; l++) {
      int g = full[l];
      int kpos = g < c->L ? g - (c->num_ter - key_ter)
                          : key_ter + key_main + (g - c->L);
      uint32_t q = c->q[g], ri = rinv_mod(q);
      const uint32_t *kb = evk_b[i] + (size_t)kpos * n;
      const uint32_t *ka = evk_a[i] + (size_t)kpos * n;
      for (int j = 0; j < n; j++) {
        uint32_t x = mu[(size_t)l * n + j];
        uint32_t pb = orc_mulmod(orc_mulmod(x, kb[j], q), ri, q);
        uint32_t pa = orc_mulmod(orc_mulmod(x, ka[j], q), ri, q);
        uint32_t sb = acc_b[(size_t)l * n + j] + pb;
        uint32_t sa = acc_a[(size_t)l * n + j] + pa;
        acc_b[(size_t)l * n + j] = sb >= q ? sb - q : sb;
        acc_a[(size_t)l * n + j] = sa >= q ? sa - q : sa;
      }
    }
  }
}

/* Context.cpp:85-98 (P mod q in M-form) and :688-699 (CAccum) */
void orc_add_p_times(const orc_ctx *c, int level, uint32_t *acc,
                     const uint32_t *x) {
  int n = c->n, nm, nt;
  level_np(c, level, &nm, &nt);
  int alpha = level_alpha(c, level);
  int lim[128], nq = np_limbs(c, nm, nt, 0, lim);
  int aux[64];
  /* P = product of the first alpha auxiliary primes (all of them except on
   * the short base, Context.cpp:100-123) */
  for (int a = 0; a < alpha; a++) aux[a] = c->L + a;
  for (int l = 0; l < nq; l++) {
    uint32_t q = c->q[lim[l]], pp = 1;
    for (int a = 0; a < alpha; a++) pp = orc_mulmod(pp, c->q[aux[a]] % q, q);
    for (int j = 0; j < n; j++) {
      size_t i = (size_t)l * n + j;
      uint32_t s = acc[i] + orc_mulmod(x[i], pp, q);
      acc[i] = s >= q ? s - q : s;
    }
  }
}

void orc_hmult(const orc_ctx *c, int level, uint32_t *out_b, uint32_t *out_a,
               const uint32_t *b1, const uint32_t *a1, const uint32_t *b2,
               const uint32_t *a2, const uint32_t *const *evk_b,
               const uint32_t *const *evk_a, int key_main, int rescale) {
  int n = c->n, nm, nt;
  level_np(c, level, &nm, &nt);
  int alpha = level_alpha(c, level), beta = orc_beta(c, level);
  int lim[128], nq = np_limbs(c, nm, nt, 0, lim);
  int ntot = nq + alpha;
  size_t lsz = (size_t)nq * n, fsz = (size_t)ntot * n;
  uint32_t *d0 = (uint32_t *)malloc(4 * lsz), *d1 = (uint32_t *)malloc(4 * lsz),
           *d2 = (uint32_t *)malloc(4 * lsz);
  uint32_t *mu = (uint32_t *)calloc(fsz * beta, 4);
  uint32_t *ab = (uint32_t *)malloc(4 * fsz), *aa = (uint32_t *)malloc(4 * fsz);
  /* Context.cpp:862-871 -> :316-330 -> :714-737 */
  orc_tensor(c, d0, d1, d2, b1, a1, b2, a2, lim, nq);
  orc_modup(c, level, mu, d2);
  orc_evk_inner(c, level, ab, aa, mu, evk_b, evk_a, key_main);
  orc_add_p_times(c, level, ab, d0);
  orc_add_p_times(c, level, aa, d1);
  orc_moddown(c, level, rescale ? 2 : 0, out_b, ab);
  orc_moddown(c, level, rescale ? 2 : 0, out_a, aa);
  free(d0);
  free(d1);
  free(d2);
  free(mu);
  free(ab);
  free(aa);
}

/* Context.cpp:584-607 with a.HasRx() == false (:700-711) */
void orc_keyswitch(const orc_ctx *c, int level, uint32_t *out_b,
                   uint32_t *out_a, const uint32_t *d, const uint32_t *bx,
                   const uint32_t *const *evk_b, const uint32_t *const *evk_a,
                   int key_main) {
  int n = c->n, nm, nt;
  level_np(c, level, &nm, &nt);
  int alpha = level_alpha(c, level), beta = orc_beta(c, level);
  int ntot = nm + nt + alpha;
  size_t fsz = (size_t)ntot * n;
  uint32_t *mu = (uint32_t *)calloc(fsz * beta, 4);
  uint32_t *ab = (uint32_t *)malloc(4 * fsz), *aa = (uint32_t *)malloc(4 * fsz);
  orc_modup(c, level, mu, d);
  orc_evk_inner(c, level, ab, aa, mu, evk_b, evk_a, key_main);
  orc_add_p_times(c, level, ab, bx);
  orc_moddown(c, level, 0, out_b, ab);
  orc_moddown(c, level, 0, out_a, aa);
  free(mu);
  free(ab);
  free(aa);
}
