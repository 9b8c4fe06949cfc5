// Level-aware pipelines: ModUp, the ModDown family, the evaluation-key inner
// product, key switching and HMult, composed from the kernels of this library.
// They follow the algebra of the reference's ModSwitchHandler
// (src/core/ModSwitch.cu:429-684) and Context (src/core/Context.cpp:584-871)
// with fewer launches: every digit's base conversion shares one launch, all
// digits' forward transforms share one launch, the digit's own limbs are read
// in place instead of copied, P*(b,a) is folded into the inner product, and
// both polynomials of a ciphertext go through ModDown together.
#include <string.h>

#include "host_math.h"
#include "pipeline.h"

namespace cfhe {
namespace {

void fill_bconv_job(const Context &c, BconvJob &j, const ConvPlan &cv,
                    const int32_t *src, uint32_t *dst,
                    const std::vector<int> *dst_pos) {
  j.src = src;
  j.dst = dst;
  j.table = cv.d_table;
  j.ns = (int)cv.src_g.size();
  j.nd = (int)cv.dst_g.size();
  for (int m = 0; m < j.nd; m++) {
    const int g = cv.dst_g[m];
    j.dst_limb[m] = (uint8_t)(dst_pos ? (*dst_pos)[m] : m);
    j.q[m] = c.q[g];
    j.qinv[m] = 0u - c.nqinv[g];
  }
}

void fill_tc_job(const Context &c, BconvTcJob &j, const ConvPlan &cv,
                 const uint32_t *src, uint32_t *dst,
                 const std::vector<int> *dst_pos) {
  j.src = src;
  j.dst = dst;
  j.btile = cv.d_tc_table;
  j.ns = (int)cv.src_g.size();
  j.nd = (int)cv.dst_g.size();
  j.kpad = cv.tc_kpad;
  j.npad = cv.tc_npad;
  for (int k = 0; k < kMaxBconvSrc + 3; k++)
    j.half[k] = k < j.ns ? c.q[cv.src_g[k]] >> 1 : 0xffffffffu;  // repeats past the last source never count
  for (int m = 0; m < j.nd; m++) {
    const int g = cv.dst_g[m];
    j.dst_limb[m] = (uint8_t)(dst_pos ? (*dst_pos)[m] : m);
    j.q[m] = c.q[g];
    j.nqinv[m] = c.nqinv[g];
  }
}

}  // namespace

size_t modup_scratch_words(const LevelPlan &lp) { return (size_t)lp.nq * kN; }

int run_modup(const Context &c, const LevelPlan &lp, uint32_t *mu,
              const uint32_t *src, bool copy_own, uint32_t *y) {
  if (lp.digits.empty()) {
    set_error("ModUp: level has no digits");
    return -1;
  }
  // 1. inverse transform of every Q limb, pre-scaled and centred
  NttArgs a;
  memset(&a, 0, sizeof(a));
  a.dst = y;
  a.src = src;
  a.table = c.d_itw;
  bool tc = c.use_tc_bconv;
  for (const DigitPlan &d : lp.digits) tc = tc && d.conv.d_tc_table;
  a.n_limbs = lp.nq;
  a.n_polys = 1;
  a.centred = tc ? 0 : 1;  // the tensor-core conversion takes canonical residues
  for (const DigitPlan &d : lp.digits)
    for (int k = d.s0; k < d.s1; k++) {
      const int g = lp.q_g[k];
      a.g[k] = (uint8_t)g;
      a.q[k] = c.q[g];
      a.src_limb[k] = a.dst_limb[k] = (uint16_t)k;
      a.kc[k] = d.conv.pre_tw[k - d.s0];
    }
  if (int r = launch_ntt(c, a, true)) return r;
  c.mark("modup_intt");
  // 2. every digit's base conversion in one launch, written straight to the
  //    limb positions of its (nq + alpha)-limb ModUp buffer
  if ((int)lp.digits.size() > kMaxBconvJobs) {
    set_error("ModUp: too many digits");
    return -1;
  }
  if (tc) {
    BconvTcArgs b;
    memset(&b, 0, sizeof(b));
    b.error_flag = c.d_error_flag;
    for (const DigitPlan &d : lp.digits)
      fill_tc_job(c, b.jobs[b.n_jobs++], d.conv, y + (size_t)d.s0 * kN,
                  mu + (size_t)d.index * lp.ntot * kN, &d.dst_pos);
    if (int r = launch_bconv_tc(c, b)) return r;
  } else {
    BconvArgs b;
    memset(&b, 0, sizeof(b));
    for (const DigitPlan &d : lp.digits)
      fill_bconv_job(c, b.jobs[b.n_jobs++], d.conv,
                     reinterpret_cast<const int32_t *>(y) + (size_t)d.s0 * kN,
                     mu + (size_t)d.index * lp.ntot * kN, &d.dst_pos);
    if (int r = launch_bconv(c, b)) return r;
  }
  c.mark("modup_bconv");
  // 3. forward transforms of all converted limbs of all digits, in place
  memset(&a, 0, sizeof(a));
  a.dst = mu;
  a.src = mu;
  a.table = c.d_tw;
  a.n_polys = 1;
  // listed prime by prime, so that the copies of a prime in different digits
  // are neighbours and one CTA can transform them with one set of twiddles
  int n = 0;
  for (int g : lp.full_g)
    for (const DigitPlan &d : lp.digits)
      for (size_t m = 0; m < d.dst_pos.size(); m++) {
        if (d.conv.dst_g[m] != g) continue;
        if (n == kMaxJobs) {
          set_error("ModUp: too many limb transforms");
          return -1;
        }
        a.g[n] = (uint8_t)g;
        a.q[n] = c.q[g];
        a.src_limb[n] = a.dst_limb[n] = (uint16_t)(d.index * lp.ntot + d.dst_pos[m]);
        n++;
      }
  a.n_limbs = n;
  if (int r = launch_ntt(c, a, false)) return r;
  c.mark("modup_ntt");
  if (copy_own)
    for (const DigitPlan &d : lp.digits)
      CFHE_CUDA(cudaMemcpyAsync(
          mu + ((size_t)d.index * lp.ntot + d.s0) * kN, src + (size_t)d.s0 * kN,
          (size_t)(d.s1 - d.s0) * kN * sizeof(uint32_t),
          cudaMemcpyDeviceToDevice, c.stream));
  return 0;
}

size_t moddown_scratch_words(const ConvPlan &cv, int n_polys) {
  return (size_t)n_polys * cv.src_g.size() * kN;
}

static int check_moddown_shape(const ConvPlan &cv, int n_polys) {
  const int ns = (int)cv.src_g.size(), nd = (int)cv.dst_g.size();
  if (ns == 0 || nd == 0 || ns > kMaxBconvSrc || n_polys > kMaxBconvJobs) {
    set_error("ModDown: unsupported shape");
    return -1;
  }
  return 0;
}

// 1. inverse transform of the limbs that disappear, y = [n_polys][ns][N]
int run_moddown_intt(const Context &c, const ConvPlan &cv, uint32_t *y, const uint32_t *src, int n_polys,
                     long long src_stride) {
  if (int r = check_moddown_shape(cv, n_polys)) return r;
  const int ns = (int)cv.src_g.size();
  const bool tc = c.use_tc_bconv && cv.d_tc_table;
  NttArgs a;
  memset(&a, 0, sizeof(a));
  a.dst = y;
  a.src = src;
  a.table = c.d_itw;
  a.n_limbs = ns;
  a.n_polys = n_polys;
  a.dst_poly_stride = (long long)ns * kN;
  a.src_poly_stride = src_stride;
  a.centred = tc ? 0 : 1;
  for (int k = 0; k < ns; k++) {
    const int g = cv.src_g[k];
    a.g[k] = (uint8_t)g;
    a.q[k] = c.q[g];
    a.src_limb[k] = (uint16_t)cv.src_pos[k];
    a.dst_limb[k] = (uint16_t)k;
    a.kc[k] = cv.pre_tw[k];
  }
  if (int r = launch_ntt(c, a, true)) return r;
  c.mark("moddown_intt");
  return 0;
}

// 2. base conversion of y into the destination buffers
int run_moddown_bconv(const Context &c, const ConvPlan &cv, uint32_t *dst, uint32_t *y, int n_polys,
                      long long dst_stride) {
  if (int r = check_moddown_shape(cv, n_polys)) return r;
  const int ns = (int)cv.src_g.size();
  const bool tc = c.use_tc_bconv && cv.d_tc_table;
  if (tc) {
    BconvTcArgs b;
    memset(&b, 0, sizeof(b));
    b.error_flag = c.d_error_flag;
    for (int p = 0; p < n_polys; p++)
      fill_tc_job(c, b.jobs[b.n_jobs++], cv, y + (size_t)p * ns * kN, dst + p * dst_stride, nullptr);
    if (int r = launch_bconv_tc(c, b)) return r;
  } else {
    BconvArgs b;
    memset(&b, 0, sizeof(b));
    for (int p = 0; p < n_polys; p++)
      fill_bconv_job(c, b.jobs[b.n_jobs++], cv,
                     reinterpret_cast<const int32_t *>(y) + (size_t)p * ns * kN,
                     dst + p * dst_stride, nullptr);
    if (int r = launch_bconv(c, b)) return r;
  }
  c.mark("moddown_bconv");
  return 0;
}

// 3. forward transform in place with the fused (pad*x - t) * P^-1 epilogue
int run_moddown_ntt(const Context &c, const ConvPlan &cv, uint32_t *dst, const uint32_t *src, int n_polys,
                    long long dst_stride, long long src_stride) {
  if (int r = check_moddown_shape(cv, n_polys)) return r;
  const int nd = (int)cv.dst_g.size();
  NttArgs a;
  memset(&a, 0, sizeof(a));
  a.dst = dst;
  a.src = dst;
  a.table = c.d_tw;
  a.n_limbs = nd;
  a.n_polys = n_polys;
  a.dst_poly_stride = a.src_poly_stride = dst_stride;
  a.ep_mode = cv.has_pad ? 2 : 1;
  a.ep_src = src;
  a.ep_poly_stride = src_stride;
  for (int m = 0; m < nd; m++) {
    const int g = cv.dst_g[m];
    const uint32_t q = c.q[g];
    a.g[m] = (uint8_t)g;
    a.q[m] = q;
    a.src_limb[m] = a.dst_limb[m] = (uint16_t)m;
    a.ep_limb[m] = cv.ep_pos[m] < 0 ? 255 : (uint8_t)cv.ep_pos[m];
    a.ep_pad[m] = cv.ep_pad_tw[m];
    a.ep_scale[m] = cv.ep_scale_tw[m];
    a.ep_ps[m] = cv.ep_ps_tw[m];
  }
  if (int r = launch_ntt(c, a, false)) return r;
  c.mark("moddown_ntt");
  return 0;
}

int run_moddown(const Context &c, const ConvPlan &cv, uint32_t *dst,
                const uint32_t *src, int n_polys, long long dst_stride,
                long long src_stride, uint32_t *y) {
  if (int r = run_moddown_intt(c, cv, y, src, n_polys, src_stride)) return r;
  if (int r = run_moddown_bconv(c, cv, dst, y, n_polys, dst_stride)) return r;
  return run_moddown_ntt(c, cv, dst, src, n_polys, dst_stride, src_stride);
}

static int run_inner_impl(const Context &c, const LevelPlan &lp, uint32_t *acc_b,
                          uint32_t *acc_a, const uint32_t *mu, const uint32_t *d,
                          const uint32_t *c0, const uint32_t *c1,
                          const uint32_t *const *kb, const uint32_t *const *ka,
                          int key_main, uint32_t galois_inv, bool accumulate = false);

int run_inner(const Context &c, const LevelPlan &lp, uint32_t *acc_b,
              uint32_t *acc_a, const uint32_t *mu, const uint32_t *d,
              const uint32_t *c0, const uint32_t *c1,
              const uint32_t *const *kb, const uint32_t *const *ka,
              int key_main) {
  return run_inner_impl(c, lp, acc_b, acc_a, mu, d, c0, c1, kb, ka, key_main, 0);
}

int run_inner_rot(const Context &c, const LevelPlan &lp, uint32_t *acc_b,
                  uint32_t *acc_a, const uint32_t *mu, const uint32_t *d,
                  const uint32_t *c0, const uint32_t *const *kb,
                  const uint32_t *const *ka, int key_main, uint32_t galois_inv) {
  return run_inner_impl(c, lp, acc_b, acc_a, mu, d, c0, nullptr, kb, ka, key_main, galois_inv);
}

static int run_inner_impl(const Context &c, const LevelPlan &lp, uint32_t *acc_b,
                          uint32_t *acc_a, const uint32_t *mu, const uint32_t *d,
                          const uint32_t *c0, const uint32_t *c1,
                          const uint32_t *const *kb, const uint32_t *const *ka,
                          int key_main, uint32_t galois_inv, bool accumulate) {
  if ((int)lp.digits.size() > kMaxDigits) {
    set_error("inner product: too many digits");
    return -1;
  }
  const int key_ter = lp.level == -1 ? lp.num_ter : c.T;
  if (key_main < lp.num_main || key_main > c.M) {
    set_error("evaluation key holds fewer main limbs than the level needs");
    return -1;
  }
  InnerArgs a;
  memset(&a, 0, sizeof(a));
  a.acc_b = acc_b;
  a.acc_a = acc_a;
  a.mu = mu;
  a.d = d;
  a.c0 = c0;
  a.c1 = c1;
  a.n_digits = (int)lp.digits.size();
  a.ntot = lp.ntot;
  a.nq = lp.nq;
  a.scatter_galois = galois_inv;
  a.accumulate = accumulate ? 1 : 0;
  for (int i = 0; i < a.n_digits; i++) {
    const int slot = lp.digits[i].index;
    a.kb[i] = kb[slot];
    a.ka[i] = ka[slot];
    a.mu_slot[i] = (uint8_t)slot;
  }
  for (int l = 0; l < lp.ntot; l++) {
    const int g = lp.full_g[l];
    a.q[l] = c.q[g];
    a.nqinv[l] = c.nqinv[g];
    a.kpos[l] = (uint8_t)(g < c.L ? g - (c.T - key_ter)
                                  : key_ter + key_main + (g - c.L));
    a.own_digit[l] = l < lp.nq ? (uint8_t)lp.own_digit[l] : 255;
    a.pm[l] = l < lp.nq ? lp.p_mont[l] : 0;
  }
  if (int r = launch_inner(c, a)) return r;
  c.mark("inner");
  return 0;
}

int run_tensor(const Context &c, const LevelPlan &lp, uint32_t *d0,
               uint32_t *d1, uint32_t *d2, const uint32_t *b1,
               const uint32_t *a1, const uint32_t *b2, const uint32_t *a2) {
  TensorArgs t;
  memset(&t, 0, sizeof(t));
  t.n_rows = lp.nq;
  for (int l = 0; l < lp.nq; l++) {
    const size_t o = (size_t)l * kN;
    const int g = lp.q_g[l];
    t.rows[l] = TensorRow{d0 + o, d1 + o, d2 + o, b1 + o, a1 + o,
                          b2 + o, a2 + o, c.q[g], c.nqinv[g]};
  }
  if (int r = launch_tensor(c, t)) return r;
  c.mark("tensor");
  return 0;
}

int run_keyswitch(Context &c, const LevelPlan &lp, int down_type,
                  uint32_t *out_b, uint32_t *out_a, const uint32_t *d,
                  const uint32_t *c0, const uint32_t *c1,
                  const uint32_t *const *kb, const uint32_t *const *ka,
                  int key_main, uint32_t *scratch) {
  const ConvPlan &cv = lp.down[down_type];
  // scratch: y (max of the two inverse-transform outputs) | mu | acc_b | acc_a
  const size_t y_words =
      std::max(modup_scratch_words(lp), moddown_scratch_words(cv, 2));
  uint32_t *y = scratch;
  uint32_t *mu = y + y_words;
  uint32_t *acc = mu + (size_t)lp.beta * lp.ntot * kN;
  const size_t acc_words = (size_t)lp.ntot * kN;
  if (int r = run_modup(c, lp, mu, d, false, y)) return r;
  if (int r = run_inner(c, lp, acc, acc + acc_words, mu, d, c0, c1, kb, ka, key_main))
    return r;
  if (out_a - out_b == 0) {
    set_error("key switch: output polynomials alias");
    return -1;
  }
  return run_moddown(c, cv, out_b, acc, 2, (long long)(out_a - out_b),
                     (long long)acc_words, y);
}

// g^-1 modulo 2N by Newton iteration on the 2-adic inverse (g odd)
static uint32_t galois_inverse(uint32_t g) {
  const uint32_t m2 = 2u * kN;
  uint32_t inv = g;
  for (int it = 0; it < 5; it++) inv = (uint32_t)((uint64_t)inv * (2u - g * inv)) & (m2 - 1);
  return inv;
}

constexpr int kHoistChunk = 4;  // rotations whose ModDowns share launches

size_t hoisted_scratch_words(const LevelPlan &lp) {
  const size_t y_words = std::max(modup_scratch_words(lp),
                                  moddown_scratch_words(lp.down[0], 2 * kHoistChunk));
  return y_words + (size_t)(lp.beta + 2 * kHoistChunk) * lp.ntot * kN;
}

int run_hoisted_rotations(Context &c, const LevelPlan &lp, uint32_t *out,
                          const uint32_t *b, const uint32_t *a, int n_rot,
                          const uint32_t *galois, const uint32_t *const *kb,
                          const uint32_t *const *ka, int key_main,
                          uint32_t *scratch) {
  const ConvPlan &cv = lp.down[0];
  const size_t y_words = std::max(modup_scratch_words(lp),
                                  moddown_scratch_words(cv, 2 * kHoistChunk));
  uint32_t *y = scratch;
  uint32_t *mu = y + y_words;
  uint32_t *acc = mu + (size_t)lp.beta * lp.ntot * kN;
  const size_t acc_words = (size_t)lp.ntot * kN, out_words = (size_t)lp.nq * kN;
  const uint32_t m2 = 2u * kN;
  // the ModUp of a is computed once and shared by every rotation
  if (int r = run_modup(c, lp, mu, a, false, y)) return r;
  for (int r0 = 0; r0 < n_rot; r0 += kHoistChunk) {
    const int cnt = std::min(kHoistChunk, n_rot - r0);
    for (int i = 0; i < cnt; i++) {
      const uint32_t g = galois[r0 + i];
      if ((g & 1u) == 0 || g >= m2) {
        set_error("hoisted rotations: invalid Galois element");
        return -1;
      }
      const uint32_t inv = galois_inverse(g);
      uint32_t *ab = acc + (size_t)(2 * i) * acc_words;
      if (int rc = run_inner_rot(c, lp, ab, ab + acc_words, mu, a, b,
                                 kb + (size_t)(r0 + i) * lp.beta,
                                 ka + (size_t)(r0 + i) * lp.beta, key_main, inv))
        return rc;
    }
    if (int rc = run_moddown(c, cv, out + (size_t)(2 * r0) * out_words, acc, 2 * cnt,
                             (long long)out_words, (long long)acc_words, y))
      return rc;
  }
  return 0;
}

// ---------------------------------------------------------------------------
// Baby-step/giant-step linear transform with both hoistings:
//   out = Down( sum_j rot_Gj( Down( sum_i pt[j][i] (*) rot_bi(in) ) ) )
// (the unrotated giant step skips its inner Down)
// * the baby rotations share one ModUp and stay on the extended basis (no
//   ModDown per rotation); the unrotated input joins them as P * in;
// * the plaintexts, given on the extended basis, are accumulated per giant
//   step by one kernel; the giant sums go through ModDown together;
// * every giant rotation is a key switch whose extended-basis result is
//   added into one accumulator, so a single (rescaling) ModDown ends the call.
// ---------------------------------------------------------------------------
static size_t lt_y_words(const LevelPlan &lp, int n_giant, bool rescale) {
  size_t y = modup_scratch_words(lp);
  y = std::max(y, moddown_scratch_words(lp.down[0], std::min(2 * n_giant, kMaxBconvJobs)));
  y = std::max(y, moddown_scratch_words(lp.down[rescale ? 2 : 0], 2));
  return y;
}

// stored_rotations: the two-kernel form keeps every baby rotation (2 * n_baby
// extended polynomials); the fused kernel keeps none
size_t linear_transform_scratch_words(const LevelPlan &lp, int n_baby, int n_giant, bool rescale,
                                      bool stored_rotations) {
  const int rot_polys = stored_rotations ? 2 * n_baby : 0;
  return lt_y_words(lp, n_giant, rescale) +
         ((size_t)(lp.beta + rot_polys + 2 * n_giant + 2) * lp.ntot + (size_t)2 * n_giant * lp.nq) * kN;
}

// dst = (P * src on the Q limbs, 0 on the auxiliary limbs) for `n_polys`
// polynomials; src polynomials are nq limbs apart, dst ntot limbs apart.
static int lift_to_extended(const Context &c, const LevelPlan &lp, uint32_t *dst,
                            const uint32_t *const *src, int n_polys) {
  EwArgs e;
  e.n_rows = 0;
  for (int p = 0; p < n_polys; p++) {
    uint32_t *d = dst + (size_t)p * lp.ntot * kN;
    for (int l = 0; l < lp.nq; l++) {
      const int g = lp.q_g[l];
      e.rows[e.n_rows++] = EwRow{d + (size_t)l * kN, src[p] + (size_t)l * kN, nullptr,
                                 c.q[g], c.nqinv[g], lp.p_mont[l], 0u};
    }
    CFHE_CUDA(cudaMemsetAsync(d + (size_t)lp.nq * kN, 0, (size_t)(lp.ntot - lp.nq) * kN * sizeof(uint32_t),
                              c.stream));
  }
  if (int r = launch_ew(c, EW_MULC, e)) return r;
  c.mark("lift");
  return 0;
}

int run_linear_transform(Context &c, const LevelPlan &lp, bool rescale, uint32_t *out_b,
                         uint32_t *out_a, const uint32_t *in_b, const uint32_t *in_a,
                         int n_baby, const uint32_t *baby_galois,
                         const uint32_t *const *baby_kb, const uint32_t *const *baby_ka,
                         int n_giant, const uint32_t *giant_galois,
                         const uint32_t *const *giant_kb, const uint32_t *const *giant_ka,
                         const uint32_t *const *pt, int key_main, uint32_t *scratch) {
  if (n_baby < 1 || n_baby > kMaxBaby || n_giant < 1 || n_giant > kMaxGiant) {
    set_error("linear transform: at most 16 baby and 16 giant steps");
    return -1;
  }
  if (baby_galois[0] != 1u) {
    set_error("linear transform: the first baby step must be the identity");
    return -1;
  }
  if (rescale && !lp.has_rescale) {
    set_error("linear transform: this level cannot be rescaled");
    return -1;
  }
  if (2 * lp.ntot > kMaxRows) {
    set_error("linear transform: too many limbs");
    return -1;
  }
  const uint32_t m2 = 2u * kN;
  const size_t ext = (size_t)lp.ntot * kN, qw = (size_t)lp.nq * kN;
  uint32_t *y = scratch;
  uint32_t *mu = y + lt_y_words(lp, n_giant, rescale);
  uint32_t *rot = mu + (size_t)lp.beta * ext;       // [n_baby][2][ntot][N], two-kernel form only
  uint32_t *acc = rot + (c.use_fused_lt ? 0 : (size_t)2 * n_baby * ext);  // [n_giant][2][ntot][N]
  uint32_t *total = acc + (size_t)2 * n_giant * ext;  // [2][ntot][N]
  uint32_t *cj = total + 2 * ext;                   // [n_giant][2][nq][N]
  // giant steps in working order: the rotating ones first, the unrotated one
  // (if any) last, so that its extended-basis sum doubles as the accumulator
  int order[kMaxGiant], n_rot = 0, plain = -1;
  for (int j = 0; j < n_giant; j++) {
    const uint32_t g = giant_galois[j];
    if (g == 1u) {
      if (plain >= 0) {
        set_error("linear transform: more than one unrotated giant step");
        return -1;
      }
      plain = j;
    } else if ((g & 1u) == 0 || g >= m2) {
      set_error("linear transform: invalid giant-step Galois element");
      return -1;
    } else {
      order[n_rot++] = j;
    }
  }
  if (plain >= 0) order[n_rot] = plain;
  // 1 + 2. baby steps and plaintext accumulation
  if (n_baby > 1)
    if (int r = run_modup(c, lp, mu, in_a, false, y)) return r;
  for (int i = 1; i < n_baby; i++) {
    const uint32_t g = baby_galois[i];
    if ((g & 1u) == 0 || g >= m2 || g == 1u) {
      set_error("linear transform: invalid baby-step Galois element");
      return -1;
    }
  }
  if (c.use_fused_lt) {
    // one kernel: every baby rotation is formed at the automorphism's source
    // index and multiplied straight into the giant-step sums
    if ((int)lp.digits.size() > kMaxDigits) {
      set_error("linear transform: too many digits");
      return -1;
    }
    if (n_baby > 1 && (key_main < lp.num_main || key_main > c.M)) {
      set_error("evaluation key holds fewer main limbs than the level needs");
      return -1;
    }
    LtBabyArgs fa;
    memset(&fa, 0, sizeof(fa));
    fa.acc = acc;
    fa.mu = mu;
    fa.in_b = in_b;
    fa.in_a = in_a;
    fa.n_baby = n_baby;
    fa.n_giant = n_giant;
    fa.n_digits = (int)lp.digits.size();
    fa.ntot = lp.ntot;
    fa.nq = lp.nq;
    for (int i = 0; i < n_baby; i++) {
      fa.galois[i] = baby_galois[i];
      if (i == 0) continue;
      for (int d = 0; d < fa.n_digits; d++) {
        const int slot = lp.digits[d].index;
        fa.kb[i * kMaxDigits + d] = baby_kb[(size_t)i * lp.beta + slot];
        fa.ka[i * kMaxDigits + d] = baby_ka[(size_t)i * lp.beta + slot];
      }
    }
    for (int d = 0; d < fa.n_digits; d++) fa.mu_slot[d] = (uint8_t)lp.digits[d].index;
    for (int j = 0; j < n_giant; j++)
      for (int i = 0; i < n_baby; i++) fa.pt[j * kMaxBaby + i] = pt[(size_t)order[j] * n_baby + i];
    const int key_ter = lp.level == -1 ? lp.num_ter : c.T;
    for (int l = 0; l < lp.ntot; l++) {
      const int g = lp.full_g[l];
      fa.q[l] = c.q[g];
      fa.nqinv[l] = c.nqinv[g];
      fa.kpos[l] = (uint8_t)(g < c.L ? g - (c.T - key_ter) : key_ter + (n_baby > 1 ? key_main : 0) + (g - c.L));
      fa.own_digit[l] = l < lp.nq ? (uint8_t)lp.own_digit[l] : 255;
      fa.pm[l] = l < lp.nq ? lp.p_mont[l] : 0;
    }
    if (int r = launch_lt_baby(c, fa)) return r;
    c.mark("lt_baby");
  } else {
    {
      const uint32_t *src[2] = {in_b, in_a};
      if (int r = lift_to_extended(c, lp, rot, src, 2)) return r;
    }
    for (int i = 1; i < n_baby; i++) {
      uint32_t *rb = rot + (size_t)(2 * i) * ext;
      if (int r = run_inner_impl(c, lp, rb, rb + ext, mu, in_a, in_b, nullptr,
                                 baby_kb + (size_t)i * lp.beta, baby_ka + (size_t)i * lp.beta,
                                 key_main, galois_inverse(baby_galois[i])))
        return r;
    }
    PtAccumArgs pa;
    memset(&pa, 0, sizeof(pa));
    pa.rot = rot;
    pa.acc = acc;
    pa.n_baby = n_baby;
    pa.n_giant = n_giant;
    pa.ntot = lp.ntot;
    for (int j = 0; j < n_giant; j++)
      for (int i = 0; i < n_baby; i++) pa.pt[j * kMaxBaby + i] = pt[(size_t)order[j] * n_baby + i];
    for (int l = 0; l < lp.ntot; l++) {
      pa.q[l] = c.q[lp.full_g[l]];
      pa.nqinv[l] = c.nqinv[lp.full_g[l]];
    }
    if (int r = launch_pt_accum(c, pa)) return r;
    c.mark("pt_accum");
  }
  // 3. Of the rotating giant steps only the a parts leave the extended basis
  // (they are what gets decomposed and switched); the b parts are rotated where
  // they are and added to the accumulator. The unrotated step stays entirely:
  // it is already what the accumulator must start from.
  for (int p0 = 0; p0 < n_rot; p0 += kMaxBconvJobs) {
    const int cnt = std::min(kMaxBconvJobs, n_rot - p0);
    if (int r = run_moddown(c, lp.down[0], cj + (size_t)p0 * qw, acc + (size_t)(2 * p0 + 1) * ext, cnt,
                            (long long)qw, (long long)(2 * ext), y))
      return r;
  }
  // 4. giant rotations accumulate on the extended basis
  if (plain >= 0)
    total = acc + (size_t)2 * n_rot * ext;
  else
    CFHE_CUDA(cudaMemsetAsync(total, 0, 2 * ext * sizeof(uint32_t), c.stream));
  for (int jj = 0; jj < n_rot; jj++) {
    const int j = order[jj];
    const uint32_t g = giant_galois[j];
    {
      EwArgs e;
      e.n_rows = lp.ntot;
      const uint32_t *sb = acc + (size_t)(2 * jj) * ext;
      for (int l = 0; l < lp.ntot; l++) {
        const int gi = lp.full_g[l];
        const size_t o = (size_t)l * kN;
        e.rows[l] = EwRow{total + o, sb + o, total + o, c.q[gi], c.nqinv[gi], 0u, 0u};
      }
      if (int r = launch_permute(c, e, g)) return r;
      c.mark("permute");
    }
    const uint32_t *ca = cj + (size_t)jj * qw;
    if (int r = run_modup(c, lp, mu, ca, false, y)) return r;
    if (int r = run_inner_impl(c, lp, total, total + ext, mu, ca, nullptr, nullptr,
                               giant_kb + (size_t)j * lp.beta, giant_ka + (size_t)j * lp.beta,
                               key_main, galois_inverse(g), true))
      return r;
  }
  // 5. one ModDown (with the rescale) for the whole transform
  if (out_a - out_b == 0) {
    set_error("linear transform: output polynomials alias");
    return -1;
  }
  return run_moddown(c, lp.down[rescale ? 2 : 0], out_b, total, 2, (long long)(out_a - out_b),
                     (long long)ext, y);
}

size_t keyswitch_scratch_words(const LevelPlan &lp, int down_type) {
  const size_t y_words = std::max(modup_scratch_words(lp),
                                  moddown_scratch_words(lp.down[down_type], 2));
  return y_words + (size_t)(lp.beta + 2) * lp.ntot * kN;
}

}  // namespace cfhe
