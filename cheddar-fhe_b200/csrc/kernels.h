// Argument blocks and launchers of the element-wise, inner-product and base
// conversion kernels. Argument blocks travel as kernel parameters (constant
// bank), so a launch needs no host-to-device copy.
#pragma once
#include <stdint.h>

#include "context.h"

namespace cfhe {

enum EwOp {
  EW_ADD = 0,
  EW_SUB,
  EW_NEG,
  EW_MUL,
  EW_ADDC,
  EW_SUBC,
  EW_RSUBC,
  EW_MULC,
  EW_MULC_ADD,
  EW_IMAG,
  EW_COPY
};

struct EwRow {
  uint32_t *dst;
  const uint32_t *a;
  const uint32_t *b;
  uint32_t q, nqinv, k, pad_;
};
constexpr int kMaxRows = 192;  // 3 polynomials x 59 limbs fit
struct EwArgs {
  int n_rows;
  EwRow rows[kMaxRows];
};

struct TensorRow {
  uint32_t *d0, *d1, *d2;
  const uint32_t *b1, *a1, *b2, *a2;
  uint32_t q, nqinv;
};
struct TensorArgs {
  int n_rows;
  TensorRow rows[kMaxLimbs];
};

// Fused sums of up to kMaxTerms terms over n_polys polynomials (the
// reference's Sum / Accum, CAccum, PAccum and PermuteAccum families,
// src/core/ElementWise.cu:32-71, 225-366, 395-501):
//   dst[p] = (add[p] if given) + sum_t term_t(p),
//   term_t(p) = src[t][p]                          NARY_SUM
//             = c[t][limb] * src[t][p]             NARY_CONST   (c in M-form)
//             = pt[t] (*) src[t][p]                NARY_PLAIN   (one plaintext polynomial per term)
//             = permute(src[t][p], galois[t])      NARY_PERMUTE
constexpr int kMaxTerms = 8;
constexpr int kMaxNaryPolys = 3;
enum NaryMode { NARY_SUM = 0, NARY_CONST, NARY_PLAIN, NARY_PERMUTE };
struct NaryArgs {
  int mode, n_terms, n_polys, n_limbs;
  uint32_t *dst[kMaxNaryPolys];
  const uint32_t *add[kMaxNaryPolys];
  const uint32_t *src[kMaxTerms][kMaxNaryPolys];
  const uint32_t *pt[kMaxTerms];
  uint32_t galois[kMaxTerms];
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs];
  uint32_t c[kMaxTerms][kMaxLimbs];
};

// Sum of up to kMaxTensorTerms tensor products in one pass:
//   (d0, d1, d2) (+)= sum_t (b1_t b2_t, b1_t a2_t + a1_t b2_t, a1_t a2_t)
constexpr int kMaxTensorTerms = 16;
struct TensorAccArgs {
  int n_terms, n_limbs, accumulate;
  uint32_t *d[3];
  const uint32_t *b1[kMaxTensorTerms], *a1[kMaxTensorTerms], *b2[kMaxTensorTerms], *a2[kMaxTensorTerms];
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs];
};

constexpr int kMaxDigits = 8;
struct InnerArgs {
  uint32_t *acc_b, *acc_a;
  const uint32_t *mu;  // ModUp buffers, slot s at mu + s*ntot*N
  const uint32_t *d;   // polynomial being switched (own limbs), or null
  const uint32_t *c0, *c1;  // optional P*c0 -> acc_b, P*c1 -> acc_a (Q limbs)
  const uint32_t *kb[kMaxDigits], *ka[kMaxDigits];
  int n_digits, ntot, nq;
  // 0: results stay in place; otherwise the inverse Galois element g^-1 of an
  // automorphism applied to the result: word i is stored at pi_{g^-1}(i)
  uint32_t scatter_galois;
  int accumulate;  // != 0: the result is added to what acc_b / acc_a hold
  uint8_t mu_slot[kMaxDigits];
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs], pm[kMaxLimbs];
  uint8_t kpos[kMaxLimbs];       // limb position inside the key
  uint8_t own_digit[kMaxLimbs];  // active-digit index owning limb l, or 255
};

constexpr int kMaxBconvSrc = 20;  // source limbs of one conversion
struct BconvJob {
  const int32_t *src;    // [ns][N] centred
  uint32_t *dst;         // limb m stored at dst + dst_limb[m]*N
  const int32_t *table;  // [nd][ns]
  int ns, nd;
  uint8_t dst_limb[kMaxLimbs];
  uint32_t q[kMaxLimbs], qinv[kMaxLimbs];
};
constexpr int kMaxBconvJobs = 8;
struct BconvArgs {
  int n_jobs;
  BconvJob jobs[kMaxBconvJobs];
};

// Tensor-core base conversion (bconv_tc.cu): sources are canonical residues.
struct BconvTcJob {
  const uint32_t *src;   // [ns][N] canonical residues in [0, s_k)
  uint32_t *dst;         // limb m stored at dst + dst_limb[m]*N
  const uint8_t *btile;  // table byte planes in operand layout
  int ns, nd, kpad, npad;
  uint32_t half[kMaxBconvSrc + 3];  // s_k >> 1; 2^32 - 1 past the last source
  uint8_t dst_limb[kMaxLimbs];
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs];
};
struct BconvTcArgs {
  int n_jobs;
  int per_unit;     // CTAs sharing the tiles of one job (filled by the launcher)
  int *error_flag;  // set to 1 when a completion wait timed out
  BconvTcJob jobs[kMaxBconvJobs];
};

// Plaintext accumulation of a baby-step/giant-step linear transform on the
// extended basis: acc_j = sum_i pt[j][i] (*) rot_i for both polynomials.
constexpr int kMaxBaby = 16, kMaxGiant = 16;
struct PtAccumArgs {
  const uint32_t *rot;  // [n_baby][2][ntot][N]: (b, a) of every baby rotation
  uint32_t *acc;        // [n_giant][2][ntot][N]
  const uint32_t *pt[kMaxGiant * kMaxBaby];  // [giant * kMaxBaby + baby], [ntot][N] each; null = absent
  int n_baby, n_giant, ntot;
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs];
};

// Fused baby steps of a linear transform: for every output word, every baby
// rotation's key inner product is formed at the source index of the
// automorphism and multiplied straight into the giant-step sums, so the
// rotated ciphertexts are never stored.
struct LtBabyArgs {
  uint32_t *acc;                // [n_giant][2][ntot][N]
  const uint32_t *mu;           // ModUp buffers of the input's a part, slot s at mu + s*ntot*N
  const uint32_t *in_b, *in_a;  // input ciphertext on the Q limbs
  const uint32_t *kb[kMaxBaby * kMaxDigits], *ka[kMaxBaby * kMaxDigits];  // [baby][active digit]
  const uint32_t *pt[kMaxGiant * kMaxBaby];  // [giant][baby], null = absent
  uint32_t galois[kMaxBaby];    // Galois element of each baby rotation (1 = identity)
  int n_baby, n_giant, n_digits, ntot, nq;
  uint8_t mu_slot[kMaxDigits];
  uint32_t q[kMaxLimbs], nqinv[kMaxLimbs], pm[kMaxLimbs];
  uint8_t kpos[kMaxLimbs], own_digit[kMaxLimbs];
};

int launch_ew(const Context &ctx, int op, const EwArgs &args);
int launch_pt_accum(const Context &ctx, const PtAccumArgs &args);
int launch_lt_baby(const Context &ctx, const LtBabyArgs &args);
int launch_tensor(const Context &ctx, const TensorArgs &args);
int launch_lift(const Context &ctx, const EwArgs &args, const uint32_t *src, uint32_t q0, uint32_t q1);
int launch_permute(const Context &ctx, const EwArgs &args, uint32_t galois);
int launch_nary(const Context &ctx, const NaryArgs &args);
int launch_tensor_accum(const Context &ctx, const TensorAccArgs &args);
// gemm_tc.cu: ciphertext x plaintext RNS GEMM on the tensor cores
size_t gemm_packed_weight_bytes(int n_in, int n_out);  // per limb
size_t gemm_scratch_bytes(int n_in);
void gemm_pack_weights_limb(uint8_t *out, const uint32_t *w, int n_in, int n_out, uint32_t q);
int launch_ctpt_gemm(const Context &c, uint32_t *const *y, const uint32_t *const *x, const uint8_t *wp,
                     uint8_t *scratch, int n_in, int n_out, const int *gidx, int n_limbs);
// sampling.cu: client-side sampling and encryption
constexpr int kErrorCdfEntries = 97;
void error_cdf_table(double sigma, uint64_t *cdf);
int launch_sample_uniform(const Context &c, uint32_t *dst, const int *gidx, int n_limbs, uint64_t seed,
                          uint32_t stream);
int launch_sample_error(const Context &c, uint32_t *dst, const int *gidx, int n_limbs, double sigma,
                        uint64_t seed, uint32_t stream);
int launch_crt_lift(const Context &c, double *out, const uint32_t *res, const int *gidx, int n_limbs,
                    const uint32_t *hat, const uint32_t *q_low);
int launch_rns_split(const Context &c, uint32_t *dst, const double *v, const int *gidx, int n_limbs);
int launch_encrypt(const Context &c, uint32_t *b, const uint32_t *a, const uint32_t *s, const uint32_t *e,
                   const uint32_t *m, const int *gidx, int n_limbs);
int launch_inner(const Context &ctx, const InnerArgs &args);
int launch_bconv(const Context &ctx, const BconvArgs &args);
int launch_bconv_tc(const Context &ctx, const BconvTcArgs &args);
int build_tc_table(const Context &ctx, ConvPlan &cv);

}  // namespace cfhe
