/*
 * Scalar CPU golden model of the CKKS RNS hot path (32-bit words).
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or
 * calls this file; it exists so that the GPU kernels can be checked bit for
 * bit on the same inputs, and so that a bounded sample of the same work can be
 * timed on host cores as a reported baseline.
 *
 * It restates, in plain C with 64-bit `%` arithmetic, the algorithms of the
 * Cheddar reference (file:line cited at each function, relative to the
 * reference project root). The reference ships no golden vectors or known-
 * answer tests for this path (its tests are randomised round trips with a
 * 1e-3 tolerance, unittest/Testbed.h:93). Limb-level parity of this model
 * with the reference is pinned by the reference itself: its CUDA sources are
 * compiled unmodified into oracle/_ref/libcheddar_ref.so (Makefile target
 * `ref`), and tests/test_reference_gpu.py feeds the same device buffers to
 * that library, to the engine and to this model and compares every word
 * (NTT, INTT, ModUp, the three ModDown forms, HMult). Algebraic identities on
 * a toy ring (tests/test_oracle_cpu.py) pin it where no GPU is present.
 *
 * Conventions (reference include/core/Parameter.h:199-206,
 * src/core/Parameter.cu:104-105):
 *   - global prime order g = 0..L+alpha-1: terminal primes reversed, main
 *     primes, auxiliary primes;
 *   - a polynomial is limb-major, each limb N consecutive uint32 words;
 *   - NTT-domain values are stored as x*2^32 mod q ("M-form"), canonical
 *     [0,q), in the bit-reversed evaluation order produced by an in-place
 *     Cooley-Tukey transform;
 *   - Mont(a,b) = a*b*2^-32 mod q.
 */
#ifndef CFHE_ORACLE_H
#define CFHE_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct orc_ctx orc_ctx;

/* level_config: 2*num_levels ints, (num_main, num_ter) per level. */
orc_ctx *orc_create(int log_degree, const uint32_t *main_primes, int num_main,
                    const uint32_t *ter_primes, int num_ter,
                    const uint32_t *aux_primes, int num_aux,
                    const int *level_config, int num_levels, int add_main,
                    int add_ter);
void orc_destroy(orc_ctx *c);

int orc_degree(const orc_ctx *c);
int orc_num_primes(const orc_ctx *c);         /* L + alpha */
uint32_t orc_prime(const orc_ctx *c, int g);  /* by global index */
uint32_t orc_psi(const orc_ctx *c, int g);    /* primitive 2N-th root used */
int32_t orc_qinv(const orc_ctx *c, int g);    /* q^-1 mod 2^32, signed */
/* Global prime indices of a polynomial at `level` (-1 = short base) with
 * `num_aux` auxiliary limbs; returns the limb count. */
int orc_level_limbs(const orc_ctx *c, int level, int num_aux, int *gidx);
int orc_beta(const orc_ctx *c, int level);

/* ---- number theory helpers (exported for tests) ---- */
uint32_t orc_mulmod(uint32_t a, uint32_t b, uint32_t q);
uint32_t orc_powmod(uint32_t a, uint64_t e, uint32_t q);
uint32_t orc_invmod(uint32_t a, uint32_t q);
uint32_t orc_find_generator(uint32_t q);
uint32_t orc_to_mont(uint32_t a, uint32_t q);
uint32_t orc_mont_mul(uint32_t a, uint32_t b, uint32_t q);

/* ---- transforms; limb i of dst/src uses prime gidx[i] ---- */
/* Forward negacyclic NTT, natural order in, bit-reversed out, canonical.
 * mont_conv != 0 multiplies the input by 2^64 mod q through Mont first. */
void orc_ntt(const orc_ctx *c, uint32_t *dst, const uint32_t *src,
             const int *gidx, int nlimbs, int mont_conv);
/* Inverse: Gentleman-Sande, then out = Mont(raw, k[i]) where raw lacks the
 * 1/N factor. consts == NULL: k = N^-1 (mode_mont_keep == 0, leaves M-form)
 * or ToMont(N^-1) (mode_mont_keep != 0). centred != 0 maps results above
 * q>>1 to x - q (stored as two's complement). */
void orc_intt(const orc_ctx *c, uint32_t *dst, const uint32_t *src,
              const int *gidx, int nlimbs, const uint32_t *consts,
              int mode_mont_keep, int centred);

/* ---- element-wise, per limb prime gidx[i] ---- */
void orc_add(const orc_ctx *c, uint32_t *d, const uint32_t *a,
             const uint32_t *b, const int *gidx, int nlimbs);
void orc_sub(const orc_ctx *c, uint32_t *d, const uint32_t *a,
             const uint32_t *b, const int *gidx, int nlimbs);
void orc_neg(const orc_ctx *c, uint32_t *d, const uint32_t *a, const int *gidx,
             int nlimbs);
void orc_mul(const orc_ctx *c, uint32_t *d, const uint32_t *a,
             const uint32_t *b, const int *gidx, int nlimbs);
/* op: 0 add const, 1 sub const (a-k), 2 const minus a (k-a), 3 Mont mult */
void orc_const_op(const orc_ctx *c, uint32_t *d, const uint32_t *a,
                  const uint32_t *k, const int *gidx, int nlimbs, int op);
void orc_tensor(const orc_ctx *c, uint32_t *d0, uint32_t *d1, uint32_t *d2,
                const uint32_t *b1, const uint32_t *a1, const uint32_t *b2,
                const uint32_t *a2, const int *gidx, int nlimbs);
void orc_permute(const orc_ctx *c, uint32_t *d, const uint32_t *a,
                 uint32_t galois, int nlimbs);
void orc_mul_imag_unit(const orc_ctx *c, uint32_t *d, const uint32_t *a,
                       const int *gidx, int nlimbs);
uint32_t orc_galois_for_rotation(const orc_ctx *c, int rot);

/* ---- base conversion: y centred int32 [n_src][N] -> out [n_dst][N] ---- */
void orc_bconv(const orc_ctx *c, uint32_t *dst, const int32_t *y,
               const int *src_gidx, int n_src, const int *dst_gidx, int n_dst);

/* ---- level-aware pipelines ---- */
/* dst: beta buffers, each (nq+alpha) limbs, stored back to back; digits that
 * hold no limb at this level are left untouched. */
void orc_modup(const orc_ctx *c, int level, uint32_t *dst, const uint32_t *src);
/* type 0 ModDown (src nq+alpha limbs -> nq), 1 Rescale (nq -> nq'),
 * 2 ModDownAndRescale (nq+alpha -> nq'). */
void orc_moddown(const orc_ctx *c, int level, int type, uint32_t *dst,
                 const uint32_t *src);
/* acc_b/acc_a (nq+alpha limbs) = sum_j modup_j * evk_{b,a}[j]; evk digit j is
 * limb-major over the key's limbs (key_main, all terminal, alpha).
 * evk_b/evk_a: arrays of beta pointers. */
void orc_evk_inner(const orc_ctx *c, int level, uint32_t *acc_b,
                   uint32_t *acc_a, const uint32_t *modup,
                   const uint32_t *const *evk_b, const uint32_t *const *evk_a,
                   int key_main);
/* acc[Q limbs] += (P mod q) * x */
void orc_add_p_times(const orc_ctx *c, int level, uint32_t *acc,
                     const uint32_t *x);
/* Full HMult = tensor, relinearise, (rescale). out_b/out_a have the limbs of
 * level-1 when rescale != 0, else of level. */
void orc_hmult(const orc_ctx *c, int level, uint32_t *out_b, uint32_t *out_a,
               const uint32_t *b1, const uint32_t *a1, const uint32_t *b2,
               const uint32_t *a2, const uint32_t *const *evk_b,
               const uint32_t *const *evk_a, int key_main, int rescale);
/* Key switch of one polynomial d with b-part bx: (out_b,out_a) =
 * ModDown(sum_j ModUp_j(d)*evk_j + P*(bx,0)). */
void orc_keyswitch(const orc_ctx *c, int level, uint32_t *out_b,
                   uint32_t *out_a, const uint32_t *d, const uint32_t *bx,
                   const uint32_t *const *evk_b, const uint32_t *const *evk_a,
                   int key_main);

#ifdef __cplusplus
}
#endif
#endif
