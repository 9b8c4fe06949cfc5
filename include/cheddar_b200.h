/*
 * C ABI of the B200 CKKS engine (libcheddar_b200.so).
 *
 * This is the boundary a host language binds. The reference (Cheddar) has no
 * C ABI or plugin mechanism of its own: its consumers include C++ headers and
 * call template classes. Each entry point below therefore names the reference
 * C++ method whose device-side work it replaces (file:line relative to the
 * reference project root); the C++ facade in cheddar-fhe_b200/host mirrors the
 * reference's class names on top of these calls.
 *
 * Conventions
 *  - every function returns 0 on success, a negative code on failure;
 *    cfhe_last_error() returns the message of the calling thread's last
 *    failure (the reference prints and exits instead, include/common/Assert.h:9-21);
 *  - all polynomial pointers are DEVICE pointers to 32-bit words, limb-major,
 *    N words per limb; limb lists (`gidx`) are HOST arrays of global prime
 *    indices in the reference's order: terminal primes reversed, main primes,
 *    auxiliary primes (include/core/Parameter.h:199-206);
 *  - NTT-domain values are x * 2^32 mod q in [0,q), in the bit-reversed
 *    evaluation order of an in-place Cooley-Tukey transform, exactly as the
 *    reference stores them;
 *  - work is enqueued on the context's stream and is asynchronous; calls on
 *    one context are ordered.
 */
#ifndef CHEDDAR_B200_H
#define CHEDDAR_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CFHE_API __attribute__((visibility("default")))
#else
#define CFHE_API
#endif

typedef struct cfhe_context cfhe_context;

CFHE_API const char *cfhe_last_error(void);
/* Number of kernels this library has launched in the calling process so far
 * (all contexts). No counterpart in the reference; benchmarks take the
 * difference around a timed region to report how many launches it held. */
CFHE_API unsigned long long cfhe_kernel_launch_count(void);

/* Builds per-prime tables on `device`. level_config holds (num_main, num_ter)
 * per level. Replaces Context<word>::Create + NTTHandler /
 * ModSwitchHandler construction (src/core/Context.cpp:62-124,
 * src/core/NTT.cu:1233-1299, src/core/ModSwitch.cu:175-318). Only
 * log_degree 16 is supported (as the reference's Parameter, Parameter.h:32). */
CFHE_API int cfhe_context_create(cfhe_context **out, int device, int log_degree,
                        const uint32_t *main_primes, int num_main,
                        const uint32_t *ter_primes, int num_ter,
                        const uint32_t *aux_primes, int num_aux,
                        const int *level_config, int num_levels, int add_main,
                        int add_ter);
CFHE_API void cfhe_context_destroy(cfhe_context *ctx);

/* Enqueue on the caller's cudaStream_t; the handle is used as given, so NULL
 * means the legacy default stream, which is what the reference runs on
 * (include/core/DeviceVector.h:88). A new context starts on a non-blocking
 * stream of its own; cfhe_use_own_stream() returns to it. */
CFHE_API int cfhe_set_stream(cfhe_context *ctx, void *cuda_stream);
CFHE_API int cfhe_use_own_stream(cfhe_context *ctx);
/* The cudaStream_t the context's work is enqueued on (for a caller that puts
 * its own work, e.g. a collective on the context's buffers, in the same order). */
CFHE_API void *cfhe_get_stream(cfhe_context *ctx);
CFHE_API int cfhe_synchronize(cfhe_context *ctx);
/* Two contexts of one GPU work side by side (each on its own stream, with its
 * own workspace and allocation cache): everything submitted to `later` after
 * this call starts after everything submitted to `earlier` before it. No host
 * synchronisation. The reference runs on the legacy default stream
 * (src/core/Context.cpp:584-871 launch without a stream argument), where this
 * ordering is implicit; it has no counterpart there. */
CFHE_API int cfhe_order_after(cfhe_context *later, cfhe_context *earlier);

CFHE_API int cfhe_degree(const cfhe_context *ctx);
CFHE_API int cfhe_num_primes(const cfhe_context *ctx);
CFHE_API uint32_t cfhe_prime(const cfhe_context *ctx, int g);
/* Limbs of a polynomial at `level` (-1: short base) with num_aux auxiliary
 * limbs (Parameter<word>::LevelToNP + GetPrimeVector,
 * src/core/Parameter.cu:277-325). Returns the count. */
CFHE_API int cfhe_level_limbs(const cfhe_context *ctx, int level, int num_aux, int *gidx);

/* Device memory (the reference's DeviceVector / MemoryPool,
 * src/core/DeviceVector.cpp, src/core/MemoryPool.cpp). */
CFHE_API int cfhe_malloc(cfhe_context *ctx, void **ptr, size_t bytes);
CFHE_API int cfhe_free(cfhe_context *ctx, void *ptr);
CFHE_API int cfhe_copy_h2d(cfhe_context *ctx, void *dst, const void *src, size_t bytes);
CFHE_API int cfhe_copy_d2h(cfhe_context *ctx, void *dst, const void *src, size_t bytes);

/* Batched forward NTT of n_polys polynomials with the same limb list.
 * NTTHandler<word>::NTT (src/core/NTT.cu:606-671); mont_conv multiplies the
 * input by 2^32 mod q first (the reference's montgomery_conversion). Strides
 * are in words between consecutive polynomials. dst may equal src. */
CFHE_API int cfhe_ntt(cfhe_context *ctx, uint32_t *dst, const uint32_t *src,
             const int *gidx, int n_limbs, int n_polys,
             long long dst_poly_stride, long long src_poly_stride,
             int mont_conv);

/* Batched inverse NTT followed by a per-limb constant.
 * consts == NULL: NTTHandler<word>::INTT (src/core/NTT.cu:673-741), the
 * constant is 1/N (mont_keep == 0, result leaves M-form) or keeps M-form
 * (mont_keep != 0). consts != NULL (HOST array, one word per limb):
 * NTTHandler<word>::INTTAndMultConst (src/core/NTT.cu:743-813), result =
 * raw * consts[l] * 2^-32 mod q. centred != 0 stores values above q/2 as
 * x - q (the reference's `normalize`). */
CFHE_API int cfhe_intt(cfhe_context *ctx, uint32_t *dst, const uint32_t *src,
              const int *gidx, int n_limbs, int n_polys,
              long long dst_poly_stride, long long src_poly_stride,
              const uint32_t *consts, int mont_keep, int centred);

/* ---- element-wise operators (ElementWiseHandler, src/core/ElementWise.cu).
 * Operands are limb-major over exactly the limbs listed in gidx. ---- */
/* op: 0 a+b (:687 Add), 1 a-b (:719 Sub), 2 -a (:751 Neg, b unused),
 * 3 a*b Montgomery (:779 Mult / :813 PMult). */
CFHE_API int cfhe_binary(cfhe_context *ctx, int op, uint32_t *dst,
                         const uint32_t *a, const uint32_t *b, const int *gidx,
                         int n_limbs);
/* consts: HOST array, one word per limb. op: 0 a+k (:821 AddConst), 1 a-k
 * (:852 SubConst), 2 k-a (:883 SubOppositeConst), 3 a*k Montgomery (:914
 * MultConst), 4 a*k + b (CAccum with one term plus src0, :1356). */
CFHE_API int cfhe_const_op(cfhe_context *ctx, int op, uint32_t *dst,
                           const uint32_t *a, const uint32_t *b,
                           const uint32_t *consts, const int *gidx, int n_limbs);
/* The operators of cfhe_binary (with_const == 0, op 0..3) or cfhe_const_op
 * (with_const != 0, op 0..4) applied to n_polys polynomials in one launch, as
 * the reference's element-wise kernels do for the two or three polynomials of
 * a ciphertext (template parameter num_poly, ElementWise.cu:32-60). dst, a, b:
 * HOST arrays of n_polys device pointers (b may be NULL where the op has no
 * second operand); consts and gidx are shared by all polynomials;
 * n_polys * n_limbs <= 192. */
CFHE_API int cfhe_elementwise_multi(cfhe_context *ctx, int with_const, int op,
                                    int n_polys, uint32_t *const *dst,
                                    const uint32_t *const *a,
                                    const uint32_t *const *b,
                                    const uint32_t *consts, const int *gidx,
                                    int n_limbs);
/* (d0,d1,d2) = (b1*b2, b1*a2 + a1*b2, a1*a2): ElementWiseHandler::Tensor
 * (:922, kernel :504-546). */
CFHE_API int cfhe_tensor(cfhe_context *ctx, uint32_t *d0, uint32_t *d1,
                         uint32_t *d2, const uint32_t *b1, const uint32_t *a1,
                         const uint32_t *b2, const uint32_t *a2,
                         const int *gidx, int n_limbs);
/* dst = automorphism_galois(src) (+ add when add != NULL):
 * ElementWiseHandler::Permute / PermuteAccum (:967, :1002; kernels :370-501).
 * galois = 5^r mod 2N for a rotation by r slots, 2N-1 for conjugation. */
CFHE_API int cfhe_permute(cfhe_context *ctx, uint32_t *dst, const uint32_t *src,
                          const uint32_t *add, uint32_t galois,
                          const int *gidx, int n_limbs);
CFHE_API uint32_t cfhe_galois_for_rotation(const cfhe_context *ctx, int rot);
/* Fused n-ary sums over n_polys (1..3) polynomials and n_terms (1..8) terms, one
 * launch each; `src` is [term * n_polys + poly], `addend` (n_polys pointers or
 * NULL) an optional extra summand per polynomial. They replace the
 * reference's variadic kernels and the workers that pick an instantiation:
 *   cfhe_accum          dst[p] = sum_t src[t][p]
 *       ElementWiseHandler::Accum / Add (:1246, kernel Sum :32-71)
 *   cfhe_caccum         dst[p] = sum_t consts[t*n_limbs + l] * src[t][p] (+ addend[p])
 *       ElementWiseHandler::CAccum (:1355-1394, kernels CPAccum / CPAccumAdd
 *       <const_accum = true> :225-366); consts are M-form words per term and limb
 *   cfhe_paccum         dst[p] = sum_t pt[t] (*) src[t][p] (+ addend[p])
 *       ElementWiseHandler::PAccum (:1396-1435, CPAccum<false>); one plaintext
 *       polynomial per term, shared by the polynomials
 *   cfhe_permute_accum  dst[p] = sum_t automorphism_{galois[t]}(src[t][p]) (+ addend[p])
 *       ElementWiseHandler::PermuteAccum (:1002-1226, kernels :395-501);
 *       no source may alias its destination. */
CFHE_API int cfhe_accum(cfhe_context *ctx, int n_polys, uint32_t *const *dst, int n_terms,
                        const uint32_t *const *src, const int *gidx, int n_limbs);
CFHE_API int cfhe_caccum(cfhe_context *ctx, int n_polys, uint32_t *const *dst, int n_terms,
                         const uint32_t *const *src, const uint32_t *consts,
                         const uint32_t *const *addend, const int *gidx, int n_limbs);
CFHE_API int cfhe_paccum(cfhe_context *ctx, int n_polys, uint32_t *const *dst, int n_terms,
                         const uint32_t *const *src, const uint32_t *const *pt,
                         const uint32_t *const *addend, const int *gidx, int n_limbs);
CFHE_API int cfhe_permute_accum(cfhe_context *ctx, int n_polys, uint32_t *const *dst, int n_terms,
                                const uint32_t *const *src, const uint32_t *galois,
                                const uint32_t *const *addend, const int *gidx, int n_limbs);
/* (d0,d1,d2) (+)= sum over n_terms (<= 16) of the tensor products
 * (b1*b2, b1*a2 + a1*b2, a1*a2); accumulate != 0 adds to what d0..d2 hold.
 * One pass over the operands instead of one Tensor and one Add per term
 * (ElementWiseHandler::Tensor, src/core/ElementWise.cu:922, kernel :504-546;
 * the reference has no n-ary form of it). Operand tables: HOST arrays of
 * DEVICE pointers. Same words as cfhe_tensor followed by cfhe_binary(add). */
CFHE_API int cfhe_tensor_accum(cfhe_context *ctx, uint32_t *d0, uint32_t *d1, uint32_t *d2, int n_terms,
                               const uint32_t *const *b1, const uint32_t *const *a1,
                               const uint32_t *const *b2, const uint32_t *const *a2, int accumulate,
                               const int *gidx, int n_limbs);
/* Plaintext products of a baby-step/giant-step linear transform, all giant
 * steps in one launch (the reference's GSFusedKernel, src/extension/Hoist.cu:80-118):
 *   acc[j] = sum_i pt[j * n_baby + i] (*) rot[i]   on both polynomials,
 * a NULL plaintext is skipped. rot: [n_baby][2][n_limbs][N] (b, a of every
 * baby rotation), acc: [n_giant][2][n_limbs][N], pt: HOST array of
 * n_giant * n_baby DEVICE pointers ([n_limbs][N] each); at most 16 baby and 16
 * giant steps. (The reference passes tables of polynomial pointers instead of
 * two contiguous buffers.) */
CFHE_API int cfhe_giantstep_paccum(cfhe_context *ctx, uint32_t *acc, const uint32_t *rot, int n_baby,
                                   int n_giant, const uint32_t *const *pt, const int *gidx, int n_limbs);
/* Ciphertext x plaintext RNS GEMM on the tensor cores (tcgen05 kind::i8, exact):
 *   y[j] = sum_k W[l][k][j] * x[k]  on every listed limb l,
 * n_in input and n_out output polynomials of n_limbs limbs each, W words in
 * M-form. Same words as cfhe_caccum applied to eight terms at a time. The
 * reference has no kernel for this contraction (its CAccum,
 * src/core/ElementWise.cu:1355-1394, is the closest operator); it is the
 * projection step of the encrypted transformer layer (one ciphertext
 * polynomial per input feature, plaintext weight matrix).
 *   cfhe_gemm_weight_bytes   device bytes of the packed weights
 *   cfhe_gemm_pack_weights   weights: HOST array [n_limbs][n_in][n_out]; packed:
 *                            DEVICE buffer of cfhe_gemm_weight_bytes bytes
 *   cfhe_ctpt_gemm           x, y: HOST arrays of n_in / n_out DEVICE pointers */
CFHE_API size_t cfhe_gemm_weight_bytes(int n_in, int n_out, int n_limbs);
CFHE_API int cfhe_gemm_pack_weights(cfhe_context *ctx, void *packed, const uint32_t *weights, int n_in,
                                    int n_out, const int *gidx, int n_limbs);
CFHE_API int cfhe_ctpt_gemm(cfhe_context *ctx, uint32_t *const *y, const uint32_t *const *x,
                            const void *packed, int n_in, int n_out, const int *gidx, int n_limbs);
/* Client-side sampling and encryption on the device (the reference samples on
 * the host and uploads: src/UserInterface.cu:223-276, 366-458; Random,
 * include/Random.h). Words are a pure function of (seed, stream, prime index,
 * word index) through the Philox-4x32-10 counter-based generator, so a draw
 * can be reproduced anywhere.
 *   cfhe_sample_uniform  n_limbs limbs of residues uniform in [0, q) (exactly
 *       uniform: multiply-and-reject). Replaces Random::SampleUniformWord +
 *       upload in UserInterface::SampleRandomPolynomial.
 *   cfhe_sample_error    ONE polynomial of rounded-normal integers (standard
 *       deviation sigma <= 8, tail cut at +-48), written mod every prime of the
 *       list in coefficient order; the caller transforms it (cfhe_ntt with
 *       mont_conv). Replaces Random::SampleDiscreteNormal + upload.
 *   cfhe_error_cdf       the 97-entry cumulative table (64-bit fixed point)
 *       the error sampler walks, for hosts that want to reproduce a draw.
 *   cfhe_encrypt         b = m + e - a * s, m == NULL for an encryption of
 *       zero: the reference's Encrypt / EncryptZero kernels (:17-80); s in
 *       M-form, everything in the NTT domain.
 *   cfhe_add_evk_part    bx += p_prod[l] * s_target on the listed limbs: the
 *       reference's AddEvkPart kernel (:82-108); p_prod in M-form. */
CFHE_API int cfhe_sample_uniform(cfhe_context *ctx, uint32_t *dst, const int *gidx, int n_limbs,
                                 unsigned long long seed, unsigned int stream);
CFHE_API int cfhe_sample_error(cfhe_context *ctx, uint32_t *dst, const int *gidx, int n_limbs,
                               double sigma, unsigned long long seed, unsigned int stream);
CFHE_API int cfhe_error_cdf(double sigma, unsigned long long *cdf, int entries);
CFHE_API int cfhe_encrypt(cfhe_context *ctx, uint32_t *b, const uint32_t *a, const uint32_t *s,
                          const uint32_t *e, const uint32_t *m, const int *gidx, int n_limbs);
CFHE_API int cfhe_add_evk_part(cfhe_context *ctx, uint32_t *bx, const uint32_t *s_target,
                               const uint32_t *p_prod, const int *gidx, int n_limbs);
/* Encoding, device half (Encoder::Encode, src/core/Encode.cpp:136-248, after
 * its special inverse FFT): coeffs is a HOST array of N doubles, the
 * plaintext polynomial's coefficients already multiplied by the scale; dst
 * receives, on every listed limb, the residues of trunc(coeffs[i]) (toward
 * zero, as the reference's conversion to a big integer truncates), transformed
 * to the evaluation domain in M-form: a finished plaintext. Any magnitude a
 * double can hold is reduced exactly (m * 2^e mod q), without big integers;
 * one 512 KiB upload instead of n_limbs * 256 KiB. */
CFHE_API int cfhe_encode_coeffs(cfhe_context *ctx, uint32_t *dst, const double *coeffs, const int *gidx,
                                int n_limbs);
/* Decoding, device half (Encoder::Decode, src/core/Encode.cpp:250-275, before
 * its special FFT): src is a plaintext on the listed limbs (evaluation domain,
 * M-form); coeffs, a HOST array of N doubles, receives the centred integer
 * coefficients of the plaintext polynomial (to be divided by the scale).
 * The caller supplies the constants of the limb set:
 *   icrt[j]    = (N * Q / q_j)^-1 mod q_j
 *   hat[4*j..] = (Q / q_j) mod 2^128, four little-endian 32-bit words
 *   q_low[4]   = Q mod 2^128
 * Exact for coefficients below 2^127 in magnitude (any decodable plaintext;
 * larger values wrap). Synchronises the context's stream. */
CFHE_API int cfhe_decode_coeffs(cfhe_context *ctx, double *coeffs, const uint32_t *src, const int *gidx,
                                int n_limbs, const uint32_t *icrt, const uint32_t *hat,
                                const uint32_t *q_low);
/* Device-to-device copy and fill on the context's stream (the reference's
 * DeviceVector copies, src/core/DeviceVector.cpp, and cudaMemsetAsync calls). */
CFHE_API int cfhe_copy_d2d(cfhe_context *ctx, void *dst, const void *src, size_t bytes);
CFHE_API int cfhe_memset(cfhe_context *ctx, void *dst, int value, size_t bytes);
/* dst = src * X^(N/2): ElementWiseHandler::MultImaginaryUnit (:1673). */
CFHE_API int cfhe_mul_imag_unit(cfhe_context *ctx, uint32_t *dst,
                                const uint32_t *src, const int *gidx,
                                int n_limbs);

/* Exact lift of a one- or two-limb value to other primes:
 * ElementWiseHandler::ModUpToMax (:1646; kernels :579-623), used by
 * BootContext::ModUpToMax. src holds plain coefficients; in the two-limb case
 * limb k must already be multiplied by (q_other)^-1 mod q_k (as the
 * reference's INTTAndMultConst with mod_max_intt_const_ does,
 * src/extension/BootContext.cpp:93-108). dst: plain coefficients mod each
 * destination prime, centred lift. */
CFHE_API int cfhe_modup_to_max(cfhe_context *ctx, uint32_t *dst,
                               const uint32_t *src, const int *src_gidx,
                               int n_src, const int *dst_gidx, int n_dst);

/* ---- mod-switch (ModSwitchHandler, src/core/ModSwitch.cu) ---- */
/* Base conversion of centred, pre-scaled coefficients y[n_src][N] (int32) to
 * M-form coefficients on the destination primes: the kernel
 * ModSwitchMatrixMult (:23-171) with its table built as in :353-366. */
CFHE_API int cfhe_bconv(cfhe_context *ctx, uint32_t *dst, const int32_t *y,
                        const int *src_gidx, int n_src, const int *dst_gidx,
                        int n_dst);
CFHE_API int cfhe_beta(const cfhe_context *ctx, int level);
/* ModSwitchHandler::ModUp (:429-509). dst: beta buffers of (nq+alpha) limbs,
 * back to back (digit i at dst + i*(nq+alpha)*N); digits holding no limb at
 * this level are left untouched. */
CFHE_API int cfhe_modup(cfhe_context *ctx, int level, uint32_t *dst,
                        const uint32_t *src);
/* ModSwitchHandler::PseudoModUp (:413-428): dst = (P mod q_l) * src on the
 * level's Q limbs, the extended-basis image of a polynomial that needs no
 * conversion (used by the reference's hoisting for the unrotated term). */
CFHE_API int cfhe_pseudo_modup(cfhe_context *ctx, int level, uint32_t *dst, const uint32_t *src);
/* type 0 ModDown (:511-527), 1 Rescale (:529-545), 2 ModDownAndRescale
 * (:547-563), all through ModDownWorker (:566-684); n_polys polynomials with
 * the given strides (words) are processed together. */
CFHE_API int cfhe_moddown(cfhe_context *ctx, int level, int type, uint32_t *dst,
                          const uint32_t *src, int n_polys,
                          long long dst_poly_stride, long long src_poly_stride);
/* The three stages of cfhe_moddown() as separate calls, for a host that
 * composes its own pipeline as the reference's handlers allow
 * (NTTHandler::INTTForModDown, src/core/NTT.cu:1018-1127;
 * ModSwitchHandler's matrix product, src/core/ModSwitch.cu:23-171;
 * NTTHandler::NTTForModDown with its (src * pad - x) * P^-1 epilogue,
 * src/core/NTT.cu:889-1016). level / type / n_polys / strides as in
 * cfhe_moddown; y is a scratch of n_polys * cfhe_moddown_source_limbs() limbs:
 *   cfhe_intt_for_moddown   y   = inverse transform of the limbs of src that
 *                                 disappear, times the conversion's constants,
 *                                 in the form the conversion reads
 *   cfhe_bconv_for_moddown  dst = base conversion of y onto the limbs that stay
 *   cfhe_ntt_for_moddown    dst = (pad * src - NTT(dst)) * P^-1, in place
 * Run in that order they leave the words of cfhe_moddown(). (The forward
 * transform that skips a digit's own limbs, NTTForModUp, is cfhe_ntt with the
 * limb list that leaves them out.) */
CFHE_API int cfhe_moddown_source_limbs(cfhe_context *ctx, int level, int type);
CFHE_API int cfhe_intt_for_moddown(cfhe_context *ctx, int level, int type, uint32_t *y, const uint32_t *src,
                                   int n_polys, long long src_poly_stride);
CFHE_API int cfhe_bconv_for_moddown(cfhe_context *ctx, int level, int type, uint32_t *dst, uint32_t *y,
                                    int n_polys, long long dst_poly_stride);
CFHE_API int cfhe_ntt_for_moddown(cfhe_context *ctx, int level, int type, uint32_t *dst, const uint32_t *src,
                                  int n_polys, long long dst_poly_stride, long long src_poly_stride);
/* Same result as cfhe_moddown() for ONE polynomial, but the call path never
 * allocates or frees device memory. This entry point has no counterpart in
 * the reference (whose every ModDown takes temporaries from its memory pool,
 * src/core/ModSwitch.cu:589-605). It is for hosts that cannot let a library
 * call cudaMalloc: processes that gave the whole GPU to their own allocator,
 * and loops that cannot afford the device-wide synchronisation an allocation
 * implies. The inverse-transform intermediate lives in a 4 MiB array built
 * into the library (16 limbs; every GPU that loads the library carries it
 * until exit); a level/type whose conversion drops more than 16 limbs is
 * refused with an error. The context's device must be current. The first call
 * on each device also looks up the array's address, so make that first call
 * before starting any stream capture. All calls on a device share the array:
 * two calls running on the GPU at the same time corrupt each other, so keep
 * them ordered (one stream, or events). Nothing needs clearing between calls:
 * every word read is written earlier in the same call. */
CFHE_API int cfhe_moddown_noalloc(cfhe_context *ctx, int level, int type,
                                  uint32_t *dst, const uint32_t *src);
/* Evaluation-key inner product, Context::MultKeyNoModDown(accum, a_modup,
 * a_orig, key) (src/core/Context.cpp:609-647) -> ElementWiseHandler::PAccum.
 * modup as produced by cfhe_modup; evk_b/evk_a: HOST arrays of beta device
 * pointers, each limb-major over (all terminal, key_main main, alpha aux)
 * limbs. c0/c1 (may be NULL): adds P*c0 to acc_b and P*c1 to acc_a on the Q
 * limbs, the CAccum step of Context.cpp:688-711. */
CFHE_API int cfhe_evk_inner(cfhe_context *ctx, int level, uint32_t *acc_b,
                            uint32_t *acc_a, const uint32_t *modup,
                            const uint32_t *c0, const uint32_t *c1,
                            const uint32_t *const *evk_b,
                            const uint32_t *const *evk_a, int key_main);
/* Context::MultKey for a ciphertext without rx (Context.cpp:584-607): the
 * polynomial d is switched, P*bx is added to the b part, both parts go
 * through ModDown. Used by HRot / HConj before the permutation. */
CFHE_API int cfhe_keyswitch(cfhe_context *ctx, int level, uint32_t *out_b,
                            uint32_t *out_a, const uint32_t *d,
                            const uint32_t *bx, const uint32_t *const *evk_b,
                            const uint32_t *const *evk_a, int key_main);
/* Hoisted rotations: n_rot homomorphic rotations of one ciphertext (bx, ax)
 * that share a single ModUp of ax; each rotation is the evaluation-key inner
 * product fused with its automorphism (the reference's HoistHandler baby step,
 * src/extension/Hoist.cu:578-691 with kernel :20-78), followed by ModDown.
 * rot[i] > 0 is the slot distance (negative: conjugation); the keys are laid
 * out as for Context::HRot (src/core/Context.cpp:776-791): evk_b/evk_a are HOST
 * arrays of n_rot*beta device pointers, rotation i digit j at [i*beta + j],
 * beta = cfhe_beta(level). out: [n_rot][2][nq][N] words; every (b, a) pair is
 * word for word what HRot with the same key returns. */
CFHE_API int cfhe_hoisted_rotations(cfhe_context *ctx, int level, uint32_t *out,
                                    const uint32_t *bx, const uint32_t *ax,
                                    int n_rot, const int *rot,
                                    const uint32_t *const *evk_b,
                                    const uint32_t *const *evk_a, int key_main);
/* Baby-step/giant-step linear transform of one ciphertext (the reference's
 * HoistHandler: BSFusedKeyMult and GSFusedPAccum, src/extension/Hoist.cu:20-120,
 * 208-360, driven by LinearTransform::Evaluate,
 * src/extension/LinearTransform.cpp:118-124):
 *   out = Down( sum_j rot_{giant_rot[j]}( Down( sum_i pt[j][i] (*) rot_{baby_rot[i]}(in) ) ) )
 * The baby rotations share one ModUp and stay on the extended basis; the
 * plaintexts are multiplied there; every giant rotation is a key switch added
 * into one extended-basis accumulator, so one ModDown ends the call, fused
 * with the rescale to level-1 when rescale != 0. The sum of the unrotated
 * giant step (giant_rot == 0) skips its inner Down: it starts the accumulator
 * as it is; of a rotating giant step only the a part goes through Down and the
 * key switch, its b part is rotated on the extended basis.
 * baby_rot[0] must be 0 (the input itself); the other baby_rot[i] and the
 * non-zero giant_rot[j] are slot distances in (0, N/2); at most one giant_rot
 * may be 0; n_baby, n_giant <= 16. Keys as for cfhe_hoisted_rotations: HOST
 * arrays of n*beta device pointers, step s digit d at [s*beta + d] (entries of
 * unrotated steps are not read). pt: HOST array of n_giant*n_baby device
 * pointers, pt[j*n_baby + i] = NTT, M-form plaintext on the level's limbs
 * followed by the alpha auxiliary limbs ((nq+alpha)*N words), or NULL. */
CFHE_API int cfhe_linear_transform(cfhe_context *ctx, int level, int rescale,
                                   uint32_t *out_b, uint32_t *out_a,
                                   const uint32_t *in_b, const uint32_t *in_a,
                                   int n_baby, const int *baby_rot,
                                   const uint32_t *const *baby_evk_b,
                                   const uint32_t *const *baby_evk_a,
                                   int n_giant, const int *giant_rot,
                                   const uint32_t *const *giant_evk_b,
                                   const uint32_t *const *giant_evk_a,
                                   const uint32_t *const *pt, int key_main);
/* Context::HMult (Context.cpp:862-871): tensor product, relinearisation and,
 * when rescale != 0, ModDownAndRescale to level-1 (RelinearizeRescale,
 * :714-737); rescale == 0 keeps the level (Relinearize, :561-565). */
CFHE_API int cfhe_hmult(cfhe_context *ctx, int level, uint32_t *out_b,
                        uint32_t *out_a, const uint32_t *b1, const uint32_t *a1,
                        const uint32_t *b2, const uint32_t *a2,
                        const uint32_t *const *evk_b,
                        const uint32_t *const *evk_a, int key_main, int rescale);

/* ---- stage timing (no counterpart in the reference, which only prints
 * wall-clock time per operator, unittest/Testbed.h:24-47). Between begin and
 * end every pipeline stage records a CUDA event on the context's stream;
 * end synchronises and returns the stage count, the milliseconds of each
 * stage in order and their names joined by ';'. ---- */
CFHE_API int cfhe_profile_begin(cfhe_context *ctx);
CFHE_API int cfhe_profile_end(cfhe_context *ctx, char *names, size_t names_cap,
                              float *ms, int cap);

#ifdef __cplusplus
}
#endif
#endif
