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

/* Use an existing cudaStream_t (NULL restores the context's own stream). The
 * reference runs everything on the legacy default stream
 * (include/core/DeviceVector.h:88). */
CFHE_API int cfhe_set_stream(cfhe_context *ctx, void *cuda_stream);
CFHE_API int cfhe_synchronize(cfhe_context *ctx);

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

#ifdef __cplusplus
}
#endif
#endif
