// Level-aware pipelines built from the kernels (see pipeline.cu).
#pragma once
#include <algorithm>

#include "context.h"
#include "kernels.h"

namespace cfhe {

size_t modup_scratch_words(const LevelPlan &lp);
size_t moddown_scratch_words(const ConvPlan &cv, int n_polys);
size_t keyswitch_scratch_words(const LevelPlan &lp, int down_type);

// mu: beta buffers of ntot limbs (slot = digit number); y: nq limbs scratch
int run_modup(const Context &c, const LevelPlan &lp, uint32_t *mu,
              const uint32_t *src, bool copy_own, uint32_t *y);
int run_moddown_intt(const Context &c, const ConvPlan &cv, uint32_t *y, const uint32_t *src, int n_polys,
                     long long src_stride);
int run_moddown_bconv(const Context &c, const ConvPlan &cv, uint32_t *dst, uint32_t *y, int n_polys,
                      long long dst_stride);
int run_moddown_ntt(const Context &c, const ConvPlan &cv, uint32_t *dst, const uint32_t *src, int n_polys,
                    long long dst_stride, long long src_stride);
int run_moddown(const Context &c, const ConvPlan &cv, uint32_t *dst,
                const uint32_t *src, int n_polys, long long dst_stride,
                long long src_stride, uint32_t *y);
int run_inner(const Context &c, const LevelPlan &lp, uint32_t *acc_b,
              uint32_t *acc_a, const uint32_t *mu, const uint32_t *d,
              const uint32_t *c0, const uint32_t *c1,
              const uint32_t *const *kb, const uint32_t *const *ka,
              int key_main);
// galois_inv != 0: the result is additionally permuted by the automorphism
// whose inverse Galois element is galois_inv (fused into the store)
int run_inner_rot(const Context &c, const LevelPlan &lp, uint32_t *acc_b,
                  uint32_t *acc_a, const uint32_t *mu, const uint32_t *d,
                  const uint32_t *c0, const uint32_t *const *kb,
                  const uint32_t *const *ka, int key_main, uint32_t galois_inv);
// Hoisted rotations: one ModUp of `a` shared by n_rot key switches, each fused
// with its automorphism; out = [n_rot][2][nq][N].
int run_hoisted_rotations(Context &c, const LevelPlan &lp, uint32_t *out,
                          const uint32_t *b, const uint32_t *a, int n_rot,
                          const uint32_t *galois, const uint32_t *const *kb,
                          const uint32_t *const *ka, int key_main,
                          uint32_t *scratch);
size_t hoisted_scratch_words(const LevelPlan &lp);
// Baby-step/giant-step linear transform with both hoistings (see pipeline.cu).
// baby_galois[0] must be 1; key arrays hold beta pointers per step (entries of
// unrotated steps are not read); pt[j*n_baby+i] on the extended basis or null.
int run_linear_transform(Context &c, const LevelPlan &lp, bool rescale, uint32_t *out_b,
                         uint32_t *out_a, const uint32_t *in_b, const uint32_t *in_a,
                         int n_baby, const uint32_t *baby_galois,
                         const uint32_t *const *baby_kb, const uint32_t *const *baby_ka,
                         int n_giant, const uint32_t *giant_galois,
                         const uint32_t *const *giant_kb, const uint32_t *const *giant_ka,
                         const uint32_t *const *pt, int key_main, uint32_t *scratch);
size_t linear_transform_scratch_words(const LevelPlan &lp, int n_baby, int n_giant, bool rescale,
                                      bool stored_rotations);
int run_tensor(const Context &c, const LevelPlan &lp, uint32_t *d0,
               uint32_t *d1, uint32_t *d2, const uint32_t *b1,
               const uint32_t *a1, const uint32_t *b2, const uint32_t *a2);
// (out_b, out_a) = Down( sum_i ModUp_i(d) * key_i + P * (c0, c1) )
int run_keyswitch(Context &c, const LevelPlan &lp, int down_type,
                  uint32_t *out_b, uint32_t *out_a, const uint32_t *d,
                  const uint32_t *c0, const uint32_t *c1,
                  const uint32_t *const *kb, const uint32_t *const *ka,
                  int key_main, uint32_t *scratch);

}  // namespace cfhe
