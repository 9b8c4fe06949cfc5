/* Minimal declarations of the GMP integer functions the reference's
 * BigInt_gmp.cpp calls, for linking against the libgmp.so.10 present in the
 * image (no gmp.h is installed). Layout of __mpz_struct and the __gmpz_* entry
 * names are GMP's public, stable ABI. Test infrastructure only. */
#ifndef CFHE_GMP_SHIM_H
#define CFHE_GMP_SHIM_H
#ifdef __cplusplus
extern "C" {
#endif
typedef unsigned long mp_limb_t;
typedef struct {
  int _mp_alloc;
  int _mp_size;
  mp_limb_t *_mp_d;
} __mpz_struct;
typedef __mpz_struct mpz_t[1];
typedef __mpz_struct *mpz_ptr;
typedef const __mpz_struct *mpz_srcptr;
#define mpz_init __gmpz_init
#define mpz_clear __gmpz_clear
#define mpz_set __gmpz_set
#define mpz_set_ui __gmpz_set_ui
#define mpz_set_d __gmpz_set_d
#define mpz_get_ui __gmpz_get_ui
#define mpz_get_d __gmpz_get_d
#define mpz_neg __gmpz_neg
#define mpz_add __gmpz_add
#define mpz_sub __gmpz_sub
#define mpz_mul __gmpz_mul
#define mpz_mod __gmpz_mod
#define mpz_cmp __gmpz_cmp
#define mpz_fdiv_q_2exp __gmpz_fdiv_q_2exp
void __gmpz_init(mpz_ptr);
void __gmpz_clear(mpz_ptr);
void __gmpz_set(mpz_ptr, mpz_srcptr);
void __gmpz_set_ui(mpz_ptr, unsigned long);
void __gmpz_set_d(mpz_ptr, double);
unsigned long __gmpz_get_ui(mpz_srcptr);
double __gmpz_get_d(mpz_srcptr);
void __gmpz_neg(mpz_ptr, mpz_srcptr);
void __gmpz_add(mpz_ptr, mpz_srcptr, mpz_srcptr);
void __gmpz_sub(mpz_ptr, mpz_srcptr, mpz_srcptr);
void __gmpz_mul(mpz_ptr, mpz_srcptr, mpz_srcptr);
void __gmpz_mod(mpz_ptr, mpz_srcptr, mpz_srcptr);
int __gmpz_cmp(mpz_srcptr, mpz_srcptr);
void __gmpz_fdiv_q_2exp(mpz_ptr, mpz_srcptr, unsigned long);
#define mpz_sgn(Z) ((Z)->_mp_size < 0 ? -1 : (Z)->_mp_size > 0)
#ifdef __cplusplus
}
#endif
#endif
