"""CPU checks of the golden model itself and of the host-side pieces of the
library (no GPU needed)."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import load_package

_client = load_package().client
Client, brev, negacyclic_mul, toy_params = _client.Client, _client.brev, _client.negacyclic_mul, _client.toy_params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def toy():
    from oracle import Oracle
    return Oracle(toy_params(5))


def test_psi_is_primitive_root_from_smallest_generator(oracle40):
    """psi = g^((q-1)/2N) for the smallest primitive root g
    (reference include/common/PrimeUtils.h:135-196)."""
    o = oracle40
    for g in (0, 4, 27, 47, 58):
        q = int(o.primes[g])
        psi = o.psi(g)
        assert pow(psi, o.n, q) == q - 1
        gen = o.L.orc_find_generator(q)
        assert pow(gen, (q - 1) // (2 * o.n), q) == psi
        # smaller candidates are not generators
        fac = [f for f in range(2, 2000) if (q - 1) % f == 0 and all(f % d for d in range(2, f))]
        for r in range(2, gen):
            assert any(pow(r, (q - 1) // f, q) == 1 for f in fac)


def test_qinv(oracle40):
    for g in range(oracle40.num_primes):
        q = int(oracle40.primes[g])
        assert (q * (oracle40.qinv(g) & 0xFFFFFFFF)) & 0xFFFFFFFF == 1


def test_ntt_is_bitreversed_evaluation_at_odd_powers(toy):
    """A[i] = sum_j a_j psi^((2*brev(i)+1) j): the ordering the reference's
    automorphism index formula relies on (src/core/ElementWise.cu:377-382)."""
    o = toy
    rng = np.random.default_rng(1)
    g = list(range(o.num_primes))
    a = np.stack([rng.integers(0, int(o.primes[i]), o.n) for i in g]).astype(np.uint32)
    A = o.ntt(a, g)
    logn = o.p["log_degree"]
    for li, gi in enumerate(g):
        q, psi = int(o.primes[gi]), o.psi(gi)
        for i in range(o.n):
            e = 2 * brev(i, logn) + 1
            assert sum(int(a[li, j]) * pow(psi, e * j, q) for j in range(o.n)) % q == int(A[li, i])
    assert np.array_equal(o.intt(A, g, mont_keep=True), a)
    # default INTT leaves the Montgomery form: result = a * 2^-32
    back = o.intt(A, g)
    for li, gi in enumerate(g):
        q = int(o.primes[gi])
        assert all((int(a[li, j]) * pow(1 << 32, -1, q)) % q == int(back[li, j]) for j in range(o.n))


def test_permute_is_the_galois_automorphism(toy):
    o = toy
    rng = np.random.default_rng(2)
    g = [0, 5]
    coefs = rng.integers(-50, 50, o.n)
    cl = Client(o, seed=1)
    A = cl.to_ntt(coefs, g)
    for rot in (1, 3, -1):
        gal = o.galois(rot)
        # sigma_gal on coefficients: X^j -> X^(j*gal mod 2N) with sign
        out = np.zeros(o.n, dtype=np.int64)
        for j in range(o.n):
            e = (j * gal) % (2 * o.n)
            if e < o.n:
                out[e] += coefs[j]
            else:
                out[e - o.n] -= coefs[j]
        assert np.array_equal(o.permute(A, gal), cl.to_ntt(out, g))


def test_bconv_is_exact_crt_lift(toy):
    """Base conversion of centred, pre-scaled residues reproduces the integer
    (up to a multiple of the source modulus bounded by half the digit size)."""
    o = toy
    rng = np.random.default_rng(3)
    src, dst = [2, 3, 4], [0, 1, 5, 6, 11, 12]
    qs = [int(o.primes[g]) for g in src]
    S = int(np.prod(np.array(qs, dtype=object)))
    x = [int(v) for v in rng.integers(-2 ** 40, 2 ** 40, o.n)]
    y = np.zeros((len(src), o.n), np.int32)
    for k, q in enumerate(qs):
        Sk = S // q
        for j in range(o.n):
            v = (x[j] * pow(Sk, -1, q)) % q
            y[k, j] = v - q if v > q // 2 else v
    out = o.bconv(y, src, dst)
    for m, g in enumerate(dst):
        p = int(o.primes[g])
        for j in range(o.n):
            lifted = sum(int(y[k, j]) * (S // qs[k]) for k in range(len(src)))
            assert (lifted - x[j]) % S == 0 and abs(lifted - x[j]) <= 2 * S
            assert int(out[m, j]) == (lifted << 32) % p


@pytest.mark.parametrize("level", [1, 2, 3, 4, 5, 6])
def test_hmult_decrypts_to_product_on_toy_ring(toy, level):
    """End-to-end meaning of ModUp / inner product / ModDown(+Rescale) with
    terminal primes dropped and restored (rational rescaling)."""
    o = toy
    cl = Client(o, seed=3)
    kb, ka = cl.mult_key(7)
    rng = np.random.default_rng(5 + level)
    m1 = rng.integers(-2 ** 18, 2 ** 18, o.n)
    m2 = rng.integers(-2 ** 18, 2 ** 18, o.n)
    b1, a1 = cl.encrypt(m1, level)
    b2, a2 = cl.encrypt(m2, level)
    g = o.level_limbs(level)
    prod = negacyclic_mul(m1, m2)
    for rescale in (False, True):
        ob, oa = o.hmult(level, b1, a1, b2, a2, kb, ka, 7, rescale)
        gd = o.level_limbs(level - 1 if rescale else level)
        dec = cl.decrypt(ob, oa, gd)
        num = den = 1
        if rescale:
            for x in set(map(int, g)) - set(map(int, gd)):
                num *= int(o.primes[x])
            for x in set(map(int, gd)) - set(map(int, g)):
                den *= int(o.primes[x])
        exp = np.array([int(v) * den / num for v in prod])
        err = np.abs(np.array([float(x) for x in dec]) - exp).max()
        assert err < (2e8 if not rescale else 64), (level, rescale, err)


def test_rotation_keyswitch_on_toy_ring(toy):
    o = toy
    cl = Client(o, seed=4)
    level, rot = 4, 3
    kb, ka = cl.rotation_key(rot, 7)
    rng = np.random.default_rng(9)
    m = rng.integers(-2 ** 18, 2 ** 18, o.n)
    b, a = cl.encrypt(m, level)
    g = o.level_limbs(level)
    ob, oa = o.keyswitch(level, a, b, kb, ka, 7)
    gal = o.galois(rot)
    rb, ra = o.permute(ob, gal), o.permute(oa, gal)
    dec = cl.decrypt(rb, ra, g)
    out = np.zeros(o.n, dtype=np.int64)
    for j in range(o.n):
        e = (j * gal) % (2 * o.n)
        if e < o.n:
            out[e] += m[j]
        else:
            out[e - o.n] -= m[j]
    assert np.abs(np.array([int(x) for x in dec]) - out).max() < 4096


def test_emulated_kernel_phases_match_oracle(oracle40):
    """The per-thread phase functions of the cluster NTT kernels, run on the
    host for every (CTA, thread), give the golden model's words."""
    so = os.path.join(ROOT, "tests", "emu", "libnttemu.so")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I",
                           os.path.join(ROOT, "cheddar-fhe_b200", "csrc"), "-o", so,
                           os.path.join(ROOT, "tests", "emu", "ntt_emu.cpp")])
    emu = C.CDLL(so)
    u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
    emu.emu_ntt_fwd.argtypes = [C.c_uint32, u32p, u32p, C.c_int, C.c_int]
    emu.emu_ntt_inv.argtypes = [C.c_uint32, u32p, u32p, C.c_uint32, C.c_int, C.c_int]
    o = oracle40
    rng = np.random.default_rng(0)
    for g in (3, 4, 5, 47):
        q = int(o.primes[g])
        a = rng.integers(0, q, o.n, dtype=np.uint64).astype(np.uint32)
        a[:4] = [0, q - 1, 1, q - 1]
        for mc in (0, 1):
            out = np.empty_like(a)
            emu.emu_ntt_fwd(q, a, out, mc, 0)
            assert np.array_equal(out, o.ntt(a[None, :], [g], bool(mc))[0])
        k = int(rng.integers(1, q))
        for cen in (0, 1):
            out = np.empty_like(a)
            emu.emu_ntt_inv(q, a, out, k, cen, 0)
            assert np.array_equal(out, o.intt(a[None, :], [g], np.array([k], np.uint32), False, bool(cen))[0])


def test_library_exports_every_declared_symbol(pkg):
    """The C-ABI library loads and exports each function the header declares
    (no compute call is made here)."""
    hdr = open(pkg.HEADER_PATH).read()
    names = set(re.findall(r"\b(cfhe_[a-z0-9_]+)\s*\(", hdr))
    assert len(names) >= 10
    if not os.path.exists(pkg.LIB_PATH):
        pkg.build()
    lib = C.CDLL(pkg.LIB_PATH)
    for n in sorted(names):
        assert hasattr(lib, n), n


def test_modup_to_max_is_the_centred_lift(oracle40):
    """Golden model of the bootstrapping lift (reference ModUpToMax1/2,
    src/core/ElementWise.cu:579-623) against Python integers."""
    o = oracle40
    rng = np.random.default_rng(9)
    base = [2, 3]
    q0, q1 = int(o.primes[2]), int(o.primes[3])
    xs = [0, 1, -1, (q0 * q1 - 1) // 2, -((q0 * q1 - 1) // 2)] + [int(v) for v in rng.integers(-2**48, 2**48, 11)]
    src = np.zeros((2, o.n), dtype=np.uint32)
    for i, x in enumerate(xs):
        src[0, i] = (x * pow(q1, -1, q0)) % q0
        src[1, i] = (x * pow(q0, -1, q1)) % q1
    dst = [0, 4, 30, 47, 58]
    out = o.modup_to_max(src, base, dst)
    for i, x in enumerate(xs):
        for m, g in enumerate(dst):
            assert int(out[m, i]) == x % int(o.primes[g])
    one = o.modup_to_max(src[:1], base[:1], dst)
    for m, g in enumerate(dst):
        assert int(one[m, 3]) == int(src[0, 3]) % int(o.primes[g])


# ---------------------------------------------------------------------------
# Golden vectors produced by the reference's own CUDA library
# ---------------------------------------------------------------------------
def _golden():
    import importlib.util
    import json
    import os
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(here, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(here, "reference_digests.json")) as f:
        return mod, json.load(f)["cases"]


def _matches(case, arr):
    import hashlib
    a = np.ascontiguousarray(arr, dtype=np.uint32)
    assert list(a.shape) == case["shape"]
    assert a.reshape(-1, a.shape[-1])[:, :len(case["head"][0])].tolist() == case["head"]
    assert hashlib.sha256(a.tobytes()).hexdigest() == case["sha256"]


def test_oracle_ntt_equals_reference_golden(oracle40):
    """NTT / INTT words of the golden model against digests of the reference's
    own kernels (tests/golden/make_golden.py generated them on a B200)."""
    g_mod, cases = _golden()
    o = oracle40
    for case in g_mod.NTT_CASES:
        g = g_mod.ntt_limbs(case)
        a = g_mod.rand_limbs(np.random.default_rng(9000 + sum(case)), o.primes, g)
        for mont in (False, True):
            _matches(cases[f"ntt{case}_inv0_mont{int(mont)}"], o.ntt(a, g, mont))
            # the reference's INTT with montgomery conversion leaves M-form
            _matches(cases[f"ntt{case}_inv1_mont{int(mont)}"], o.intt(a, g, mont_keep=not mont))


def test_oracle_modswitch_equals_reference_golden(oracle40):
    g_mod, cases = _golden()
    o = oracle40
    for level in g_mod.MODUP_LEVELS:
        a = g_mod.rand_limbs(np.random.default_rng(9100 + level), o.primes, o.level_limbs(level))
        _matches(cases[f"modup_level{level}"], o.modup(level, a))
    for level in g_mod.MODDOWN_LEVELS:
        full = o.level_limbs(level, 12)
        a = g_mod.rand_limbs(np.random.default_rng(9200 + level), o.primes, full)
        nq = len(full) - 12
        for kind in (0, 1, 2):
            x = a if kind != 1 else np.ascontiguousarray(a[:nq])
            _matches(cases[f"moddown_level{level}_kind{kind}"], o.moddown(level, kind, x))


def test_oracle_hmult_equals_reference_golden(oracle40):
    g_mod, cases = _golden()
    o = oracle40
    kg = list(range(47)) + [47 + a for a in range(12)]
    for level, rescale in g_mod.HMULT_CASES:
        rng = np.random.default_rng(9300 + level)
        g = o.level_limbs(level)
        ins = [g_mod.rand_limbs(rng, o.primes, g) for _ in range(4)]
        beta = o.beta(28)
        kb = [g_mod.rand_limbs(rng, o.primes, kg) for _ in range(beta)]
        ka = [g_mod.rand_limbs(rng, o.primes, kg) for _ in range(beta)]
        b, a = o.hmult(level, *ins, kb, ka, 43, rescale)
        _matches(cases[f"hmult_level{level}_rescale{int(rescale)}"], np.stack([b, a]))
