"""Device-side sampling and the fused client kernels.

cfhe_sample_uniform and cfhe_sample_error are reproduced word for word on the
host from the published Philox-4x32-10 round function and the library's own
cumulative table; the fused Encrypt / AddEvkPart / PseudoModUp kernels are
compared with the same expressions composed from the golden model's
single operators."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = np.uint64(0xFFFFFFFF)


def philox(c0, c1, c2, c3, k0, k1):
    """Ten Philox-4x32 rounds on arrays of counters (uint64 holding 32-bit values)."""
    c = [np.asarray(x, dtype=np.uint64) for x in (c0, c1, c2, c3)]
    k0, k1 = np.uint64(k0), np.uint64(k1)
    for _ in range(10):
        p0, p1 = np.uint64(M0) * c[0], np.uint64(M1) * c[2]
        c = [(p1 >> np.uint64(32)) ^ c[1] ^ k0, p1 & MASK, (p0 >> np.uint64(32)) ^ c[3] ^ k1, p0 & MASK]
        k0 = (k0 + np.uint64(W0)) & MASK
        k1 = (k1 + np.uint64(W1)) & MASK
    return c


def host_uniform(n, g, q, seed, stream):
    """The library's multiply-and-reject map, limb with prime index g."""
    v = np.arange(n // 4, dtype=np.uint64)
    out = np.zeros((n // 4, 4), dtype=np.uint64)
    done = np.zeros((n // 4, 4), dtype=bool)
    reject_below = np.uint64((1 << 32) % q)
    for d in range(16):
        r = philox(v, np.full_like(v, g), np.full_like(v, d), np.full_like(v, stream), seed & 0xFFFFFFFF, seed >> 32)
        for e in range(4):
            m = r[e] * np.uint64(q)
            take = ~done[:, e]
            out[take, e] = (m >> np.uint64(32))[take]
            ok = ((m & MASK) >= reject_below) | (d == 15)
            done[:, e] |= take & ok
        if done.all():
            break
    return out.reshape(-1).astype(np.uint32)


def test_uniform_samples_are_reproducible_and_uniform(engine40):
    e = engine40
    g = [0, 3, 30, 50, 58]  # terminal, main below 2^30, main above, auxiliary primes
    dst = e.empty(len(g), e.n)
    seed = 0x1234_5678_9ABC_DEF0
    e.sample_uniform_(dst, g, seed, stream=7)
    got = e.to_host(dst)
    for l, gi in enumerate(g):
        q = int(e.primes[gi])
        assert np.array_equal(got[l], host_uniform(e.n, gi, q, seed, 7)), gi
        assert got[l].max() < q
        # crude uniformity: mean within 5 standard errors of (q - 1) / 2
        assert abs(got[l].mean() - (q - 1) / 2) < 5 * q / math.sqrt(12 * e.n)
    again = e.empty(len(g), e.n)
    e.sample_uniform_(again, g, seed, stream=7)
    assert e.torch.equal(again, dst)
    e.sample_uniform_(again, g, seed + 1, stream=7)
    assert not e.torch.equal(again, dst)


def test_error_samples_follow_the_table(engine40):
    e = engine40
    sigma, seed = 3.2, 0xDEADBEEF
    cdf = e.error_cdf(sigma)
    # the table is the rounded normal's cumulative distribution in 64-bit fixed point
    for k in (-10, -1, 0, 1, 10):
        p = 0.5 * math.erfc(-(k + 0.5) / (sigma * math.sqrt(2)))
        assert abs(int(cdf[k + 48]) / 2.0 ** 64 - p) < 1e-12
    assert int(cdf[-1]) == 2 ** 64 - 1 and np.all(np.diff(cdf.astype(object)) >= 0)
    g = [0, 10, 47]
    dst = e.empty(len(g), e.n)
    e.sample_error_(dst, g, sigma, seed, stream=1)
    got = e.to_host(dst)
    v = np.arange(e.n // 2, dtype=np.uint64)
    r = philox(v, np.full_like(v, 0xE0E0E0E0), np.zeros_like(v), np.full_like(v, 1), seed & 0xFFFFFFFF, seed >> 32)
    u = np.stack([(r[1] << np.uint64(32)) | r[0], (r[3] << np.uint64(32)) | r[2]], axis=1).reshape(-1)
    err = np.searchsorted(cdf, u, side="right").astype(np.int64) - 48
    for l, gi in enumerate(g):
        q = int(e.primes[gi])
        assert np.array_equal(got[l], np.where(err < 0, q + err, err).astype(np.uint32)), gi
    assert abs(err.mean()) < 5 * sigma / math.sqrt(e.n)
    assert abs(err.std() - math.sqrt(sigma ** 2 + 1 / 12)) < 0.05


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


def test_fused_client_kernels_match_the_composition(engine40, oracle40):
    e, o = engine40, oracle40
    rng = np.random.default_rng(5150)
    level = 12
    g = e.level_limbs(level)
    a, s, err, m = (rand_limbs(rng, o.primes, g, o.n) for _ in range(4))
    da, ds, de, dm = (e.to_dev(x) for x in (a, s, err, m))
    b = e.empty(len(g), e.n)
    e.encrypt_(b, da, ds, de, dm, g)           # m + e - a*s
    want = o.add(o.sub(err, o.mul(a, s, g), g), m, g)
    assert np.array_equal(e.to_host(b), want)
    e.encrypt_(b, da, ds, de, None, g)         # encryption of zero
    zero = o.sub(err, o.mul(a, s, g), g)
    assert np.array_equal(e.to_host(b), zero)
    k = np.array([rng.integers(0, int(o.primes[gi])) for gi in g], dtype=np.uint32)
    e.add_evk_part_(b, ds, k, g)               # b += k * s
    assert np.array_equal(e.to_host(b), o.add(zero, o.const_op(s, k, g, 3), g))
    # PseudoModUp: multiplication by P mod q_l in M-form
    P = 1
    for p in e.p["auxiliary_primes"]:
        P *= int(p)
    pm = np.array([((P % int(o.primes[gi])) << 32) % int(o.primes[gi]) for gi in g], dtype=np.uint32)
    out = e.empty(len(g), e.n)
    e.pseudo_modup_(level, out, da)
    assert np.array_equal(e.to_host(out), o.const_op(a, pm, g, 3))


def test_encode_coeffs_reduces_any_double_exactly(engine40, oracle40):
    """cfhe_encode_coeffs against exact integer arithmetic: residues of
    trunc(v) (toward zero, as the reference's conversion of a scaled
    coefficient to a big integer, src/core/Encode.cpp:136-248) for magnitudes
    from fractions to 2^120, then the golden model's forward NTT with
    Montgomery conversion. Every word must match."""
    e, o = engine40, oracle40
    rng = np.random.default_rng(4242)
    n = o.n
    v = np.zeros(n, dtype=np.float64)
    mags = [0.0, 0.49, 0.99, 1.0, 1.5, 2.0 ** 31, 2.0 ** 40 + 0.75, 2.0 ** 52 + 1, 2.0 ** 53, 2.0 ** 62,
            2.0 ** 63, 2.0 ** 64 + 2.0 ** 13, 2.0 ** 80 * 1.2345678901234567, 2.0 ** 100 * 1.999999, 2.0 ** 120]
    for i, m in enumerate(mags):
        v[2 * i], v[2 * i + 1] = m, -m
    k = 2 * len(mags)
    expo = rng.integers(-3, 110, n - k)
    v[k:] = rng.uniform(-1.0, 1.0, n - k) * np.exp2(expo.astype(np.float64))
    g = e.level_limbs(16, 12)  # main, terminal and auxiliary primes
    want_coeff = np.stack([np.array([int(x) % int(o.primes[gi]) for x in v], dtype=np.uint64).astype(np.uint32)
                           for gi in g])
    want = o.ntt(want_coeff, g, mont_conv=True)
    dst = e.empty(len(g), n)
    e.encode_coeffs_(dst, v, g)
    assert np.array_equal(e.to_host(dst), want)
