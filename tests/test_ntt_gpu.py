"""GPU parity of the batched NTT / INTT against the CPU golden model, through
the C ABI. Bit-exact: every output word must match."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rand_poly(rng, primes, gidx, n, polys=None):
    shape = (n,) if polys is None else (polys, n)
    cols = [rng.integers(0, int(primes[g]), shape, dtype=np.uint64).astype(np.uint32) for g in gidx]
    return np.stack(cols, axis=0 if polys is None else 1)


def test_ntt_matches_oracle_all_primes(engine40, oracle40):
    rng = np.random.default_rng(11)
    g = np.arange(engine40.num_primes)
    a = rand_poly(rng, oracle40.primes, g, oracle40.n)
    # edge values in the first words of every limb
    for l, gi in enumerate(g):
        q = int(oracle40.primes[gi])
        a[l, :4] = [0, q - 1, 1, q - 1]
    for mc in (False, True):
        assert np.array_equal(engine40.ntt(a, g, mc), oracle40.ntt(a, g, mc))


def test_intt_matches_oracle_all_primes(engine40, oracle40):
    rng = np.random.default_rng(12)
    g = np.arange(engine40.num_primes)
    a = rand_poly(rng, oracle40.primes, g, oracle40.n)
    k = np.array([rng.integers(1, int(oracle40.primes[gi])) for gi in g], dtype=np.uint32)
    assert np.array_equal(engine40.intt(a, g), oracle40.intt(a, g))
    assert np.array_equal(engine40.intt(a, g, mont_keep=True), oracle40.intt(a, g, mont_keep=True))
    for cen in (False, True):
        assert np.array_equal(engine40.intt(a, g, k, centred=cen), oracle40.intt(a, g, k, centred=cen))


def test_config1_batch_roundtrip_and_sample_parity(engine40, oracle40):
    """Config 1: 16 polynomials x the first 40 Q limbs; forward then inverse
    is the identity at full size, and two polynomials are checked word for
    word against the golden model."""
    rng = np.random.default_rng(13)
    g = engine40.level_limbs(28)[:40]
    a = rand_poly(rng, oracle40.primes, g, oracle40.n, polys=16)
    d = engine40.to_dev(a)
    f = engine40.torch.empty_like(d)
    engine40.ntt_(f, d, g)
    back = engine40.torch.empty_like(d)
    engine40.intt_(back, f, g, mont_keep=True)
    assert np.array_equal(engine40.to_host(back), a)
    fh = engine40.to_host(f)
    for p in (0, 15):
        assert np.array_equal(fh[p], oracle40.ntt(a[p], g))
    # in place
    engine40.ntt_(d, d, g)
    assert np.array_equal(engine40.to_host(d), fh)


def test_single_limb_and_subset(engine40, oracle40):
    rng = np.random.default_rng(14)
    for g in ([58], [0, 46, 47], [5]):
        a = rand_poly(rng, oracle40.primes, g, oracle40.n)
        assert np.array_equal(engine40.ntt(a, g), oracle40.ntt(a, g))


def test_bad_arguments_fail_loudly(engine40, pkg):
    a = engine40.empty(1, engine40.n)
    with pytest.raises(pkg.CfheError):
        engine40.ntt_(a, a, [engine40.num_primes])
