"""Pins the golden model and the engine to the reference itself: the
reference's own CUDA library (built unmodified into oracle/_ref by
`make -C oracle ref`) runs on the same device buffers and every output word
must match. Skipped when that library was not built (it needs the reference
tree at build time; the tests never read the tree)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(params40):
    from oracle import ref_binding
    if not ref_binding.available():
        pytest.skip("oracle/_ref/libcheddar_ref.so not built")
    r = ref_binding.Reference(params40)
    yield r
    r.close()


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


@pytest.mark.parametrize("np_", [(43, 4, 12), (23, 0, 0), (0, 2, 0), (36, 4, 0)])
def test_ntt_words_equal_reference(engine40, oracle40, ref, np_):
    e, o = engine40, oracle40
    nm, nt, na = np_
    T, L = 4, 47
    g = list(range(T - nt, T + nm)) + [L + a for a in range(na)]
    rng = np.random.default_rng(sum(np_))
    a = rand_limbs(rng, o.primes, g, e.n)
    src = e.to_dev(a)
    for mont in (False, True):
        out_ref = e.torch.empty_like(src)
        ref.ntt(out_ref, src, nm, nt, na, inverse=False, mont_conv=mont)
        want = e.to_host(out_ref)
        assert np.array_equal(e.ntt(a, g, mont), want)
        assert np.array_equal(o.ntt(a, g, mont), want)
    for mont in (False, True):  # reference INTT: mont_conv=True leaves M-form
        out_ref = e.torch.empty_like(src)
        ref.ntt(out_ref, src, nm, nt, na, inverse=True, mont_conv=mont)
        want = e.to_host(out_ref)
        assert np.array_equal(e.intt(a, g, mont_keep=not mont), want)
        assert np.array_equal(o.intt(a, g, mont_keep=not mont), want)


@pytest.mark.parametrize("level", [28, 16, 9, 2, 0])
def test_modup_words_equal_reference(engine40, oracle40, ref, level):
    e, o = engine40, oracle40
    rng = np.random.default_rng(600 + level)
    g = e.level_limbs(level)
    a = rand_limbs(rng, o.primes, g, e.n)
    src = e.to_dev(a)
    ntot = len(g) + 12
    out = e.torch.zeros((e.beta(level), ntot, e.n), dtype=e.torch.int32, device=src.device)
    ref.modup(level, out, src)
    want = e.to_host(out)
    got = e.modup(level, a)
    assert np.array_equal(got, want)
    assert np.array_equal(o.modup(level, a), want)


@pytest.mark.parametrize("level", [28, 27, 17, 14, 3, 2, 1])
def test_moddown_family_words_equal_reference(engine40, oracle40, ref, level):
    e, o = engine40, oracle40
    rng = np.random.default_rng(700 + level)
    full = e.level_limbs(level, 12)
    a = rand_limbs(rng, o.primes, full, e.n)
    src = e.to_dev(a)
    nq = len(full) - 12
    for kind in (0, 2, 1):
        x = a if kind != 1 else np.ascontiguousarray(a[:nq])
        xs = src if kind != 1 else e.to_dev(x)
        nd = len(e.level_limbs(level if kind == 0 else level - 1))
        out = e.empty(nd, e.n)
        ref.moddown(level, kind, out, xs)
        want = e.to_host(out)
        assert np.array_equal(e.moddown(level, kind, x), want), kind
        assert np.array_equal(o.moddown(level, kind, x), want), kind


@pytest.mark.parametrize("level,rescale", [(28, True), (28, False), (16, True), (3, True), (1, True)])
def test_hmult_words_equal_reference(engine40, oracle40, ref, level, rescale):
    e, o = engine40, oracle40
    rng = np.random.default_rng(800 + level)
    g = e.level_limbs(level)
    ins = [rand_limbs(rng, o.primes, g, e.n) for _ in range(4)]
    kg = list(range(47)) + [47 + a for a in range(12)]
    beta = e.beta(28)
    kb = [rand_limbs(rng, o.primes, kg, e.n) for _ in range(beta)]
    ka = [rand_limbs(rng, o.primes, kg, e.n) for _ in range(beta)]
    d_ins = [e.to_dev(x) for x in ins]
    dkb, dka = [e.to_dev(x) for x in kb], [e.to_dev(x) for x in ka]
    nd = len(e.level_limbs(level - 1 if rescale else level))
    rb, ra = e.empty(nd, e.n), e.empty(nd, e.n)
    ref.hmult(level, rb, ra, *d_ins, dkb, dka, 43, rescale)
    got = e.hmult(level, *ins, kb, ka, 43, rescale)
    assert np.array_equal(got[0], e.to_host(rb)) and np.array_equal(got[1], e.to_host(ra))
    if level in (28, 1):
        exp = o.hmult(level, *ins, kb, ka, 43, rescale)
        assert np.array_equal(exp[0], e.to_host(rb)) and np.array_equal(exp[1], e.to_host(ra))
