"""The ciphertext x plaintext RNS GEMM on the tensor cores (cfhe_ctpt_gemm)
against the same contraction composed from the golden model's constant
multiplication and addition: every output word must match. Parity for this
operator is pinned by the golden model only; the reference has no kernel for
it (its nearest operator is CAccum, src/core/ElementWise.cu:1355-1394)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


@pytest.mark.parametrize("n_in,n_out", [(16, 64), (40, 100), (5, 3), (272, 64)])
def test_ctpt_gemm_matches_oracle(engine40, oracle40, n_in, n_out):
    e, o = engine40, oracle40
    rng = np.random.default_rng(6000 + n_in)
    g = [0, 10, 30, 52]  # a terminal prime, main primes on both sides of 2^30, an auxiliary prime
    xs_h = [rand_limbs(rng, o.primes, g, o.n) for _ in range(n_in)]
    for l, gi in enumerate(g):  # extreme residues
        q = int(o.primes[gi])
        xs_h[0][l, :3] = [q - 1, 0, 1]
        xs_h[-1][l, :2] = [q - 1, q - 1]
    w = np.stack([rng.integers(0, int(o.primes[gi]), (n_in, n_out), dtype=np.uint64).astype(np.uint32) for gi in g])
    for l, gi in enumerate(g):
        w[l, 0, 0] = int(o.primes[gi]) - 1
        w[l, -1, -1] = int(o.primes[gi]) - 1
    xs = [e.to_dev(x) for x in xs_h]
    ys = [e.empty(len(g), e.n) for _ in range(n_out)]
    for y in ys:
        y.fill_(-1)
    packed = e.gemm_pack_weights(w, g)
    e.ctpt_gemm_(ys, xs, packed, g)
    e.synchronize()
    check = sorted({0, n_out - 1, n_out // 2, int(rng.integers(0, n_out)), int(rng.integers(0, n_out))})
    for j in check:
        want = None
        for k in range(n_in):
            term = o.const_op(xs_h[k], w[:, k, j], g, 3)
            want = term if want is None else o.add(want, term, g)
        assert np.array_equal(e.to_host(ys[j]), want), (n_in, n_out, j)


def test_ctpt_gemm_equals_caccum(engine40):
    """The tensor-core path and the fused SIMT sum give the same words."""
    e = engine40
    rng = np.random.default_rng(6100)
    g = list(e.level_limbs(6))
    n_in, n_out = 8, 2
    primes = [int(e.primes[gi]) for gi in g]
    xs = [e.to_dev(rand_limbs(rng, e.primes, g, e.n)) for _ in range(n_in)]
    w = np.stack([rng.integers(0, q, (n_in, n_out), dtype=np.uint64).astype(np.uint32) for q in primes])
    ys = [e.empty(len(g), e.n) for _ in range(n_out)]
    e.ctpt_gemm_(ys, xs, e.gemm_pack_weights(w, g), g)
    for j in range(n_out):
        ref = e.empty(len(g), e.n)
        e.nary_("const", [ref], [[x] for x in xs], g, consts=w[:, :, j].T)
        e.synchronize()
        assert e.torch.equal(ref, ys[j]), j


def test_ctpt_gemm_argument_checks(engine40, pkg):
    e = engine40
    g = [0, 1]
    x = e.empty(2, e.n)
    w = np.zeros((2, 1, 1), dtype=np.uint32)
    packed = e.gemm_pack_weights(w, g)
    with pytest.raises(pkg.CfheError):
        e.ctpt_gemm_([x], [x], packed, [0, 999])
