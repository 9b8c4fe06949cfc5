"""The fused n-ary element-wise entry points (cfhe_accum, cfhe_caccum,
cfhe_paccum, cfhe_permute_accum) against the same sums composed from the golden
model's single operators: every word must match. Shapes follow the reference's
uses: up to eight terms, one to three polynomials, with and without the extra
summand (reference src/core/ElementWise.cu:1002-1226, 1246-1435)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


def mont(x, q):
    return (int(x) << 32) % int(q)


@pytest.mark.parametrize("n_terms,n_polys,with_add", [(1, 1, False), (2, 2, True), (5, 3, False), (8, 2, True)])
def test_accum_and_caccum(engine40, oracle40, n_terms, n_polys, with_add):
    e, o = engine40, oracle40
    rng = np.random.default_rng(1100 + n_terms)
    g = e.level_limbs(20, 12)
    host = [[rand_limbs(rng, o.primes, g, o.n) for _ in range(n_polys)] for _ in range(n_terms)]
    for l, gi in enumerate(g):  # extreme residues in the first words
        q = int(o.primes[gi])
        for t in range(n_terms):
            host[t][0][l, :3] = [q - 1, 0, 1]
    dev = [[e.to_dev(x) for x in term] for term in host]
    add_h = [rand_limbs(rng, o.primes, g, o.n) for _ in range(n_polys)]
    add_d = [e.to_dev(x) for x in add_h]
    out = [e.empty(len(g), e.n) for _ in range(n_polys)]
    # plain sum
    e.nary_("sum", out, dev, g)
    for p in range(n_polys):
        want = host[0][p]
        for t in range(1, n_terms):
            want = o.add(want, host[t][p], g)
        assert np.array_equal(e.to_host(out[p]), want), ("sum", p)
    # constants in M-form, one per term and limb
    k = np.array([[rng.integers(0, int(o.primes[gi])) for gi in g] for _ in range(n_terms)], dtype=np.uint32)
    k[0, 0] = int(o.primes[g[0]]) - 1
    e.nary_("const", out, dev, g, consts=k, addend=add_d if with_add else None)
    for p in range(n_polys):
        want = o.const_op(host[0][p], k[0], g, 3)
        for t in range(1, n_terms):
            want = o.add(want, o.const_op(host[t][p], k[t], g, 3), g)
        if with_add:
            want = o.add(want, add_h[p], g)
        assert np.array_equal(e.to_host(out[p]), want), ("const", p)


@pytest.mark.parametrize("n_terms,n_polys,with_add", [(1, 2, False), (3, 2, True), (8, 2, False)])
def test_paccum_and_permute_accum(engine40, oracle40, n_terms, n_polys, with_add):
    e, o = engine40, oracle40
    rng = np.random.default_rng(1200 + n_terms)
    g = e.level_limbs(16)
    host = [[rand_limbs(rng, o.primes, g, o.n) for _ in range(n_polys)] for _ in range(n_terms)]
    dev = [[e.to_dev(x) for x in term] for term in host]
    pts_h = [rand_limbs(rng, o.primes, g, o.n) for _ in range(n_terms)]
    pts_d = [e.to_dev(x) for x in pts_h]
    add_h = [rand_limbs(rng, o.primes, g, o.n) for _ in range(n_polys)]
    add_d = [e.to_dev(x) for x in add_h]
    out = [e.empty(len(g), e.n) for _ in range(n_polys)]
    e.nary_("plain", out, dev, g, pts=pts_d, addend=add_d if with_add else None)
    for p in range(n_polys):
        want = o.mul(host[0][p], pts_h[0], g)
        for t in range(1, n_terms):
            want = o.add(want, o.mul(host[t][p], pts_h[t], g), g)
        if with_add:
            want = o.add(want, add_h[p], g)
        assert np.array_equal(e.to_host(out[p]), want), ("plain", p)
    rots = [1, 1234, 32767, -1, 5, 64, 4096, 77][:n_terms]
    gal = [o.galois(r) for r in rots]
    e.nary_("permute", out, dev, g, galois=gal, addend=add_d if with_add else None)
    for p in range(n_polys):
        want = o.permute(host[0][p], gal[0])
        for t in range(1, n_terms):
            want = o.add(want, o.permute(host[t][p], gal[t]), g)
        if with_add:
            want = o.add(want, add_h[p], g)
        assert np.array_equal(e.to_host(out[p]), want), ("permute", p)


def test_nary_argument_checks(engine40, pkg):
    e = engine40
    g = e.level_limbs(2)
    a = e.empty(len(g), e.n)
    b = e.empty(len(g), e.n)
    with pytest.raises(pkg.CfheError):
        e.nary_("sum", [a], [[b]] * 9, g)           # more than eight terms
    with pytest.raises(pkg.CfheError):
        e.nary_("sum", [a] * 4, [[b] * 4], g)       # more than three polynomials
    with pytest.raises(pkg.CfheError):
        e.nary_("permute", [a], [[a]], g, galois=[5])   # in place
    with pytest.raises(pkg.CfheError):
        e.nary_("permute", [a], [[b]], g, galois=[4])   # even Galois element


@pytest.mark.parametrize("n_terms,accumulate", [(1, False), (3, True), (16, False), (16, True)])
def test_tensor_accum(engine40, oracle40, n_terms, accumulate):
    """cfhe_tensor_accum against the golden model's Tensor and Add applied term by term."""
    e, o = engine40, oracle40
    rng = np.random.default_rng(1300 + n_terms)
    g = e.level_limbs(12)
    ops = [[rand_limbs(rng, o.primes, g, o.n) for _ in range(4)] for _ in range(n_terms)]
    for l, gi in enumerate(g):  # extreme residues: the 64-bit accumulators see their largest sums
        q = int(o.primes[gi])
        for t in range(n_terms):
            for x in ops[t]:
                x[l, :2] = [q - 1, q - 1]
            ops[t][0][l, 2:4] = [0, 1]
    dev = [[e.to_dev(x) for x in term] for term in ops]
    start = [rand_limbs(rng, o.primes, g, o.n) for _ in range(3)]
    out = [e.to_dev(x) for x in start]
    e.tensor_accum_(out[0], out[1], out[2], [t[0] for t in dev], [t[1] for t in dev], [t[2] for t in dev],
                    [t[3] for t in dev], g, accumulate=accumulate)
    want = [x.copy() for x in start] if accumulate else None
    for t in range(n_terms):
        d = o.tensor(ops[t][0], ops[t][1], ops[t][2], ops[t][3], g)
        want = list(d) if want is None else [o.add(w, x, g) for w, x in zip(want, d)]
    for p in range(3):
        assert np.array_equal(e.to_host(out[p]), want[p]), p


@pytest.mark.parametrize("n_baby,n_giant", [(1, 1), (5, 3), (16, 4)])
def test_giantstep_paccum(engine40, oracle40, n_baby, n_giant):
    """cfhe_giantstep_paccum (the reference's GSFusedKernel, src/extension/Hoist.cu:80-118)
    against products and sums of the golden model; some plaintexts absent."""
    e, o = engine40, oracle40
    t = e.torch
    rng = np.random.default_rng(1400 + n_baby)
    g = e.level_limbs(16, 12)
    rot_h = np.stack([np.stack([rand_limbs(rng, o.primes, g, o.n) for _ in range(2)]) for _ in range(n_baby)])
    for l, gi in enumerate(g):
        rot_h[:, :, l, :2] = int(o.primes[gi]) - 1
    pts_h = [[None if (i + j) % 4 == 3 else rand_limbs(rng, o.primes, g, o.n) for i in range(n_baby)]
             for j in range(n_giant)]
    for l, gi in enumerate(g):
        for row in pts_h:
            if row[0] is not None:
                row[0][l, :2] = int(o.primes[gi]) - 1
    rot = e.to_dev(rot_h.reshape(-1, o.n)).reshape(n_baby, 2, len(g), o.n)
    pts = [[None if p is None else e.to_dev(p) for p in row] for row in pts_h]
    acc = t.empty((n_giant, 2, len(g), o.n), dtype=t.int32, device=rot.device)
    e.giantstep_paccum_(acc, rot, pts, g)
    got = e.to_host(acc.reshape(-1, o.n)).reshape(n_giant, 2, len(g), o.n)
    for j in range(n_giant):
        for part in range(2):
            want = np.zeros((len(g), o.n), dtype=np.uint32)
            for i in range(n_baby):
                if pts_h[j][i] is not None:
                    want = o.add(want, o.mul(rot_h[i, part], pts_h[j][i], g), g)
            assert np.array_equal(got[j, part], want), (j, part)
