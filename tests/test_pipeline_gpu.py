"""GPU parity of the element-wise operators, base conversion, ModUp, the
ModDown family, the evaluation-key inner product, key switching and HMult
against the CPU golden model, through the C ABI. Every word must match."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


def test_elementwise_matches_oracle(engine40, oracle40):
    e, o = engine40, oracle40
    rng = np.random.default_rng(21)
    g = e.level_limbs(28, 12)
    a, b = rand_limbs(rng, o.primes, g, o.n), rand_limbs(rng, o.primes, g, o.n)
    for l, gi in enumerate(g):  # edge values
        q = int(o.primes[gi])
        a[l, :4] = [0, q - 1, q - 1, 1]
        b[l, :4] = [0, q - 1, 1, q - 1]
    assert np.array_equal(e.add(a, b, g), o.add(a, b, g))
    assert np.array_equal(e.sub(a, b, g), o.sub(a, b, g))
    assert np.array_equal(e.neg(a, g), o.neg(a, g))
    assert np.array_equal(e.mul(a, b, g), o.mul(a, b, g))
    k = np.array([rng.integers(0, int(o.primes[gi])) for gi in g], dtype=np.uint32)
    for op in range(4):
        assert np.array_equal(e.const_op(a, k, g, op), o.const_op(a, k, g, op)), op
    assert np.array_equal(e.const_op(a, k, g, 4, b=b), o.add(o.const_op(a, k, g, 3), b, g))
    assert np.array_equal(e.mul_imag_unit(a, g), o.mul_imag_unit(a, g))


def test_elementwise_multi_equals_single_calls(engine40, oracle40):
    """Two and three polynomials in one launch give the words of one launch per
    polynomial, for every binary and constant operator."""
    e, o = engine40, oracle40
    rng = np.random.default_rng(23)
    g = e.level_limbs(20)
    polys = [[e.to_dev(rand_limbs(rng, o.primes, g, o.n)) for _ in range(3)] for _ in range(2)]
    k = np.array([rng.integers(0, int(o.primes[gi])) for gi in g], dtype=np.uint32)
    t = e.torch
    for n in (2, 3):
        a, b = polys[0][:n], polys[1][:n]
        for op in range(4):
            multi = [t.empty_like(x) for x in a]
            e.elementwise_multi_(0, op, multi, a, b if op != 2 else None, None, g)
            for i in range(n):
                single = t.empty_like(a[i])
                e.binary_(op, single, a[i], b[i] if op != 2 else None, g)
                assert t.equal(multi[i], single), (n, op, i)
        for op in range(5):
            multi = [t.empty_like(x) for x in a]
            e.elementwise_multi_(1, op, multi, a, b if op == 4 else None, k, g)
            for i in range(n):
                single = t.empty_like(a[i])
                e.const_op_(op, single, a[i], b[i] if op == 4 else None, k, g)
                assert t.equal(multi[i], single), (n, op, i)


def test_tensor_matches_oracle(engine40, oracle40):
    e, o = engine40, oracle40
    rng = np.random.default_rng(22)
    g = e.level_limbs(28)
    ins = [rand_limbs(rng, o.primes, g, o.n) for _ in range(4)]
    for x in ins:
        for l, gi in enumerate(g):
            x[l, 0] = int(o.primes[gi]) - 1
    for got, exp in zip(e.tensor(*ins, g), o.tensor(*ins, g)):
        assert np.array_equal(got, exp)


def test_permute_matches_oracle(engine40, oracle40):
    e, o = engine40, oracle40
    rng = np.random.default_rng(23)
    g = e.level_limbs(16)
    a, b = rand_limbs(rng, o.primes, g, o.n), rand_limbs(rng, o.primes, g, o.n)
    for rot in (1, 1234, 32767, -1):
        gal = o.galois(rot)
        assert gal == e.galois(rot)
        assert np.array_equal(e.permute(a, gal, g), o.permute(a, gal))
    gal = o.galois(5)
    assert np.array_equal(e.permute(a, gal, g, add=b), o.add(o.permute(a, gal), b, g))


def test_two_contexts_ordered_across_streams(engine40, params40, pkg):
    """A second context on its own stream consumes what the first produced and
    hands its result back, with cfhe_order_after in both directions and no host
    synchronisation in between; the words equal the single-context result."""
    e = engine40
    side = pkg.Engine(params40, device=0)
    rng = np.random.default_rng(31)
    level = 20
    g = e.level_limbs(level)
    nq, n = len(g), e.n
    primes = np.array([e.primes[x] for x in g], dtype=np.uint64)
    a = e.to_dev((rng.integers(0, 1 << 62, (nq, n), dtype=np.uint64) % primes[:, None]).astype(np.uint32))
    b = e.to_dev((rng.integers(0, 1 << 62, (nq, n), dtype=np.uint64) % primes[:, None]).astype(np.uint32))
    t = e.torch
    ref1, ref2, ref3 = t.empty_like(a), t.empty_like(a), t.empty_like(a)
    e.binary_(3, ref1, a, b, g)       # product on the main context
    e.binary_(0, ref2, ref1, a, g)    # the step the side context takes below
    e.binary_(1, ref3, ref2, b, g)    # back on the main context
    e.synchronize()
    for _ in range(20):               # many rounds: an ordering bug shows as a stale read
        x1, x2, x3 = t.zeros_like(a), t.zeros_like(a), t.zeros_like(a)
        e.synchronize()
        e.binary_(3, x1, a, b, g)
        side.order_after(e)
        side.binary_(0, x2, x1, a, g)
        e.order_after(side)
        e.binary_(1, x3, x2, b, g)
        e.synchronize()
        assert t.equal(x3, ref3)


def test_bconv_matches_oracle(engine40, oracle40):
    e, o = engine40, oracle40
    rng = np.random.default_rng(24)
    full = list(e.level_limbs(28, 12))
    for src in (full[12:24], full[0:12], full[36:47], full[47:59] + full[45:47], full[0:2], [full[5]]):
        dst = [x for x in full if x not in src]
        y = np.stack([rng.integers(-(int(o.primes[g]) // 2), int(o.primes[g]) // 2 + 1, o.n) for g in src]).astype(np.int32)
        for k, g in enumerate(src):  # extreme centred values
            h = int(o.primes[g]) // 2
            y[k, :2] = [h, -h]
        assert np.array_equal(e.bconv(y, src, dst), o.bconv(y, src, dst)), len(src)


@pytest.mark.parametrize("level", [28, 27, 26, 17, 16, 13, 9, 8, 2, 1, 0])
def test_modup_matches_oracle(engine40, oracle40, level):
    e, o = engine40, oracle40
    rng = np.random.default_rng(100 + level)
    g = e.level_limbs(level)
    src = rand_limbs(rng, o.primes, g, o.n)
    assert e.beta(level) == o.beta(level)
    assert np.array_equal(e.modup(level, src), o.modup(level, src))


@pytest.mark.parametrize("level", [28, 27, 26, 17, 16, 15, 14, 13, 12, 3, 2, 1])
def test_moddown_family_matches_oracle(engine40, oracle40, level):
    e, o = engine40, oracle40
    rng = np.random.default_rng(200 + level)
    full = e.level_limbs(level, 12)
    src = np.stack([rand_limbs(rng, o.primes, full, o.n) for _ in range(2)])
    nq = len(full) - 12
    got = e.moddown(level, 0, src)
    for p in range(2):
        assert np.array_equal(got[p], o.moddown(level, 0, src[p]))
    got = e.moddown(level, 2, src)
    for p in range(2):
        assert np.array_equal(got[p], o.moddown(level, 2, src[p]))
    q_only = np.ascontiguousarray(src[0, :nq])
    assert np.array_equal(e.moddown(level, 1, q_only), o.moddown(level, 1, q_only))


@pytest.mark.parametrize("level", [28, 16, 3])
def test_moddown_stage_entries_compose_to_moddown(engine40, oracle40, level):
    """cfhe_intt_for_moddown, cfhe_bconv_for_moddown and cfhe_ntt_for_moddown run
    in that order leave the words of the golden model's ModDown, Rescale and
    ModDownAndRescale (two polynomials at once)."""
    e, o = engine40, oracle40
    t = e.torch
    rng = np.random.default_rng(260 + level)
    full = e.level_limbs(level, 12)
    nq = len(full) - 12
    src = np.stack([rand_limbs(rng, o.primes, full, o.n) for _ in range(2)])
    for kind in (0, 2, 1):
        host = src if kind != 1 else np.ascontiguousarray(src[:, :nq])
        s = e.to_dev(host.reshape(-1, o.n)).reshape(host.shape)
        nd = len(e.level_limbs(level if kind == 0 else level - 1))
        d = t.empty((2, nd, o.n), dtype=t.int32, device=s.device)
        e.moddown_staged_(level, kind, d, s)
        got = e.to_host(d.reshape(-1, o.n)).reshape(2, nd, o.n)
        for p in range(2):
            assert np.array_equal(got[p], o.moddown(level, kind, host[p])), (kind, p)


def fake_key(rng, e, o, key_main, beta):
    T = len(e.p["terminal_primes"])
    L = T + len(e.p["main_primes"])
    g = list(range(0, T + key_main)) + [L + a for a in range(e.alpha)]
    kb = [rand_limbs(rng, o.primes, g, o.n) for _ in range(beta)]
    ka = [rand_limbs(rng, o.primes, g, o.n) for _ in range(beta)]
    return kb, ka


@pytest.mark.parametrize("level,key_main", [(28, 43), (16, 43), (16, 23), (5, 43)])
def test_inner_product_matches_oracle(engine40, oracle40, level, key_main):
    e, o = engine40, oracle40
    rng = np.random.default_rng(300 + level)
    full = e.level_limbs(level, 12)
    beta = e.beta(level)
    kb, ka = fake_key(rng, e, o, key_main, beta)
    mu = np.stack([rand_limbs(rng, o.primes, full, o.n) for _ in range(beta)])
    ab, aa = e.evk_inner(level, mu, kb, ka, key_main)
    rb, ra = o.evk_inner(level, mu, kb, ka, key_main)
    assert np.array_equal(ab, rb) and np.array_equal(aa, ra)


@pytest.mark.parametrize("level,rescale", [(28, True), (28, False), (16, True), (8, True), (2, True), (1, True)])
def test_hmult_matches_oracle(engine40, oracle40, level, rescale):
    """Config 2 path: tensor, ModUp, inner product with the key, P*(d0,d1),
    ModDown(AndRescale). Random words stand in for ciphertexts and keys:
    limb-level parity does not depend on them being valid encryptions."""
    e, o = engine40, oracle40
    rng = np.random.default_rng(400 + level)
    g = e.level_limbs(level)
    ins = [rand_limbs(rng, o.primes, g, o.n) for _ in range(4)]
    kb, ka = fake_key(rng, e, o, 43, e.beta(28))
    got = e.hmult(level, *ins, kb, ka, 43, rescale)
    exp = o.hmult(level, *ins, kb, ka, 43, rescale)
    assert np.array_equal(got[0], exp[0]) and np.array_equal(got[1], exp[1])


def test_keyswitch_matches_oracle(engine40, oracle40):
    e, o = engine40, oracle40
    rng = np.random.default_rng(500)
    level = 20
    g = e.level_limbs(level)
    d, bx = rand_limbs(rng, o.primes, g, o.n), rand_limbs(rng, o.primes, g, o.n)
    kb, ka = fake_key(rng, e, o, 43, e.beta(28))
    got = e.keyswitch(level, d, bx, kb, ka, 43)
    exp = o.keyswitch(level, d, bx, kb, ka, 43)
    assert np.array_equal(got[0], exp[0]) and np.array_equal(got[1], exp[1])


def test_errors_are_reported(engine40, pkg):
    e = engine40
    a = e.empty(2, e.n)
    with pytest.raises(pkg.CfheError):
        e.moddown_(0, 2, a, a)  # level 0 cannot be rescaled
    with pytest.raises(pkg.CfheError):
        e.modup_(99, a, a)


@pytest.fixture(scope="module")
def engine40_simt(pkg, params40):
    """A second context whose base conversions run on the SIMT kernel instead
    of the tensor cores (CFHE_BCONV=simt is read at context creation)."""
    import os
    os.environ["CFHE_BCONV"] = "simt"
    try:
        e = pkg.Engine(params40, device=0)
    finally:
        del os.environ["CFHE_BCONV"]
    yield e
    e.close()


@pytest.mark.parametrize("level", [28, 16, 2, 1])
def test_simt_and_tensor_core_conversions_agree(engine40, engine40_simt, oracle40, level):
    rng = np.random.default_rng(900 + level)
    full = engine40.level_limbs(level, 12)
    nq = len(full) - 12
    src = rand_limbs(rng, oracle40.primes, full, oracle40.n)
    q_only = np.ascontiguousarray(src[:nq])
    want = oracle40.modup(level, q_only)
    assert np.array_equal(engine40.modup(level, q_only), want)
    assert np.array_equal(engine40_simt.modup(level, q_only), want)
    for kind in (0, 2):
        want = oracle40.moddown(level, kind, src)
        assert np.array_equal(engine40.moddown(level, kind, src), want)
        assert np.array_equal(engine40_simt.moddown(level, kind, src), want)


def test_extreme_residues_through_the_tensor_core_conversion(engine40, oracle40):
    """Residues 0, 1, (q-1)/2, (q+1)/2 and q-1 in every limb: the boundary of
    the centred representation and the largest byte planes."""
    level = 28
    g = engine40.level_limbs(level)
    src = np.zeros((len(g), oracle40.n), np.uint32)
    for l, gi in enumerate(g):
        q = int(oracle40.primes[gi])
        vals = np.array([0, 1, (q - 1) // 2, (q + 1) // 2, q - 1, q - 2, 255, 256, 65535, 65536], dtype=np.uint32)
        src[l] = np.resize(np.roll(vals, l), oracle40.n)
    # feed the values as NTT-domain words: ModUp first inverts the transform,
    # so also run the conversion on the transform of these coefficient patterns
    assert np.array_equal(engine40.modup(level, src), oracle40.modup(level, src))
    coef = oracle40.ntt(src, g)
    assert np.array_equal(engine40.modup(level, coef), oracle40.modup(level, coef))


@pytest.mark.parametrize("level,rots", [(16, [1, 1234, 32767, -1, 5, 64]), (28, [7, 4096])])
def test_hoisted_rotations_equal_hrot(engine40, oracle40, level, rots):
    """Every output of the hoisted path equals MultKey + Permute (the
    reference's HRot, src/core/Context.cpp:776-791) with the same key."""
    e, o = engine40, oracle40
    rng = np.random.default_rng(1000 + level)
    g = e.level_limbs(level)
    bx, ax = rand_limbs(rng, o.primes, g, o.n), rand_limbs(rng, o.primes, g, o.n)
    keys = [fake_key(rng, e, o, 43, e.beta(28)) for _ in rots]
    dk = [([e.to_dev(x) for x in kb], [e.to_dev(x) for x in ka]) for kb, ka in keys]
    out = e.empty(len(rots), 2, len(g), e.n)
    beta = e.beta(level)
    e.hoisted_rotations_(level, out, e.to_dev(bx), e.to_dev(ax), rots,
                         [k[0][:beta] for k in dk], [k[1][:beta] for k in dk], 43)
    got = e.to_host(out)
    for i, r in enumerate(rots):
        kb, ka = keys[i]
        sb, sa = o.keyswitch(level, ax, bx, kb, ka, 43)
        gal = o.galois(r)
        assert np.array_equal(got[i, 0], o.permute(sb, gal)), r
        assert np.array_equal(got[i, 1], o.permute(sa, gal)), r


def _extra_ntt_primes(existing, count, n=1 << 16):
    """`count` primes below 2^31, = 1 mod 2n, not in `existing` (deterministic Miller-Rabin)."""
    def is_prime(p):
        d, s = p - 1, 0
        while d % 2 == 0:
            d //= 2
            s += 1
        for a in (2, 3, 5, 7, 11, 13, 17):
            x = pow(a, d, p)
            if x in (1, p - 1):
                continue
            for _ in range(s - 1):
                x = x * x % p
                if x == p - 1:
                    break
            else:
                return False
        return True
    out, p = [], (1 << 31) - (1 << 31) % (2 * n) + 1 - 2 * n * 300
    while len(out) < count:
        if p not in existing and is_prime(p):
            out.append(p)
        p -= 2 * n
    return out


def test_modup_moddown_with_sixteen_auxiliary_primes(pkg, params40):
    """A parameter set with 16 auxiliary primes makes digits of 16 limbs, which
    take the widest operand rows of the tensor-core base conversion (more than
    15 source limbs); ModUp and the ModDown family still equal the golden model."""
    import copy
    import torch
    from oracle import Oracle
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    p = copy.deepcopy(params40)
    used = set(p["main_primes"]) | set(p["terminal_primes"]) | set(p["auxiliary_primes"])
    p["auxiliary_primes"] = list(p["auxiliary_primes"]) + _extra_ntt_primes(used, 4)
    e, o = pkg.Engine(p, device=0), Oracle(p)
    rng = np.random.default_rng(77)
    for level in (28, 20):
        g = e.level_limbs(level)
        src = rand_limbs(rng, o.primes, g, o.n)
        assert e.beta(level) == o.beta(level)
        assert np.array_equal(e.modup(level, src), o.modup(level, src)), level
        full = e.level_limbs(level, 16)
        acc = np.stack([rand_limbs(rng, o.primes, full, o.n) for _ in range(2)])
        for kind in (0, 2):
            got = e.moddown(level, kind, acc)
            for i in range(2):
                assert np.array_equal(got[i], o.moddown(level, kind, acc[i])), (level, kind)


def test_limb_sharded_hmult_on_one_rank_equals_hmult(engine40, params40):
    """The limb-sharded HMult (cheddar-fhe_b200/sharded.py) run with a single
    rank, i.e. the same per-limb algebra without the all-gathers, returns the
    words of cfhe_hmult without rescaling. (With more ranks the exchanged limbs
    are the same tensors, moved by NCCL; bench.py --shard limbs checks that on
    the GPUs it runs on.)"""
    import importlib.util
    import os
    e = engine40
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("cfhe_sharded", os.path.join(root, "cheddar-fhe_b200", "sharded.py"))
    sh = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sh)
    for level in (28, 9):
        plan = sh.LimbShardPlan(params40, level, 1)
        rng = np.random.default_rng(7700 + level)
        g = list(e.level_limbs(level))
        T, M = len(params40["terminal_primes"]), len(params40["main_primes"])
        kg = list(range(T + M)) + [T + M + a for a in range(e.alpha)]
        ins = [rand_limbs(rng, e.primes, g, e.n) for _ in range(4)]
        kb = [rand_limbs(rng, e.primes, kg, e.n) for _ in range(e.beta(28))]
        ka = [rand_limbs(rng, e.primes, kg, e.n) for _ in range(e.beta(28))]
        rows = [kg.index(x) for x in plan.full_g]
        active = [d[0] for d in plan.digits]
        got_b, got_a, _ = sh.sharded_hmult(e, plan, 0, None, *[e.to_dev(x) for x in ins],
                                           [e.to_dev(kb[i][rows]) for i in active],
                                           [e.to_dev(ka[i][rows]) for i in active])
        want_b, want_a = e.hmult(level, *ins, kb, ka, M, False)
        assert np.array_equal(e.to_host(got_b), want_b) and np.array_equal(e.to_host(got_a), want_a), level
