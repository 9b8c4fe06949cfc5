"""Word-level GPU parity on bootparam_30 and bootparam_35, every level.

The level tables of these two sets take terminal <-> main prime transitions
that bootparam_40 never does (bootparam_35 drops one terminal prime per level
near the top and trades five terminal primes for three main ones lower down;
bootparam_30 has no terminal primes at all), so ModUp, ModDown, Rescale and
ModDownAndRescale are compared with the CPU golden model word for word on
every level of both sets, and HMult / key switching on a few levels each.
Everything goes through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SETS = ["bootparam_30.json", "bootparam_35.json"]
_cache = {}


def _pair(pkg, name):
    """(engine, oracle) of a parameter set, created once per session."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if name not in _cache:
        from oracle import Oracle
        p = pkg.load_params(name)
        _cache[name] = (pkg.Engine(p, device=0), Oracle(p), p)
    return _cache[name]


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


def _levels(name):
    import json
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "cheddar-fhe_b200", "parameters", name)) as f:
        return len(json.load(f)["level_config"])


CASES = [(name, level) for name in SETS for level in range(_levels(name))]


@pytest.mark.parametrize("name,level", CASES)
def test_modup_every_level(pkg, name, level):
    e, o, _ = _pair(pkg, name)
    rng = np.random.default_rng(7000 + level)
    g = e.level_limbs(level)
    assert list(g) == list(o.level_limbs(level))
    src = rand_limbs(rng, o.primes, g, o.n)
    assert e.beta(level) == o.beta(level)
    assert np.array_equal(e.modup(level, src), o.modup(level, src))


@pytest.mark.parametrize("name,level", CASES)
def test_moddown_family_every_level(pkg, name, level):
    """ModDown on every level; Rescale and ModDownAndRescale on every level that
    can be rescaled (the engine and the golden model must agree on which)."""
    e, o, p = _pair(pkg, name)
    rng = np.random.default_rng(8000 + level)
    alpha = len(p["auxiliary_primes"])
    full = e.level_limbs(level, alpha)
    nq = len(full) - alpha
    src = np.stack([rand_limbs(rng, o.primes, full, o.n) for _ in range(2)])
    got = e.moddown(level, 0, src)
    for i in range(2):
        assert np.array_equal(got[i], o.moddown(level, 0, src[i]))
    if level == 0:
        with pytest.raises(pkg.CfheError):
            e.moddown(level, 2, src)
        return
    got = e.moddown(level, 2, src)
    for i in range(2):
        assert np.array_equal(got[i], o.moddown(level, 2, src[i]))
    q_only = np.ascontiguousarray(src[0, :nq])
    assert np.array_equal(e.moddown(level, 1, q_only), o.moddown(level, 1, q_only))


def fake_key(rng, e, o, p, key_main, beta):
    T = len(p["terminal_primes"])
    L = T + len(p["main_primes"])
    g = list(range(0, T + key_main)) + [L + a for a in range(len(p["auxiliary_primes"]))]
    kb = [rand_limbs(rng, o.primes, g, o.n) for _ in range(beta)]
    ka = [rand_limbs(rng, o.primes, g, o.n) for _ in range(beta)]
    return kb, ka


def _hmult_levels(name):
    n = _levels(name)
    # the top level, the middle level, level 4 (inside the range where levels
    # trade terminal for main primes) and level 1 (the last that can be rescaled)
    return sorted({n - 1, n // 2, 4, 1})


@pytest.mark.parametrize("name,level", [(s, l) for s in SETS for l in _hmult_levels(s)])
def test_hmult_and_keyswitch(pkg, name, level):
    e, o, p = _pair(pkg, name)
    rng = np.random.default_rng(9000 + level)
    g = e.level_limbs(level)
    key_main = len(p["main_primes"])
    top = len(p["level_config"]) - 1
    kb, ka = fake_key(rng, e, o, p, key_main, e.beta(top))
    ins = [rand_limbs(rng, o.primes, g, o.n) for _ in range(4)]
    got = e.hmult(level, *ins, kb, ka, key_main, True)
    exp = o.hmult(level, *ins, kb, ka, key_main, True)
    assert np.array_equal(got[0], exp[0]) and np.array_equal(got[1], exp[1])
    got = e.keyswitch(level, ins[0], ins[1], kb, ka, key_main)
    exp = o.keyswitch(level, ins[0], ins[1], kb, ka, key_main)
    assert np.array_equal(got[0], exp[0]) and np.array_equal(got[1], exp[1])
