"""The engine against the committed digests of the reference's own CUDA
library (tests/golden/reference_digests.json): same seeded inputs, through the
C ABI, every output word must hash to what the reference produced. Unlike
tests/test_reference_gpu.py this needs no reference library at run time."""
import numpy as np
import pytest

from test_oracle_cpu import _golden, _matches

pytestmark = pytest.mark.gpu


def test_engine_ntt_equals_reference_golden(engine40):
    g_mod, cases = _golden()
    e = engine40
    for case in g_mod.NTT_CASES:
        g = g_mod.ntt_limbs(case)
        a = g_mod.rand_limbs(np.random.default_rng(9000 + sum(case)), e.primes, g)
        for mont in (False, True):
            _matches(cases[f"ntt{case}_inv0_mont{int(mont)}"], e.ntt(a, g, mont))
            _matches(cases[f"ntt{case}_inv1_mont{int(mont)}"], e.intt(a, g, mont_keep=not mont))


def test_engine_modswitch_equals_reference_golden(engine40):
    g_mod, cases = _golden()
    e = engine40
    for level in g_mod.MODUP_LEVELS:
        a = g_mod.rand_limbs(np.random.default_rng(9100 + level), e.primes, e.level_limbs(level))
        _matches(cases[f"modup_level{level}"], e.modup(level, a))
    for level in g_mod.MODDOWN_LEVELS:
        full = e.level_limbs(level, 12)
        a = g_mod.rand_limbs(np.random.default_rng(9200 + level), e.primes, full)
        nq = len(full) - 12
        for kind in (0, 1, 2):
            x = a if kind != 1 else np.ascontiguousarray(a[:nq])
            _matches(cases[f"moddown_level{level}_kind{kind}"], e.moddown(level, kind, x))


def test_engine_hmult_equals_reference_golden(engine40):
    g_mod, cases = _golden()
    e = engine40
    kg = list(range(47)) + [47 + a for a in range(12)]
    for level, rescale in g_mod.HMULT_CASES:
        rng = np.random.default_rng(9300 + level)
        g = e.level_limbs(level)
        ins = [g_mod.rand_limbs(rng, e.primes, g) for _ in range(4)]
        beta = e.beta(28)
        kb = [g_mod.rand_limbs(rng, e.primes, kg) for _ in range(beta)]
        ka = [g_mod.rand_limbs(rng, e.primes, kg) for _ in range(beta)]
        b, a = e.hmult(level, *ins, kb, ka, 43, rescale)
        _matches(cases[f"hmult_level{level}_rescale{int(rescale)}"], np.stack([b, a]))
