"""The allocation-free ModDown entry point against the regular one.

Some hosts cannot let a library allocate device memory (the application owns
every byte through its own allocator, or a loop cannot tolerate the
synchronisation an allocation brings), so cfhe_moddown_noalloc keeps its
intermediate in an array that is part of the library image. This file checks,
through the C ABI, that it returns exactly the words of cfhe_moddown, twice in
a row with different inputs and conversion types, so that stale contents of
the shared array from the first call would show up in the second. The file
name sorts last: a run that stops at the first failure has already executed
every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rand_limbs(rng, primes, gidx, n):
    return np.stack([rng.integers(0, int(primes[g]), n, dtype=np.uint64).astype(np.uint32) for g in gidx])


def test_noalloc_moddown_equals_regular_twice(engine40, oracle40):
    e = engine40
    rng = np.random.default_rng(777)
    # back-to-back calls with different data: ModDownAndRescale 28 -> 27 (14 limbs
    # dropped), plain ModDown at level 17 (12 dropped), ModDownAndRescale 2 -> 1
    # (16 dropped, the most the built-in array holds, and 2 limbs restored)
    for level, kind in ((28, 2), (17, 0), (2, 2)):
        full = e.level_limbs(level, 12)
        src = e.to_dev(rand_limbs(rng, oracle40.primes, full, e.n))
        nd = len(e.level_limbs(level if kind == 0 else level - 1))
        want = e.empty(nd, e.n)
        got = e.empty(nd, e.n)
        got.fill_(-1)
        e.moddown_(level, kind, want, src)
        e.moddown_noalloc_(level, kind, got, src)
        e.synchronize()
        assert e.torch.equal(got, want), (level, kind)


def test_noalloc_moddown_on_a_fresh_context_allocates_nothing(pkg, params40, oracle40):
    """A context that has run no other operator (its workspace arena is still
    empty) converts through the allocation-free entry point and returns the
    golden model's words; a second call leaves the amount of free device
    memory exactly where the first left it."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    e = pkg.Engine(params40, device=0)
    rng = np.random.default_rng(778)
    level, kind = 16, 2
    full = e.level_limbs(level, 12)
    host = rand_limbs(rng, oracle40.primes, full, e.n)
    src = e.to_dev(host)
    got = e.empty(len(e.level_limbs(level - 1)), e.n)
    got.fill_(-1)
    e.moddown_noalloc_(level, kind, got, src)   # first call on this context: nothing else has run
    e.synchronize()
    assert np.array_equal(e.to_host(got), oracle40.moddown(level, kind, host))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    got.fill_(-1)
    e.moddown_noalloc_(level, kind, got, src)
    e.synchronize()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert np.array_equal(e.to_host(got), oracle40.moddown(level, kind, host))
    e.close()


def test_noalloc_moddown_rejects_bad_requests(engine40, pkg):
    e = engine40
    a = e.empty(2, e.n)
    with pytest.raises(pkg.CfheError):
        e.moddown_noalloc_(0, 2, a, a)  # level 0 has no rescale
    with pytest.raises(pkg.CfheError):
        e.moddown_noalloc_(28, 7, a, a)  # unknown type


def test_noalloc_moddown_refuses_more_than_16_dropped_limbs(pkg):
    """bootparam_35 level 3 -> 2 drops 5 terminal + 12 auxiliary limbs."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    e = pkg.Engine(pkg.load_params("bootparam_35.json"), device=0)
    src = e.empty(len(e.level_limbs(3, 12)), e.n)
    dst = e.empty(len(e.level_limbs(2)), e.n)
    src.zero_()
    with pytest.raises(pkg.CfheError, match="16"):
        e.moddown_noalloc_(3, 2, dst, src)
    e.close()
