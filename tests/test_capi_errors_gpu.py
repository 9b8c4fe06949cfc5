"""Error behaviour of the C ABI: bad arguments come back as a negative status
with a message from cfhe_last_error(), never as a crash or a CUDA fault, and
the context stays usable. (The reference prints and exits on the same
conditions, include/common/Assert.h:9-21; the C++ mirror maps the status to
that behaviour.) Only argument checks that fail before any launch are used."""
import ctypes as C

import numpy as np
import pytest

from test_pipeline_gpu import rand_limbs

pytestmark = pytest.mark.gpu


def test_bad_arguments_are_refused_and_the_context_survives(pkg, engine40, oracle40):
    e, o = engine40, oracle40
    Err = pkg.CfheError
    g = list(e.level_limbs(5))
    a = e.to_dev(rand_limbs(np.random.default_rng(1), o.primes, g, o.n))
    d = e.torch.empty_like(a)
    with pytest.raises(Err, match="unknown"):
        e.binary_(9, d, a, a, g)
    with pytest.raises(Err, match="out of range"):
        e.binary_(0, d, a, a, [0, 1, 99])
    with pytest.raises(Err, match="null"):
        e.binary_(0, d, a, None, g)
    with pytest.raises(Err):
        e.modup_(99, d, a)  # no such level
    with pytest.raises(Err):
        e.moddown_(0, 1, d, a)  # level 0 cannot be rescaled
    with pytest.raises(Err, match="too many|unsupported"):
        e._check(e.L.cfhe_bconv(e.h, e._p(d), e._p(a), (C.c_int * 30)(*range(30)), 30,
                                (C.c_int * 2)(0, 1), 2))
    with pytest.raises(Err, match="one or two"):
        e.modup_to_max_(d, a, [0, 1, 2], g)
    # linear transform: first baby step must be the identity, at most 16 steps
    out_b, out_a = e.empty(len(e.level_limbs(4)), e.n), e.empty(len(e.level_limbs(4)), e.n)
    with pytest.raises(Err, match="identity"):
        e.linear_transform_(5, out_b, out_a, a, a, [1], [None], [0], [None], [[None]], 43)
    with pytest.raises(Err, match="16"):
        e.linear_transform_(5, out_b, out_a, a, a, [0] + list(range(1, 17)), [None] * 17, [0], [None],
                            [[None] * 17], 43)
    with pytest.raises(Err, match="not returned"):
        e._check(e.L.cfhe_free(e.h, C.c_void_p(a.data_ptr())))  # not this allocator's pointer
    # the context still works
    assert np.array_equal(e.to_host(a), e.intt(e.ntt(e.to_host(a), g), g, mont_keep=True))


def test_allocator_reuses_blocks(engine40):
    e = engine40
    p1, p2 = C.c_void_p(), C.c_void_p()
    e._check(e.L.cfhe_malloc(e.h, C.byref(p1), C.c_size_t(3 << 20)))
    e._check(e.L.cfhe_free(e.h, p1))
    e._check(e.L.cfhe_malloc(e.h, C.byref(p2), C.c_size_t(3 << 20)))
    assert p1.value == p2.value  # the freed block is handed out again, no cudaMalloc
    e._check(e.L.cfhe_free(e.h, p2))
    e._check(e.L.cfhe_free(e.h, None))  # freeing NULL is a no-op


def test_allocator_merges_free_neighbours(engine40):
    """Three blocks carved side by side out of one slab, freed in the order
    first, last, middle, come back as one range: a request of their total size
    gets the first block's address, and the words written through it survive."""
    e = engine40
    sizes = [3 << 20, 5 << 20, (1 << 20) + 1]
    ptrs = [C.c_void_p() for _ in sizes]
    for p, s in zip(ptrs, sizes):
        e._check(e.L.cfhe_malloc(e.h, C.byref(p), C.c_size_t(s)))
    rounded = [(s + (256 << 10) - 1) // (256 << 10) * (256 << 10) for s in sizes]
    if ptrs[1].value != ptrs[0].value + rounded[0] or ptrs[2].value != ptrs[1].value + rounded[1]:
        for p in ptrs:
            e._check(e.L.cfhe_free(e.h, p))
        pytest.skip("the three blocks did not come out of one free range")
    for i in (0, 2, 1):
        e._check(e.L.cfhe_free(e.h, ptrs[i]))
    big = C.c_void_p()
    e._check(e.L.cfhe_malloc(e.h, C.byref(big), C.c_size_t(sum(rounded))))
    assert big.value == ptrs[0].value
    words = sum(rounded) // 4
    host = np.arange(words, dtype=np.uint32)
    back = np.empty_like(host)
    e._check(e.L.cfhe_copy_h2d(e.h, big, host.ctypes.data_as(C.c_void_p), C.c_size_t(host.nbytes)))
    e._check(e.L.cfhe_copy_d2h(e.h, back.ctypes.data_as(C.c_void_p), big, C.c_size_t(host.nbytes)))
    e.synchronize()
    assert np.array_equal(host, back)
    e._check(e.L.cfhe_free(e.h, big))
    with pytest.raises(Exception, match="not returned"):
        e._check(e.L.cfhe_free(e.h, big))  # double free is refused
