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
