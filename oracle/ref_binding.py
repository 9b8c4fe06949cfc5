"""ctypes binding of oracle/_ref/libcheddar_ref.so: the UNMODIFIED reference
library built by `make -C oracle ref` (test infrastructure; GPU only)."""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(_HERE, "_ref", "libcheddar_ref.so")


def available():
    return os.path.exists(REF_LIB)


class Reference:
    """The reference's Context on the current device; buffers are torch int32
    CUDA tensors holding the same words as the engine's."""

    def __init__(self, p):
        self.L = C.CDLL(REF_LIB)
        self.L.ref_create.restype = C.c_void_p
        u = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
        main, ter, aux = u(p["main_primes"]), u(p["terminal_primes"] or [0]), u(p["auxiliary_primes"])
        lc = np.ascontiguousarray(np.array(p["level_config"], dtype=np.int32).reshape(-1))
        self.p = p
        self.h = C.c_void_p(self.L.ref_create(
            p["log_degree"], C.c_double(float(2 ** p["log_default_scale"])), p["default_encryption_level"],
            main.ctypes.data_as(C.c_void_p), len(p["main_primes"]),
            ter.ctypes.data_as(C.c_void_p), len(p["terminal_primes"]),
            aux.ctypes.data_as(C.c_void_p), len(p["auxiliary_primes"]),
            lc.ctypes.data_as(C.c_void_p), len(p["level_config"])))

    def close(self):
        if self.h:
            self.L.ref_destroy(self.h)
            self.h = None

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def ntt(self, dst, src, num_main, num_ter, num_aux, inverse=False, mont_conv=False):
        rc = self.L.ref_ntt(self.h, self._p(dst), self._p(src), num_main, num_ter, num_aux,
                            int(inverse), int(mont_conv))
        assert rc == 0, rc

    def modup(self, level, dst, src):
        assert self.L.ref_modup(self.h, level, self._p(dst), self._p(src)) == 0

    def moddown(self, level, kind, dst, src):
        assert self.L.ref_moddown(self.h, level, kind, self._p(dst), self._p(src)) == 0

    def hmult(self, level, out_b, out_a, b1, a1, b2, a2, kb, ka, key_main, rescale=True, iters=1):
        beta = len(kb)
        pb = (C.c_void_p * beta)(*[t.data_ptr() for t in kb])
        pa = (C.c_void_p * beta)(*[t.data_ptr() for t in ka])
        usec = C.c_float(0)
        rc = self.L.ref_hmult(self.h, level, self._p(out_b), self._p(out_a), self._p(b1), self._p(a1),
                              self._p(b2), self._p(a2), pb, pa, key_main, beta, int(rescale), iters,
                              C.byref(usec))
        assert rc == 0, rc
        return usec.value

    def rotations_time(self, level, bx, ax, kb, ka, key_main, rots, iters=3):
        """Config 3 on the reference: (microseconds for len(rots) x Context::HRot,
        microseconds for one hoisted HoistHandler::EvaluateBabyStep over the
        same rotations); see ref_rotations_time in ref_driver.cu."""
        beta = len(kb)
        pb = (C.c_void_p * beta)(*[t.data_ptr() for t in kb])
        pa = (C.c_void_p * beta)(*[t.data_ptr() for t in ka])
        r = np.ascontiguousarray(rots, dtype=np.int32)
        usec = (C.c_float * 2)()
        rc = self.L.ref_rotations_time(self.h, level, self._p(bx), self._p(ax), pb, pa, key_main, beta,
                                       len(r), r.ctypes.data_as(C.c_void_p), iters, usec)
        assert rc == 0, rc
        return float(usec[0]), float(usec[1])

    def ntt_batch_time(self, buf_a, buf_b, polys, num_main, num_ter, iters):
        usec = C.c_float(0)
        rc = self.L.ref_ntt_batch_time(self.h, self._p(buf_a), self._p(buf_b), polys, num_main, num_ter,
                                       iters, C.byref(usec))
        assert rc == 0, rc
        return usec.value


def boot(p, iters=3, min_ks=False):
    """Runs the reference's own bootstrapping (BootContext::Boot) on random
    slots and returns its latency and error; see ref_boot in ref_driver.cu."""
    L = C.CDLL(REF_LIB)
    u = lambda a: np.ascontiguousarray(a, dtype=np.uint32)
    main, ter, aux = u(p["main_primes"]), u(p["terminal_primes"] or [0]), u(p["auxiliary_primes"])
    lc = np.ascontiguousarray(np.array(p["level_config"], dtype=np.int32).reshape(-1))
    out = (C.c_double * 6)()
    rc = L.ref_boot(
        p["log_degree"], C.c_double(float(2 ** p["log_default_scale"])), p["default_encryption_level"],
        main.ctypes.data_as(C.c_void_p), len(p["main_primes"]),
        ter.ctypes.data_as(C.c_void_p), len(p["terminal_primes"]),
        aux.ctypes.data_as(C.c_void_p), len(p["auxiliary_primes"]),
        lc.ctypes.data_as(C.c_void_p), len(p["level_config"]),
        int(p.get("dense_hamming_weight", 0)), int(p.get("sparse_hamming_weight", 0)),
        int(p["num_cts_levels"]), int(p["num_stc_levels"]), int(min_ks), iters, out)
    assert rc == 0, rc
    return {"ms": out[0], "max_err": out[1], "mean_err": out[2], "prepare_s": out[3],
            "rotation_keys": int(out[4]), "end_level": int(out[5])}
