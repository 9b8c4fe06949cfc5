"""ctypes binding of oracle/liboracle.so (test infrastructure only)."""
import ctypes as C
import json
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build():
    """Compile liboracle.so with gcc (no-op when up to date)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_create.restype = C.c_void_p
        L.orc_create.argtypes = [C.c_int, u32p, C.c_int, u32p, C.c_int, u32p,
                                 C.c_int, i32p, C.c_int, C.c_int, C.c_int]
        L.orc_destroy.argtypes = [C.c_void_p]
        for name in ("orc_degree", "orc_num_primes"):
            getattr(L, name).argtypes = [C.c_void_p]
        L.orc_prime.restype = C.c_uint32
        L.orc_prime.argtypes = [C.c_void_p, C.c_int]
        L.orc_psi.restype = C.c_uint32
        L.orc_psi.argtypes = [C.c_void_p, C.c_int]
        L.orc_qinv.restype = C.c_int32
        L.orc_qinv.argtypes = [C.c_void_p, C.c_int]
        L.orc_level_limbs.argtypes = [C.c_void_p, C.c_int, C.c_int, i32p]
        L.orc_beta.argtypes = [C.c_void_p, C.c_int]
        L.orc_galois_for_rotation.restype = C.c_uint32
        L.orc_galois_for_rotation.argtypes = [C.c_void_p, C.c_int]
        for name in ("orc_mulmod", "orc_to_mont", "orc_mont_mul"):
            f = getattr(L, name)
            f.restype = C.c_uint32
        L.orc_mulmod.argtypes = [C.c_uint32] * 3
        L.orc_mont_mul.argtypes = [C.c_uint32] * 3
        L.orc_to_mont.argtypes = [C.c_uint32] * 2
        L.orc_invmod.restype = C.c_uint32
        L.orc_invmod.argtypes = [C.c_uint32] * 2
        L.orc_powmod.restype = C.c_uint32
        L.orc_powmod.argtypes = [C.c_uint32, C.c_uint64, C.c_uint32]
        L.orc_find_generator.restype = C.c_uint32
        L.orc_find_generator.argtypes = [C.c_uint32]
        _LIB = L
    return _LIB


def load_params(path):
    """Parameter JSON with the keys of the reference's test fixture
    (unittest/Testbed.h:103-210)."""
    with open(path) as f:
        j = json.load(f)
    return {
        "log_degree": j["log_degree"],
        "log_default_scale": j["log_default_scale"],
        "default_encryption_level": j["default_encryption_level"],
        "main_primes": j["main_primes"],
        "terminal_primes": j.get("terminal_primes", []),
        "auxiliary_primes": j["auxiliary_primes"],
        "level_config": j["level_config"],
        "additional_base": j.get("additional_base", [0, 0]),
        "dense_hamming_weight": j.get("dense_hamming_weight"),
        "sparse_hamming_weight": j.get("sparse_hamming_weight"),
    }


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _ptr_array(arrs):
    T = C.c_void_p * len(arrs)
    return T(*[a.ctypes.data for a in arrs])


class Oracle:
    """Golden model context; arrays are numpy uint32, limb-major [limbs, N]."""

    def __init__(self, p):
        L = _lib()
        self.L = L
        self.p = p
        lc = np.ascontiguousarray(np.array(p["level_config"], dtype=np.int32).reshape(-1))
        ter = _u32(p["terminal_primes"]) if p["terminal_primes"] else np.zeros(1, np.uint32)
        self.h = L.orc_create(p["log_degree"], _u32(p["main_primes"]), len(p["main_primes"]),
                              ter, len(p["terminal_primes"]),
                              _u32(p["auxiliary_primes"]), len(p["auxiliary_primes"]),
                              lc, len(p["level_config"]),
                              p["additional_base"][0], p["additional_base"][1])
        self.n = L.orc_degree(self.h)
        self.num_primes = L.orc_num_primes(self.h)
        self.primes = np.array([L.orc_prime(self.h, g) for g in range(self.num_primes)], dtype=np.uint64)
        self.alpha = len(p["auxiliary_primes"])
        self.max_level = len(p["level_config"]) - 1

    def __del__(self):
        try:
            self.L.orc_destroy(self.h)
        except Exception:
            pass

    # ---- metadata
    def level_limbs(self, level, num_aux=0):
        buf = np.zeros(128, np.int32)
        k = self.L.orc_level_limbs(self.h, level, num_aux, buf)
        return buf[:k].copy()

    def beta(self, level):
        return self.L.orc_beta(self.h, level)

    def psi(self, g):
        return self.L.orc_psi(self.h, g)

    def qinv(self, g):
        return self.L.orc_qinv(self.h, g)

    def galois(self, rot):
        return self.L.orc_galois_for_rotation(self.h, rot)

    def _g(self, gidx):
        return np.ascontiguousarray(gidx, dtype=np.int32)

    def _call(self, name, *args):
        f = getattr(self.L, name)
        f.restype = None
        conv = []
        for a in args:
            if isinstance(a, np.ndarray):
                conv.append(C.c_void_p(a.ctypes.data))
            elif a is None:
                conv.append(C.c_void_p(0))
            elif isinstance(a, int):
                conv.append(C.c_int(a))
            else:
                conv.append(a)
        f(C.c_void_p(self.h), *conv)

    # ---- transforms
    def ntt(self, src, gidx, mont_conv=False):
        src = _u32(src)
        g = self._g(gidx)
        dst = np.empty_like(src)
        self._call("orc_ntt", dst, src, g, len(g), int(mont_conv))
        return dst

    def intt(self, src, gidx, consts=None, mont_keep=False, centred=False):
        src = _u32(src)
        g = self._g(gidx)
        dst = np.empty_like(src)
        k = _u32(consts) if consts is not None else None
        self._call("orc_intt", dst, src, g, len(g), k, int(mont_keep), int(centred))
        return dst

    # ---- element-wise
    def _bin(self, name, a, b, gidx):
        a, b, g = _u32(a), _u32(b), self._g(gidx)
        d = np.empty_like(a)
        self._call(name, d, a, b, g, len(g))
        return d

    def add(self, a, b, gidx):
        return self._bin("orc_add", a, b, gidx)

    def sub(self, a, b, gidx):
        return self._bin("orc_sub", a, b, gidx)

    def mul(self, a, b, gidx):
        return self._bin("orc_mul", a, b, gidx)

    def neg(self, a, gidx):
        a, g = _u32(a), self._g(gidx)
        d = np.empty_like(a)
        self._call("orc_neg", d, a, g, len(g))
        return d

    def const_op(self, a, k, gidx, op):
        a, k, g = _u32(a), _u32(k), self._g(gidx)
        d = np.empty_like(a)
        self._call("orc_const_op", d, a, k, g, len(g), int(op))
        return d

    def tensor(self, b1, a1, b2, a2, gidx):
        b1, a1, b2, a2 = map(_u32, (b1, a1, b2, a2))
        g = self._g(gidx)
        d0, d1, d2 = (np.empty_like(b1) for _ in range(3))
        self._call("orc_tensor", d0, d1, d2, b1, a1, b2, a2, g, len(g))
        return d0, d1, d2

    def permute(self, a, galois):
        a = _u32(a)
        d = np.empty_like(a)
        self._call("orc_permute", d, a, C.c_uint32(int(galois)), a.shape[0])
        return d

    def mul_imag_unit(self, a, gidx):
        a, g = _u32(a), self._g(gidx)
        d = np.empty_like(a)
        self._call("orc_mul_imag_unit", d, a, g, len(g))
        return d

    def bconv(self, y, src_gidx, dst_gidx):
        y = np.ascontiguousarray(y, dtype=np.int32)
        sg, dg = self._g(src_gidx), self._g(dst_gidx)
        d = np.empty((len(dg), self.n), np.uint32)
        self._call("orc_bconv", d, y, sg, len(sg), dg, len(dg))
        return d

    # ---- pipelines
    def modup(self, level, src):
        src = _u32(src)
        ntot = len(self.level_limbs(level, self._alpha(level)))
        d = np.zeros((self.beta(level), ntot, self.n), np.uint32)
        self._call("orc_modup", level, d, src)
        return d

    def _alpha(self, level):
        return len(self.level_limbs(-1)) if level == -1 else self.alpha

    def moddown(self, level, kind, src):
        src = _u32(src)
        nd = len(self.level_limbs(level if kind == 0 else level - 1))
        d = np.empty((nd, self.n), np.uint32)
        self._call("orc_moddown", level, int(kind), d, src)
        return d

    def evk_inner(self, level, modup, evk_b, evk_a, key_main):
        modup = _u32(modup)
        evk_b = [_u32(x) for x in evk_b]
        evk_a = [_u32(x) for x in evk_a]
        ntot = modup.shape[1]
        ab = np.empty((ntot, self.n), np.uint32)
        aa = np.empty((ntot, self.n), np.uint32)
        self._call("orc_evk_inner", level, ab, aa, modup, _ptr_array(evk_b), _ptr_array(evk_a), int(key_main))
        return ab, aa

    def add_p_times(self, level, acc, x):
        acc = _u32(acc).copy()
        self._call("orc_add_p_times", level, acc, _u32(x))
        return acc

    def modup_to_max(self, src, src_gidx, dst_gidx):
        """Exact centred lift of a value known modulo one or two primes to
        other primes (reference kernels ModUpToMax1 / ModUpToMax2,
        src/core/ElementWise.cu:579-623). src: plain coefficients; in the
        two-limb case limb k is already multiplied by (q_other)^-1 mod q_k."""
        src = np.asarray(src, dtype=np.uint32).astype(np.int64)
        q = [int(self.primes[g]) for g in src_gidx]
        out = np.empty((len(dst_gidx), self.n), dtype=np.uint32)
        if len(q) == 1:
            x = src[0]
        else:
            prod = q[0] * q[1]
            x = (src[0] * q[1] + src[1] * q[0]) % prod
            x = np.where(x > prod // 2, x - prod, x)
        for m, g in enumerate(dst_gidx):
            out[m] = (x % int(self.primes[g])).astype(np.uint32)
        return out

    def hmult(self, level, b1, a1, b2, a2, evk_b, evk_a, key_main, rescale=True):
        b1, a1, b2, a2 = map(_u32, (b1, a1, b2, a2))
        evk_b = [_u32(x) for x in evk_b]
        evk_a = [_u32(x) for x in evk_a]
        nd = len(self.level_limbs(level - 1 if rescale else level))
        ob = np.empty((nd, self.n), np.uint32)
        oa = np.empty((nd, self.n), np.uint32)
        self._call("orc_hmult", level, ob, oa, b1, a1, b2, a2, _ptr_array(evk_b), _ptr_array(evk_a),
                   int(key_main), int(rescale))
        return ob, oa

    def keyswitch(self, level, d, bx, evk_b, evk_a, key_main):
        d, bx = _u32(d), _u32(bx)
        evk_b = [_u32(x) for x in evk_b]
        evk_a = [_u32(x) for x in evk_a]
        nd = len(self.level_limbs(level))
        ob = np.empty((nd, self.n), np.uint32)
        oa = np.empty((nd, self.n), np.uint32)
        self._call("orc_keyswitch", level, ob, oa, d, bx, _ptr_array(evk_b), _ptr_array(evk_a), int(key_main))
        return ob, oa
