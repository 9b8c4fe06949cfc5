"""Python binding of libcheddar_b200.so through its C ABI (ctypes).

The directory name carries a hyphen, so load it with
`importlib.util.spec_from_file_location("cheddar_fhe_b200", ".../__init__.py")`
(tests/conftest.py, bench.py and __graft_entry__.py show how). PyTorch is used
only for device memory and streams; every operation goes through the shared
library, and a missing library is an error, never a fallback.
"""
import ctypes as C
import json
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libcheddar_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "cheddar_b200.h")
PARAM_DIR = os.path.join(_HERE, "parameters")

_lib = None


def build(verbose=False):
    """Compile every CUDA source for sm_100a into lib/libcheddar_b200.so."""
    cmd = ["make", "-C", _HERE, "-j8"]
    if not verbose:
        cmd.insert(1, "-s")
    subprocess.check_call(cmd)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {_HERE}`; there is no fallback path")
        L = C.CDLL(LIB_PATH)
        L.cfhe_last_error.restype = C.c_char_p
        L.cfhe_prime.restype = C.c_uint32
        _lib = L
    return _lib


class CfheError(RuntimeError):
    pass


def load_params(path_or_name):
    """Parameter JSON with the keys the reference's test fixture reads
    (reference unittest/Testbed.h:103-210)."""
    path = path_or_name
    if not os.path.exists(path):
        path = os.path.join(PARAM_DIR, path_or_name)
    with open(path) as f:
        j = json.load(f)
    j.setdefault("terminal_primes", [])
    j.setdefault("additional_base", [0, 0])
    return j


def _ints(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int))


def _u32s(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


class Engine:
    """One context on one GPU. Device buffers are torch int32 CUDA tensors of
    shape [..., limbs, N] holding the 32-bit words (reinterpreted)."""

    def __init__(self, params, device=0):
        import torch

        self.torch = torch
        self.L = lib()
        self.p = params
        self.device = device
        main, mp = _u32s(params["main_primes"])
        ter, tp = _u32s(params["terminal_primes"] if params["terminal_primes"] else [0])
        aux, ap = _u32s(params["auxiliary_primes"])
        lc, lp = _ints(np.array(params["level_config"]).reshape(-1))
        h = C.c_void_p()
        self._check(self.L.cfhe_context_create(
            C.byref(h), device, params["log_degree"], mp, len(params["main_primes"]),
            tp, len(params["terminal_primes"]), ap, len(params["auxiliary_primes"]),
            lp, len(params["level_config"]), params["additional_base"][0], params["additional_base"][1]))
        self.h = h
        self.n = self.L.cfhe_degree(h)
        self.num_primes = self.L.cfhe_num_primes(h)
        self.primes = np.array([self.L.cfhe_prime(h, g) for g in range(self.num_primes)], dtype=np.uint64)
        self.alpha = len(params["auxiliary_primes"])
        self.max_level = len(params["level_config"]) - 1
        self.use_torch_stream()

    def close(self):
        if getattr(self, "h", None):
            self.L.cfhe_context_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc < 0:
            raise CfheError(self.L.cfhe_last_error().decode())
        return rc

    def use_torch_stream(self):
        """Enqueue on torch's current stream so torch.cuda.Event brackets it."""
        s = self.torch.cuda.current_stream(self.device).cuda_stream
        self._check(self.L.cfhe_set_stream(self.h, C.c_void_p(s)))

    def synchronize(self):
        self._check(self.L.cfhe_synchronize(self.h))

    # ---- helpers
    def to_dev(self, a):
        t = self.torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint32).view(np.int32))
        return t.to(f"cuda:{self.device}")

    def to_host(self, t):
        return t.cpu().numpy().view(np.uint32)

    def empty(self, *shape):
        return self.torch.empty(shape, dtype=self.torch.int32, device=f"cuda:{self.device}")

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def level_limbs(self, level, num_aux=0):
        buf = np.zeros(128, np.int32)
        k = self._check(self.L.cfhe_level_limbs(self.h, level, num_aux, buf.ctypes.data_as(C.POINTER(C.c_int))))
        return buf[:k].copy()

    # ---- device-resident API: tensors [polys, limbs, N] or [limbs, N]
    def ntt_(self, dst, src, gidx, mont_conv=False):
        g, gp = _ints(gidx)
        polys = 1 if src.dim() == 2 else src.shape[0]
        stride_s = src.stride(0) if src.dim() == 3 else 0
        stride_d = dst.stride(0) if dst.dim() == 3 else 0
        self._check(self.L.cfhe_ntt(self.h, self._p(dst), self._p(src), gp, len(g), polys,
                                    C.c_longlong(stride_d), C.c_longlong(stride_s), int(mont_conv)))

    def intt_(self, dst, src, gidx, consts=None, mont_keep=False, centred=False):
        g, gp = _ints(gidx)
        polys = 1 if src.dim() == 2 else src.shape[0]
        stride_s = src.stride(0) if src.dim() == 3 else 0
        stride_d = dst.stride(0) if dst.dim() == 3 else 0
        if consts is not None:
            k, kp = _u32s(consts)
        else:
            kp = None
        self._check(self.L.cfhe_intt(self.h, self._p(dst), self._p(src), gp, len(g), polys,
                                     C.c_longlong(stride_d), C.c_longlong(stride_s), kp,
                                     int(mont_keep), int(centred)))

    # ---- host-array API with the golden model's signatures (copies in/out)
    def ntt(self, src, gidx, mont_conv=False):
        s = self.to_dev(src)
        d = self.torch.empty_like(s)
        self.ntt_(d, s, gidx, mont_conv)
        return self.to_host(d)

    def intt(self, src, gidx, consts=None, mont_keep=False, centred=False):
        s = self.to_dev(src)
        d = self.torch.empty_like(s)
        self.intt_(d, s, gidx, consts, mont_keep, centred)
        return self.to_host(d)
