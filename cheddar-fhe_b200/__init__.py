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

from . import client  # noqa: F401  (host-side keygen / encrypt / encode)

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
        L.cfhe_kernel_launch_count.restype = C.c_ulonglong
        _lib = L
    return _lib


def kernel_launch_count():
    """Kernels the library has launched in this process so far."""
    return int(lib().cfhe_kernel_launch_count())


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

    def order_after(self, earlier):
        """Work submitted to this engine from now on starts after everything
        already submitted to `earlier` (another engine on the same GPU)."""
        self._check(self.L.cfhe_order_after(self.h, earlier.h))

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

    def profile_begin(self):
        self._check(self.L.cfhe_profile_begin(self.h))

    def profile_end(self, cap=4096):
        """[(stage, ms)] of every pipeline stage since profile_begin()."""
        names = C.create_string_buffer(64 * cap)
        ms = (C.c_float * cap)()
        n = self._check(self.L.cfhe_profile_end(self.h, names, C.c_size_t(len(names)), ms, cap))
        return list(zip(names.value.decode().split(";")[:n], [float(ms[i]) for i in range(n)]))

    def beta(self, level):
        return self._check(self.L.cfhe_beta(self.h, level))

    def galois(self, rot):
        self.L.cfhe_galois_for_rotation.restype = C.c_uint32
        return self.L.cfhe_galois_for_rotation(self.h, int(rot))

    def _alpha(self, level):
        return len(self.level_limbs(-1)) if level == -1 else self.alpha

    def _ptrs(self, tensors):
        arr = (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
        return arr

    # ---- device-resident operators
    def binary_(self, op, dst, a, b, gidx):
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_binary(self.h, op, self._p(dst), self._p(a),
                                       self._p(b) if b is not None else None, gp, len(g)))

    def const_op_(self, op, dst, a, b, consts, gidx):
        g, gp = _ints(gidx)
        k, kp = _u32s(consts)
        self._check(self.L.cfhe_const_op(self.h, op, self._p(dst), self._p(a),
                                         self._p(b) if b is not None else None, kp, gp, len(g)))

    def elementwise_multi_(self, with_const, op, dsts, a_list, b_list, consts, gidx):
        """One launch for several polynomials (cfhe_elementwise_multi)."""
        g, gp = _ints(gidx)
        n = len(dsts)
        arr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() if t is not None else None for t in ts])
        kp = None
        if consts is not None:
            k, kp = _u32s(consts)
        self._check(self.L.cfhe_elementwise_multi(self.h, int(with_const), int(op), n, arr(dsts), arr(a_list),
                                                  arr(b_list) if b_list is not None else None, kp, gp, len(g)))

    def tensor_(self, d0, d1, d2, b1, a1, b2, a2, gidx):
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_tensor(self.h, *[self._p(t) for t in (d0, d1, d2, b1, a1, b2, a2)], gp, len(g)))

    def tensor_accum_(self, d0, d1, d2, b1s, a1s, b2s, a2s, gidx, accumulate=False):
        """(d0, d1, d2) (+)= sum_t tensor(b1s[t], a1s[t], b2s[t], a2s[t]) (cfhe_tensor_accum)."""
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_tensor_accum(self.h, self._p(d0), self._p(d1), self._p(d2), len(b1s),
                                             self._ptrs(b1s), self._ptrs(a1s), self._ptrs(b2s), self._ptrs(a2s),
                                             1 if accumulate else 0, gp, len(g)))

    def giantstep_paccum_(self, acc, rot, pts, gidx):
        """acc[j] = sum_i pts[j][i] (*) rot[i] (cfhe_giantstep_paccum); rot [n_baby][2][limbs][N],
        acc [n_giant][2][limbs][N], pts[j][i] a tensor or None."""
        g, gp = _ints(gidx)
        n_giant, n_baby = len(pts), len(pts[0])
        flat = (C.c_void_p * (n_giant * n_baby))(*[self._p(t) if t is not None else None
                                                     for row in pts for t in row])
        self._check(self.L.cfhe_giantstep_paccum(self.h, self._p(acc), self._p(rot), n_baby, n_giant, flat,
                                                 gp, len(g)))

    def permute_(self, dst, src, add, galois, gidx):
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_permute(self.h, self._p(dst), self._p(src),
                                        self._p(add) if add is not None else None,
                                        C.c_uint32(int(galois)), gp, len(g)))

    def nary_(self, kind, dsts, terms, gidx, consts=None, pts=None, galois=None, addend=None):
        """Fused n-ary sums (cfhe_accum / cfhe_caccum / cfhe_paccum /
        cfhe_permute_accum): dsts[p] = (addend[p]) + sum_t term_t(terms[t][p]).
        kind: "sum", "const" (consts[t][limb], M-form), "plain" (pts[t]) or
        "permute" (galois[t])."""
        g, gp = _ints(gidx)
        n_polys, n_terms = len(dsts), len(terms)
        dst = self._ptrs(dsts)
        src = self._ptrs([terms[t][p] for t in range(n_terms) for p in range(n_polys)])
        add = self._ptrs(addend) if addend is not None else None
        if kind == "sum":
            rc = self.L.cfhe_accum(self.h, n_polys, dst, n_terms, src, gp, len(g))
        elif kind == "const":
            k, kp = _u32s(np.asarray(consts, dtype=np.uint32).reshape(-1))
            rc = self.L.cfhe_caccum(self.h, n_polys, dst, n_terms, src, kp, add, gp, len(g))
        elif kind == "plain":
            rc = self.L.cfhe_paccum(self.h, n_polys, dst, n_terms, src, self._ptrs(pts), add, gp, len(g))
        elif kind == "permute":
            k, kp = _u32s(galois)
            rc = self.L.cfhe_permute_accum(self.h, n_polys, dst, n_terms, src, kp, add, gp, len(g))
        else:
            raise ValueError(kind)
        self._check(rc)

    def gemm_pack_weights(self, weights, gidx):
        """weights: uint32 [n_limbs][n_in][n_out] in M-form; returns the packed device buffer."""
        w = np.ascontiguousarray(weights, dtype=np.uint32)
        n_limbs, n_in, n_out = w.shape
        g, gp = _ints(gidx)
        self.L.cfhe_gemm_weight_bytes.restype = C.c_size_t
        nbytes = self.L.cfhe_gemm_weight_bytes(n_in, n_out, n_limbs)
        packed = self.torch.empty(nbytes, dtype=self.torch.uint8, device=f"cuda:{self.device}")
        self._check(self.L.cfhe_gemm_pack_weights(self.h, C.c_void_p(packed.data_ptr()),
                                                  w.ctypes.data_as(C.POINTER(C.c_uint32)), n_in, n_out, gp, len(g)))
        return packed

    def ctpt_gemm_(self, ys, xs, packed, gidx):
        """ys[j] = sum_k W[k][j] * xs[k] on the tensor cores (cfhe_ctpt_gemm)."""
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_ctpt_gemm(self.h, self._ptrs(ys), self._ptrs(xs), C.c_void_p(packed.data_ptr()),
                                          len(xs), len(ys), gp, len(g)))

    def sample_uniform_(self, dst, gidx, seed, stream=0):
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_sample_uniform(self.h, self._p(dst), gp, len(g), C.c_ulonglong(seed),
                                               C.c_uint(stream)))

    def sample_error_(self, dst, gidx, sigma, seed, stream=0):
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_sample_error(self.h, self._p(dst), gp, len(g), C.c_double(sigma),
                                             C.c_ulonglong(seed), C.c_uint(stream)))

    def error_cdf(self, sigma):
        out = np.zeros(97, dtype=np.uint64)
        self._check(self.L.cfhe_error_cdf(C.c_double(sigma), out.ctypes.data_as(C.c_void_p), 97))
        return out

    def encrypt_(self, b, a, s, e, m, gidx):
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_encrypt(self.h, self._p(b), self._p(a), self._p(s), self._p(e),
                                        self._p(m) if m is not None else None, gp, len(g)))

    def encode_coeffs_(self, dst, coeffs, gidx):
        """dst = NTT (M-form) of the residues of trunc(coeffs[i]) on the limbs of gidx
        (cfhe_encode_coeffs); coeffs: N float64 values on the host."""
        g, gp = _ints(gidx)
        c = np.ascontiguousarray(coeffs, dtype=np.float64)
        assert c.shape == (self.n,)
        self._check(self.L.cfhe_encode_coeffs(self.h, self._p(dst), c.ctypes.data_as(C.c_void_p), gp, len(g)))

    def add_evk_part_(self, bx, s_target, p_prod, gidx):
        g, gp = _ints(gidx)
        k, kp = _u32s(p_prod)
        self._check(self.L.cfhe_add_evk_part(self.h, self._p(bx), self._p(s_target), kp, gp, len(g)))

    def pseudo_modup_(self, level, dst, src):
        self._check(self.L.cfhe_pseudo_modup(self.h, level, self._p(dst), self._p(src)))

    def modup_(self, level, dst, src):
        self._check(self.L.cfhe_modup(self.h, level, self._p(dst), self._p(src)))

    def moddown_(self, level, kind, dst, src):
        """dst/src: [limbs, N] or [polys, limbs, N]."""
        polys = 1 if src.dim() == 2 else src.shape[0]
        ss = src.stride(0) if src.dim() == 3 else 0
        ds = dst.stride(0) if dst.dim() == 3 else 0
        self._check(self.L.cfhe_moddown(self.h, level, kind, self._p(dst), self._p(src), polys,
                                        C.c_longlong(ds), C.c_longlong(ss)))

    def moddown_staged_(self, level, kind, dst, src):
        """The same as moddown_, composed from the three stage entries
        (cfhe_intt_for_moddown, cfhe_bconv_for_moddown, cfhe_ntt_for_moddown)."""
        polys = 1 if src.dim() == 2 else src.shape[0]
        ss = src.stride(0) if src.dim() == 3 else 0
        ds = dst.stride(0) if dst.dim() == 3 else 0
        ns = self.L.cfhe_moddown_source_limbs(self.h, level, kind)
        if ns < 0:
            self._check(ns)
        y = self.torch.empty((polys, ns, self.n), dtype=self.torch.int32, device=src.device)
        self._check(self.L.cfhe_intt_for_moddown(self.h, level, kind, self._p(y), self._p(src), polys,
                                                 C.c_longlong(ss)))
        self._check(self.L.cfhe_bconv_for_moddown(self.h, level, kind, self._p(dst), self._p(y), polys,
                                                  C.c_longlong(ds)))
        self._check(self.L.cfhe_ntt_for_moddown(self.h, level, kind, self._p(dst), self._p(src), polys,
                                                C.c_longlong(ds), C.c_longlong(ss)))

    def moddown_noalloc_(self, level, kind, dst, src):
        """One polynomial, [limbs, N]; no device allocation on the call path."""
        self._check(self.L.cfhe_moddown_noalloc(self.h, level, kind, self._p(dst), self._p(src)))

    def evk_inner_(self, level, acc_b, acc_a, modup, c0, c1, evk_b, evk_a, key_main):
        self._check(self.L.cfhe_evk_inner(self.h, level, self._p(acc_b), self._p(acc_a), self._p(modup),
                                          self._p(c0) if c0 is not None else None,
                                          self._p(c1) if c1 is not None else None,
                                          self._ptrs(evk_b), self._ptrs(evk_a), int(key_main)))

    def keyswitch_(self, level, out_b, out_a, d, bx, evk_b, evk_a, key_main):
        self._check(self.L.cfhe_keyswitch(self.h, level, self._p(out_b), self._p(out_a), self._p(d),
                                          self._p(bx) if bx is not None else None,
                                          self._ptrs(evk_b), self._ptrs(evk_a), int(key_main)))

    def hoisted_rotations_(self, level, out, bx, ax, rots, evk_b, evk_a, key_main):
        """out: [n_rot, 2, nq, N]; evk_b/evk_a: per rotation a list of beta digit tensors."""
        r, rp = _ints(rots)
        flat_b = [t for key in evk_b for t in key]
        flat_a = [t for key in evk_a for t in key]
        self._check(self.L.cfhe_hoisted_rotations(self.h, level, self._p(out), self._p(bx), self._p(ax),
                                                  len(r), rp, self._ptrs(flat_b), self._ptrs(flat_a),
                                                  int(key_main)))

    def linear_transform_(self, level, out_b, out_a, in_b, in_a, baby_rots, baby_keys, giant_rots,
                          giant_keys, pts, key_main, rescale=True):
        """Baby-step/giant-step linear transform (cfhe_linear_transform).
        baby_rots[0] must be 0. baby_keys / giant_keys: per step a pair
        (digits_b, digits_a) of lists of beta device tensors, or None for an
        unrotated step. pts[j][i]: device tensor [(nq+alpha), N] or None."""
        beta = self.beta(level)

        def flat(keys, part):
            out = []
            for k in keys:
                out += [None] * beta if k is None else list(k[part][:beta])
            return (C.c_void_p * len(out))(*[t.data_ptr() if t is not None else None for t in out])

        br, brp = _ints(baby_rots)
        gr, grp = _ints(giant_rots)
        ptl = [pts[j][i] for j in range(len(gr)) for i in range(len(br))]
        pta = (C.c_void_p * len(ptl))(*[t.data_ptr() if t is not None else None for t in ptl])
        self._check(self.L.cfhe_linear_transform(
            self.h, level, int(rescale), self._p(out_b), self._p(out_a), self._p(in_b), self._p(in_a),
            len(br), brp, flat(baby_keys, 0), flat(baby_keys, 1),
            len(gr), grp, flat(giant_keys, 0), flat(giant_keys, 1), pta, int(key_main)))

    def modup_to_max_(self, dst, src, src_gidx, dst_gidx):
        """Exact centred lift of a one- or two-limb value (cfhe_modup_to_max)."""
        sg, sgp = _ints(src_gidx)
        dg, dgp = _ints(dst_gidx)
        self._check(self.L.cfhe_modup_to_max(self.h, self._p(dst), self._p(src), sgp, len(sg), dgp, len(dg)))

    def modup_to_max(self, src, src_gidx, dst_gidx):
        d = self.empty(len(dst_gidx), self.n)
        self.modup_to_max_(d, self.to_dev(src), src_gidx, dst_gidx)
        return self.to_host(d)

    def hmult_(self, level, out_b, out_a, b1, a1, b2, a2, evk_b, evk_a, key_main, rescale=True):
        self._check(self.L.cfhe_hmult(self.h, level, self._p(out_b), self._p(out_a),
                                      self._p(b1), self._p(a1), self._p(b2), self._p(a2),
                                      self._ptrs(evk_b), self._ptrs(evk_a), int(key_main), int(rescale)))

    # ---- host-array operators with the golden model's signatures
    def _bin(self, op, a, b, gidx):
        da = self.to_dev(a)
        db = self.to_dev(b) if b is not None else None
        d = self.torch.empty_like(da)
        self.binary_(op, d, da, db, gidx)
        return self.to_host(d)

    def add(self, a, b, gidx):
        return self._bin(0, a, b, gidx)

    def sub(self, a, b, gidx):
        return self._bin(1, a, b, gidx)

    def neg(self, a, gidx):
        return self._bin(2, a, None, gidx)

    def mul(self, a, b, gidx):
        return self._bin(3, a, b, gidx)

    def const_op(self, a, k, gidx, op, b=None):
        da = self.to_dev(a)
        db = self.to_dev(b) if b is not None else None
        d = self.torch.empty_like(da)
        self.const_op_(op, d, da, db, k, gidx)
        return self.to_host(d)

    def tensor(self, b1, a1, b2, a2, gidx):
        ins = [self.to_dev(x) for x in (b1, a1, b2, a2)]
        outs = [self.torch.empty_like(ins[0]) for _ in range(3)]
        self.tensor_(*outs, *ins, gidx)
        return tuple(self.to_host(o) for o in outs)

    def permute(self, a, galois, gidx=None, add=None):
        da = self.to_dev(a)
        if gidx is None:
            gidx = [0] * da.shape[0]
        d = self.torch.empty_like(da)
        self.permute_(d, da, self.to_dev(add) if add is not None else None, galois, gidx)
        return self.to_host(d)

    def mul_imag_unit(self, a, gidx):
        da = self.to_dev(a)
        d = self.torch.empty_like(da)
        g, gp = _ints(gidx)
        self._check(self.L.cfhe_mul_imag_unit(self.h, self._p(d), self._p(da), gp, len(g)))
        return self.to_host(d)

    def bconv_(self, dst, y, src_gidx, dst_gidx):
        """Base conversion of centred residues y [n_src][N] (int32 words) into
        the limbs dst_gidx, device-resident (cfhe_bconv)."""
        sg, sp = _ints(src_gidx)
        dg, dp = _ints(dst_gidx)
        self._check(self.L.cfhe_bconv(self.h, self._p(dst), self._p(y), sp, len(sg), dp, len(dg)))

    def bconv(self, y, src_gidx, dst_gidx):
        dy = self.to_dev(np.ascontiguousarray(y, dtype=np.int32).view(np.uint32))
        sg, sp = _ints(src_gidx)
        dg, dp = _ints(dst_gidx)
        d = self.empty(len(dg), self.n)
        self._check(self.L.cfhe_bconv(self.h, self._p(d), self._p(dy), sp, len(sg), dp, len(dg)))
        return self.to_host(d)

    def modup(self, level, src):
        ntot = len(self.level_limbs(level, self._alpha(level)))
        d = self.torch.zeros((self.beta(level), ntot, self.n), dtype=self.torch.int32,
                             device=f"cuda:{self.device}")
        self.modup_(level, d, self.to_dev(src))
        return self.to_host(d)

    def moddown(self, level, kind, src):
        s = self.to_dev(src)
        nd = len(self.level_limbs(level if kind == 0 else level - 1))
        shape = (nd, self.n) if s.dim() == 2 else (s.shape[0], nd, self.n)
        d = self.empty(*shape)
        self.moddown_(level, kind, d, s)
        return self.to_host(d)

    def evk_inner(self, level, modup, evk_b, evk_a, key_main, c0=None, c1=None):
        mu = self.to_dev(modup)
        kb = [self.to_dev(x) for x in evk_b]
        ka = [self.to_dev(x) for x in evk_a]
        ab = self.empty(mu.shape[1], self.n)
        aa = self.empty(mu.shape[1], self.n)
        self.evk_inner_(level, ab, aa, mu, self.to_dev(c0) if c0 is not None else None,
                        self.to_dev(c1) if c1 is not None else None, kb, ka, key_main)
        return self.to_host(ab), self.to_host(aa)

    def keyswitch(self, level, d, bx, evk_b, evk_a, key_main):
        kb = [self.to_dev(x) for x in evk_b]
        ka = [self.to_dev(x) for x in evk_a]
        nd = len(self.level_limbs(level))
        ob, oa = self.empty(nd, self.n), self.empty(nd, self.n)
        self.keyswitch_(level, ob, oa, self.to_dev(d), self.to_dev(bx), kb, ka, key_main)
        return self.to_host(ob), self.to_host(oa)

    def hmult(self, level, b1, a1, b2, a2, evk_b, evk_a, key_main, rescale=True):
        kb = [self.to_dev(x) for x in evk_b]
        ka = [self.to_dev(x) for x in evk_a]
        nd = len(self.level_limbs(level - 1 if rescale else level))
        ob, oa = self.empty(nd, self.n), self.empty(nd, self.n)
        self.hmult_(level, ob, oa, *[self.to_dev(x) for x in (b1, a1, b2, a2)], kb, ka, key_main, rescale)
        return self.to_host(ob), self.to_host(oa)
