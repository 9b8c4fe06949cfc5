"""Python mirror of the reference's client side: key generation, encryption,
decryption (reference src/UserInterface.cu:131-190, :223-276, :366-458) and
CKKS encoding (reference src/core/Encode.cpp:23-275).

Like the reference's UserInterface it is host code that samples on the CPU and
calls the engine for the transforms and the element-wise products. It works on
any engine object that offers `ntt`, `intt`, `mul`, `add`, `sub`, `const_op`,
`permute`, `level_limbs` on host arrays, i.e. the CUDA `Engine` of this
package; the tests also drive the CPU golden model with it.
"""
import numpy as np


def brev(v, bits):
    r = 0
    for i in range(bits):
        r |= ((v >> i) & 1) << (bits - 1 - i)
    return r


class Client:
    def __init__(self, eng, seed=0, hamming=None, sigma=3.2):
        self.e = eng
        self.n = eng.n
        self.rng = np.random.default_rng(seed)
        self.sigma = sigma
        self.all = list(range(eng.num_primes))
        h = hamming if hamming is not None else self.n // 2
        # ternary secret with fixed Hamming weight (UserInterface.cu:223-276)
        s = np.zeros(self.n, dtype=np.int64)
        pos = self.rng.choice(self.n, size=h, replace=False)
        s[pos] = self.rng.choice([-1, 1], size=h)
        self.s_coef = s
        self.s = self.to_ntt(s, self.all)  # every prime, M-form

    # integer coefficient vector -> NTT domain, M-form, on limbs gidx
    def to_ntt(self, coefs, gidx):
        res = np.stack([np.mod(coefs, int(self.e.primes[g])).astype(np.uint32) for g in gidx])
        return self.e.ntt(res, gidx, True)

    def uniform(self, gidx):
        return np.stack([self.rng.integers(0, int(self.e.primes[g]), self.n, dtype=np.uint64).astype(np.uint32)
                         for g in gidx])

    def error(self, gidx):
        e = np.rint(self.rng.normal(0, self.sigma, self.n)).astype(np.int64)
        return self.to_ntt(e, gidx)

    def secret(self, gidx, s=None):
        s = self.s if s is None else s
        return s[np.asarray(gidx)]

    def encrypt(self, coefs, level):
        """b = m - a*s + e on the limbs of `level` (UserInterface.cu:17-50)."""
        g = self.e.level_limbs(level)
        a = self.uniform(g)
        m = self.to_ntt(coefs, g)
        b = self.e.add(self.e.sub(m, self.e.mul(a, self.secret(g), g), g), self.error(g), g)
        return b, a

    def decrypt(self, b, a, gidx):
        """Centred integer coefficients of b + a*s (UserInterface.cu:170-190)."""
        g = list(gidx)
        m = self.e.add(b, self.e.mul(a, self.secret(g), g), g)
        c = self.e.intt(m, g)  # leaves M-form: plain residues
        return self.crt(c, g)

    def encrypt_message(self, msg, level, scale):
        """Encode complex slots at `scale`, then encrypt at `level`."""
        return self.encrypt(encode_coefs(msg, self.n, scale), level)

    def decrypt_message(self, b, a, gidx, scale, num_slots):
        return decode_coefs(self.decrypt(b, a, gidx), self.n, scale, num_slots)

    def crt(self, res, gidx):
        qs = [int(self.e.primes[g]) for g in gidx]
        Q = 1
        for q in qs:
            Q *= q
        acc = np.zeros(self.n, dtype=object)
        for r, q in zip(res, qs):
            Qi = Q // q
            acc = (acc + r.astype(object) * (Qi * pow(Qi, -1, q))) % Q
        return np.array([int(x) - Q if int(x) > Q // 2 else int(x) for x in acc], dtype=object)

    def key_limbs(self, key_main):
        T = len(self.e.p["terminal_primes"])
        L = T + len(self.e.p["main_primes"])
        return list(range(0, T + key_main)) + [L + a for a in range(self.e.alpha)]

    def switching_key(self, s_enc, s_target, key_main):
        """Digit j: b_j = e_j - a_j*s_enc, plus P*s_target on digit j's limbs
        (UserInterface.cu:366-458). s_enc/s_target: M-form on every prime."""
        g = self.key_limbs(key_main)
        alpha = self.e.alpha
        nq = len(g) - alpha
        beta = -(-nq // alpha)
        L = self.e.num_primes - alpha
        P = 1
        for a in range(alpha):
            P *= int(self.e.primes[L + a])
        kb, ka = [], []
        for j in range(beta):
            a = self.uniform(g)
            b = self.e.sub(self.error(g), self.e.mul(a, s_enc[g], g), g)
            lo, hi = j * alpha, min((j + 1) * alpha, nq)
            gd = g[lo:hi]
            pk = np.array([((P % int(self.e.primes[x])) << 32) % int(self.e.primes[x]) for x in gd], dtype=np.uint32)
            add = self.e.const_op(s_target[gd], pk, gd, 3)
            b[lo:hi] = self.e.add(b[lo:hi], add, gd)
            kb.append(b)
            ka.append(a)
        return kb, ka

    def mult_key(self, key_main):
        s2 = self.e.mul(self.s, self.s, self.all)
        return self.switching_key(self.s, s2, key_main)

    def rotation_key(self, rot, key_main):
        """Key for sigma_rot: encryption secret = secret permuted by the
        opposite rotation (UserInterface.cu:303-306)."""
        gal = self.e.galois(self.n // 2 - rot) if rot >= 0 else self.e.galois(-1)
        s_rot = self.e.permute(self.s, gal)
        return self.switching_key(s_rot, self.s, key_main)


def negacyclic_mul(a, b):
    n = len(a)
    out = np.zeros(n, dtype=object)
    for i in range(n):
        if a[i] == 0:
            continue
        for j in range(n):
            k = i + j
            if k < n:
                out[k] += int(a[i]) * int(b[j])
            else:
                out[k - n] -= int(a[i]) * int(b[j])
    return out


def toy_params(logn=5):
    """A small ring with the same shape of level table as the shipped sets:
    terminal primes that are dropped and restored by rational rescaling."""
    n = 1 << logn

    def isprime(x):
        i = 2
        while i * i <= x:
            if x % i == 0:
                return False
            i += 1
        return x > 1

    def gen(lo, cnt):
        out, x = [], lo - lo % (2 * n) + 1
        while len(out) < cnt:
            if x > lo and isprime(x):
                out.append(x)
            x += 2 * n
        return out

    main = gen(1 << 26, 7)
    ter = gen(1 << 19, 4)
    aux = gen((1 << 31) - (1 << 22), 3)
    return dict(log_degree=logn, log_default_scale=20, default_encryption_level=4,
                main_primes=main, terminal_primes=ter, auxiliary_primes=aux,
                level_config=[[0, 2], [3, 0], [1, 4], [4, 2], [7, 0], [7, 2], [7, 4]],
                additional_base=[0, 0])


# ---------------------------------------------------------------------------
# CKKS encoding (reference src/core/Encode.cpp:85-248), numpy version
# ---------------------------------------------------------------------------
def _bitrev_perm(n):
    bits = n.bit_length() - 1
    idx = np.arange(n)
    out = np.zeros(n, dtype=np.int64)
    for b in range(bits):
        out |= ((idx >> b) & 1) << (bits - 1 - b)
    return out


def _galois_pows(count, m):
    g = np.ones(max(count, 1), dtype=np.int64)
    for i in range(1, count):
        g[i] = (g[i - 1] * 5) % m
    return g


def special_ifft(vals, degree):
    """Encode.cpp:85-109."""
    d = np.array(vals, dtype=np.complex128)
    n = len(d)
    m = 2 * degree
    tw = np.exp(2j * np.pi * np.arange(m) / m)
    gal = _galois_pows(n // 2 if n > 1 else 1, m)
    s = n // 2
    while s >= 1:
        st8 = s << 3
        gap = m // st8
        idx = (st8 - (gal[:s] % st8)) * gap
        v = d.reshape(-1, 2, s)
        x = v[:, 0, :] + v[:, 1, :]
        y = (v[:, 0, :] - v[:, 1, :]) * tw[idx % m]
        d = np.stack([x, y], axis=1).reshape(-1)
        s //= 2
    return d[_bitrev_perm(n)] / n


def special_fft(vals, degree):
    """Encode.cpp:111-133."""
    d = np.array(vals, dtype=np.complex128)
    n = len(d)
    m = 2 * degree
    tw = np.exp(2j * np.pi * np.arange(m) / m)
    gal = _galois_pows(n // 2 if n > 1 else 1, m)
    d = d[_bitrev_perm(n)]
    s = 1
    while s < n:
        st8 = s << 3
        gap = m // st8
        idx = (gal[:s] % st8) * gap
        v = d.reshape(-1, 2, s)
        y = v[:, 1, :] * tw[idx]
        d = np.stack([v[:, 0, :] + y, v[:, 0, :] - y], axis=1).reshape(-1)
        s *= 2
    return d


def encode_coefs(msg, degree, scale):
    """Complex slots -> integer coefficients (truncated toward zero, as
    BigInt(double) does, src/core/BigInt_gmp.cpp:22-25). Real parts at
    i*gap, imaginary parts at i*gap + N/2 (Encode.cpp:169-182)."""
    n = len(msg)
    gap = (degree // 2) // n
    v = special_ifft(msg, degree) * scale
    coefs = np.zeros(degree, dtype=object)
    re = [int(x) for x in np.trunc(v.real)]
    im = [int(x) for x in np.trunc(v.imag)]
    for i in range(n):
        coefs[i * gap] = re[i]
        coefs[i * gap + degree // 2] = im[i]
    return coefs


def decode_coefs(coefs, degree, scale, num_slots):
    gap = (degree // 2) // num_slots
    re = np.array([float(coefs[i * gap]) for i in range(num_slots)])
    im = np.array([float(coefs[i * gap + degree // 2]) for i in range(num_slots)])
    return special_fft((re + 1j * im) / scale, degree)


def level_scale(params, level):
    """Scale used by the reference's tests at `level` (unittest/Testbed.h:236-243
    with the schedule of src/core/Parameter.cu:149-193)."""
    lc = params["level_config"]
    main, ter = params["main_primes"], params["terminal_primes"]
    scale = float(2 ** params["log_default_scale"])
    prods = [None]
    for i in range(1, len(lc)):
        (um, ut), (lm, lt) = lc[i], lc[i - 1]
        num = den = 1.0
        if ut >= lt:
            for j in range(ut - lt):
                num *= ter[lt + j]
        else:
            for j in range(lt - ut):
                den *= ter[ut + j]
        if um >= lm:
            for j in range(um - lm):
                num *= main[lm + j]
        else:
            for j in range(lm - um):
                den *= main[um + j]
        prods.append(num / den)
    scales = [scale]
    for i in range(1, params["default_encryption_level"] + 1):
        scale = (scale * prods[i]) ** 0.5
        scales.append(scale)
    if level <= params["default_encryption_level"]:
        return scales[level], prods
    return prods[level], prods
