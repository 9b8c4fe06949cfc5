"""Small Python CKKS client used by the tests (test infrastructure).

It follows the reference's test client (src/UserInterface.cu:131-190 encrypt /
decrypt, :223-276 secrets, :366-458 switching keys) on top of any engine that
offers `ntt`, `intt`, `mul`, `add`, `sub` with the golden model's signatures,
so the same client drives the CPU model and the CUDA library.
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
