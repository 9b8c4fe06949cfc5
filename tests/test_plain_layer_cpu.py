"""The float64 transformer layer used as the checker of the encrypted layer
(oracle/transformer_plain.h) against PyTorch's own float64 operators
(softmax, erf-GELU, layer_norm, matmul): with the exact functions the two must
agree to rounding, and with the Chebyshev series the layer evaluates (fitted
here as the product fits them: interpolation at Chebyshev nodes) to the
series' approximation error. Host only."""
import os
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")


def cheb_coefficients(f, degree, points=256):
    th = np.pi * (np.arange(points) + 0.5) / points
    y = f(np.cos(th))
    c = np.array([(y * np.cos(k * th)).sum() * 2.0 / points for k in range(degree + 1)])
    c[0] /= 2.0
    return c


def torch_layer(x, w, heads, eps):
    import torch
    import torch.nn.functional as F
    t = {k: torch.tensor(v, dtype=torch.float64) for k, v in w.items()}
    x = torch.tensor(x, dtype=torch.float64)
    T, H = x.shape
    D = H // heads
    q = (x @ t["wq"] + t["bq"]).view(T, heads, D).transpose(0, 1)
    k = (x @ t["wk"] + t["bk"]).view(T, heads, D).transpose(0, 1)
    v = (x @ t["wv"] + t["bv"]).view(T, heads, D).transpose(0, 1)
    att = F.softmax(q @ k.transpose(1, 2) / D ** 0.5, dim=-1) @ v
    o = att.transpose(0, 1).reshape(T, H) @ t["wo"] + t["bo"]
    h1 = F.layer_norm(x + o, (H,), t["gamma1"], t["beta1"], eps)
    a = F.gelu(h1 @ t["w1"] + t["b1"])
    h2 = F.layer_norm(h1 + a @ t["w2"] + t["b2"], (H,), t["gamma2"], t["beta2"], eps)
    return h2.numpy()


@pytest.mark.parametrize("exact", [True, False])
def test_plain_layer_matches_torch_float64(tmp_path, exact):
    subprocess.check_call(["make", "-s", "-C", CPP, "plain_layer"])
    rng = np.random.default_rng(31 + exact)
    T, H, heads, Fn = 16, 32, 2, 64
    R, lo, hi, vlo, vhi, G, eps = 2.0, 0.04, 0.8, 0.15, 6.5, 4.0, 1e-5
    deg = (15, 63, 63, 31)
    from math import erf
    verf = np.vectorize(erf)
    series = [
        cheb_coefficients(lambda u: np.exp(R * (u - 1.0)), deg[0]),
        cheb_coefficients(lambda w: 1.0 / (T * 0.5 * ((hi - lo) * w + hi + lo)), deg[1]),
        cheb_coefficients(lambda w: 0.5 / np.sqrt(0.5 * ((vhi - vlo) * w + vhi + vlo) + eps), deg[2]),
        cheb_coefficients(lambda t: 0.5 * (G * t) * (1.0 + verf(G * t / np.sqrt(2.0))) / G, deg[3]),
    ]
    shapes = [("wq", (H, H)), ("wk", (H, H)), ("wv", (H, H)), ("wo", (H, H)), ("w1", (H, Fn)), ("w2", (Fn, H)),
              ("bq", (H,)), ("bk", (H,)), ("bv", (H,)), ("bo", (H,)), ("b1", (Fn,)), ("b2", (H,)),
              ("gamma1", (H,)), ("beta1", (H,)), ("gamma2", (H,)), ("beta2", (H,))]
    w = {}
    for name, shape in shapes:
        centre = 1.0 if name.startswith("gamma") else 0.0
        w[name] = centre + 0.08 * rng.standard_normal(shape)
    x = rng.standard_normal((T, H))
    blob = struct.pack("<9i", T, H, heads, Fn, int(exact), *deg) + struct.pack("<7d", R, lo, hi, vlo, vhi, G, eps)
    for c in series:
        blob += np.asarray(c, dtype="<f8").tobytes()
    for name, _ in shapes:
        blob += np.ascontiguousarray(w[name], dtype="<f8").tobytes()
    blob += np.ascontiguousarray(x, dtype="<f8").tobytes()
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    fin.write_bytes(blob)
    subprocess.check_call([os.path.join(CPP, "plain_layer"), str(fin), str(fout)])
    got = np.frombuffer(fout.read_bytes(), dtype="<f8").reshape(T, H)
    want = torch_layer(x, w, heads, eps)
    err = np.abs(got - want).max()
    print("max |oracle - torch|", err)
    assert err < (1e-12 if exact else 1e-6)


def test_block_partition_of_the_sharded_layer():
    """Every item of a sharded vector is owned by exactly one rank, block sizes
    differ by at most one, and the owner lookup agrees (host/cheddar/RankGroup.h)."""
    subprocess.check_call(["make", "-s", "-C", CPP, "plain_layer"])
    r = subprocess.run([os.path.join(CPP, "plain_layer"), "--blocks"], capture_output=True, text=True)
    assert r.returncode == 0 and "blocks ok" in r.stdout
