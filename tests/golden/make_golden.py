"""Generates tests/golden/reference_digests.json on a GPU box from the
reference's own CUDA library (oracle/_ref/libcheddar_ref.so, built unmodified
from the reference sources by `make -C oracle ref`).

For seeded inputs it runs the reference's NTT / INTT, ModUp, the three ModDown
forms and HMult and stores, per case, the SHA-256 of the output words and the
first words of every limb. The CPU suite regenerates the same inputs, runs the
golden model on them and compares: that pins the model to the reference on
machines without a GPU.

    python tests/golden/make_golden.py        # needs a GPU and oracle/_ref
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

N = 1 << 16
HEAD = 4  # words kept per limb beside the digest


def rand_limbs(rng, primes, gidx):
    return np.stack([rng.integers(0, int(primes[g]), N, dtype=np.uint64).astype(np.uint32) for g in gidx])


def record(arr):
    a = np.ascontiguousarray(arr, dtype=np.uint32)
    return {"shape": list(a.shape), "sha256": hashlib.sha256(a.tobytes()).hexdigest(),
            "head": a.reshape(-1, N)[:, :HEAD].tolist()}


# the cases, shared with the CPU test (tests/test_oracle_cpu.py)
NTT_CASES = [(2, 2, 2), (0, 2, 0), (5, 0, 1)]          # (num_main, num_ter, num_aux)
MODUP_LEVELS = [0, 2, 5]
MODDOWN_LEVELS = [1, 2, 3]
HMULT_CASES = [(3, True), (1, True), (2, False)]


def ntt_limbs(case, T=4, L=47):
    nm, nt, na = case
    return list(range(T - nt, T + nm)) + [L + a for a in range(na)]


def main():
    import torch
    from conftest import load_package
    from oracle import ref_binding

    pkg = load_package()
    params = pkg.load_params("bootparam_40.json")
    eng = pkg.Engine(params, device=0)  # only for limb lists and device buffers
    ref = ref_binding.Reference(params)
    primes = eng.primes
    out = {"parameter_set": "bootparam_40.json", "head_words": HEAD, "cases": {}}
    for case in NTT_CASES:
        g = ntt_limbs(case)
        a = rand_limbs(np.random.default_rng(9000 + sum(case)), primes, g)
        src = eng.to_dev(a)
        for inverse in (False, True):
            for mont in (False, True):
                dst = torch.empty_like(src)
                ref.ntt(dst, src, *case, inverse=inverse, mont_conv=mont)
                out["cases"][f"ntt{case}_inv{int(inverse)}_mont{int(mont)}"] = record(eng.to_host(dst))
    for level in MODUP_LEVELS:
        g = eng.level_limbs(level)
        a = rand_limbs(np.random.default_rng(9100 + level), primes, g)
        dst = torch.zeros((eng.beta(level), len(g) + eng.alpha, N), dtype=torch.int32, device="cuda:0")
        ref.modup(level, dst, eng.to_dev(a))
        out["cases"][f"modup_level{level}"] = record(eng.to_host(dst))
    for level in MODDOWN_LEVELS:
        full = eng.level_limbs(level, eng.alpha)
        a = rand_limbs(np.random.default_rng(9200 + level), primes, full)
        nq = len(full) - eng.alpha
        for kind in (0, 1, 2):
            x = a if kind != 1 else np.ascontiguousarray(a[:nq])
            nd = len(eng.level_limbs(level if kind == 0 else level - 1))
            dst = eng.empty(nd, N)
            ref.moddown(level, kind, dst, eng.to_dev(x))
            out["cases"][f"moddown_level{level}_kind{kind}"] = record(eng.to_host(dst))
    params_max_level = len(params["level_config"]) - 1
    M, T = len(params["main_primes"]), len(params["terminal_primes"])
    kg = list(range(T + M)) + [T + M + a for a in range(eng.alpha)]
    for level, rescale in HMULT_CASES:
        rng = np.random.default_rng(9300 + level)
        g = eng.level_limbs(level)
        ins = [rand_limbs(rng, primes, g) for _ in range(4)]
        beta = eng.beta(params_max_level)  # a key made for the top level serves every level
        kb = [rand_limbs(rng, primes, kg) for _ in range(beta)]
        ka = [rand_limbs(rng, primes, kg) for _ in range(beta)]
        nd = len(eng.level_limbs(level - 1 if rescale else level))
        rb, ra = eng.empty(nd, N), eng.empty(nd, N)
        ref.hmult(level, rb, ra, *[eng.to_dev(x) for x in ins], [eng.to_dev(x) for x in kb],
                  [eng.to_dev(x) for x in ka], M, rescale)
        out["cases"][f"hmult_level{level}_rescale{int(rescale)}"] = record(
            np.stack([eng.to_host(rb), eng.to_host(ra)]))
    ref.close()
    path = os.path.join(HERE, "reference_digests.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
    print("wrote", path, len(out["cases"]), "cases")


if __name__ == "__main__":
    main()
