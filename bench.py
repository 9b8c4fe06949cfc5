#!/usr/bin/env python
"""Benchmark of the CKKS hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload hmult|ntt]
    python bench.py --impl reference ...      # CPU golden model on host cores

Prints ONE JSON line (rank 0). Under torchrun every rank works on its own
ciphertexts / polynomials (independent units: weak scaling, no data-path
collective).

Workload "hmult" (default): one CKKS HMult + relinearise + rescale with
bootparam_40 at the top level 28 (47 Q limbs, 12 auxiliary limbs, 4 digits):
two ciphertexts encrypting 2^15 complex slots uniform in [-1,1]^2, seeded
secret / error / key sampling. A step is one cfhe_hmult call (tensor, ModUp,
inner product with the 118 MiB multiplication key, ModDownAndRescale of both
polynomials). The key plus the temporaries exceed the 126 MB L2, so every step
streams from HBM. The NTT workload is run too and reported under "ntt".

Workload "ntt": batched forward + inverse negacyclic NTT, 16 polynomials x the
first 40 Q limbs (N = 2^16), residues uniform in [0,q); a step is one forward
and one inverse transform of the batch: 16*40*65536*4 B * 2 * 2 = 671 MB of
algorithmic traffic, through three different 168 MB buffers.
"""
import argparse
import concurrent.futures as cf
import importlib.util
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def load_package():
    path = os.path.join(ROOT, "cheddar-fhe_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("cheddar_fhe_b200", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["cheddar_fhe_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


N = 65536
LIMB = N * 4
NTT_POLYS, NTT_LIMBS = 16, 40
NTT_BYTES_PER_STEP = NTT_POLYS * NTT_LIMBS * LIMB * 2 * 2
NTT_BYTES_PER_LAUNCH = NTT_POLYS * NTT_LIMBS * LIMB * 2
HM_LEVEL = 28


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region
    runs (read-only queries)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            time.sleep(0.3)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def make_batch(rng, primes, gidx, polys):
    cols = [rng.integers(0, int(primes[g]), (polys, N), dtype=np.uint64).astype(np.uint32) for g in gidx]
    return np.ascontiguousarray(np.stack(cols, axis=1))


def rand_limbs(rng, primes, gidx):
    return np.stack([rng.integers(0, int(primes[g]), N, dtype=np.uint64).astype(np.uint32) for g in gidx])


# --------------------------------------------------------------------------
# CPU legs (golden model; the reference has no CPU implementation of the path)
# --------------------------------------------------------------------------
def cpu_ntt_sample(params, gidx, polys, threads, seed=0xC0FFEE01):
    from oracle import Oracle
    o = Oracle(params)
    rng = np.random.default_rng(seed)
    a = make_batch(rng, o.primes, gidx, polys)

    def one(p):
        o.intt(o.ntt(a[p], gidx), gidx, mont_keep=True)

    t0 = time.perf_counter()
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(one, range(polys)))
    return time.perf_counter() - t0, polys * len(gidx) * LIMB * 2 * 2


def cpu_hmult_sample(params, count, threads, seed=0xC0FFEE02):
    """`count` independent HMults at level 28 with the golden model on
    `threads` host threads; returns seconds for all of them."""
    from oracle import Oracle
    o = Oracle(params)
    rng = np.random.default_rng(seed)
    g = o.level_limbs(HM_LEVEL)
    T, M = len(params["terminal_primes"]), len(params["main_primes"])
    kg = list(range(T + M)) + [T + M + a for a in range(o.alpha)]
    beta = o.beta(HM_LEVEL)
    kb = [rand_limbs(rng, o.primes, kg) for _ in range(beta)]
    ka = [rand_limbs(rng, o.primes, kg) for _ in range(beta)]
    ins = [rand_limbs(rng, o.primes, g) for _ in range(4)]

    def one(_):
        o.hmult(HM_LEVEL, *ins, kb, ka, M, True)

    t0 = time.perf_counter()
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(one, range(count)))
    return time.perf_counter() - t0


def run_reference(args, pkg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    params = pkg.load_params("bootparam_40.json")
    threads = os.cpu_count() or 1
    if args.workload == "ntt":
        gidx = list(range(NTT_LIMBS))
        polys = max(2, min(NTT_POLYS, threads))
        times = []
        ran_steps, ran_warmup = args.steps, 0
        for _ in range(args.steps):
            dt, nbytes = cpu_ntt_sample(params, gidx, polys, threads)
            times.append(dt)
        dt = float(np.mean(times))
        val, unit, metric, hib = nbytes / dt / 1e9, "GB/s", "NTT GB/s", True
        sample = f"{polys} of {NTT_POLYS} polynomials x {NTT_LIMBS} limbs, forward+inverse, per step"
        workload = "batched fwd+inv negacyclic NTT, N=2^16, 40 limbs (bootparam_40), 16 polynomials"
    else:
        count = threads
        ran_steps = max(1, min(args.steps, 2))   # one step is `threads` HMults, about 2.5 s each
        ran_warmup = 0
        times = [cpu_hmult_sample(params, count, threads) for _ in range(ran_steps)]
        dt = float(np.mean(times)) / count
        val, unit, metric, hib = dt * 1e6, "us", "HMult us", False
        sample = (f"{count} independent HMult+relin+rescale (level 28, random residues) on {threads} "
                  f"threads per step; value = step time / {count}")
        workload = "HMult+relinearise+rescale, bootparam_40 level 28, N=2^16"
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": unit,
        "n_gpus": args.gpus, "steps": ran_steps, "warmup": ran_warmup,
        "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": hib, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": workload, "timed": sample,
                   "note": "the reference has no CPU implementation; this is the scalar C restatement (oracle/)"},
        "cpu_baseline": {"value": val, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------
# GPU legs
# --------------------------------------------------------------------------
def bench_ntt(eng, pkg, torch, steps, warmup, rank, barrier):
    gidx = list(range(NTT_LIMBS))
    rng = np.random.default_rng(0xC0FFEE01 + rank)
    host = make_batch(rng, eng.primes, gidx, NTT_POLYS)
    src = eng.to_dev(host)
    mid = torch.empty_like(src)
    out = torch.empty_like(src)
    pin_in = torch.from_numpy(host.view(np.int32)).pin_memory()
    pin_out = torch.empty_like(pin_in).pin_memory()

    def step():
        eng.ntt_(mid, src, gidx)
        eng.intt_(out, mid, gidx, mont_keep=True)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    assert torch.equal(out, src), "forward+inverse NTT is not the identity"
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    barrier()
    launches0 = pkg.kernel_launch_count()
    for k in range(steps):
        ev[k][0].record()
        eng.ntt_(mid, src, gidx)
        ev[k][1].record()
        eng.intt_(out, mid, gidx, mont_keep=True)
        ev[k][2].record()
    launches = pkg.kernel_launch_count() - launches0
    barrier()
    ms_total = ev[0][0].elapsed_time(ev[-1][2])
    fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
    inv_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in ev]))
    for _ in range(2):
        src.copy_(pin_in, non_blocking=True)
        step()
        pin_out.copy_(out, non_blocking=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        src.copy_(pin_in, non_blocking=True)
        step()
        pin_out.copy_(out, non_blocking=True)
    e1.record()
    barrier()
    return {"ms_step": ms_total / steps, "ms_e2e": e0.elapsed_time(e1) / steps, "fwd_ms": fwd_ms,
            "inv_ms": inv_ms, "h2d": int(src.numel() * 4), "d2h": int(out.numel() * 4), "launches": launches}


# algorithmic bytes of each HMult stage at a level with nq Q limbs, alpha aux
# limbs, digit sizes ds, nd limbs after the rescale and ns limbs dropped by it
# DRAM bytes of each HMult stage measured with ncu (warm L2) at level 28
HMULT_STAGE_TRAFFIC = {"tensor": 60_600_000, "modup_intt": 47_800_000, "modup_bconv": 30_100_000,
                       "modup_ntt": 69_600_000, "inner": 232_400_000, "moddown_intt": 13_200_000,
                       "moddown_bconv": 9_200_000, "moddown_ntt": 64_000_000}


HMULT_TRAFFIC_SOURCE = ("ncu dram read+write of the stage's launches inside one HMult, warm L2 "
                        "(--cache-control none), profiles/hmult_level28_dram_traffic.md")
NTT_KERNEL_NOTE = "ntt_cols_kernel + ntt_rows_kernel, forward (one batch = one column-pass and one row-pass launch)"
NTT_TRAFFIC = 652_600_000
NTT_TRAFFIC_SOURCE = ("ncu dram read+write summed over the two launches of one forward batch, warm L2, "
                      "profiles/ntt_cols_rows_kernels_batch16x40.md")


def hmult_compulsory_bytes(nq, alpha, beta, nd):
    """Bytes an HMult cannot avoid: four input polynomials, the key (both
    halves, beta digits on nq + alpha limbs) and two output polynomials."""
    return (4 * nq + 2 * beta * (nq + alpha) + 2 * nd) * LIMB


def hmult_stage_bytes(nq, alpha, ds, nd, ns):
    ntot = nq + alpha
    conv = sum(ntot - d for d in ds)
    beta = len(ds)
    return {
        "tensor": (4 + 3) * nq * LIMB,
        "modup_intt": 2 * nq * LIMB,
        "modup_bconv": (nq + conv) * LIMB,
        "modup_ntt": 2 * conv * LIMB,
        "inner": (beta * ntot + 2 * beta * ntot + 2 * nq + 2 * ntot) * LIMB,
        "moddown_intt": 2 * 2 * ns * LIMB,
        "moddown_bconv": 2 * (ns + nd) * LIMB,
        "moddown_ntt": 2 * (2 * nd + (nq - (ns - alpha))) * LIMB,
    }


def bench_hmult(eng, pkg, torch, params, steps, warmup, rank, barrier, check):
    client = pkg.client
    level = HM_LEVEL
    M = len(params["main_primes"])
    cl = client.Client(eng, seed=0xC0FFEE02 + rank)
    scale, prods = client.level_scale(params, level)
    rng = np.random.default_rng(0xC0FFEE12 + rank)
    slots = N // 2
    m1 = rng.uniform(-1, 1, slots) + 1j * rng.uniform(-1, 1, slots)
    m2 = rng.uniform(-1, 1, slots) + 1j * rng.uniform(-1, 1, slots)
    b1, a1 = cl.encrypt_message(m1, level, scale)
    b2, a2 = cl.encrypt_message(m2, level, scale)
    kb, ka = cl.mult_key(M)
    dkb = [eng.to_dev(x) for x in kb]
    dka = [eng.to_dev(x) for x in ka]
    host_in = np.ascontiguousarray(np.stack([b1, a1, b2, a2]))
    dev_in = eng.to_dev(host_in)
    nd = len(eng.level_limbs(level - 1))
    dev_out = eng.empty(2, nd, N)
    pin_in = torch.from_numpy(host_in.view(np.int32)).pin_memory()
    pin_out = torch.empty((2, nd, N), dtype=torch.int32).pin_memory()

    def step():
        eng.hmult_(level, dev_out[0], dev_out[1], dev_in[0], dev_in[1], dev_in[2], dev_in[3],
                   dkb, dka, M, True)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    precision_bits = None
    if check and rank == 0:
        out = eng.to_host(dev_out)
        g = eng.level_limbs(level - 1)
        dec = cl.decrypt_message(out[0], out[1], g, scale * scale / prods[level], slots)
        err = np.abs(dec - m1 * m2)
        assert err.max() < 1e-3, f"HMult result is off by {err.max()}"
        precision_bits = float(-np.log2(err.mean()))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = pkg.kernel_launch_count()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    launches = pkg.kernel_launch_count() - launches0
    barrier()
    ms_step = e0.elapsed_time(e1) / steps
    # per-stage device times, CUDA events inside the library on the same stream
    eng.profile_begin()
    for _ in range(steps):
        step()
    stages = {}
    for name, ms in eng.profile_end():
        stages.setdefault(name, []).append(ms)
    stage_ms = {k: float(np.mean(v)) for k, v in stages.items()}
    # end to end: every step copies its ciphertexts from pinned host memory and
    # its result back to the host. The copies run on two side streams with
    # double buffers, so the upload of step t+1 and the download of step t-1
    # overlap the multiplication of step t (PCIe is full duplex); the events
    # order each buffer's upload -> HMult -> download -> next upload.
    compute = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ins = [dev_in, torch.empty_like(dev_in)]
    outs = [dev_out, torch.empty_like(dev_out)]
    pins_out = [pin_out, torch.empty_like(pin_out).pin_memory()]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(count):
        for t in range(count):
            i = t & 1
            with torch.cuda.stream(s_in):
                if t >= 2:
                    s_in.wait_event(comp_done[i])  # the HMult that last read this input buffer
                ins[i].copy_(pin_in, non_blocking=True)
                in_ready[i].record(s_in)
            compute.wait_event(in_ready[i])
            if t >= 2:
                compute.wait_event(out_done[i])  # the download that last read this output buffer
            eng.hmult_(level, outs[i][0], outs[i][1], ins[i][0], ins[i][1], ins[i][2], ins[i][3],
                       dkb, dka, M, True)
            comp_done[i].record(compute)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[i])
                pins_out[i].copy_(outs[i], non_blocking=True)
                out_done[i].record(s_out)
        compute.wait_stream(s_in)
        compute.wait_stream(s_out)

    e2e_steps(4)
    barrier()
    e0.record()
    e2e_steps(steps)
    e1.record()
    barrier()
    if check and rank == 0:
        assert torch.equal(pins_out[(steps - 1) & 1], dev_out.cpu()) or steps < 1, "pipelined result differs"
    return {"ms_step": ms_step, "ms_e2e": e0.elapsed_time(e1) / steps, "stage_ms": stage_ms,
            "h2d": int(dev_in.numel() * 4), "d2h": int(dev_out.numel() * 4),
            "precision_bits": precision_bits, "launches": launches}


def bench_hmult_level(eng, torch, params, level, steps, with_ref):
    """HMult + relinearise + rescale at another level (16 = the default
    encryption level) on random residues and a random key: device-resident
    time of the engine and, when it is built, of the reference's library on the
    same buffers."""
    rng = np.random.default_rng(0xC0FFEE16)
    g = eng.level_limbs(level)
    M, T = len(params["main_primes"]), len(params["terminal_primes"])
    kg = list(range(T + M)) + [T + M + a for a in range(eng.alpha)]
    beta = eng.beta(level)                                  # digits this level uses
    key_digits = eng.beta(len(params["level_config"]) - 1)  # digits a key holds
    ins = [eng.to_dev(rand_limbs(rng, eng.primes, g)) for _ in range(4)]
    kb = [eng.to_dev(rand_limbs(rng, eng.primes, kg)) for _ in range(key_digits)]
    ka = [eng.to_dev(rand_limbs(rng, eng.primes, kg)) for _ in range(key_digits)]
    nd = len(eng.level_limbs(level - 1))
    ob, oa = eng.empty(nd, N), eng.empty(nd, N)
    for _ in range(3):
        eng.hmult_(level, ob, oa, *ins, kb, ka, M, True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        eng.hmult_(level, ob, oa, *ins, kb, ka, M, True)
    e1.record()
    torch.cuda.synchronize()
    nq = len(g)
    out = {"level": level, "us": e0.elapsed_time(e1) / steps * 1e3,
           "compulsory_bytes": (4 * nq + 2 * beta * (nq + eng.alpha) + 2 * nd) * N * 4,
           "note": "inputs, the key limbs of the level and outputs once each; one key and two ciphertexts "
                   "are smaller than L2 at this level, so repeated calls find part of them there"}
    out["GB/s"] = out["compulsory_bytes"] / (out["us"] * 1e-6) / 1e9
    if with_ref:
        try:
            from oracle import ref_binding
            if ref_binding.available():
                ref = ref_binding.Reference(params)
                rb, ra = eng.empty(nd, N), eng.empty(nd, N)
                out["reference_cuda_us"] = ref.hmult(level, rb, ra, *ins, kb, ka, M, True, iters=max(steps, 2))
                out["words_equal_reference"] = bool(torch.equal(rb, ob) and torch.equal(ra, oa))
                ref.close()
        except Exception as exc:  # the reference library is optional
            out["reference_cuda_error"] = str(exc)[:200]
    return out


def bench_reference_cuda(eng, torch, params, steps, with_boot=True):
    """The reference's own CUDA library (oracle/_ref, built unmodified from
    the reference tree) on the same GPU: HMult at level 28 on random residues
    and the config-1 NTT batch, timed with CUDA events inside its driver.
    Reported beside the engine's numbers; absent when the library was not
    built."""
    try:
        from oracle import ref_binding
    except Exception:
        return None
    if not ref_binding.available():
        return None
    ref = ref_binding.Reference(params)
    rng = np.random.default_rng(0xC0FFEE22)
    g = eng.level_limbs(HM_LEVEL)
    M, T = len(params["main_primes"]), len(params["terminal_primes"])
    kg = list(range(T + M)) + [T + M + a for a in range(eng.alpha)]
    beta = eng.beta(HM_LEVEL)
    ins = [eng.to_dev(rand_limbs(rng, eng.primes, g)) for _ in range(4)]
    kb = [eng.to_dev(rand_limbs(rng, eng.primes, kg)) for _ in range(beta)]
    ka = [eng.to_dev(rand_limbs(rng, eng.primes, kg)) for _ in range(beta)]
    nd = len(eng.level_limbs(HM_LEVEL - 1))
    ob, oa = eng.empty(nd, N), eng.empty(nd, N)
    torch.cuda.synchronize()
    hm_us = ref.hmult(HM_LEVEL, ob, oa, *ins, kb, ka, M, True, iters=max(steps, 2))
    mine_b, mine_a = eng.empty(nd, N), eng.empty(nd, N)
    eng.hmult_(HM_LEVEL, mine_b, mine_a, *ins, kb, ka, M, True)
    torch.cuda.synchronize()
    same = bool(torch.equal(mine_b, ob) and torch.equal(mine_a, oa))
    a = eng.to_dev(make_batch(rng, eng.primes, list(range(NTT_LIMBS)), NTT_POLYS))
    b = torch.empty_like(a)
    torch.cuda.synchronize()
    ntt_us = ref.ntt_batch_time(a, b, NTT_POLYS, NTT_LIMBS - T, T, max(steps, 2))
    # config 3: 64 rotations at the top level, unhoisted and with the reference's hoisted baby step
    rots = [1 << i for i in range(15)]
    r3 = np.random.default_rng(0xC0FFEE03)
    while len(rots) < 64:
        r = int(r3.integers(1, N // 2))
        if r not in rots:
            rots.append(r)
    hrot_us, hoisted_us = ref.rotations_time(HM_LEVEL, ins[0], ins[1], kb, ka, M, rots, iters=2)
    ref.close()
    boot = None
    if with_boot:
        torch.cuda.empty_cache()
        boot = ref_binding.boot(params, iters=min(max(steps, 2), 10))
    return {"bootstrap": boot, "hmult_us": hm_us, "hmult_words_equal_engine": same,
            "rotations64_unhoisted_ms": hrot_us / 1e3, "rotations64_hoisted_baby_step_ms": hoisted_us / 1e3,
            "rotations_note": "64 x Context::HRot, and HoistHandler::EvaluateBabyStep (one shared ModUp; its "
                              "outputs stay on the extended basis, no ModDown per rotation)",
            "ntt_fwd_inv_us": ntt_us, "ntt_GBps": NTT_BYTES_PER_STEP / (ntt_us * 1e-6) / 1e9,
            "how": "unmodified reference sources compiled for sm_100a, legacy stream, CUDA events"}


def bench_bootstrap(pkg, local, iters, warmup):
    """Config 4: full bootstrapping of a level-0 ciphertext with 2^15 random
    complex slots (bootparam_40, BootParameter(28, 4, 3)) through the C++
    mirror of the reference API, one bootstrap per GPU per step. The host
    program lib/boot_bench builds the keys and plaintext diagonals (tens of
    seconds, untimed) and times Boot with the host clock around a device
    synchronisation, as the reference's test does."""
    exe = os.path.join(os.path.dirname(pkg.LIB_PATH), "boot_bench")
    if not os.path.exists(exe):
        raise RuntimeError("lib/boot_bench is missing: run the package build")
    env = dict(os.environ)
    visible = env.get("CUDA_VISIBLE_DEVICES")
    env["CUDA_VISIBLE_DEVICES"] = visible.split(",")[local] if visible else str(local)
    r = subprocess.run([exe, os.path.join(pkg.PARAM_DIR, "bootparam_40.json"), "--iters", str(iters),
                        "--warmup", str(warmup)], capture_output=True, text=True, env=env, timeout=900)
    if r.returncode != 0:
        raise RuntimeError("boot_bench failed: " + r.stderr[-500:])
    return json.loads(r.stdout.strip().splitlines()[-1])


def bench_bert_layer(pkg, local, rank=0, world=1, rendezvous=None):
    """Config 5: one encrypted BERT-base encoder layer (128 tokens, hidden 768,
    12 heads of 64, feed-forward 3072; weights N(0, 0.02), activations N(0, 1))
    on 256 sequences at once, one ciphertext per feature, through the C++
    layer driver (host/cheddar/Transformer.h) built on cfhe_ctpt_gemm, hoisted
    rotations, EvalPoly and Boot. The host program lib/bert_bench generates the
    keys, encrypts the 768 input ciphertexts and packs the weights (untimed,
    reported), then times one layer stage by stage with the host clock around
    device synchronisations. With several ranks the ONE layer call is sharded
    over the GPUs by heads and blocks of ciphertexts (NCCL all-gathers between
    the stages, strong scaling); rank 0's process reports. The reference has no
    transformer code, so there is no reference figure."""
    exe = os.path.join(os.path.dirname(pkg.LIB_PATH), "bert_bench")
    if not os.path.exists(exe):
        raise RuntimeError("lib/bert_bench is missing: run the package build")
    env = dict(os.environ)
    visible = env.get("CUDA_VISIBLE_DEVICES")
    env["CUDA_VISIBLE_DEVICES"] = visible.split(",")[local] if visible else str(local)
    cmd = [exe, os.path.join(pkg.PARAM_DIR, "bootparam_40.json"), "--warmup", "1", "--passes", "1"]
    if world > 1:
        cmd += ["--rank", str(rank), "--world", str(world), "--rendezvous", rendezvous]
        env.setdefault("NCCL_DEBUG", "WARN")
        env.setdefault("NCCL_NVLS_ENABLE", "0")  # plain peer transfers: broadcasts gain nothing from multicast
    # A rank that fails leaves the others waiting inside a collective: every rank's
    # process is bounded, and a failure is reported in the line instead of ending the run.
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=420)
    except subprocess.TimeoutExpired:
        return {"error": "bert_bench did not finish within 420 s"} if rank == 0 else None
    if r.returncode != 0:
        return {"error": "bert_bench failed: " + r.stderr[-300:]} if rank == 0 else None
    if rank != 0:
        return None
    return json.loads(r.stdout.strip().splitlines()[-1])


def bert_entry(bert, world):
    """The `bert_layer` object of the line, from rank 0's process: one layer
    call of 256 sequences on all `world` GPUs together (its stage times include
    the waits inside the all-gathers, so they are the job's times)."""
    if "error" in bert:
        return dict(bert)
    peak = None
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            peak = 2.0 * json.load(f)["bf16_tflops"]
    out = dict(bert)
    out["unit"] = f"s per layer call of 256 sequences on {world} GPU(s)"
    out["scaling"] = "strong: one call sharded by heads and ciphertext blocks" if world > 1 else "one GPU"
    out["sequences_per_s"] = bert["sequences_per_layer_call"] / bert["seconds_per_layer"]
    out["projection_tensor_pipe"] = {
        "int8_TOPS": bert["gemm_int8_TOPS"], "peak_TOPS": peak,
        "frac": bert["gemm_int8_TOPS"] / peak if peak else None,
        "peak_source": "2 x measured bf16 burst (MEASURED_PEAKS.json)" if peak else None,
        "share_of_layer_time": bert["gemm_seconds_per_layer"] / bert["seconds_per_layer"]}
    out["parity"] = ("unpinned by the reference (it has no transformer code); tests/test_transformer_gpu.py "
                     "checks the same driver against a float64 layer at reduced width")
    return out


def bench_hoisted(eng, torch, params, n_rot, steps):
    """Config 3: n_rot rotations of one level-28 ciphertext sharing one ModUp
    (power-of-two distances first, then seeded random ones). Keys hold random
    residues below every prime: timing does not depend on their values."""
    rng = np.random.default_rng(0xC0FFEE03)
    level, M = HM_LEVEL, len(params["main_primes"])
    g = eng.level_limbs(level)
    beta = eng.beta(level)
    nkey = len(params["terminal_primes"]) + M + eng.alpha
    rots = [1 << i for i in range(min(15, n_rot))]
    while len(rots) < n_rot:
        r = int(rng.integers(1, N // 2))
        if r not in rots:
            rots.append(r)
    dev = f"cuda:{eng.device}"
    keys = torch.randint(0, 1 << 24, (n_rot, 2, beta, nkey, N), dtype=torch.int32, device=dev)
    kb = [[keys[i, 0, j] for j in range(beta)] for i in range(n_rot)]
    ka = [[keys[i, 1, j] for j in range(beta)] for i in range(n_rot)]
    bx = eng.to_dev(rand_limbs(rng, eng.primes, g))
    ax = eng.to_dev(rand_limbs(rng, eng.primes, g))
    out = eng.empty(n_rot, 2, len(g), N)
    for _ in range(2):
        eng.hoisted_rotations_(level, out, bx, ax, rots, kb, ka, M)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        eng.hoisted_rotations_(level, out, bx, ax, rots, kb, ka, M)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # unhoisted: one full key switch + permutation per rotation
    tmp_b, tmp_a = eng.empty(len(g), N), eng.empty(len(g), N)
    e0.record()
    for i in range(n_rot):
        eng.keyswitch_(level, tmp_b, tmp_a, ax, bx, kb[i], ka[i], M)
        eng.permute_(out[i, 0], tmp_b, None, eng.galois(rots[i]), g)
        eng.permute_(out[i, 1], tmp_a, None, eng.galois(rots[i]), g)
    e1.record()
    torch.cuda.synchronize()
    ms_plain = e0.elapsed_time(e1)
    nbytes = (2 * len(g) + n_rot * 2 * beta * (len(g) + eng.alpha) + n_rot * 2 * len(g)) * LIMB
    return {"rotations": n_rot, "hoisted_ms": ms, "unhoisted_ms": ms_plain,
            "algorithmic_bytes": nbytes, "GB/s": nbytes / (ms * 1e-3) / 1e9,
            "key_bytes_resident": int(keys.numel() * 4)}


def reduce_max(values, device="cpu"):
    """Maximum over ranks of a list of numbers (every rank gets the result).
    Works on whatever process group is initialised: NCCL with CUDA tensors in
    the benchmark, gloo with CPU tensors in the world-size-2 CPU test."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]


def reduce_over_ranks(ntt, hm, boot, hoist, device="cpu"):
    """Every time-like figure of the line is the maximum over ranks."""
    red = {}
    red["ntt_ms"], red["ntt_e2e"], red["fwd_ms"], red["inv_ms"] = reduce_max(
        [ntt["ms_step"], ntt["ms_e2e"], ntt["fwd_ms"], ntt["inv_ms"]], device)
    if hm:
        red["hm_ms"], red["hm_e2e"] = reduce_max([hm["ms_step"], hm["ms_e2e"]], device)
    if boot:
        red["boot_ms"], red["boot_err"] = reduce_max([boot["boot_ms"], boot["mean_err"]], device)
    if hoist:
        red["hoisted_ms"], red["unhoisted_ms"] = reduce_max([hoist["hoisted_ms"], hoist["unhoisted_ms"]], device)
    return red


def assemble_line(args, world, warmup, clocks, red, ntt, hm, hoist, boot, shape):
    """The JSON line rank 0 prints. `red` holds the maxima over ranks, the
    other arguments rank 0's own measurements (used for figures that are not
    times: bytes, stage split, precision); `shape` = limb counts at the HMult
    level. Values aggregate over ranks: `world` units were processed in the
    maximum time."""
    peak, how = measured_peaks()
    ntt_ms, ntt_e2e, fwd_ms, inv_ms = red["ntt_ms"], red["ntt_e2e"], red["fwd_ms"], red["inv_ms"]
    ntt_val = world * NTT_BYTES_PER_STEP / (ntt_ms * 1e-3) / 1e9
    ntt_ach = NTT_BYTES_PER_LAUNCH / (fwd_ms * 1e-3) / 1e9
    ntt_roof = {"bound": "hbm", "kernel": NTT_KERNEL_NOTE,
                "achieved": ntt_ach,
                "peak": peak, "unit": "GB/s", "frac": ntt_ach / peak, "peak_source": how,
                "traffic": NTT_TRAFFIC, "traffic_source": NTT_TRAFFIC_SOURCE,
                "fwd_ms": fwd_ms, "inv_ms": inv_ms,
                "inv_achieved": NTT_BYTES_PER_LAUNCH / (inv_ms * 1e-3) / 1e9}
    if hm:
        hm_ms, hm_e2e = red["hm_ms"], red["hm_e2e"]
        sb = hmult_stage_bytes(shape["nq"], shape["alpha"], [12, 12, 12, 11], shape["nd"], shape["alpha"] + 2)
        stage = {k: {"ms": v, "GB/s": sb[k] / (v * 1e-3) / 1e9 if k in sb else None,
                     "frac": sb[k] / (v * 1e-3) / 1e9 / peak if k in sb else None}
                 for k, v in hm["stage_ms"].items()}
        top = max(hm["stage_ms"], key=hm["stage_ms"].get)
        compulsory = hmult_compulsory_bytes(shape["nq"], shape["alpha"], 4, shape["nd"])
        line = {
            "metric": "HMult us", "value": hm_ms * 1e3 / world, "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": hm_ms,
            "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic",
            "config": {"workload": "HMult+relinearise+rescale, bootparam_40 level 28 (47+12 limbs, 4 digits), "
                                   "N=2^16, 2^15 complex slots uniform in [-1,1]^2, one HMult per GPU per step",
                       "value_is": "step time / n_gpus",
                       "l2": "118 MiB key + 200 MiB of temporaries per step, larger than the 126 MB L2",
                       "parallelism": f"independent ciphertexts x{world}",
                       "e2e_note": "every step uploads its two ciphertexts from pinned host memory and downloads "
                                   "its result; uploads, HMult and downloads run on three streams with double "
                                   "buffers; the multiplication key stays resident"},
            "e2e": {"value": hm_e2e * 1e3 / world, "unit": "us", "h2d_bytes_per_step": hm["h2d"],
                    "d2h_bytes_per_step": hm["d2h"]},
            "gpu_launches": hm["launches"],
            "gpu_launches_note": "kernels the library launched inside the timed region of `value` (counted)",
            "clocks": clocks,
            "precision_bits": hm["precision_bits"],
            "roofline": {"bound": "hbm",
                         "kernel": f"stage {top}",
                         "achieved": stage[top]["GB/s"],
                         "peak": peak, "unit": "GB/s", "frac": stage[top]["frac"], "peak_source": how,
                         "traffic": HMULT_STAGE_TRAFFIC.get(top),
                         "traffic_source": HMULT_TRAFFIC_SOURCE},
            "whole_op": {"compulsory_bytes": compulsory, "GB/s": compulsory / (hm_ms * 1e-3) / 1e9,
                         "frac": compulsory / (hm_ms * 1e-3) / 1e9 / peak,
                         "note": "inputs, key and outputs once each, over the whole HMult"},
            "stages": stage,
            "ntt": {"value": ntt_val, "unit": "GB/s", "ms_per_step": ntt_ms,
                    "e2e": world * NTT_BYTES_PER_STEP / (ntt_e2e * 1e-3) / 1e9, "roofline": ntt_roof,
                    "gpu_launches": ntt["launches"]},
        }
    else:
        line = {
            "metric": "NTT GB/s", "value": ntt_val, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ntt_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic",
            "config": {"workload": "batched fwd+inv negacyclic NTT, N=2^16, 40 limbs (bootparam_40), "
                                   "16 polynomials per GPU",
                       "l2": "three 168 MB buffers per step, larger than L2",
                       "parallelism": f"independent batches x{world}"},
            "e2e": {"value": world * NTT_BYTES_PER_STEP / (ntt_e2e * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": ntt["h2d"], "d2h_bytes_per_step": ntt["d2h"]},
            "gpu_launches": ntt["launches"], "clocks": clocks, "roofline": ntt_roof,
        }
    if hoist:
        h = dict(hoist)
        h["hoisted_ms"], h["unhoisted_ms"] = red["hoisted_ms"], red["unhoisted_ms"]
        h["GB/s"] = h["algorithmic_bytes"] / (h["hoisted_ms"] * 1e-3) / 1e9
        h["frac"] = h["GB/s"] / peak
        h["rotations_per_s_all_ranks"] = world * h["rotations"] / (h["hoisted_ms"] * 1e-3)
        line["hoisted_rotations"] = h
    if boot:
        line["bootstrap"] = {"ms": red["boot_ms"], "unit": "ms per bootstrap (max over ranks)",
                             "bootstraps_per_s": world / (red["boot_ms"] * 1e-3),
                             "precision_bits": -math.log2(red["boot_err"]), "rank0": boot,
                             "workload": "bootparam_40, BootParameter(28,4,3), level 0 -> 13, 2^15 complex "
                                         "slots uniform in [-1,1]^2, one ciphertext per GPU"}
    return line


def bench_gemm(eng, torch, steps, n_in=768, n_out=768, n_limbs=8):
    """Config 5's projection step: y_j = sum_k W[k][j] x_k for 768 input and 768
    output polynomials (one ciphertext polynomial per hidden feature of
    BERT-base) on n_limbs limbs, exact, on the tensor cores (cfhe_ctpt_gemm).
    Inputs are uniform residues (what NTT-domain ciphertext limbs look like),
    weights uniform words standing in for N(0, 0.02) weights times the scale
    reduced modulo each prime (equally uniform)."""
    rng = np.random.default_rng(0xC0FFEE05)
    g = list(range(4, 4 + n_limbs))
    dev = f"cuda:{eng.device}"
    x = torch.randint(0, 1 << 24, (n_in, n_limbs, N), dtype=torch.int32, device=dev)
    y = torch.empty((n_out, n_limbs, N), dtype=torch.int32, device=dev)
    w = np.stack([rng.integers(0, int(eng.primes[gi]), (n_in, n_out), dtype=np.uint64).astype(np.uint32) for gi in g])
    packed = eng.gemm_pack_weights(w, g)
    xs, ys = [x[k] for k in range(n_in)], [y[j] for j in range(n_out)]
    for _ in range(2):
        eng.ctpt_gemm_(ys, xs, packed, g)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        eng.ctpt_gemm_(ys, xs, packed, g)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ops = 2.0 * N * (4 * n_in) * (4 * n_out) * n_limbs       # 8-bit multiply-adds of the byte-plane GEMM, x2
    useful = 2.0 * N * n_in * n_out * n_limbs                # modular multiply-adds, x2
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = None
    if os.path.exists(p):
        with open(p) as f:
            peak = 2.0 * json.load(f)["bf16_tflops"]         # dense 8-bit rate is twice the bf16 rate
    return {"n_in": n_in, "n_out": n_out, "n_limbs": n_limbs, "ms": ms, "int8_TOPS": ops / (ms * 1e-3) / 1e12,
            "modular_GMACs_per_s": useful / 2 / (ms * 1e-3) / 1e9,
            "tensor_peak_TOPS": peak, "peak_source": "2 x measured bf16 burst (MEASURED_PEAKS.json)" if peak else None,
            "frac": ops / (ms * 1e-3) / 1e12 / peak if peak else None,
            "includes": "packing the activations into operand layout (one pass over the inputs per limb)"}


def run_limb_sharded(args, pkg):
    """One HMult (no rescale) at level 28 with the RNS limbs sharded over the
    ranks: rank r owns the limbs at positions r mod G of ciphertexts, key and
    result; all-gathers at the two base conversions (cheddar-fhe_b200/sharded.py).
    Strong scaling of ONE operation: reports its latency at G GPUs, the share
    of the collectives, the same HMult on one GPU, and checks that the gathered
    result equals the one-GPU words."""
    import torch
    import torch.distributed as dist
    import importlib.util
    spec = importlib.util.spec_from_file_location("cfhe_sharded", os.path.join(ROOT, "cheddar-fhe_b200", "sharded.py"))
    sh = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sh)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    params = pkg.load_params("bootparam_40.json")
    eng = pkg.Engine(params, device=local)
    plan = sh.LimbShardPlan(params, HM_LEVEL, world)
    rng = np.random.default_rng(0xC0FFEE44)  # the same data on every rank
    M, T = len(params["main_primes"]), len(params["terminal_primes"])
    g = list(eng.level_limbs(HM_LEVEL))
    kg = list(range(T + M)) + [T + M + a for a in range(eng.alpha)]
    beta = eng.beta(HM_LEVEL)
    ins = [rand_limbs(rng, eng.primes, g) for _ in range(4)]
    kb = [rand_limbs(rng, eng.primes, kg) for _ in range(beta)]
    ka = [rand_limbs(rng, eng.primes, kg) for _ in range(beta)]
    own, own_q = plan.owned(rank), plan.owned_q(rank)
    key_rows = [kg.index(plan.full_g[k]) for k in own]   # rows of the full key that this rank keeps
    mine = [eng.to_dev(x[own_q]) for x in ins]
    kb_own = [eng.to_dev(x[key_rows]) for x in kb]
    ka_own = [eng.to_dev(x[key_rows]) for x in ka]
    warmup = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        out_b, out_a, _ = sh.sharded_hmult(eng, plan, rank, dist, *mine, kb_own, ka_own)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    coll = 0.0
    e0.record()
    for _ in range(args.steps):
        out_b, out_a, c = sh.sharded_hmult(eng, plan, rank, dist, *mine, kb_own, ka_own)
        coll += c
    e1.record()
    barrier()
    ms, coll_ms = reduce_max([e0.elapsed_time(e1) / args.steps, coll * 1e3 / args.steps], f"cuda:{local}")
    # assemble the result on every rank and compare with the one-GPU operator on rank 0
    gathered = [sh.gather_limbs(dist, torch, t, list(range(plan.nq)), plan, rank) for t in (out_b, out_a)]
    same, single_ms = None, None
    if rank == 0:
        full = [eng.to_dev(x) for x in ins]
        dkb, dka = [eng.to_dev(x) for x in kb], [eng.to_dev(x) for x in ka]
        rb, ra = eng.empty(len(g), N), eng.empty(len(g), N)
        for _ in range(warmup):
            eng.hmult_(HM_LEVEL, rb, ra, *full, dkb, dka, M, False)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            eng.hmult_(HM_LEVEL, rb, ra, *full, dkb, dka, M, False)
        e1.record()
        torch.cuda.synchronize()
        single_ms = e0.elapsed_time(e1) / args.steps
        same = all(torch.equal(gathered[0][k], rb[k]) and torch.equal(gathered[1][k], ra[k]) for k in range(plan.nq))
        exchanged = (plan.nq + 2 * plan.alpha) * LIMB
        print(json.dumps({
            "metric": "HMult us (limb-sharded, no rescale)", "value": ms * 1e3, "unit": "us", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": "one HMult + relinearise (ModDown, no rescale), bootparam_40 level 28, limbs "
                                   "sharded by position mod n_gpus, all-gather before each base conversion",
                       "parallelism": f"limbs x{world}"},
            "collective_ms": coll_ms, "collective_share": coll_ms / ms,
            "bytes_exchanged_per_hmult": exchanged,
            "one_gpu_fused_operator_us": single_ms * 1e3,
            "words_equal_one_gpu": bool(same),
            "note": "the sharded path is orchestrated per limb group from Python with the library's fine-grained "
                    "operators (more launches than the fused one-GPU cfhe_hmult), so its one-rank time is above "
                    "the fused operator's"}))
    if world > 1:
        dist.destroy_process_group()


def run_gpu(args, pkg):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        # keep the communicator's set-up lines (ranks, transports) in the log
        os.environ.setdefault("NCCL_DEBUG", "INFO")
        os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    params = pkg.load_params("bootparam_40.json")
    eng = pkg.Engine(params, device=local)
    warmup = max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.workload == "gemm":
        # the projection kernel alone (profiling runs): no other workload is launched
        if rank == 0:
            print(json.dumps({"metric": "ct-pt GEMM", "ctpt_gemm": bench_gemm(eng, torch, args.steps,
                                                                             n_limbs=args.gemm_limbs)}))
        if world > 1:
            dist.destroy_process_group()
        return
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ntt = bench_ntt(eng, pkg, torch, args.steps, warmup, rank, barrier)
    hm = None
    if args.workload == "hmult":
        hm = bench_hmult(eng, pkg, torch, params, args.steps, warmup, rank, barrier, not args.no_check)
    clocks = sampler.stop() if rank == 0 else None
    hoist = None
    if args.workload == "hmult" and not args.no_hoist:
        hoist = bench_hoisted(eng, torch, params, 64, max(2, args.steps // 5))
    gemm = None
    if rank == 0 and args.workload == "hmult" and not args.no_gemm:
        gemm = bench_gemm(eng, torch, max(2, args.steps // 5))
        torch.cuda.empty_cache()
    hm16 = None
    if rank == 0 and args.workload == "hmult":
        hm16 = bench_hmult_level(eng, torch, params, 16, args.steps, world == 1 and not args.no_ref)
        torch.cuda.empty_cache()
    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_ref:
        ref_cuda = bench_reference_cuda(eng, torch, params, args.steps, not args.no_boot)
    boot = None
    if args.workload == "hmult" and not args.no_boot:
        barrier()
        boot = bench_bootstrap(pkg, local, min(max(args.steps, 2), 10), 3)

    bert = None
    if args.workload == "hmult" and not args.no_bert:
        torch.cuda.empty_cache()
        barrier()
        token = [f"/tmp/cfhe_bert_{os.getpid()}_{int(time.time())}"]
        if world > 1:
            dist.broadcast_object_list(token, src=0)
        bert = bench_bert_layer(pkg, local, rank, world, token[0])
        barrier()

    shape = {"nq": len(eng.level_limbs(HM_LEVEL)), "nd": len(eng.level_limbs(HM_LEVEL - 1)), "alpha": eng.alpha}
    red = reduce_over_ranks(ntt, hm, boot, hoist, device=f"cuda:{local}")
    if rank == 0:
        line = assemble_line(args, world, warmup, clocks, red, ntt, hm, hoist, boot, shape)
        if gemm:
            line["ctpt_gemm"] = gemm
        if hm16:
            line["hmult_level16"] = hm16
        if bert:
            line["bert_layer"] = bert_entry(bert, world)
        if ref_cuda:
            line["reference_cuda"] = ref_cuda
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            if hm:
                dt = cpu_hmult_sample(params, 1, 1)
                line["cpu_baseline"] = {"value": dt * 1e6, "unit": "us", "cores": 1, "kind": "port",
                                        "sample": f"1 HMult+relin+rescale at level 28, 1 thread of {threads}"}
            else:
                dt, nbytes = cpu_ntt_sample(params, list(range(NTT_LIMBS)), 2, 1)
                line["cpu_baseline"] = {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                                        "sample": f"2 of 16 polynomials x 40 limbs fwd+inv, 1 thread of {threads}"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="hmult", choices=["hmult", "ntt", "gemm"])
    ap.add_argument("--no-gemm", action="store_true", help="skip the ct-pt GEMM (config 5 projection) leg")
    ap.add_argument("--gemm-limbs", type=int, default=8, help="limbs of the --workload gemm run")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip decrypting the HMult result")
    ap.add_argument("--no-hoist", action="store_true", help="skip the 64-rotation hoisting sweep")
    ap.add_argument("--no-ref", action="store_true", help="skip timing the reference's CUDA library")
    ap.add_argument("--no-boot", action="store_true", help="skip the bootstrapping workload")
    ap.add_argument("--no-bert", action="store_true", help="skip the encrypted transformer layer (about a minute)")
    ap.add_argument("--shard", default="ciphertexts", choices=["ciphertexts", "limbs"],
                    help="limbs: one HMult with its RNS limbs sharded over the ranks (strong scaling)")
    args = ap.parse_args()
    pkg = load_package()
    if args.impl == "reference":
        run_reference(args, pkg)
    elif args.shard == "limbs":
        run_limb_sharded(args, pkg)
    else:
        run_gpu(args, pkg)


if __name__ == "__main__":
    main()
