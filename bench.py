#!/usr/bin/env python
"""Benchmark of the CKKS hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload ntt]
    python bench.py --impl reference ...      # CPU golden model on host cores

Prints ONE JSON line (rank 0). Under torchrun every rank processes its own
batch (independent polynomials: weak scaling, no data-path collective).

Workload "ntt" is the batched forward + inverse negacyclic NTT: 16 polynomials
x the first 40 Q limbs of bootparam_40 (N = 2^16), residues uniform in [0,q).
A step is one forward and one inverse transform of the whole batch; the
algorithmic bytes per step are 16*40*65536*4 B * 2 (read+write) * 2 = 671 MB.
Source, intermediate and destination are three different 168 MB buffers, so
every pass streams more than the 126 MB L2.
"""
import argparse
import concurrent.futures as cf
import importlib.util
import json
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


NTT_POLYS, NTT_LIMBS, N = 16, 40, 65536
NTT_BYTES_PER_STEP = NTT_POLYS * NTT_LIMBS * N * 4 * 2 * 2
NTT_BYTES_PER_LAUNCH = NTT_POLYS * NTT_LIMBS * N * 4 * 2


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
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
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


def cpu_ntt_sample(params, gidx, polys, threads, seed=0xC0FFEE01):
    """Golden model (plain C, 64-bit %) on `threads` host threads: forward +
    inverse NTT of `polys` polynomials. Returns (seconds, bytes)."""
    from oracle import Oracle
    o = Oracle(params)
    rng = np.random.default_rng(seed)
    a = make_batch(rng, o.primes, gidx, polys)

    def one(p):
        f = o.ntt(a[p], gidx)
        o.intt(f, gidx, mont_keep=True)

    t0 = time.perf_counter()
    with cf.ThreadPoolExecutor(threads) as ex:
        list(ex.map(one, range(polys)))
    dt = time.perf_counter() - t0
    return dt, polys * len(gidx) * N * 4 * 2 * 2


def run_reference(args, pkg):
    """The reference ships no CPU implementation of this path; this arm times
    the scalar restatement (oracle/) on every host core."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    params = pkg.load_params("bootparam_40.json")
    threads = os.cpu_count() or 1
    gidx = list(range(0, NTT_LIMBS))
    polys = max(2, min(NTT_POLYS, threads))
    for _ in range(min(args.warmup, 1)):
        cpu_ntt_sample(params, gidx, 1, 1)
    times = []
    for _ in range(args.steps):
        dt, nbytes = cpu_ntt_sample(params, gidx, polys, threads)
        times.append(dt)
    dt = float(np.mean(times))
    val = nbytes / dt / 1e9
    sample = f"{polys} of {NTT_POLYS} polynomials x {NTT_LIMBS} limbs, forward+inverse, per step"
    print(json.dumps({
        "impl": "reference", "metric": "NTT GB/s", "value": val, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": "batched fwd+inv negacyclic NTT, N=2^16, 40 limbs (bootparam_40), "
                               "16 polynomials", "timed": sample},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ntt(args, pkg):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    params = pkg.load_params("bootparam_40.json")
    eng = pkg.Engine(params, device=local)
    gidx = list(range(0, NTT_LIMBS))
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    assert torch.equal(out, src), "forward+inverse NTT is not the identity"

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # ---- device-resident throughput
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    t_all0 = torch.cuda.Event(enable_timing=True)
    t_all1 = torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for k in range(args.steps):
        ev[k][0].record()
        eng.ntt_(mid, src, gidx)
        ev[k][1].record()
        eng.intt_(out, mid, gidx, mont_keep=True)
        ev[k][2].record()
    t_all1.record()
    barrier()
    ms_total = t_all0.elapsed_time(t_all1)
    fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
    inv_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in ev]))

    # ---- end to end: pinned host -> device -> fwd+inv -> pinned host
    for _ in range(2):
        src.copy_(pin_in, non_blocking=True)
        step()
        pin_out.copy_(out, non_blocking=True)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        src.copy_(pin_in, non_blocking=True)
        step()
        pin_out.copy_(out, non_blocking=True)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_total, ms_e2e, fwd_ms, inv_ms], device=f"cuda:{local}", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e, fwd_ms, inv_ms = [float(x) for x in t.cpu()]
    if rank == 0:
        peak, how = measured_peaks()
        ms_step = ms_total / args.steps
        value = world * NTT_BYTES_PER_STEP / (ms_step * 1e-3) / 1e9
        e2e = world * NTT_BYTES_PER_STEP / (ms_e2e / args.steps * 1e-3) / 1e9
        achieved = NTT_BYTES_PER_LAUNCH / (fwd_ms * 1e-3) / 1e9
        line = {
            "metric": "NTT GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic",
            "config": {"workload": "batched fwd+inv negacyclic NTT, N=2^16, 40 limbs (bootparam_40), "
                                   "16 polynomials per GPU", "l2": "three 168 MB buffers per step, larger than L2",
                       "parallelism": f"independent batches x{world}"},
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": int(src.numel() * 4),
                    "d2h_bytes_per_step": int(out.numel() * 4)},
            "gpu_launches": 2 * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "ntt_cluster_kernel<forward>",
                         "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": how, "traffic": None,
                         "fwd_ms": fwd_ms, "inv_ms": inv_ms,
                         "inv_achieved": NTT_BYTES_PER_LAUNCH / (inv_ms * 1e-3) / 1e9},
        }
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            dt, nbytes = cpu_ntt_sample(params, gidx, 2, 1)
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
    ap.add_argument("--workload", default="ntt", choices=["ntt"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    args = ap.parse_args()
    pkg = load_package()
    if args.impl == "reference":
        run_reference(args, pkg)
    else:
        run_ntt(args, pkg)


if __name__ == "__main__":
    main()
