"""World-size-2 check of the multi-rank bench logic on CPU (gloo): bench.py's
own reduction over ranks and its assembly of the JSON line run on two ranks
with made-up per-rank measurements. Ranks work on independent units, every
time is the maximum over ranks, and only rank 0 reports. No GPU and no CUDA
library call is involved."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import argparse, json, os, sys
    sys.path.insert(0, os.environ["BENCH_ROOT"])
    import torch.distributed as dist
    import bench                      # the benchmark's own reduction and line assembly
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # per-rank measurements: rank r pretends to be (r + 1) times slower
    k = float(rank + 1)
    ntt = {"ms_step": 0.4 * k, "ms_e2e": 40.0 * k, "fwd_ms": 0.2 * k, "inv_ms": 0.21 * k,
           "h2d": 1, "d2h": 1, "launches": 20}
    hm = {"ms_step": 0.2 * k, "ms_e2e": 1.0 * k, "stage_ms": {"tensor": 0.02, "modup_ntt": 0.05},
          "h2d": 49283072, "d2h": 23592960, "precision_bits": 25.0, "launches": 14}
    boot = {"boot_ms": 9.0 * k, "mean_err": 2.0 ** -22 * k}
    hoist = {"rotations": 64, "hoisted_ms": 6.0 * k, "unhoisted_ms": 13.0 * k,
             "algorithmic_bytes": 9_000_000_000, "GB/s": 0.0, "key_bytes_resident": 1}
    dist.barrier()
    red = bench.reduce_over_ranks(ntt, hm, boot, hoist)
    if rank == 0:
        args = argparse.Namespace(steps=20, warmup=5)
        shape = {"nq": 47, "nd": 45, "alpha": 12}
        print(json.dumps(bench.assemble_line(args, world, 5, None, red, ntt, hm, hoist, boot, shape)))
    dist.destroy_process_group()
""")


def test_two_ranks_report_max_time_from_rank0(tmp_path):
    """Runs bench.py's reduce_over_ranks and assemble_line on two gloo ranks:
    every time in the line is the slower rank's, values count both ranks'
    units, and only rank 0 prints."""
    script = tmp_path / "two_ranks.py"
    script.write_text(SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", BENCH_ROOT=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout  # only rank 0 prints
    import json
    import math
    j = json.loads(lines[0])
    assert j["n_gpus"] == 2 and j["scaling"] == "weak"
    assert j["ms_per_step"] == 0.4                      # the slower rank's HMult step
    assert j["value"] == 0.4 * 1e3 / 2                  # two HMults in that time
    assert j["e2e"]["value"] == 2.0 * 1e3 / 2
    assert j["ntt"]["ms_per_step"] == 0.8 and j["ntt"]["roofline"]["fwd_ms"] == 0.4
    assert j["hoisted_rotations"]["hoisted_ms"] == 12.0  # reduced over ranks like the other legs
    assert j["hoisted_rotations"]["unhoisted_ms"] == 26.0
    assert j["bootstrap"]["ms"] == 18.0 and abs(j["bootstrap"]["bootstraps_per_s"] - 2 / 18e-3) < 1e-6
    assert abs(j["bootstrap"]["precision_bits"] - 21.0) < 1e-9  # the worse rank's error
    assert j["gpu_launches"] == 14
    assert math.isclose(j["whole_op"]["compulsory_bytes"], (4 * 47 + 2 * 4 * 59 + 2 * 45) * 65536 * 4)


def test_reference_arm_runs_on_rank0_only():
    """bench.py --impl reference under a 2-rank launch: rank 1 exits at once,
    rank 0 prints one line carrying impl=reference."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=120, env=env, cwd=ROOT)
    assert r.returncode == 0 and r.stdout.strip() == ""
