"""World-size-2 check of the multi-rank bench logic on CPU (gloo): ranks work
on independent units, the step time is the maximum over ranks, and only rank 0
reports. No GPU and no CUDA library call is involved."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent("""
    import os, json, sys
    import torch, torch.distributed as dist
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # per-rank "step time": rank r pretends to need (r+1) ms; units are independent
    t = torch.tensor([float(rank + 1), 2.0 * (rank + 1)], dtype=torch.float64)
    dist.barrier()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t[0])
        print(json.dumps({"n_gpus": world, "ms_per_step": ms, "value": ms * 1e3 / world,
                          "scaling": "weak"}))
    dist.destroy_process_group()
""")


def test_two_ranks_report_max_time_from_rank0(tmp_path):
    script = tmp_path / "two_ranks.py"
    script.write_text(SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout  # only rank 0 prints
    import json
    j = json.loads(lines[0])
    assert j["n_gpus"] == 2 and j["ms_per_step"] == 2.0 and j["value"] == 1000.0


def test_reference_arm_runs_on_rank0_only():
    """bench.py --impl reference under a 2-rank launch: rank 1 exits at once,
    rank 0 prints one line carrying impl=reference."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=120, env=env, cwd=ROOT)
    assert r.returncode == 0 and r.stdout.strip() == ""
