"""Partition logic of the limb-sharded HMult on two gloo ranks (CPU): every
limb has exactly one owner, the digits and pre-scale constants agree with the
engine's level plan as the golden model sees it, and the padded all-gather
returns every rank's limbs to everyone in the right places. No GPU involved."""
import importlib.util
import os
import subprocess
import sys
import textwrap

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_sharded():
    spec = importlib.util.spec_from_file_location("cfhe_sharded", os.path.join(ROOT, "cheddar-fhe_b200", "sharded.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_plan_matches_the_golden_model(pkg):
    from oracle import Oracle
    sh = load_sharded()
    p = pkg.load_params("bootparam_40.json")
    o = Oracle(p)
    for level in (28, 16, 5, 1):
        for world in (1, 2, 4, 8):
            plan = sh.LimbShardPlan(p, level, world)
            assert plan.q_g == list(o.level_limbs(level))
            assert plan.full_g == list(o.level_limbs(level, plan.alpha))
            assert len(plan.digits) == o.beta(level) or level < 5  # low levels have inactive digits
            owners = [plan.owned(r) for r in range(world)]
            assert sorted(sum(owners, [])) == list(range(plan.ntot))
            for k in range(plan.ntot):
                assert plan.q(k) == int(o.primes[plan.full_g[k]])
            covered = sorted(k for (_, s0, s1) in plan.digits for k in range(s0, s1))
            assert covered == list(range(plan.nq))
            pre = {}
            for d in plan.digits:
                pre.update(plan.modup_prescale(d))
            n = 1 << p["log_degree"]
            for (_, s0, s1) in plan.digits:
                for k in range(s0, s1):
                    shat = n
                    for i in range(s0, s1):
                        if i != k:
                            shat *= plan.q(i)
                    assert pre[k] * shat % plan.q(k) == 1


SCRIPT = textwrap.dedent("""
    import importlib.util, json, os, sys
    import torch, torch.distributed as dist
    root = os.environ["BENCH_ROOT"]
    spec = importlib.util.spec_from_file_location("cfhe_sharded", os.path.join(root, "cheddar-fhe_b200", "sharded.py"))
    sh = importlib.util.module_from_spec(spec); spec.loader.exec_module(sh)
    with open(os.path.join(root, "cheddar-fhe_b200", "parameters", "bootparam_40.json")) as f:
        p = json.load(f)
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    plan = sh.LimbShardPlan(p, 28, world)
    n = 64
    positions = list(range(plan.nq, plan.ntot))          # the auxiliary limbs, as ModDown gathers them
    mine = [k for k in positions if plan.owner(k) == rank]
    local = torch.stack([torch.full((n,), 1000 * k + rank, dtype=torch.int32) for k in mine])
    got = sh.gather_limbs(dist, torch, local, positions, plan, rank)
    ok = tuple(got.shape) == (len(positions), n) and all(
        int(got[i][0]) == 1000 * k + plan.owner(k) and int(got[i][n - 1]) == 1000 * k + plan.owner(k)
        for i, k in enumerate(positions))
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"ok": bool(flag.item()), "world": world, "gathered": len(got)}))
    dist.destroy_process_group()
""")


def test_gather_on_two_gloo_ranks(tmp_path):
    script = tmp_path / "gather.py"
    script.write_text(SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", BENCH_ROOT=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
                       capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    import json
    j = json.loads(lines[0])
    assert j == {"ok": True, "world": 2, "gathered": 12}
