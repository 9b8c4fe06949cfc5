"""One layer call of the encrypted transformer sharded over two GPUs (heads
and blocks of ciphertexts per rank, NCCL all-gathers between the stages) must
leave exactly the ciphertext words a one-GPU call leaves: every rank starts
from the same keys and inputs (seeded device sampling) and all arithmetic is
exact. Skipped on a box with one GPU."""
import json
import os
import subprocess
import tempfile

import pytest

pytestmark = pytest.mark.gpu


def _run(exe, params, extra, env, out):
    with open(out, "w") as f:
        return subprocess.Popen([exe, params, "--small", "--warmup", "0"] + extra, stdout=f,
                                stderr=subprocess.DEVNULL, env=env)


def test_two_ranks_leave_the_words_of_one(pkg):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    exe = os.path.join(os.path.dirname(pkg.LIB_PATH), "bert_bench")
    params = os.path.join(pkg.PARAM_DIR, "bootparam_40.json")
    base = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    with tempfile.TemporaryDirectory() as tmp:
        one = os.path.join(tmp, "one.json")
        assert _run(exe, params, [], dict(base, CUDA_VISIBLE_DEVICES="0"), one).wait(timeout=600) == 0
        rv = os.path.join(tmp, "rendezvous")
        outs = [os.path.join(tmp, f"two_{r}.json") for r in range(2)]
        procs = [_run(exe, params, ["--rank", str(r), "--world", "2", "--rendezvous", rv],
                      dict(base, CUDA_VISIBLE_DEVICES=str(r)), outs[r]) for r in range(2)]
        try:
            codes = [p.wait(timeout=600) for p in procs]
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
        assert codes == [0, 0]
        a = json.loads([l for l in open(one) if l.startswith("{")][0])
        b = json.loads([l for l in open(outs[0]) if l.startswith("{")][0])
    assert a["gpus"] == 1 and b["gpus"] == 2
    assert a["output_digest"] == b["output_digest"]
    assert any(k.startswith("all-gather") for k in b["stages_s"])
