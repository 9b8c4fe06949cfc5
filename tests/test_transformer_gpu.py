"""The encrypted transformer encoder layer (one attention block and one
feed-forward block, with both LayerNorms and the bootstraps between them)
against the float64 layer that evaluates the same Chebyshev series.

Parity unpinned by the reference: the reference has no transformer code
(CMakeLists.txt:63-75 lists every extension source), so the checker is the
textbook layer in double precision (oracle/transformer_plain.h). The bar is
stated in bits: max over every slot of every output ciphertext of
|encrypted - float64| must stay below 2^-12 on outputs of magnitude up to ~5
(the two bootstraps on the way each leave about 2^-19 on values scaled to
[-1, 1], the LayerNorms multiply that by up to 1/sqrt(var_lo))."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
pytestmark = pytest.mark.gpu


def build_transformer_test(pkg):
    if not os.path.exists(pkg.LIB_PATH):
        pkg.build()
    subprocess.check_call(["make", "-s", "-C", CPP, "transformer_test"])
    return os.path.join(CPP, "transformer_test")


@pytest.mark.parametrize("extra", [[], ["--no-pair", "--seed", "7", "--workers", "1"]],
                         ids=["paired-bootstraps-4-host-threads", "single-bootstraps-1-host-thread"])
def test_encrypted_layer_matches_float64_layer(pkg, extra):
    exe = build_transformer_test(pkg)
    cmd = [exe, os.path.join(pkg.PARAM_DIR, "bootparam_40.json")] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    print(r.stdout[-6000:])
    print(r.stderr[-3000:])
    assert r.returncode == 0, "transformer_test failed"
    assert "PASS" in r.stdout
    bits = float(re.search(r"precision_bits ([0-9.]+)", r.stdout).group(1))
    assert bits >= 12.0


def test_bert_base_layer_matches_float64_layer(pkg):
    """The full BERT-base shape (128 tokens, hidden 768, 12 heads, feed-forward
    3072; weights N(0, 0.02), activations N(0, 1)), 256 sequences encrypted,
    the first two compared slot by slot with the float64 layer; the test also
    fails when any value leaves the interval its series was fitted on."""
    exe = build_transformer_test(pkg)
    r = subprocess.run([exe, os.path.join(pkg.PARAM_DIR, "bootparam_40.json"), "--base"], capture_output=True,
                       text=True, timeout=1500)
    print(r.stdout[-6000:])
    print(r.stderr[-3000:])
    assert r.returncode == 0, "transformer_test --base failed"
    assert "PASS" in r.stdout
    assert float(re.search(r"precision_bits ([0-9.]+)", r.stdout).group(1)) >= 12.0
