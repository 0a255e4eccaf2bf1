"""Drop-in proof on the GPU: the reference's own attention test programs and benchmark,
compiled unmodified from the reference tree (oracle/Makefile) and linked against
libboat_b200.so, must run and pass."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref")


def run(name, tmp_path):
    path = os.path.join(BIN, name)
    if not os.path.exists(path):
        pytest.skip("%s was not built (needs the reference source tree at build time)" % name)
    proc = subprocess.run([path], cwd=str(tmp_path), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:]
    return proc.stdout


def test_reference_training_test_program(gpu_lib, tmp_path):
    out = run("dropin_test_attention_training", tmp_path)
    losses = [float(x) for x in re.findall(r"Loss = ([0-9.]+)", out)]
    assert len(losses) == 5 and all(b < a for a, b in zip(losses, losses[1:])), out
    # the reference prints 0.324671 for the first iteration when its weights come from the
    # C library's default rand() state, which is how this program starts too
    assert abs(losses[0] - 0.324671) < 5e-6, losses
    assert "completed successfully" in out


def test_reference_gradient_check_program(gpu_lib, tmp_path):
    out = run("dropin_test_attention_gradient_check", tmp_path)
    assert "FAIL" not in out.upper().replace("FAILED: 0", ""), out[-3000:]


def test_reference_benchmark_program(gpu_lib, tmp_path):
    out = run("dropin_attention_performance", tmp_path)
    assert "forward" in out.lower()
