"""The C++ host layer (planner, NvidiaBackend, Runtime, KernelCache, vendor dispatch): its own test
executable, built by cantors-gift_b200/build.py, run here in its CPU and GPU modes."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "cantors-gift_b200", "lib", "host_tests")


def _run(mode):
    if not os.path.exists(EXE):
        pytest.fail(f"{EXE} missing: run `python __graft_entry__.py` (build) first")
    r = subprocess.run([EXE, mode], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout


def test_host_layer_cpu():
    _run("cpu")


@pytest.mark.gpu
def test_host_layer_gpu():
    _run("gpu")
