"""The shipped example must run: two gloo ranks on CPU here, one rank on a GPU in the gpu tier."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = ["--batch-size", "16", "--hidden", "256", "--intermediate", "128", "--experts", "8", "--top-k", "2"]


def _run(extra, env=None):
    cmd = [sys.executable, "-m", "umdk_original_b200.examples.fused_deep_moe_sample", *SMALL, *extra]
    return subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env=env)


@pytest.mark.multi_process_test
def test_example_two_cpu_ranks():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = _run(["--world", "2", "--with-mask"], env)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--with-mask"], ["--dynamic-eplb"]])
def test_example_one_gpu(extra):
    r = _run(["--world", "1", *extra])
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
