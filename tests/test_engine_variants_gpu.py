"""The kernel variants that the defaults do not reach, each checked against the oracle by running the convolution parity
cases in a child process with the switch that selects it: the 256-column strip kernel and the 256-filter filter
gradient on single CTAs (the defaults run them on CTA pairs), the filter gradient's tile shapes forced either way, the
first TMA engine (boxes of 32 pixels per tap, the
fallback for filters wider than nine taps), and PERF_OPT on the gather-fed kernels alone."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("switches", [
    {"VDNN_STRIP_PAIRS": "0", "VDNN_WGRAD_PAIRS": "0"},
    {"VDNN_WGRAD_STRIPS": "0"},
    {"VDNN_WGRAD_SHAPE": "tall"},
    {"VDNN_WGRAD_SHAPE": "flat"},
    {"VDNN_TMA_BOXES": "1"},
    {"VDNN_TMA_WGRAD": "0"},
    {"VDNN_NO_TMA": "1"},
], ids=lambda s: "+".join(f"{k}={v}" for k, v in s.items()))
def test_convolution_parity_with_the_other_kernel_variants(switches):
    env = dict(os.environ, **switches)
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_kernels_gpu.py"), "-x", "-q", "-m", "gpu",
           "-k", "convolution_trio and tcgen05", "-p", "no:cacheprovider"]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, cwd=ROOT, timeout=900)
    assert p.returncode == 0, p.stdout[-3000:]
    assert " passed" in p.stdout and "failed" not in p.stdout
