"""The drop-in claim made concrete: the reference's own driver sources (vdnn.cu + network.cu, compiled unmodified by
oracle/build_ref.py with csrc/ref_dropin.h force-included) linked against this library's Layer class.  The build
needs a checkout of the reference; where there is none and no prebuilt binary either, the tests skip."""
import json
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "oracle", "_ref", "vdnn_dropin")
MEMORY = json.load(open(os.path.join(ROOT, "tests", "golden", "ref_memory.json")))


def test_reference_driver_links_against_this_librarys_layer_class():
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/vdnn_dropin not built (no reference checkout at hand)")
    needed = subprocess.run(["ldd", EXE], stdout=subprocess.PIPE, text=True).stdout
    assert "libvdnn_b200.so" in needed
    assert "libcudnn" not in needed and "libcublas" not in needed        # nothing of the reference's libraries is left


@pytest.mark.gpu
@pytest.mark.parametrize("policy", ["BASELINE", "VDNN_ALL", "VDNN_CONV"])
def test_reference_driver_runs_on_this_library_with_the_reference_memory_lines(policy):
    """The stock program, argument parsing, banners and loops of the reference, with every layer computed by this
    library: the per-layer pool figures it prints equal the ones the reference printed on cuDNN (zero-workspace mode,
    where no library-specific workspace size enters)."""
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/vdnn_dropin not built")
    env = dict(os.environ, VDNN_POOL_BYTES=str(60_000_000_000))
    p = subprocess.run([EXE, "ALEXNET", policy, "VDNN_MEMORY_OPT_ALGO"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                       text=True, env=env, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:]
    assert "Elapsed Time:" in p.stdout
    rec = MEMORY[f"ALEXNET/{policy}/VDNN_MEMORY_OPT_ALGO"]
    lines = re.findall(r"\[(Fwd|Bwd)\] Layer (\d+), Free Memory: (\d+), Total Memory: (\d+), Memory Usage: (\d+)", p.stdout)
    fwd = [[int(l), int(t) - int(f), int(u)] for k, l, f, t, u in lines if k == "Fwd"]
    bwd = [[int(l), int(t) - int(f), int(u)] for k, l, f, t, u in lines if k == "Bwd"]
    assert fwd == rec["fwd"] and bwd == rec["bwd"]
