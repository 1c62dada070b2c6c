"""Data-parallel training on two GPUs of one box (skipped where fewer are visible): weights identical
across ranks after several steps, and equal (to rounding) to one GPU training on the whole batch."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("fused", [0, 1])
@pytest.mark.parametrize("model,policy,per_rank,steps,lr", [("ALEXNET", "VDNN_CONV", 4, 10, 0.01), ("VGG16_64", "VDNN_ALL", 2, 1, 1e-4)])
def test_two_gpu_data_parallel(vdnn, model, policy, per_rank, steps, lr, fused):
    """fused = 0: per-layer NCCL all-reduce + axpy; fused = 1: the peer-memory kernel that reduces, gathers and applies the
    SGD step in one launch (plain loads / stores over NVLink, bounded flag waits; NVLS off, no multimem)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_port()), os.path.join(HERE, "dp_worker.py"), model, policy, str(per_rank), str(steps), str(lr)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", VDNN_DP_FUSED=str(fused))
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:]
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("DPRESULT ")][-1]
    r = json.loads(line[len("DPRESULT "):])
    assert len(set(r["checksums"])) == 1, r                   # bit-identical weights on both ranks
    assert r["max_rel_err_vs_single_gpu"] < 1e-4, r
    assert r["grad_buffer_bytes"] > 0 and r["engine_status"] == 0
    assert r["dp_mode"] == (2 if fused else 1), r
