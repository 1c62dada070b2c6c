"""Host-side logic of the data-parallel path on CPU: two gloo ranks, batch sharded across them,
per-layer gradient all-reduce with SUM.  The arithmetic is the CPU oracle's; what is under test is the
rule the CUDA path implements (csrc/network.cu reduceAndApply): gradients of the shards add up to the
gradient of the whole batch, so w += -lr * sum_r grad_r reproduces the single-process update exactly,
and every rank ends with identical parameters."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import rel_err, tiny_net


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, per_rank, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import binding as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the 128-byte communicator id travels from rank 0 to everyone (what bench.py does over NCCL)
        uid = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            uid = torch.arange(128, dtype=torch.uint8)
        dist.broadcast(uid, 0)
        assert uid.tolist() == list(range(128))

        lr = 0.05
        specs = tiny_net(per_rank)
        net = orc.Net(specs, lr, init_mode=0)                 # identical seeded weights on every rank
        for step in range(2):
            before = {l: (net.weights(l), net.bias(l)) for l in range(net.num_layers) if net.weights(l) is not None}
            # rank-specific shard: sample s of rank r is global sample r * per_rank + s of the seeded batch
            full_x = orc.fill_normal(world * net.input_size, 1000 + step).reshape(world, -1)
            full_t = orc.fill_onehot(world * per_rank, 10, 2000 + step).reshape(world, -1)
            net.set_input(full_x[rank], full_t[rank])
            net.forward()
            net.backward()                                    # local fused update: w_r = w - lr * grad_r
            for l, (w0, b0) in before.items():
                for get, old in ((net.weights, w0), (net.bias, b0)):
                    delta = torch.from_numpy(get(l) - old)    # = -lr * grad_r
                    dist.all_reduce(delta, op=dist.ReduceOp.SUM)
                    new = old + delta.numpy()
                    ptr = net._L.orc_net_weights(net.h, l) if get == net.weights else net._L.orc_net_bias(net.h, l)
                    np.ctypeslib.as_array(ptr, shape=(new.size,))[:] = new
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"),
                 **{f"w{l}": net.weights(l) for l in range(net.num_layers) if net.weights(l) is not None},
                 **{f"b{l}": net.bias(l) for l in range(net.num_layers) if net.weights(l) is not None})
    finally:
        dist.destroy_process_group()


def test_sharded_sum_allreduce_equals_one_big_batch(oracle, tmp_path):
    world, per_rank = 2, 2
    mp.spawn(_rank_main, args=(world, _free_port(), per_rank, str(tmp_path)), nprocs=world, join=True)
    r0 = np.load(tmp_path / "rank0.npz")
    r1 = np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), k                # weights identical across ranks, bit for bit
    # single process, whole batch
    lr = 0.05
    net = oracle.Net(tiny_net(world * per_rank), lr, init_mode=0)
    for step in range(2):
        x = oracle.fill_normal(net.input_size, 1000 + step)
        t = oracle.fill_onehot(world * per_rank, 10, 2000 + step)
        net.set_input(x, t)
        net.forward()
        net.backward()
    for l in range(net.num_layers):
        if net.weights(l) is not None:
            assert rel_err(r0[f"w{l}"], net.weights(l)) < 1e-5, l
            assert rel_err(r0[f"b{l}"], net.bias(l)) < 1e-5, l


def test_dry_run_network_accepts_dp_configuration(vdnn):
    net = vdnn.Network("ALEXNET", "VDNN_CONV", "VDNN_MEMORY_OPT_ALGO", device=-1, pool_bytes=8e9)
    try:
        net.enable_dp(1, 2, b"\0" * 128)
        net.step()
        with pytest.raises(vdnn.VdnnError):
            net.enable_dp(2, 2, b"\0" * 128)              # rank out of range
    finally:
        net.close()
