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


def _two_shot_rank(rank, world, port, count, out_dir):
    """The partition arithmetic of the fused peer all-reduce (csrc/dp_peer.cu), replayed on CPU ranks over gloo: rank r
    reduces the slice vdnn_dp_slice gives it -- the contributions of all ranks added in rank order -- and the reduced
    slices are then handed to everybody."""
    import ctypes as C
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import vdnn_implementation_b200 as v
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        padded = (count + 3) // 4 * 4                     # staging buffers are padded to whole groups of 4 floats
        mine = np.zeros(padded, np.float32)
        mine[:count] = np.random.default_rng(100 + rank).standard_normal(count).astype(np.float32)
        everyone = [torch.zeros(padded) for _ in range(world)]
        dist.all_gather(everyone, torch.from_numpy(mine))                       # "peer-mapped arenas"
        b, e = C.c_size_t(), C.c_size_t()
        assert v.lib().vdnn_dp_slice(count, world, rank, C.byref(b), C.byref(e)) == 0
        assert b.value % 4 == 0 and e.value % 4 == 0 and b.value <= e.value <= padded
        reduced = np.zeros(e.value - b.value, np.float32)
        for r in range(world):                                                   # rank order, as the kernel adds
            reduced += everyone[r].numpy()[b.value:e.value]
        bounds = [None] * world
        dist.all_gather_object(bounds, (b.value, e.value))
        assert bounds[0][0] == 0 and bounds[-1][1] == padded                     # the slices tile the buffer ...
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))   # ... without gap or overlap
        pieces = [None] * world
        dist.all_gather_object(pieces, reduced)                                  # "stores into every peer's arena"
        total = np.concatenate(pieces)
        want = torch.from_numpy(mine.copy())
        dist.all_reduce(want, op=dist.ReduceOp.SUM)
        np.save(os.path.join(out_dir, f"two_shot_{count}_{rank}.npy"), np.stack([total, want.numpy()]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,count", [(2, 1000), (2, 7), (3, 4097), (4, 2)])
def test_two_shot_slices_cover_the_gradient_and_sum_like_allreduce(vdnn, tmp_path, world, count):
    mp.spawn(_two_shot_rank, args=(world, _free_port(), count, str(tmp_path)), nprocs=world, join=True)
    results = [np.load(tmp_path / f"two_shot_{count}_{r}.npy") for r in range(world)]
    for r in range(world):
        assert np.array_equal(results[r][0], results[0][0])                      # every rank ends with the same bits
        assert np.allclose(results[r][0], results[r][1], rtol=1e-6, atol=1e-6)   # and with the all-reduce sum
