"""Worker for tests/test_dp_gpu.py: one process per GPU under torch.distributed.run.

Each rank trains its shard of a seeded batch with per-layer gradient all-reduce (NCCL, sum) overlapped
with backward; afterwards rank 0 repeats the same steps alone on the whole batch.  Prints one JSON line."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import vdnn_implementation_b200 as vdnn  # noqa: E402
from vdnn_implementation_b200.network import dp_unique_id  # noqa: E402


def fill(fn, *args):
    import ctypes as C
    return fn(*args)


def batches(world, per_rank, steps, in_per_image, classes):
    import ctypes as C
    L = vdnn.lib()
    out = []
    for step in range(steps):
        x = np.empty(world * per_rank * in_per_image, np.float32)
        t = np.empty((world * per_rank, classes), np.float32)
        L.vdnn_host_fill_normal(x.ctypes.data_as(C.c_void_p), x.size, 1000 + step, 0.0, 1.0)
        L.vdnn_host_fill_onehot(t.ctypes.data_as(C.c_void_p), world * per_rank, classes, 2000 + step)
        out.append((x.reshape(world, -1), t.reshape(world, -1)))
    return out


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    model, policy, per_rank, steps, lr = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), float(sys.argv[5])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    net = vdnn.Network(model, policy, "VDNN_PERF_OPT_ALGO", batch_size=per_rank, device=local, pool_bytes=8e9,
                       learning_rate=lr, init_mode=0)
    uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        uid.copy_(torch.frombuffer(bytearray(dp_unique_id()), dtype=torch.uint8))
    dist.broadcast(uid, 0)
    net.enable_dp(rank, world, uid.cpu().numpy().tobytes())
    data = batches(world, per_rank, steps, net.input_size // per_rank, net.output_size // per_rank)
    for x, t in data:
        net.set_input(np.ascontiguousarray(x[rank]), np.ascontiguousarray(t[rank]))
        net.step()
    net.synchronize()
    sums = [None] * world
    dist.all_gather_object(sums, net.weight_checksum())
    stats = net.stats()
    probe_layers = [l for l in range(net.num_layers) if net.tensor_size(l, 2) > 0]
    dp_weights = {l: net.weights(l) for l in (probe_layers[0], probe_layers[len(probe_layers) // 2], probe_layers[-1])}
    dp_bias = {l: net.bias(l) for l in dp_weights}
    status = vdnn.ops.engine_status()
    net.close()
    result = {"checksums": [str(s) for s in sums], "grad_buffer_bytes": stats["grad_buffer_bytes"], "engine_status": status}
    if rank == 0:
        # the same steps on one GPU with the whole batch: sum-of-shard-gradients == gradient of the batch
        one = vdnn.Network(model, policy, "VDNN_PERF_OPT_ALGO", batch_size=per_rank * world, device=local, pool_bytes=8e9,
                           learning_rate=lr, init_mode=0)
        for x, t in data:
            one.set_input(np.ascontiguousarray(x.ravel()), np.ascontiguousarray(t.ravel()))
            one.step()
        one.synchronize()
        errs = []
        for l in dp_weights:
            for a, b in ((dp_weights[l], one.weights(l)), (dp_bias[l], one.bias(l))):
                errs.append(float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)))
        result["max_rel_err_vs_single_gpu"] = max(errs)
        one.close()
        print("DPRESULT " + json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
