"""Worker for tests/test_dp_gpu.py: one process per GPU under torch.distributed.run.

Each rank trains its shard of a seeded batch with per-layer gradient all-reduce (NCCL, sum) overlapped
with backward; afterwards rank 0 repeats the same steps alone on the whole batch.  Prints one JSON line."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vdnn_implementation_b200.network import dp_consistency_check  # noqa: E402


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    model, policy, per_rank, steps, lr = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), float(sys.argv[5])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    result = dp_consistency_check(model, policy, per_rank, steps, lr, dist, local)
    if rank == 0:
        print("DPRESULT " + json.dumps(result), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
