"""Per-call timing of the contraction engines on the convolution shapes of VGG16.

    python opbench.py --engine tcgen05 --batch 32
    python opbench.py --engine tcgen05 --batch 32 --layer 5 --op fwd --reps 3   (one kernel, for ncu)

Times vdnn_conv_fwd / vdnn_conv_bwd_data / vdnn_conv_bwd_filter (and, with --op bwd, the three gradients in one call:
vdnn_conv_bwd_data_filter_bias) through the C ABI with CUDA events on the launching stream; PyTorch only owns the
buffers.  Prints algorithmic TFLOP/s (2*M*N*K per call; twice that for bwd).
"""
import argparse

import torch

import vdnn_implementation_b200 as v

SHAPES = [(3, 64, 224), (64, 64, 224), (64, 128, 112), (128, 128, 112), (128, 256, 56), (256, 256, 56),
          (256, 512, 28), (512, 512, 28), (512, 512, 14)]


def timeit(fn, reps):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def elementwise(ops, n, args):
    """ReLU and 2x2/s2 max-pool, forward and backward, on the first VGG16 activation shape (64 x 224 x 224 per image).
    GB/s = algorithmic bytes (each tensor the layer must read or write, once) / time."""
    c, h = 64, 224
    count = n * c * h * h
    x = torch.randn(n, c, h, h, device="cuda")
    y = torch.empty_like(x)
    dy = torch.randn_like(x)
    dx = torch.empty_like(x)
    yp = torch.empty(n, c, h // 2, h // 2, device="cuda")
    dyp = torch.randn_like(yp)
    cases = [
        ("relu_fwd", lambda: ops.relu_fwd(count, x, y), 8.0 * count),
        ("relu_bwd", lambda: ops.relu_bwd(count, y, dy, x, dx), 12.0 * count),
        ("maxpool_fwd", lambda: ops.maxpool_fwd(n, c, h, h, (2, 2), (2, 2), x, yp), 4.0 * (count + count / 4)),
        ("maxpool_bwd", lambda: ops.maxpool_bwd(n, c, h, h, (2, 2), (2, 2), yp, dyp, x, dx), 4.0 * (2 * count + count / 4)),
    ]
    for name, fn, nbytes in cases:
        ms = timeit(fn, args.reps)
        print(f"{name:12s} {count} elements  {ms:7.3f} ms  {nbytes / ms / 1e6:7.0f} GB/s", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--engine", default="tcgen05", choices=["ffma", "tcgen05"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--layer", type=int, default=-1, help="index into the VGG16 shape list; -1 = all")
    ap.add_argument("--op", default="all", choices=["all", "fwd", "dgrad", "wgrad", "bwd", "elementwise"])
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--algo", type=int, default=1, help="0 MEMORY_OPT, 1 PERF_OPT")
    args = ap.parse_args()
    ops = v.ops
    ops.set_engine({"ffma": v.ENGINE_FFMA, "tcgen05": v.ENGINE_TCGEN05}[args.engine])
    n = args.batch
    if args.op == "elementwise":
        return elementwise(ops, n, args)
    total = {"fwd": 0.0, "dgrad": 0.0, "wgrad": 0.0, "bwd": 0.0}
    flops = 0.0
    for idx, (c, k, h) in enumerate(SHAPES):
        if args.layer >= 0 and idx != args.layer:
            continue
        d = ops.conv_desc(n, c, h, h, k, 3, 3, (1, 1), (1, 1))
        x = torch.randn(n, c, h, h, device="cuda")
        w = torch.randn(k, c, 3, 3, device="cuda") * 0.05
        y = torch.empty(n, k, h, h, device="cuda")
        dy = torch.randn(n, k, h, h, device="cuda")
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        bias = torch.zeros(k, device="cuda")
        need = max(ops.conv_workspace_bytes(op, args.algo, d) for op in range(4))
        ws = torch.empty(max(need, 4) // 4, device="cuda")
        calls = {
            "fwd": lambda: ops.conv_fwd(d, x, w, y, bias=bias, algo_mode=args.algo, workspace=ws, workspace_bytes=need),
            "dgrad": lambda: ops.conv_bwd_data(d, w, dy, dx, algo_mode=args.algo, workspace=ws, workspace_bytes=need),
            "wgrad": lambda: ops.conv_bwd_filter(d, x, dy, dw, alpha=-0.01, beta=1.0, algo_mode=args.algo, workspace=ws,
                                                 workspace_bytes=need),
            "bwd": lambda: ops.conv_bwd_data_filter_bias(d, w, x, dy, dx, dw, bias, alpha_w=-0.01, beta_w=1.0, alpha_b=-0.01, beta_b=1.0,
                                                         algo_mode=args.algo, workspace=ws, workspace_bytes=need),
        }
        fl = 2.0 * n * h * h * k * c * 9
        flops += fl
        line = f"conv {c:4d}->{k:4d} @{h:3d}x{h:<3d} batch {n}:"
        for name, fn in calls.items():
            if args.op != name and not (args.op == "all" and name != "bwd"):
                continue
            ms = timeit(fn, args.reps)
            total[name] += ms
            line += f"  {name} {ms:8.3f} ms {(2 if name == 'bwd' else 1) * fl / ms / 1e9:7.1f} TFLOP/s"
        print(line, flush=True)
    for name, ms in total.items():
        if ms > 0:
            print(f"{name}: {ms:.2f} ms, {(2 if name == 'bwd' else 1) * flops / ms / 1e9:.1f} TFLOP/s")
    print("engine status", ops.engine_status())


if __name__ == "__main__":
    main()
