#!/usr/bin/env python
"""Benchmark of the vDNN training hot path on B200.

    python bench.py --gpus N --steps K --warmup W            this library (CUDA, sm_100a)
    python bench.py --impl reference --steps K --warmup W    the reference program itself (oracle/_ref, cuDNN build)
                                                             where it was built, else the CPU restatement

One "step" is forward + backward (SGD folded into backward) of the named network under the named
vDNN policy on one synthetic batch per GPU.  Prints ONE JSON line on rank 0.

  value     images/s over all ranks, batch already resident in HBM, CUDA-event time, max over ranks
  e2e       the same through the public API with the batch in pinned host memory: every step uploads
            input + labels and reads the loss back
  roofline  CONV/FC contraction layers: algorithmic FLOP/s achieved over the timed region
  cpu_baseline  the CPU restatement of the same layer math on this box's host cores (bounded sample)
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODELS = {"ALEXNET": (128, 227), "ALEXNET_LRN": (128, 227), "OVERFEAT": (128, 231), "VGG16_64": (64, 224),
          "VGG16_128": (128, 224), "VGG16_256": (256, 224)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="VGG16_128", choices=sorted(MODELS))
    ap.add_argument("--policy", default="VDNN_ALL", choices=["BASELINE", "VDNN_NONE", "VDNN_ALL", "VDNN_CONV"])
    ap.add_argument("--algo", default="VDNN_PERF_OPT_ALGO", choices=["VDNN_MEMORY_OPT_ALGO", "VDNN_PERF_OPT_ALGO"])
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (0 = the model's own)")
    ap.add_argument("--pool-gb", type=float, default=24.0, help="device pool capacity (BASELINE config: 24 GB cap)")
    ap.add_argument("--lr", type=float, default=1e-6,
                    help="SGD rate for one GPU (divided by the world size under data parallelism).  The reference's constant is "
                         "1e-5 (vdnn.h:8); gradients are batch sums, and on this seeded He-normal VGG16 that rate makes the loss "
                         "rise from the first steps on, 1e-6 makes it fall")
    ap.add_argument("--engine", default="auto", choices=["auto", "ffma", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-warm", action="store_true", help="skip the warm runs of the reference's own Network")
    ap.add_argument("--no-by-policy", action="store_true", help="skip the short VDNN_NONE / VDNN_CONV measurements")
    ap.add_argument("--no-probes", action="store_true", help="skip the TF32 tensor-pipe and PCIe copy-rate probes")
    ap.add_argument("--no-dp-check", action="store_true", help="skip the data-parallel == single-GPU check (world > 1)")
    ap.add_argument("--reference-kind", default="auto", choices=["auto", "cpu"],
                    help="--impl reference: auto = the built reference program when present and a GPU is visible, else the CPU port")
    ap.add_argument("--cpu-batch", type=int, default=0, help="images in the CPU sample (0 = sized for ~10-30 s)")
    return ap.parse_args()


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops_sustained"], "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "tflops": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------ CPU arm
def cpu_step_rate(model, batch, steps, warmup, lr):
    """Times the CPU restatement (float accumulation build, all host threads) on `batch` images."""
    from oracle import binding as orc
    specs = orc.model_layers(getattr(orc, model), batch)
    net = orc.Net(specs, lr, init_mode=0, f32=True)
    rows = batch
    x = orc.fill_normal(net.input_size, 1000)
    t = orc.fill_onehot(rows, net.output_size // rows, 2000)
    net.set_input(x, t)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        net.forward()
        net.backward()
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    net.close()
    return batch / (sum(times) / len(times)), sum(times) / len(times)


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference_binary(args, exe):
    """One forward + backward of the unmodified reference program per step; it times itself (vdnn.cu:72-79:
    wall clock around forwardPropagation + backwardPropagation, host-side input generation included) and
    prints microseconds.  Returns (images/s, mean seconds, steps used) or None if it could not run."""
    import re
    batch = MODELS[args.model][0]
    env = dict(os.environ, VDNN_POOL_BYTES=str(int(max(args.pool_gb, 24.0) * 1e9)))
    runs = max(1, min(args.steps, 5))           # every run re-initialises the network (seconds): keep the arm bounded
    warm = 1 if args.warmup > 0 else 0
    times = []
    for i in range(warm + runs):
        try:
            out = subprocess.run([exe, args.model, args.policy, args.algo], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                 text=True, env=env, timeout=600).stdout
        except Exception:
            return None
        m = re.search(r"Elapsed Time: (\d+)", out)
        if not m:
            return None
        if i >= warm:
            times.append(int(m.group(1)) / 1e6)
    mean = sum(times) / len(times)
    return batch / mean, mean, runs, warm


def run_reference(args):
    """Reference arm.  When the reference was built here (oracle/_ref/vdnn_ref, its unmodified sources on
    cuDNN / cuBLAS) and a GPU is present, the reference program itself is run and timed by its own clock.
    Otherwise the CPU restatement of the same layer math (oracle port) is timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    exe = os.path.join(ROOT, "oracle", "_ref", "vdnn_ref")
    res = None
    import shutil
    has_gpu = bool(shutil.which("nvidia-smi")) and subprocess.run(["nvidia-smi", "-L"], stdout=subprocess.DEVNULL,
                                                                 stderr=subprocess.DEVNULL).returncode == 0
    if os.path.exists(exe) and has_gpu and args.reference_kind != "cpu":
        res = run_reference_binary(args, exe)
    cores = host_threads()
    if res:
        value, step_s, runs, warm = res
        batch = MODELS[args.model][0]
        line = {
            "impl": "reference", "metric": "train images/s", "value": value, "unit": "images/s", "n_gpus": 1,
            "steps": runs, "warmup": warm, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.model} {args.policy} {args.algo}, batch {batch}, the reference program on cuDNN/cuBLAS "
                                   f"(one iteration per process, timed by its own clock incl. host input generation)"},
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": 1, "kind": "reference",
                             "sample": f"{runs} runs of oracle/_ref/vdnn_ref {args.model} {args.policy} {args.algo} (unmodified reference "
                                       f"sources, cuDNN default math, one host thread driving the same GPU)"},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line), flush=True)
        return
    batch = args.cpu_batch or 1
    value, step_s = cpu_step_rate(args.model, batch, max(args.steps, 1), min(args.warmup, 1), args.lr)
    line = {
        "impl": "reference", "metric": "train images/s", "value": value, "unit": "images/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.model} forward+backward+SGD on host cores, batch {batch} per step "
                               f"(bounded sample of the batch-{MODELS[args.model][0]} workload)"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port",
                         "sample": f"{args.model} batch {batch}, {args.steps} steps, OpenMP over {cores} threads"},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.proc = None
        self.device = device

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.device), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def pcie_probe(torch, device, mib=1024, reps=3):
    """Pinned-memory copy rates of this GPU's link: device->host alone, host->device alone, both at once (GB/s)."""
    n = mib << 20
    h_out = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    h_in = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    h_in.zero_(); h_out.zero_()
    d_src = torch.zeros(n, dtype=torch.uint8, device=device)
    d_dst = torch.empty(n, dtype=torch.uint8, device=device)
    s_out, s_in = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(out, inn):
        best = [0.0, 0.0]
        for _ in range(reps):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            torch.cuda.synchronize()
            if out:
                with torch.cuda.stream(s_out):
                    ev[0].record(); h_out.copy_(d_src, non_blocking=True); ev[1].record()
            if inn:
                with torch.cuda.stream(s_in):
                    ev[2].record(); d_dst.copy_(h_in, non_blocking=True); ev[3].record()
            torch.cuda.synchronize()
            if out:
                best[0] = max(best[0], n / ev[0].elapsed_time(ev[1]) / 1e6)
            if inn:
                best[1] = max(best[1], n / ev[2].elapsed_time(ev[3]) / 1e6)
        return best

    run(True, True)                                   # first touch of the pinned pages
    d2h, h2d = run(True, False)[0], run(False, True)[1]
    both = run(True, True)
    return {"d2h_alone_gbs": d2h, "h2d_alone_gbs": h2d, "d2h_with_h2d_gbs": both[0], "h2d_with_d2h_gbs": both[1],
            "pcie_how": f"{mib} MiB pinned <-> device copies on two streams, best of {reps}, CUDA events"}


def tf32_probe(torch, vdnn, stream):
    """Dense TF32 rate of the tensor pipe: the library's probe kernel (MMAs on resident operands, no loads), as one
    short launch (burst) and back to back for about two seconds (sustained, under the power cap)."""
    ops = vdnn.ops

    def once(iters, launches):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flops = 0.0
        a.record(stream)
        for _ in range(launches):
            flops += ops.engine_mma_rate_probe(iters, stream.cuda_stream)
        b.record(stream)
        torch.cuda.synchronize()
        return flops / (a.elapsed_time(b) / 1e3) / 1e12

    once(2000, 1)
    burst = max(once(20000, 1) for _ in range(3))                    # ~25 ms each
    sustained = once(20000, 80)                                      # ~2 s back to back
    assert ops.engine_status() == 0
    return {"tf32_dense_tflops_burst": burst, "tf32_dense_tflops_sustained": sustained,
            "tf32_how": "vdnn_engine_mma_rate_probe: one CTA per SM issuing tcgen05.mma kind::tf32 128x256x8 on resident operands"}


def reference_warm(args, policies):
    """The reference's own Network (oracle/_ref/ref_warm: its unmodified sources on cuDNN / cuBLAS) iterated in one
    process: warm steps, host-side input generation measured and subtracted.  cuDNN default math (TF32 allowed for
    fp32 convolutions on this architecture) and FMA math (NVIDIA_TF32_OVERRIDE=0)."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_warm")
    if not os.path.exists(exe):
        return {"unavailable": "oracle/_ref/ref_warm not built (reference sources were not at hand)"}
    import tempfile
    out = {}
    for policy in policies:
        for math, override in (("default_math", None), ("fma_math", "0")):
            env = dict(os.environ, VDNN_POOL_BYTES=str(int(max(args.pool_gb, 24.0) * 1e9)))
            env.pop("NVIDIA_TF32_OVERRIDE", None)
            if override is not None:
                env["NVIDIA_TF32_OVERRIDE"] = override
            with tempfile.NamedTemporaryFile(suffix=".json") as tmp:
                try:
                    rc = subprocess.run([exe, args.model, policy, args.algo, "10", "2", tmp.name], stdout=subprocess.DEVNULL,
                                        stderr=subprocess.PIPE, text=True, env=env, timeout=300)
                    if rc.returncode != 0:
                        out[f"{policy}/{math}"] = {"failed": rc.stderr[-300:]}
                        continue
                    r = json.load(open(tmp.name))
                except Exception as e:                      # noqa: BLE001
                    out[f"{policy}/{math}"] = {"failed": repr(e)[:300]}
                    continue
            out[f"{policy}/{math}"] = {"images_per_s": r["images_per_s"], "ms_per_step": r["net_ms_mean"],
                                       "wall_ms_per_step": r["wall_ms_mean"], "host_input_generation_ms": r["rng_ms_mean"],
                                       "steps": r["iterations"], "warmup": r["warmup"]}
    out["how"] = ("oracle/_ref/ref_warm MODEL POLICY ALGO 10 2: the reference's forwardPropagation + backwardPropagation per step, "
                  "cudaDeviceSynchronize + wall clock around each, minus the measured host-side input/label generation")
    return out


def profile_traffic():
    """Measured DRAM bytes per launch of the dominant kernel, from the committed ncu summary (a line
    `roofline.traffic_bytes_per_launch = N` in a file under profiles/); None when no summary states it."""
    import glob
    import re
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        m = re.search(r"roofline\.traffic_bytes_per_launch\s*=\s*(\d+)", open(path).read())
        if m:
            return int(m.group(1)), os.path.basename(path)
    return None, None


def run_b200(args):
    import torch
    import torch.distributed as dist
    import vdnn_implementation_b200 as vdnn
    from vdnn_implementation_b200.network import dp_unique_id, dp_consistency_check
    import ctypes as C
    import math

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    vdnn.ops.set_engine({"auto": vdnn.ENGINE_AUTO, "ffma": vdnn.ENGINE_FFMA, "tcgen05": vdnn.ENGINE_TCGEN05}[args.engine])
    L = vdnn.lib()
    batch = args.batch or MODELS[args.model][0]
    # Gradients are batch sums and the all-reduce adds the ranks' sums: the update of one step grows with the global
    # batch.  Dividing the rate by the world size keeps the step per sample, and so the trajectory, the same at every N.
    lr = args.lr / world

    dp_check = None
    if world > 1 and not args.no_dp_check:
        # data parallel == one GPU on the whole batch, on a small model, before anything is timed
        dp_check = dp_consistency_check("ALEXNET", "VDNN_CONV", 4, 3, 0.01, dist, local)

    def make_net(policy, lean=False):
        net = vdnn.Network(args.model, policy, args.algo, batch_size=batch, device=local,
                           pool_bytes=args.pool_gb * 1e9, learning_rate=lr, init_mode=0, lean_offload=lean)
        if world > 1:
            uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
            if rank == 0:
                uid.copy_(torch.frombuffer(bytearray(dp_unique_id()), dtype=torch.uint8))
            dist.broadcast(uid, 0)
            net.enable_dp(rank, world, bytes(uid.cpu().numpy().tobytes()))
        return net

    def barrier(net):
        net.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(net, stream, hosts, steps, upload):
        """K steps between two CUDA events on the compute stream (the other streams are joined to it)."""
        beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier(net)
        launches0 = L.vdnn_kernel_launch_count()
        beg.record(stream)
        losses = []
        for i in range(steps):
            if upload:
                net.set_input(*hosts[i % 2])
            net.forwardPropagation()
            net.backwardPropagation()
            if upload:
                losses.append(net.loss())       # device -> host read of the step's result (blocks on the loss only)
        net.join()
        end.record(stream)
        barrier(net)
        ms = beg.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, L.vdnn_kernel_launch_count() - launches0, losses

    def copy_rates(stats):
        off = stats["offload_bytes"] / stats["offload_ms"] / 1e6 if stats["offload_ms"] > 0 else None
        pre = stats["prefetch_bytes"] / stats["prefetch_ms"] / 1e6 if stats["prefetch_ms"] > 0 else None
        return off, pre

    net = make_net(args.policy)
    # rank-specific synthetic batches in pinned host memory (two, alternated, so that the e2e upload
    # never re-sends a buffer the copy engine may have cached)
    rows = batch
    cols = net.output_size // rows
    hosts = []
    for j in range(2):
        x = torch.empty(net.input_size, dtype=torch.float32, pin_memory=True)
        t = torch.empty(net.output_size, dtype=torch.float32, pin_memory=True)
        L.vdnn_host_fill_normal(C.c_void_p(x.data_ptr()), net.input_size, 1000 + j * world + rank, 0.0, 1.0)
        L.vdnn_host_fill_onehot(C.c_void_p(t.data_ptr()), rows, cols, 2000 + j * world + rank)
        hosts.append((x, t))
    h2d_bytes = 4 * (net.input_size + net.output_size)
    stream = torch.cuda.ExternalStream(net.stream(0), device=local)

    # warm-up (also first-touch of pinned offload buffers), batch resident afterwards
    net.set_input(*hosts[0])
    for _ in range(max(args.warmup, 3)):
        net.step()
    barrier(net)

    net.set_profiling(True)
    # the clock sampler is started one (untimed) step early: nvidia-smi's own start-up takes driver locks for a few hundred
    # milliseconds, which must not fall into the timed region; it then samples every 200 ms through that region
    sampler = ClockSampler(local)
    sampler.start()
    net.step()
    barrier(net)
    ms, launches, _ = timed(net, stream, hosts, args.steps, upload=False)
    clocks = sampler.stop()
    stats = net.stats()
    net.set_profiling(False)
    ms_e2e, _, losses = timed(net, stream, hosts, args.steps, upload=True)
    status = vdnn.ops.engine_status()
    if status != 0:
        raise SystemExit(f"a bounded wait of the tensor-core engine expired during the timed region (code {status}): no valid number")
    if not all(math.isfinite(v) for pair in losses for v in pair):
        raise SystemExit(f"non-finite loss in the timed region: {losses}")
    layer_specs = net.layer_specs()
    checksum = net.weight_checksum() if world > 1 else None
    dp_mode = net.dp_mode()
    net.close()

    # the other policies, a few steps each, same process and same data (BASELINE config 5 names VDNN_CONV for the 1/2/4/8 runs;
    # VDNN_NONE is the kernel-bound rate).  VDNN_ALL_LEAN is this library's opt-in variant of VDNN_ALL that does not offload
    # ReLU inputs: it moves fewer bytes than the reference's policy, so it is reported here and never as the headline.
    by_policy = {}
    for policy in ([] if args.no_by_policy else [p for p in ("VDNN_NONE", "VDNN_CONV", "VDNN_ALL_LEAN") if p != args.policy]):
        try:
            other = make_net("VDNN_ALL", lean=True) if policy == "VDNN_ALL_LEAN" else make_net(policy)
        except vdnn.VdnnError as e:
            by_policy[policy] = {"unavailable": str(e)[:200]}
            continue
        ostream = torch.cuda.ExternalStream(other.stream(0), device=local)
        other.set_input(*hosts[0])
        for _ in range(3):
            other.step()
        barrier(other)
        other.set_profiling(True)
        k = max(3, min(args.steps, 8))
        oms, _, _ = timed(other, ostream, hosts, k, upload=False)
        ost = other.stats()
        off, pre = copy_rates(ost)
        by_policy[policy] = {"images_per_s": batch * world * k / (oms / 1e3), "ms_per_step": oms / k, "steps": k, "warmup": 3,
                             "pool_peak_bytes": ost["pool_peak_bytes"], "contraction_ms": ost["contraction_ms"],
                             "elementwise_ms": ost["elementwise_ms"],
                             "contraction_tflops": ost["contraction_flops"] / (ost["contraction_ms"] / 1e3) / 1e12 if ost["contraction_ms"] > 0 else None,
                             "offload_gbs": off, "prefetch_gbs": pre, "offload_bytes_per_step": ost["offload_bytes"]}
        if vdnn.ops.engine_status() != 0:
            by_policy[policy]["engine_error"] = True
        other.close()

    # algorithmic bytes of the contraction layers per step: each of forward, data gradient and filter gradient reads
    # or writes the layer's input-sized, output-sized and weight tensors once
    contraction_bytes = 0
    for sp in layer_specs:
        if sp.type in (vdnn.FC_GEMM, vdnn.CONV, vdnn.FC_CONV):
            src = sp.n * sp.c * sp.h * sp.w
            if sp.type == vdnn.FC_GEMM:
                dst = sp.n * sp.k
            else:
                dst = sp.n * sp.k * ((sp.h + 2 * sp.pad_h - sp.r) // sp.stride_h + 1) * ((sp.w + 2 * sp.pad_w - sp.s) // sp.stride_w + 1)
            contraction_bytes += 3 * 4 * (src + dst + sp.k * sp.c * sp.r * sp.s)
    peaks = measured_peaks()
    measured = None
    if rank == 0 and not args.no_probes:
        measured = tf32_probe(torch, vdnn, torch.cuda.current_stream())
        measured.update(pcie_probe(torch, torch.device("cuda", local)))
    images = batch * world * args.steps
    value = images / (ms / 1e3)
    e2e = images / (ms_e2e / 1e3)
    achieved_tf = stats["contraction_flops"] / (stats["contraction_ms"] / 1e3) / 1e12 if stats["contraction_ms"] > 0 else None
    elem_gbs = stats["elementwise_bytes"] / (stats["elementwise_ms"] / 1e3) / 1e9 if stats["elementwise_ms"] > 0 else None
    copy_ms = stats["offload_ms"] + stats["prefetch_ms"]
    off_gbs, pre_gbs = copy_rates(stats)
    traffic, traffic_file = profile_traffic()
    # squared-error loss (what the reference's backward differentiates, network.cu:1042-1054) of the e2e steps;
    # the two host batches alternate, so steps of equal parity see the same data
    sq = [v[0] for v in losses]
    same_batch_last = len(sq) - 1 - ((len(sq) - 1) % 2)
    line = {
        "metric": "train images/s", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.model} {args.policy} {args.algo}, batch {batch} per GPU, pool cap {args.pool_gb:g} GB",
                   "engine": args.engine, "l2": "activations per step (GBs) far exceed the 126 MB L2; no flush needed",
                   "parallelism": f"dp{world}" if world > 1 else "single",
                   "learning_rate": lr, "learning_rate_note": "--lr / world size: gradients are batch sums and the all-reduce sums over ranks"},
        "e2e": {"value": e2e, "unit": "images/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 16,
                "ms_per_step": ms_e2e / args.steps,
                "loss": [sq[0], sq[same_batch_last]] if sq else None,
                "loss_note": "0.5*sum((y-label)^2)/batch of the first and the last timed step that saw the same host batch (rank 0)",
                "loss_decreasing": bool(sq and sq[same_batch_last] < sq[0]),
                "cross_entropy": [losses[0][1], losses[same_batch_last][1]] if losses else None,
                "loss_trace": [round(v, 6) for v in sq]},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved_tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": (achieved_tf / peaks["tflops"]) if achieved_tf else None, "traffic": traffic,
                     "traffic_source": traffic_file, "algorithmic_bytes_per_step": contraction_bytes,
                     "kernel": "CONV/FC contraction layers (forward, data gradient, filter gradient)",
                     "peak_source": peaks["source"] + " bf16 sustained (cuBLAS); a product exact to fp32 costs three TF32 MMAs, each at half the bf16 rate",
                     "elementwise_gbs": elem_gbs, "hbm_peak_gbs": peaks["hbm_gbs"]},
        "vdnn": {"pool_peak_bytes": stats["pool_peak_bytes"], "pinned_bytes": stats["pinned_bytes"],
                 "offload_bytes": stats["offload_bytes"], "prefetch_bytes": stats["prefetch_bytes"],
                 "workspace_bytes_max": stats["workspace_bytes_max"], "grad_buffer_bytes": stats["grad_buffer_bytes"],
                 "step_ms_profiled": stats["step_ms"], "contraction_ms": stats["contraction_ms"],
                 "elementwise_ms": stats["elementwise_ms"],
                 "offload_gbs": off_gbs, "prefetch_gbs": pre_gbs,
                 "offload_gbs_all_gpus": off_gbs * world if off_gbs else None,
                 "prefetch_gbs_all_gpus": pre_gbs * world if pre_gbs else None,
                 "copy_overlap_frac": stats["copy_overlap_ms"] / copy_ms if copy_ms > 0 else None,
                 "forced_offloads": stats["forced_offloads"],
                 "dp_mode": {0: "single", 1: "nccl all-reduce + axpy per layer", 2: "fused peer all-reduce + SGD kernel"}[dp_mode],
                 "by_policy": by_policy},
    }
    if measured:
        line["measured_peaks"] = measured
        if achieved_tf:
            line["roofline"]["frac_of_3xtf32_ceiling"] = achieved_tf / (measured["tf32_dense_tflops_sustained"] / 3.0)
    if world > 1:
        sums = [None] * world
        dist.all_gather_object(sums, checksum)
        line["vdnn"]["weights_identical_across_ranks"] = len(set(sums)) == 1
        if dp_check is not None:
            line["vdnn"]["dp_matches_single_gpu"] = bool(dp_check["max_rel_err_vs_single_gpu"] < 1e-4 and
                                                         len(set(dp_check["checksums"])) == 1)
            line["vdnn"]["dp_check"] = {"model": "ALEXNET VDNN_CONV, 4 images per rank, 3 steps, lr 0.01",
                                        "max_rel_err_vs_single_gpu": dp_check["max_rel_err_vs_single_gpu"]}
    if rank == 0 and world == 1 and not args.no_reference_warm:
        line["reference_warm"] = reference_warm(args, ["VDNN_NONE"] + ([args.policy] if args.policy != "VDNN_NONE" else []))
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_batch = args.cpu_batch or (8 if args.model.startswith("VGG") else 64)
        v, step_s = cpu_step_rate(args.model, cpu_batch, 1, 1, args.lr)
        line["cpu_baseline"] = {"value": v, "unit": "images/s", "cores": host_threads(), "kind": "port",
                                "sample": f"{args.model} batch {cpu_batch}: 1 warm-up + 1 timed step ({step_s:.1f} s) of the CPU "
                                          f"restatement, float accumulation, OpenMP"}
    elif rank == 0:
        line["cpu_baseline"] = None
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
