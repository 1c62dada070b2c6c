"""Python mirror of the driver's Network class (reference network.h:15-95) over the C ABI."""
import ctypes as C

import numpy as np

from . import abi
from .abi import check, lib


class Network:
    """Builds one of the reference topologies (or a custom layer list) under a vDNN policy.

    forwardPropagation / backwardPropagation keep the reference's names.  `device=-1` makes a
    dry-run network: the allocation / offload / prefetch schedule is replayed against a
    bookkeeping-only pool and nothing touches a GPU.
    """

    def __init__(self, cnn_type, vdnn_type, algo_mode, batch_size=0, device=0, pool_bytes=0, learning_rate=0.0,
                 init_mode=0, weight_seed_base=3000, fix_input_leak=True, host_sync_per_layer=False,
                 verbose=False, capture=False, custom_layers=None, lean_offload=None):
        cnn_type = abi.CNN_NAMES.get(cnn_type, cnn_type)
        vdnn_type = abi.VDNN_NAMES.get(vdnn_type, vdnn_type)
        algo_mode = abi.ALGO_NAMES.get(algo_mode, algo_mode)
        cfg = abi.NetworkConfig()
        cfg.cnn_type, cfg.vdnn_type, cfg.algo_mode, cfg.batch_size = cnn_type, vdnn_type, algo_mode, batch_size
        cfg.device, cfg.pool_bytes, cfg.learning_rate = device, int(pool_bytes), learning_rate
        cfg.init_mode, cfg.weight_seed_base = init_mode, weight_seed_base
        cfg.fix_input_leak, cfg.host_sync_per_layer = int(fix_input_leak), int(host_sync_per_layer)
        cfg.verbose, cfg.capture = int(verbose), int(capture)
        self._custom = None
        if custom_layers is not None:
            self._custom = (abi.LayerSpec * len(custom_layers))()
            for i, s in enumerate(custom_layers):
                self._custom[i] = s if isinstance(s, abi.LayerSpec) else abi.LayerSpec(*s)
            cfg.custom_layers = self._custom
            cfg.num_custom_layers = len(custom_layers)
        self._h = C.c_void_p()
        # lean_offload: None = the environment decides (VDNN_LEAN_OFFLOAD), True / False = this network's own choice
        if lean_offload is not None:
            lib().vdnn_set_lean_offload(int(bool(lean_offload)))
        try:
            check(lib().vdnn_network_create(C.byref(self._h), C.byref(cfg)), "vdnn_network_create")
        finally:
            if lean_offload is not None:
                lib().vdnn_set_lean_offload(-1)
        self.lean_offload = bool(lib().vdnn_network_lean(self._h))
        self.num_layers = lib().vdnn_network_num_layers(self._h)
        self.input_size = lib().vdnn_network_input_size(self._h)
        self.output_size = lib().vdnn_network_output_size(self._h)
        self.dry_run = device < 0

    def close(self):
        if getattr(self, "_h", None):
            lib().vdnn_network_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def layer_spec(self, layer):
        s = abi.LayerSpec()
        check(lib().vdnn_network_layer_spec(self._h, layer, C.byref(s)), "layer_spec")
        return s

    def layer_specs(self):
        return [self.layer_spec(i) for i in range(self.num_layers)]

    def set_input(self, input_h, label_h):
        """input_h / label_h: contiguous float32 host arrays (numpy, or pinned torch CPU tensors)."""
        pi, pl = _host_ptr(input_h, self.input_size), _host_ptr(label_h, self.output_size)
        check(lib().vdnn_network_set_input(self._h, pi, pl), "set_input")

    def seed_input(self, input_seed, label_seed):
        check(lib().vdnn_network_seed_input(self._h, input_seed, label_seed), "seed_input")

    def forwardPropagation(self):
        check(lib().vdnn_network_forward(self._h), "forwardPropagation")

    def backwardPropagation(self):
        check(lib().vdnn_network_backward(self._h), "backwardPropagation")

    def step(self):
        self.forwardPropagation()
        self.backwardPropagation()

    def synchronize(self):
        check(lib().vdnn_network_synchronize(self._h), "synchronize")

    def stream(self, which=0):
        """Raw cudaStream_t (int) of the compute (0), offload (1), prefetch (2) or collective (3) stream."""
        return lib().vdnn_network_stream(self._h, which) or 0

    def join(self):
        check(lib().vdnn_network_join(self._h), "join")

    def loss(self):
        out = (C.c_double * 2)()
        check(lib().vdnn_network_loss(self._h, out), "loss")
        return out[0], out[1]

    def tensor_size(self, layer, kind):
        return lib().vdnn_network_tensor_size(self._h, layer, kind)

    def read_tensor(self, layer, kind):
        n = self.tensor_size(layer, kind)
        if n == 0:
            return None
        out = np.empty(n, np.float32)
        check(lib().vdnn_network_read_tensor(self._h, layer, kind, out.ctypes.data_as(C.c_void_p), n), "read_tensor")
        return out

    def write_tensor(self, layer, kind, values):
        v = np.ascontiguousarray(values, np.float32).ravel()
        check(lib().vdnn_network_write_tensor(self._h, layer, kind, v.ctypes.data_as(C.c_void_p), v.size), "write_tensor")

    def dst(self, layer):
        return self.read_tensor(layer, abi.TENSOR_DST)

    def grad(self, layer):
        return self.read_tensor(layer, abi.TENSOR_GRAD)

    def weights(self, layer):
        return self.read_tensor(layer, abi.TENSOR_WEIGHT)

    def bias(self, layer):
        return self.read_tensor(layer, abi.TENSOR_BIAS)

    def trace(self):
        n = C.c_int()
        check(lib().vdnn_network_trace(self._h, None, 0, C.byref(n)), "trace")
        buf = (abi.TraceEvent * max(n.value, 1))()
        check(lib().vdnn_network_trace(self._h, buf, n.value, C.byref(n)), "trace")
        return [(e.kind, e.layer, e.tag, e.bytes, e.used) for e in buf[:n.value]]

    def trace_reset(self):
        check(lib().vdnn_network_trace_reset(self._h), "trace_reset")

    def set_profiling(self, enabled=True):
        check(lib().vdnn_network_set_profiling(self._h, int(enabled)), "set_profiling")

    def selected(self):
        """(vdnn_type, algo_mode) the constructor settled on; algo_mode 2 (VDNN_DYNAMIC_ALGO) = chosen per layer."""
        t, a = C.c_int(), C.c_int()
        check(lib().vdnn_network_selected(self._h, C.byref(t), C.byref(a)), "selected")
        return t.value, a.value

    def layer_algos(self, layer):
        """VDNN_ALGO_MEMORY_OPT (0) / VDNN_ALGO_PERF_OPT (1) for forward, data gradient, filter gradient."""
        out = (C.c_int * 3)()
        check(lib().vdnn_network_layer_algos(self._h, layer, out), "layer_algos")
        return tuple(out)

    def set_offload_order(self, forward_order=False):
        """False (default): offload copies reach the copy engine in the order backward needs them;
        True: in layer order, as the reference enqueues them."""
        check(lib().vdnn_network_set_offload_order(self._h, int(forward_order)), "set_offload_order")

    def timeline(self):
        """(num_layers, 8) array of ms since step start: fwd beg/end, offload beg/end, bwd beg/end, prefetch beg/end."""
        out = np.empty(8 * self.num_layers, np.float32)
        check(lib().vdnn_network_timeline(self._h, out.ctypes.data_as(C.c_void_p)), "timeline")
        return out.reshape(self.num_layers, 8)

    def stats(self):
        s = abi.NetworkStats()
        check(lib().vdnn_network_get_stats(self._h, C.byref(s)), "get_stats")
        return s.asdict()

    def enable_dp(self, rank, world_size, unique_id):
        check(lib().vdnn_network_enable_dp(self._h, rank, world_size, unique_id), "enable_dp")

    def dp_mode(self):
        """0 single device, 1 NCCL all-reduce + axpy, 2 fused peer all-reduce + SGD kernel."""
        return lib().vdnn_network_dp_mode(self._h)

    def weight_checksum(self):
        out = C.c_uint64()
        check(lib().vdnn_network_weight_checksum(self._h, C.byref(out)), "weight_checksum")
        return out.value


def dp_unique_id():
    buf = C.create_string_buffer(128)
    check(lib().vdnn_dp_unique_id(buf), "dp_unique_id")
    return buf.raw


def _host_ptr(a, expect):
    if isinstance(a, np.ndarray):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"] and a.size == expect
        return a.ctypes.data_as(C.c_void_p)
    # torch CPU tensor (possibly pinned)
    assert a.device.type == "cpu" and a.is_contiguous() and a.numel() == expect and a.element_size() == 4
    return C.c_void_p(a.data_ptr())


def dp_consistency_check(model, policy, per_rank, steps, lr, dist, local_device, algo="VDNN_PERF_OPT_ALGO", pool_bytes=8e9):
    """Data-parallel training against one GPU on the whole batch (call on every rank of an initialised NCCL group).

    Every rank trains its shard of `steps` seeded batches with the per-layer gradient all-reduce; then rank 0 repeats
    the same steps alone on the whole batches.  Gradients are batch sums (layer.cu:631-660, 736-760 of the reference
    fold alpha = -lr sums into the weights), so the sum over the shards' gradients is the whole batch's gradient and
    the two runs must agree to rounding.  Returns on rank 0 a dict with `checksums` (one per rank; equal = weights
    bit-identical across ranks), `max_rel_err_vs_single_gpu`, `grad_buffer_bytes`, `engine_status`, `dp_mode` (1 NCCL,
    2 the fused peer kernel, chosen by VDNN_DP_FUSED in the environment); None elsewhere."""
    import torch
    from . import ops
    rank, world = dist.get_rank(), dist.get_world_size()
    L = lib()
    net = Network(model, policy, algo, batch_size=per_rank, device=local_device, pool_bytes=pool_bytes, learning_rate=lr, init_mode=0)
    uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        uid.copy_(torch.frombuffer(bytearray(dp_unique_id()), dtype=torch.uint8))
    dist.broadcast(uid, 0)
    net.enable_dp(rank, world, uid.cpu().numpy().tobytes())
    in_per_image, classes = net.input_size // per_rank, net.output_size // per_rank
    data = []
    for step in range(steps):
        x = np.empty(world * per_rank * in_per_image, np.float32)
        t = np.empty((world * per_rank, classes), np.float32)
        L.vdnn_host_fill_normal(x.ctypes.data_as(C.c_void_p), x.size, 1000 + step, 0.0, 1.0)
        L.vdnn_host_fill_onehot(t.ctypes.data_as(C.c_void_p), world * per_rank, classes, 2000 + step)
        data.append((x.reshape(world, -1), t.reshape(world, -1)))
    for x, t in data:
        net.set_input(np.ascontiguousarray(x[rank]), np.ascontiguousarray(t[rank]))
        net.step()
    net.synchronize()
    sums = [None] * world
    dist.all_gather_object(sums, net.weight_checksum())
    stats = net.stats()
    mode = net.dp_mode()
    with_weights = [l for l in range(net.num_layers) if net.tensor_size(l, abi.TENSOR_WEIGHT) > 0]
    probe = (with_weights[0], with_weights[len(with_weights) // 2], with_weights[-1])
    dp_weights = {l: net.weights(l) for l in probe}
    dp_bias = {l: net.bias(l) for l in probe}
    status = ops.engine_status()
    net.close()
    result = None
    if rank == 0:
        one = Network(model, policy, algo, batch_size=per_rank * world, device=local_device, pool_bytes=pool_bytes,
                      learning_rate=lr, init_mode=0)
        for x, t in data:
            one.set_input(np.ascontiguousarray(x.ravel()), np.ascontiguousarray(t.ravel()))
            one.step()
        one.synchronize()
        errs = []
        for l in probe:
            for a, b in ((dp_weights[l], one.weights(l)), (dp_bias[l], one.bias(l))):
                errs.append(float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)))
        one.close()
        result = {"checksums": [str(s) for s in sums], "grad_buffer_bytes": stats["grad_buffer_bytes"], "engine_status": status,
                  "max_rel_err_vs_single_gpu": max(errs), "dp_mode": mode}
    dist.barrier()
    return result
