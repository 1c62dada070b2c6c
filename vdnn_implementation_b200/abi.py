"""ctypes declarations for include/vdnn_b200.h."""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))

# vdnn_t, vdnnAlgoMode_t, Layer_t, CNN_t (reference vdnn.h:23-61; LRN / ALEXNET_LRN are additions)
BASELINE, VDNN_NONE, VDNN_ALL, VDNN_CONV = range(4)
VDNN_MEMORY_OPT_ALGO, VDNN_PERF_OPT_ALGO, VDNN_DYNAMIC_ALGO = range(3)
FC_GEMM, CONV, FC_CONV, RELU, TANH, SIGMOID, SOFTMAX, POOL, CONCATENATE, LRN = range(10)
ALEXNET, OVERFEAT, GOOGLENET, VGG16_64, VGG16_128, VGG16_256, CUSTOM_CNN, ALEXNET_LRN = range(8)
ENGINE_AUTO, ENGINE_FFMA, ENGINE_TCGEN05 = range(3)
CONV_FWD, CONV_BWD_DATA, CONV_BWD_FILTER = range(3)
TENSOR_DST, TENSOR_GRAD, TENSOR_WEIGHT, TENSOR_BIAS = range(4)

CNN_NAMES = {"ALEXNET": ALEXNET, "OVERFEAT": OVERFEAT, "GOOGLENET": GOOGLENET, "VGG16_64": VGG16_64,
             "VGG16_128": VGG16_128, "VGG16_256": VGG16_256, "CUSTOM_CNN": CUSTOM_CNN, "ALEXNET_LRN": ALEXNET_LRN}
VDNN_NAMES = {"BASELINE": BASELINE, "VDNN_NONE": VDNN_NONE, "VDNN_ALL": VDNN_ALL, "VDNN_CONV": VDNN_CONV}
ALGO_NAMES = {"VDNN_MEMORY_OPT_ALGO": VDNN_MEMORY_OPT_ALGO, "VDNN_PERF_OPT_ALGO": VDNN_PERF_OPT_ALGO,
              "VDNN_DYNAMIC_ALGO": VDNN_DYNAMIC_ALGO}


class VdnnError(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        name = lib().vdnn_status_string(status).decode()
        super().__init__(f"{what}: {name} ({status}), cuda error {lib().vdnn_last_cuda_error()}")


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n", "c", "h", "w", "k", "r", "s", "pad_h", "pad_w", "stride_h", "stride_w")]


class LayerSpec(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("type", "n", "c", "h", "w", "pad_h", "pad_w", "stride_h", "stride_w", "k", "r", "s")]

    def astuple(self):
        return tuple(getattr(self, f) for f, _ in self._fields_)


class NetworkConfig(C.Structure):
    _fields_ = [("cnn_type", C.c_int), ("vdnn_type", C.c_int), ("algo_mode", C.c_int), ("batch_size", C.c_int),
                ("device", C.c_int), ("pool_bytes", C.c_size_t), ("learning_rate", C.c_float),
                ("init_mode", C.c_int), ("weight_seed_base", C.c_uint64), ("fix_input_leak", C.c_int),
                ("host_sync_per_layer", C.c_int), ("verbose", C.c_int), ("capture", C.c_int),
                ("custom_layers", C.POINTER(LayerSpec)), ("num_custom_layers", C.c_int)]


class TraceEvent(C.Structure):
    _fields_ = [("kind", C.c_int), ("layer", C.c_int), ("tag", C.c_int), ("bytes", C.c_int64), ("used", C.c_int64)]


class NetworkStats(C.Structure):
    _fields_ = [("pool_peak_bytes", C.c_int64), ("pool_used_bytes", C.c_int64), ("pool_capacity_bytes", C.c_int64),
                ("pinned_bytes", C.c_int64), ("offload_bytes", C.c_int64), ("prefetch_bytes", C.c_int64),
                ("workspace_bytes_max", C.c_int64), ("grad_buffer_bytes", C.c_int64), ("step_ms", C.c_float),
                ("offload_ms", C.c_float), ("prefetch_ms", C.c_float), ("copy_overlap_ms", C.c_float),
                ("kernel_launches", C.c_int), ("contraction_ms", C.c_float), ("elementwise_ms", C.c_float),
                ("contraction_flops", C.c_double), ("elementwise_bytes", C.c_double), ("forced_offloads", C.c_int64)]

    def asdict(self):
        return {f: getattr(self, f) for f, _ in self._fields_}


def lib_path():
    """The in-tree shared object; VDNN_B200_LIB may point at another build of the same library."""
    return os.environ.get("VDNN_B200_LIB") or os.path.join(PKG, "libvdnn_b200.so")


_lib = None

_P, _F, _I, _Z, _D = C.c_void_p, C.c_float, C.c_int, C.c_size_t, C.POINTER(ConvDesc)
# name -> (restype, argtypes); every symbol declared in include/vdnn_b200.h
SIGNATURES = {
    "vdnn_status_string": (C.c_char_p, [_I]),
    "vdnn_last_cuda_error": (_I, []),
    "vdnn_build_info": (C.c_char_p, []),
    "vdnn_set_engine": (_I, [_I]),
    "vdnn_get_engine": (_I, []),
    "vdnn_engine_status": (_I, [C.POINTER(_I)]),
    "vdnn_engine_status_publish": (_I, [_P, _P]),
    "vdnn_engine_wait_selftest": (_I, [C.c_ulonglong, _P]),
    "vdnn_engine_mma_rate_probe": (_I, [_I, C.POINTER(C.c_double), _P]),
    "vdnn_conv_out_dims": (_I, [_D, C.POINTER(_I), C.POINTER(_I)]),
    "vdnn_pool_out_dims": (_I, [_I] * 6 + [C.POINTER(_I), C.POINTER(_I)]),
    "vdnn_conv_workspace_bytes": (_Z, [_I, _I, _D]),
    "vdnn_conv_fwd": (_I, [_D, _I, _F, _P, _P, _P, _F, _P, _P, _Z, _P]),
    "vdnn_add_bias": (_I, [_I, _I, _I, _F, _P, _P, _P]),
    "vdnn_conv_bwd_data": (_I, [_D, _I, _F, _P, _P, _F, _P, _P, _Z, _P]),
    "vdnn_conv_bwd_bias": (_I, [_I, _I, _I, _F, _P, _F, _P, _P]),
    "vdnn_conv_bwd_filter": (_I, [_D, _I, _F, _P, _P, _F, _P, _P, _Z, _P]),
    "vdnn_conv_bwd_filter_bias": (_I, [_D, _I, _F, _P, _P, _F, _P, _F, _F, _P, _P, _Z, _P]),
    "vdnn_conv_bwd_data_filter_bias": (_I, [_D, _I, _F, _P, _P, _P, _F, _P, _F, _F, _P, _F, _F, _P, _P, _Z, _P]),
    "vdnn_conv_bwd_shares_dy": (_I, [_D, _I]),
    "vdnn_conv_bwd_filter_static": (_I, [_D, _F, _P, _P, _F, _P, _P]),
    "vdnn_sgemm_workspace_bytes": (_Z, [_I, _I, _I, _I]),
    "vdnn_sgemm": (_I, [_I, _I, _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I, _I, _P, _Z, _P]),
    "vdnn_fill": (_I, [_Z, _F, _P, _P]),
    "vdnn_relu_fwd": (_I, [_Z, _P, _P, _P]),
    "vdnn_relu_bwd": (_I, [_Z, _P, _P, _P, _P, _P]),
    "vdnn_activation_fwd": (_I, [_I, _Z, _P, _P, _P]),
    "vdnn_activation_bwd": (_I, [_I, _Z, _P, _P, _P, _P, _P]),
    "vdnn_maxpool_fwd": (_I, [_I] * 8 + [_P, _P, _P]),
    "vdnn_maxpool_bwd": (_I, [_I] * 8 + [_P, _P, _P, _P, _P]),
    "vdnn_softmax_fwd": (_I, [_I, _I, _P, _P, _P]),
    "vdnn_softmax_bwd": (_I, [_I, _I, _P, _P, _P, _P]),
    "vdnn_sub": (_I, [_Z, _P, _P, _P, _P]),
    "vdnn_lrn_fwd": (_I, [_I, _I, _I, _I, _F, _F, _F, _P, _P, _P]),
    "vdnn_lrn_bwd": (_I, [_I, _I, _I, _I, _F, _F, _F, _P, _P, _P, _P, _P]),
    "vdnn_axpy": (_I, [_Z, _F, _P, _P, _P]),
    "vdnn_loss": (_I, [_I, _I, _P, _P, _P, _P]),
    "vdnn_offload": (_I, [_P, _P, _Z, _P, _P, _P]),
    "vdnn_prefetch": (_I, [_P, _P, _Z, _P, _P, _P]),
    "vdnn_network_create": (_I, [C.POINTER(_P), C.POINTER(NetworkConfig)]),
    "vdnn_network_destroy": (_I, [_P]),
    "vdnn_network_num_layers": (_I, [_P]),
    "vdnn_network_layer_spec": (_I, [_P, _I, C.POINTER(LayerSpec)]),
    "vdnn_network_input_size": (_Z, [_P]),
    "vdnn_network_output_size": (_Z, [_P]),
    "vdnn_network_set_input": (_I, [_P, _P, _P]),
    "vdnn_network_seed_input": (_I, [_P, C.c_uint64, C.c_uint64]),
    "vdnn_network_forward": (_I, [_P]),
    "vdnn_network_backward": (_I, [_P]),
    "vdnn_network_synchronize": (_I, [_P]),
    "vdnn_network_stream": (_P, [_P, _I]),
    "vdnn_network_join": (_I, [_P]),
    "vdnn_kernel_launch_count": (C.c_ulonglong, []),
    "vdnn_network_loss": (_I, [_P, C.POINTER(C.c_double)]),
    "vdnn_network_tensor_size": (_Z, [_P, _I, _I]),
    "vdnn_network_read_tensor": (_I, [_P, _I, _I, _P, _Z]),
    "vdnn_network_write_tensor": (_I, [_P, _I, _I, _P, _Z]),
    "vdnn_network_trace": (_I, [_P, C.POINTER(TraceEvent), _I, C.POINTER(_I)]),
    "vdnn_network_trace_reset": (_I, [_P]),
    "vdnn_network_get_stats": (_I, [_P, C.POINTER(NetworkStats)]),
    "vdnn_network_set_profiling": (_I, [_P, _I]),
    "vdnn_network_set_offload_order": (_I, [_P, _I]),
    "vdnn_set_lean_offload": (_I, [_I]),
    "vdnn_network_lean": (_I, [_P]),
    "vdnn_network_selected": (_I, [_P, C.POINTER(_I), C.POINTER(_I)]),
    "vdnn_network_layer_algos": (_I, [_P, _I, C.POINTER(_I)]),
    "vdnn_network_timeline": (_I, [_P, _P]),
    "vdnn_dp_unique_id": (_I, [C.c_char_p]),
    "vdnn_network_enable_dp": (_I, [_P, _I, _I, C.c_char_p]),
    "vdnn_network_dp_mode": (_I, [_P]),
    "vdnn_dp_slice": (_I, [_Z, _I, _I, C.POINTER(_Z), C.POINTER(_Z)]),
    "vdnn_network_weight_checksum": (_I, [_P, C.POINTER(C.c_uint64)]),
    "vdnn_host_fill_normal": (None, [_P, _Z, C.c_uint64, _F, _F]),
    "vdnn_host_fill_uniform": (None, [_P, _Z, C.c_uint64, _F, _F]),
    "vdnn_host_fill_onehot": (None, [_P, _I, _I, C.c_uint64]),
}


def lib():
    """The loaded CUDA library.  Raises if it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: build it with `python -m vdnn_implementation_b200.build` "
                              "(the package has no CPU or PyTorch fallback)")
        L = C.CDLL(path, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            if os.environ.get("VDNN_B200_LIB") and not hasattr(L, name):
                continue        # an experimental build may lack the newest entry points
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status, what):
    if status != 0:
        raise VdnnError(status, what)
