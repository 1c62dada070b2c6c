"""Thin wrappers that call the layer kernels of the C ABI on device pointers.

Arguments are objects with `data_ptr()` (torch CUDA tensors: PyTorch is only the owner of the
device memory here) or raw integer device addresses.  Every function enqueues on `stream`
(a raw cudaStream_t integer, 0 = legacy default stream) and returns nothing.
"""
import ctypes as C

from . import abi
from .abi import ConvDesc, check, lib


def _p(t):
    if t is None:
        return None
    return C.c_void_p(t.data_ptr() if hasattr(t, "data_ptr") else int(t))


def _s(stream):
    return C.c_void_p(int(stream) if stream else 0)


def conv_desc(n, c, h, w, k, r, s, pad, stride):
    return ConvDesc(n, c, h, w, k, r, s, pad[0], pad[1], stride[0], stride[1])


def conv_out_dims(desc):
    p, q = C.c_int(), C.c_int()
    check(lib().vdnn_conv_out_dims(C.byref(desc), C.byref(p), C.byref(q)), "conv_out_dims")
    return p.value, q.value


def conv_workspace_bytes(op, algo_mode, desc):
    return lib().vdnn_conv_workspace_bytes(op, algo_mode, C.byref(desc))


def conv_fwd(desc, x, w, y, bias=None, alpha=1.0, beta=0.0, algo_mode=0, workspace=None, workspace_bytes=0, stream=0):
    check(lib().vdnn_conv_fwd(C.byref(desc), algo_mode, alpha, _p(x), _p(w), _p(bias), beta, _p(y), _p(workspace),
                              workspace_bytes, _s(stream)), "conv_fwd")


def add_bias(n, k, pq, bias, y, alpha=1.0, stream=0):
    check(lib().vdnn_add_bias(n, k, pq, alpha, _p(bias), _p(y), _s(stream)), "add_bias")


def conv_bwd_data(desc, w, dy, dx, alpha=1.0, beta=0.0, algo_mode=0, workspace=None, workspace_bytes=0, stream=0):
    check(lib().vdnn_conv_bwd_data(C.byref(desc), algo_mode, alpha, _p(w), _p(dy), beta, _p(dx), _p(workspace),
                                   workspace_bytes, _s(stream)), "conv_bwd_data")


def conv_bwd_bias(n, k, pq, dy, db, alpha=1.0, beta=0.0, stream=0):
    check(lib().vdnn_conv_bwd_bias(n, k, pq, alpha, _p(dy), beta, _p(db), _s(stream)), "conv_bwd_bias")


def conv_bwd_filter(desc, x, dy, dw, alpha=1.0, beta=0.0, algo_mode=0, workspace=None, workspace_bytes=0, stream=0):
    check(lib().vdnn_conv_bwd_filter(C.byref(desc), algo_mode, alpha, _p(x), _p(dy), beta, _p(dw), _p(workspace),
                                     workspace_bytes, _s(stream)), "conv_bwd_filter")


def conv_bwd_filter_bias(desc, x, dy, dw, db, alpha=1.0, beta=0.0, alpha_b=1.0, beta_b=0.0, algo_mode=0, workspace=None,
                         workspace_bytes=0, stream=0):
    check(lib().vdnn_conv_bwd_filter_bias(C.byref(desc), algo_mode, alpha, _p(x), _p(dy), beta, _p(dw), alpha_b, beta_b, _p(db),
                                          _p(workspace), workspace_bytes, _s(stream)), "conv_bwd_filter_bias")


def conv_bwd_data_filter_bias(desc, w, x, dy, dx, dw, db, alpha_dx=1.0, beta_dx=0.0, alpha_w=1.0, beta_w=0.0, alpha_b=1.0, beta_b=0.0,
                              algo_mode=0, workspace=None, workspace_bytes=0, stream=0):
    check(lib().vdnn_conv_bwd_data_filter_bias(C.byref(desc), algo_mode, alpha_dx, _p(w), _p(x), _p(dy), beta_dx, _p(dx), alpha_w, beta_w,
                                               _p(dw), alpha_b, beta_b, _p(db), _p(workspace), workspace_bytes, _s(stream)),
          "conv_bwd_data_filter_bias")


def conv_bwd_shares_dy(desc, algo_mode):
    return bool(lib().vdnn_conv_bwd_shares_dy(C.byref(desc), algo_mode))


STATIC_SCRATCH_BYTES = 16 << 20


def conv_bwd_filter_static(desc, x, dy, dw, alpha=1.0, beta=0.0, stream=0):
    """Filter gradient without caller workspace: the split-K partial sums go to the library's own
    16 MiB device array.  For hosts that may not allocate after start-up.  Raises VdnnError
    (VDNN_ERR_SCRATCH_LIMIT) when the shape needs more than that."""
    check(lib().vdnn_conv_bwd_filter_static(C.byref(desc), alpha, _p(x), _p(dy), beta, _p(dw), _s(stream)),
          "conv_bwd_filter_static")


def sgemm_workspace_bytes(algo_mode, m, n, k):
    return lib().vdnn_sgemm_workspace_bytes(algo_mode, m, n, k)


def sgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, Cm, ldc, algo_mode=0, workspace=None,
          workspace_bytes=0, stream=0):
    check(lib().vdnn_sgemm(int(transa), int(transb), m, n, k, alpha, _p(A), lda, _p(B), ldb, beta, _p(Cm), ldc,
                           algo_mode, _p(workspace), workspace_bytes, _s(stream)), "sgemm")


def fill(count, value, dst, stream=0):
    check(lib().vdnn_fill(count, value, _p(dst), _s(stream)), "fill")


def relu_fwd(count, x, y, stream=0):
    check(lib().vdnn_relu_fwd(count, _p(x), _p(y), _s(stream)), "relu_fwd")


def relu_bwd(count, y, dy, x, dx, stream=0):
    check(lib().vdnn_relu_bwd(count, _p(y), _p(dy), _p(x), _p(dx), _s(stream)), "relu_bwd")


ACT_RELU, ACT_TANH, ACT_SIGMOID = 0, 1, 2


def activation_fwd(mode, count, x, y, stream=0):
    check(lib().vdnn_activation_fwd(mode, count, _p(x), _p(y), _s(stream)), "activation_fwd")


def activation_bwd(mode, count, y, dy, x, dx, stream=0):
    check(lib().vdnn_activation_bwd(mode, count, _p(y), _p(dy), _p(x), _p(dx), _s(stream)), "activation_bwd")


def maxpool_fwd(n, c, h, w, win, stride, x, y, stream=0):
    check(lib().vdnn_maxpool_fwd(n, c, h, w, win[0], win[1], stride[0], stride[1], _p(x), _p(y), _s(stream)), "maxpool_fwd")


def maxpool_bwd(n, c, h, w, win, stride, y, dy, x, dx, stream=0):
    check(lib().vdnn_maxpool_bwd(n, c, h, w, win[0], win[1], stride[0], stride[1], _p(y), _p(dy), _p(x), _p(dx),
                                 _s(stream)), "maxpool_bwd")


def softmax_fwd(rows, cols, x, y, stream=0):
    check(lib().vdnn_softmax_fwd(rows, cols, _p(x), _p(y), _s(stream)), "softmax_fwd")


def softmax_bwd(rows, cols, y, dy, dx, stream=0):
    check(lib().vdnn_softmax_bwd(rows, cols, _p(y), _p(dy), _p(dx), _s(stream)), "softmax_bwd")


def sub(count, a, b, out, stream=0):
    check(lib().vdnn_sub(count, _p(a), _p(b), _p(out), _s(stream)), "sub")


def lrn_fwd(n, c, hw, x, y, win=5, alpha=1e-4, beta=0.75, k=2.0, stream=0):
    check(lib().vdnn_lrn_fwd(n, c, hw, win, alpha, beta, k, _p(x), _p(y), _s(stream)), "lrn_fwd")


def lrn_bwd(n, c, hw, x, y, dy, dx, win=5, alpha=1e-4, beta=0.75, k=2.0, stream=0):
    check(lib().vdnn_lrn_bwd(n, c, hw, win, alpha, beta, k, _p(x), _p(y), _p(dy), _p(dx), _s(stream)), "lrn_bwd")


def axpy(count, alpha, g, w, stream=0):
    check(lib().vdnn_axpy(count, alpha, _p(g), _p(w), _s(stream)), "axpy")


def loss(rows, cols, y, label, out2, stream=0):
    check(lib().vdnn_loss(rows, cols, _p(y), _p(label), _p(out2), _s(stream)), "loss")


def set_engine(engine):
    return lib().vdnn_set_engine(engine)


def get_engine():
    return lib().vdnn_get_engine()


def engine_status():
    """Synchronises the device; returns the tensor-core engine's error code (0 = healthy) and clears it."""
    code = C.c_int()
    check(lib().vdnn_engine_status(C.byref(code)), "engine_status")
    return code.value


def engine_wait_selftest(limit_cycles=2_000_000, stream=0):
    """Runs the engine's bounded barrier wait on a barrier nothing arrives at: it runs out after `limit_cycles` SM
    cycles, records code 104 and the kernel returns.  engine_status() then reports (and clears) 104."""
    check(lib().vdnn_engine_wait_selftest(limit_cycles, _s(stream)), "engine_wait_selftest")


def engine_mma_rate_probe(iterations, stream=0):
    """Enqueues the tensor-pipe rate probe; returns the hardware flops of the launch (time it with events)."""
    flops = C.c_double()
    check(lib().vdnn_engine_mma_rate_probe(iterations, C.byref(flops), _s(stream)), "engine_mma_rate_probe")
    return flops.value
