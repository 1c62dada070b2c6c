"""ctypes binding of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Imported by the tests, by the smoke check and by the CPU-baseline leg of the benchmark.
The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# Layer_t / vdnn_t / CNN_t values of the reference (vdnn.h:23-61) plus the LRN extension.
FC_GEMM, CONV, FC_CONV, RELU, TANH, SIGMOID, SOFTMAX, POOL, CONCATENATE, LRN = range(10)
BASELINE, VDNN_NONE, VDNN_ALL, VDNN_CONV = range(4)
ALEXNET, OVERFEAT, GOOGLENET, VGG16_64, VGG16_128, VGG16_256, CUSTOM_CNN, ALEXNET_LRN = range(8)

EV_ALLOC, EV_FREE, EV_OFFLOAD, EV_PREFETCH, EV_FWD_DONE, EV_BWD_DONE = range(6)
(TAG_WEIGHT, TAG_BIAS, TAG_DST, TAG_DIFF, TAG_GRAD, TAG_SRC, TAG_WS, TAG_ONES, TAG_INPUT,
 TAG_LABEL, TAG_DXDY, TAG_NONE) = range(12)


class LayerSpec(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("type", "n", "c", "h", "w", "pad_h", "pad_w", "stride_h", "stride_w", "k", "r", "s")]

    def astuple(self):
        return tuple(getattr(self, f) for f, _ in self._fields_)


class Event(C.Structure):
    _fields_ = [("kind", C.c_int), ("layer", C.c_int), ("tag", C.c_int),
                ("bytes", C.c_int64), ("used", C.c_int64)]


class TraceSummary(C.Structure):
    _fields_ = [("peak_bytes", C.c_int64), ("static_bytes", C.c_int64), ("offload_bytes", C.c_int64),
                ("prefetch_bytes", C.c_int64), ("pinned_bytes", C.c_int64), ("num_events", C.c_int)]


def build():
    subprocess.check_call(["make", "-s", "-C", HERE], stdout=subprocess.DEVNULL)


_libs = {}


def lib(f32=False):
    name = "liboracle_f32.so" if f32 else "liboracle.so"
    if name not in _libs:
        path = os.path.join(HERE, name)
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        fp = C.POINTER(C.c_float)
        L.orc_net_create.restype = C.c_void_p
        L.orc_net_create.argtypes = [C.POINTER(LayerSpec), C.c_int, C.c_float, C.c_int, C.c_uint64]
        for fn in ("orc_net_dst", "orc_net_grad", "orc_net_weights", "orc_net_bias"):
            getattr(L, fn).restype = fp
            getattr(L, fn).argtypes = [C.c_void_p, C.c_int]
        for fn in ("orc_net_weight_count", "orc_net_src_size", "orc_net_dst_size"):
            getattr(L, fn).restype = C.c_size_t
            getattr(L, fn).argtypes = [C.c_void_p, C.c_int]
        for fn in ("orc_net_input_size", "orc_net_output_size"):
            getattr(L, fn).restype = C.c_size_t
            getattr(L, fn).argtypes = [C.c_void_p]
        for fn in ("orc_net_forward", "orc_net_backward", "orc_net_destroy"):
            getattr(L, fn).restype = None
            getattr(L, fn).argtypes = [C.c_void_p]
        L.orc_net_set_input.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_net_loss.argtypes = [C.c_void_p, C.POINTER(C.c_double)]
        L.orc_model_layers.argtypes = [C.c_int, C.c_int, C.POINTER(LayerSpec), C.c_int]
        L.orc_policy_trace.argtypes = [C.POINTER(LayerSpec), C.c_int, C.c_int, C.POINTER(C.c_int64),
                                       C.c_int, C.c_int, C.POINTER(Event), C.c_int,
                                       C.POINTER(TraceSummary), C.c_int]
        _libs[name] = L
    return _libs[name]


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fill_uniform(n, seed, lo, hi):
    out = np.empty(n, np.float32)
    lib().orc_fill_uniform(_p(out), C.c_size_t(n), C.c_uint64(seed), C.c_float(lo), C.c_float(hi))
    return out


def fill_normal(n, seed, mean=0.0, std=1.0):
    out = np.empty(n, np.float32)
    lib().orc_fill_normal(_p(out), C.c_size_t(n), C.c_uint64(seed), C.c_float(mean), C.c_float(std))
    return out


def fill_onehot(rows, cols, seed):
    out = np.empty((rows, cols), np.float32)
    lib().orc_fill_onehot(_p(out), rows, cols, C.c_uint64(seed))
    return out


def conv_out_dims(h, w, pad, stride, r, s):
    return (h + 2 * pad[0] - r) // stride[0] + 1, (w + 2 * pad[1] - s) // stride[1] + 1


def conv_fwd(x, w, pad, stride, alpha=1.0, beta=0.0, y=None, f32=False):
    x, w = _f32(x), _f32(w)
    n, c, h, wd = x.shape
    k, _, r, s = w.shape
    P, Q = conv_out_dims(h, wd, pad, stride, r, s)
    y = np.zeros((n, k, P, Q), np.float32) if y is None else _f32(y).copy()
    lib(f32).orc_conv_fwd(n, c, h, wd, k, r, s, pad[0], pad[1], stride[0], stride[1],
                          C.c_float(alpha), _p(x), _p(w), C.c_float(beta), _p(y))
    return y


def add_bias(y, bias):
    y = _f32(y).copy()
    bias = _f32(bias)
    n, k = y.shape[:2]
    lib().orc_add_bias(n, k, int(np.prod(y.shape[2:])), _p(bias), _p(y))
    return y


def conv_bwd_data(w, dy, xshape, pad, stride, alpha=1.0, beta=0.0, dx=None, f32=False):
    w, dy = _f32(w), _f32(dy)
    n, c, h, wd = xshape
    k, _, r, s = w.shape
    dx = np.zeros(xshape, np.float32) if dx is None else _f32(dx).copy()
    lib(f32).orc_conv_bwd_data(n, c, h, wd, k, r, s, pad[0], pad[1], stride[0], stride[1],
                               C.c_float(alpha), _p(w), _p(dy), C.c_float(beta), _p(dx))
    return dx


def conv_bwd_bias(dy, alpha=1.0, beta=0.0, db=None):
    dy = _f32(dy)
    n, k = dy.shape[:2]
    db = np.zeros(k, np.float32) if db is None else _f32(db).copy()
    lib().orc_conv_bwd_bias(n, k, int(np.prod(dy.shape[2:])), C.c_float(alpha), _p(dy),
                            C.c_float(beta), _p(db))
    return db


def conv_bwd_filter(x, dy, wshape, pad, stride, alpha=1.0, beta=0.0, dw=None, f32=False):
    x, dy = _f32(x), _f32(dy)
    n, c, h, wd = x.shape
    k, _, r, s = wshape
    dw = np.zeros(wshape, np.float32) if dw is None else _f32(dw).copy()
    lib(f32).orc_conv_bwd_filter(n, c, h, wd, k, r, s, pad[0], pad[1], stride[0], stride[1],
                                 C.c_float(alpha), _p(x), _p(dy), C.c_float(beta), _p(dw))
    return dw


def sgemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, Cm, ldc, f32=False):
    """Column-major cuBLAS semantics; A, B, Cm are flat float32 arrays. Returns the new C."""
    A, B = _f32(A), _f32(B)
    Cm = _f32(Cm).copy()
    lib(f32).orc_sgemm(int(transa), int(transb), m, n, k, C.c_float(alpha), _p(A), lda, _p(B), ldb,
                       C.c_float(beta), _p(Cm), ldc)
    return Cm


def relu_fwd(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_relu_fwd(C.c_size_t(x.size), _p(x), _p(y))
    return y


def act_fwd(mode, x):
    """mode 1 tanh, 2 sigmoid."""
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_act_fwd(C.c_int(mode), C.c_size_t(x.size), _p(x), _p(y))
    return y


def act_bwd(mode, y, dy):
    y, dy = _f32(y), _f32(dy)
    dx = np.empty_like(y)
    lib().orc_act_bwd(C.c_int(mode), C.c_size_t(y.size), _p(y), _p(dy), _p(dx))
    return dx


def relu_bwd(y, dy, x):
    y, dy, x = _f32(y), _f32(dy), _f32(x)
    dx = np.empty_like(x)
    lib().orc_relu_bwd(C.c_size_t(x.size), _p(y), _p(dy), _p(x), _p(dx))
    return dx


def maxpool_fwd(x, win, stride):
    x = _f32(x)
    n, c, h, w = x.shape
    P, Q = (h - win[0]) // stride[0] + 1, (w - win[1]) // stride[1] + 1
    y = np.empty((n, c, P, Q), np.float32)
    lib().orc_maxpool_fwd(n, c, h, w, win[0], win[1], stride[0], stride[1], _p(x), _p(y))
    return y


def maxpool_bwd(y, dy, x, win, stride):
    y, dy, x = _f32(y), _f32(dy), _f32(x)
    n, c, h, w = x.shape
    dx = np.empty_like(x)
    lib().orc_maxpool_bwd(n, c, h, w, win[0], win[1], stride[0], stride[1], _p(y), _p(dy), _p(x), _p(dx))
    return dx


def softmax_fwd(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_softmax_fwd(x.shape[0], int(np.prod(x.shape[1:])), _p(x), _p(y))
    return y


def softmax_bwd(y, dy):
    y, dy = _f32(y), _f32(dy)
    dx = np.empty_like(y)
    lib().orc_softmax_bwd(y.shape[0], int(np.prod(y.shape[1:])), _p(y), _p(dy), _p(dx))
    return dx


def sub(a, b):
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().orc_sub(C.c_size_t(a.size), _p(a), _p(b), _p(out))
    return out


def lrn_fwd(x, win=5, alpha=1e-4, beta=0.75, k=2.0):
    x = _f32(x)
    n, c = x.shape[:2]
    y = np.empty_like(x)
    lib().orc_lrn_fwd(n, c, int(np.prod(x.shape[2:])), win, C.c_float(alpha), C.c_float(beta),
                      C.c_float(k), _p(x), _p(y))
    return y


def lrn_bwd(x, y, dy, win=5, alpha=1e-4, beta=0.75, k=2.0):
    x, y, dy = _f32(x), _f32(y), _f32(dy)
    n, c = x.shape[:2]
    dx = np.empty_like(x)
    lib().orc_lrn_bwd(n, c, int(np.prod(x.shape[2:])), win, C.c_float(alpha), C.c_float(beta),
                      C.c_float(k), _p(x), _p(y), _p(dy), _p(dx))
    return dx


def loss(y, label):
    y, label = _f32(y), _f32(label)
    out = (C.c_double * 2)()
    lib().orc_loss(y.shape[0], int(np.prod(y.shape[1:])), _p(y), _p(label), out)
    return out[0], out[1]


def model_layers(cnn_type, batch):
    arr = (LayerSpec * 64)()
    n = lib().orc_model_layers(cnn_type, batch, arr, 64)
    return [arr[i] for i in range(n)]


def make_specs(tuples):
    arr = (LayerSpec * len(tuples))()
    for i, t in enumerate(tuples):
        arr[i] = t if isinstance(t, LayerSpec) else LayerSpec(*t)
    return arr


def policy_trace(specs, vdnn_type, ws=None, iterations=1, fix_input_leak=False, max_events=8192, wide_workspace=False):
    arr = make_specs(list(specs))
    ev = (Event * max_events)()
    summ = TraceSummary()
    wsp = None
    if ws is not None:
        flat = [int(v) for row in ws for v in row]
        wsp = (C.c_int64 * len(flat))(*flat)
    rc = lib().orc_policy_trace(arr, len(arr), vdnn_type, wsp, iterations, int(fix_input_leak), ev,
                                max_events, C.byref(summ), int(wide_workspace))
    assert rc == 0, "event buffer too small"
    events = [(e.kind, e.layer, e.tag, e.bytes, e.used) for e in ev[:summ.num_events]]
    return events, summ


def dynamic_choice(specs, capacity, ws_perf, fix_input_leak=True):
    """VDNN_DYNAMIC_ALGO as network.cu:946-1008 orders it, decided on the simulated peak of two iterations:
    VDNN_ALL + MEMORY_OPT must fit (else None); then the first of VDNN_NONE, VDNN_CONV, VDNN_ALL that fits
    with the workspace-using algorithms (`ws_perf`: per layer, bytes for forward / data gradient / filter
    gradient); else (VDNN_ALL, "per layer").  Peak bytes ignore fragmentation, so a pool within a few large
    tensors of a peak can be judged differently by a real allocator."""
    BASELINE, VDNN_NONE, VDNN_ALL, VDNN_CONV = 0, 1, 2, 3
    zero = [[0, 0, 0] for _ in specs]

    def fits(policy, ws):
        return policy_trace(specs, policy, ws=ws, iterations=2, fix_input_leak=fix_input_leak)[1].peak_bytes <= capacity

    if not fits(VDNN_ALL, zero):
        return None
    for policy in (VDNN_NONE, VDNN_CONV, VDNN_ALL):
        if fits(policy, ws_perf):
            return policy, 1
    return VDNN_ALL, 2


class Net:
    """Whole-network CPU training step (forward, backward with fused SGD)."""

    def __init__(self, specs, lr, init_mode=0, weight_seed_base=3000, f32=False):
        self._L = lib(f32)
        self.specs = make_specs(list(specs))
        self.h = self._L.orc_net_create(self.specs, len(self.specs), C.c_float(lr), init_mode,
                                        C.c_uint64(weight_seed_base))
        self.num_layers = len(self.specs)

    def close(self):
        if self.h:
            self._L.orc_net_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    @property
    def input_size(self):
        return self._L.orc_net_input_size(self.h)

    @property
    def output_size(self):
        return self._L.orc_net_output_size(self.h)

    def set_input(self, x, label):
        x, label = _f32(x), _f32(label)
        assert x.size == self.input_size and label.size == self.output_size
        self._L.orc_net_set_input(self.h, _p(x), _p(label))

    def forward(self):
        self._L.orc_net_forward(self.h)

    def backward(self):
        self._L.orc_net_backward(self.h)

    def _arr(self, ptr, n):
        return np.ctypeslib.as_array(ptr, shape=(n,)).copy() if n else np.zeros(0, np.float32)

    def dst(self, l):
        return self._arr(self._L.orc_net_dst(self.h, l), self._L.orc_net_dst_size(self.h, l))

    def grad(self, l):
        return self._arr(self._L.orc_net_grad(self.h, l), self._L.orc_net_src_size(self.h, l))

    def weights(self, l):
        n = self._L.orc_net_weight_count(self.h, l)
        return self._arr(self._L.orc_net_weights(self.h, l), n) if n else None

    def bias(self, l):
        n = self._L.orc_net_weight_count(self.h, l)
        return self._arr(self._L.orc_net_bias(self.h, l), self.specs[l].k) if n else None

    def loss(self):
        out = (C.c_double * 2)()
        self._L.orc_net_loss(self.h, out)
        return out[0], out[1]
