"""Parity of every layer kernel with the CPU oracle, called through the C ABI on a B200.
PyTorch only owns the device buffers.  Tolerance for floating point: tensor-normalised
max|a-b| <= 1e-4 * max|b| (the bar the specification states for activations and gradients);
integer-like results (ReLU masks, pooling routes) must be exact."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


CONV_CASES = [  # n, c, h, w, k, r, pad, stride
    (2, 3, 27, 27, 6, 11, 0, 4),
    (2, 5, 9, 9, 7, 5, 2, 1),
    (2, 4, 12, 12, 6, 5, 0, 1),
    (2, 6, 13, 13, 5, 3, 1, 1),
    (3, 6, 6, 6, 8, 6, 0, 1),
    (2, 8, 1, 1, 4, 1, 0, 1),
    (1, 1, 5, 7, 1, 3, 1, 1),
    (4, 64, 28, 28, 128, 3, 1, 1),     # several full tiles, K = 576
    (3, 3, 32, 32, 64, 3, 1, 1),       # first-layer shape (C = 3, K = 27)
    (2, 130, 7, 7, 130, 3, 1, 1),      # ragged tile edges in every dimension
    (2, 3, 17, 17, 8, 5, 2, 2),        # few input channels with stride and padding: the phase-class data gradient
    (2, 2, 12, 12, 5, 3, 1, 2),
    (2, 4, 11, 11, 6, 3, 0, 3),
    (1, 3, 70, 150, 9, 3, 1, 1),       # wider than one 128-column tile of that kernel
    # stride 1 with reduction channels in whole blocks of 32: in PERF_OPT forward and data gradient fetch their operand by
    # tensor copies from channels-last images (boxes of 32 pixels, zero fill outside the image)
    (2, 32, 14, 14, 40, 3, 1, 1),      # 14 x 14 grid under 16 x 2 boxes: overhang on both edges, 40 of 64 columns used
    (3, 64, 13, 13, 96, 5, 2, 1),      # 5 x 5 taps, padding 2, odd grid
    (2, 96, 12, 12, 32, 5, 0, 1),      # no padding: the output grid (8 x 8) is smaller than the image
    (1, 256, 9, 30, 288, 3, 1, 1),     # 256-column tile plus a ragged second one, wide rows
    (2, 32, 10, 10, 64, 1, 0, 1),      # 1 x 1 filter
    (5, 32, 7, 7, 32, 3, 2, 1),        # padding beyond the filter radius: the output grid (9 x 9) is larger than the image
    (2, 512, 6, 6, 64, 3, 1, 1),       # one output tile, 4608-long reduction: split along k with partial sums
    (9, 64, 40, 24, 64, 3, 1, 1),      # many tiles of 64 columns, tiles that straddle images
    (2, 32, 12, 12, 160, 3, 1, 1),     # 256-column tiles on CTA pairs with an odd number of row tiles: the last pair is half empty
    (3, 288, 10, 10, 512, 3, 1, 1),    # two full 256-column tiles, 81 row groups (ragged last row tile), pairs in every kernel
    (2, 128, 16, 16, 128, 3, 1, 1),    # 128 filters, 36 row groups: the filter gradient's two-half tiles (the fifth is half empty)
]
ENGINES = ["ffma", "tcgen05"]


def _engine(vdnn, name):
    vdnn.ops.set_engine({"ffma": vdnn.ENGINE_FFMA, "tcgen05": vdnn.ENGINE_TCGEN05, "auto": vdnn.ENGINE_AUTO}[name])


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("algo", [0, 1])
@pytest.mark.parametrize("case", CONV_CASES)
def test_convolution_trio(vdnn, oracle, case, algo, engine):
    n, c, h, w, k, r, pad, st = case
    ops = vdnn.ops
    _engine(vdnn, engine)
    try:
        rng = np.random.default_rng(sum(case) + algo)
        x = rng.standard_normal((n, c, h, w), dtype=np.float32)
        wt = (rng.standard_normal((k, c, r, r), dtype=np.float32) * 0.2).astype(np.float32)
        bias = rng.standard_normal(k).astype(np.float32)
        d = ops.conv_desc(n, c, h, w, k, r, r, (pad, pad), (st, st))
        P, Q = ops.conv_out_dims(d)
        ws_bytes = max(ops.conv_workspace_bytes(op, algo, d) for op in range(3))
        ws = torch.empty(max(ws_bytes, 4) // 4, dtype=torch.float32, device="cuda")
        # forward with the bias in the same pass
        xd, wd, bd = dev(x), dev(wt), dev(bias)
        yd = torch.full((n, k, P, Q), 7.0, device="cuda")
        ops.conv_fwd(d, xd, wd, yd, bias=bd, algo_mode=algo, workspace=ws, workspace_bytes=ws_bytes)
        want = oracle.add_bias(oracle.conv_fwd(x, wt, (pad, pad), (st, st)), bias)
        assert rel_err(host(yd), want) < TOL
        # forward with alpha / beta and a separate bias add (the reference's two calls)
        y0 = rng.standard_normal((n, k, P, Q), dtype=np.float32)
        yd = dev(y0)
        ops.conv_fwd(d, xd, wd, yd, alpha=0.5, beta=2.0, algo_mode=algo, workspace=ws, workspace_bytes=ws_bytes)
        ops.add_bias(n, k, P * Q, bd, yd)
        want2 = oracle.add_bias(oracle.conv_fwd(x, wt, (pad, pad), (st, st), alpha=0.5, beta=2.0, y=y0), bias)
        assert rel_err(host(yd), want2) < TOL
        # data gradient
        dy = rng.standard_normal((n, k, P, Q), dtype=np.float32)
        dyd = dev(dy)
        dxd = torch.full((n, c, h, w), -3.0, device="cuda")
        ops.conv_bwd_data(d, wd, dyd, dxd, algo_mode=algo, workspace=ws, workspace_bytes=ws_bytes)
        assert rel_err(host(dxd), oracle.conv_bwd_data(wt, dy, x.shape, (pad, pad), (st, st))) < TOL
        # filter and bias gradient folded into the parameters: w += -lr * grad (alpha = -lr, beta = 1)
        lr = 0.01
        wupd = dev(wt)
        ops.conv_bwd_filter(d, xd, dyd, wupd, alpha=-lr, beta=1.0, algo_mode=algo, workspace=ws, workspace_bytes=ws_bytes)
        assert rel_err(host(wupd), oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st), alpha=-lr, beta=1.0, dw=wt)) < TOL
        # plain gradient (alpha = 1, beta = 0), as the data-parallel path stages it
        gd = torch.full((k, c, r, r), 5.0, device="cuda")
        ops.conv_bwd_filter(d, xd, dyd, gd, algo_mode=algo, workspace=ws, workspace_bytes=ws_bytes)
        assert rel_err(host(gd), oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st))) < TOL
        bupd = dev(bias)
        ops.conv_bwd_bias(n, k, P * Q, dyd, bupd, alpha=-lr, beta=1.0)
        assert rel_err(host(bupd), oracle.conv_bwd_bias(dy, alpha=-lr, beta=1.0, db=bias)) < TOL
        # both gradients in one call (where the filter gradient prepares dy as operand images, that pass sums dy per
        # channel): folded into the parameters, then staged
        wupd, bupd = dev(wt), dev(bias)
        ops.conv_bwd_filter_bias(d, xd, dyd, wupd, bupd, alpha=-lr, beta=1.0, alpha_b=-lr, beta_b=1.0, algo_mode=algo, workspace=ws,
                                 workspace_bytes=ws_bytes)
        assert rel_err(host(wupd), oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st), alpha=-lr, beta=1.0, dw=wt)) < TOL
        assert rel_err(host(bupd), oracle.conv_bwd_bias(dy, alpha=-lr, beta=1.0, db=bias)) < TOL
        gd, gb = torch.full((k, c, r, r), 5.0, device="cuda"), torch.full((k,), 9.0, device="cuda")
        ops.conv_bwd_filter_bias(d, xd, dyd, gd, gb, algo_mode=algo, workspace=ws, workspace_bytes=ws_bytes)
        assert rel_err(host(gd), oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st))) < TOL
        assert rel_err(host(gb), oracle.conv_bwd_bias(dy)) < TOL
        # the three gradients in one call and one workspace (one pass over dy where both gradients are TMA-fed); dw aliases
        # w as in training: the data gradient must see the weights as they were
        need = ops.conv_workspace_bytes(3, algo, d)
        assert need <= max(ws_bytes, ops.conv_workspace_bytes(2, algo, d))
        ws3 = torch.empty(max(need, 4) // 4, dtype=torch.float32, device="cuda")
        wupd, bupd = dev(wt), dev(bias)
        dxd = torch.full((n, c, h, w), -3.0, device="cuda")
        ops.conv_bwd_data_filter_bias(d, wupd, xd, dyd, dxd, wupd, bupd, alpha_w=-lr, beta_w=1.0, alpha_b=-lr, beta_b=1.0, algo_mode=algo,
                                      workspace=ws3, workspace_bytes=need)
        assert rel_err(host(dxd), oracle.conv_bwd_data(wt, dy, x.shape, (pad, pad), (st, st))) < TOL
        assert rel_err(host(wupd), oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st), alpha=-lr, beta=1.0, dw=wt)) < TOL
        assert rel_err(host(bupd), oracle.conv_bwd_bias(dy, alpha=-lr, beta=1.0, db=bias)) < TOL
        assert ops.engine_status() == 0
    finally:
        _engine(vdnn, "auto")


def test_perf_opt_filter_gradient_is_deterministic(vdnn):
    ops = vdnn.ops
    n, c, h, w, k = 8, 32, 28, 28, 32
    d = ops.conv_desc(n, c, h, w, k, 3, 3, (1, 1), (1, 1))
    need = ops.conv_workspace_bytes(2, 1, d)
    assert need > 0
    x = torch.randn(n, c, h, w, device="cuda")
    dy = torch.randn(n, k, h, w, device="cuda")
    ws = torch.empty(need // 4, device="cuda")
    outs = []
    for _ in range(3):
        g = torch.empty(k, c, 3, 3, device="cuda")
        ops.conv_bwd_filter(d, x, dy, g, algo_mode=1, workspace=ws, workspace_bytes=need)
        outs.append(host(g).copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    # too little workspace is an error, not a silent change of algorithm
    with pytest.raises(vdnn.VdnnError) as e:
        ops.conv_bwd_filter(d, x, dy, g, algo_mode=1, workspace=ws, workspace_bytes=need - 4)
    assert e.value.status == -3


SGEMM_CASES = [  # transa, transb, m, n, k  (the five cublasSgemm shapes of the FC layers, scaled down, plus ragged)
    (1, 0, 96, 16, 200),      # forward      W^T X
    (0, 0, 200, 16, 96),      # data grad    W dY
    (0, 1, 200, 96, 16),      # filter grad  X dY^T
    (0, 0, 96, 16, 1),        # bias broadcast (rank 1)
    (0, 0, 96, 1, 16),        # bias gradient
    (1, 1, 33, 45, 67),
    (1, 0, 1000, 128, 4096),  # VGG16 fc3 at full size
    (0, 1, 300, 260, 128),
]


@pytest.mark.parametrize("engine", ENGINES)
@pytest.mark.parametrize("algo", [0, 1])
@pytest.mark.parametrize("case", SGEMM_CASES)
def test_sgemm(vdnn, oracle, case, algo, engine):
    ta, tb, m, n, k = case
    ops = vdnn.ops
    _engine(vdnn, engine)
    try:
        rng = np.random.default_rng(m * 7 + n + k + algo)
        lda = (k if ta else m) + 3
        ldb = (n if tb else k) + 1
        A = rng.standard_normal(lda * (m if ta else k), dtype=np.float32)
        B = rng.standard_normal(ldb * (k if tb else n), dtype=np.float32)
        for ldc, alpha, beta in [(m, 1.0, 0.0), (m, -0.01, 1.0), (m + 5, 0.5, 2.0)]:
            C0 = rng.standard_normal(ldc * n, dtype=np.float32)
            Cd = dev(C0)
            need = ops.sgemm_workspace_bytes(algo, m, n, k)
            ws = torch.empty(max(need, 4) // 4, device="cuda")
            ops.sgemm(ta, tb, m, n, k, alpha, dev(A), lda, dev(B), ldb, beta, Cd, ldc, algo_mode=algo, workspace=ws,
                      workspace_bytes=need)
            want = oracle.sgemm(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C0, ldc)
            got = host(Cd)
            # only the m x n window is defined; the padding rows of C must be untouched
            assert rel_err(got.reshape(n, ldc)[:, :m], want.reshape(n, ldc)[:, :m]) < TOL
            assert np.array_equal(got.reshape(n, ldc)[:, m:], C0.reshape(n, ldc)[:, m:])
        assert ops.engine_status() == 0
    finally:
        _engine(vdnn, "auto")


@pytest.mark.parametrize("count", [1, 3, 1024, 4097, 3 * 224 * 224 + 1])
def test_relu(vdnn, oracle, count):
    ops = vdnn.ops
    rng = np.random.default_rng(count)
    x = rng.standard_normal(count, dtype=np.float32)
    x[0] = 0.0
    if count > 2:
        x[1], x[2] = np.nan, -0.0
    xd = dev(x)
    yd = torch.empty_like(xd)
    ops.relu_fwd(count, xd, yd)
    y = host(yd)
    assert np.array_equal(y, oracle.relu_fwd(x), equal_nan=True)
    dy = rng.standard_normal(count, dtype=np.float32)
    dxd = torch.empty_like(xd)
    ops.relu_bwd(count, yd, dev(dy), xd, dxd)
    assert np.array_equal(host(dxd), oracle.relu_bwd(y, dy, x))
    # unaligned views take the scalar path
    if count > 8:
        big = dev(np.concatenate([[0.0], x]))
        out = torch.zeros(count + 1, device="cuda")
        ops.relu_fwd(count, big.data_ptr() + 4, out.data_ptr() + 4)
        assert np.array_equal(host(out)[1:], oracle.relu_fwd(x), equal_nan=True)


POOL_CASES = [  # n, c, h, w, win, stride
    (2, 3, 55, 55, 3, 2), (2, 4, 27, 27, 3, 2), (2, 5, 13, 13, 3, 2),      # AlexNet (overlapping)
    (2, 3, 56, 56, 2, 2), (2, 3, 24, 24, 2, 2), (3, 7, 12, 12, 2, 2),      # OverFeat / VGG (fast path)
    (2, 3, 14, 14, 2, 2), (1, 2, 7, 7, 2, 2), (1, 1, 6, 10, 2, 2),         # W % 4 != 0, odd sizes: generic path
]


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("count", [1, 5, 4096, 3 * 55 * 55 + 3])
def test_tanh_sigmoid(vdnn, oracle, mode, count):
    """The two activation modes besides ReLU that the reference's Layer accepts (layer.cu:361-368)."""
    ops = vdnn.ops
    rng = np.random.default_rng(100 * mode + count)
    x = (4.0 * rng.standard_normal(count)).astype(np.float32)
    x[0] = 0.0
    xd = dev(x)
    yd = torch.empty_like(xd)
    ops.activation_fwd(mode, count, xd, yd)
    y = host(yd)
    assert np.abs(y - oracle.act_fwd(mode, x)).max() < 3e-7          # values are in [-1, 1]: a few ulp
    dy = rng.standard_normal(count, dtype=np.float32)
    dxd = torch.empty_like(xd)
    ops.activation_bwd(mode, count, yd, dev(dy), xd, dxd)
    assert rel_err(host(dxd), oracle.act_bwd(mode, y, dy)) < 1e-6
    # mode 0 is the ReLU entry point
    ops.activation_fwd(0, count, xd, yd)
    assert np.array_equal(host(yd), oracle.relu_fwd(x))
    with pytest.raises(vdnn.VdnnError):
        ops.activation_fwd(3, count, xd, yd)


@pytest.mark.parametrize("case", POOL_CASES)
@pytest.mark.parametrize("ties", [False, True])
def test_maxpool(vdnn, oracle, case, ties):
    n, c, h, w, win, st = case
    ops = vdnn.ops
    rng = np.random.default_rng(h * 31 + w + win)
    x = rng.standard_normal((n, c, h, w), dtype=np.float32)
    if ties:
        x = np.maximum(x, 0).astype(np.float32)        # what a pool sees after ReLU: many equal zeros
        x[:, :, : h // 2] = 0
    P, Q = (h - win) // st + 1, (w - win) // st + 1
    xd = dev(x)
    yd = torch.empty(n, c, P, Q, device="cuda")
    ops.maxpool_fwd(n, c, h, w, (win, win), (st, st), xd, yd)
    y = host(yd)
    assert np.array_equal(y, oracle.maxpool_fwd(x, (win, win), (st, st)))
    dy = rng.standard_normal((n, c, P, Q), dtype=np.float32)
    dxd = torch.full((n, c, h, w), 9.0, device="cuda")
    ops.maxpool_bwd(n, c, h, w, (win, win), (st, st), yd, dev(dy), xd, dxd)
    want = oracle.maxpool_bwd(y, dy, x, (win, win), (st, st))
    assert rel_err(host(dxd), want) < 1e-6
    assert np.array_equal(host(dxd) != 0, want != 0)


def test_softmax_sub_loss(vdnn, oracle):
    ops = vdnn.ops
    rng = np.random.default_rng(3)
    for rows, cols in [(128, 1000), (3, 10), (5, 33)]:
        x = (rng.standard_normal((rows, cols), dtype=np.float32) * 4).astype(np.float32)
        xd = dev(x)
        yd = torch.empty_like(xd)
        ops.softmax_fwd(rows, cols, xd, yd)
        y = host(yd)
        assert rel_err(y, oracle.softmax_fwd(x)) < 1e-5
        label = oracle.fill_onehot(rows, cols, 2000)
        dd = torch.empty_like(xd)
        ops.sub(rows * cols, yd, dev(label), dd)
        assert np.array_equal(host(dd), oracle.sub(y, label))
        dxd = torch.empty_like(xd)
        ops.softmax_bwd(rows, cols, yd, dd, dxd)
        assert rel_err(host(dxd), oracle.softmax_bwd(y, host(dd))) < 1e-5
        out = torch.zeros(2, dtype=torch.float64, device="cuda")
        ops.loss(rows, cols, yd, dev(label), out)
        sq, ce = oracle.loss(y, label)
        got = host(out)
        assert abs(got[0] - sq) < 1e-5 * max(1.0, abs(sq)) and abs(got[1] - ce) < 1e-5 * max(1.0, abs(ce))


@pytest.mark.parametrize("shape", [(2, 96, 55 * 55), (2, 256, 27 * 27), (3, 7, 5), (1, 3, 1)])
def test_lrn(vdnn, oracle, shape):
    n, c, hw = shape
    ops = vdnn.ops
    rng = np.random.default_rng(c)
    x = (rng.standard_normal((n, c, hw), dtype=np.float32) * 5).astype(np.float32)
    xd = dev(x)
    yd = torch.empty_like(xd)
    ops.lrn_fwd(n, c, hw, xd, yd)
    y = host(yd)
    assert rel_err(y, oracle.lrn_fwd(x)) < 1e-5
    dy = rng.standard_normal((n, c, hw), dtype=np.float32)
    dxd = torch.empty_like(xd)
    ops.lrn_bwd(n, c, hw, xd, yd, dev(dy), dxd)
    assert rel_err(host(dxd), oracle.lrn_bwd(x, y, dy)) < 1e-5


def test_axpy_fill_bias(vdnn, oracle):
    ops = vdnn.ops
    rng = np.random.default_rng(11)
    g = rng.standard_normal(100003, dtype=np.float32)
    w = rng.standard_normal(100003, dtype=np.float32)
    wd = dev(w)
    ops.axpy(g.size, -0.01, dev(g), wd)
    assert rel_err(host(wd), w + np.float32(-0.01) * g) < 1e-6
    t = torch.empty(1000, device="cuda")
    ops.fill(1000, 1.0, t)
    assert (host(t) == 1.0).all()
    # FC-shaped bias add / bias gradient (pq = 1)
    y = rng.standard_normal((128, 1000), dtype=np.float32)
    b = rng.standard_normal(1000).astype(np.float32)
    yd = dev(y)
    ops.add_bias(128, 1000, 1, dev(b), yd)
    assert np.array_equal(host(yd), oracle.add_bias(y.reshape(128, 1000, 1), b).reshape(128, 1000))
    bd = dev(b)
    ops.conv_bwd_bias(128, 1000, 1, dev(y), bd, alpha=-0.01, beta=1.0)
    assert rel_err(host(bd), oracle.conv_bwd_bias(y.reshape(128, 1000, 1), alpha=-0.01, beta=1.0, db=b)) < 1e-5


def test_offload_prefetch_round_trip(vdnn):
    L = vdnn.lib()
    n = 1 << 20
    src = torch.randn(n, device="cuda")
    pinned = torch.empty(n, pin_memory=True)
    back = torch.zeros(n, device="cuda")
    s = torch.cuda.Stream()
    ready, done = torch.cuda.Event(), torch.cuda.Event()
    ready.record()
    assert L.vdnn_offload(C.c_void_p(pinned.data_ptr()), C.c_void_p(src.data_ptr()), n * 4, C.c_void_p(ready.cuda_event),
                          None, C.c_void_p(s.cuda_stream)) == 0
    assert L.vdnn_prefetch(C.c_void_p(back.data_ptr()), C.c_void_p(pinned.data_ptr()), n * 4, None, None,
                           C.c_void_p(s.cuda_stream)) == 0
    s.synchronize()
    assert torch.equal(src, back)
