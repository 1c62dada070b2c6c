"""The CPU oracle against an independent implementation (PyTorch CPU, float64) and against the
schedule facts read off the reference's network.cu.  No GPU."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import rel_err

CONV_CASES = [  # n, c, h, w, k, r, pad, stride  -- every filter/stride/pad combination of the three networks
    (2, 3, 27, 27, 6, 11, 0, 4),   # AlexNet / OverFeat conv1
    (2, 5, 9, 9, 7, 5, 2, 1),      # AlexNet conv2
    (2, 4, 12, 12, 6, 5, 0, 1),    # OverFeat conv2
    (2, 6, 13, 13, 5, 3, 1, 1),    # 3x3 pad 1 (VGG16, AlexNet, OverFeat)
    (3, 6, 6, 6, 8, 6, 0, 1),      # OverFeat 6x6 valid "FC"
    (2, 8, 1, 1, 4, 1, 0, 1),      # OverFeat 1x1 "FC"
    (1, 1, 5, 7, 1, 3, 1, 1),      # ragged minimum
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_matches_torch(oracle, case):
    n, c, h, w, k, r, pad, st = case
    rng = np.random.default_rng(sum(case))
    x = rng.standard_normal((n, c, h, w), dtype=np.float32)
    wt = rng.standard_normal((k, c, r, r), dtype=np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    wtt = torch.tensor(wt, dtype=torch.float64, requires_grad=True)
    yt = F.conv2d(xt, wtt, stride=st, padding=pad)
    y = oracle.conv_fwd(x, wt, (pad, pad), (st, st))
    assert rel_err(y, yt.detach().numpy()) < 1e-6
    dy = rng.standard_normal(y.shape, dtype=np.float32)
    yt.backward(torch.tensor(dy, dtype=torch.float64))
    assert rel_err(oracle.conv_bwd_data(wt, dy, x.shape, (pad, pad), (st, st)), xt.grad.numpy()) < 1e-6
    # in-place SGD form used by the reference: w <- w + (-lr) * grad
    w0 = rng.standard_normal(wt.shape, dtype=np.float32)
    got = oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st), alpha=-0.25, beta=1.0, dw=w0)
    assert rel_err(got, w0 - 0.25 * wtt.grad.numpy()) < 1e-6
    b0 = rng.standard_normal(k).astype(np.float32)
    assert rel_err(oracle.conv_bwd_bias(dy, alpha=-0.25, beta=1.0, db=b0), b0 - 0.25 * dy.sum((0, 2, 3))) < 1e-5
    # alpha / beta on the forward path
    y0 = rng.standard_normal(y.shape, dtype=np.float32)
    assert rel_err(oracle.conv_fwd(x, wt, (pad, pad), (st, st), alpha=0.5, beta=2.0, y=y0),
                   0.5 * yt.detach().numpy() + 2.0 * y0) < 1e-6


@pytest.mark.parametrize("win,stride,h", [(3, 2, 13), (2, 2, 12), (3, 2, 55), (2, 2, 7)])
def test_maxpool_matches_torch(oracle, win, stride, h):
    rng = np.random.default_rng(h)
    x = rng.standard_normal((2, 3, h, h), dtype=np.float32)
    xt = torch.tensor(x, requires_grad=True)
    yt = F.max_pool2d(xt, win, stride)
    y = oracle.maxpool_fwd(x, (win, win), (stride, stride))
    assert np.array_equal(y, yt.detach().numpy())
    dy = rng.standard_normal(y.shape, dtype=np.float32)
    yt.backward(torch.tensor(dy))
    assert rel_err(oracle.maxpool_bwd(y, dy, x, (win, win), (stride, stride)), xt.grad.numpy()) < 1e-6


def test_maxpool_tie_goes_to_first_element(oracle):
    # pools follow ReLU, so all-zero windows are common: the first element in scan order takes dy
    x = np.zeros((1, 1, 4, 4), np.float32)
    y = oracle.maxpool_fwd(x, (2, 2), (2, 2))
    dy = np.arange(1, 5, dtype=np.float32).reshape(1, 1, 2, 2)
    dx = oracle.maxpool_bwd(y, dy, x, (2, 2), (2, 2))
    expect = np.zeros((4, 4), np.float32)
    expect[0, 0], expect[0, 2], expect[2, 0], expect[2, 2] = 1, 2, 3, 4
    assert np.array_equal(dx[0, 0], expect)


def test_tanh_sigmoid_against_numpy(oracle):
    rng = np.random.default_rng(5)
    x = (3.0 * rng.standard_normal(1000)).astype(np.float32)
    dy = rng.standard_normal(1000).astype(np.float32)
    t = oracle.act_fwd(1, x)
    s = oracle.act_fwd(2, x)
    assert np.allclose(t, np.tanh(x.astype(np.float64)), atol=1e-7)
    assert np.allclose(s, 1.0 / (1.0 + np.exp(-x.astype(np.float64))), atol=1e-7)
    assert np.allclose(oracle.act_bwd(1, t, dy), dy * (1.0 - t.astype(np.float64) ** 2), atol=1e-6)
    assert np.allclose(oracle.act_bwd(2, s, dy), dy * s.astype(np.float64) * (1.0 - s), atol=1e-6)


def test_relu_softmax_lrn_sub(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 1000), dtype=np.float32) * 3
    x[0, :4] = [0.0, -0.0, np.nan, -1.0]
    y = oracle.relu_fwd(x)
    assert y[0, 0] == 0 and y[0, 1] == 0 and np.isnan(y[0, 2]) and y[0, 3] == 0      # PROPAGATE_NAN
    x = np.nan_to_num(x)
    dy = rng.standard_normal(x.shape, dtype=np.float32)
    assert np.array_equal(oracle.relu_bwd(y, dy, x), np.where(x > 0, dy, 0).astype(np.float32))
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    st = F.softmax(xt, 1)
    s = oracle.softmax_fwd(x)
    assert rel_err(s, st.detach().numpy()) < 1e-6
    st.backward(torch.tensor(dy, dtype=torch.float64))
    assert rel_err(oracle.softmax_bwd(st.detach().numpy().astype(np.float32), dy), xt.grad.numpy()) < 1e-5
    assert np.array_equal(oracle.sub(s, dy), s - dy)
    x4 = rng.standard_normal((2, 9, 5, 5), dtype=np.float32) * 4
    xt = torch.tensor(x4, dtype=torch.float64, requires_grad=True)
    lt = F.local_response_norm(xt, 5, 1e-4, 0.75, 2.0)
    l = oracle.lrn_fwd(x4)
    assert rel_err(l, lt.detach().numpy()) < 1e-6
    d4 = rng.standard_normal(x4.shape, dtype=np.float32)
    lt.backward(torch.tensor(d4, dtype=torch.float64))
    assert rel_err(oracle.lrn_bwd(x4, l, d4), xt.grad.numpy()) < 1e-6


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_sgemm_column_major(oracle, ta, tb):
    rng = np.random.default_rng(ta * 2 + tb)
    m, n, k = 7, 5, 9
    A = rng.standard_normal((k, m) if not ta else (m, k), dtype=np.float32)     # numpy rows = BLAS columns
    B = rng.standard_normal((n, k) if not tb else (k, n), dtype=np.float32)
    Cm = rng.standard_normal((n, m), dtype=np.float32)
    opA = A.T if not ta else A
    opB = B.T if not tb else B
    ref = (0.5 * opA.astype(np.float64) @ opB + 2 * Cm.T).T
    out = oracle.sgemm(ta, tb, m, n, k, 0.5, A.ravel(), A.shape[1], B.ravel(), B.shape[1], 2.0, Cm.ravel(), m)
    assert rel_err(out.reshape(n, m), ref) < 1e-6


def test_network_step_matches_torch_autograd(oracle):
    """Whole step on a small topology: forward values, the (y - label) seed, input gradient and the
    fused SGD update against autograd on the loss 0.5*sum((softmax - label)^2)."""
    from helpers import tiny_net
    specs = tiny_net(3, with_lrn=True)
    lr = 0.05
    net = oracle.Net(specs, lr, init_mode=0)
    x = oracle.fill_normal(net.input_size, 1000)
    t = oracle.fill_onehot(3, 10, 2000)
    net.set_input(x, t)
    params = {l: (net.weights(l), net.bias(l)) for l in range(net.num_layers) if net.weights(l) is not None}
    net.forward()
    net.backward()
    # torch model with the same parameters
    xt = torch.tensor(x.reshape(3, 3, 20, 20), dtype=torch.float64, requires_grad=True)
    P = {l: (torch.tensor(w, dtype=torch.float64, requires_grad=True), torch.tensor(b, dtype=torch.float64, requires_grad=True))
         for l, (w, b) in params.items()}
    h = xt
    for l, s in enumerate(specs):
        ty = s[0]
        if ty == 2:
            h = F.conv2d(h, P[l][0].reshape(s[9], s[2], s[10], s[11]), P[l][1], stride=s[7], padding=s[5])
        elif ty == 3:
            h = F.relu(h)
        elif ty == 9:
            h = F.local_response_norm(h, 5, 1e-4, 0.75, 2.0)
        elif ty == 7:
            h = F.max_pool2d(h, s[10], s[7])
        elif ty == 0:
            h = F.linear(h.reshape(3, -1), P[l][0].reshape(s[9], s[2]), P[l][1])
        elif ty == 6:
            h = F.softmax(h.reshape(3, -1), 1)
        assert rel_err(net.dst(l), h.detach().numpy()) < 1e-5, l
    loss = 0.5 * ((h - torch.tensor(t, dtype=torch.float64)) ** 2).sum()
    loss.backward()
    assert rel_err(net.grad(0), xt.grad.numpy()) < 1e-5
    for l, (w, b) in params.items():
        assert rel_err(net.weights(l), w - lr * P[l][0].grad.numpy().ravel()) < 1e-5, l
        assert rel_err(net.bias(l), b - lr * P[l][1].grad.numpy().ravel()) < 1e-5, l
    sq, ce = net.loss()
    assert abs(sq - float(loss.detach()) / 3) < 1e-6


def test_topologies_follow_reference_tables(oracle):
    # layer counts and the shapes that network.cu spells out
    a = oracle.model_layers(oracle.ALEXNET, 128)
    assert len(a) == 19 and a[0].astuple() == (2, 128, 3, 227, 227, 0, 0, 4, 4, 96, 11, 11)
    assert a[13].astuple() == (0, 128, 9216, 1, 1, 0, 0, 0, 0, 4096, 1, 1)
    o = oracle.model_layers(oracle.OVERFEAT, 128)
    assert len(o) == 19 and o[13].astuple() == (2, 128, 1024, 6, 6, 0, 0, 1, 1, 3072, 6, 6)
    v = oracle.model_layers(oracle.VGG16_128, 128)
    assert len(v) == 37 and v[31].astuple() == (0, 128, 25088, 1, 1, 0, 0, 0, 0, 4096, 1, 1)
    assert len(oracle.model_layers(oracle.ALEXNET_LRN, 128)) == 21


def _prefetch_pairs(oracle, model, batch, policy):
    ev, _ = oracle.policy_trace(oracle.model_layers(model, batch), policy)
    pairs, cur = [], None
    # the layer whose backward issues a prefetch is the one that allocates its gradData just before it
    for kind, layer, tag, _, _ in ev:
        if kind == oracle.EV_ALLOC and tag == oracle.TAG_GRAD:
            cur = layer
        if kind == oracle.EV_PREFETCH:
            pairs.append((cur, layer))
    return pairs


def test_prefetch_schedule(oracle):
    # worked out by hand from findPrefetchLayer (network.cu:1198-1207) and the layer tables
    assert _prefetch_pairs(oracle, oracle.VGG16_128, 128, oracle.VDNN_CONV) == [
        (36, 28), (28, 26), (26, 24), (24, 21), (21, 19), (19, 17), (17, 14), (14, 12), (12, 10), (10, 7), (7, 5), (5, 2), (2, 0)]
    assert _prefetch_pairs(oracle, oracle.ALEXNET, 128, oracle.VDNN_CONV) == [(18, 10), (10, 8), (8, 6), (6, 3), (3, 0)]
    assert _prefetch_pairs(oracle, oracle.OVERFEAT, 128, oracle.VDNN_CONV) == [
        (18, 17), (17, 15), (15, 13), (13, 10), (10, 8), (8, 6), (6, 3), (3, 0)]
    assert _prefetch_pairs(oracle, oracle.VGG16_64, 64, oracle.VDNN_ALL) == [(l, l - 1) for l in range(36, 0, -1)]
    assert _prefetch_pairs(oracle, oracle.ALEXNET, 128, oracle.VDNN_NONE) == []


PEAKS = {  # pool high-water marks in bytes with zero workspace: BASELINE, NONE, ALL, CONV
    ("ALEXNET", 128): (1364340736, 1097141760, 1003062272, 1044581888),
    ("ALEXNET_LRN", 128): (1608577024, 1341378048, 1072598528, 1288818176),
    ("OVERFEAT", 128): (1895851520, 1711326720, 1364683776, 1616168448),
    ("VGG16_64", 64): (9569200640, 7965284352, 4702640128, 5833005056),
    ("VGG16_128", 128): (18584969728, 15377137664, 8851849216, 11112579072),
}


@pytest.mark.parametrize("key", sorted(PEAKS))
def test_peak_bytes_per_policy(oracle, key):
    model = getattr(oracle, key[0])
    specs = oracle.model_layers(model, key[1])
    got = tuple(oracle.policy_trace(specs, p)[1].peak_bytes for p in range(4))
    assert got == PEAKS[key]
    ev, s = oracle.policy_trace(specs, oracle.VDNN_ALL)
    assert s.offload_bytes == s.prefetch_bytes == s.pinned_bytes
    assert s.offload_bytes == sum(4 * x.n * x.c * x.h * x.w for x in specs[:-1])


def test_input_leak_is_replayed_or_fixed(oracle):
    specs = oracle.model_layers(oracle.ALEXNET, 16)
    leak = [oracle.policy_trace(specs, oracle.VDNN_ALL, iterations=i)[0][-1][4] for i in (1, 2, 3)]
    fixed = [oracle.policy_trace(specs, oracle.VDNN_ALL, iterations=i, fix_input_leak=True)[0][-1][4] for i in (1, 2, 3)]
    in_bytes = (4 * 16 * 3 * 227 * 227 + 511) // 512 * 512
    assert leak[1] - leak[0] == in_bytes and leak[2] - leak[1] == in_bytes     # network.cu:1156,1185
    assert fixed[0] == fixed[1] == fixed[2]


def test_rng_is_counter_based(oracle):
    a = oracle.fill_normal(1000, 7)
    b = oracle.fill_normal(2000, 7)
    assert np.array_equal(a, b[:1000])
    assert abs(float(oracle.fill_normal(200000, 1).std()) - 1.0) < 0.01
    u = oracle.fill_uniform(100000, 3, -0.01, 0.01)
    assert u.min() >= -0.01 and u.max() < 0.01
    oh = oracle.fill_onehot(64, 1000, 9)
    assert (oh.sum(1) == 1).all()
