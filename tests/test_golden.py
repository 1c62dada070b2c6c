"""Pins the CPU oracle to what the reference itself computed on a B200 (its own Layer class on cuDNN 9.10 /
cuBLAS, FMA arithmetic) and to the memory figures its program printed.  The fixtures under tests/golden/
were produced by tests/golden/make_golden.py.  No GPU."""
import json
import os

import numpy as np
import pytest

from helpers import rel_err

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LAYERS = json.load(open(os.path.join(GOLD, "ref_layers.json")))
ARR = np.load(os.path.join(GOLD, "ref_layers.npz"))
MEMORY = json.load(open(os.path.join(GOLD, "ref_memory.json")))
CASES = {c["id"]: c for c in LAYERS["cases"]}
TOL = 1e-5      # cuDNN / cuBLAS fp32 (FMA) against a double-accumulating restatement


def _inputs(oracle, cid, xs, ws, bs, ys, wstd):
    x = oracle.fill_normal(xs, 100 * cid + 1)
    w = oracle.fill_normal(ws, 100 * cid + 2, 0.0, wstd) if ws else None
    b = oracle.fill_normal(bs, 100 * cid + 3) if bs else None
    dy = oracle.fill_normal(ys, 100 * cid + 4)
    return x, w, b, dy


@pytest.mark.parametrize("cid", [c["id"] for c in LAYERS["cases"] if c["kind"] == "conv"])
def test_convolution_layer_against_reference(oracle, cid):
    c = CASES[cid]
    n, ch, h, w, k, r, pad, st, P, Q = (c[x] for x in ("n", "c", "h", "w", "k", "r", "pad", "stride", "p", "q"))
    x, wt, b, dy = _inputs(oracle, cid, n * ch * h * w, k * ch * r * r, k, n * k * P * Q, 0.2)
    x, wt, dy = x.reshape(n, ch, h, w), wt.reshape(k, ch, r, r), dy.reshape(n, k, P, Q)
    assert oracle.conv_out_dims(h, w, (pad, pad), (st, st), r, r) == (P, Q)
    y = oracle.add_bias(oracle.conv_fwd(x, wt, (pad, pad), (st, st)), b)
    assert rel_err(y, ARR[f"conv{cid}_y"]) < TOL
    assert rel_err(oracle.conv_bwd_data(wt, dy, x.shape, (pad, pad), (st, st)), ARR[f"conv{cid}_dx"]) < TOL
    lr = np.float32(c["lr"])
    zero_w, zero_b = np.zeros_like(wt), np.zeros(k, np.float32)
    wstep = oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st), alpha=-lr, beta=1.0, dw=zero_w)
    bstep = oracle.conv_bwd_bias(dy, alpha=-lr, beta=1.0, db=zero_b)
    assert rel_err(wstep, ARR[f"conv{cid}_wstep"]) < TOL      # in-place SGD: w <- w + (-lr) * grad
    assert rel_err(bstep, ARR[f"conv{cid}_bstep"]) < TOL


@pytest.mark.parametrize("cid", [c["id"] for c in LAYERS["cases"] if c["kind"] == "fc"])
def test_fully_connected_layer_against_reference(oracle, cid):
    c = CASES[cid]
    n, cin, cout = c["n"], c["cin"], c["cout"]
    x, wt, b, dy = _inputs(oracle, cid, n * cin, cin * cout, cout, n * cout, 0.1)
    lr = np.float32(c["lr"])
    # the three cublasSgemm calls of layer.cu:677-744 with the reference's operand order
    y = oracle.sgemm(1, 0, cout, n, cin, 1.0, wt, cin, x, cin, 0.0, np.zeros(n * cout, np.float32), cout)
    y = oracle.add_bias(y.reshape(n, cout, 1), b).ravel()
    assert rel_err(y, ARR[f"fc{cid}_y"]) < TOL
    dx = oracle.sgemm(0, 0, cin, n, cout, 1.0, wt, cin, dy, cout, 0.0, np.zeros(n * cin, np.float32), cin)
    assert rel_err(dx, ARR[f"fc{cid}_dx"]) < TOL
    wstep = oracle.sgemm(0, 1, cin, cout, n, -lr, x, cin, dy, cout, 1.0, np.zeros(cin * cout, np.float32), cin)
    assert rel_err(wstep, ARR[f"fc{cid}_wstep"]) < TOL
    bstep = oracle.conv_bwd_bias(dy.reshape(n, cout, 1), alpha=-lr, beta=1.0, db=np.zeros(cout, np.float32))
    assert rel_err(bstep, ARR[f"fc{cid}_bstep"]) < TOL


def _simple_input(oracle, c):
    n, ch, h, w = c["n"], c["c"], c["h"], c["w"]
    std = 4.0 if c["kind"] == "softmax" else 1.0
    x = oracle.fill_normal(n * ch * h * w, 100 * c["id"] + 1, 0.0, std).reshape(n, ch, h, w)
    if c["mode"] == 1:
        rows = np.arange(h).reshape(1, 1, h, 1)
        x = np.where((x > 0) & (rows >= h // 2), x, 0).astype(np.float32)
    elif c["mode"] == 2:
        x = np.ones_like(x)
    dy = oracle.fill_normal(n * ch * c["p"] * c["q"], 100 * c["id"] + 4).reshape(n, ch, c["p"], c["q"])
    return x, dy


@pytest.mark.parametrize("cid", [c["id"] for c in LAYERS["cases"] if c["kind"] == "pool"])
def test_max_pooling_against_reference_including_ties(oracle, cid):
    """Modes 1 and 2 are full of equal values inside a window: this is where cuDNN's undocumented
    routing rule shows, and the oracle's rule (first maximum in scan order) has to reproduce it."""
    c = CASES[cid]
    x, dy = _simple_input(oracle, c)
    win, st = (c["win"], c["win"]), (c["stride"], c["stride"])
    y = oracle.maxpool_fwd(x, win, st)
    assert np.array_equal(y.ravel(), ARR[f"pool{cid}_y"])
    dx = oracle.maxpool_bwd(y, dy, x, win, st)
    assert rel_err(dx, ARR[f"pool{cid}_dx"]) < 1e-6
    assert np.array_equal(dx.ravel() != 0, ARR[f"pool{cid}_dx"] != 0)


def test_relu_and_softmax_against_reference(oracle):
    for c in LAYERS["cases"]:
        if c["kind"] == "relu":
            x, dy = _simple_input(oracle, c)
            y = oracle.relu_fwd(x)
            assert np.array_equal(y.ravel(), ARR[f"relu{c['id']}_y"])
            assert np.array_equal(oracle.relu_bwd(y, dy, x).ravel(), ARR[f"relu{c['id']}_dx"])
        if c["kind"] == "softmax":
            x, dy = _simple_input(oracle, c)
            y = oracle.softmax_fwd(x.reshape(c["n"], -1))
            assert rel_err(y, ARR[f"softmax{c['id']}_y"]) < TOL
            dx = oracle.softmax_bwd(ARR[f"softmax{c['id']}_y"].reshape(c["n"], -1), dy.reshape(c["n"], -1))
            assert rel_err(dx, ARR[f"softmax{c['id']}_dx"]) < 1e-4     # float cancellation inside cuDNN's own sum


@pytest.mark.parametrize("run", sorted(MEMORY))
def test_schedule_simulator_reproduces_the_reference_programs_memory_lines(oracle, run):
    """The reference prints pool usage after every layer of forward and backward.  With the workspace
    sizes cuDNN reported in that run fed in, the simulator must give the same byte counts line by line."""
    model, policy, algo = run.split("/")
    rec = MEMORY[run]
    batch = 64 if model == "VGG16_64" else 128
    specs = oracle.model_layers(getattr(oracle, model), batch)
    ws = [rec["workspace"].get(str(l), [0, 0, 0]) for l in range(len(specs))]
    if model == "OVERFEAT":
        assert all(rec["workspace"][str(l)] == [0, 0, 0] for l in (13, 15, 17))      # pinned to MEMORY_OPT (network.cu:447-486)
    ev, _ = oracle.policy_trace(specs, getattr(oracle, policy), ws=ws, iterations=1, fix_input_leak=False)
    fwd = [(l, used) for kind, l, tag, b, used in ev if kind == oracle.EV_FWD_DONE]
    bwd = [(l, used) for kind, l, tag, b, used in ev if kind == oracle.EV_BWD_DONE]
    assert fwd == [(l, used) for l, used, _ in rec["fwd"]]
    assert bwd == [(l, used) for l, used, _ in rec["bwd"]]
    # the printed "Memory Usage" adds the layer's workspace sizes to the pool usage
    for l, used, printed in rec["fwd"]:
        assert printed == used + ws[l][0]
    for l, used, printed in rec["bwd"]:
        assert printed == used + ws[l][1] + ws[l][2]
