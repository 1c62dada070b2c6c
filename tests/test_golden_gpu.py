"""The CUDA kernels against the tensors the reference's own Layer class produced on cuDNN / cuBLAS
(tests/golden/ref_layers.npz), through the C ABI, on both contraction engines."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LAYERS = json.load(open(os.path.join(GOLD, "ref_layers.json")))
ARR = np.load(os.path.join(GOLD, "ref_layers.npz"))
TOL = 1e-4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy().ravel()


@pytest.mark.parametrize("engine", ["ffma", "tcgen05"])
def test_kernels_reproduce_reference_layer_outputs(vdnn, oracle, engine):
    ops = vdnn.ops
    ops.set_engine({"ffma": vdnn.ENGINE_FFMA, "tcgen05": vdnn.ENGINE_TCGEN05}[engine])
    try:
        for c in LAYERS["cases"]:
            cid = c["id"]
            if c["kind"] == "conv":
                n, ch, h, w, k, r, pad, st, P, Q = (c[x] for x in ("n", "c", "h", "w", "k", "r", "pad", "stride", "p", "q"))
                x = oracle.fill_normal(n * ch * h * w, 100 * cid + 1)
                wt = oracle.fill_normal(k * ch * r * r, 100 * cid + 2, 0.0, 0.2)
                b = oracle.fill_normal(k, 100 * cid + 3)
                dy = oracle.fill_normal(n * k * P * Q, 100 * cid + 4)
                d = ops.conv_desc(n, ch, h, w, k, r, r, (pad, pad), (st, st))
                xd, wd, bd, dyd = dev(x), dev(wt), dev(b), dev(dy)
                yd = torch.empty(n * k * P * Q, device="cuda")
                ops.conv_fwd(d, xd, wd, yd, bias=bd)
                assert rel_err(host(yd), ARR[f"conv{cid}_y"]) < TOL, (cid, "y")
                dxd = torch.empty(n * ch * h * w, device="cuda")
                ops.conv_bwd_data(d, wd, dyd, dxd)
                assert rel_err(host(dxd), ARR[f"conv{cid}_dx"]) < TOL, (cid, "dx")
                lr = float(np.float32(c["lr"]))
                wz, bz = torch.zeros(k * ch * r * r, device="cuda"), torch.zeros(k, device="cuda")
                ops.conv_bwd_filter(d, xd, dyd, wz, alpha=-lr, beta=1.0)
                ops.conv_bwd_bias(n, k, P * Q, dyd, bz, alpha=-lr, beta=1.0)
                assert rel_err(host(wz), ARR[f"conv{cid}_wstep"]) < TOL, (cid, "w")
                assert rel_err(host(bz), ARR[f"conv{cid}_bstep"]) < TOL, (cid, "b")
            elif c["kind"] == "fc":
                n, cin, cout = c["n"], c["cin"], c["cout"]
                x = oracle.fill_normal(n * cin, 100 * cid + 1)
                wt = oracle.fill_normal(cin * cout, 100 * cid + 2, 0.0, 0.1)
                b = oracle.fill_normal(cout, 100 * cid + 3)
                dy = oracle.fill_normal(n * cout, 100 * cid + 4)
                lr = float(np.float32(c["lr"]))
                xd, wd, bd, dyd = dev(x), dev(wt), dev(b), dev(dy)
                yd = torch.empty(n * cout, device="cuda")
                ops.sgemm(1, 0, cout, n, cin, 1.0, wd, cin, xd, cin, 0.0, yd, cout)
                ops.add_bias(n, cout, 1, bd, yd)
                assert rel_err(host(yd), ARR[f"fc{cid}_y"]) < TOL
                dxd = torch.empty(n * cin, device="cuda")
                ops.sgemm(0, 0, cin, n, cout, 1.0, wd, cin, dyd, cout, 0.0, dxd, cin)
                assert rel_err(host(dxd), ARR[f"fc{cid}_dx"]) < TOL
                wz, bz = torch.zeros(cin * cout, device="cuda"), torch.zeros(cout, device="cuda")
                ops.sgemm(0, 1, cin, cout, n, -lr, xd, cin, dyd, cout, 1.0, wz, cin)
                ops.conv_bwd_bias(n, cout, 1, dyd, bz, alpha=-lr, beta=1.0)
                assert rel_err(host(wz), ARR[f"fc{cid}_wstep"]) < TOL
                assert rel_err(host(bz), ARR[f"fc{cid}_bstep"]) < TOL
            else:
                n, ch, h, w = c["n"], c["c"], c["h"], c["w"]
                std = 4.0 if c["kind"] == "softmax" else 1.0
                x = oracle.fill_normal(n * ch * h * w, 100 * cid + 1, 0.0, std).reshape(n, ch, h, w)
                if c["mode"] == 1:
                    rows = np.arange(h).reshape(1, 1, h, 1)
                    x = np.where((x > 0) & (rows >= h // 2), x, 0).astype(np.float32)
                elif c["mode"] == 2:
                    x = np.ones_like(x)
                dy = oracle.fill_normal(n * ch * c["p"] * c["q"], 100 * cid + 4)
                xd, dyd = dev(x), dev(dy)
                yd = torch.empty(n * ch * c["p"] * c["q"], device="cuda")
                dxd = torch.empty(x.size, device="cuda")
                if c["kind"] == "relu":
                    ops.relu_fwd(x.size, xd, yd)
                    ops.relu_bwd(x.size, yd, dyd, xd, dxd)
                    assert np.array_equal(host(yd), ARR[f"relu{cid}_y"]) and np.array_equal(host(dxd), ARR[f"relu{cid}_dx"])
                elif c["kind"] == "pool":
                    win, st = (c["win"], c["win"]), (c["stride"], c["stride"])
                    ops.maxpool_fwd(n, ch, h, w, win, st, xd, yd)
                    ops.maxpool_bwd(n, ch, h, w, win, st, yd, dyd, xd, dxd)
                    assert np.array_equal(host(yd), ARR[f"pool{cid}_y"])
                    assert rel_err(host(dxd), ARR[f"pool{cid}_dx"]) < 1e-6
                    assert np.array_equal(host(dxd) != 0, ARR[f"pool{cid}_dx"] != 0)      # same routing, ties included
                else:
                    rows, cols = n, ch * h * w
                    ops.softmax_fwd(rows, cols, xd, yd)
                    assert rel_err(host(yd), ARR[f"softmax{cid}_y"]) < 1e-5
                    ops.softmax_bwd(rows, cols, dev(ARR[f"softmax{cid}_y"]), dyd, dxd)
                    assert rel_err(host(dxd), ARR[f"softmax{cid}_dx"]) < 1e-4
        assert ops.engine_status() == 0
    finally:
        ops.set_engine(vdnn.ENGINE_AUTO)


BIG_HAVE = os.path.exists(os.path.join(GOLD, "ref_big.json"))
BIG = json.load(open(os.path.join(GOLD, "ref_big.json"))) if BIG_HAVE else {"cases": [], "tensors": []}
BIG_ARR = np.load(os.path.join(GOLD, "ref_big.npz")) if BIG_HAVE else {}
BIG_META = {t["name"]: t for t in BIG["tensors"]}


@pytest.mark.skipif(not BIG_HAVE, reason="tests/golden/ref_big.* not generated")
@pytest.mark.parametrize("algo_mode", [0, 1])
@pytest.mark.parametrize("cid", [c["id"] for c in BIG["cases"]])
def test_kernels_reproduce_reference_at_benchmark_sizes(vdnn, oracle, cid, algo_mode):
    """Layers at or near the sizes the benchmarked networks run them at (every tile width, split plan and special-case
    kernel of the tensor-core engine) against what the reference's Layer class computed on cuDNN / cuBLAS: strided
    samples, L2 norm and sum of every output tensor, in the zero-workspace and the workspace-using mode."""
    from helpers import check_reduced
    from test_golden_big import big_inputs
    ops = vdnn.ops
    c = next(c for c in BIG["cases"] if c["id"] == cid)
    x, wt, b, dy = big_inputs(oracle, c)
    lr = float(np.float32(c["lr"]))
    xd, wd, bd, dyd = dev(x), dev(wt), dev(b), dev(dy)
    out = {}
    if c["kind"] == "conv":
        n, ch, h, w, k, r, pad, st, P, Q = (c[x_] for x_ in ("n", "c", "h", "w", "k", "r", "pad", "stride", "p", "q"))
        d = ops.conv_desc(n, ch, h, w, k, r, r, (pad, pad), (st, st))
        need = max(ops.conv_workspace_bytes(op, algo_mode, d) for op in range(3))
        ws = torch.empty(max(need, 16) // 4 + 64, device="cuda")
        tag = f"conv{cid}"
        yd = torch.empty(n * k * P * Q, device="cuda")
        ops.conv_fwd(d, xd, wd, yd, bias=bd, algo_mode=algo_mode, workspace=ws, workspace_bytes=need)
        dxd = torch.empty(n * ch * h * w, device="cuda")
        ops.conv_bwd_data(d, wd, dyd, dxd, algo_mode=algo_mode, workspace=ws, workspace_bytes=need)
        wz, bz = torch.zeros(k * ch * r * r, device="cuda"), torch.zeros(k, device="cuda")
        ops.conv_bwd_filter(d, xd, dyd, wz, alpha=-lr, beta=1.0, algo_mode=algo_mode, workspace=ws, workspace_bytes=need)
        ops.conv_bwd_bias(n, k, P * Q, dyd, bz, alpha=-lr, beta=1.0)
    else:
        n, cin, cout = c["n"], c["cin"], c["cout"]
        tag = f"fc{cid}"
        yd = torch.empty(n * cout, device="cuda")
        ops.sgemm(1, 0, cout, n, cin, 1.0, wd, cin, xd, cin, 0.0, yd, cout)
        ops.add_bias(n, cout, 1, bd, yd)
        dxd = torch.empty(n * cin, device="cuda")
        ops.sgemm(0, 0, cin, n, cout, 1.0, wd, cin, dyd, cout, 0.0, dxd, cin)
        wz, bz = torch.zeros(cin * cout, device="cuda"), torch.zeros(cout, device="cuda")
        ops.sgemm(0, 1, cin, cout, n, -lr, xd, cin, dyd, cout, 1.0, wz, cin)
        ops.conv_bwd_bias(n, cout, 1, dyd, bz, alpha=-lr, beta=1.0)
    for name, t in (("y", yd), ("dx", dxd), ("wstep", wz), ("bstep", bz)):
        check_reduced(host(t), BIG_ARR[f"{tag}_{name}"], BIG_META[f"{tag}_{name}"], TOL, f"{tag}_{name} mode {algo_mode}")
    assert ops.engine_status() == 0
