"""Pins the CPU oracle to the reference's own Layer class (cuDNN 9.10 / cuBLAS, FMA arithmetic, run on a B200) on
layers at or near the sizes the benchmarked networks run them at.  The tensors are too large to keep, so the
fixture (tests/golden/ref_big.npz + ref_big.json, made by tests/golden/make_golden.py --big from the output of
`oracle/_ref/ref_harness <dir> big`) holds 4096 strided samples, the sum, the sum of squares and the largest
magnitude of each.  No GPU."""
import json
import os

import numpy as np
import pytest

from helpers import check_reduced

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
HAVE = os.path.exists(os.path.join(GOLD, "ref_big.json"))
BIG = json.load(open(os.path.join(GOLD, "ref_big.json"))) if HAVE else {"cases": [], "tensors": []}
ARR = np.load(os.path.join(GOLD, "ref_big.npz")) if HAVE else {}
META = {t["name"]: t for t in BIG["tensors"]}
TOL = 2e-5      # fp32 FMA sums of up to 25088 terms against double accumulation


def big_inputs(oracle, c):
    cid = c["id"]
    if c["kind"] == "conv":
        n, ch, h, w, k, r = (c[x] for x in ("n", "c", "h", "w", "k", "r"))
        sizes = (n * ch * h * w, k * ch * r * r, k, n * k * c["p"] * c["q"])
    else:
        sizes = (c["n"] * c["cin"], c["cin"] * c["cout"], c["cout"], c["n"] * c["cout"])
    x = oracle.fill_normal(sizes[0], 100 * cid + 1)
    wt = oracle.fill_normal(sizes[1], 100 * cid + 2, 0.0, float(np.float32(c["wstd"])))
    b = oracle.fill_normal(sizes[2], 100 * cid + 3)
    dy = oracle.fill_normal(sizes[3], 100 * cid + 4)
    return x, wt, b, dy


@pytest.mark.skipif(not HAVE, reason="tests/golden/ref_big.* not generated")
@pytest.mark.parametrize("cid", [c["id"] for c in BIG["cases"]])
def test_oracle_against_reference_at_benchmark_sizes(oracle, cid):
    c = next(c for c in BIG["cases"] if c["id"] == cid)
    x, wt, b, dy = big_inputs(oracle, c)
    lr = np.float32(c["lr"])
    if c["kind"] == "conv":
        n, ch, h, w, k, r, pad, st, P, Q = (c[x_] for x_ in ("n", "c", "h", "w", "k", "r", "pad", "stride", "p", "q"))
        x, wt, dy = x.reshape(n, ch, h, w), wt.reshape(k, ch, r, r), dy.reshape(n, k, P, Q)
        tag = f"conv{cid}"
        y = oracle.add_bias(oracle.conv_fwd(x, wt, (pad, pad), (st, st)), b)
        dx = oracle.conv_bwd_data(wt, dy, x.shape, (pad, pad), (st, st))
        wstep = oracle.conv_bwd_filter(x, dy, wt.shape, (pad, pad), (st, st), alpha=-lr, beta=1.0, dw=np.zeros_like(wt))
        bstep = oracle.conv_bwd_bias(dy, alpha=-lr, beta=1.0, db=np.zeros(k, np.float32))
    else:
        n, cin, cout = c["n"], c["cin"], c["cout"]
        tag = f"fc{cid}"
        y = oracle.sgemm(1, 0, cout, n, cin, 1.0, wt, cin, x, cin, 0.0, np.zeros(n * cout, np.float32), cout)
        y = oracle.add_bias(y.reshape(n, cout, 1), b).ravel()
        dx = oracle.sgemm(0, 0, cin, n, cout, 1.0, wt, cin, dy, cout, 0.0, np.zeros(n * cin, np.float32), cin)
        wstep = oracle.sgemm(0, 1, cin, cout, n, -lr, x, cin, dy, cout, 1.0, np.zeros(cin * cout, np.float32), cin)
        bstep = oracle.conv_bwd_bias(dy.reshape(n, cout, 1), alpha=-lr, beta=1.0, db=np.zeros(cout, np.float32))
    for name, t in (("y", y), ("dx", dx), ("wstep", wstep), ("bstep", bstep)):
        check_reduced(t, ARR[f"{tag}_{name}"], META[f"{tag}_{name}"], TOL, f"{tag}_{name}")
