import numpy as np

FC_GEMM, CONV, FC_CONV, RELU, SOFTMAX, POOL, LRN = 0, 1, 2, 3, 6, 7, 9


def rel_err(a, b):
    """Tensor-normalised error: max|a-b| / max|b|."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    denom = max(float(np.abs(b).max()), 1e-30)
    return float(np.abs(a - b).max()) / denom


def relu_knife_edges(onet, specs, eps=5e-8, live=2e-5):
    """Count ReLU inputs the oracle holds within `eps` (tensor-normalised; an fp32 convolution output near
    zero carries a rounding error around 1e-8 of the tensor's maximum) of zero while a gradient above
    `live` of the largest arrives there.  The sign of such an input is decided by the last rounding of the
    convolution below it, so two correct fp32 implementations may disagree on that mask bit, and the
    disagreement then spreads through every gradient underneath.  Whole-network parity is only meaningful
    on inputs where this count is zero."""
    count = 0
    for l, spec in enumerate(specs):
        if tuple(spec)[0] != RELU:
            continue
        x = np.abs(onet.dst(l - 1).ravel())
        dy = np.abs(onet.grad(l + 1).ravel()) if l + 1 < len(specs) else None
        near = x < eps * x.max()
        if dy is not None:
            near &= dy > live * max(float(dy.max()), 1e-30)
        count += int(near.sum())
    return count


# Small topologies in the reference's constructor order: (type, n, c, h, w, pad_h, pad_w, stride_h, stride_w, k, r, s)


def tiny_net(n=4, with_lrn=False):
    """conv3x3 -> relu -> [lrn] -> pool2 -> conv5x5/s2 -> relu -> pool3/s2 -> fc -> relu -> fc -> softmax."""
    L = []
    L.append((FC_CONV, n, 3, 20, 20, 1, 1, 1, 1, 8, 3, 3))      # -> 8x20x20
    L.append((RELU, n, 8, 20, 20, 0, 0, 0, 0, 0, 0, 0))
    if with_lrn:
        L.append((LRN, n, 8, 20, 20, 0, 0, 0, 0, 0, 5, 5))
    L.append((POOL, n, 8, 20, 20, 0, 0, 2, 2, 0, 2, 2))          # -> 8x10x10
    L.append((FC_CONV, n, 8, 10, 10, 2, 2, 1, 1, 16, 5, 5))      # -> 16x10x10
    L.append((RELU, n, 16, 10, 10, 0, 0, 0, 0, 0, 0, 0))
    L.append((POOL, n, 16, 10, 10, 0, 0, 2, 2, 0, 3, 3))         # -> 16x4x4
    L.append((FC_GEMM, n, 256, 1, 1, 0, 0, 0, 0, 32, 1, 1))
    L.append((RELU, n, 32, 1, 1, 0, 0, 0, 0, 0, 0, 0))
    L.append((FC_GEMM, n, 32, 1, 1, 0, 0, 0, 0, 10, 1, 1))
    L.append((SOFTMAX, n, 10, 1, 1, 0, 0, 0, 0, 0, 0, 0))
    return L


def check_reduced(tensor, samples, meta, tol, what=""):
    """Compares a full tensor with the reduced fixture of a tensor too large to keep: `samples` are its elements at
    indices 0, stride, 2*stride, ...; `meta` holds count, stride, sum, sumsq and maxabs over the whole tensor.
      * every sample within tol of the reference, normalised by the reference tensor's largest magnitude;
      * the L2 norm within tol (relative);
      * the sum within tol * sqrt(count * sumsq): what per-element errors of tol * rms can add up to at most."""
    t = np.asarray(tensor, np.float64).ravel()
    assert t.size == meta["count"], (what, t.size, meta["count"])
    got = t[::meta["stride"]][:meta["samples"]]
    err = float(np.abs(got - samples.astype(np.float64)).max()) / max(meta["maxabs"], 1e-30)
    assert err < tol, (what, "samples", err)
    norm, ref_norm = float(np.sqrt((t * t).sum())), float(np.sqrt(meta["sumsq"]))
    assert abs(norm - ref_norm) <= tol * ref_norm, (what, "norm", norm, ref_norm)
    assert abs(float(t.sum()) - meta["sum"]) <= tol * np.sqrt(meta["count"] * meta["sumsq"]), (what, "sum", float(t.sum()), meta["sum"])
    return err


def outlier_fraction(a, b, tol=1e-4):
    """Fraction of elements of `a` further than tol (normalised by max|b|) from `b`."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    denom = max(float(np.abs(b).max()), 1e-30)
    return float((np.abs(a - b) > tol * denom).mean())


def l2_err(a, b):
    """Relative L2 error ||a - b|| / ||b||."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    return float(np.sqrt(((a - b) ** 2).sum()) / max(np.sqrt((b * b).sum()), 1e-30))
