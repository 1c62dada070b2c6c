import numpy as np


def rel_err(a, b):
    """Tensor-normalised error: max|a-b| / max|b|."""
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    denom = max(float(np.abs(b).max()), 1e-30)
    return float(np.abs(a - b).max()) / denom


# Small topologies in the reference's constructor order: (type, n, c, h, w, pad_h, pad_w, stride_h, stride_w, k, r, s)
FC_GEMM, CONV, FC_CONV, RELU, SOFTMAX, POOL, LRN = 0, 1, 2, 3, 6, 7, 9


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
