"""The workspace-free filter gradient (vdnn_conv_bwd_filter_static) against the ordinary entry point.

Some hosts of this library cannot allocate device memory once they are running: their memory budget
is fixed at start-up, or they sit inside a process whose allocator they cannot reach, or an
allocation's implicit device-wide synchronisation is not acceptable in their steady-state loop.
They have no buffer to pass as `workspace`, so this entry point keeps the split-K partial sums in a
16 MiB array that is part of the library image.  The file is named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu


def _case(vdnn, n, c, h, k, seed):
    ops = vdnn.ops
    d = ops.conv_desc(n, c, h, h, k, 3, 3, (1, 1), (1, 1))
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, c, h, h, device="cuda", generator=g)
    dy = torch.randn(n, k, h, h, device="cuda", generator=g)
    w0 = torch.randn(k, c, 3, 3, device="cuda", generator=g)
    return ops, d, x, dy, w0


def test_static_scratch_matches_workspace_entry_point_twice(vdnn):
    results = []
    # two calls in a row with different shapes and data: the second reuses the array the first left dirty
    for (n, c, h, k, seed) in [(8, 32, 28, 32, 1), (4, 64, 14, 48, 2)]:
        ops, d, x, dy, w0 = _case(vdnn, n, c, h, k, seed)
        need = ops.conv_workspace_bytes(2, 1, d)
        assert 0 < need <= ops.STATIC_SCRATCH_BYTES          # the shape really does use scratch
        ws = torch.empty(need // 4, device="cuda")
        want = w0.clone()
        ops.conv_bwd_filter(d, x, dy, want, alpha=-0.01, beta=1.0, algo_mode=1, workspace=ws, workspace_bytes=need)
        got = w0.clone()
        ops.conv_bwd_filter_static(d, x, dy, got, alpha=-0.01, beta=1.0)
        torch.cuda.synchronize()
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < 1e-4
        assert torch.equal(got, want)                         # same kernels, fixed summation order
        # plain gradient (alpha = 1, beta = 0) as well
        ops.conv_bwd_filter(d, x, dy, want, algo_mode=1, workspace=ws, workspace_bytes=need)
        ops.conv_bwd_filter_static(d, x, dy, got)
        torch.cuda.synchronize()
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < 1e-4
        results.append(float(got.abs().sum()))
    assert all(np.isfinite(results)) and ops.engine_status() == 0


def test_static_scratch_with_packed_operand_images_against_oracle(vdnn, oracle):
    """Shapes with at least 128 filters also keep the tile images of dy in the scratch array (images first, partial
    sums behind them), and a filter as large as its input runs as a plain matrix product.  Each case runs right after a
    call that left other data in the array, is checked against the CPU oracle, and must not change the amount of free
    device memory: the entry point allocates nothing."""
    ops = vdnn.ops
    # make the array dirty first
    o0, d0, x0, dy0, w0 = _case(vdnn, 8, 32, 28, 32, 7)
    ops.conv_bwd_filter_static(d0, x0, dy0, w0.clone())
    torch.cuda.synchronize()
    for (n, c, h, k, r, pad) in [(4, 64, 14, 128, 3, 1), (2, 32, 12, 256, 3, 1), (256, 64, 6, 48, 6, 0)]:
        d = ops.conv_desc(n, c, h, h, k, r, r, (pad, pad), (1, 1))
        assert ops.conv_workspace_bytes(2, 1, d) <= ops.STATIC_SCRATCH_BYTES
        p = h + 2 * pad - r + 1
        x = oracle.fill_normal(n * c * h * h, 11).reshape(n, c, h, h)
        dy = oracle.fill_normal(n * k * p * p, 12).reshape(n, k, p, p)
        w0 = oracle.fill_normal(k * c * r * r, 13, 0.0, 0.1).reshape(k, c, r, r)
        want = oracle.conv_bwd_filter(x, dy, w0.shape, (pad, pad), (1, 1), alpha=-0.01, beta=1.0, dw=w0.copy())
        xd, dyd = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()
        for rep in range(2):                     # the second call finds the array as the first left it
            got = torch.from_numpy(w0.copy()).cuda()
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            ops.conv_bwd_filter_static(d, xd, dyd, got, alpha=-0.01, beta=1.0)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before, (n, c, h, k, rep)
            assert rel_err(got.cpu().numpy(), want) < 1e-4, (n, c, h, k, rep)
    assert ops.engine_status() == 0


def test_static_scratch_refuses_what_does_not_fit(vdnn):
    ops = vdnn.ops
    # 512 -> 512 channels at 14x14: few output tiles, many splits, 18 MiB of partial sums, beyond the 16 MiB array
    d = ops.conv_desc(8, 512, 14, 14, 512, 3, 3, (1, 1), (1, 1))
    assert ops.conv_workspace_bytes(2, 1, d) > ops.STATIC_SCRATCH_BYTES
    x = torch.zeros(8, 512, 14, 14, device="cuda")
    dy = torch.zeros(8, 512, 14, 14, device="cuda")
    dw = torch.full((512, 512, 3, 3), 3.0, device="cuda")
    with pytest.raises(vdnn.VdnnError) as e:
        ops.conv_bwd_filter_static(d, x, dy, dw)
    assert e.value.status == -8 and "SCRATCH_LIMIT" in str(e.value)
    torch.cuda.synchronize()
    assert bool((dw == 3.0).all())                            # nothing was launched
