"""The path "a bounded device-side wait ran out -> status word -> host error", exercised without disturbing the GPU:
the library's self-test kernel waits a few hundred microseconds on a barrier nothing arrives at, gives up, records
its code and returns normally."""
import pytest
import torch

from helpers import tiny_net

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_cleared(vdnn):
    ops = vdnn.ops
    assert ops.engine_status() == 0
    ops.engine_wait_selftest(500_000)              # about a quarter of a millisecond
    torch.cuda.synchronize()                       # the kernel returned by itself
    assert ops.engine_status() == 104              # reading clears the word
    assert ops.engine_status() == 0
    with pytest.raises(vdnn.VdnnError):
        ops.engine_wait_selftest(10 ** 10)         # limits beyond about a second are refused


def test_network_synchronize_reports_an_expired_wait(vdnn):
    """The network publishes the status word behind every backward pass; synchronize() turns a non-zero word into
    VDNN_ERR_TIMEOUT, so a step whose contraction kernels gave up is never taken for a valid one."""
    ops = vdnn.ops
    specs = tiny_net(4)
    net = vdnn.Network("CUSTOM_CNN", "VDNN_NONE", "VDNN_MEMORY_OPT_ALGO", pool_bytes=1e9, custom_layers=specs)
    try:
        net.seed_input(1000, 2000)
        net.step()
        net.synchronize()                          # healthy
        ops.engine_wait_selftest(500_000, net.stream(0))
        net.step()
        with pytest.raises(vdnn.VdnnError) as e:
            net.synchronize()
        assert e.value.status == -6
        assert ops.engine_status() == 104
        net.step()                                 # the word is clear again: the next step is healthy
        net.synchronize()
    finally:
        net.close()
    assert ops.engine_status() == 0
