"""Whole-network parity on a B200: the driver's Network against the CPU oracle's network step on
the same seeded inputs -- per-layer activations and gradients within 1e-4 (tensor-normalised),
loss within 1e-5, updated parameters, and the allocation / offload / prefetch trace."""
import numpy as np
import pytest

from helpers import rel_err, relu_knife_edges, tiny_net

pytestmark = pytest.mark.gpu
TOL = 1e-4
POLICIES = ["BASELINE", "VDNN_NONE", "VDNN_ALL", "VDNN_CONV"]
# Two runs of the same network differ by the order of their atomic sums (bias gradients of the TMA-fed layers, reduction
# splits of the zero-workspace kernels).  The first layer's bias gradient is a sum of up to 1.6 M terms of either sign
# per channel, so the second step's value carries that noise amplified by the cancellation: 1.2e-3 of the largest bias
# was measured between runs; the bound leaves room for the tail.
BIAS_NOISE = 5e-3


def _run(vdnn, oracle, specs, cnn, policy, algo, batch, lr, steps=2, host_sync=False, init_mode=0, seed0=1000, pool_bytes=4e9,
         expect_selected=None):
    onet = oracle.Net(specs, lr, init_mode=init_mode)
    net = vdnn.Network(cnn, policy, algo, batch_size=batch, pool_bytes=pool_bytes, learning_rate=lr, init_mode=init_mode,
                       capture=True, custom_layers=specs if cnn == "CUSTOM_CNN" else None, host_sync_per_layer=host_sync)
    try:
        if expect_selected is not None:
            assert net.selected() == expect_selected
        assert [s.astuple() for s in net.layer_specs()] == [tuple(s) if not hasattr(s, "astuple") else s.astuple() for s in specs]
        rows = specs[-1][1] if not hasattr(specs[-1], "n") else specs[-1].n
        cols = net.output_size // rows
        for step in range(steps):
            x = oracle.fill_normal(net.input_size, seed0 + step)
            t = oracle.fill_onehot(rows, cols, 2000 + step)
            onet.set_input(x, t)
            onet.forward()
            onet.backward()
            net.set_input(x, t)
            net.forwardPropagation()
            net.backwardPropagation()
            net.synchronize()
            for l in range(net.num_layers):
                assert rel_err(net.dst(l), onet.dst(l)) < TOL, ("dst", step, l)
            for l in range(net.num_layers - 1, -1, -1):
                assert rel_err(net.grad(l), onet.grad(l)) < TOL, ("grad", step, l)
                if onet.weights(l) is not None:
                    assert rel_err(net.weights(l), onet.weights(l)) < TOL, ("w", step, l)
                    assert rel_err(net.bias(l), onet.bias(l)) < TOL, ("b", step, l)
            sq, ce = net.loss()
            osq, oce = onet.loss()
            assert abs(sq - osq) < 1e-5 * max(1.0, abs(osq)) and abs(ce - oce) < 1e-5 * max(1.0, abs(oce))
        tr = net.trace()
        st = net.stats()
        assert vdnn.ops.engine_status() == 0
    finally:
        net.close()
        onet.close()
    return tr, st


@pytest.mark.parametrize("policy", POLICIES)
@pytest.mark.parametrize("algo", ["VDNN_MEMORY_OPT_ALGO", "VDNN_PERF_OPT_ALGO"])
def test_tiny_network_all_policies(vdnn, oracle, policy, algo):
    specs = tiny_net(4, with_lrn=True)
    tr, st = _run(vdnn, oracle, specs, "CUSTOM_CNN", policy, algo, 4, 0.05)
    if algo == "VDNN_MEMORY_OPT_ALGO":
        ev, summ = oracle.policy_trace(specs, vdnn.abi.VDNN_NAMES[policy], iterations=2, fix_input_leak=True)
        assert tr == ev
        assert st["pool_peak_bytes"] == summ.peak_bytes


def test_tanh_and_sigmoid_layers(vdnn, oracle):
    # the activation types besides RELU that the Layer class takes (vdnn.h:28-29); no stock model uses them
    TANH, SIGMOID = 4, 5
    specs = tiny_net(4)
    relus = [i for i, s in enumerate(specs) if s[0] == 3]
    specs[relus[0]] = (TANH,) + tuple(specs[relus[0]][1:])
    specs[relus[1]] = (SIGMOID,) + tuple(specs[relus[1]][1:])
    assert [s[0] for s in specs].count(TANH) == 1 and [s[0] for s in specs].count(SIGMOID) == 1
    _run(vdnn, oracle, specs, "CUSTOM_CNN", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", 4, 0.05)


def test_dynamic_algo_trains_with_mixed_algorithms(vdnn, oracle):
    """VDNN_DYNAMIC_ALGO on a pool that leaves room for the second convolution's workspace only: VDNN_ALL is kept,
    layer 0 runs its zero-workspace kernels, layer 2 the workspace-using ones, and the step equals the oracle's."""
    from test_host_logic import workspace_heavy_net
    specs = workspace_heavy_net()
    _run(vdnn, oracle, specs, "CUSTOM_CNN", "BASELINE", "VDNN_DYNAMIC_ALGO", 2, 0.01, pool_bytes=9_000_000, expect_selected=(2, 2))
    # and with room for everything the first candidate (VDNN_NONE, workspace-using algorithms) is taken
    _run(vdnn, oracle, specs, "CUSTOM_CNN", "BASELINE", "VDNN_DYNAMIC_ALGO", 2, 0.01, pool_bytes=64e6, expect_selected=(1, 1))


def test_reference_schedule_mode_gives_same_numbers(vdnn, oracle):
    # host synchronisation after every layer, as the reference does, instead of event ordering
    _run(vdnn, oracle, tiny_net(4), "CUSTOM_CNN", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", 4, 0.05, host_sync=True)


def test_reference_init_mode(vdnn, oracle):
    # U(-0.01, 0.01) weights and biases as layer.cu:925-967
    _run(vdnn, oracle, tiny_net(4), "CUSTOM_CNN", "VDNN_CONV", "VDNN_MEMORY_OPT_ALGO", 4, 0.01, init_mode=1)


@pytest.mark.parametrize("cnn,policy", [("ALEXNET", "VDNN_ALL"), ("ALEXNET_LRN", "BASELINE"), ("OVERFEAT", "VDNN_CONV")])
def test_reference_topologies_small_batch(vdnn, oracle, cnn, policy):
    batch = 2
    specs = [s.astuple() for s in oracle.model_layers(getattr(oracle, cnn), batch)]
    algo = "VDNN_PERF_OPT_ALGO" if cnn == "OVERFEAT" else "VDNN_MEMORY_OPT_ALGO"
    _run(vdnn, oracle, specs, cnn, policy, algo, batch, 0.01, steps=1)


def test_vgg16_single_image(vdnn, oracle):
    specs = [s.astuple() for s in oracle.model_layers(oracle.VGG16_64, 1)]
    # 13 ReLU layers over up to 3.2 M activations each: take the first input seed on which the oracle has
    # no ReLU input within rounding of zero under a live gradient (seed 1000 has two; one is 2e-8 against
    # a tensor maximum of 11 where the gradient is half the tensor's largest, and its mask bit depends on
    # the summation order of the convolution below).
    for seed0 in range(1000, 1016):
        onet = oracle.Net(specs, 0.01, init_mode=0)
        try:
            onet.set_input(oracle.fill_normal(3 * 224 * 224, seed0), oracle.fill_onehot(1, 1000, 2000))
            onet.forward()
            onet.backward()
            if relu_knife_edges(onet, specs) == 0:
                break
        finally:
            onet.close()
    else:
        pytest.fail("no seed without a knife-edge ReLU input")
    _run(vdnn, oracle, specs, "VGG16_64", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", 1, 0.01, steps=1, seed0=seed0)


def test_policies_agree_at_full_width(vdnn):
    """Size-independent property at a size the CPU oracle cannot reach in seconds: the four
    policies move data differently but compute the same step, so losses and parameters after two
    steps agree (to rounding: bias gradients and split FC products are summed with atomics)."""
    seen = {}
    for policy in POLICIES:
        net = vdnn.Network("ALEXNET", policy, "VDNN_PERF_OPT_ALGO", batch_size=32, pool_bytes=6e9, learning_rate=0.01)
        try:
            for step in range(2):
                net.seed_input(1000 + step, 2000 + step)
                net.step()
            seen[policy] = (net.loss(), [net.weights(l) for l in (0, 6, 13, 17)], [net.bias(l) for l in (0, 17)])
        finally:
            net.close()
    assert vdnn.ops.engine_status() == 0
    ref = seen["VDNN_NONE"]
    for policy, (loss, ws, bs) in seen.items():
        assert abs(loss[0] - ref[0][0]) < 1e-5 * abs(ref[0][0]) and abs(loss[1] - ref[0][1]) < 1e-5 * abs(ref[0][1]), policy
        for a, b in zip(ws + bs, ref[1] + ref[2]):
            assert rel_err(a, b) < 5e-5, policy


def test_resident_batch_is_reused_correctly_across_steps(vdnn):
    """Several steps on one uploaded batch.  Under VDNN_ALL / VDNN_CONV layer 0 is offloaded too, and the
    prefetched copy becomes the next step's input buffer (network.cu:1185): the next offload of layer 0
    must wait for that prefetch.  Compared with VDNN_NONE, which never moves the input."""
    import ctypes as C
    res = {}
    for policy in ("VDNN_NONE", "VDNN_ALL", "VDNN_CONV"):
        net = vdnn.Network("ALEXNET", policy, "VDNN_PERF_OPT_ALGO", batch_size=16, pool_bytes=4e9, learning_rate=1e-4)
        try:
            net.seed_input(1000, 2000)
            for _ in range(4):
                net.step()
            res[policy] = ([net.weights(l) for l in (0, 3, 17)], [net.bias(l) for l in (0, 17)], net.loss())
        finally:
            net.close()
    # Biases start at zero and are pure sums of gradients, so they show every flipped ReLU / pooling route that
    # run-to-run rounding (atomic sums) causes over several steps; a buffer read too early shows as a gross
    # difference in everything, which is what this test is after.
    for policy in ("VDNN_ALL", "VDNN_CONV"):
        for a, b in zip(res[policy][0], res["VDNN_NONE"][0]):
            assert rel_err(a, b) < 1e-4, policy
        for a, b in zip(res[policy][1], res["VDNN_NONE"][1]):
            assert rel_err(a, b) < 2e-2, policy
        assert abs(res[policy][2][0] - res["VDNN_NONE"][2][0]) < 1e-3


def test_offload_bytes_and_overlap_are_reported(vdnn, oracle):
    net = vdnn.Network("VGG16_64", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", batch_size=8, pool_bytes=6e9)
    try:
        net.set_profiling(True)
        for step in range(2):
            net.seed_input(1000 + step, 2000 + step)
            net.step()
        st = net.stats()
        specs = [s.astuple() for s in net.layer_specs()]
        _, summ = oracle.policy_trace(specs, oracle.VDNN_ALL, fix_input_leak=True)
        assert st["offload_bytes"] == summ.offload_bytes == st["prefetch_bytes"]
        assert st["pool_peak_bytes"] == summ.peak_bytes
        assert st["step_ms"] > 0 and st["offload_ms"] > 0 and st["prefetch_ms"] > 0
        assert 0 <= st["copy_overlap_ms"] <= st["offload_ms"] + st["prefetch_ms"] + 1e-3
        assert st["kernel_launches"] > 37
    finally:
        net.close()


def _steps(vdnn, pool_bytes, forward_order, model="ALEXNET", batch=32, layers=(0, 6, 13, 17), steps=2, lean=None,
           algo="VDNN_PERF_OPT_ALGO"):
    net = vdnn.Network(model, "VDNN_ALL", algo, batch_size=batch, pool_bytes=pool_bytes, learning_rate=1e-4, lean_offload=lean)
    try:
        net.set_offload_order(forward_order)
        forced = 0
        for step in range(steps):
            net.seed_input(1000 + step, 2000 + step)
            net.forwardPropagation()
            forced += net.stats()["forced_offloads"]
            net.backwardPropagation()
        net.synchronize()
        return ([net.weights(l) for l in layers], [net.bias(l) for l in (layers[0], layers[-1])], net.loss(), net.trace(),
                net.stats()["pool_peak_bytes"], forced, net.stats())
    finally:
        net.close()


def test_offload_order_is_not_observable(vdnn):
    """Offload copies enqueued in the order backward needs them (the default) or in layer order (the
    reference's): same host-side trace (allocations, releases, offloads, prefetches with the pool's byte
    count after each), same peak, same step to rounding."""
    by_need = _steps(vdnn, 6e9, False)
    in_order = _steps(vdnn, 6e9, True)
    assert by_need[3] == in_order[3] and by_need[4] == in_order[4]
    assert by_need[5] == 0 and in_order[5] == 0
    # losses of the second step: they carry the first step's atomically summed bias gradients (run-to-run noise); 1e-5 is
    # the bar the specification sets for the loss
    assert abs(by_need[2][0] - in_order[2][0]) < 1e-5 * abs(in_order[2][0]) and abs(by_need[2][1] - in_order[2][1]) < 1e-5 * abs(in_order[2][1])
    for a, b in zip(by_need[0], in_order[0]):
        assert rel_err(a, b) < 5e-5
    for a, b in zip(by_need[1], in_order[1]):        # bias gradients are summed with atomics: run-to-run noise
        assert rel_err(a, b) < BIAS_NOISE
    assert vdnn.ops.engine_status() == 0


@pytest.mark.parametrize("model,batch,layers", [("ALEXNET_LRN", 32, (0, 8, 15, 19)), ("VGG16_64", 8, (0, 5, 31, 35))])
def test_lean_offload_moves_fewer_bytes_and_trains_the_same(vdnn, model, batch, layers):
    """The opt-in lean form of VDNN_ALL drops the input of every ReLU that follows a CONV / FC layer instead of offloading
    it, and takes the ReLU's mask from its output in backward.  Same step as VDNN_ALL (the mask is the same bit for bit;
    what differs run to run is the order of the atomic sums), fewer bytes over PCIe, a lower peak, nothing leaked."""
    full = _steps(vdnn, 8e9, False, model=model, batch=batch, layers=layers, lean=False)
    lean = _steps(vdnn, 8e9, False, model=model, batch=batch, layers=layers, lean=True)
    assert lean[6]["offload_bytes"] == lean[6]["prefetch_bytes"] == lean[6]["pinned_bytes"]
    assert lean[6]["offload_bytes"] < 0.75 * full[6]["offload_bytes"]
    assert lean[4] <= full[4] and lean[6]["pool_used_bytes"] == full[6]["pool_used_bytes"]
    assert abs(lean[2][0] - full[2][0]) < 1e-5 * abs(full[2][0]) and abs(lean[2][1] - full[2][1]) < 1e-5 * abs(full[2][1])
    for a, b in zip(lean[0], full[0]):
        assert rel_err(a, b) < 5e-5
    for a, b in zip(lean[1], full[1]):          # layer 0's bias gradient: up to 1.6 M terms per channel, summed with atomics
        assert rel_err(a, b) < BIAS_NOISE
    assert vdnn.ops.engine_status() == 0


def test_workspace_reserve_keeps_a_roomy_pool_trainable(vdnn):
    """PERF_OPT at a pool of 1.45 x the peak, where the largest workspace (1 GB of operand images at this batch size) is a
    quarter of the pool: placement by pending events spreads the tensors, and the workspace finds its bytes in one piece
    only because the top of the pool is kept for it.  Same step as in a roomy pool."""
    vgg = dict(model="VGG16_64", batch=32, layers=(0, 5, 31, 35))
    dry = vdnn.Network("VGG16_64", "VDNN_ALL", "VDNN_PERF_OPT_ALGO", batch_size=32, device=-1, pool_bytes=20e9)
    try:
        dry.step()
        dry.step()
        peak = dry.stats()["pool_peak_bytes"]
    finally:
        dry.close()
    tight = _steps(vdnn, int(peak * 1.45), False, steps=3, **vgg)
    roomy = _steps(vdnn, 12e9, False, steps=3, **vgg)
    assert tight[3] == roomy[3] and tight[4] == roomy[4] == peak
    for a, b in zip(tight[0], roomy[0]):           # three steps of atomically summed bias / FC gradients apart
        assert rel_err(a, b) < 5e-5
    assert vdnn.ops.engine_status() == 0


def test_held_blocks_are_given_back_under_pool_pressure(vdnn):
    """VGG16 at batch 32 in a pool of 1.45 x the policy's peak: enough room for placement by pending events, but less
    than forward needs if nothing is reused, so forward can only go on by taking the bytes of tensors whose offload
    copy is still held back, and the pool has those copies enqueued early (oldest first).  Same step as in a roomy
    pool, and as in a pool so tight (1.15 x peak) that the driver packs it and sends the copies in layer order.
    (With the zero-workspace algorithms: the peak of PERF_OPT contains a workspace of 1 GB at this batch size, and
    1.45 x that peak holds all of forward without reuse.  The pressure is there in the first step; from the second on
    the measured budget of copies that leave during forward relieves it.)"""
    vgg = dict(model="VGG16_64", batch=32, layers=(0, 5, 31, 35), algo="VDNN_MEMORY_OPT_ALGO")
    dry = vdnn.Network("VGG16_64", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", batch_size=32, device=-1, pool_bytes=20e9)
    try:
        dry.step()
        dry.step()
        peak = dry.stats()["pool_peak_bytes"]
    finally:
        dry.close()
    pressed = _steps(vdnn, int(peak * 1.45), False, **vgg)
    roomy = _steps(vdnn, 12e9, False, **vgg)
    packed = _steps(vdnn, int(peak * 1.15), False, **vgg)
    assert pressed[5] > 0 and roomy[5] == 0 and packed[5] == 0
    for other in (pressed, packed):
        assert other[3] == roomy[3] and other[4] == roomy[4] == peak
        for a, b in zip(other[0], roomy[0]):       # the zero-workspace kernels sum their reduction splits with atomics
            assert rel_err(a, b) < 5e-5
        for a, b in zip(other[1], roomy[1]):       # layer 0's bias gradient: 1.6 M terms per channel, summed with atomics
            assert rel_err(a, b) < BIAS_NOISE
    assert vdnn.ops.engine_status() == 0


@pytest.mark.parametrize("cnn,policy,algo,batch", [
    ("ALEXNET", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", 128),          # BASELINE.json configuration 1 (without / with LRN)
    ("ALEXNET_LRN", "BASELINE", "VDNN_MEMORY_OPT_ALGO", 128),
    ("OVERFEAT", "VDNN_CONV", "VDNN_PERF_OPT_ALGO", 128),          # configuration 2
    ("VGG16_64", "VDNN_ALL", "VDNN_PERF_OPT_ALGO", 8),             # configurations 3-5 at the largest batch the oracle steps in seconds
    ("VGG16_64", "VDNN_NONE", "VDNN_MEMORY_OPT_ALGO", 8),
])
def test_benchmark_configurations_against_oracle(vdnn, oracle, cnn, policy, algo, batch):
    """One training step of the benchmarked networks at their own batch size (VGG16: batch 8) against the CPU oracle.

    Activations of every layer and the loss are compared in full (tensor-normalised 1e-4, loss 1e-5).  Gradients cannot
    be at these sizes: a few ReLU inputs and pooling windows lie within rounding of a tie (helpers.relu_knife_edges), two
    correct fp32 implementations may route those differently, and every such difference is spread by the layers below
    (one flipped element reaches 9 x C inputs of the next 3 x 3 convolution).  What the gradients are checked for here is
    what this test can see and the per-kernel tests cannot: a buffer used before its copy landed, a block reused too
    early, a tile never written -- gross errors.  So: relative L2 error below 1 %, and fewer than 2 % of the elements
    further than 1e-3 (tensor-normalised) from the oracle (measured: 0.2 - 0.3 % and about 1 %, depending on which way
    the first layers' roundings tip the ties).  (The kernels themselves are held to 1e-4 at these sizes by
    the reference fixtures of test_golden_gpu.py.)"""
    from helpers import l2_err, outlier_fraction
    specs = [s.astuple() for s in oracle.model_layers(getattr(oracle, cnn), batch)]
    lr = 1e-3
    onet = oracle.Net(specs, lr, init_mode=0)
    net = vdnn.Network(cnn, policy, algo, batch_size=batch, pool_bytes=12e9, learning_rate=lr, init_mode=0, capture=True)
    try:
        x = oracle.fill_normal(net.input_size, 1000)
        t = oracle.fill_onehot(batch, net.output_size // batch, 2000)
        before = {l: (net.weights(l), net.bias(l)) for l in range(net.num_layers) if net.tensor_size(l, 2) > 0}
        onet.set_input(x, t)
        onet.forward()
        onet.backward()
        net.set_input(x, t)
        net.step()
        net.synchronize()
        for l in range(net.num_layers):
            assert rel_err(net.dst(l), onet.dst(l)) < TOL, ("dst", l)
        sq, ce = net.loss()
        osq, oce = onet.loss()
        assert abs(sq - osq) < 1e-5 * max(1.0, abs(osq)) and abs(ce - oce) < 1e-5 * max(1.0, abs(oce))
        for l in range(net.num_layers - 1, -1, -1):
            g, og = net.grad(l), onet.grad(l)
            assert l2_err(g, og) < 1e-2 and outlier_fraction(g, og, 1e-3) < 2e-2, ("grad", l, l2_err(g, og))
            if l in before:
                w0, b0 = before[l]
                dw, odw = net.weights(l) - w0, onet.weights(l) - w0
                assert l2_err(dw, odw) < 1e-2, ("dw", l, l2_err(dw, odw))
                assert l2_err(net.bias(l) - b0, onet.bias(l) - b0) < 1e-2, ("db", l)
        assert vdnn.ops.engine_status() == 0
    finally:
        net.close()
        onet.close()


def test_vgg16_256_trains_on_the_gpu(vdnn, oracle):
    """VGG16 at batch 256 (vdnn.cu:20, network.cu:146-147): tensors of 822 M elements, byte counts beyond 2^31
    (network.cu:1010-1023 keeps them in an int).  One step under VDNN_ALL: the schedule equals the oracle's
    simulator, the loss is finite and equals the loss of the same step under VDNN_CONV, and so do the updated parameters."""
    seen = {}
    for policy in ("VDNN_ALL", "VDNN_CONV"):
        net = vdnn.Network("VGG16_256", policy, "VDNN_MEMORY_OPT_ALGO", pool_bytes=40e9, learning_rate=1e-6)
        try:
            net.seed_input(1000, 2000)
            net.step()
            net.synchronize()
            seen[policy] = (net.loss(), [net.weights(l) for l in (0, 10, 31, 35)], net.stats(), net.trace())
            if policy == "VDNN_ALL":
                specs = [s.astuple() for s in net.layer_specs()]
                assert specs[1][1:5] == (256, 64, 224, 224)
                ev, summ = oracle.policy_trace(specs, oracle.VDNN_ALL, fix_input_leak=True)
                assert seen[policy][3] == ev and seen[policy][2]["pool_peak_bytes"] == summ.peak_bytes
                assert seen[policy][2]["offload_bytes"] == summ.offload_bytes > 2 ** 34       # 29.5 GB each way
        finally:
            net.close()
    assert vdnn.ops.engine_status() == 0
    (la, wa, _, _), (lc, wc, _, _) = seen["VDNN_ALL"], seen["VDNN_CONV"]
    assert np.isfinite(la[0]) and np.isfinite(la[1])
    assert abs(la[0] - lc[0]) < 1e-6 and abs(la[1] - lc[1]) < 1e-5 * abs(lc[1])
    for a, b in zip(wa, wc):
        assert rel_err(a, b) < 1e-5
