"""Host-side logic of the product library, exercised without a GPU: exported symbols, the pool
allocator, the host generators, and the Network's allocation / offload / prefetch schedule
(dry-run networks against the oracle's schedule simulator)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(vdnn):
    header = open(os.path.join(ROOT, "include", "vdnn_b200.h")).read()
    declared = set(re.findall(r"\b(vdnn_[a-z0-9_]+)\s*\(", header))
    declared -= {"vdnn_status", "vdnn_network"}        # type names followed by '(' never occur, but be safe
    assert len(declared) >= 50
    L = C.CDLL(vdnn.lib_path())
    missing = [n for n in sorted(declared) if not hasattr(L, n)]
    assert not missing, missing
    from vdnn_implementation_b200 import abi
    assert declared == set(abi.SIGNATURES), declared ^ set(abi.SIGNATURES)
    pool_header = open(os.path.join(ROOT, "include", "cnmem", "include", "cnmem.h")).read()
    for name in set(re.findall(r"\b((?:cnmem|vdnnPool)[A-Za-z]+)\s*\(", pool_header)):
        assert hasattr(L, name), name


def test_status_strings_and_bad_arguments(vdnn):
    L = vdnn.lib()
    assert L.vdnn_status_string(0) == b"VDNN_OK"
    assert L.vdnn_status_string(-3) == b"VDNN_ERR_WORKSPACE"
    assert b"sm_100a" in L.vdnn_build_info()
    # argument validation happens before any CUDA call
    assert L.vdnn_relu_fwd(16, None, None, None) == -1
    d = vdnn.ConvDesc(1, 1, 2, 2, 1, 3, 3, 0, 0, 1, 1)          # filter larger than the padded input
    p, q = C.c_int(), C.c_int()
    assert L.vdnn_conv_out_dims(C.byref(d), C.byref(p), C.byref(q)) == -1
    d = vdnn.ConvDesc(128, 3, 227, 227, 96, 11, 11, 0, 0, 4, 4)
    assert L.vdnn_conv_out_dims(C.byref(d), C.byref(p), C.byref(q)) == 0 and (p.value, q.value) == (55, 55)
    assert L.vdnn_pool_out_dims(55, 55, 3, 3, 2, 2, C.byref(p), C.byref(q)) == 0 and (p.value, q.value) == (27, 27)
    assert L.vdnn_conv_workspace_bytes(0, 0, C.byref(d)) == 0     # MEMORY_OPT never needs workspace
    assert L.vdnn_set_engine(7) == -1


def test_host_generators_match_oracle_bit_for_bit(vdnn, oracle):
    L = vdnn.lib()
    n = 100003
    a = np.empty(n, np.float32)
    L.vdnn_host_fill_normal(a.ctypes.data_as(C.c_void_p), n, 1234, 0.0, 1.0)
    assert np.array_equal(a, oracle.fill_normal(n, 1234))
    L.vdnn_host_fill_normal(a.ctypes.data_as(C.c_void_p), n, 3001, 0.0, float(np.sqrt(np.float32(2.0) / np.float32(27))))
    assert np.array_equal(a, oracle.fill_normal(n, 3001, 0.0, float(np.sqrt(np.float32(2.0) / np.float32(27)))))
    L.vdnn_host_fill_uniform(a.ctypes.data_as(C.c_void_p), n, 77, -0.01, 0.01)
    assert np.array_equal(a, oracle.fill_uniform(n, 77, -0.01, 0.01))
    oh = np.empty((128, 1000), np.float32)
    L.vdnn_host_fill_onehot(oh.ctypes.data_as(C.c_void_p), 128, 1000, 2000)
    assert np.array_equal(oh, oracle.fill_onehot(128, 1000, 2000))


def test_pool_allocator_bookkeeping(vdnn):
    L = C.CDLL(vdnn.lib_path())
    L.vdnnPoolInitVirtual.argtypes = [C.c_size_t]
    L.cnmemMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p]
    L.cnmemFree.argtypes = [C.c_void_p, C.c_void_p]
    L.cnmemMemGetInfo.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_void_p]
    L.cnmemGetErrorString.restype = C.c_char_p
    assert L.cnmemMalloc(C.byref(C.c_void_p()), 16, None) == 3            # NOT_INITIALIZED
    assert L.vdnnPoolInitVirtual(1 << 20) == 0
    try:
        free, total = C.c_size_t(), C.c_size_t()

        def used():
            L.cnmemMemGetInfo(C.byref(free), C.byref(total), None)
            return total.value - free.value

        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        assert L.cnmemMalloc(C.byref(a), 1, None) == 0 and used() == 512          # 512-byte granularity
        assert L.cnmemMalloc(C.byref(b), 513, None) == 0 and used() == 512 + 1024
        assert L.cnmemMalloc(C.byref(c), 1 << 20, None) == 4                       # OUT_OF_MEMORY
        assert L.cnmemGetErrorString(4) == b"CNMEM_STATUS_OUT_OF_MEMORY"
        assert L.cnmemFree(a, None) == 0 and used() == 1024
        assert L.cnmemFree(a, None) == 2                                           # double free rejected
        # best fit: a 512-byte request goes back into the 512-byte hole, not the big tail
        d = C.c_void_p()
        assert L.cnmemMalloc(C.byref(d), 100, None) == 0 and d.value == a.value
        assert L.cnmemFree(d, None) == 0 and L.cnmemFree(b, None) == 0 and used() == 0
        # coalescing: the whole pool is one block again
        assert L.cnmemMalloc(C.byref(c), 1 << 20, None) == 0 and L.cnmemFree(c, None) == 0
        peak = C.c_size_t()
        assert L.vdnnPoolHighWater(C.byref(peak), 1) == 0 and peak.value == 1 << 20
        # host-side fault injection for the soft out-of-memory path
        assert L.vdnnPoolFailAfter(2) == 0
        assert L.cnmemMalloc(C.byref(a), 16, None) == 0
        assert L.cnmemMalloc(C.byref(b), 16, None) == 4
        assert L.cnmemMalloc(C.byref(b), 16, None) == 0
    finally:
        assert L.cnmemFinalize() == 0


def test_pool_held_bytes_are_avoided_then_resolved_oldest_first(vdnn):
    """Bytes released with vdnnPoolFreeHeld (their last reader is not enqueued yet) count as free, are
    passed over while anything else fits -- also by placing a request behind them inside a coalesced free
    block -- and are claimed through the resolver, lowest token first, when nothing else fits."""
    L = C.CDLL(vdnn.lib_path())
    L.vdnnPoolInitVirtual.argtypes = [C.c_size_t]
    L.cnmemMalloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p]
    L.cnmemFree.argtypes = [C.c_void_p, C.c_void_p]
    L.cnmemMemGetInfo.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_void_p]
    L.vdnnPoolFreeHeld.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_ulonglong]
    L.vdnnPoolResolve.argtypes = [C.c_ulonglong, C.c_void_p]
    RESOLVER = C.CFUNCTYPE(None, C.c_void_p, C.c_ulonglong)
    L.vdnnPoolSetResolver.argtypes = [RESOLVER, C.c_void_p]
    L.vdnnPoolMallocFor.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p, C.c_int]
    K = 256 << 10
    asked = []

    def resolve(user, token):
        asked.append(token)
        assert L.vdnnPoolResolve(token, None) == 0

    cb = RESOLVER(resolve)
    assert L.vdnnPoolInitVirtual(4 * K) == 0
    try:
        assert L.vdnnPoolSetResolver(cb, None) == 0
        a, b, c, d, e = (C.c_void_p() for _ in range(5))
        for p in (a, b, c):
            assert L.cnmemMalloc(C.byref(p), K, None) == 0
        free, total = C.c_size_t(), C.c_size_t()
        assert L.vdnnPoolFreeHeld(b, None, 0, 2) == 0 and L.vdnnPoolFreeHeld(a, None, 0, 1) == 0
        L.cnmemMemGetInfo(C.byref(free), C.byref(total), None)
        assert total.value - free.value == K                       # held bytes are free bytes
        assert L.cnmemFree(c, None) == 0                            # [a b c tail] is one free block now; a and b held
        assert L.vdnnPoolMallocFor(C.byref(d), K, None, 0) == 0
        assert d.value == c.value and asked == []                   # placed behind the held bytes, nobody asked
        assert L.vdnnPoolMallocFor(C.byref(e), K, None, 0) == 0
        assert e.value == c.value + K and asked == []
        assert L.vdnnPoolMallocFor(C.byref(c), 2 * K, None, 0) == 0 # only the held bytes are left
        assert c.value == a.value and asked == [1, 2]
        assert L.vdnnPoolMallocFor(C.byref(b), 512, None, 0) == 4   # OUT_OF_MEMORY: the pool is full
        L.vdnnPoolSetResolver(RESOLVER(0), None)
    finally:
        assert L.cnmemFinalize() == 0


MODELS = [("ALEXNET", 128), ("ALEXNET_LRN", 128), ("OVERFEAT", 128), ("VGG16_64", 64), ("VGG16_128", 128),
          ("VGG16_256", 256)]      # 822 M-element tensors: byte counts beyond 2^31 (the reference's int sizes wrap there)


@pytest.mark.parametrize("model,batch", MODELS)
@pytest.mark.parametrize("policy", [0, 1, 2, 3])
def test_network_schedule_equals_reference_schedule(vdnn, oracle, model, batch, policy):
    """Event-for-event: every pool allocation and release, every offload and prefetch, and the pool
    usage after each of them, over two iterations."""
    for fix in (True, False):
        net = vdnn.Network(model, policy, vdnn.VDNN_MEMORY_OPT_ALGO, device=-1, pool_bytes=170e9, fix_input_leak=fix)
        try:
            specs = [s.astuple() for s in net.layer_specs()]
            assert specs == [s.astuple() for s in oracle.model_layers(getattr(oracle, model), batch)]
            net.step()
            net.step()
            ev, summ = oracle.policy_trace(specs, policy, iterations=2, fix_input_leak=fix)
            assert net.trace() == ev
            st = net.stats()
            assert st["pool_peak_bytes"] == summ.peak_bytes
            assert st["pinned_bytes"] == summ.pinned_bytes
            assert st["offload_bytes"] * 2 == summ.offload_bytes and st["prefetch_bytes"] * 2 == summ.prefetch_bytes
        finally:
            net.close()


def test_perf_opt_workspace_enters_the_schedule(vdnn, oracle):
    net = vdnn.Network("VGG16_64", "VDNN_ALL", "VDNN_PERF_OPT_ALGO", device=-1, pool_bytes=40e9)
    try:
        specs = [s.astuple() for s in net.layer_specs()]
        L = vdnn.lib()
        ws = []
        for s in specs:
            if s[0] in (1, 2):
                d = vdnn.ConvDesc(s[1], s[2], s[3], s[4], s[9], s[10], s[11], s[5], s[6], s[7], s[8])
                ws.append([L.vdnn_conv_workspace_bytes(op, 1, C.byref(d)) for op in range(3)])
            else:
                ws.append([0, 0, 0])
        assert any(w[2] > 0 for w in ws)            # filter gradients of the wide layers split along K
        net.step()
        ev, summ = oracle.policy_trace(specs, oracle.VDNN_ALL, ws=ws, fix_input_leak=True)
        assert net.trace() == ev and net.stats()["pool_peak_bytes"] == summ.peak_bytes
    finally:
        net.close()


def test_pool_too_small_is_reported_not_fatal(vdnn):
    net = vdnn.Network("VGG16_128", "VDNN_NONE", "VDNN_MEMORY_OPT_ALGO", device=-1, pool_bytes=12e9)
    try:
        with pytest.raises(vdnn.VdnnError) as e:
            net.step()
        assert e.value.status == -5
    finally:
        net.close()        # the pool is per process: one network at a time, as with the reference's cnmem
    # the same model fits under VDNN_ALL, which is the point of the policy
    net = vdnn.Network("VGG16_128", "VDNN_ALL", "VDNN_MEMORY_OPT_ALGO", device=-1, pool_bytes=12e9)
    net.step()
    net.close()


def _perf_workspaces(vdnn, specs):
    L = vdnn.lib()
    ws = []
    for s in specs:
        if s[0] in (1, 2):
            d = vdnn.ConvDesc(s[1], s[2], s[3], s[4], s[9], s[10], s[11], s[5], s[6], s[7], s[8])
            ws.append([L.vdnn_conv_workspace_bytes(op, 1, C.byref(d)) for op in range(3)])
        else:
            ws.append([0, 0, 0])
    return ws


@pytest.mark.parametrize("pool_gb,expect", [(40, (1, 1)), (14.5, (3, 1)), (11, (2, 1)), (5, None)])
def test_dynamic_algo_picks_the_first_policy_that_fits(vdnn, oracle, pool_gb, expect):
    """VDNN_DYNAMIC_ALGO (network.cu:946-1008): NONE, then CONV, then ALL with the workspace-using algorithms;
    a model that does not even fit under VDNN_ALL with zero workspace is refused.  Pool sizes are chosen away
    from the boundaries (peaks 15.6 / 11.8 / 9.2 GB with the workspace-using algorithms), where peak bytes and a real
    allocator agree."""
    specs = [s.astuple() for s in oracle.model_layers(oracle.VGG16_128, 128)]
    assert oracle.dynamic_choice(specs, pool_gb * 1e9, _perf_workspaces(vdnn, specs)) == expect
    if expect is None:
        with pytest.raises(vdnn.VdnnError) as e:
            vdnn.Network("VGG16_128", "BASELINE", "VDNN_DYNAMIC_ALGO", device=-1, pool_bytes=pool_gb * 1e9)
        assert e.value.status == -5
        return
    net = vdnn.Network("VGG16_128", "BASELINE", "VDNN_DYNAMIC_ALGO", device=-1, pool_bytes=pool_gb * 1e9)   # the given policy is ignored
    try:
        assert net.selected() == expect
        net.step()
        net.step()
        ev, summ = oracle.policy_trace(specs, expect[0], ws=_perf_workspaces(vdnn, specs), iterations=2, fix_input_leak=True)
        assert net.trace() == ev and net.stats()["pool_peak_bytes"] == summ.peak_bytes
    finally:
        net.close()


def workspace_heavy_net(n=2):
    """Two 3x3 convolutions on 7x7 maps with many channels: their packed-weight workspaces (8.3 and 4.2 MB)
    dwarf the activations, so the pool size decides which operations may use them."""
    return [(2, n, 256, 7, 7, 1, 1, 1, 1, 256, 3, 3), (3, n, 256, 7, 7, 0, 0, 0, 0, 0, 0, 0),
            (2, n, 256, 7, 7, 1, 1, 1, 1, 128, 3, 3), (3, n, 128, 7, 7, 0, 0, 0, 0, 0, 0, 0),
            (0, n, 128 * 49, 1, 1, 0, 0, 0, 0, 10, 1, 1), (6, n, 10, 1, 1, 0, 0, 0, 0, 0, 0, 0)]


def test_dynamic_algo_per_layer(vdnn, oracle):
    """Step 5 of the dynamic mode (layer.cu:1091-1147): under VDNN_ALL every convolution operation gets the
    workspace-using algorithm only where the iteration still fits the pool."""
    specs = workspace_heavy_net()
    ws = _perf_workspaces(vdnn, specs)
    assert ws[0][0] > 8e6 and ws[2][0] > 4e6
    picks = {}
    for pool in (3_500_000, 4_496_896, 10_000_000, 16_000_000):
        assert (oracle.dynamic_choice(specs, pool, ws) is None) == (pool == 3_500_000)
        try:
            net = vdnn.Network("CUSTOM_CNN", "VDNN_NONE", "VDNN_DYNAMIC_ALGO", device=-1, pool_bytes=pool, custom_layers=specs)
        except vdnn.VdnnError as e:
            picks[pool] = e.status
            continue
        try:
            picks[pool] = (net.selected(), net.layer_algos(0), net.layer_algos(2))
            net.step()
            net.step()            # what was chosen does train within the pool
        finally:
            net.close()
    assert picks[3_500_000] == -5                                         # not even VDNN_ALL with zero workspace
    assert picks[4_496_896] == ((2, 2), (0, 0, 0), (0, 0, 0))             # VDNN_ALL, no room for any workspace
    assert picks[10_000_000] == ((2, 2), (0, 0, 1), (1, 1, 1))            # room for the second layer's workspaces and the first one's smallest
    assert picks[16_000_000] == ((1, 1), (1, 1, 1), (1, 1, 1))            # everything fits without offloading


def test_unsupported_modes_are_refused(vdnn):
    with pytest.raises(vdnn.VdnnError):
        vdnn.Network("GOOGLENET", "BASELINE", "VDNN_MEMORY_OPT_ALGO", device=-1)
    with pytest.raises(vdnn.VdnnError):
        vdnn.Network("CUSTOM_CNN", "BASELINE", "VDNN_MEMORY_OPT_ALGO", device=-1)


def test_custom_topology_dry_run(vdnn, oracle):
    from helpers import tiny_net
    specs = tiny_net(4, with_lrn=True)
    net = vdnn.Network("CUSTOM_CNN", "VDNN_CONV", "VDNN_MEMORY_OPT_ALGO", device=-1, custom_layers=specs)
    try:
        net.step()
        ev, _ = oracle.policy_trace(specs, oracle.VDNN_CONV, fix_input_leak=True)
        assert net.trace() == ev
    finally:
        net.close()


@pytest.mark.parametrize("model", ["ALEXNET", "OVERFEAT", "VGG16_64", "VGG16_128", "VGG16_256"])
def test_baseline_shared_workspace_covers_every_layer(vdnn, oracle, model):
    """BASELINE hands one workspace block to all layers (network.cu:894-906).  The reference sizes it as a maximum
    kept in an int, which wraps for requests beyond 2^31 bytes; a kernel that then writes the workspace it asked for
    would overrun the block.  Here the maximum is kept in 64 bits: the block is at least as large as every request."""
    net = vdnn.Network(model, "BASELINE", "VDNN_PERF_OPT_ALGO", device=-1, pool_bytes=170e9)
    try:
        specs = [s.astuple() for s in net.layer_specs()]
        ws = _perf_workspaces(vdnn, specs)
        largest = max(max(w) for w in ws)
        shared = [e for e in net.trace() if e[0] == 0 and e[1] == -1 and e[2] == 6]       # alloc, network-owned, workspace
        assert len(shared) == 1 and shared[0][3] == largest
        net.step()
        ev, summ = oracle.policy_trace(specs, oracle.BASELINE, ws=ws, fix_input_leak=True, wide_workspace=True)
        assert net.trace() == ev and net.stats()["pool_peak_bytes"] == summ.peak_bytes
    finally:
        net.close()


def test_padded_pooling_is_refused(vdnn):
    specs = [(7, 2, 3, 8, 8, 1, 1, 2, 2, 0, 2, 2), (6, 2, 3, 5, 5, 0, 0, 0, 0, 0, 0, 0)]
    with pytest.raises(vdnn.VdnnError):
        vdnn.Network("CUSTOM_CNN", "VDNN_NONE", "VDNN_MEMORY_OPT_ALGO", device=-1, custom_layers=specs)


def test_lean_offload_schedule_on_the_bookkeeping_pool(vdnn):
    """Lean VDNN_ALL (opt-in, not in the reference): ReLU inputs behind CONV / FC layers are released instead of
    offloaded.  Replayed without a device: fewer offloaded bytes (VGG16: about half), prefetches match offloads, a lower
    peak, the pool back at the same level after every step; the other policies do not change with the switch."""
    def run(policy, lean):
        net = vdnn.Network("VGG16_128", policy, "VDNN_PERF_OPT_ALGO", device=-1, pool_bytes=int(24e9), lean_offload=lean)
        try:
            used = []
            for _ in range(3):
                net.step()
                used.append(net.stats()["pool_used_bytes"])
            return net.stats(), used, net.lean_offload
        finally:
            net.close()
    full, used_full, flag_full = run("VDNN_ALL", False)
    lean, used_lean, flag_lean = run("VDNN_ALL", True)
    assert (flag_full, flag_lean) == (False, True)
    assert lean["offload_bytes"] == lean["prefetch_bytes"] == lean["pinned_bytes"]
    assert 0.45 * full["offload_bytes"] < lean["offload_bytes"] < 0.6 * full["offload_bytes"]
    assert lean["pool_peak_bytes"] < full["pool_peak_bytes"]
    assert used_lean == used_full and len(set(used_lean)) == 1
    for policy in ("VDNN_CONV", "VDNN_NONE"):
        a, _, _ = run(policy, False)
        b, _, _ = run(policy, True)
        assert a["offload_bytes"] == b["offload_bytes"] and a["pool_peak_bytes"] == b["pool_peak_bytes"]


def test_backward_in_one_workspace_is_covered_by_the_filter_gradient_figure(vdnn):
    """Where the two gradients share an image pass over dy, vdnn_conv_bwd_data_filter_bias runs inside the filter gradient's
    workspace window of the reference's schedule, so the figure reported for VDNN_CONV_BWD_FILTER must cover what the
    combined call needs (VDNN_CONV_BWD_ALL) there; elsewhere VDNN_CONV_BWD_ALL is the larger of the two separate figures.
    VGG16's first layer (3 channels) is the one layer of that network that does not share, and the workspace stays at
    about 1 GiB whatever the batch size."""
    L = vdnn.lib()
    for model, batch in (("VGG16_128", 128), ("VGG16_256", 256), ("ALEXNET", 128), ("OVERFEAT", 128)):
        net = vdnn.Network(model, "VDNN_NONE", "VDNN_PERF_OPT_ALGO", device=-1, pool_bytes=int(60e9))
        try:
            specs = net.layer_specs()
        finally:
            net.close()
        shares = []
        for sp in specs:
            if sp.type not in (vdnn.CONV, vdnn.FC_CONV):
                continue
            d = vdnn.ConvDesc(sp.n, sp.c, sp.h, sp.w, sp.k, sp.r, sp.s, sp.pad_h, sp.pad_w, sp.stride_h, sp.stride_w)
            everything, filt = L.vdnn_conv_workspace_bytes(3, 1, C.byref(d)), L.vdnn_conv_workspace_bytes(2, 1, C.byref(d))
            data = L.vdnn_conv_workspace_bytes(1, 1, C.byref(d))
            shares.append(L.vdnn_conv_bwd_shares_dy(C.byref(d), 1))
            if shares[-1]:
                assert everything <= filt <= int(1.25 * 2 ** 30), (model, sp.astuple())
            else:
                assert everything == max(data, filt), (model, sp.astuple())
            assert L.vdnn_conv_workspace_bytes(3, 0, C.byref(d)) == 0 and L.vdnn_conv_bwd_shares_dy(C.byref(d), 0) == 0
        if model.startswith("VGG16"):
            assert shares == [0] + [1] * 12
