"""GPU test of tnns_cuda_conv_noalloc, the layer entry point for hosts that may not
allocate device memory (arena-owning servers, plug-ins under a foreign caching allocator,
allocation-free latency loops).  Its scratch is a fixed array inside the library, shared
by all calls, so the test makes calls in a row with different geometry and data -- a later
call must not see anything of an earlier one -- and compares each, bit for bit, with the
ordinary entry point (tnns_cuda_conv), which owns a cudaMalloc'd workspace, and with the
CPU checker.  It also watches the device's free memory: a start-up call with an empty batch
is what reserves the array, and no call after it may change the amount of free memory.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import numpy as np
import pytest

import fastertnn_b200 as ft
from fastertnn_b200 import api
from cases import BTN, TNN, make_case, wgt_ternary
from fastertnn_b200.workloads import Layer

pytestmark = pytest.mark.gpu


def run_both(ctx, case):
    """Returns (allocating entry point's output, no-allocation entry point's output, change of
    free device memory across the no-allocation call)."""
    L = case.layer
    shape = L.shape(case.N)
    wp = (ft.pack_weights_ternary if wgt_ternary(case.type) else ft.pack_weights_binary)(case.w, case.w_thr)
    w = ctx.upload_weights(case.type, wp, L.C, L.KH, L.KW)
    d_w = ctx.to_device(wp)            # the caller's own device copy of the packed kernel rows
    d_x, d_t = ctx.to_device(case.x), ctx.to_device(case.thr)
    count = case.N * L.KN * L.OH * L.OW
    d_ref, d_new = ctx.malloc(count * 4), ctx.malloc(count * 4)
    try:
        ctx.conv(w, d_x, d_t, d_ref, shape, case.alpha)
        ctx.sync()
        free_before = ctx.mem_info()[0]
        api.conv_noalloc(case.type, d_w, d_x, d_t, d_new, shape, case.alpha)
        ctx.sync()
        free_after = ctx.mem_info()[0]
        return (ctx.to_host(d_ref, (count,), np.float32), ctx.to_host(d_new, (count,), np.float32), free_before - free_after, wp)
    finally:
        for p in (d_w, d_x, d_t, d_ref, d_new):
            ctx.free(p)
        w.free()


def test_noalloc_layer_matches_allocating_layer_and_checker_in_a_row(checker):
    ctx = ft.Context(0)
    try:
        # the start-up call a host makes before its arena takes the memory: an empty batch launches
        # nothing but resolves (and, with lazy module loading, thereby reserves) the scratch array
        empty = Layer(64, 8, 8, 16, 3, 3, 1, 1).shape(0)
        api.conv_noalloc(TNN, 256, 256, 256, 256, empty, 0.5)
        first = make_case(TNN, Layer(192, 20, 20, 80, 3, 3, 1, 1), 6, 8101, "uniform")
        second = make_case(BTN, Layer(100, 9, 13, 33, 3, 3, 1, 2), 3, 8102, "uniform")  # smaller, other type and row width
        for i, case in enumerate((first, second, first, second)):
            want, got, taken, wp = run_both(ctx, case)
            assert got.tobytes() == want.tobytes()
            cpu = checker.conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
            assert got.tobytes() == cpu.tobytes()
            # the first call of each kind may still load its kernels' code onto the device (lazy
            # module loading); a repeated call must leave the amount of free memory untouched
            if i >= 2:
                assert taken == 0, f"the no-allocation call changed free device memory by {taken} bytes"
    finally:
        ctx.close()


def test_noalloc_rejects_layers_beyond_its_scratch():
    limit = api.noalloc_scratch_bytes()
    assert limit == 32 << 20
    big = Layer(512, 32, 32, 512, 3, 3, 1, 1).shape(64)   # packed matrix of 75.5 MB
    assert ft.packed_bytes(TNN, big) > limit
    with pytest.raises(ft.TnnsError) as e:
        api.conv_noalloc(TNN, 256, 256, 256, 256, big, 0.5)   # refused on sizes alone, before any pointer is used
    assert e.value.status == 4 and "scratch" in e.value.detail
