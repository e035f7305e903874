"""GPU test of tnns_cuda_conv_noalloc, the layer entry point for hosts that may not
allocate device memory (arena-owning servers, plug-ins under a foreign caching allocator,
allocation-free latency loops).  Its scratch is a fixed array inside the library, shared
by all calls, so the test makes two calls in a row with different geometry and data -- the
second must not see anything of the first -- and compares each, bit for bit, with the
ordinary entry point (tnns_cuda_conv), which owns a cudaMalloc'd workspace.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import numpy as np
import pytest

import fastertnn_b200 as ft
from fastertnn_b200 import api
from cases import BTN, TNN, make_case, wgt_ternary
from fastertnn_b200.workloads import Layer

pytestmark = pytest.mark.gpu


def run_both(ctx, case):
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
        api.conv_noalloc(case.type, d_w, d_x, d_t, d_new, shape, case.alpha)
        ctx.sync()
        return ctx.to_host(d_ref, (count,), np.float32), ctx.to_host(d_new, (count,), np.float32)
    finally:
        for p in (d_w, d_x, d_t, d_ref, d_new):
            ctx.free(p)
        w.free()


def test_noalloc_layer_matches_allocating_layer_twice_in_a_row():
    ctx = ft.Context(0)
    try:
        first = make_case(TNN, Layer(192, 20, 20, 80, 3, 3, 1, 1), 6, 8101, "uniform")
        second = make_case(BTN, Layer(100, 9, 13, 33, 3, 3, 1, 2), 3, 8102, "uniform")  # smaller, other type and row width
        for case in (first, second, first):
            want, got = run_both(ctx, case)
            assert got.tobytes() == want.tobytes()
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
