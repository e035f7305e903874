"""GPU suite, second part: parity at the sizes the metric is quoted on.  Every byte of the CUDA
result is compared with the CPU checker run over the whole tensor (the reference's protocol,
src/timing_layers.c:142-165, compares whole tensors too), with the checker's images spread over
the host threads so that a full-size layer costs a fraction of a second."""
import ctypes

import numpy as np
import pytest

import fastertnn_b200 as ft
from cases import BNN, BTN, TBN, TNN, act_ternary, make_case, threaded_conv, wgt_ternary
from fastertnn_b200 import synth
from fastertnn_b200.workloads import CONV_LARGE, RESNET18_STACK, RESNET18_STACK_BATCH, Layer, model_layers

pytestmark = pytest.mark.gpu


def weights_for(checker, type_, layer, seed):
    shape_w = (layer.KN, layer.C, layer.KH, layer.KW)
    tern = wgt_ternary(type_)
    w = synth.ternary_values(seed, shape_w) if tern else synth.binary_values(seed, shape_w)
    return checker.pack_weights(tern, w, np.full(layer.KN, 0.5 if tern else 0.0, np.float32))


@pytest.mark.parametrize("type_", [TNN, TBN])
def test_large_layer_full_batch_on_the_default_route(type_, gpu_ctx, checker):
    """The large single layer at its full size -- 64 x 512x32x32 -> 512, 3x3 s1 p1, M = 65536,
    K = 4608, N = 512 -- through tnns_cuda_conv with TNNS_GEMM_AUTO.  At this size the library's
    own rule takes the one-launch kernel on block pairs (asserted), and all 134 MB of output are
    compared with the checker."""
    N, layer = CONV_LARGE
    ctx = gpu_ctx
    x = synth.uniform_pm1(0xC0FFEE40 + type_, (N, layer.C, layer.H, layer.W))
    thr = np.full(N, 0.25, np.float32)
    wp = weights_for(checker, type_, layer, 0xC0FFEE41 + type_)
    want = threaded_conv(checker, type_, x, thr, wp, layer)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    d_x, d_t, d_y = ctx.to_device(x), ctx.to_device(thr), ctx.malloc(want.nbytes)
    try:
        assert ctx.conv_fused_preferred(w, layer.shape(N), d_x, ft.NCHW), "the full-size layer must take the one-launch route"
        for rep in range(2):
            ctx.fill(d_y, np.full(1 << 20, np.nan, np.float32))
            ctx.conv(w, d_x, d_t, d_y, layer.shape(N), 0.5)
            ctx.sync()
            got = ctx.to_host(d_y, want.shape, np.float32)
            assert got.tobytes() == want.tobytes(), f"call {rep}"
        # the slice a rank of an 8-GPU run owns (8 images) takes the small-batch route: same bytes
        ctx.fill(d_y, np.full(1 << 20, np.nan, np.float32))
        ctx.conv(w, d_x + 24 * layer.C * layer.H * layer.W * 4, d_t, d_y, layer.shape(8), 0.5)
        ctx.sync()
        assert ctx.to_host(d_y, (8,) + want.shape[1:], np.float32).tobytes() == want[24:32].tobytes()
        # the same layer pixel-major (NHWC in and out): also the one-launch kernel, its quantiser warps reading
        # swizzled boxes of pixels x channels and its epilogue writing whole sectors of pixel rows
        ctx.free(d_x)
        d_x = ctx.to_device(np.ascontiguousarray(x.transpose(0, 2, 3, 1)))
        assert ctx.conv_fused_preferred(w, layer.shape(N), d_x, ft.NHWC)
        ctx.fill(d_y, np.full(1 << 20, np.nan, np.float32))
        ctx.conv(w, d_x, d_t, d_y, layer.shape(N), 0.5, ft.NHWC)
        ctx.sync()
        got = ctx.to_host(d_y, (N, layer.OH, layer.OW, layer.KN), np.float32)
        assert np.ascontiguousarray(got.transpose(0, 3, 1, 2)).tobytes() == want.tobytes(), "NHWC"
    finally:
        for p in (d_x, d_t, d_y):
            ctx.free(p)
        w.free()


def test_resnet18_style_stack_at_batch_256(gpu_ctx, checker):
    """The 11-layer ternary stack at the batch its figure is quoted on (256): all three ways of
    chaining on the device against the checker chained on the host, every byte of the final
    256 x 512 x 7 x 7 output.  At this batch every layer has thousands of tiles and block pairs and
    the one-launch forms are reached, which a small batch never does."""
    from fastertnn_b200.stack import ConvStack
    N = RESNET18_STACK_BATCH
    L0 = RESNET18_STACK[0]
    x = synth.uniform_pm1(0xC0FFEE50, (N, L0.C, L0.H, L0.W))
    thr = np.full(N, 0.25, np.float32)
    pws = [weights_for(checker, TNN, L, 0xC0FFEE51 + i) for i, L in enumerate(RESNET18_STACK)]
    want = x
    for L, pw in zip(RESNET18_STACK, pws):
        want = threaded_conv(checker, TNN, want, thr, pw, L)
    assert np.count_nonzero(want) > 0
    for chain in ("image", "packed", "fp32"):
        st = ConvStack(gpu_ctx, TNN, RESNET18_STACK, pws, N, 0.25, chain=chain)
        try:
            if chain == "image":
                assert st.mode[:2] == ["slab", "slab"], "the two 64-channel layers take the slab-fed route"
            gpu_ctx.fill(st.input_ptr(), x)
            st.run()
            gpu_ctx.sync()
            got = gpu_ctx.to_host(st.output_ptr(), want.shape, np.float32)
        finally:
            st.close()
        assert got.tobytes() == want.tobytes(), chain


@pytest.mark.parametrize("model", ["resnet18", "resnet34", "vgg16", "darknet19"])
def test_reference_model_tables_chained_like_the_reference(model, gpu_ctx, checker):
    """The layer tables of the reference's end-to-end mode, batch 1, chained as its driver chains
    them (src/timing_layers.c:186-202: every layer's output buffer is the next layer's input, read
    with the next layer's shape), on the device against the checker on the host."""
    from fastertnn_b200.stack import ConvStack
    layers = model_layers(model)
    N = 1
    L0 = layers[0]
    x = synth.ternary_values(0xC0FFEE60, (N, L0.C, L0.H, L0.W))  # the reference's protocol: inputs in the alphabet, thresholds 0.5
    thr = np.full(N, 0.5, np.float32)
    pws = [weights_for(checker, TNN, L, 0xC0FFEE61 + i) for i, L in enumerate(layers)]
    want = x
    for L, pw in zip(layers, pws):
        need = N * L.C * L.H * L.W
        src = np.ascontiguousarray(want.reshape(-1)[:need]).reshape(N, L.C, L.H, L.W)  # where shapes do not chain, the buffer's first floats
        want = checker.conv(TNN, src, thr, pw, (L.KH, L.KW), (L.P, L.P), (L.S, L.S), 0.5)
    for chain in ("fp32", "image"):
        st = ConvStack(gpu_ctx, TNN, layers, pws, N, 0.5, chain=chain, reinterpret_links=True)
        try:
            gpu_ctx.fill(st.input_ptr(), x)
            st.run()
            gpu_ctx.sync()
            got = gpu_ctx.to_host(st.output_ptr(), want.shape, np.float32)
        finally:
            st.close()
        assert got.tobytes() == want.tobytes(), chain


def _device_count():
    import torch
    return torch.cuda.device_count()


def test_device_group_runs_one_host_batch_over_all_devices(checker):
    """tnns_cuda_multi_conv_host: one host batch, split by image index over every visible device
    (a group of one on a single-GPU box still goes through the sharding code), page-locked and
    pageable buffers, a batch smaller than the group, every byte against the checker."""
    G = min(_device_count(), 8)
    layer = Layer(256, 16, 16, 320, 3, 3, 1, 1)
    for type_, N in ((TNN, 37), (BTN, 5), (TBN, max(G - 1, 1))):
        case = make_case(type_, layer, N, 7300 + N, "uniform")
        wp = weights_for(checker, type_, layer, 7400 + type_)
        want = threaded_conv(checker, type_, case.x, case.thr, wp, layer)
        with ft.MultiContext(list(range(G))) as grp:
            w = grp.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
            y = np.full_like(want, np.nan)
            grp.conv_host(w, case.x.ctypes.data, case.thr.ctypes.data, y.ctypes.data, layer.shape(N), 0.5)   # pageable
            assert grp.shard_status == [0] * G
            assert y.tobytes() == want.tobytes()
            ctx0 = ft.Context(0)
            h_x, h_y = ctx0.malloc_host(case.x.nbytes), ctx0.malloc_host(want.nbytes)
            try:
                ctypes.memmove(h_x, case.x.ctypes.data, case.x.nbytes)
                yy = np.ctypeslib.as_array(ctypes.cast(h_y, ctypes.POINTER(ctypes.c_float)), shape=want.shape)
                for _ in range(2):
                    yy.fill(np.nan)
                    grp.conv_host(w, h_x, case.thr.ctypes.data, h_y, layer.shape(N), 0.5)
                    assert yy.tobytes() == want.tobytes()
            finally:
                ctx0.free_host(h_x)
                ctx0.free_host(h_y)
                ctx0.close()
            w.free()


def test_drop_in_layer_over_the_device_group(checker, monkeypatch):
    """The reference's own entry point, tnns_conv(testcase_t*), spreading its batch over the devices
    that TNNS_B200_DEVICES names (from a thread of its own: the variable is read once per thread)."""
    import threading
    G = min(_device_count(), 8)
    if G < 2:
        pytest.skip("needs two devices")
    monkeypatch.setenv("TNNS_B200_DEVICES", ",".join(str(i) for i in range(G)))
    case = make_case(TNN, Layer(128, 12, 12, 96, 3, 3, 1, 1), 19, 7500, "uniform")
    wp = ft.pack_weights_ternary(case.w, case.w_thr)
    want = checker.conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    out = {}

    def run():
        out["y"] = ft.tnns_conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
        out["y2"] = ft.tnns_conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
        ft.load_library().tnns_b200_thread_shutdown()

    t = threading.Thread(target=run)
    t.start()
    t.join()
    assert out["y"].tobytes() == want.tobytes() and out["y2"].tobytes() == want.tobytes()


def test_context_and_weights_of_different_devices_are_refused():
    """A thread that holds contexts on two devices is left on the second one's device; a call on the
    first context must still run on the first device, and weights uploaded through one context are
    refused by the other."""
    if _device_count() < 2:
        pytest.skip("needs two devices")
    layer = Layer(64, 8, 8, 16, 3, 3, 1, 1)
    case = make_case(TNN, layer, 2, 7600, "uniform")
    wp = ft.pack_weights_ternary(case.w, case.w_thr)
    c0, c1 = ft.Context(0), ft.Context(1)   # the thread's current device is now 1
    try:
        w0 = c0.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
        d_x, d_t, d_y = c0.to_device(case.x), c0.to_device(case.thr), c0.malloc(2 * 16 * 8 * 8 * 4)
        c1.sync()                             # leaves device 1 current
        c0.conv(w0, d_x, d_t, d_y, layer.shape(2), 0.5)
        c0.sync()
        y = c0.to_host(d_y, (2, 16, 8, 8), np.float32)
        from oracle import binding
        assert y.tobytes() == binding.best().conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, 0.5).tobytes()
        with pytest.raises(ft.TnnsError) as e:
            c1.conv(w0, d_x, d_t, d_y, layer.shape(2), 0.5)
        assert e.value.status == 1 and "device" in e.value.detail
        for p in (d_x, d_t, d_y):
            c0.free(p)
        w0.free()
    finally:
        c0.close()
        c1.close()
