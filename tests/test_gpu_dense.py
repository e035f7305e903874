"""GPU suite: layers with few input channels as a dense 1x1 layer over the real positions of every window
(the first layer of an image network: C = 3).  Outputs must be the checker's bits whatever the route."""
import numpy as np
import pytest

import fastertnn_b200 as ft
from cases import BNN, BTN, TBN, TNN, act_ternary, make_case, to_nchw, to_nhwc, wgt_ternary
from fastertnn_b200 import synth
from fastertnn_b200.workloads import Layer

pytestmark = pytest.mark.gpu

DENSE_LAYERS = [
    (TNN, Layer(3, 30, 30, 64, 7, 7, 3, 2), 3),       # the ResNet entry layer's shape: 147 positions -> 256
    (TBN, Layer(3, 20, 24, 64, 3, 3, 1, 1), 2),       # the VGG entry layer's shape: 27 positions -> 64; binary weights
    (TNN, Layer(3, 21, 17, 40, 3, 3, 1, 2), 5),       # odd sizes, stride 2, ragged kernel tile
    (TNN, Layer(1, 16, 16, 33, 5, 5, 2, 1), 4),       # one channel: 25 positions
    (TNN, Layer(8, 14, 14, 100, 3, 3, 1, 2), 3),      # 72 positions -> 128
    (TBN, Layer(16, 12, 12, 128, 3, 3, 1, 1), 2),     # 144 positions -> 256, the widest channel count taken
    (TNN, Layer(3, 13, 13, 300, 11, 11, 5, 4), 2),    # 363 positions -> 512 (two 256-position groups), stride 4
    (TNN, Layer(4, 6, 9, 64, 6, 9, 0, 1), 9),         # the filter is the image: one output pixel per image
]


@pytest.mark.parametrize("type_,layer,N", DENSE_LAYERS, ids=lambda v: str(v).replace(" ", ""))
def test_dense_route_matches_the_checker(type_, layer, N, gpu_ctx, checker):
    ctx = gpu_ctx
    case = make_case(type_, layer, N, 9900 + layer.C * 7 + layer.KN, "uniform")
    # thresholds of zero, negative and ordinary size
    case.thr[:] = np.resize(np.array([0.25, 0.0, -0.1, 0.6], np.float32), N)
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    assert ctx.dense_supported(w, shape)
    nws = ft.api.dense_workspace_bytes(shape)
    d_t = ctx.to_device(case.thr)
    d_x, d_xh = ctx.to_device(case.x), ctx.to_device(to_nhwc(case.x))
    d_y, d_ws = ctx.malloc(want.nbytes), ctx.malloc(nws)
    thr_next = np.resize(np.array([0.0, 0.4, 3.0, -0.2], np.float32), N)
    d_tn, d_f = ctx.to_device(thr_next), ctx.to_device(want)
    nb_o = max(ft.api.e2m1_image_bytes(N, layer.KN, layer.OH, layer.OW), ft.api.packed_image_bytes(True, N, layer.KN, layer.OH, layer.OW))
    d_o, d_q = ctx.malloc(nb_o), ctx.malloc(nb_o)
    try:
        assert ctx.conv_auto_algo(w, shape, d_x) == ft.GEMM_F4_DENSE
        for layout, src in ((ft.NCHW, d_x), (ft.NHWC, d_xh)):
            for how in ("entry", "auto", "request"):
                ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
                ctx.fill(d_ws, np.full(nws // 4, 0x5A5A5A5A, np.uint32))
                if how == "entry":
                    ctx.conv_dense(w, src, d_t, d_y, d_ws, nws, shape, case.alpha, layout)
                elif how == "auto":
                    ctx.conv(w, src, d_t, d_y, shape, case.alpha, layout)
                else:
                    ctx.conv_ws(w, src, d_t, d_y, d_ws, nws, shape, case.alpha, layout, ft.PACK_AUTO, ft.GEMM_F4_DENSE)
                ctx.sync()
                got = ctx.to_host(d_y, want.shape if layout == ft.NCHW else (N, layer.OH, layer.OW, layer.KN), np.float32)
                if layout == ft.NHWC:
                    got = to_nchw(got)
                assert got.tobytes() == want.tobytes(), (layout, how)
        # the padded routes give the same bits (they are what the dense one replaces)
        ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
        ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, ft.NCHW, ft.PACK_AUTO, ft.GEMM_F4_TC)
        ctx.sync()
        assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes(), "padded route"
        # quantising epilogue: the next layer's activations == the quantise kernels' image of the fp32 output
        for fmt in (2, 1, 0):
            ctx.fill(d_q, np.zeros(nb_o // 4, np.uint32))
            ctx.fill(d_o, np.zeros(nb_o // 4, np.uint32))
            if fmt == 2:
                ctx.quantise_e2m1(d_f, d_tn, d_q, N, layer.KN, layer.OH, layer.OW)
            else:
                ctx.quantise(fmt == 1, d_f, d_tn, d_q, N, layer.KN, layer.OH, layer.OW)
            ctx.conv_dense_packed_out(w, d_x, d_t, d_o, d_tn, fmt, d_ws, nws, shape, case.alpha)
            ctx.sync()
            assert np.array_equal(ctx.to_host(d_o, (nb_o // 4,), np.uint32), ctx.to_host(d_q, (nb_o // 4,), np.uint32)), fmt
        # ... and bordered for a slab-fed next layer (padding 1, then 2 rows / 0 columns), over a buffer of stale bytes
        for pad in ((1, 1), (2, 0)):
            nb_b = ft.api.bordered_image_bytes(N, layer.KN, layer.OH, layer.OW, pad[0], pad[1])
            d_ob, d_qb = ctx.malloc(nb_b), ctx.malloc(nb_b)
            if (layer.OH * layer.OW) % 4 == 0 and layer.OH * layer.OW >= 32:
                ctx.fill(d_ob, np.full(nb_b // 4, 0x77777777, np.uint32))
                ctx.quantise_e2m1_bordered(True, d_f, d_tn, d_qb, N, layer.KN, layer.OH, layer.OW, pad[0], pad[1])
                ctx.conv_dense_packed_out(w, d_x, d_t, d_ob, d_tn, 3, d_ws, nws, shape, case.alpha, ft.NCHW, 0, pad)
                ctx.sync()
                assert np.array_equal(ctx.to_host(d_ob, (nb_b // 4,), np.uint32), ctx.to_host(d_qb, (nb_b // 4,), np.uint32)), ("bordered", pad)
            ctx.free(d_ob)
            ctx.free(d_qb)
        with pytest.raises(ft.TnnsError):
            ctx.conv_dense(w, d_x, d_t, d_y, d_ws, nws - 128, shape, case.alpha)
    finally:
        for p in (d_t, d_x, d_xh, d_y, d_ws, d_tn, d_f, d_o, d_q):
            ctx.free(p)
        w.free()


def test_dense_route_declines_what_it_cannot_do(gpu_ctx, checker):
    ctx = gpu_ctx
    for type_, layer, why in ((BTN, Layer(3, 12, 12, 64, 3, 3, 1, 1), "binary activations pad with +1"),
                              (BNN, Layer(3, 12, 12, 64, 3, 3, 1, 1), "binary activations"),
                              (TNN, Layer(64, 12, 12, 64, 3, 3, 1, 1), "a full channel group"),
                              (TNN, Layer(24, 12, 12, 64, 3, 3, 1, 1), "more than 16 channels")):
        case = make_case(type_, layer, 2, 9950, "uniform")
        wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
        want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
        w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
        shape = layer.shape(2)
        assert not ctx.dense_supported(w, shape), why
        d_x, d_t, d_y = ctx.to_device(case.x), ctx.to_device(case.thr), ctx.malloc(want.nbytes)
        with pytest.raises(ft.TnnsError) as e:
            ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, ft.NCHW, ft.PACK_AUTO, ft.GEMM_F4_DENSE)
        assert e.value.status == 4
        ctx.conv(w, d_x, d_t, d_y, shape, case.alpha)
        ctx.sync()
        assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes(), why
        for p in (d_x, d_t, d_y):
            ctx.free(p)
        w.free()


def test_image_chain_starts_with_the_dense_layer(gpu_ctx, checker):
    """A small network whose first layer has three input channels: the image chain quantises it through the dense
    route, hands a plain 4-bit image to the second layer, and ends with the checker's bits."""
    from fastertnn_b200.stack import ConvStack
    layers = [Layer(3, 20, 20, 64, 3, 3, 1, 1), Layer(64, 20, 20, 64, 3, 3, 1, 1), Layer(64, 20, 20, 48, 3, 3, 1, 2)]
    N = 5
    x = synth.uniform_pm1(9970, (N, 3, 20, 20))
    thr = np.full(N, 0.25, np.float32)
    pws = []
    for i, L in enumerate(layers):
        wv = synth.ternary_values(9971 + i, (L.KN, L.C, L.KH, L.KW))
        pws.append(checker.pack_weights(True, wv, np.full(L.KN, 0.5, np.float32)))
    want = x
    for L, pw in zip(layers, pws):
        want = checker.conv(TNN, want, thr, pw, (L.KH, L.KW), (L.P, L.P), (L.S, L.S), 0.5)
    st = ConvStack(gpu_ctx, TNN, layers, pws, N, 0.25, chain="image")
    try:
        # the second layer (64 channels, stride 1) is slab-fed: the dense layer's epilogue writes its bordered image
        assert st.mode[0] == "dense" and st.mode[1] == "slab"
        for rep in range(2):
            gpu_ctx.fill(st.input_ptr(), x)
            st.run()
            gpu_ctx.sync()
            got = gpu_ctx.to_host(st.output_ptr(), want.shape, np.float32)
            assert got.tobytes() == want.tobytes(), rep
    finally:
        st.close()
