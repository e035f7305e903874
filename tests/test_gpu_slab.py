"""GPU suite, third part: stride-1 layers from a bordered 4-bit image (the slab-fed GEMM).  The
bordered image is compared with a numpy construction from the checker's packed pixels, every layer
output bit for bit with the CPU checker, for all four network types (binary activations: the
border holds +1), in every form: single blocks, block pairs, one launch, quantising epilogues."""
import numpy as np
import pytest

import fastertnn_b200 as ft
from cases import BNN, BTN, TBN, TNN, act_ternary, make_case, to_nchw, to_nhwc, wgt_ternary
from fastertnn_b200 import synth
from fastertnn_b200.workloads import Layer
from test_gpu_parity import _expand32_f4_numpy, expected_image

pytestmark = pytest.mark.gpu


def expected_bordered(checker, case):
    """[n][Hp][Wp][ic][lo, hi][4 words]: the e2m1 expansion of the checker's packed pixels in the
    interior, the padding value (ternary 0 -> bytes 0x00, binary +1 -> nibbles 0x2) in the border."""
    L = case.layer
    tern = act_ternary(case.type)
    Cp = (L.C + 63) // 64
    planes = expected_image(checker, case).view(np.uint32).reshape(case.N, 2 if tern else 1, L.H * L.W, Cp, 2)
    sign = planes[:, 0]
    zero = planes[:, 1] if tern else np.zeros_like(sign)
    inner = _expand32_f4_numpy(sign, zero).reshape(case.N, L.H, L.W, Cp, 2, 4)
    Hp, Wp = L.H + 2 * L.P, L.W + 2 * L.P
    img = np.full((case.N, Hp, Wp, Cp, 2, 4), 0 if tern else 0x22222222, np.uint32)
    img[:, L.P:L.P + L.H, L.P:L.P + L.W] = inner
    return img


SLAB_LAYERS = [
    (TNN, Layer(256, 14, 14, 256, 3, 3, 1, 1), 4),     # 128-byte pixels, tiles straddle images
    (TNN, Layer(512, 12, 12, 300, 3, 3, 1, 1), 3),     # two channel groups = two slabs per tile, ragged kernel tile
    (TBN, Layer(256, 10, 10, 100, 3, 3, 1, 1), 3),     # binary weights
    (BTN, Layer(256, 10, 12, 96, 3, 3, 1, 1), 3),      # binary activations: the border is +1
    (BNN, Layer(256, 8, 8, 64, 3, 3, 1, 1), 2),
    (TNN, Layer(64, 12, 12, 64, 3, 3, 1, 1), 5),       # 32-byte pixels (32-byte swizzle), weights resident in the ring
    (TNN, Layer(64, 20, 20, 200, 3, 3, 1, 1), 3),      # 32-byte pixels, two kernel tiles: weights through the ring
    (TBN, Layer(64, 10, 10, 200, 3, 3, 1, 1), 5),
    (BTN, Layer(64, 12, 8, 64, 3, 3, 1, 1), 3),
    (BNN, Layer(50, 8, 12, 40, 3, 3, 1, 1), 3),        # binary with a channel tail: absent channels read +1 on both sides
    (TNN, Layer(128, 14, 14, 256, 5, 3, 1, 1), 4),     # 64-byte pixels (64-byte swizzle), 5 x 3 kernel, 15 taps: one pad tap
    (TBN, Layer(100, 10, 10, 100, 3, 3, 1, 1), 3),     # 64-byte pixels with a channel tail
    (TNN, Layer(250, 10, 12, 64, 3, 3, 2, 1), 3),       # padding wider than the kernel reach, channel tail
    (TNN, Layer(256, 10, 10, 128, 3, 3, 0, 1), 3),       # no padding: the lattice is the image itself
    (TNN, Layer(256, 6, 6, 64, 1, 1, 0, 1), 9),        # 1x1: the slab is the tile
    (TNN, Layer(64, 40, 40, 64, 7, 7, 3, 1), 2),       # 49 taps, slab of 128 + 6*46 + 6 rows: two tensor copies per slab
    (TNN, Layer(1024, 8, 8, 512, 3, 3, 1, 1), 3),      # four channel groups, two kernel tiles
]


@pytest.mark.parametrize("type_,layer,N", SLAB_LAYERS, ids=lambda v: str(v).replace(" ", ""))
def test_bordered_image_and_slab_gemm(type_, layer, N, gpu_ctx, checker):
    ctx = gpu_ctx
    case = make_case(type_, layer, N, 9100 + layer.C + layer.KN, "uniform")
    tern = act_ternary(type_)
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    assert ctx.slab_supported(w, shape)
    nb = ft.api.bordered_image_bytes(N, layer.C, layer.H, layer.W, layer.P, layer.P)
    nb_ws = ft.api.slab_workspace_bytes(N, layer.C, layer.H, layer.W, layer.P, layer.P)
    d_t, d_x = ctx.to_device(case.thr), ctx.to_device(case.x)
    d_y, d_img, d_ws = ctx.malloc(want.nbytes), ctx.malloc(nb), ctx.malloc(nb_ws)
    try:
        ctx.fill(d_img, np.full(nb // 4, 0x5A5A5A5A, np.uint32))
        ctx.quantise_e2m1_bordered(tern, d_x, d_t, d_img, N, layer.C, layer.H, layer.W, layer.P, layer.P)
        ctx.sync()
        image = ctx.to_host(d_img, (nb // 4,), np.uint32)
        assert np.array_equal(image, expected_bordered(checker, case).reshape(-1)), "bordered image"
        # the same image from NHWC input (channel counts that are multiples of four)
        d_xh = ctx.to_device(to_nhwc(case.x))
        if layer.C % 4 == 0 and N * layer.H * layer.W >= 128:
            ctx.fill(d_img, np.full(nb // 4, 0x5A5A5A5A, np.uint32))
            ctx.quantise_e2m1_bordered(tern, d_xh, d_t, d_img, N, layer.C, layer.H, layer.W, layer.P, layer.P, ft.NHWC)
            ctx.sync()
            assert np.array_equal(ctx.to_host(d_img, (nb // 4,), np.uint32), image), "bordered image from NHWC input"
            got = np.empty((N, layer.OH, layer.OW, layer.KN), np.float32)
            ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
            assert ctx.conv_auto_algo(w, shape, d_xh, ft.NHWC) in (ft.GEMM_F4_SLAB, ft.GEMM_F4_TC, ft.GEMM_F4_FUSED)
            ctx.conv(w, d_xh, d_t, d_y, shape, case.alpha, ft.NHWC, ft.PACK_AUTO, ft.GEMM_F4_SLAB)
            ctx.sync()
            assert to_nchw(ctx.to_host(d_y, got.shape, np.float32)).tobytes() == want.tobytes(), "slab route, NHWC in and out"
        else:
            with pytest.raises(ft.TnnsError):
                ctx.quantise_e2m1_bordered(tern, d_xh, d_t, d_img, N, layer.C, layer.H, layer.W, layer.P, layer.P, ft.NHWC)
        ctx.free(d_xh)
        for layout in (ft.NCHW, ft.NHWC):
            for pairs in (1, 2):
                if pairs == 2 and layer.KN <= 128:
                    with pytest.raises(ft.TnnsError):
                        ctx.gemm_slab(w, d_img, d_y, shape, case.alpha, layout, 0, 2)
                    continue
                ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
                ctx.gemm_slab(w, d_img, d_y, shape, case.alpha, layout, 0, pairs)
                ctx.sync()
                got = ctx.to_host(d_y, want.shape if layout == ft.NCHW else (N, layer.OH, layer.OW, layer.KN), np.float32)
                if layout == ft.NHWC:
                    got = to_nchw(got)
                assert got.tobytes() == want.tobytes(), (layout, pairs)
        # one launch: quantiser warps write the bordered image (workspace full of stale bytes), twice in a row
        assert ctx.conv_slab_supported(w, shape, d_x, ft.NCHW)
        for pairs in (1, 2, 0):
            if pairs == 2 and layer.KN <= 128:
                continue
            for rep in range(2):
                ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
                ctx.fill(d_ws, np.full(nb_ws // 4, 0xFFFFFFFF, np.uint32))
                ctx.conv_slab(w, d_x, d_t, d_y, d_ws, nb_ws, shape, case.alpha, pairs)
                ctx.sync()
                assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes(), ("one launch", pairs, rep)
                assert np.array_equal(ctx.to_host(d_ws, (nb // 4,), np.uint32), image), "bordered image written by the quantiser warps"
        # through the layer entry point, both forms
        for algo in (ft.GEMM_F4_SLAB, ft.GEMM_F4_SLAB_FUSED):
            ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
            ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, ft.NCHW, ft.PACK_AUTO, algo)
            ctx.sync()
            assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes(), algo
    finally:
        for p in (d_t, d_x, d_y, d_img, d_ws):
            ctx.free(p)
        w.free()


@pytest.mark.parametrize("type_", [TNN, TBN, BTN, BNN])
@pytest.mark.parametrize("channels", [64, 256])
def test_slab_chain_with_quantising_epilogues(type_, channels, gpu_ctx, checker):
    """Three same-size stride-1 layers chained through bordered 4-bit images: the first launch quantises
    the fp32 input itself, every epilogue writes the next layer's image INCLUDING its border (rows on
    border positions write the padding value), the buffers start full of stale bytes, and the last
    layer writes fp32 -- equal to the checker chained on the host.  Then the same producers writing a
    plain 4-bit image and bit planes, compared with what the quantise kernels make of the fp32 tensor."""
    ctx = gpu_ctx
    N, H, W = 3, 14, 10
    tern = act_ternary(type_)
    layers = [Layer(channels, H, W, 100 if channels == 64 else 256, 3, 3, 1, 1), Layer(100 if channels == 64 else 256, H, W, channels, 3, 3, 1, 1),
              Layer(channels, H, W, 72, 3, 3, 1, 1)]
    if channels == 64:
        layers[0] = Layer(64, H, W, 64, 3, 3, 1, 1)
        layers[1] = Layer(64, H, W, 64, 3, 3, 1, 1)
    x = synth.uniform_pm1(9300 + type_, (N, channels, H, W))
    thr = np.array([0.25, 0.4, 0.1], np.float32) if tern else np.array([0.0, 0.1, -0.2], np.float32)
    pws = []
    for i, L in enumerate(layers):
        shape_w = (L.KN, L.C, L.KH, L.KW)
        wv = synth.ternary_values(9400 + i, shape_w) if wgt_ternary(type_) else synth.binary_values(9400 + i, shape_w)
        pws.append(checker.pack_weights(wgt_ternary(type_), wv, np.full(L.KN, 0.5 if wgt_ternary(type_) else 0.0, np.float32)))
    mids = [x]
    for L, pw in zip(layers, pws):
        mids.append(checker.conv(type_, mids[-1], thr, pw, (L.KH, L.KW), (L.P, L.P), (L.S, L.S), 0.5))
    want = mids[-1]
    ws = [ctx.upload_weights(type_, pw, L.C, L.KH, L.KW) for L, pw in zip(layers, pws)]
    bordered = 3 if tern else 5
    nb = max(ft.api.bordered_image_bytes(N, max(L.C, L.KN), H, W, 1, 1) for L in layers)
    nb_ws = ft.api.slab_workspace_bytes(N, channels, H, W, 1, 1)
    d_x, d_t = ctx.to_device(x), ctx.to_device(thr)
    d_a, d_b, d_ws, d_y = ctx.malloc(nb), ctx.malloc(nb), ctx.malloc(nb_ws), ctx.malloc(want.nbytes)
    try:
        for rep in range(2):
            for d in (d_a, d_b):
                ctx.fill(d, np.full(nb // 4, 0x77777777, np.uint32))
            ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
            ctx.conv_slab_packed_out(ws[0], d_x, d_t, d_a, d_t, bordered, (1, 1), d_ws, nb_ws, layers[0].shape(N), 0.5)
            ctx.gemm_slab_packed_out(ws[1], d_a, d_b, d_t, bordered, (1, 1), layers[1].shape(N), 0.5)
            ctx.gemm_slab(ws[2], d_b, d_y, layers[2].shape(N), 0.5)
            ctx.sync()
            assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes(), rep
        # the image a producer wrote for its consumer == the quantise kernel's image of the fp32 intermediate
        mid = mids[1]
        d_m = ctx.to_device(mid)
        L1 = layers[1]
        nb1 = ft.api.bordered_image_bytes(N, L1.C, H, W, 1, 1)
        ctx.quantise_e2m1_bordered(tern, d_m, d_t, d_b, N, L1.C, H, W, 1, 1)
        ctx.sync()
        assert np.array_equal(ctx.to_host(d_a, (nb1 // 4,), np.uint32), ctx.to_host(d_b, (nb1 // 4,), np.uint32)), "bordered image from the epilogue"
        # plain 4-bit image (ternary) and bit planes from the same producer
        if tern:
            ctx.gemm_slab_packed_out(ws[1], d_a, d_b, d_t, 2, (0, 0), layers[1].shape(N), 0.5)
            d_m2 = ctx.to_device(mids[2])
            nbp = ft.api.e2m1_image_bytes(N, layers[1].KN, H, W)
            d_c = ctx.malloc(nbp)
            ctx.quantise_e2m1(d_m2, d_t, d_c, N, layers[1].KN, H, W)
            ctx.sync()
            assert np.array_equal(ctx.to_host(d_b, (nbp // 4,), np.uint32), ctx.to_host(d_c, (nbp // 4,), np.uint32)), "plain image from the epilogue"
            ctx.free(d_m2)
            ctx.free(d_c)
        ctx.gemm_slab_packed_out(ws[1], d_a, d_b, d_t, 1 if tern else 0, (0, 0), layers[1].shape(N), 0.5)
        d_m2 = ctx.to_device(mids[2])
        nbp = ft.api.packed_image_bytes(tern, N, layers[1].KN, H, W)
        d_c = ctx.malloc(nbp)
        ctx.quantise(tern, d_m2, d_t, d_c, N, layers[1].KN, H, W)
        ctx.sync()
        assert np.array_equal(ctx.to_host(d_b, (nbp // 4,), np.uint32), ctx.to_host(d_c, (nbp // 4,), np.uint32)), "bit planes from the epilogue"
        for p in (d_m, d_m2, d_c):
            ctx.free(p)
    finally:
        for p in (d_x, d_t, d_a, d_b, d_ws, d_y):
            ctx.free(p)
        for w in ws:
            w.free()


def test_slab_route_declines_what_it_cannot_do(gpu_ctx, checker):
    ctx = gpu_ctx
    for layer, why in ((Layer(256, 14, 14, 64, 3, 3, 1, 2), "stride 2"), (Layer(192, 14, 14, 64, 3, 3, 1, 1), "three 64-channel groups")):
        case = make_case(TNN, layer, 2, 9500, "uniform")
        wp = checker.pack_weights(True, case.w, case.w_thr)
        w = ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
        assert not ctx.slab_supported(w, layer.shape(2)), why
        d = ctx.malloc(1 << 20)
        with pytest.raises(ft.TnnsError) as e:
            ctx.gemm_slab(w, d, d, layer.shape(2), 0.5)
        assert e.value.status == 4
        with pytest.raises(ft.TnnsError):
            ctx.conv(w, d, d, d, layer.shape(2), 0.5, ft.NCHW, ft.PACK_AUTO, ft.GEMM_F4_SLAB)
        ctx.free(d)
        w.free()
    # a bordered output needs the next layer's padded size to equal this layer's
    layer = Layer(256, 10, 10, 256, 3, 3, 1, 1)
    case = make_case(TNN, layer, 2, 9501, "uniform")
    w = ctx.upload_weights(TNN, checker.pack_weights(True, case.w, case.w_thr), 256, 3, 3)
    d = ctx.malloc(1 << 22)
    with pytest.raises(ft.TnnsError) as e:
        ctx.gemm_slab_packed_out(w, d, d + (1 << 21), d, 3, (2, 2), layer.shape(2), 0.5)
    assert e.value.status == 4
    ctx.free(d)
    w.free()


@pytest.mark.parametrize("tern", [True, False])
@pytest.mark.parametrize("C,H,W,N", [(64, 12, 12, 3), (512, 9, 7, 5), (100, 13, 11, 2), (4, 16, 16, 1), (260, 5, 5, 6), (1024, 3, 3, 15),
                                     (36, 1, 1, 130)])
def test_quantise_from_nhwc_through_the_copy_engine(tern, C, H, W, N, gpu_ctx, checker):
    """NHWC input arrives as 128-byte-swizzled boxes of 128 pixels x 32 channels; the bit planes and the
    4-bit image must equal those made from the same tensor in NCHW (odd pixel counts, channel tails,
    bands that straddle images, 1x1 images)."""
    ctx = gpu_ctx
    x = synth.uniform_pm1(9700 + C + H, (N, C, H, W))
    thr = (synth.uniform_pm1(9701, (N,)) * 0.3 + (0.35 if tern else 0.0)).astype(np.float32)
    d_x, d_xh, d_t = ctx.to_device(x), ctx.to_device(to_nhwc(x)), ctx.to_device(thr)
    nbp = ft.api.packed_image_bytes(tern, N, C, H, W)
    nbe = ft.api.e2m1_image_bytes(N, C, H, W)
    d_a, d_b = ctx.malloc(max(nbp, nbe)), ctx.malloc(max(nbp, nbe))
    try:
        for d in (d_a, d_b):
            ctx.fill(d, np.full(max(nbp, nbe) // 4, 0x3C3C3C3C, np.uint32))
        ctx.quantise(tern, d_x, d_t, d_a, N, C, H, W, ft.NCHW)
        ctx.quantise(tern, d_xh, d_t, d_b, N, C, H, W, ft.NHWC)
        ctx.sync()
        assert np.array_equal(ctx.to_host(d_a, (nbp // 4,), np.uint32), ctx.to_host(d_b, (nbp // 4,), np.uint32)), "bit planes"
        if tern:
            ctx.quantise_e2m1(d_x, d_t, d_a, N, C, H, W, ft.NCHW)
            ctx.quantise_e2m1(d_xh, d_t, d_b, N, C, H, W, ft.NHWC)
            ctx.sync()
            assert np.array_equal(ctx.to_host(d_a, (nbe // 4,), np.uint32), ctx.to_host(d_b, (nbe // 4,), np.uint32)), "4-bit image"
    finally:
        for p in (d_x, d_xh, d_t, d_a, d_b):
            ctx.free(p)


@pytest.mark.parametrize("layer,N", [(Layer(256, 14, 14, 128, 3, 3, 1, 2), 5), (Layer(64, 16, 16, 64, 3, 3, 1, 1), 3), (Layer(128, 12, 20, 200, 5, 3, 2, 2), 4)],
                         ids=lambda v: str(v).replace(" ", ""))
def test_im2col_fed_layer_writes_a_bordered_image(layer, N, gpu_ctx, checker):
    """A layer on the im2col-fed GEMM (strided ones too) hands a slab-fed successor its bordered 4-bit image: every
    output pixel inside the border, the frame written by the same launch -- the bytes the bordered quantise kernel
    makes of the fp32 output, over a buffer of stale bytes, and the successor's output equal to the checker's."""
    ctx = gpu_ctx
    case = make_case(TNN, layer, N, 9600 + layer.C, "uniform")
    wp = checker.pack_weights(True, case.w, case.w_thr)
    mid = checker.conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
    nxt = Layer(layer.KN, layer.OH, layer.OW, 64, 3, 3, 1, 1)
    wv = synth.ternary_values(9601, (nxt.KN, nxt.C, 3, 3))
    wp2 = checker.pack_weights(True, wv, np.full(nxt.KN, 0.5, np.float32))
    thr2 = np.linspace(0.3, 2.0, N).astype(np.float32)
    want = checker.conv(TNN, mid, thr2, wp2, (3, 3), (1, 1), (1, 1), 0.5)
    w2 = ctx.upload_weights(TNN, wp2, nxt.C, 3, 3)
    assert ctx.slab_supported(w2, nxt.shape(N))
    nb_in = ft.api.e2m1_image_bytes(N, layer.C, layer.H, layer.W)
    nb_b = ft.api.bordered_image_bytes(N, nxt.C, nxt.H, nxt.W, 1, 1)
    d_x, d_t, d_t2, d_m = ctx.to_device(case.x), ctx.to_device(case.thr), ctx.to_device(thr2), ctx.to_device(mid)
    d_in, d_b, d_q, d_y = ctx.malloc(nb_in), ctx.malloc(nb_b), ctx.malloc(nb_b), ctx.malloc(want.nbytes)
    try:
        ctx.quantise_e2m1(d_x, d_t, d_in, N, layer.C, layer.H, layer.W)
        for rep in range(2):
            ctx.fill(d_b, np.full(nb_b // 4, 0x66666666, np.uint32))
            ctx.gemm_im2col_bordered_out(w, d_in, d_b, d_t2, (1, 1), layer.shape(N), case.alpha)
            ctx.sync()
            got = ctx.to_host(d_b, (nb_b // 4,), np.uint32)
            if (nxt.H * nxt.W) % 4 == 0 and nxt.H * nxt.W >= 32:
                ctx.quantise_e2m1_bordered(True, d_m, d_t2, d_q, N, nxt.C, nxt.H, nxt.W, 1, 1)
                ctx.sync()
                assert np.array_equal(got, ctx.to_host(d_q, (nb_b // 4,), np.uint32)), ("bordered image", rep)
            ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
            ctx.gemm_slab(w2, d_b, d_y, nxt.shape(N), 0.5)
            ctx.sync()
            assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes(), ("successor", rep)
    finally:
        for p in (d_x, d_t, d_t2, d_m, d_in, d_b, d_q, d_y):
            ctx.free(p)
        w.free()
        w2.free()
