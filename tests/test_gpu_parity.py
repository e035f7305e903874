"""GPU suite: every result of the CUDA path, obtained through the C ABI, is compared
bit-for-bit with the CPU checker (the reference's own objects when oracle/_ref was built,
else the restatement) and with the committed digests."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import fastertnn_b200 as ft
from cases import (BNN, BTN, TBN, TNN, act_ternary, extra_cases, make_case, reference_test_cases, special_value_case, to_nchw,
                   to_nhwc, wgt_ternary)
from fastertnn_b200.workloads import CONV_56, FC_GEMM, Layer

pytestmark = pytest.mark.gpu

DIGESTS = json.loads((Path(__file__).resolve().parent / "golden" / "digests.json").read_text())
CASES = (reference_test_cases(N=2, dist="uniform", max_ops=3e9) + reference_test_cases(N=2, dist="alphabet", max_ops=3e9)
         + extra_cases())


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def device_pack(ctx, case, layout, algo):
    tern = act_ternary(case.type)
    L = case.layer
    shape = L.shape(case.N)
    x = case.x if layout == ft.NCHW else to_nhwc(case.x)
    d_x, d_t = ctx.to_device(x), ctx.to_device(case.thr)
    nbytes = ft.packed_bytes(case.type, shape)
    d_p = ctx.malloc(nbytes + 64)
    try:
        ctx.pack(tern, d_x, d_t, d_p, shape, layout, algo)
        ctx.sync()
        rows = case.N * L.OH * L.OW
        return ctx.to_host(d_p, (rows, nbytes // 8 // rows), np.int64)
    finally:
        for p in (d_x, d_t, d_p):
            ctx.free(p)


def device_conv(ctx, case, wp, layout, pack_algo, gemm_algo):
    L = case.layer
    shape = L.shape(case.N)
    w = ctx.upload_weights(case.type, wp, L.C, L.KH, L.KW)
    x = case.x if layout == ft.NCHW else to_nhwc(case.x)
    d_x, d_t = ctx.to_device(x), ctx.to_device(case.thr)
    d_y = ctx.malloc(case.N * L.KN * L.OH * L.OW * 4)
    try:
        ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, layout, pack_algo, gemm_algo)
        ctx.sync()
        if layout == ft.NCHW:
            return ctx.to_host(d_y, (case.N, L.KN, L.OH, L.OW), np.float32)
        return to_nchw(ctx.to_host(d_y, (case.N, L.OH, L.OW, L.KN), np.float32))
    finally:
        for p in (d_x, d_t, d_y):
            ctx.free(p)
        w.free()


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_layer_matches_checker_and_golden(case, gpu_ctx, checker):
    """pack (both kernels, both layouts) and GEMM (both kernels) against the checker."""
    case = case.build()
    tern = act_ternary(case.type)
    wp = checker.pack_weights(wgt_ternary(case.type), case.w, case.w_thr)
    a_ref = checker.pack(tern, case.x, case.thr, case.kernel_hw, case.padding, case.stride)
    y_ref = checker.conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    d = DIGESTS[case.name]
    assert sha(a_ref) == d["packed"] and sha(y_ref) == d["output"]
    for layout in (ft.NCHW, ft.NHWC):
        for algo in (ft.PACK_GATHER, ft.PACK_STAGED, ft.PACK_AUTO):
            a = device_pack(gpu_ctx, case, layout, algo)
            assert np.array_equal(a, a_ref), f"packed matrix differs (layout {layout}, algo {algo})"
    for layout in (ft.NCHW, ft.NHWC):
        for galgo in (ft.GEMM_POPC_SIMPLE, ft.GEMM_POPC_TILED, ft.GEMM_I8_TC, ft.GEMM_F4_TC, ft.GEMM_AUTO):
            y = device_conv(gpu_ctx, case, wp, layout, ft.PACK_AUTO, galgo)
            assert y.tobytes() == y_ref.tobytes(), f"output differs (layout {layout}, gemm {galgo})"
    assert sha(device_conv(gpu_ctx, case, wp, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO)) == d["output"]


@pytest.mark.parametrize("case", (reference_test_cases(N=2, dist="uniform", max_ops=3e9)[::5] + extra_cases()[::7]),
                         ids=lambda c: c.name)
def test_drop_in_entry_points(case, checker):
    """The seven reference symbols, host pointers in and malloc'd host buffers out."""
    case = case.build()
    tern = act_ternary(case.type)
    L = case.layer
    wp = ft.pack_weights_ternary(case.w, case.w_thr) if wgt_ternary(case.type) else ft.pack_weights_binary(case.w, case.w_thr)
    assert np.array_equal(wp, checker.pack_weights(wgt_ternary(case.type), case.w, case.w_thr))
    y_ref = checker.conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    y = ft.tnns_conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    assert y.tobytes() == y_ref.tobytes()
    a = (ft.t2r_p2_opt if tern else ft.b2r)(case.x, case.thr, case.kernel_hw, case.padding, case.stride)
    assert np.array_equal(a, checker.pack(tern, case.x, case.thr, case.kernel_hw, case.padding, case.stride))
    K = L.KH * L.KW * ((L.C + 63) // 64)
    if case.type == BNN:
        y2 = ft.mm_bnn(a, wp, case.N, L.OH, L.OW, L.KN, K, L.C * L.KH * L.KW, case.alpha)
    else:
        y2 = {TNN: ft.mm_tnn, TBN: ft.mm_tbn, BTN: ft.mm_btn}[case.type](a, wp, case.N, L.OH, L.OW, L.KN, K, case.alpha)
    assert y2.tobytes() == y_ref.tobytes()


@pytest.mark.parametrize("type_", [TNN, TBN, BTN, BNN])
def test_special_values(type_, gpu_ctx, checker):
    """+-0, values equal to and next to the thresholds, denormals and infinities quantise as
    in the reference, in every pack kernel and layout."""
    case = special_value_case(type_)
    a_ref = checker.pack(act_ternary(type_), case.x, case.thr, case.kernel_hw, case.padding, case.stride)
    for layout in (ft.NCHW, ft.NHWC):
        for algo in (ft.PACK_GATHER, ft.PACK_STAGED):
            assert np.array_equal(device_pack(gpu_ctx, case, layout, algo), a_ref), (layout, algo)
    # W not a multiple of four takes the scalar-load variant of the staged kernel
    odd = special_value_case(type_)
    odd.layer = Layer(96, 6, 7, 16, 3, 3, 1, 1)
    odd.x = np.ascontiguousarray(odd.x[:, :, :, :7])
    a_ref = checker.pack(act_ternary(type_), odd.x, odd.thr, odd.kernel_hw, odd.padding, odd.stride)
    assert np.array_equal(device_pack(gpu_ctx, odd, ft.NCHW, ft.PACK_STAGED), a_ref)


def test_tnns_gemm_entry_point(checker):
    """tnns_gemm: packed TNN operands, alpha fixed to 1, optional caller-owned output."""
    m, n, words = 70, 45, 8
    rng = np.random.default_rng(5)
    x = rng.integers(-1, 2, size=(m, words * 64)).astype(np.float32).reshape(m, words * 64, 1, 1)
    w = rng.integers(-1, 2, size=(n, words * 64)).astype(np.float32).reshape(n, words * 64, 1, 1)
    xa = checker.pack(True, x, np.full(m, 0.5, np.float32), (1, 1))
    wa = checker.pack_weights(True, w, np.full(n, 0.5, np.float32))
    ref = checker.mm(TNN, xa, wa, m, 1, 1, n, words, 1.0).reshape(m, n)
    got = ft.tnns_gemm(xa, wa, m, n, words)
    assert got.tobytes() == ref.tobytes()
    assert np.array_equal(got, x.reshape(m, -1) @ w.reshape(n, -1).T)  # alpha = 1: plain integer product
    out = np.full((m, n), -7.0, np.float32)
    ft.tnns_gemm(xa, wa, m, n, words, out=out)
    assert out.tobytes() == ref.tobytes()


@pytest.mark.parametrize("type_", [TNN, TBN, BTN])
def test_benchmark_configs_small_enough_for_the_checker(type_, gpu_ctx, checker):
    """The FC (GEMM) configuration and the batch-1 56x56x256 conv, at full size."""
    for N, layer in (FC_GEMM, CONV_56):
        if type_ != TNN and layer is FC_GEMM[1]:
            continue
        case = make_case(type_, layer, N, 31337 + type_, "uniform")
        case.thr[:] = 0.25 if act_ternary(type_) else 0.0
        wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
        y_ref = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
        for layout in (ft.NCHW, ft.NHWC):
            for galgo in (ft.GEMM_AUTO, ft.GEMM_I8_TC, ft.GEMM_F4_TC, ft.GEMM_POPC_TILED):
                y = device_conv(gpu_ctx, case, wp, layout, ft.PACK_AUTO, galgo)
                assert y.tobytes() == y_ref.tobytes(), (layout, galgo)


def test_host_buffer_layer_matches_device_layer(gpu_ctx, checker):
    """tnns_cuda_conv_host slices the batch and overlaps copies; results must not change."""
    layer = Layer(128, 12, 12, 96, 3, 3, 1, 1)
    case = make_case(TNN, layer, 19, 99, "uniform")  # 19 images -> slices of 3 with a ragged tail
    wp = checker.pack_weights(True, case.w, case.w_thr)
    y_ref = checker.conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = gpu_ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
    y = np.empty_like(y_ref)
    for _ in range(2):  # second call reuses the staging buffers
        y.fill(np.nan)
        gpu_ctx.conv_host(w, case.x.ctypes.data, case.thr.ctypes.data, y.ctypes.data, layer.shape(case.N), case.alpha)
        assert y.tobytes() == y_ref.tobytes()
    w.free()


@pytest.mark.gpu
def test_host_buffer_layer_on_page_locked_buffers(gpu_ctx, checker):
    """Page-locked host buffers (tnns_cuda_malloc_host) through the host-buffer layer call: same
    bytes as the reference on two calls in a row, for batches whose slices take the one-launch
    route, 64-channel pixels, and a ragged last slice."""
    import ctypes
    ctx = gpu_ctx
    for layer, N in ((Layer(256, 16, 16, 320, 3, 3, 1, 1), 160), (Layer(64, 48, 48, 64, 3, 3, 1, 1), 264), (Layer(128, 12, 12, 96, 3, 3, 1, 1), 19)):
        case = make_case(TNN, layer, N, 4200 + N, "uniform")
        wp = checker.pack_weights(True, case.w, case.w_thr)
        want = checker.conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
        w = ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
        h_x, h_y = ctx.malloc_host(case.x.nbytes), ctx.malloc_host(want.nbytes)
        try:
            ctypes.memmove(h_x, case.x.ctypes.data, case.x.nbytes)
            y = np.ctypeslib.as_array(ctypes.cast(h_y, ctypes.POINTER(ctypes.c_float)), shape=want.shape)
            for _ in range(2):
                y.fill(np.nan)
                ctx.conv_host(w, h_x, case.thr.ctypes.data, h_y, layer.shape(N), case.alpha)
                assert y.tobytes() == want.tobytes()
        finally:
            ctx.free_host(h_x)
            ctx.free_host(h_y)
            w.free()


def test_empty_batch_is_a_no_op(gpu_ctx):
    layer = Layer(64, 4, 4, 8, 3, 3, 1, 1)
    shape = layer.shape(0)
    wp = ft.pack_weights_ternary(np.zeros((8, 64, 3, 3), np.float32), np.full(8, 0.5, np.float32))
    w = gpu_ctx.upload_weights(TNN, wp, 64, 3, 3)
    d = gpu_ctx.malloc(64)
    gpu_ctx.conv(w, d, d, d, shape, 0.5)
    gpu_ctx.sync()
    gpu_ctx.free(d)
    w.free()


def test_argument_errors_are_reported_not_fatal(gpu_ctx):
    layer = Layer(64, 4, 4, 8, 3, 3, 1, 1)
    wp = ft.pack_weights_ternary(np.zeros((8, 64, 3, 3), np.float32), np.full(8, 0.5, np.float32))
    w = gpu_ctx.upload_weights(TNN, wp, 64, 3, 3)
    d = gpu_ctx.malloc(1 << 16)
    with pytest.raises(ft.TnnsError) as e:
        gpu_ctx.conv(w, 0, d, d, layer.shape(1), 0.5)          # NULL input
    assert e.value.status == 1
    with pytest.raises(ft.TnnsError):
        gpu_ctx.conv(w, d, d, d, Layer(32, 4, 4, 8, 3, 3, 1, 1).shape(1), 0.5)   # weights are for C=64
    with pytest.raises(ft.TnnsError):
        gpu_ctx.conv(w, d, d, d, Layer(64, 2, 2, 8, 3, 3, 0, 1).shape(1), 0.5)   # kernel larger than image
    with pytest.raises(ft.TnnsError):
        gpu_ctx.pack(True, d, d, d + 8, layer.shape(1))          # misaligned output
    with pytest.raises(ft.TnnsError) as e:
        gpu_ctx.conv(w, d, d, d, layer.shape(1), 0.5, gemm_algo=99)
    assert e.value.status == 1
    # the context is still usable afterwards
    gpu_ctx.conv(w, d, d, d + 4096, layer.shape(1), 0.5)
    gpu_ctx.sync()
    gpu_ctx.free(d)
    w.free()


def test_large_layer_properties(gpu_ctx, checker):
    """The large-layer configuration (512 channels, 32x32, 512 kernels) at a batch the GPU
    runs in milliseconds, checked through properties that need no full-size CPU run:
    (1) images 0..1 of the batch equal the checker's result for those images alone;
    (2) the tiled and the one-thread-per-output GEMM agree on every element;
    (3) negating the activations negates the integer accumulator (ternary quantisation with
        symmetric thresholds is odd, the GEMM is linear)."""
    layer = Layer(512, 32, 32, 512, 3, 3, 1, 1)
    N = 16
    case = make_case(TNN, layer, N, 2024, "uniform")
    case.thr[:] = 0.25
    wp = checker.pack_weights(True, case.w, case.w_thr)
    y = device_conv(gpu_ctx, case, wp, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO)
    y2 = checker.conv(TNN, case.x[:2], case.thr[:2], wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    assert y[:2].tobytes() == y2.tobytes()
    y_simple = device_conv(gpu_ctx, case, wp, ft.NCHW, ft.PACK_GATHER, ft.GEMM_POPC_SIMPLE)
    assert y.tobytes() == y_simple.tobytes()
    for galgo in (ft.GEMM_POPC_TILED, ft.GEMM_I8_TC, ft.GEMM_F4_TC):
        assert device_conv(gpu_ctx, case, wp, ft.NCHW, ft.PACK_AUTO, galgo).tobytes() == y_simple.tobytes(), galgo
    neg = make_case(TNN, layer, N, 2024, "uniform")
    neg.thr[:] = 0.25
    neg.x = -neg.x
    yn = device_conv(gpu_ctx, neg, wp, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO)
    acc = np.where(y > 0, y, y / 0.5)
    accn = np.where(yn > 0, yn, yn / 0.5)
    assert np.array_equal(acc, -accn)
    assert np.abs(acc).max() <= 4608


def test_resnet18_style_stack_chained_on_device(gpu_ctx, checker):
    """The 11-layer ternary stack (two convs per stage, stride-2 transitions), batch 2: layers
    chained on the device, each output re-ternarised with +-0.25 as the next input, against the
    checker chained the same way on the host."""
    from fastertnn_b200 import synth
    from fastertnn_b200.stack import ConvStack
    from fastertnn_b200.workloads import RESNET18_STACK
    N = 2
    x = synth.uniform_pm1(77, (N, 64, 56, 56))
    thr = np.full(N, 0.25, np.float32)
    pws = []
    for i, L in enumerate(RESNET18_STACK):
        w = synth.ternary_values(500 + i, (L.KN, L.C, L.KH, L.KW))
        pws.append(checker.pack_weights(True, w, np.full(L.KN, 0.5, np.float32)))
    want = x
    for L, pw in zip(RESNET18_STACK, pws):
        want = checker.conv(TNN, want, thr, pw, (L.KH, L.KW), (L.P, L.P), (L.S, L.S), 0.5)
    for chain in ("fp32", "packed", "image"):
        st = ConvStack(gpu_ctx, TNN, RESNET18_STACK, pws, N, 0.25, chain=chain)
        gpu_ctx.lib.tnns_cuda_memcpy_h2d(gpu_ctx.handle, st.input_ptr(), x.ctypes.data, x.nbytes)
        st.run()
        gpu_ctx.sync()
        got = gpu_ctx.to_host(st.output_ptr(), want.shape, np.float32)
        st.close()
        assert got.tobytes() == want.tobytes(), chain
        assert np.count_nonzero(got) > 0


@pytest.mark.parametrize("type_", [TNN, TBN])
def test_image_chain_switches_formats_between_layers(type_, gpu_ctx, checker):
    """A stack whose layers alternate between the copy-engine route (4-bit image in) and the gathering
    route (bit planes in): 64 -> 192 channels (three 64-channel groups: not eligible) -> 256 -> 100
    (ragged) -> 128.  Every producer writes the format its consumer reads; final output bit-identical
    to the checker chained on the host, for ternary and for binary weights."""
    from fastertnn_b200 import synth
    from fastertnn_b200.stack import ConvStack
    layers = [Layer(64, 12, 12, 192, 3, 3, 1, 1), Layer(192, 12, 12, 256, 3, 3, 1, 2), Layer(256, 6, 6, 100, 3, 3, 1, 1),
              Layer(100, 6, 6, 128, 1, 1, 0, 1), Layer(128, 6, 6, 40, 3, 3, 1, 1)]
    N = 3
    x = synth.uniform_pm1(31, (N, 64, 12, 12))
    thr = np.full(N, 0.25, np.float32)
    tern_w = wgt_ternary(type_)
    pws = []
    for i, L in enumerate(layers):
        shape_w = (L.KN, L.C, L.KH, L.KW)
        w = synth.ternary_values(900 + i, shape_w) if tern_w else synth.binary_values(900 + i, shape_w)
        pws.append(checker.pack_weights(tern_w, w, np.full(L.KN, 0.5 if tern_w else 0.0, np.float32)))
    want = x
    for L, pw in zip(layers, pws):
        want = checker.conv(type_, want, thr, pw, (L.KH, L.KW), (L.P, L.P), (L.S, L.S), 0.5)
    st = ConvStack(gpu_ctx, type_, layers, pws, N, 0.25, chain="image")
    assert st.fast == [True, False, True, True, True]
    gpu_ctx.fill(st.input_ptr(), x)
    st.run()
    gpu_ctx.sync()
    got = gpu_ctx.to_host(st.output_ptr(), want.shape, np.float32)
    st.close()
    assert got.tobytes() == want.tobytes()
    assert np.count_nonzero(got) > 0


@pytest.mark.parametrize("type_", [TNN, TBN, BTN, BNN])
def test_quantising_epilogue_and_packed_im2row(type_, gpu_ctx, checker):
    """Two chained layers with the intermediate kept as bit planes: the im2row matrix built from the
    GEMM's quantised output equals the checker's pack of the fp32 intermediate, and the second
    layer's fp32 output equals the checker's.  Kernel counts 100 and 40 leave ragged 32- and
    64-channel tails in the planes; per-image thresholds differ."""
    l1, l2 = Layer(96, 10, 9, 100, 3, 3, 1, 1), Layer(100, 10, 9, 40, 3, 3, 1, 2)
    c1 = make_case(type_, l1, 3, 700 + type_, "uniform")
    c2 = make_case(type_, l2, 3, 710 + type_, "uniform")
    tern = act_ternary(type_)
    thr2 = np.array([0.25, 3.0, 0.0], np.float32) if tern else np.array([0.0, -2.0, 1.5], np.float32)
    w1 = checker.pack_weights(wgt_ternary(type_), c1.w, c1.w_thr)
    w2 = checker.pack_weights(wgt_ternary(type_), c2.w, c2.w_thr)
    y1 = checker.conv(type_, c1.x, c1.thr, w1, c1.kernel_hw, c1.padding, c1.stride, 0.5)
    a2_ref = checker.pack(tern, y1, thr2, c2.kernel_hw, c2.padding, c2.stride)
    y2_ref = checker.conv(type_, y1, thr2, w2, c2.kernel_hw, c2.padding, c2.stride, 0.5)
    ctx = gpu_ctx
    W1 = ctx.upload_weights(type_, w1, l1.C, l1.KH, l1.KW)
    W2 = ctx.upload_weights(type_, w2, l2.C, l2.KH, l2.KW)
    s1, s2 = l1.shape(3), l2.shape(3)
    d_x, d_t1, d_t2 = ctx.to_device(c1.x), ctx.to_device(c1.thr), ctx.to_device(thr2)
    d_a1 = ctx.malloc(ft.packed_bytes(type_, s1))
    d_img = ctx.malloc(ft.api.packed_image_bytes(tern, 3, l1.KN, l1.OH, l1.OW))
    d_a2 = ctx.malloc(ft.packed_bytes(type_, s2))
    d_y2 = ctx.malloc(y2_ref.nbytes)
    try:
        ctx.pack(tern, d_x, d_t1, d_a1, s1)
        ctx.gemm_packed_out(W1, d_a1, d_img, d_t2, tern, 3, l1.OH, l1.OW, 0.5)
        ctx.im2row_packed(tern, d_img, d_a2, s2)
        ctx.gemm(W2, d_a2, d_y2, 3, l2.OH, l2.OW, 0.5)
        ctx.sync()
        a2 = ctx.to_host(d_a2, a2_ref.shape, np.int64)
        assert np.array_equal(a2, a2_ref)
        assert ctx.to_host(d_y2, y2_ref.shape, np.float32).tobytes() == y2_ref.tobytes()
    finally:
        for p in (d_x, d_t1, d_t2, d_a1, d_img, d_a2, d_y2):
            ctx.free(p)
        W1.free()
        W2.free()


def expected_image(checker, case):
    """Packed image [n][plane][pixel][ic] derived from the checker's 1x1 pack of the same tensor
    (for a 1x1 window plane word j is channel group j of the pixel)."""
    tern = act_ternary(case.type)
    L = case.layer
    Cp = (L.C + 63) // 64
    rows = checker.pack(tern, case.x, case.thr, (1, 1)).view(np.uint64)          # [N*H*W][planes*Kp]
    Kp = rows.shape[1] // (2 if tern else 1)
    j = np.arange(Cp)
    if tern:
        sign = rows[:, (j // 4) * 8 + j % 4]
        zero = rows[:, (j // 4) * 8 + j % 4 + 4]
        img = np.stack([sign.reshape(case.N, L.H * L.W, Cp), zero.reshape(case.N, L.H * L.W, Cp)], axis=1)
    else:
        img = rows[:, :Cp].reshape(case.N, 1, L.H * L.W, Cp)
    assert Kp >= Cp
    return np.ascontiguousarray(img)


IMPLICIT_LAYERS = [
    Layer(256, 12, 10, 72, 3, 3, 1, 1),    # C_pack = 4: a stage is one tap, 128-bit gathers
    Layer(512, 9, 9, 300, 3, 3, 1, 2),     # stride 2, kernel count with a tail
    Layer(64, 11, 13, 64, 3, 3, 1, 1),     # C_pack = 1: a stage spans four taps, Kw = 9 -> pad words
    Layer(200, 7, 7, 40, 5, 3, 2, 1),      # C_pack = 4 with a channel tail, non-square kernel, pad 2
    Layer(130, 6, 6, 33, 2, 2, 3, 1),      # padding wider than the kernel, C_pack = 3
    Layer(320, 1, 1, 96, 1, 1, 0, 1),      # fully connected
]


@pytest.mark.parametrize("type_", [TNN, TBN, BTN, BNN])
@pytest.mark.parametrize("layer", IMPLICIT_LAYERS, ids=str)
def test_quantise_and_implicit_im2row_gemm(type_, layer, gpu_ctx, checker):
    """The default layer route: quantise to a packed image, then the GEMM gathers its im2row rows
    itself.  Image against the checker's 1x1 pack, output against the checker's layer, both layouts."""
    case = make_case(type_, layer, 3, 900 + type_, "uniform")
    tern = act_ternary(type_)
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    y_ref = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    img_ref = expected_image(checker, case)
    ctx = gpu_ctx
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    d_t = ctx.to_device(case.thr)
    d_img = ctx.malloc(ft.api.packed_image_bytes(tern, case.N, layer.C, layer.H, layer.W))
    d_y = ctx.malloc(y_ref.nbytes)
    try:
        for layout in (ft.NCHW, ft.NHWC):
            d_x = ctx.to_device(case.x if layout == ft.NCHW else to_nhwc(case.x))
            ctx.quantise(tern, d_x, d_t, d_img, case.N, layer.C, layer.H, layer.W, layout)
            ctx.gemm_implicit(w, d_img, d_y, layer.shape(case.N), case.alpha, layout)
            ctx.sync()
            ctx.free(d_x)
            img = ctx.to_host(d_img, img_ref.shape, np.uint64)
            assert np.array_equal(img, img_ref), layout
            if layout == ft.NCHW:
                y = ctx.to_host(d_y, y_ref.shape, np.float32)
            else:
                y = to_nchw(ctx.to_host(d_y, (case.N, layer.OH, layer.OW, layer.KN), np.float32))
            assert y.tobytes() == y_ref.tobytes(), layout
    finally:
        for p in (d_t, d_img, d_y):
            ctx.free(p)
        w.free()


@pytest.mark.parametrize("case", extra_cases()[::5] + reference_test_cases(N=1, dist="uniform", max_ops=3e9)[5::7], ids=lambda c: c.name)
def test_device_weight_packing(case, gpu_ctx, checker):
    """fp32 weights packed on the device equal the reference's host packers byte for byte; weights
    uploaded from that device buffer give the same layer output."""
    case = case.build()
    L = case.layer
    tern = wgt_ternary(case.type)
    w = case.w.copy()
    w.reshape(-1)[::7] *= 0.3      # values strictly inside the thresholds, not only the alphabet
    w.reshape(-1)[3::11] = 0.5     # and exactly on the ternary threshold
    want = checker.pack_weights(tern, w, case.w_thr)
    ctx = gpu_ctx
    d_w, d_t = ctx.to_device(w), ctx.to_device(case.w_thr)
    d_p = ctx.malloc(want.nbytes)
    try:
        ctx.pack_weights_device(tern, d_w, d_t, d_p, L.KN, L.C, L.KH, L.KW)
        ctx.sync()
        got = ctx.to_host(d_p, want.shape, np.int64)
        assert np.array_equal(got, want)
        h = ft.api.C.c_void_p()
        ft.api._check(ctx.lib.tnns_cuda_upload_weights(ctx.handle, case.type, d_p, L.KN, L.C, L.KH, L.KW, ft.api.C.byref(h)))
        wd = ft.Weights(ctx, h.value, case.type, L.KN)
        y_ref = checker.conv(case.type, case.x, case.thr, want, case.kernel_hw, case.padding, case.stride, case.alpha)
        d_x, d_thr = ctx.to_device(case.x), ctx.to_device(case.thr)
        d_y = ctx.malloc(y_ref.nbytes)
        ctx.conv(wd, d_x, d_thr, d_y, L.shape(case.N), case.alpha)
        ctx.sync()
        assert ctx.to_host(d_y, y_ref.shape, np.float32).tobytes() == y_ref.tobytes()
        for p in (d_x, d_thr, d_y):
            ctx.free(p)
        wd.free()
    finally:
        for p in (d_w, d_t, d_p):
            ctx.free(p)


def test_bounded_wait_expiry_is_reported_and_context_survives(gpu_ctx):
    """Every on-device wait has a limit.  A kernel whose wait nothing satisfies returns after about
    a second with the status word set; sync reports it once, and the same context then runs a layer."""
    ctx = gpu_ctx
    ft.api._check(ctx.lib.tnns_cuda_selftest_wait_expiry(ctx.handle))
    with pytest.raises(ft.TnnsError) as e:
        ctx.sync()
    assert e.value.status == 5 and "wait" in e.value.detail
    ctx.sync()  # the status word was cleared: no error the second time
    layer = Layer(64, 6, 6, 16, 3, 3, 1, 1)
    case = make_case(TNN, layer, 2, 4321, "uniform")
    wp = ft.pack_weights_ternary(case.w, case.w_thr)
    y = device_conv(ctx, case, wp, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO)
    assert np.isfinite(y).all() and y.shape == (2, 16, 6, 6)


def test_pipe_rate_microbenchmarks_report_plausible_rates(gpu_ctx):
    """The denominators of the pipe-utilisation figures: integer issue rates and the rate of a bare
    tcgen05.mma loop.  LOP3 issues faster than POPC; the 4-bit MMA kind runs faster than int8;
    both tensor rates lie between 0.5 and 20 peta-operations per second on this part."""
    ctx = gpu_ctx
    lop3, popc = ctx.pipe_rate(0), ctx.pipe_rate(1)
    assert lop3 > popc > 0
    i8, f4 = ctx.pipe_rate(3), ctx.pipe_rate(4)
    assert 0.5e6 < i8 < f4 < 20e6
    ctx.sync()
    with pytest.raises(ft.TnnsError):
        ctx.pipe_rate(5)


def _expand32_f4_numpy(s, z):
    """numpy restatement of the library's 32-element e2m1 expansion (uint32 in, four uint32 out)."""
    s = s.astype(np.uint32)
    z = z.astype(np.uint32)
    x = (s & np.uint32(0xCCCCCCCC)) | (~(z >> np.uint32(2)) & np.uint32(0x33333333))
    y = ((s << np.uint32(2)) & np.uint32(0xCCCCCCCC)) | (~z & np.uint32(0x33333333))
    a = np.uint32(0xAAAAAAAA)
    return np.stack([x & a, (x << np.uint32(1)) & a, y & a, (y << np.uint32(1)) & a], axis=-1)


IM2COL_LAYERS = [
    (TNN, Layer(256, 14, 14, 256, 3, 3, 1, 1), 4),     # straddles images: 196 pixels per image, 128-row tiles
    (TNN, Layer(256, 14, 14, 256, 5, 3, 1, 2), 8),     # 5 x 3 kernel, stride 2
    (TBN, Layer(256, 10, 10, 100, 3, 3, 1, 2), 3),     # binary weights, kernel count below one tile
    (TNN, Layer(1024, 14, 14, 1024, 5, 5, 1, 2), 2),   # 16 channel groups, four kernel tiles
    (TNN, Layer(256, 7, 7, 32, 3, 3, 1, 2), 1),        # image far below 128 KiB
    (TNN, Layer(512, 1, 1, 512, 1, 1, 0, 1), 8),       # fully connected
    (TNN, Layer(250, 9, 11, 64, 3, 3, 2, 3), 3),       # channel tail, padding 2, stride 3
    (TBN, Layer(512, 9, 11, 300, 3, 3, 0, 1), 3),      # no padding, ragged kernel tile
    (TNN, Layer(64, 9, 9, 200, 3, 3, 1, 1), 5),        # C_pack = 1: four taps per stage row (32-byte swizzle), three pad taps
    (TBN, Layer(64, 9, 9, 200, 3, 3, 1, 1), 5),        # the same against binary weights (pad words must not count)
    (TNN, Layer(128, 14, 14, 256, 5, 3, 1, 2), 4),     # C_pack = 2: two taps per stage row (64-byte swizzle), one pad tap
    (TBN, Layer(128, 10, 10, 100, 3, 3, 1, 2), 3),
    (TNN, Layer(100, 9, 11, 64, 3, 3, 2, 3), 3),       # C_pack = 2 with a channel tail
    (TNN, Layer(64, 12, 12, 32, 1, 1, 0, 1), 3),       # C_pack = 1, 1x1: one real tap, three pad taps
]


@pytest.mark.gpu
@pytest.mark.parametrize("type_,layer,N", IM2COL_LAYERS, ids=lambda v: str(v).replace(" ", ""))
def test_e2m1_image_and_im2col_tensor_copy_gemm(type_, layer, N, gpu_ctx, checker):
    """The copy-engine route: the 4-bit image holds the expansion of the bit-plane image, and the GEMM
    fed by im2col tensor copies equals the reference layer bit for bit, in both tensor layouts."""
    ctx = gpu_ctx
    case = make_case(type_, layer, N, 6100 + layer.C + layer.KN, "uniform")
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    assert ctx.im2col_supported(w, shape)
    Cp = (layer.C + 63) // 64
    nb_e = ft.api.e2m1_image_bytes(N, layer.C, layer.H, layer.W)
    nb_p = ft.api.packed_image_bytes(True, N, layer.C, layer.H, layer.W)
    assert nb_e == N * layer.H * layer.W * Cp * 32
    d_t = ctx.to_device(case.thr)
    d_y = ctx.malloc(want.nbytes)
    d_e = ctx.malloc(nb_e)
    d_p = ctx.malloc(nb_p)
    try:
        for layout in (ft.NCHW, ft.NHWC):
            d_x = ctx.to_device(case.x if layout == ft.NCHW else to_nhwc(case.x))
            ctx.quantise_e2m1(d_x, d_t, d_e, N, layer.C, layer.H, layer.W, layout)
            ctx.quantise(True, d_x, d_t, d_p, N, layer.C, layer.H, layer.W, layout)
            ctx.gemm_im2col(w, d_e, d_y, shape, case.alpha, layout, 0, 1)   # single blocks
            ctx.sync()
            planes = ctx.to_host(d_p, (N, 2, layer.H * layer.W, Cp, 2), np.uint32)   # [n][plane][pixel][ic][lo, hi]
            e2m1 = ctx.to_host(d_e, (N, layer.H * layer.W, Cp, 2, 4), np.uint32)     # [n][pixel][ic][lo, hi][4 words]
            assert np.array_equal(e2m1, _expand32_f4_numpy(planes[:, 0], planes[:, 1]))
            got = ctx.to_host(d_y, want.shape if layout == ft.NCHW else (N, layer.OH, layer.OW, layer.KN), np.float32)
            if layout == ft.NHWC:
                got = to_nchw(got)
            assert got.tobytes() == want.tobytes()
            if layer.KN > 128:
                # block pairs (two SMs on one 256-row tile) forced at a size the heuristic would not pick
                ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
                ctx.gemm_im2col(w, d_e, d_y, shape, case.alpha, layout, 0, 2)
                ctx.sync()
                got2 = ctx.to_host(d_y, got.shape if layout == ft.NCHW else (N, layer.OH, layer.OW, layer.KN), np.float32)
                if layout == ft.NHWC:
                    got2 = to_nchw(got2)
                assert got2.tobytes() == want.tobytes()
            else:
                with pytest.raises(ft.TnnsError):
                    ctx.gemm_im2col(w, d_e, d_y, shape, case.alpha, layout, 0, 2)
            ctx.free(d_x)
        # the layer entry point takes this route by itself and gives the same bytes
        y = device_conv(ctx, case, wp, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO)
        assert y.tobytes() == want.tobytes()
    finally:
        for p in (d_t, d_y, d_e, d_p):
            ctx.free(p)
        w.free()


FUSED_LAYERS = [
    (TNN, Layer(256, 14, 14, 256, 3, 3, 1, 1), 4),     # 196 pixels per image: a ragged second band of pixels
    (TNN, Layer(256, 14, 14, 256, 5, 3, 1, 2), 8),     # 5 x 3 kernel, stride 2
    (TBN, Layer(256, 10, 10, 100, 3, 3, 1, 2), 3),     # binary weights, images below one band
    (TNN, Layer(1024, 14, 14, 1024, 5, 5, 1, 2), 2),   # 16 channel groups, four kernel tiles
    (TNN, Layer(250, 10, 12, 64, 3, 3, 2, 3), 3),      # channel tail in the last group, padding 2, stride 3
    (TNN, Layer(64, 12, 12, 200, 3, 3, 1, 1), 5),      # C_pack = 1
    (TBN, Layer(128, 10, 10, 100, 3, 3, 1, 2), 3),     # C_pack = 2
    (TNN, Layer(100, 8, 8, 64, 3, 3, 1, 1), 7),        # C_pack = 2 with a channel tail
    (TNN, Layer(512, 6, 6, 512, 1, 1, 0, 1), 40),      # 36 pixels per image: a tile waits for several images
    (TNN, Layer(256, 16, 16, 320, 3, 3, 1, 1), 80),    # more tiles than SMs: tiles of later images wait while earlier ones multiply
]


@pytest.mark.gpu
@pytest.mark.parametrize("type_,layer,N", FUSED_LAYERS, ids=lambda v: str(v).replace(" ", ""))
def test_fused_quantise_and_tensor_copy_gemm(type_, layer, N, gpu_ctx, checker):
    """One launch for the whole layer: quantiser warps write the 4-bit image while the GEMM's tensor
    copies wait per image.  Output and image equal the two-kernel route and the reference bit for
    bit, with single blocks and block pairs, on two calls in a row (the synchronisation words are
    cleared by every call) and through the layer entry point."""
    ctx = gpu_ctx
    case = make_case(type_, layer, N, 6300 + layer.C + layer.KN, "uniform")
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    nb_e = ft.api.e2m1_image_bytes(N, layer.C, layer.H, layer.W)
    nb_ws = ft.api.fused_workspace_bytes(N, layer.C, layer.H, layer.W)
    assert nb_ws >= nb_e + 4 * N
    d_t = ctx.to_device(case.thr)
    d_x = ctx.to_device(case.x)
    d_y = ctx.malloc(want.nbytes)
    d_e = ctx.malloc(nb_e)
    d_ws = ctx.malloc(nb_ws)
    try:
        assert ctx.conv_fused_supported(w, shape, d_x, ft.NCHW)
        assert not ctx.conv_fused_supported(w, shape, d_x + 4, ft.NCHW)
        ctx.quantise_e2m1(d_x, d_t, d_e, N, layer.C, layer.H, layer.W, ft.NCHW)
        ctx.sync()
        image = ctx.to_host(d_e, (nb_e // 4,), np.uint32)
        for pairs in (1, 2, 0):
            if pairs == 2 and layer.KN <= 128:
                continue
            for rep in range(2):
                ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
                ctx.fill(d_ws, np.full(nb_ws // 4, 0xFFFFFFFF, np.uint32))   # stale image and stale counters
                ctx.conv_fused(w, d_x, d_t, d_y, d_ws, nb_ws, shape, case.alpha, pairs)
                ctx.sync()
                assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes()
                assert np.array_equal(ctx.to_host(d_ws, (nb_e // 4,), np.uint32), image)
        with pytest.raises(ft.TnnsError):
            ctx.conv_fused(w, d_x, d_t, d_y, d_ws, nb_ws - 128, shape, case.alpha)
        # the layer entry point on request
        ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
        ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, ft.NCHW, ft.PACK_AUTO, ft.GEMM_F4_FUSED)
        ctx.sync()
        assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes()
        # pixel-major input and output: the quantiser warps read 128-byte-swizzled boxes of 128 pixels x 32 channels
        # (channel counts that are multiples of four, at least 128 pixels in the batch), twice over stale workspace bytes
        d_xh = ctx.to_device(to_nhwc(case.x))
        nhwc_ok = layer.C % 4 == 0 and N * layer.H * layer.W >= 128
        assert ctx.conv_fused_supported(w, shape, d_xh, ft.NHWC) == nhwc_ok
        if nhwc_ok:
            for rep in range(2):
                ctx.fill(d_y, np.full(want.size, np.nan, np.float32))
                ctx.fill(d_ws, np.full(nb_ws // 4, 0xFFFFFFFF, np.uint32))
                ctx.conv_ws(w, d_xh, d_t, d_y, d_ws, nb_ws, shape, case.alpha, ft.NHWC, ft.PACK_AUTO, ft.GEMM_F4_FUSED)
                ctx.sync()
                got = ctx.to_host(d_y, (N, layer.OH, layer.OW, layer.KN), np.float32)
                assert to_nchw(got).tobytes() == want.tobytes(), ("NHWC one launch", rep)
                assert np.array_equal(ctx.to_host(d_ws, (nb_e // 4,), np.uint32), image)
        else:
            with pytest.raises(ft.TnnsError):
                ctx.conv_ws(w, d_xh, d_t, d_y, d_ws, nb_ws, shape, case.alpha, ft.NHWC, ft.PACK_AUTO, ft.GEMM_F4_FUSED)
        ctx.free(d_xh)
    finally:
        for p in (d_t, d_x, d_y, d_e, d_ws):
            ctx.free(p)
        w.free()


@pytest.mark.gpu
@pytest.mark.parametrize("next_format", [2, 1, 0])
def test_fused_first_layer_of_a_chain(next_format, gpu_ctx, checker):
    """The one-launch kernel with the quantising epilogue: fp32 input in, the next layer's quantised
    activations out -- the same bytes as the quantise kernel followed by the GEMM with that epilogue."""
    ctx = gpu_ctx
    layer, N = Layer(128, 12, 12, 200, 3, 3, 1, 1), 6
    case = make_case(TNN, layer, N, 8100 + next_format, "uniform")
    wp = checker.pack_weights(True, case.w, case.w_thr)
    w = ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    nb_in = ft.api.e2m1_image_bytes(N, layer.C, layer.H, layer.W)
    nb_ws = ft.api.fused_workspace_bytes(N, layer.C, layer.H, layer.W)
    nb_out = max(ft.api.e2m1_image_bytes(N, layer.KN, layer.OH, layer.OW), ft.api.packed_image_bytes(True, N, layer.KN, layer.OH, layer.OW))
    thr_next = np.linspace(0.2, 3.0, N).astype(np.float32)
    d_x, d_t, d_tn = ctx.to_device(case.x), ctx.to_device(case.thr), ctx.to_device(thr_next)
    d_in, d_ws = ctx.malloc(nb_in), ctx.malloc(nb_ws)
    d_o = [ctx.malloc(nb_out) for _ in range(2)]
    try:
        for p in d_o:
            ctx.fill(p, np.zeros(nb_out // 4, np.uint32))
        ctx.quantise_e2m1(d_x, d_t, d_in, N, layer.C, layer.H, layer.W, ft.NCHW)
        ctx.gemm_im2col_packed_out(w, d_in, d_o[0], d_tn, next_format, shape, case.alpha)
        ctx.conv_fused_packed_out(w, d_x, d_t, d_o[1], d_tn, next_format, d_ws, nb_ws, shape, case.alpha)
        ctx.sync()
        a, b = (ctx.to_host(p, (nb_out // 4,), np.uint32) for p in d_o)
        assert a.any() and np.array_equal(a, b)
    finally:
        for p in (d_x, d_t, d_tn, d_in, d_ws, *d_o):
            ctx.free(p)
        w.free()


@pytest.mark.gpu
@pytest.mark.parametrize("type_", [TNN, TBN])
def test_fused_quantiser_on_special_values(type_, gpu_ctx, checker):
    """+-0, values equal to and next to the thresholds, denormals, infinities, thresholds of 0 and -0:
    the quantiser warps inside the GEMM launch decide exactly as the reference does (strict compares,
    src/tnns/ternarize2row_avx2.c:444-449), seen through the layer output."""
    ctx = gpu_ctx
    case = special_value_case(type_)
    layer, N = case.layer, case.N
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    d_x, d_t = ctx.to_device(case.x), ctx.to_device(case.thr)
    d_y = ctx.malloc(want.nbytes)
    try:
        ctx.conv(w, d_x, d_t, d_y, layer.shape(N), case.alpha, ft.NCHW, ft.PACK_AUTO, ft.GEMM_F4_FUSED)
        ctx.sync()
        assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes()
    finally:
        for p in (d_x, d_t, d_y):
            ctx.free(p)
        w.free()


@pytest.mark.gpu
def test_fused_launches_on_two_streams(gpu_ctx, checker):
    """The context's own synchronisation words serve the stream that used the fused form first (they
    are left zeroed by every launch); launches on another stream use the words in the caller's
    workspace, cleared per call.  Both give the reference's bytes, interleaved and back to back."""
    import torch
    ctx = gpu_ctx
    layer = Layer(256, 12, 12, 300, 3, 3, 1, 1)
    N = 9
    case = make_case(TNN, layer, N, 7300, "uniform")
    wp = checker.pack_weights(True, case.w, case.w_thr)
    want = checker.conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    nb_ws = ft.api.fused_workspace_bytes(N, layer.C, layer.H, layer.W)
    d_x, d_t = ctx.to_device(case.x), ctx.to_device(case.thr)
    d_y = [ctx.malloc(want.nbytes) for _ in range(2)]
    d_ws = [ctx.malloc(nb_ws) for _ in range(2)]
    streams = [0, torch.cuda.Stream().cuda_stream]
    try:
        ctx.conv_fused(w, d_x, d_t, d_y[0], d_ws[0], nb_ws, shape, case.alpha, 0, streams[0])   # binds the default stream
        ctx.sync()
        for rep in range(3):
            for k in (0, 1):
                ctx.fill(d_y[k], np.full(want.size, np.nan, np.float32))
                ctx.fill(d_ws[k], np.full(nb_ws // 4, 0xFFFFFFFF, np.uint32))
            for k in (1, 0, 1, 0):
                ctx.conv_fused(w, d_x, d_t, d_y[k], d_ws[k], nb_ws, shape, case.alpha, 1 + (rep % 2), streams[k])
            ctx.sync()
            for k in (0, 1):
                assert ctx.to_host(d_y[k], want.shape, np.float32).tobytes() == want.tobytes()
    finally:
        for p in (d_x, d_t, *d_y, *d_ws):
            ctx.free(p)
        w.free()


@pytest.mark.gpu
def test_fused_route_declines_what_it_cannot_do(gpu_ctx, checker):
    """Pixel counts that are not a multiple of four (the rows of an NCHW input tensor must be 16-byte
    multiples for the copy engine) stay on the two-kernel route; asking for the fused one is an error."""
    ctx = gpu_ctx
    layer = Layer(256, 7, 7, 64, 3, 3, 1, 1)
    case = make_case(TNN, layer, 3, 91, "uniform")
    wp = checker.pack_weights(True, case.w, case.w_thr)
    want = checker.conv(TNN, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    w = ctx.upload_weights(TNN, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(3)
    d_x, d_t = ctx.to_device(case.x), ctx.to_device(case.thr)
    d_y = ctx.malloc(want.nbytes)
    try:
        assert ctx.im2col_supported(w, shape) and not ctx.conv_fused_supported(w, shape, d_x, ft.NCHW)
        with pytest.raises(ft.TnnsError):
            ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, ft.NCHW, ft.PACK_AUTO, ft.GEMM_F4_FUSED)
        ctx.conv(w, d_x, d_t, d_y, shape, case.alpha, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO)
        ctx.sync()
        assert ctx.to_host(d_y, want.shape, np.float32).tobytes() == want.tobytes()
    finally:
        for p in (d_x, d_t, d_y):
            ctx.free(p)
        w.free()


@pytest.mark.gpu
def test_im2col_route_declines_what_it_cannot_do(gpu_ctx, checker):
    """Binary activations (padding is +1, which a zero-filling copy cannot produce) and channel counts
    whose pixels are neither 32, 64 nor a multiple of 128 bytes stay on the gathering GEMM; asking for
    the route anyway is an error."""
    ctx = gpu_ctx
    for type_, layer in ((BTN, Layer(256, 8, 8, 64, 3, 3, 1, 1)), (TNN, Layer(192, 8, 8, 64, 3, 3, 1, 1))):
        case = make_case(type_, layer, 2, 77, "uniform")
        wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
        w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
        shape = layer.shape(2)
        assert not ctx.im2col_supported(w, shape)
        d = ctx.malloc(1 << 20)
        with pytest.raises(ft.TnnsError):
            ctx.gemm_im2col(w, d, d, shape, 0.5)
        ctx.free(d)
        want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
        assert device_conv(ctx, case, wp, ft.NCHW, ft.PACK_AUTO, ft.GEMM_AUTO).tobytes() == want.tobytes()
        w.free()


@pytest.mark.gpu
@pytest.mark.parametrize("alpha", [0.0, 1.0, 0.3, -0.25, 2.5])
def test_prelu_slopes_other_than_one_half(alpha, gpu_ctx, checker):
    """PReLU is acc > 0 ? acc : acc*alpha in fp32 (include/tnns/mm.h:60-66 of the reference).  Every GEMM
    kernel must give the reference's bits for any slope, including the sign of zero (alpha = 0 turns
    negative sums into -0, a negative alpha turns zero sums into -0).  Sparse activations (threshold
    0.9) make zero sums common."""
    ctx = gpu_ctx
    for type_, layer in ((TNN, Layer(256, 6, 6, 40, 3, 3, 1, 1)), (TBN, Layer(64, 6, 6, 72, 3, 3, 1, 1)), (BNN, Layer(70, 5, 5, 33, 2, 2, 1, 1))):
        case = make_case(type_, layer, 3, 1234, "uniform")
        case.thr[:] = 0.9 if act_ternary(type_) else 0.0
        wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
        want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, alpha)
        assert (want == 0).any()
        case.alpha = alpha
        for galgo in (ft.GEMM_AUTO, ft.GEMM_I8_TC, ft.GEMM_F4_TC, ft.GEMM_POPC_TILED, ft.GEMM_POPC_SIMPLE):
            got = device_conv(ctx, case, wp, ft.NCHW, ft.PACK_AUTO, galgo)
            bad = np.flatnonzero(got.view(np.uint32).ravel() != want.view(np.uint32).ravel())
            assert bad.size == 0, (type_, alpha, galgo, bad.size, got.ravel()[bad[:3]], want.ravel()[bad[:3]])


@pytest.mark.gpu
@pytest.mark.parametrize("type_", [TNN, BNN])
@pytest.mark.parametrize("alpha", [0.5, 0.3, 1.0, 0.07, -0.25, 1.5])
def test_quantising_epilogue_for_any_slope(type_, alpha, gpu_ctx, checker):
    """The chaining epilogues decide the next layer's activations from the raw accumulator by thresholds when
    0 < alpha <= 1 and by evaluating the PReLU otherwise.  Either way the bits must be those the quantise
    kernels make of the layer's fp32 output: thresholds of 0, small, integer-valued, large and negative, all
    three output formats, on the im2col-fed and the slab-fed GEMM (BNN: accumulator offset; its binary input
    takes the slab-fed GEMM only)."""
    ctx = gpu_ctx
    layer, N = Layer(256, 10, 10, 256, 3, 3, 1, 1), 7
    tern_in = act_ternary(type_)
    case = make_case(type_, layer, N, 9800 + type_, "uniform")
    wp = checker.pack_weights(wgt_ternary(type_), case.w, case.w_thr)
    want = checker.conv(type_, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, alpha)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(N)
    thr_next = np.array([0.0, 0.4, 3.0, 17.5, 250.0, -0.2, 1.0], np.float32)
    nb_b = ft.api.bordered_image_bytes(N, layer.C, layer.H, layer.W, 1, 1)
    nb_e = ft.api.e2m1_image_bytes(N, layer.C, layer.H, layer.W)
    nb_o = max(ft.api.e2m1_image_bytes(N, layer.KN, layer.OH, layer.OW), ft.api.packed_image_bytes(True, N, layer.KN, layer.OH, layer.OW))
    d_x, d_t, d_tn = ctx.to_device(case.x), ctx.to_device(case.thr), ctx.to_device(thr_next)
    d_f = ctx.to_device(want)
    d_b, d_e, d_o, d_q = ctx.malloc(nb_b), ctx.malloc(nb_e), ctx.malloc(nb_o), ctx.malloc(nb_o)
    try:
        ctx.quantise_e2m1_bordered(tern_in, d_x, d_t, d_b, N, layer.C, layer.H, layer.W, 1, 1)
        if tern_in:
            ctx.quantise_e2m1(d_x, d_t, d_e, N, layer.C, layer.H, layer.W)
        for fmt in (2, 1, 0):
            # what the quantise kernels make of the checker's fp32 output
            ctx.fill(d_q, np.zeros(nb_o // 4, np.uint32))
            if fmt == 2:
                ctx.quantise_e2m1(d_f, d_tn, d_q, N, layer.KN, layer.OH, layer.OW)
            else:
                ctx.quantise(fmt == 1, d_f, d_tn, d_q, N, layer.KN, layer.OH, layer.OW)
            ctx.sync()
            expect = ctx.to_host(d_q, (nb_o // 4,), np.uint32)
            producers = [("slab", lambda: ctx.gemm_slab_packed_out(w, d_b, d_o, d_tn, fmt, (0, 0), shape, alpha))]
            if tern_in:
                producers.append(("im2col", lambda: ctx.gemm_im2col_packed_out(w, d_e, d_o, d_tn, fmt, shape, alpha)))
            for name, run in producers:
                ctx.fill(d_o, np.zeros(nb_o // 4, np.uint32))
                run()
                ctx.sync()
                assert np.array_equal(ctx.to_host(d_o, (nb_o // 4,), np.uint32), expect), (name, fmt, alpha)
    finally:
        for p in (d_x, d_t, d_tn, d_f, d_b, d_e, d_o, d_q):
            ctx.free(p)
        w.free()
