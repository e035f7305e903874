"""Python host side of libtnns_b200: the reference's operator interface over numpy arrays
(host pointers, same argument meaning and ownership as include/tnns/tnns_cpu.h,
include/tnns/mm.h, include/tnns/ternarize2row.h, include/tnns/binarize2row.h of the
reference) and the device-resident API over raw device pointers.

Every function here ends in a call into the shared library; none computes anything on
the CPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import GemmTestcase, Shape, Testcase, load_library

TNN, TBN, BTN, BNN = 0, 1, 2, 3
NCHW, NHWC = 0, 1
PACK_AUTO, PACK_GATHER, PACK_STAGED = 0, 1, 2
GEMM_AUTO, GEMM_POPC_SIMPLE, GEMM_POPC_TILED, GEMM_I8_TC, GEMM_F4_TC, GEMM_F4_FUSED, GEMM_F4_SLAB, GEMM_F4_SLAB_FUSED, GEMM_F4_DENSE = 0, 1, 2, 3, 4, 5, 6, 7, 8


class TnnsError(RuntimeError):
    def __init__(self, status: int, detail: str):
        super().__init__(f"tnns_b200 error {status}: {detail}")
        self.status = status
        self.detail = detail


def _check(rc: int):
    if rc != 0:
        lib = load_library()
        raise TnnsError(rc, f"{lib.tnns_cuda_strerror(rc).decode()}: {lib.tnns_cuda_error_detail().decode()}")


def _last_error() -> TnnsError:
    lib = load_library()
    rc = lib.tnns_cuda_last_error()
    return TnnsError(rc, f"{lib.tnns_cuda_strerror(rc).decode()}: {lib.tnns_cuda_error_detail().decode()}")


def out_dim(size: int, pad: int, k: int, stride: int) -> int:
    return load_library().tnns_out_dim(size, pad, k, stride)


def k_words(C_: int, KH: int, KW: int) -> int:
    return load_library().tnns_k_words(C_, KH, KW)


def k_padded(C_: int, KH: int, KW: int) -> int:
    return load_library().tnns_k_padded(C_, KH, KW)


def packed_bytes(type_: int, shape: Shape) -> int:
    return load_library().tnns_packed_bytes(type_, C.byref(shape))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int64)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _take_floats(ptr: int, count: int) -> np.ndarray:
    """Copy a malloc'd float buffer returned by the library into numpy and free it."""
    lib = load_library()
    out = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(count,)).copy()
    lib.libc_free(ptr)
    return out


def _take_words(ptr: int, count: int) -> np.ndarray:
    lib = load_library()
    out = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_int64)), shape=(count,)).copy()
    lib.libc_free(ptr)
    return out


# --------------------------------------------------------------------------------------------
# Drop-in interface (host arrays)
# --------------------------------------------------------------------------------------------

def pack_weights_ternary(w, thresholds) -> np.ndarray:
    """fp32 [KN][C][KH][KW] -> packing-2 rows (reference: ternarize_opt_avx2, src/utils.c:468)."""
    w = _f32(w)
    KN, C_, KH, KW = w.shape
    thr = _f32(thresholds)
    assert thr.shape == (KN,)
    p = load_library().tnns_pack_weights_ternary(_ptr(w), _ptr(thr), KN, C_, KH, KW)
    if not p:
        raise MemoryError("tnns_pack_weights_ternary")
    return _take_words(p, KN * 2 * k_padded(C_, KH, KW)).reshape(KN, -1)


def pack_weights_binary(w, thresholds) -> np.ndarray:
    """fp32 [KN][C][KH][KW] -> one-plane rows (reference: binarize_opt_avx2, src/utils.c:672)."""
    w = _f32(w)
    KN, C_, KH, KW = w.shape
    thr = _f32(thresholds)
    assert thr.shape == (KN,)
    p = load_library().tnns_pack_weights_binary(_ptr(w), _ptr(thr), KN, C_, KH, KW)
    if not p:
        raise MemoryError("tnns_pack_weights_binary")
    return _take_words(p, KN * k_padded(C_, KH, KW)).reshape(KN, -1)


def tnns_conv(type_: int, x, thresholds, packed_kernel, kernel_hw, padding=(0, 0), stride=(1, 1), alpha=0.5) -> np.ndarray:
    """One layer through the drop-in ``tnns_conv(testcase_t*)``.

    x: fp32 NCHW; thresholds: one per image; packed_kernel: KN rows in the layout the type
    expects.  Returns fp32 NCHW [N][KN][OH][OW].
    """
    lib = load_library()
    x = _f32(x)
    N, C_, H, W = x.shape
    thr = _f32(thresholds)
    pk = _i64(packed_kernel)
    KN = pk.shape[0]
    KH, KW = kernel_hw
    t = Testcase()
    t.type = type_
    t.batchcount, t.channelcount, t.inputH, t.inputW = N, C_, H, W
    t.kernelcount, t.kernelH, t.kernelW = KN, KH, KW
    t.paddingH, t.paddingW = padding
    t.strideH, t.strideW = stride
    t.preluAlpha = alpha
    t.input_thresholds = thr.ctypes.data_as(C.POINTER(C.c_float))
    t.input = x.ctypes.data_as(C.POINTER(C.c_float))
    t.quantized_kernel_packing2 = pk.ctypes.data_as(C.POINTER(C.c_int64))
    lib.tnns_conv(C.byref(t))
    if not t.output:
        raise _last_error()
    OH = out_dim(H, padding[0], KH, stride[0])
    OW = out_dim(W, padding[1], KW, stride[1])
    return _take_floats(C.cast(t.output, C.c_void_p).value, N * KN * OH * OW).reshape(N, KN, OH, OW)


def tnns_gemm(x_packing2, w_packing2, m: int, n: int, p_packed: int, out: np.ndarray | None = None) -> np.ndarray:
    """Packed TNN GEMM with alpha = 1 through ``tnns_gemm(testcase_tnns_gemm_t*)``."""
    lib = load_library()
    xa, wa = _i64(x_packing2), _i64(w_packing2)
    t = GemmTestcase()
    t.m, t.n, t.p_packed, t.p = m, n, p_packed, p_packed * 64
    t.x_packing2 = xa.ctypes.data_as(C.POINTER(C.c_int64))
    t.w_packing2 = wa.ctypes.data_as(C.POINTER(C.c_int64))
    if out is not None:
        assert out.dtype == np.float32 and out.flags.c_contiguous and out.size == m * n
        t.output = out.ctypes.data_as(C.POINTER(C.c_float))
        lib.tnns_gemm(C.byref(t))
        return out
    lib.tnns_gemm(C.byref(t))
    if not t.output:
        raise _last_error()
    return _take_floats(C.cast(t.output, C.c_void_p).value, m * n).reshape(m, n)


def _mm(name, a, b, N, OH, OW, KN, K, alpha, K_unpack=None):
    lib = load_library()
    a, b = _i64(a), _i64(b)
    fn = getattr(lib, name)
    p = fn(_ptr(a), _ptr(b), N, OH, OW, KN, K, alpha) if K_unpack is None else fn(_ptr(a), _ptr(b), N, OH, OW, KN, K, K_unpack, alpha)
    if not p:
        raise _last_error()
    return _take_floats(p, N * KN * OH * OW).reshape(N, KN, OH, OW)


def mm_tnn(a, b, N, OH, OW, KN, K, alpha):
    return _mm("mm_tnn", a, b, N, OH, OW, KN, K, alpha)


def mm_tbn(a, b, N, OH, OW, KN, K, alpha):
    return _mm("mm_tbn", a, b, N, OH, OW, KN, K, alpha)


def mm_btn(a, b, N, OH, OW, KN, K, alpha):
    return _mm("mm_btn", a, b, N, OH, OW, KN, K, alpha)


def mm_bnn(a, b, N, OH, OW, KN, K, K_unpack, alpha):
    return _mm("mm_bnn", a, b, N, OH, OW, KN, K, alpha, K_unpack=K_unpack)


def _pack_host(name, planes, x, thresholds, kernel_hw, padding, stride):
    lib = load_library()
    x = _f32(x)
    N, C_, H, W = x.shape
    thr = _f32(thresholds)
    KH, KW = kernel_hw
    p = getattr(lib, name)(_ptr(x), _ptr(thr), N, C_, H, W, padding[0], padding[1], KH, KW, stride[0], stride[1])
    if not p:
        raise _last_error()
    rows = N * out_dim(H, padding[0], KH, stride[0]) * out_dim(W, padding[1], KW, stride[1])
    return _take_words(p, rows * planes * k_padded(C_, KH, KW)).reshape(rows, -1)


def t2r_p2_opt(x, thresholds, kernel_hw, padding=(0, 0), stride=(1, 1)) -> np.ndarray:
    """Ternarize + pack + im2row of a host NCHW tensor; rows of 2*Kp int64 (packing-2)."""
    return _pack_host("t2r_p2_opt", 2, x, thresholds, kernel_hw, padding, stride)


def b2r(x, thresholds, kernel_hw, padding=(0, 0), stride=(1, 1)) -> np.ndarray:
    """Binarize + pack + im2row of a host NCHW tensor; rows of Kp int64 (one plane)."""
    return _pack_host("b2r", 1, x, thresholds, kernel_hw, padding, stride)


# --------------------------------------------------------------------------------------------
# Device-resident interface (raw device pointers; torch supplies memory and streams)
# --------------------------------------------------------------------------------------------

class Weights:
    """Device copy of one layer's packed kernel."""

    def __init__(self, ctx: "Context", handle: int, type_: int, KN: int):
        self.ctx, self.handle, self.type, self.KN = ctx, handle, type_, KN

    def free(self):
        if self.handle:
            load_library().tnns_cuda_free_weights(self.ctx.handle, self.handle)
            self.handle = None


class Context:
    """One ``tnns_cuda_ctx`` (per host thread and device)."""

    def __init__(self, device: int = 0):
        lib = load_library()
        h = C.c_void_p()
        _check(lib.tnns_cuda_create(device, C.byref(h)))
        self.handle = h.value
        self.device = device
        self.lib = lib

    def close(self):
        if self.handle:
            self.lib.tnns_cuda_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- weights
    def upload_weights(self, type_: int, packed: np.ndarray, C_: int, KH: int, KW: int) -> Weights:
        pk = _i64(packed)
        KN = pk.shape[0]
        h = C.c_void_p()
        _check(self.lib.tnns_cuda_upload_weights(self.handle, type_, _ptr(pk), KN, C_, KH, KW, C.byref(h)))
        return Weights(self, h.value, type_, KN)

    def upload_weights_packed(self, type_: int, packed: np.ndarray, K_words: int, K_unpack: int = 0) -> Weights:
        pk = _i64(packed)
        KN = pk.shape[0]
        h = C.c_void_p()
        _check(self.lib.tnns_cuda_upload_weights_packed(self.handle, type_, _ptr(pk), KN, K_words, K_unpack, C.byref(h)))
        return Weights(self, h.value, type_, KN)

    def pack_weights_device(self, ternary: bool, d_w: int, d_thr: int, d_packed: int, KN: int, C_: int, KH: int, KW: int, stream=0):
        """fp32 weights on the device -> packed rows on the device (same bytes as the host packers)."""
        _check(self.lib.tnns_cuda_pack_weights(self.handle, int(ternary), d_w, d_thr, d_packed, KN, C_, KH, KW, stream))

    # -- kernels on device pointers
    def pack(self, ternary: bool, d_x: int, d_thr: int, d_packed: int, shape: Shape, layout=NCHW, algo=PACK_AUTO, stream=0):
        _check(self.lib.tnns_cuda_pack(self.handle, int(ternary), d_x, d_thr, d_packed, C.byref(shape), layout, algo, stream))

    def gemm(self, w: Weights, d_a: int, d_y: int, N: int, OH: int, OW: int, alpha: float, layout=NCHW, algo=GEMM_AUTO, stream=0):
        _check(self.lib.tnns_cuda_gemm(self.handle, w.handle, d_a, d_y, N, OH, OW, alpha, layout, algo, stream))

    def conv(self, w: Weights, d_x: int, d_thr: int, d_y: int, shape: Shape, alpha: float, layout=NCHW, pack_algo=PACK_AUTO,
             gemm_algo=GEMM_AUTO, stream=0):
        _check(self.lib.tnns_cuda_conv(self.handle, w.handle, d_x, d_thr, d_y, C.byref(shape), alpha, layout, pack_algo,
                                       gemm_algo, stream))

    def conv_ws(self, w: Weights, d_x: int, d_thr: int, d_y: int, d_ws: int, ws_bytes: int, shape: Shape, alpha: float,
                layout=NCHW, pack_algo=PACK_AUTO, gemm_algo=GEMM_AUTO, stream=0):
        _check(self.lib.tnns_cuda_conv_ws(self.handle, w.handle, d_x, d_thr, d_y, d_ws, ws_bytes, C.byref(shape), alpha, layout,
                                          pack_algo, gemm_algo, stream))

    def quantise(self, ternary: bool, d_x: int, d_thr: int, d_image: int, N: int, C_: int, H: int, W: int, layout=NCHW, stream=0):
        """fp32 tensor -> packed image (bit planes [n][plane][pixel][ic])."""
        _check(self.lib.tnns_cuda_quantise(self.handle, int(ternary), d_x, d_thr, d_image, N, C_, H, W, layout, stream))

    def gemm_implicit(self, w: Weights, d_image: int, d_y: int, shape: Shape, alpha: float, layout=NCHW, stream=0):
        """GEMM + PReLU gathering its im2row rows from the packed image of the layer input."""
        _check(self.lib.tnns_cuda_gemm_implicit(self.handle, w.handle, d_image, d_y, C.byref(shape), alpha, layout, stream))

    def quantise_e2m1(self, d_x: int, d_thr: int, d_image: int, N: int, C_: int, H: int, W: int, layout=NCHW, stream=0):
        """fp32 tensor -> 4-bit operand image ([n][pixel][C/2 bytes], ternary activations)."""
        _check(self.lib.tnns_cuda_quantise_e2m1(self.handle, d_x, d_thr, d_image, N, C_, H, W, layout, stream))

    def gemm_im2col(self, w: Weights, d_image: int, d_y: int, shape: Shape, alpha: float, layout=NCHW, stream=0, pairs=0):
        """GEMM + PReLU whose activation tiles the copy engine gathers from the 4-bit image.
        pairs: 0 = by size, 1 = single blocks, 2 = block pairs (tcgen05.mma.cta_group::2)."""
        _check(self.lib.tnns_cuda_gemm_im2col(self.handle, w.handle, d_image, d_y, C.byref(shape), alpha, layout, pairs, stream))

    def conv_fused_supported(self, w: Weights, shape: Shape, d_x: int, layout=NCHW) -> bool:
        return bool(self.lib.tnns_cuda_conv_fused_supported(w.handle, C.byref(shape), d_x, layout))

    def conv_fused_preferred(self, w: Weights, shape: Shape, d_x: int, layout=NCHW) -> bool:
        """Whether conv() with GEMM_AUTO takes the one-launch route for this layer by itself."""
        return bool(self.lib.tnns_cuda_conv_fused_preferred(self.handle, w.handle, C.byref(shape), d_x, layout))

    def conv_fused_packed_out(self, w: Weights, d_x: int, d_thr: int, d_image_out: int, d_thr_next: int, next_format: int, d_ws: int,
                              ws_bytes: int, shape: Shape, alpha: float, pairs=0, stream=0):
        """conv_fused whose epilogue writes the next layer's quantised activations instead of fp32."""
        _check(self.lib.tnns_cuda_conv_fused_packed_out(self.handle, w.handle, d_x, d_thr, d_image_out, d_thr_next, next_format, d_ws,
                                                        ws_bytes, C.byref(shape), alpha, pairs, stream))

    def conv_fused(self, w: Weights, d_x: int, d_thr: int, d_y: int, d_ws: int, ws_bytes: int, shape: Shape, alpha: float,
                   pairs=0, stream=0):
        """Whole layer in ONE launch: quantiser warps beside the tensor-copy fed GEMM (NCHW input).
        d_ws: fused_workspace_bytes() bytes, 128-byte aligned."""
        _check(self.lib.tnns_cuda_conv_fused(self.handle, w.handle, d_x, d_thr, d_y, d_ws, ws_bytes, C.byref(shape), alpha, pairs,
                                             stream))

    def gemm_im2col_packed_out(self, w: Weights, d_image: int, d_image_out: int, d_thr_next: int, next_format: int, shape: Shape,
                               alpha: float, stream=0, pairs=0):
        """The copy-engine GEMM with the quantising epilogue: writes the next layer's activations as binary (0) or
        ternary (1) bit planes or as a ternary 4-bit operand image (2) instead of fp32."""
        _check(self.lib.tnns_cuda_gemm_im2col_packed_out(self.handle, w.handle, d_image, d_image_out, d_thr_next, next_format,
                                                         C.byref(shape), alpha, pairs, stream))

    def gemm_im2col_bordered_out(self, w: Weights, d_image: int, d_image_out: int, d_thr_next: int, next_pad, shape: Shape, alpha: float,
                                 stream=0, pairs=0):
        """The copy-engine GEMM writing the next layer's 4-bit image bordered by next_pad = (PH, PW): what a slab-fed layer reads."""
        _check(self.lib.tnns_cuda_gemm_im2col_bordered_out(self.handle, w.handle, d_image, d_image_out, d_thr_next, next_pad[0], next_pad[1],
                                                           C.byref(shape), alpha, pairs, stream))

    # -- stride-1 layers from a bordered 4-bit image (slab-fed GEMM)
    def slab_supported(self, w: Weights, shape: Shape) -> bool:
        return bool(self.lib.tnns_cuda_slab_supported(self.handle, w.handle, C.byref(shape)))

    def slab_preferred(self, w: Weights, shape: Shape) -> bool:
        """Whether the library's own rule takes the slab-fed route for this layer."""
        return bool(self.lib.tnns_cuda_slab_preferred(self.handle, w.handle, C.byref(shape)))

    def conv_auto_algo(self, w: Weights, shape: Shape, d_x: int, layout=NCHW) -> int:
        """The GEMM_* value conv() with GEMM_AUTO resolves to for this layer and input."""
        return int(self.lib.tnns_cuda_conv_auto_algo(self.handle, w.handle, C.byref(shape), d_x, layout))

    def slab_auto(self, w: Weights, shape: Shape, d_x: int, layout=NCHW) -> int:
        """0: conv() with GEMM_AUTO does not take the slab-fed route; 1: it does, as two launches; 2: as one launch."""
        return {GEMM_F4_SLAB: 1, GEMM_F4_SLAB_FUSED: 2}.get(self.conv_auto_algo(w, shape, d_x, layout), 0)

    def conv_slab_one_launch_preferred(self, w: Weights, shape: Shape, d_x: int, layout=NCHW) -> bool:
        return bool(self.lib.tnns_cuda_conv_slab_one_launch_preferred(self.handle, w.handle, C.byref(shape), d_x, layout))

    def conv_slab_supported(self, w: Weights, shape: Shape, d_x: int, layout=NCHW) -> bool:
        return bool(self.lib.tnns_cuda_conv_slab_supported(self.handle, w.handle, C.byref(shape), d_x, layout))

    def quantise_e2m1_bordered(self, ternary: bool, d_x: int, d_thr: int, d_image: int, N: int, C_: int, H: int, W: int, PH: int, PW: int,
                               layout=NCHW, stream=0):
        """fp32 NCHW tensor -> 4-bit operand image with the layer's padding stored around every image."""
        _check(self.lib.tnns_cuda_quantise_e2m1_bordered(self.handle, int(ternary), d_x, d_thr, d_image, N, C_, H, W, PH, PW, layout, stream))

    def gemm_slab(self, w: Weights, d_image: int, d_y: int, shape: Shape, alpha: float, layout=NCHW, stream=0, pairs=0):
        """GEMM + PReLU from a bordered 4-bit image: one slab of pixels per tile serves every filter tap."""
        _check(self.lib.tnns_cuda_gemm_slab(self.handle, w.handle, d_image, d_y, C.byref(shape), alpha, layout, pairs, stream))

    def gemm_slab_packed_out(self, w: Weights, d_image: int, d_image_out: int, d_thr_next: int, next_format: int, next_pad, shape: Shape,
                             alpha: float, stream=0, pairs=0):
        """next_format: 0 / 1 bit planes (binary / ternary), 2 plain 4-bit image, 3 / 5 bordered 4-bit image for a
        ternary / binary next layer with padding next_pad = (PH, PW)."""
        _check(self.lib.tnns_cuda_gemm_slab_packed_out(self.handle, w.handle, d_image, d_image_out, d_thr_next, next_format, next_pad[0],
                                                       next_pad[1], C.byref(shape), alpha, pairs, stream))

    def conv_slab(self, w: Weights, d_x: int, d_thr: int, d_y: int, d_ws: int, ws_bytes: int, shape: Shape, alpha: float, pairs=0, stream=0):
        """Whole stride-1 layer in ONE launch: quantiser warps write the bordered image beside the slab-fed GEMM."""
        _check(self.lib.tnns_cuda_conv_slab(self.handle, w.handle, d_x, d_thr, d_y, d_ws, ws_bytes, C.byref(shape), alpha, pairs, stream))

    def conv_slab_packed_out(self, w: Weights, d_x: int, d_thr: int, d_image_out: int, d_thr_next: int, next_format: int, next_pad, d_ws: int,
                             ws_bytes: int, shape: Shape, alpha: float, pairs=0, stream=0):
        _check(self.lib.tnns_cuda_conv_slab_packed_out(self.handle, w.handle, d_x, d_thr, d_image_out, d_thr_next, next_format, next_pad[0],
                                                       next_pad[1], d_ws, ws_bytes, C.byref(shape), alpha, pairs, stream))

    # -- layers with few input channels as a dense 1x1 layer over the real positions of every window
    def dense_supported(self, w: Weights, shape: Shape) -> bool:
        return bool(self.lib.tnns_cuda_dense_supported(self.handle, w.handle, C.byref(shape)))

    def conv_dense(self, w: Weights, d_x: int, d_thr: int, d_y: int, d_ws: int, ws_bytes: int, shape: Shape, alpha: float, layout=NCHW, stream=0):
        """Whole layer with at most 16 input channels: quantise straight into the virtual layer's 4-bit image, then the GEMM."""
        _check(self.lib.tnns_cuda_conv_dense(self.handle, w.handle, d_x, d_thr, d_y, d_ws, ws_bytes, C.byref(shape), alpha, layout, stream))

    def conv_dense_packed_out(self, w: Weights, d_x: int, d_thr: int, d_image_out: int, d_thr_next: int, next_format: int, d_ws: int,
                              ws_bytes: int, shape: Shape, alpha: float, layout=NCHW, stream=0, next_pad=(0, 0)):
        """next_format 0 / 1 bit planes, 2 plain 4-bit image, 3 the 4-bit image bordered by next_pad = (PH, PW)."""
        _check(self.lib.tnns_cuda_conv_dense_packed_out(self.handle, w.handle, d_x, d_thr, d_image_out, d_thr_next, next_format, next_pad[0],
                                                        next_pad[1], d_ws, ws_bytes, C.byref(shape), alpha, layout, stream))

    def im2col_supported(self, w: Weights, shape: Shape) -> bool:
        return bool(self.lib.tnns_cuda_im2col_supported(w.handle, C.byref(shape)))

    def gemm_packed_out(self, w: Weights, d_a: int, d_image: int, d_thr_next: int, next_ternary: bool, N: int, OH: int, OW: int,
                        alpha: float, stream=0):
        """GEMM + PReLU whose epilogue writes the next layer's quantised bit planes instead of fp32."""
        _check(self.lib.tnns_cuda_gemm_packed_out(self.handle, w.handle, d_a, d_image, d_thr_next, int(next_ternary), N, OH, OW,
                                                  alpha, stream))

    def im2row_packed(self, ternary: bool, d_image: int, d_packed: int, shape: Shape, stream=0):
        """Packed image (bit planes) -> im2row matrix of the next layer."""
        _check(self.lib.tnns_cuda_im2row_packed(self.handle, int(ternary), d_image, d_packed, C.byref(shape), stream))

    def conv_host(self, w: Weights, h_x: int, h_thr: int, h_y: int, shape: Shape, alpha: float, layout=NCHW):
        """Host-pointer layer (addresses of pinned or pageable buffers)."""
        _check(self.lib.tnns_cuda_conv_host(self.handle, w.handle, h_x, h_thr, h_y, C.byref(shape), alpha, layout))

    def pipe_rate(self, op: int) -> float:
        """Issue rate of LOP3 (0), POPC (1) or IADD (2) in 1e9 thread-instructions per second, or of an
        issue-bound tcgen05.mma loop, kind::i8 (3) or kind::mxf4 (4), in 1e9 operations (2*M*N*K) per second."""
        v = C.c_double()
        _check(self.lib.tnns_cuda_pipe_rate(self.handle, op, C.byref(v)))
        return v.value

    def sync(self):
        _check(self.lib.tnns_cuda_sync(self.handle))

    # -- memory helpers (so tests need nothing but numpy)
    def malloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        _check(self.lib.tnns_cuda_malloc(self.handle, nbytes, C.byref(p)))
        return p.value

    def free(self, p: int):
        self.lib.tnns_cuda_free(self.handle, p)

    def mem_info(self) -> tuple[int, int]:
        """(free, total) bytes of device memory on this context's device."""
        f, t = C.c_size_t(), C.c_size_t()
        _check(self.lib.tnns_cuda_mem_info(self.handle, C.byref(f), C.byref(t)))
        return f.value, t.value

    def malloc_host(self, nbytes: int) -> int:
        """Page-locked host memory (tnns_cuda_conv_host moves it at full PCIe speed)."""
        p = C.c_void_p()
        _check(self.lib.tnns_cuda_malloc_host(self.handle, nbytes, C.byref(p)))
        return p.value

    def free_host(self, p: int):
        self.lib.tnns_cuda_free_host(self.handle, p)

    def to_device(self, a: np.ndarray) -> int:
        a = np.ascontiguousarray(a)
        p = self.malloc(max(a.nbytes, 16))
        _check(self.lib.tnns_cuda_memcpy_h2d(self.handle, p, _ptr(a), a.nbytes))
        return p

    def fill(self, p: int, a: np.ndarray):
        """Overwrite an existing device buffer with a host array."""
        a = np.ascontiguousarray(a)
        _check(self.lib.tnns_cuda_memcpy_h2d(self.handle, p, _ptr(a), a.nbytes))

    def to_host(self, p: int, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        _check(self.lib.tnns_cuda_memcpy_d2h(self.handle, _ptr(out), p, out.nbytes))
        return out


def shard_range(N: int, shard: int, shards: int) -> tuple[int, int]:
    """[n0, n1) of the images shard `shard` of `shards` owns (``tnns_shard_range``)."""
    a, b = C.c_int(), C.c_int()
    load_library().tnns_shard_range(N, shard, shards, C.byref(a), C.byref(b))
    return a.value, b.value


def shard_run(shards: int, N: int, fn) -> tuple[int, list[int]]:
    """``tnns_shard_run``: fn(shard, shards, n0, n1) -> status on one host thread per shard behind a
    start barrier.  Returns (overall status, status of every shard); never raises for a failed shard."""
    from ._lib import SHARD_FN
    cb = SHARD_FN(lambda g, G, n0, n1, _arg: int(fn(g, G, n0, n1)))
    st = (C.c_int * shards)()
    rc = load_library().tnns_shard_run(shards, N, cb, None, st)
    return rc, list(st)


class MultiWeights:
    def __init__(self, group: "MultiContext", handle: int):
        self.group, self.handle = group, handle

    def free(self):
        if self.handle:
            load_library().tnns_cuda_multi_free_weights(self.group.handle, self.handle)
            self.handle = None


class MultiContext:
    """A group of devices behind one call (``tnns_cuda_multi``): one host batch in, split by image
    index over the devices, one host thread per device, weights replicated, no exchange between devices."""

    def __init__(self, devices):
        lib = load_library()
        devs = (C.c_int * len(devices))(*devices)
        h = C.c_void_p()
        _check(lib.tnns_cuda_multi_create(devs, len(devices), C.byref(h)))
        self.handle, self.devices, self.lib = h.value, list(devices), lib
        self.shard_status: list[int] = []

    def close(self):
        if self.handle:
            self.lib.tnns_cuda_multi_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def upload_weights(self, type_: int, packed: np.ndarray, C_: int, KH: int, KW: int) -> MultiWeights:
        pk = _i64(packed)
        h = C.c_void_p()
        _check(self.lib.tnns_cuda_multi_upload_weights(self.handle, type_, _ptr(pk), pk.shape[0], C_, KH, KW, C.byref(h)))
        return MultiWeights(self, h.value)

    def conv_host(self, w: MultiWeights, h_x: int, h_thr: int, h_y: int, shape: Shape, alpha: float, layout=NCHW):
        """Host-pointer layer over all devices of the group; shard statuses are kept in ``shard_status``."""
        st = (C.c_int * len(self.devices))()
        rc = self.lib.tnns_cuda_multi_conv_host(self.handle, w.handle, h_x, h_thr, h_y, C.byref(shape), alpha, layout, st)
        self.shard_status = list(st)
        _check(rc)


def prelu_thresholds(t: float, alpha: float, bias: float = 0.0, ternary: bool = True) -> tuple[float, float]:
    """The constants (n1, t2) of the quantising epilogues' threshold rule (tnns_prelu_thresholds): for an integer
    accumulator v, sign = v + n1 < 0 and above = t2 - v < 0 reproduce PReLU(v + bias) followed by the next layer's
    quantiser with threshold t.  Host code; needs no GPU."""
    n1, t2 = C.c_float(), C.c_float()
    _check(load_library().tnns_prelu_thresholds(t, alpha, bias, int(ternary), C.byref(n1), C.byref(t2)))
    return n1.value, t2.value


def noalloc_scratch_bytes() -> int:
    return load_library().tnns_cuda_noalloc_scratch_bytes()


def conv_noalloc(type_: int, d_packed_weights: int, d_x: int, d_thr: int, d_y: int, shape: Shape, alpha: float, layout=NCHW,
                 stream=0):
    """Whole layer on the current device without any allocation: the packed matrix goes to
    the library's built-in scratch array (see tnns_cuda_conv_noalloc in the header)."""
    _check(load_library().tnns_cuda_conv_noalloc(type_, d_packed_weights, d_x, d_thr, d_y, C.byref(shape), alpha, layout, stream))


def packed_image_bytes(ternary: bool, N: int, C_: int, H: int, W: int) -> int:
    return load_library().tnns_packed_image_bytes(int(ternary), N, C_, H, W)


def fused_workspace_bytes(N: int, C_: int, H: int, W: int) -> int:
    return int(load_library().tnns_fused_workspace_bytes(N, C_, H, W))


def dense_workspace_bytes(shape: Shape) -> int:
    return load_library().tnns_dense_workspace_bytes(C.byref(shape))


def bordered_image_bytes(N: int, C_: int, H: int, W: int, PH: int, PW: int) -> int:
    return int(load_library().tnns_e2m1_bordered_image_bytes(N, C_, H, W, PH, PW))


def slab_workspace_bytes(N: int, C_: int, H: int, W: int, PH: int, PW: int) -> int:
    return int(load_library().tnns_slab_workspace_bytes(N, C_, H, W, PH, PW))


def e2m1_image_bytes(N: int, C_: int, H: int, W: int) -> int:
    return load_library().tnns_e2m1_image_bytes(N, C_, H, W)


def launch_count() -> int:
    return load_library().tnns_cuda_launch_count()
