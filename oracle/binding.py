"""TEST INFRASTRUCTURE ONLY: ctypes bindings of the CPU checkers.

``port``  -> oracle/liboracle_port.so, the in-repo C restatement (tnns_oracle.c).
``ref``   -> oracle/_ref/libtnns_ref.so, the reference's own AVX2 objects when they were
             built (oracle/Makefile); ``None`` otherwise.
``naive`` -> oracle/_ref/libtnns_ref_naive.so, the reference's naive packing-0 path.

Only tests, the smoke check and the CPU-baseline / reference arm of the benchmark may
import this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

from fastertnn_b200._lib import Testcase

HERE = Path(__file__).resolve().parent
_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
TNN, TBN, BTN, BNN = 0, 1, 2, 3


def reference_checkout() -> str:
    """Where the reference's sources lie: the environment variable TNNS_REFERENCE_DIR, else a
    checkout named ``reference`` beside this repository; empty when there is none."""
    import os
    env = os.environ.get("TNNS_REFERENCE_DIR")
    if env:
        return env
    cand = HERE.parent.parent / "reference"
    return str(cand) if (cand / "src" / "tnns" / "tnns_cpu_mm_p2.c").exists() else ""


def build(reference: str | None = None):
    """(Re)build the checkers; the _ref targets are skipped when the reference sources are absent."""
    ref = reference_checkout() if reference is None else reference
    subprocess.run(["make", "-s", "-C", str(HERE), f"REF={ref}"], check=True)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(a):
    """int64, C-contiguous and 64-byte aligned: the reference's AVX2 kernels use aligned
    256-bit loads on packed operands (they come from aligned_alloc(32, ..) there)."""
    a = np.ascontiguousarray(a, dtype=np.int64)
    if a.ctypes.data % 64 == 0:
        return a
    raw = np.empty(a.size + 8, dtype=np.int64)
    off = (-raw.ctypes.data % 64) // 8
    out = raw[off:off + a.size].reshape(a.shape)
    out[...] = a
    return out


def out_dim(size, pad, k, stride):
    return (size + 2 * pad - k) // stride + 1


def k_padded(C_, KH, KW):
    return 4 * ((KH * KW * ((C_ + 63) // 64) + 3) // 4)


class _Lib:
    def __init__(self, path: Path):
        self.path = path
        self.lib = C.CDLL(str(path))
        self.free = C.CDLL(None).free
        self.free.argtypes = [_vp]
        self.free.restype = None

    def _take(self, ptr, count, ctype, dtype):
        if not ptr:
            raise MemoryError(f"{self.path.name}: NULL result")
        out = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ctype)), shape=(count,)).astype(dtype, copy=True)
        self.free(ptr)
        return out


class PortOracle(_Lib):
    """The in-repo restatement."""

    kind = "port"

    def __init__(self):
        path = HERE / "liboracle_port.so"
        if not path.exists():
            build()
        super().__init__(path)
        L = self.lib
        for name in ("orc_t2r", "orc_b2r"):
            getattr(L, name).restype = _vp
            getattr(L, name).argtypes = [_vp, _vp] + [_i] * 10
        for name in ("orc_pack_w_ternary", "orc_pack_w_binary"):
            getattr(L, name).restype = _vp
            getattr(L, name).argtypes = [_vp, _vp, _i, _i, _i, _i]
        for name in ("orc_mm_tnn", "orc_mm_tbn", "orc_mm_btn"):
            getattr(L, name).restype = _vp
            getattr(L, name).argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _f]
        L.orc_mm_bnn.restype = _vp
        L.orc_mm_bnn.argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _i, _f]
        L.orc_conv.restype = _vp
        L.orc_conv.argtypes = [_i, _vp, _vp, _vp] + [_i] * 11 + [_f]

    def pack(self, ternary, x, thr, kernel_hw, padding=(0, 0), stride=(1, 1)):
        x, thr = _f32(x), _f32(thr)
        N, C_, H, W = x.shape
        KH, KW = kernel_hw
        fn = self.lib.orc_t2r if ternary else self.lib.orc_b2r
        p = fn(x.ctypes.data, thr.ctypes.data, N, C_, H, W, padding[0], padding[1], KH, KW, stride[0], stride[1])
        rows = N * out_dim(H, padding[0], KH, stride[0]) * out_dim(W, padding[1], KW, stride[1])
        width = (2 if ternary else 1) * k_padded(C_, KH, KW)
        return self._take(p, rows * width, C.c_int64, np.int64).reshape(rows, width)

    def pack_weights(self, ternary, w, thr):
        w, thr = _f32(w), _f32(thr)
        KN, C_, KH, KW = w.shape
        fn = self.lib.orc_pack_w_ternary if ternary else self.lib.orc_pack_w_binary
        p = fn(w.ctypes.data, thr.ctypes.data, KN, C_, KH, KW)
        width = (2 if ternary else 1) * k_padded(C_, KH, KW)
        return self._take(p, KN * width, C.c_int64, np.int64).reshape(KN, width)

    def mm(self, type_, a, b, N, OH, OW, KN, K, alpha, K_unpack=0):
        a, b = _i64(a), _i64(b)
        if type_ == BNN:
            p = self.lib.orc_mm_bnn(a.ctypes.data, b.ctypes.data, N, OH, OW, KN, K, K_unpack, alpha)
        else:
            fn = {TNN: self.lib.orc_mm_tnn, TBN: self.lib.orc_mm_tbn, BTN: self.lib.orc_mm_btn}[type_]
            p = fn(a.ctypes.data, b.ctypes.data, N, OH, OW, KN, K, alpha)
        return self._take(p, N * KN * OH * OW, C.c_float, np.float32).reshape(N, KN, OH, OW)

    def conv(self, type_, x, thr, packed_w, kernel_hw, padding=(0, 0), stride=(1, 1), alpha=0.5):
        x, thr, pw = _f32(x), _f32(thr), _i64(packed_w)
        N, C_, H, W = x.shape
        KH, KW = kernel_hw
        KN = pw.shape[0]
        p = self.lib.orc_conv(type_, x.ctypes.data, thr.ctypes.data, pw.ctypes.data, N, C_, H, W, KN, KH, KW, padding[0],
                              padding[1], stride[0], stride[1], alpha)
        OH, OW = out_dim(H, padding[0], KH, stride[0]), out_dim(W, padding[1], KW, stride[1])
        return self._take(p, N * KN * OH * OW, C.c_float, np.float32).reshape(N, KN, OH, OW)


class RefOracle(_Lib):
    """The reference's own compiled objects (final / packing-2 AVX2 build)."""

    kind = "reference"

    def __init__(self, path: Path | None = None):
        super().__init__(path or HERE / "_ref" / "libtnns_ref.so")
        L = self.lib
        L.tnns_conv.restype = None
        L.tnns_conv.argtypes = [C.POINTER(Testcase)]
        self.has_final = hasattr(L, "t2r_p2_opt")
        if self.has_final:
            for name in ("t2r_p2_opt", "b2r"):
                getattr(L, name).restype = _vp
                getattr(L, name).argtypes = [_vp, _vp] + [_i] * 10
            for name in ("mm_tnn", "mm_tbn", "mm_btn"):
                getattr(L, name).restype = _vp
                getattr(L, name).argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _f]
            L.mm_bnn.restype = _vp
            L.mm_bnn.argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _i, _f]
        for name in ("ternarize_opt_avx2", "binarize_opt_avx2"):
            getattr(L, name).restype = _vp
            getattr(L, name).argtypes = [_vp, _vp, _i, _i, _i, _i]
        for name in ("ternarize_naive", "binarize_naive"):
            getattr(L, name).restype = _vp
            getattr(L, name).argtypes = [_vp, _vp, _i, _i, _i, _i, _i, _i]
        L.direct_pad.restype = _vp
        L.direct_pad.argtypes = [_vp, _i, _i, _i, _i, _i, _i, _i]
        L.direct_conv2d.restype = _vp
        L.direct_conv2d.argtypes = [_vp, _vp] + [_i] * 9 + [_f]

    def pack(self, ternary, x, thr, kernel_hw, padding=(0, 0), stride=(1, 1)):
        x, thr = _f32(x), _f32(thr)
        N, C_, H, W = x.shape
        KH, KW = kernel_hw
        fn = self.lib.t2r_p2_opt if ternary else self.lib.b2r
        p = fn(x.ctypes.data, thr.ctypes.data, N, C_, H, W, padding[0], padding[1], KH, KW, stride[0], stride[1])
        rows = N * out_dim(H, padding[0], KH, stride[0]) * out_dim(W, padding[1], KW, stride[1])
        width = (2 if ternary else 1) * k_padded(C_, KH, KW)
        return self._take(p, rows * width, C.c_int64, np.int64).reshape(rows, width)

    def pack_weights(self, ternary, w, thr):
        w, thr = _f32(w), _f32(thr)
        KN, C_, KH, KW = w.shape
        fn = self.lib.ternarize_opt_avx2 if ternary else self.lib.binarize_opt_avx2
        p = fn(w.ctypes.data, thr.ctypes.data, KN, C_, KH, KW)
        width = (2 if ternary else 1) * k_padded(C_, KH, KW)
        return self._take(p, KN * width, C.c_int64, np.int64).reshape(KN, width)

    def pack_weights_naive(self, ternary, w, thr):
        """Packing-0 weights for the naive library (its tnns_conv reads quantized_kernel_packing0)."""
        w, thr = _f32(w), _f32(thr)
        KN, C_, KH, KW = w.shape
        fn = self.lib.ternarize_naive if ternary else self.lib.binarize_naive
        p = fn(w.ctypes.data, thr.ctypes.data, KN, C_, KH, KW, 0, 0)
        count = KN * KH * KW * ((C_ + 63) // 64) * (2 if ternary else 1)
        return self._take(p, count, C.c_int64, np.int64)

    def mm(self, type_, a, b, N, OH, OW, KN, K, alpha, K_unpack=0):
        a, b = _i64(a), _i64(b)
        if type_ == BNN:
            p = self.lib.mm_bnn(a.ctypes.data, b.ctypes.data, N, OH, OW, KN, K, K_unpack, alpha)
        else:
            fn = {TNN: self.lib.mm_tnn, TBN: self.lib.mm_tbn, BTN: self.lib.mm_btn}[type_]
            p = fn(a.ctypes.data, b.ctypes.data, N, OH, OW, KN, K, alpha)
        return self._take(p, N * KN * OH * OW, C.c_float, np.float32).reshape(N, KN, OH, OW)

    def conv(self, type_, x, thr, packed_w, kernel_hw, padding=(0, 0), stride=(1, 1), alpha=0.5, packing0=None):
        """The reference's tnns_conv(testcase_t*).  ``packing0`` feeds the naive library."""
        x, thr = _f32(x), _f32(thr)
        N, C_, H, W = x.shape
        KH, KW = kernel_hw
        t = Testcase()
        t.type = type_
        t.batchcount, t.channelcount, t.inputH, t.inputW = N, C_, H, W
        t.kernelH, t.kernelW = KH, KW
        t.paddingH, t.paddingW = padding
        t.strideH, t.strideW = stride
        t.preluAlpha = alpha
        t.input_thresholds = thr.ctypes.data_as(C.POINTER(C.c_float))
        t.input = x.ctypes.data_as(C.POINTER(C.c_float))
        if packed_w is not None:
            pw = _i64(packed_w)
            t.kernelcount = pw.shape[0]
            t.quantized_kernel_packing2 = pw.ctypes.data_as(C.POINTER(C.c_int64))
        if packing0 is not None:
            p0, KN = packing0
            p0 = _i64(p0)
            t.kernelcount = KN
            t.quantized_kernel_packing0 = p0.ctypes.data_as(C.POINTER(C.c_int64))
        self.lib.tnns_conv(C.byref(t))
        KN = t.kernelcount
        OH, OW = out_dim(H, padding[0], KH, stride[0]), out_dim(W, padding[1], KW, stride[1])
        return self._take(C.cast(t.output, _vp).value, N * KN * OH * OW, C.c_float, np.float32).reshape(N, KN, OH, OW)

    def float_conv(self, x, w, padding, stride, alpha, pad_val):
        """direct_pad + direct_conv2d (src/utils.c:101-155): the reference's float checker."""
        x, w = _f32(x), _f32(w)
        N, C_, H, W = x.shape
        KN, _, KH, KW = w.shape
        px = self.lib.direct_pad(x.ctypes.data, padding[0], padding[1], N, C_, H, W, pad_val)
        HP, WP = H + 2 * padding[0], W + 2 * padding[1]
        y = self.lib.direct_conv2d(px, w.ctypes.data, stride[0], stride[1], N, C_, HP, WP, KN, KH, KW, alpha)
        self.free(px)
        OH, OW = (HP - KH) // stride[0] + 1, (WP - KW) // stride[1] + 1
        return self._take(y, N * KN * OH * OW, C.c_float, np.float32).reshape(N, KN, OH, OW)


_port = None
_ref = None
_naive = None


def port() -> PortOracle:
    global _port
    if _port is None:
        _port = PortOracle()
    return _port


def ref() -> RefOracle | None:
    global _ref
    path = HERE / "_ref" / "libtnns_ref.so"
    if _ref is None and path.exists():
        _ref = RefOracle(path)
    return _ref


def naive() -> RefOracle | None:
    global _naive
    path = HERE / "_ref" / "libtnns_ref_naive.so"
    if _naive is None and path.exists():
        _naive = RefOracle(path)
    return _naive


def best():
    """The reference's own objects when present, else the restatement."""
    return ref() or port()
