"""ctypes loader for libtnns_b200.so.  There is no fallback: if the library is missing
or does not load, importing a symbol raises."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_LIB = None


class Shape(C.Structure):
    """``tnns_shape_t`` of include/tnns_b200.h."""
    _fields_ = [(n, C.c_int) for n in ("N", "C", "H", "W", "KN", "KH", "KW", "PH", "PW", "SH", "SW")]

    @property
    def OH(self):
        return (self.H + 2 * self.PH - self.KH) // self.SH + 1

    @property
    def OW(self):
        return (self.W + 2 * self.PW - self.KW) // self.SW + 1


class Testcase(C.Structure):
    """``testcase_t``: field order of the reference's include/tnns/data.h:4-25."""
    _fields_ = [
        ("type", C.c_int), ("batchcount", C.c_int), ("channelcount", C.c_int),
        ("inputW", C.c_int), ("inputH", C.c_int), ("kernelcount", C.c_int),
        ("kernelW", C.c_int), ("kernelH", C.c_int), ("paddingW", C.c_int), ("paddingH", C.c_int),
        ("strideW", C.c_int), ("strideH", C.c_int), ("preluAlpha", C.c_float),
        ("input_thresholds", C.POINTER(C.c_float)), ("input", C.POINTER(C.c_float)),
        ("kernel", C.POINTER(C.c_float)),
        ("quantized_kernel_packing0", C.POINTER(C.c_int64)),
        ("quantized_kernel_packing1", C.POINTER(C.c_int64)),
        ("quantized_kernel_packing2", C.POINTER(C.c_int64)),
        ("output", C.POINTER(C.c_float)),
    ]


class GemmTestcase(C.Structure):
    """``testcase_tnns_gemm_t``: include/tnns/data.h:27-41 of the reference."""
    _fields_ = [
        ("m", C.c_int), ("p", C.c_int), ("p_packed", C.c_int), ("n", C.c_int),
        ("x", C.POINTER(C.c_float)), ("w", C.POINTER(C.c_float)),
        ("x_packing0", C.POINTER(C.c_int64)), ("x_packing1", C.POINTER(C.c_int64)),
        ("x_packing2", C.POINTER(C.c_int64)), ("w_packing0", C.POINTER(C.c_int64)),
        ("w_packing1", C.POINTER(C.c_int64)), ("w_packing2", C.POINTER(C.c_int64)),
        ("output", C.POINTER(C.c_float)),
    ]


# name -> (restype, argtypes); every symbol include/tnns_b200.h declares
_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
_pf, _pi64 = C.POINTER(C.c_float), C.POINTER(C.c_int64)
_pshape = C.POINTER(Shape)
SHARD_FN = C.CFUNCTYPE(C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p)  # tnns_shard_fn
SIGNATURES = {
    "tnns_conv": (None, [C.POINTER(Testcase)]),
    "tnns_gemm": (None, [C.POINTER(GemmTestcase)]),
    "tnns_b200_thread_shutdown": (None, []),
    "mm_tnn": (_vp, [_vp, _vp, _i, _i, _i, _i, _i, _f]),
    "mm_tbn": (_vp, [_vp, _vp, _i, _i, _i, _i, _i, _f]),
    "mm_btn": (_vp, [_vp, _vp, _i, _i, _i, _i, _i, _f]),
    "mm_bnn": (_vp, [_vp, _vp, _i, _i, _i, _i, _i, _i, _f]),
    "t2r_p2_opt": (_vp, [_vp, _vp] + [_i] * 10),
    "b2r": (_vp, [_vp, _vp] + [_i] * 10),
    "tnns_pack_weights_ternary": (_vp, [_vp, _vp, _i, _i, _i, _i]),
    "tnns_pack_weights_binary": (_vp, [_vp, _vp, _i, _i, _i, _i]),
    "tnns_cuda_create": (_i, [_i, C.POINTER(_vp)]),
    "tnns_cuda_destroy": (None, [_vp]),
    "tnns_out_dim": (_i, [_i, _i, _i, _i]),
    "tnns_k_words": (_i, [_i, _i, _i]),
    "tnns_k_padded": (_i, [_i, _i, _i]),
    "tnns_packed_bytes": (_sz, [_i, _pshape]),
    "tnns_cuda_upload_weights": (_i, [_vp, _i, _vp, _i, _i, _i, _i, C.POINTER(_vp)]),
    "tnns_cuda_upload_weights_packed": (_i, [_vp, _i, _vp, _i, _i, _i, C.POINTER(_vp)]),
    "tnns_cuda_pack_weights": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tnns_cuda_free_weights": (None, [_vp, _vp]),
    "tnns_cuda_pack": (_i, [_vp, _i, _vp, _vp, _vp, _pshape, _i, _i, _vp]),
    "tnns_cuda_gemm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _i, _vp]),
    "tnns_cuda_conv": (_i, [_vp, _vp, _vp, _vp, _vp, _pshape, _f, _i, _i, _i, _vp]),
    "tnns_cuda_conv_ws": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _pshape, _f, _i, _i, _i, _vp]),
    "tnns_packed_image_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "tnns_cuda_quantise": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "tnns_cuda_gemm_implicit": (_i, [_vp, _vp, _vp, _vp, _pshape, _f, _i, _vp]),
    "tnns_cuda_gemm_packed_out": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]),
    "tnns_cuda_im2row_packed": (_i, [_vp, _i, _vp, _vp, _pshape, _vp]),
    "tnns_cuda_conv_host": (_i, [_vp, _vp, _vp, _vp, _vp, _pshape, _f, _i]),
    "tnns_shard_range": (None, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "tnns_shard_run": (_i, [_i, _i, SHARD_FN, _vp, C.POINTER(_i)]),
    "tnns_cuda_multi_create": (_i, [C.POINTER(_i), _i, C.POINTER(_vp)]),
    "tnns_cuda_multi_destroy": (None, [_vp]),
    "tnns_cuda_multi_device_count": (_i, [_vp]),
    "tnns_cuda_multi_context": (_vp, [_vp, _i]),
    "tnns_cuda_multi_upload_weights": (_i, [_vp, _i, _vp, _i, _i, _i, _i, C.POINTER(_vp)]),
    "tnns_cuda_multi_free_weights": (None, [_vp, _vp]),
    "tnns_cuda_multi_conv_host": (_i, [_vp, _vp, _vp, _vp, _vp, _pshape, _f, _i, C.POINTER(_i)]),
    "tnns_cuda_noalloc_scratch_bytes": (_sz, []),
    "tnns_cuda_conv_noalloc": (_i, [_i, _vp, _vp, _vp, _vp, _pshape, _f, _i, _vp]),
    "tnns_cuda_pipe_rate": (_i, [_vp, _i, C.POINTER(C.c_double)]),
    "tnns_cuda_selftest_wait_expiry": (_i, [_vp]),
    "tnns_prelu_thresholds": (_i, [_f, _f, _f, _i, C.POINTER(_f), C.POINTER(_f)]),
    "tnns_cuda_sync": (_i, [_vp]),
    "tnns_cuda_malloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "tnns_cuda_free": (None, [_vp, _vp]),
    "tnns_cuda_mem_info": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "tnns_cuda_malloc_host": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "tnns_cuda_free_host": (None, [_vp, _vp]),
    "tnns_e2m1_image_bytes": (_sz, [_i, _i, _i, _i]),
    "tnns_cuda_im2col_supported": (_i, [_vp, _vp]),
    "tnns_cuda_quantise_e2m1": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "tnns_cuda_gemm_im2col": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_float, _i, _i, _vp]),
    "tnns_fused_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "tnns_e2m1_bordered_image_bytes": (_sz, [_i] * 6),
    "tnns_slab_workspace_bytes": (_sz, [_i] * 6),
    "tnns_cuda_slab_supported": (_i, [_vp, _vp, _vp]),
    "tnns_cuda_conv_slab_supported": (_i, [_vp, _vp, _vp, _vp, _i]),
    "tnns_cuda_slab_preferred": (_i, [_vp, _vp, _vp]),
    "tnns_cuda_conv_auto_algo": (_i, [_vp, _vp, _vp, _vp, _i]),
    "tnns_cuda_conv_slab_one_launch_preferred": (_i, [_vp, _vp, _vp, _vp, _i]),
    "tnns_cuda_quantise_e2m1_bordered": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tnns_cuda_gemm_slab": (_i, [_vp, _vp, _vp, _vp, _pshape, C.c_float, _i, _i, _vp]),
    "tnns_cuda_gemm_slab_packed_out": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _pshape, C.c_float, _i, _vp]),
    "tnns_dense_workspace_bytes": (_sz, [_pshape]),
    "tnns_cuda_dense_supported": (_i, [_vp, _vp, _pshape]),
    "tnns_cuda_conv_dense": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_conv_dense_packed_out": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_gemm_im2col_bordered_out": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_conv_slab": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_conv_slab_packed_out": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_conv_fused_supported": (_i, [_vp, _vp, _vp, _i]),
    "tnns_cuda_conv_fused_preferred": (_i, [_vp, _vp, _vp, _vp, _i]),
    "tnns_cuda_conv_fused_packed_out": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _sz, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_conv_fused": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _pshape, C.c_float, _i, _vp]),
    "tnns_cuda_gemm_im2col_packed_out": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, C.c_float, _i, _vp]),
    "tnns_cuda_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "tnns_cuda_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "tnns_cuda_launch_count": (C.c_ulonglong, []),
    "tnns_cuda_last_error": (_i, []),
    "tnns_cuda_strerror": (C.c_char_p, [_i]),
    "tnns_cuda_error_detail": (C.c_char_p, []),
}


def library_path() -> Path:
    return _PKG / "libtnns_b200.so"


def load_library():
    """Load libtnns_b200.so and bind every declared symbol.  Raises if it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -m fastertnn_b200._build` (needs nvcc). "
            "There is no CPU fallback.")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    lib.libc_free = C.CDLL(None).free
    lib.libc_free.argtypes = [C.c_void_p]
    lib.libc_free.restype = None
    _LIB = lib
    return lib
