"""fastertnn_b200 -- B200-native ternary/binary convolution + GEMM inference path.

The product is ``libtnns_b200.so`` (CUDA kernels for sm_100a behind a C ABI, see
``include/tnns_b200.h``).  This package is the Python host side: it loads the library,
mirrors the reference's operator interface (``tnns_conv``, ``tnns_gemm``, ``mm_*``,
``t2r_p2_opt``, ``b2r``) over numpy arrays, and exposes the device-resident API over
raw device pointers (torch tensors supply memory and streams).
"""
from .api import (  # noqa: F401
    TNN, TBN, BTN, BNN, NCHW, NHWC,
    PACK_AUTO, PACK_GATHER, PACK_STAGED,
    GEMM_AUTO, GEMM_POPC_SIMPLE, GEMM_POPC_TILED, GEMM_I8_TC, GEMM_F4_TC, GEMM_F4_FUSED, GEMM_F4_SLAB, GEMM_F4_SLAB_FUSED, GEMM_F4_DENSE,
    Shape, Testcase, GemmTestcase, TnnsError, Context, Weights, MultiContext, MultiWeights, shard_range, shard_run,
    tnns_conv, tnns_gemm, mm_tnn, mm_tbn, mm_btn, mm_bnn, t2r_p2_opt, b2r,
    pack_weights_ternary, pack_weights_binary, out_dim, k_words, k_padded, packed_bytes,
)
from ._lib import library_path, load_library  # noqa: F401
