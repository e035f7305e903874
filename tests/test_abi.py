"""CPU suite: the shared library loads without a GPU and exports every symbol that
include/tnns_b200.h declares; struct layouts match the header; host-only helpers agree
with the oracle.  No kernel is launched here."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import fastertnn_b200 as ft
from fastertnn_b200 import _lib
from cases import extra_cases, wgt_ternary

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "tnns_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)  # preprocessor lines declare no functions
    text = re.sub(r"typedef[^;]*\(\s*\*[^;]*;", "", text)  # function-pointer typedefs declare no functions
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}]*\)\s*;", text)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_header_declares_the_reference_entry_points():
    names = declared_functions()
    for n in ("tnns_conv", "tnns_gemm", "mm_tnn", "mm_tbn", "mm_btn", "mm_bnn", "t2r_p2_opt", "b2r"):
        assert n in names


def test_library_exports_every_declared_symbol():
    lib = ft.load_library()
    names = declared_functions()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/tnns_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"


def test_struct_layouts():
    # testcase_t: 12 ints + float, padding to 8, 7 pointers (include/tnns/data.h:4-25 of the reference)
    assert C.sizeof(_lib.Testcase) == 13 * 4 + 4 + 7 * 8
    assert _lib.Testcase.input.offset == 64
    assert C.sizeof(_lib.GemmTestcase) == 4 * 4 + 9 * 8
    assert C.sizeof(_lib.Shape) == 11 * 4


def test_size_helpers():
    assert ft.out_dim(56, 1, 3, 1) == 56
    assert ft.out_dim(14, 1, 5, 2) == 6
    assert ft.k_words(64, 3, 3) == 9 and ft.k_padded(64, 3, 3) == 12
    assert ft.k_words(257, 3, 3) == 45 and ft.k_padded(257, 3, 3) == 48
    s = ft.Shape(64, 512, 32, 32, 512, 3, 3, 1, 1, 1, 1)
    assert ft.packed_bytes(ft.TNN, s) == 65536 * 72 * 16
    assert ft.packed_bytes(ft.BTN, s) == 65536 * 72 * 8
    bad = ft.Shape(1, 8, 2, 2, 1, 3, 3, 0, 0, 1, 1)  # kernel larger than the image
    assert ft.packed_bytes(ft.TNN, bad) == 0


@pytest.mark.parametrize("case", extra_cases()[::2], ids=lambda c: c.name)
def test_host_weight_packers_match_oracle(case, port_oracle):
    case = case.build()
    t = wgt_ternary(case.type)
    mine = (ft.pack_weights_ternary if t else ft.pack_weights_binary)(case.w, case.w_thr)
    assert np.array_equal(mine, port_oracle.pack_weights(t, case.w, case.w_thr))


def test_error_strings():
    lib = ft.load_library()
    assert lib.tnns_cuda_strerror(0) == b"success"
    assert b"invalid" in lib.tnns_cuda_strerror(1)
