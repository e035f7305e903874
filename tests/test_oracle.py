"""CPU suite: pins the oracle.  The restatement (oracle/tnns_oracle.c) and, when built,
the reference's own objects (oracle/_ref) must reproduce the committed digests, and the
reference's three statements of the maths (final AVX2, naive packing-0, float conv) must
agree on the reference's own test protocol."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from cases import act_ternary, extra_cases, make_case, reference_test_cases, special_value_case, wgt_ternary

GOLDEN = Path(__file__).resolve().parent / "golden"
DIGESTS = json.loads((GOLDEN / "digests.json").read_text())


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def golden_cases():
    return (reference_test_cases(N=2, dist="uniform", max_ops=3e9)
            + reference_test_cases(N=2, dist="alphabet", max_ops=3e9) + extra_cases())


CASES = golden_cases()


def test_every_digest_has_a_case():
    assert sorted(DIGESTS) == sorted(c.name for c in CASES)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_port_matches_golden(case, port_oracle):
    case = case.build()
    d = DIGESTS[case.name]
    wp = port_oracle.pack_weights(wgt_ternary(case.type), case.w, case.w_thr)
    assert sha(wp) == d["weights"]
    ap = port_oracle.pack(act_ternary(case.type), case.x, case.thr, case.kernel_hw, case.padding, case.stride)
    assert sha(ap) == d["packed"]
    y = port_oracle.conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    assert sha(y) == d["output"]
    # the GEMM entry point on its own, fed the packed matrix
    L = case.layer
    K = L.KH * L.KW * ((L.C + 63) // 64)
    y2 = port_oracle.mm(case.type, ap, wp, case.N, L.OH, L.OW, L.KN, K, case.alpha, K_unpack=L.C * L.KH * L.KW)
    assert y2.tobytes() == y.tobytes()


@pytest.mark.parametrize("case", CASES[::3], ids=lambda c: c.name)
def test_reference_objects_match_golden(case, ref_oracle):
    case = case.build()
    d = DIGESTS[case.name]
    wp = ref_oracle.pack_weights(wgt_ternary(case.type), case.w, case.w_thr)
    assert sha(wp) == d["weights"]
    ap = ref_oracle.pack(act_ternary(case.type), case.x, case.thr, case.kernel_hw, case.padding, case.stride)
    assert sha(ap) == d["packed"]
    y = ref_oracle.conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    assert sha(y) == d["output"]


@pytest.mark.parametrize("case", reference_test_cases(N=2, dist="alphabet", max_ops=3e9)[::2], ids=lambda c: c.name)
def test_reference_statements_agree(case, ref_oracle):
    """The reference's own protocol (src/timing_layers.c:142-165): tnns_conv against
    direct_pad + direct_conv2d, plus its naive packing-0 implementation."""
    case = case.build()
    from oracle import binding
    nv = binding.naive()
    wt = wgt_ternary(case.type)
    wp = ref_oracle.pack_weights(wt, case.w, case.w_thr)
    y = ref_oracle.conv(case.type, case.x, case.thr, wp, case.kernel_hw, case.padding, case.stride, case.alpha)
    yf = ref_oracle.float_conv(case.x, case.w, case.padding, case.stride, case.alpha, 0 if act_ternary(case.type) else 1)
    assert np.abs(yf - y).max() <= 0.01  # the reference's tolerance; the values are in fact equal
    assert np.array_equal(yf, y)
    if nv is not None:
        p0 = nv.pack_weights_naive(wt, case.w, case.w_thr)
        yn = nv.conv(case.type, case.x, case.thr, None, case.kernel_hw, case.padding, case.stride, case.alpha,
                     packing0=(p0, case.layer.KN))
        assert yn.tobytes() == y.tobytes()


def test_tiny_vector(port_oracle):
    z = np.load(GOLDEN / "tiny_tnn.npz")
    wp = port_oracle.pack_weights(True, z["w"], z["w_thr"])
    assert np.array_equal(wp, z["packed_w"])
    ap = port_oracle.pack(True, z["x"], z["thr"], (3, 3), (1, 1), (1, 1))
    assert np.array_equal(ap, z["packed_a"])
    y = port_oracle.conv(0, z["x"], z["thr"], wp, (3, 3), (1, 1), (1, 1), 0.5)
    assert y.tobytes() == z["y"].tobytes()


def test_prelu_zero_is_positive_zero(port_oracle):
    """An all-zero ternary activation gives acc = 0 everywhere; the reference stores +0.0f."""
    x = np.zeros((1, 64, 3, 3), np.float32)
    w = np.ones((4, 64, 3, 3), np.float32)
    wp = port_oracle.pack_weights(True, w, np.full(4, 0.5, np.float32))
    y = port_oracle.conv(0, x, np.array([0.25], np.float32), wp, (3, 3), (1, 1), (1, 1), 0.5)
    assert np.all(y.view(np.uint32) == 0)


@pytest.mark.parametrize("type_", [0, 1, 2, 3])
def test_special_values_port_equals_reference_objects(type_, port_oracle, ref_oracle):
    """+-0, values equal to and next to the thresholds, denormals, infinities."""
    c = special_value_case(type_)
    t = act_ternary(type_)
    a_p = port_oracle.pack(t, c.x, c.thr, c.kernel_hw, c.padding, c.stride)
    a_r = ref_oracle.pack(t, c.x, c.thr, c.kernel_hw, c.padding, c.stride)
    assert np.array_equal(a_p, a_r)


@pytest.mark.parametrize("alpha", [0.0, 1.0, 0.3, -0.25, 2.5])
@pytest.mark.parametrize("type_", [0, 1, 2, 3])
def test_prelu_slopes_port_equals_reference_objects(type_, alpha, port_oracle, ref_oracle):
    """The reference has two PReLU expressions (mm_tnn scales every non-positive sum, the other three
    pass a zero sum through), which differ in the sign of zero for a negative slope; the restatement
    follows both.  Sparse activations make zero sums common."""
    from fastertnn_b200.workloads import Layer
    layer = Layer(70, 5, 5, 33, 2, 2, 1, 1)
    c = make_case(type_, layer, 2, 4321, "uniform")
    c.thr[:] = 0.9 if act_ternary(type_) else 0.0
    wp = ref_oracle.pack_weights(wgt_ternary(type_), c.w, c.w_thr)
    y_r = ref_oracle.conv(type_, c.x, c.thr, wp, c.kernel_hw, c.padding, c.stride, alpha)
    y_p = port_oracle.conv(type_, c.x, c.thr, wp, c.kernel_hw, c.padding, c.stride, alpha)
    assert y_p.tobytes() == y_r.tobytes()
