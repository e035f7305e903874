"""The quantising epilogues replace "PReLU, then the next layer's quantiser" by thresholds on the raw
integer accumulator.  The constants come from host-callable code shared with the kernels
(tnns_prelu_thresholds), so the equivalence is checked here exhaustively over every accumulator value a
layer can produce, against the reference's expressions evaluated in fp32 by numpy."""
import numpy as np
import pytest

import fastertnn_b200 as ft

R = 5000  # |accumulator| <= K = C*KH*KW; the largest layer of the workloads has 4608


def reference_bits(v, bias, alpha, t, ternary):
    """mm_p2_final_*: a > 0 ? a : a * alpha (one fp32 rounding); ternarize2row: sign = f < -t, non-zero = |f| > t;
    binarize2row: sign = f < t."""
    a = (v + np.float32(bias)).astype(np.float32)
    f = np.where(a > 0, a, (a * np.float32(alpha)).astype(np.float32)).astype(np.float32)
    t = np.float32(t)
    if ternary:
        return f < -t, np.abs(f) > t
    return f < t, None


def threshold_bits(v, n1, t2, ternary):
    sign = np.signbit((v + np.float32(n1)).astype(np.float32))
    if not ternary:
        return sign, None
    above = np.signbit((np.float32(t2) - v).astype(np.float32))
    return sign, sign | above


ALPHAS = [0.5, 1.0, 0.25, 0.3, 0.7, 0.1, 1e-3, 0.9999999, 1.1754944e-38, 3e-42]
THRESHOLDS = [0.0, -0.0, 0.25, 0.5, 1.0, 1.5, 2.0, 0.1, 3.3, 17.0, 100.5, 4607.9, 4608.0, 6000.0, 1e-30, 1e30, -0.2, -1.0, -2.5, -1e30,
              float("inf"), float("-inf"), float("nan")]


@pytest.mark.parametrize("ternary", [True, False])
@pytest.mark.parametrize("bias", [0.0, -37.0, 1000.0])
def test_threshold_rule_equals_prelu_then_quantise(ternary, bias):
    v = np.arange(-R, R + 1, dtype=np.float32)
    v_with_minus_zero = np.concatenate([v, np.array([-0.0], np.float32)])
    for alpha in ALPHAS:
        for t in THRESHOLDS:
            n1, t2 = ft.api.prelu_thresholds(t, alpha, bias, ternary)
            want = reference_bits(v_with_minus_zero, bias, alpha, t, ternary)
            got = threshold_bits(v_with_minus_zero, n1, t2, ternary)
            assert np.array_equal(want[0], got[0]), ("sign", alpha, t, bias)
            if ternary:
                assert np.array_equal(want[1], got[1]), ("non-zero", alpha, t, bias)


def test_threshold_rule_random():
    rng = np.random.default_rng(77)
    v = np.arange(-R, R + 1, dtype=np.float32)
    for _ in range(400):
        alpha = float(np.float32(rng.uniform(1e-4, 1.0)))
        t = float(np.float32(rng.normal(0, 3) if rng.random() < 0.5 else rng.uniform(-R * alpha, R)))
        for ternary in (True, False):
            n1, t2 = ft.api.prelu_thresholds(t, alpha, 0.0, ternary)
            want = reference_bits(v, 0.0, alpha, t, ternary)
            got = threshold_bits(v, n1, t2, ternary)
            assert np.array_equal(want[0], got[0]), ("sign", alpha, t)
            if ternary:
                assert np.array_equal(want[1], got[1]), ("non-zero", alpha, t)


def test_threshold_rule_needs_alpha_in_unit_interval():
    for alpha in (0.0, -0.5, 1.5, float("nan")):
        with pytest.raises(ft.TnnsError):
            ft.api.prelu_thresholds(0.25, alpha)
