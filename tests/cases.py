"""Seeded test cases shared by the CPU and GPU suites."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from fastertnn_b200 import synth
from fastertnn_b200.workloads import Layer, REFERENCE_TEST_LAYERS

TNN, TBN, BTN, BNN = 0, 1, 2, 3
TYPE_NAMES = {TNN: "tnn", TBN: "tbn", BTN: "btn", BNN: "bnn"}


def act_ternary(t):
    return t in (TNN, TBN)


def wgt_ternary(t):
    return t in (TNN, BTN)


@dataclass
class Case:
    name: str
    type: int
    layer: Layer
    N: int
    x: np.ndarray          # fp32 NCHW
    thr: np.ndarray        # fp32 [N]
    w: np.ndarray          # fp32 [KN][C][KH][KW], values in the weight alphabet
    w_thr: np.ndarray      # fp32 [KN]
    alpha: float = 0.5

    @property
    def kernel_hw(self):
        return (self.layer.KH, self.layer.KW)

    @property
    def padding(self):
        return (self.layer.P, self.layer.P)

    @property
    def stride(self):
        return (self.layer.S, self.layer.S)


def make_case(type_: int, layer: Layer, N: int, seed: int, dist: str = "uniform", name: str = "") -> Case:
    """dist 'uniform': activations uniform in [-1,1), thresholds 0.25 / 0.0 with a different
    value on odd images (exercises the per-image threshold); 'alphabet': activations already
    in {-1,0,+1} / {-1,+1} with thresholds 0.5 / 0.0, the reference's own test protocol
    (src/timing_layers.c:97-107 of the reference)."""
    xs = (N, layer.C, layer.H, layer.W)
    ws = (layer.KN, layer.C, layer.KH, layer.KW)
    if dist == "uniform":
        x = synth.uniform_pm1(seed, xs)
        if act_ternary(type_):
            thr = np.where(np.arange(N) % 2 == 0, 0.25, 0.4).astype(np.float32)
        else:
            thr = np.where(np.arange(N) % 2 == 0, 0.0, 0.1).astype(np.float32)
    elif dist == "alphabet":
        x = synth.ternary_values(seed, xs) if act_ternary(type_) else synth.binary_values(seed, xs)
        thr = np.full(N, 0.5 if act_ternary(type_) else 0.0, np.float32)
    else:
        raise ValueError(dist)
    if wgt_ternary(type_):
        w = synth.ternary_values(seed + 1, ws)
        w_thr = np.full(layer.KN, 0.5, np.float32)
    else:
        w = synth.binary_values(seed + 1, ws)
        w_thr = np.full(layer.KN, 0.0, np.float32)
    return Case(name or f"{TYPE_NAMES[type_]}-{layer}", type_, layer, N, x, thr, w, w_thr)


def reference_test_cases(N: int = 2, dist: str = "uniform", types=(TNN, TBN, BTN, BNN), max_ops: float | None = None):
    """The 12 shapes of the reference's correctness run, for each network type."""
    out = []
    for t in types:
        for i, layer in enumerate(REFERENCE_TEST_LAYERS):
            n = N
            if max_ops is not None:
                while n > 1 and layer.ops(n) > max_ops:
                    n -= 1
            out.append(make_case(t, layer, n, 1000 * (t + 1) + i, dist, name=f"{TYPE_NAMES[t]}-shape{i}-{dist}"))
    return out


# Small odd geometries: non-square kernels and strides are covered by the reference shapes;
# these add channel counts around the 32/64 boundaries, batch 1 and 3, kernel = image,
# padding wider than the kernel reach, a 7x7 kernel, stride 3 and KN tails.
EXTRA_LAYERS = [
    Layer(1, 5, 5, 3, 3, 3, 1, 1),
    Layer(31, 6, 9, 5, 3, 3, 1, 1),
    Layer(33, 9, 6, 65, 3, 3, 1, 2),
    Layer(64, 8, 8, 64, 3, 3, 1, 1),     # Kw = 9 -> Kp = 12: three pad-to-four words
    Layer(65, 4, 4, 7, 1, 1, 0, 1),
    Layer(96, 5, 7, 33, 5, 5, 2, 1),
    Layer(100, 3, 3, 10, 3, 3, 0, 1),    # kernel covers the whole image: one output pixel
    Layer(70, 6, 6, 12, 2, 2, 3, 1),     # padding wider than the kernel: all-padding windows
    Layer(130, 12, 12, 20, 7, 7, 3, 3),
    Layer(256, 1, 1, 100, 1, 1, 0, 1),   # fully connected
    Layer(320, 1, 1, 64, 1, 1, 0, 1),    # fully connected, C % 256 != 0
    Layer(128, 16, 16, 128, 3, 3, 1, 1),
]


def extra_cases(types=(TNN, TBN, BTN, BNN)):
    out = []
    for t in types:
        for i, layer in enumerate(EXTRA_LAYERS):
            N = 3 if i % 2 else 1
            out.append(make_case(t, layer, N, 5000 * (t + 1) + i, "uniform", name=f"{TYPE_NAMES[t]}-extra{i}"))
    return out


def to_nhwc(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x.transpose(0, 2, 3, 1))


def to_nchw(y: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(y.transpose(0, 3, 1, 2))
