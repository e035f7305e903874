"""The benchmark configurations and the reference's own test shapes, as data.

Layer tuples are (C, H, W, KN, KH, KW, P, S), the same eight quantities the reference's
shape tables hold (include/timing/shapes_test.h of the reference lists them as
c, ih, iw, kn, kw, kh, p, s).
"""
from __future__ import annotations

from dataclasses import dataclass

import json
from pathlib import Path

from ._lib import Shape


@dataclass(frozen=True)
class Layer:
    C: int
    H: int
    W: int
    KN: int
    KH: int
    KW: int
    P: int
    S: int

    def shape(self, N: int) -> Shape:
        return Shape(N, self.C, self.H, self.W, self.KN, self.KH, self.KW, self.P, self.P, self.S, self.S)

    @property
    def OH(self):
        return (self.H + 2 * self.P - self.KH) // self.S + 1

    @property
    def OW(self):
        return (self.W + 2 * self.P - self.KW) // self.S + 1

    def ops(self, N: int) -> int:
        """2*M*N*K with the unpadded K = C*KH*KW."""
        return 2 * N * self.OH * self.OW * self.KN * self.C * self.KH * self.KW


# The 12 shapes of the reference's correctness run (batch 8 there).
REFERENCE_TEST_LAYERS = [
    Layer(32, 7, 7, 32, 3, 3, 0, 1),
    Layer(32, 7, 7, 32, 3, 3, 1, 2),
    Layer(127, 7, 7, 32, 3, 3, 1, 1),
    Layer(127, 7, 7, 32, 3, 3, 1, 1),
    Layer(128, 7, 7, 32, 3, 3, 1, 2),
    Layer(193, 7, 7, 32, 3, 3, 1, 2),
    Layer(256, 14, 14, 256, 5, 3, 1, 2),   # kernel 5 high x 3 wide (table order is kw, kh)
    Layer(256, 14, 14, 256, 3, 3, 1, 2),
    Layer(257, 14, 14, 257, 3, 3, 1, 2),
    Layer(320, 15, 23, 320, 3, 3, 1, 2),
    Layer(512, 1, 1, 512, 1, 1, 0, 1),
    Layer(1024, 14, 14, 1024, 5, 5, 1, 2),
]
REFERENCE_TEST_BATCH = 8

# Benchmark configurations.
FC_GEMM = (1024, Layer(4096, 1, 1, 1024, 1, 1, 0, 1))        # M=1024 K=4096 N=1024
CONV_56 = (1, Layer(256, 56, 56, 256, 3, 3, 1, 1))            # M=3136 K=2304 N=256
CONV_LARGE = (64, Layer(512, 32, 32, 512, 3, 3, 1, 1))        # M=65536 K=4608 N=512

# ResNet-18-style stack: two convs per stage, stride-2 transitions between stages.
RESNET18_STACK_BATCH = 256
RESNET18_STACK = [
    Layer(64, 56, 56, 64, 3, 3, 1, 1), Layer(64, 56, 56, 64, 3, 3, 1, 1),
    Layer(64, 56, 56, 128, 3, 3, 1, 2),
    Layer(128, 28, 28, 128, 3, 3, 1, 1), Layer(128, 28, 28, 128, 3, 3, 1, 1),
    Layer(128, 28, 28, 256, 3, 3, 1, 2),
    Layer(256, 14, 14, 256, 3, 3, 1, 1), Layer(256, 14, 14, 256, 3, 3, 1, 1),
    Layer(256, 14, 14, 512, 3, 3, 1, 2),
    Layer(512, 7, 7, 512, 3, 3, 1, 1), Layer(512, 7, 7, 512, 3, 3, 1, 1),
]


# Layer tables of the reference's end-to-end timing mode (its include/timing/shapes_e2e.h: ResNet18/34/152,
# VGG16/19, DarkNet19/53), kept as numbers in model_tables.json; batch 8 there (src/timing_layers.c:46).
_MODEL_TABLES = None


def model_tables() -> dict:
    global _MODEL_TABLES
    if _MODEL_TABLES is None:
        _MODEL_TABLES = json.loads((Path(__file__).resolve().parent / "model_tables.json").read_text())
    return _MODEL_TABLES


def model_names() -> list[str]:
    return sorted(model_tables()["models"])


def model_layers(name: str) -> list[Layer]:
    """The layers of one of the reference's model tables, in the order its driver runs them."""
    return [Layer(*row) for row in model_tables()["models"][name]]


REFERENCE_MODEL_BATCH = 8
