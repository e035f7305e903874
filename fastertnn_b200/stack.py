"""Chained layers on the device: the output of one layer is the next layer's input, as the
reference's end-to-end timing mode does on the host (src/timing_layers.c:188-201 of the
reference: ``test->input = test->output`` between layers).  Activations stay in HBM as fp32
in the chosen layout; every layer re-quantises its input with its own thresholds.

``chain="packed"`` removes that fp32 round trip: every layer but the last runs its GEMM with
the quantising epilogue (``tnns_cuda_gemm_packed_out``) and the next layer starts from the bit
planes (``tnns_cuda_im2row_packed``); the final fp32 output is bit-identical.

``chain="image"`` goes one step further where the layers qualify for the copy-engine route:
the input is quantised once into a 4-bit operand image, every layer is ONE kernel -- the GEMM fed
by im2col tensor copies, whose epilogue writes the next layer's 4-bit image
(``tnns_cuda_gemm_im2col_packed_out``) -- and only the last layer writes fp32; where the first layer
is large enough for the one-launch route, its kernel also quantises the input
(``tnns_cuda_conv_fused_packed_out``).  A layer that does
not qualify takes the bit-plane steps of the packed chain; the format between two layers is
chosen by what the consumer reads.  The final output is again bit-identical."""
from __future__ import annotations

import numpy as np

from . import api
from .workloads import Layer


class ConvStack:
    def __init__(self, ctx: api.Context, type_: int, layers: list[Layer], packed_weights: list[np.ndarray], batch: int,
                 threshold: float, alpha: float = 0.5, layout: int = api.NCHW, chain: str = "fp32"):
        assert len(layers) == len(packed_weights)
        for a, b in zip(layers, layers[1:]):
            if (a.KN, a.OH, a.OW) != (b.C, b.H, b.W):
                raise ValueError(f"layer output {a.KN}x{a.OH}x{a.OW} does not feed {b.C}x{b.H}x{b.W}")
        self.ctx, self.type, self.layers, self.batch, self.alpha, self.layout = ctx, type_, layers, batch, alpha, layout
        self.weights = [ctx.upload_weights(type_, pw, L.C, L.KH, L.KW) for L, pw in zip(layers, packed_weights)]
        sizes = [batch * layers[0].C * layers[0].H * layers[0].W] + [batch * L.KN * L.OH * L.OW for L in layers]
        self.sizes = sizes
        big = max(sizes) * 4
        self.buf = [ctx.malloc(big), ctx.malloc(big)]  # ping-pong activation buffers
        self.d_thr = ctx.to_device(np.full(batch, threshold, np.float32))
        self.chain = chain
        self.act_ternary = type_ in (api.TNN, api.TBN)
        self.extra = []
        if chain == "packed":
            if layout != api.NCHW:
                raise ValueError("the packed chain is defined for NCHW input and output")
            img = max(api.packed_image_bytes(self.act_ternary, batch, L.KN, L.OH, L.OW) for L in layers)
            a = max(api.packed_bytes(type_, L.shape(batch)) for L in layers)
            self.d_img = ctx.malloc(img)
            self.d_a = ctx.malloc(a)
            self.extra = [self.d_img, self.d_a]
        elif chain == "image":
            if layout != api.NCHW:
                raise ValueError("the image chain is defined for NCHW input and output")
            if not self.act_ternary:
                raise ValueError("4-bit operand images hold ternary activations")
            self.fast = [ctx.im2col_supported(w, L.shape(batch)) for w, L in zip(self.weights, layers)]
            img = max([api.e2m1_image_bytes(batch, layers[0].C, layers[0].H, layers[0].W)] +
                      [api.e2m1_image_bytes(batch, L.KN, L.OH, L.OW) for L in layers])
            self.d_imgs = [ctx.malloc(img), ctx.malloc(img)]  # ping-pong quantised activations (either format fits)
            self.extra = list(self.d_imgs)
            # first layer in one launch (quantise step inside the GEMM kernel) where the library itself
            # would choose that route; its workspace holds the input's 4-bit image
            L0 = layers[0]
            self.fuse_first = bool(self.fast[0]) and ctx.conv_fused_preferred(self.weights[0], L0.shape(batch), self.buf[0], layout)
            self.ws0_bytes = api.fused_workspace_bytes(batch, L0.C, L0.H, L0.W)
            if self.fuse_first:
                self.d_ws0 = ctx.malloc(self.ws0_bytes)
                self.extra.append(self.d_ws0)
            self.d_a = None
            if not all(self.fast):
                self.d_a = ctx.malloc(max(api.packed_bytes(type_, L.shape(batch)) for L, f in zip(layers, self.fast) if not f))
                self.extra.append(self.d_a)
        elif chain != "fp32":
            raise ValueError(chain)

    def input_ptr(self) -> int:
        return self.buf[0]

    def output_ptr(self) -> int:
        return self.buf[1] if self.chain in ("packed", "image") else self.buf[len(self.layers) % 2]

    def run(self, stream: int = 0):
        """Enqueue all layers; input must already be in input_ptr()."""
        if self.chain == "packed":
            last = len(self.layers) - 1
            for i, (L, w) in enumerate(zip(self.layers, self.weights)):
                shape = L.shape(self.batch)
                if i == 0:
                    self.ctx.pack(self.act_ternary, self.buf[0], self.d_thr, self.d_a, shape, self.layout, stream=stream)
                else:
                    self.ctx.im2row_packed(self.act_ternary, self.d_img, self.d_a, shape, stream=stream)
                if i < last:
                    self.ctx.gemm_packed_out(w, self.d_a, self.d_img, self.d_thr, self.act_ternary, self.batch, L.OH, L.OW, self.alpha,
                                             stream=stream)
                else:
                    self.ctx.gemm(w, self.d_a, self.buf[1], self.batch, L.OH, L.OW, self.alpha, self.layout, stream=stream)
            return
        if self.chain == "image":
            last = len(self.layers) - 1
            L0 = self.layers[0]
            # the input, in the format the first layer reads
            if self.fuse_first:
                pass
            elif self.fast[0]:
                self.ctx.quantise_e2m1(self.buf[0], self.d_thr, self.d_imgs[0], self.batch, L0.C, L0.H, L0.W, self.layout, stream)
            else:
                self.ctx.quantise(True, self.buf[0], self.d_thr, self.d_imgs[0], self.batch, L0.C, L0.H, L0.W, self.layout, stream)
            for i, (L, w) in enumerate(zip(self.layers, self.weights)):
                shape = L.shape(self.batch)
                src, dst = self.d_imgs[i % 2], self.d_imgs[(i + 1) % 2]
                nxt = 2 if (i < last and self.fast[i + 1]) else 1  # 4-bit image or ternary bit planes for the consumer
                if i == 0 and self.fuse_first:
                    if i < last:
                        self.ctx.conv_fused_packed_out(w, self.buf[0], self.d_thr, dst, self.d_thr, nxt, self.d_ws0, self.ws0_bytes, shape,
                                                       self.alpha, 0, stream)
                    else:
                        self.ctx.conv_fused(w, self.buf[0], self.d_thr, self.buf[1], self.d_ws0, self.ws0_bytes, shape, self.alpha, 0, stream)
                elif self.fast[i]:
                    if i < last:
                        self.ctx.gemm_im2col_packed_out(w, src, dst, self.d_thr, nxt, shape, self.alpha, stream)
                    else:
                        self.ctx.gemm_im2col(w, src, self.buf[1], shape, self.alpha, self.layout, stream)
                else:
                    self.ctx.im2row_packed(True, src, self.d_a, shape, stream=stream)
                    if i < last:
                        self.ctx.gemm_packed_out(w, self.d_a, dst, self.d_thr, nxt, self.batch, L.OH, L.OW, self.alpha, stream=stream)
                    else:
                        self.ctx.gemm(w, self.d_a, self.buf[1], self.batch, L.OH, L.OW, self.alpha, self.layout, stream=stream)
            return
        for i, (L, w) in enumerate(zip(self.layers, self.weights)):
            self.ctx.conv(w, self.buf[i % 2], self.d_thr, self.buf[(i + 1) % 2], L.shape(self.batch), self.alpha, self.layout,
                          stream=stream)

    def ops(self) -> int:
        return sum(L.ops(self.batch) for L in self.layers)

    def close(self):
        for w in self.weights:
            w.free()
        for p in self.buf + [self.d_thr] + self.extra:
            self.ctx.free(p)
