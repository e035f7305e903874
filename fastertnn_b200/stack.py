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
    """reinterpret_links: the reference's driver hands every layer's output BUFFER to the next layer
    and reads it with the next layer's shape; in its model tables a few consecutive shapes do not
    chain (a pooling step the tables leave out), and the next layer then reads the first
    N*C*H*W floats of the larger buffer.  With reinterpret_links=True such links are accepted and
    behave exactly so (the link goes through fp32; chain="image" starts a new run of 4-bit images
    behind it); otherwise they are an error."""

    def __init__(self, ctx: api.Context, type_: int, layers: list[Layer], packed_weights: list[np.ndarray], batch: int,
                 threshold: float, alpha: float = 0.5, layout: int = api.NCHW, chain: str = "fp32", reinterpret_links: bool = False, use_slab: bool = True):
        assert len(layers) == len(packed_weights)
        self.link_ok = []
        for a, b in zip(layers, layers[1:]):
            ok = (a.KN, a.OH, a.OW) == (b.C, b.H, b.W)
            if not ok and not (reinterpret_links and b.C * b.H * b.W <= a.KN * a.OH * a.OW and chain in ("fp32", "image")):
                raise ValueError(f"layer output {a.KN}x{a.OH}x{a.OW} does not feed {b.C}x{b.H}x{b.W}")
            self.link_ok.append(ok)
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
        self._out = self.buf[len(layers) % 2]
        if chain == "packed":
            if layout != api.NCHW:
                raise ValueError("the packed chain is defined for NCHW input and output")
            img = max(api.packed_image_bytes(self.act_ternary, batch, L.KN, L.OH, L.OW) for L in layers)
            a = max(api.packed_bytes(type_, L.shape(batch)) for L in layers)
            self.d_img = ctx.malloc(img)
            self.d_a = ctx.malloc(a)
            self.extra = [self.d_img, self.d_a]
            self._out = self.buf[1]
        elif chain == "image":
            if layout != api.NCHW:
                raise ValueError("the image chain is defined for NCHW input and output")
            n = len(layers)
            shapes = [L.shape(batch) for L in layers]
            self.fast = [self.act_ternary and ctx.im2col_supported(w, sh) for w, sh in zip(self.weights, shapes)]
            self.run_first = [i == 0 or not self.link_ok[i - 1] for i in range(n)]
            self.run_last = [i == n - 1 or not self.link_ok[i] for i in range(n)]
            # mode of every layer = the format its input arrives in:
            #   "slab"    bordered 4-bit image (stride-1 layers; the only 4-bit form of binary activations).  Its
            #             producer is the quantise step of a run's first layer, a slab-fed predecessor whose
            #             padded lattice is this layer's (its epilogue then writes this image with its border), or --
            #             ternary activations -- an im2col-fed or dense predecessor (any stride: its epilogue places
            #             every output pixel inside the border and writes the frame)
            #   "im2col"  plain 4-bit image read through im2col tensor copies
            #   "planes"  bit planes + im2row from planes
            want_slab = [use_slab and ctx.slab_preferred(w, sh) for w, sh in zip(self.weights, shapes)]
            self.mode = []
            for i, L in enumerate(layers):
                ok = want_slab[i] and (self.run_first[i] or (self.mode[i - 1] == "slab" and
                                                            (layers[i - 1].H + 2 * layers[i - 1].P, layers[i - 1].W + 2 * layers[i - 1].P) ==
                                                            (L.H + 2 * L.P, L.W + 2 * L.P)) or
                                       (self.act_ternary and self.mode[i - 1] in ("im2col", "dense") and
                                        not (self.run_first[i - 1] and self.mode[i - 1] == "im2col" and
                                             ctx.conv_fused_preferred(self.weights[i - 1], shapes[i - 1], self.buf[0], layout))))
                # "dense": a run's first layer with few input channels (an image network's first layer) -- fp32 in, only
                # the real positions of every window multiplied (the library's dense few-channel route)
                dense = self.run_first[i] and ctx.dense_supported(self.weights[i], shapes[i])
                self.mode.append("dense" if dense else "slab" if ok else "im2col" if self.fast[i] else "planes")
            if not self.act_ternary and any(m not in ("slab",) for m in self.mode):
                raise ValueError("binary activations travel as 4-bit images only between slab-fed (stride-1, same-size) layers; use chain='packed'")
            img = max([max(api.bordered_image_bytes(batch, L.C, L.H, L.W, L.P, L.P), api.e2m1_image_bytes(batch, L.KN, L.OH, L.OW),
                           api.bordered_image_bytes(batch, L.KN, L.OH, L.OW, L.P, L.P)) for L in layers])
            self.d_imgs = [ctx.malloc(img), ctx.malloc(img)]  # ping-pong quantised activations (any format fits)
            self.extra = list(self.d_imgs)
            # a layer that starts a run (the first layer, and every layer behind a reinterpreted link)
            # reads fp32: in one launch (quantise step inside the GEMM kernel) where the library itself
            # would choose that form; its workspace holds the input's 4-bit image
            self.fuse = []
            for i, (L, w, sh) in enumerate(zip(layers, self.weights, shapes)):
                if not self.run_first[i] or self.mode[i] == "dense":
                    self.fuse.append(False)
                elif self.mode[i] == "slab":
                    self.fuse.append(bool(ctx.conv_slab_one_launch_preferred(w, sh, self.buf[0], layout)))
                else:
                    self.fuse.append(bool(self.mode[i] == "im2col" and ctx.conv_fused_preferred(w, sh, self.buf[0], layout)))
            self.fuse_first = self.fuse[0]
            self.ws0_bytes = max([max(api.fused_workspace_bytes(batch, L.C, L.H, L.W), api.slab_workspace_bytes(batch, L.C, L.H, L.W, L.P, L.P))
                                  for L, f in zip(layers, self.fuse) if f] +
                                 [api.dense_workspace_bytes(sh) for sh, m in zip(shapes, self.mode) if m == "dense"] + [0])
            if self.ws0_bytes:
                self.d_ws0 = ctx.malloc(self.ws0_bytes)
                self.extra.append(self.d_ws0)
            self.d_a = None
            if any(m == "planes" for m in self.mode):
                self.d_a = ctx.malloc(max(api.packed_bytes(type_, L.shape(batch)) for L, m in zip(layers, self.mode) if m == "planes"))
                self.extra.append(self.d_a)
            self._out = self.buf[sum(self.run_last) % 2]
        elif chain != "fp32":
            raise ValueError(chain)

    def input_ptr(self) -> int:
        return self.buf[0]

    def output_ptr(self) -> int:
        return self._out

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
            fp, k = self.buf[0], 0  # fp32 tensor the current run of layers starts from; runs finished so far
            tern = self.act_ternary
            for i, (L, w) in enumerate(zip(self.layers, self.weights)):
                shape = L.shape(self.batch)
                src, dst = self.d_imgs[i % 2], self.d_imgs[(i + 1) % 2]
                last = self.run_last[i]
                out_fp = self.buf[(k + 1) % 2]
                mode = self.mode[i]
                # what the consumer reads: bordered 4-bit image (3 ternary / 5 binary), plain 4-bit image (2), bit planes (1 / 0)
                nxt, nxt_pad = 1 if tern else 0, (0, 0)
                if not last:
                    Ln = self.layers[i + 1]
                    if self.mode[i + 1] == "slab":
                        nxt, nxt_pad = (3 if tern else 5), (Ln.P, Ln.P)
                    elif self.mode[i + 1] == "im2col":
                        nxt = 2
                if mode == "dense":
                    if not last:
                        self.ctx.conv_dense_packed_out(w, fp, self.d_thr, dst, self.d_thr, nxt, self.d_ws0, self.ws0_bytes, shape, self.alpha, self.layout, stream,
                                                       nxt_pad)
                    else:
                        self.ctx.conv_dense(w, fp, self.d_thr, out_fp, self.d_ws0, self.ws0_bytes, shape, self.alpha, self.layout, stream)
                    if last:
                        fp, k = out_fp, k + 1
                    continue
                if self.run_first[i] and not self.fuse[i]:
                    # the run's input, in the format its first layer reads
                    if mode == "slab":
                        self.ctx.quantise_e2m1_bordered(tern, fp, self.d_thr, src, self.batch, L.C, L.H, L.W, L.P, L.P, self.layout, stream)
                    elif mode == "im2col":
                        self.ctx.quantise_e2m1(fp, self.d_thr, src, self.batch, L.C, L.H, L.W, self.layout, stream)
                    else:
                        self.ctx.quantise(tern, fp, self.d_thr, src, self.batch, L.C, L.H, L.W, self.layout, stream)
                if mode == "slab":
                    if self.fuse[i]:
                        if not last:
                            self.ctx.conv_slab_packed_out(w, fp, self.d_thr, dst, self.d_thr, nxt, nxt_pad, self.d_ws0, self.ws0_bytes, shape, self.alpha, 0, stream)
                        else:
                            self.ctx.conv_slab(w, fp, self.d_thr, out_fp, self.d_ws0, self.ws0_bytes, shape, self.alpha, 0, stream)
                    elif not last:
                        self.ctx.gemm_slab_packed_out(w, src, dst, self.d_thr, nxt, nxt_pad, shape, self.alpha, stream)
                    else:
                        self.ctx.gemm_slab(w, src, out_fp, shape, self.alpha, self.layout, stream)
                elif mode == "im2col":
                    if self.fuse[i]:
                        if not last:
                            self.ctx.conv_fused_packed_out(w, fp, self.d_thr, dst, self.d_thr, nxt, self.d_ws0, self.ws0_bytes, shape, self.alpha, 0, stream)
                        else:
                            self.ctx.conv_fused(w, fp, self.d_thr, out_fp, self.d_ws0, self.ws0_bytes, shape, self.alpha, 0, stream)
                    elif not last and nxt == 3:
                        self.ctx.gemm_im2col_bordered_out(w, src, dst, self.d_thr, nxt_pad, shape, self.alpha, stream)
                    elif not last:
                        self.ctx.gemm_im2col_packed_out(w, src, dst, self.d_thr, nxt, shape, self.alpha, stream)
                    else:
                        self.ctx.gemm_im2col(w, src, out_fp, shape, self.alpha, self.layout, stream)
                else:
                    self.ctx.im2row_packed(tern, src, self.d_a, shape, stream=stream)
                    if not last:
                        self.ctx.gemm_packed_out(w, self.d_a, dst, self.d_thr, nxt, self.batch, L.OH, L.OW, self.alpha, stream=stream)
                    else:
                        self.ctx.gemm(w, self.d_a, out_fp, self.batch, L.OH, L.OW, self.alpha, self.layout, stream=stream)
                if last:
                    fp, k = out_fp, k + 1
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
