/*
 * tnns_b200 -- C ABI of the B200 (sm_100a) implementation of FasterTNN's ternary /
 * binary convolution + GEMM inference path.
 *
 * Two groups of entry points:
 *
 *  1. DROP-IN: the seven functions and two structs of the reference's CPU library,
 *     with identical names, signatures, layouts and ownership rules, so the
 *     reference's drivers (src/timing_layers.c, src/timing_gemm.c) link against
 *     libtnns_b200.so instead of tnns_cpu_mm_p2.o + mm_p2_final_*.o +
 *     {ternarize,binarize}2row_*.o.  They take HOST pointers and return malloc-family
 *     host buffers.
 *
 *  2. DEVICE-RESIDENT: tnns_cuda_* functions over device pointers and an explicit
 *     stream, for chained layers, per-kernel timing and multi-GPU sharding.  The
 *     drop-in functions are thin wrappers over these.
 *
 * All functions have C linkage and use only plain pointers, integers and floats.
 * File:line citations name the interface of the reference project
 * (fpgasystems/FasterTNN) that each declaration replaces.
 */
#ifndef TNNS_B200_H
#define TNNS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------
 * Types shared with the reference
 * ---------------------------------------------------------------------------------------- */

/* Network type: which operand is ternary (T) or binary (B); activations first.
 * Replaces include/tnns/common.h:16. */
enum tnns_type { TNN = 0, TBN = 1, BTN = 2, BNN = 3 };

/* One convolution layer invocation.  Field order and types replace
 * include/tnns/data.h:4-25 exactly (the struct crosses the boundary by pointer). */
typedef struct testcase {
    enum tnns_type type;
    int batchcount;
    int channelcount;
    int inputW;
    int inputH;
    int kernelcount;
    int kernelW;
    int kernelH;
    int paddingW;
    int paddingH;
    int strideW;
    int strideH;
    float preluAlpha;
    float* input_thresholds;            /* one symmetric threshold per image            */
    float* input;                       /* fp32 NCHW                                    */
    float* kernel;                      /* fp32 weights; not read by tnns_conv          */
    int64_t* quantized_kernel_packing0; /* not read                                     */
    int64_t* quantized_kernel_packing1; /* not read                                     */
    int64_t* quantized_kernel_packing2; /* packed weights, layout by type (see below)   */
    float* output;                      /* set by tnns_conv; caller frees with free()   */
} testcase_t;

/* One packed GEMM invocation.  Replaces include/tnns/data.h:27-41. */
typedef struct testcase_tnns_gemm {
    int m;
    int p;
    int p_packed; /* 64-bit words per plane and row */
    int n;
    float* x;
    float* w;
    int64_t* x_packing0;
    int64_t* x_packing1;
    int64_t* x_packing2;
    int64_t* w_packing0;
    int64_t* w_packing1;
    int64_t* w_packing2;
    float* output;
} testcase_tnns_gemm_t;

/*
 * Packed layouts (identical to the reference, so its host-packed weights upload
 * unchanged and packed activations can be compared with memcmp):
 *
 *   C_pack = ceil(C/64); Kw = KH*KW*C_pack; Kp = 4*ceil(Kw/4).
 *   Plane word j = (kh*KW + kw)*C_pack + ic holds channels 64*ic .. 64*ic+63 of the
 *   tap (kh,kw), channel c at bit c%64, LSB first.
 *   "packing-2" row (ternary operand): 2*Kp int64; sign word j at (j/4)*8 + j%4, zero
 *   word j four words later (alternating 256-bit sign / 256-bit zero groups).
 *   value -1: sign=1,zero=0; 0: sign=0,zero=1; +1: both 0.  Padding pixels, channels
 *   past C and the words j in [Kw,Kp) are zeros (sign=0, zero=all ones).
 *   "one-plane" row (binary operand): Kp int64, word j at j; bit=1 is -1, bit=0 is +1;
 *   padding and tails are 0 (= +1).
 */

/* ------------------------------------------------------------------------------------------
 * 1. Drop-in entry points (host pointers)
 * ---------------------------------------------------------------------------------------- */

/* Runs one layer on GPU 0 (or the device named by the environment variable
 * TNNS_B200_DEVICE; or spread by image index over the devices TNNS_B200_DEVICES lists,
 * e.g. "0,1,2,3", see tnns_cuda_multi_conv_host): quantise + pack + im2row, bitwise GEMM, PReLU.  Always sets
 * data->output to a fresh calloc'd NCHW buffer of batch*kernelcount*OH*OW floats that
 * the caller frees; on failure sets it to NULL and records an error (see
 * tnns_cuda_last_error).  Replaces include/tnns/tnns_cpu.h:4 /
 * src/tnns/tnns_cpu_mm_p2.c:83-120. */
void tnns_conv(testcase_t* data);

/* The drop-in entry points keep, per calling host thread, a context (or device group), uploaded
 * weights and page-locked staging.  They are released when the thread exits; a long-lived thread
 * can release them earlier with this call (the next drop-in call sets them up again). */
void tnns_b200_thread_shutdown(void);

/* TNN GEMM on pre-packed operands with PReLU alpha fixed to 1, as the reference's
 * final build does.  If data->output is non-NULL the m*n result is copied into it,
 * otherwise a fresh buffer is handed over.  Replaces include/tnns/tnns_cpu.h:6 /
 * src/tnns/tnns_cpu_mm_p2.c:122-133. */
void tnns_gemm(testcase_tnns_gemm_t* data);

/* Bitwise GEMM + PReLU on packed host operands; K = 64-bit words per plane BEFORE the
 * pad-to-four (buffers must already be Kp wide).  a has N*OH*OW rows, b has KN rows.
 * Returns a calloc'd NCHW float buffer or NULL.  Replace include/tnns/mm.h:5-8. */
float* mm_tnn(int64_t* a, int64_t* b, int N, int OH, int OW, int KN, int K, float prelu_alpha);
float* mm_tbn(int64_t* a, int64_t* b, int N, int OH, int OW, int KN, int K, float prelu_alpha);
float* mm_btn(int64_t* a, int64_t* b, int N, int OH, int OW, int KN, int K, float prelu_alpha);
float* mm_bnn(int64_t* a, int64_t* b, int N, int OH, int OW, int KN, int K, int K_unpack, float prelu_alpha);

/* Quantise + bit-pack + im2row of an fp32 NCHW host tensor.  Return a 32-byte aligned
 * host buffer (aligned_alloc; caller frees) of N*OH*OW rows, packing-2 (t2r_p2_opt) or
 * one-plane (b2r).  Replace include/tnns/ternarize2row.h:7 and
 * include/tnns/binarize2row.h:4. */
int64_t* t2r_p2_opt(float* x, float* q_thresholds, int N, int C, int H, int W, int H_pad, int W_pad,
                    int kH, int kW, int H_stride, int W_stride);
int64_t* b2r(float* x, float* q_thresholds, int N, int C, int H, int W, int H_pad, int W_pad, int kH,
             int kW, int H_stride, int W_stride);

/* Host-side weight packers, run once per model: fp32 [KN][C][KH][KW] plus one
 * threshold per kernel -> packing-2 rows (ternary) or one-plane rows (binary).
 * Buffers come from aligned_alloc(32, ..); caller frees.  Replace
 * ternarize_opt_avx2 / binarize_opt_avx2 (include/utils.h:22,27; src/utils.c:468-521,
 * 634-675). */
int64_t* tnns_pack_weights_ternary(const float* w, const float* thresholds, int KN, int C, int KH, int KW);
int64_t* tnns_pack_weights_binary(const float* w, const float* thresholds, int KN, int C, int KH, int KW);

/* ------------------------------------------------------------------------------------------
 * 2. Device-resident API
 * ---------------------------------------------------------------------------------------- */

typedef struct tnns_cuda_ctx tnns_cuda_ctx;         /* per (host thread, device) state   */
typedef struct tnns_cuda_weights tnns_cuda_weights; /* device copy of one packed kernel  */

/* Geometry of one layer; the same quantities as the testcase_t fields. */
typedef struct tnns_shape {
    int N, C, H, W;  /* input batch, channels, height, width   */
    int KN, KH, KW;  /* kernels, kernel height, kernel width   */
    int PH, PW;      /* zero padding                           */
    int SH, SW;      /* strides                                */
} tnns_shape_t;

/* Memory layout of the fp32 activation tensors at the device boundary. */
enum tnns_layout { TNNS_NCHW = 0, TNNS_NHWC = 1 };

/* Kernel selection.  AUTO picks per shape; the others force one implementation (used
 * by tests to cross-check them and by the benchmark to compare them). */
enum tnns_pack_algo { TNNS_PACK_AUTO = 0, TNNS_PACK_GATHER = 1, TNNS_PACK_STAGED = 2 };
enum tnns_gemm_algo {
    TNNS_GEMM_AUTO = 0,
    TNNS_GEMM_POPC_SIMPLE = 1, /* one thread per output, integer pipe            */
    TNNS_GEMM_POPC_TILED = 2,  /* tiled carry-save popcount GEMM, integer pipe   */
    TNNS_GEMM_I8_TC = 3,       /* tcgen05 int8 tensor-core GEMM                  */
    TNNS_GEMM_F4_TC = 4,       /* tcgen05 4-bit (e2m1, unit scales) tensor-core GEMM */
    TNNS_GEMM_F4_FUSED = 5,    /* whole layers only: the 4-bit GEMM fed by tensor copies with the quantise step in the same launch */
    TNNS_GEMM_F4_SLAB = 6,     /* whole stride-1 layers only: bordered 4-bit image, then the slab-fed 4-bit GEMM */
    TNNS_GEMM_F4_SLAB_FUSED = 7, /* the same as one launch */
    TNNS_GEMM_F4_DENSE = 8     /* whole layers with few input channels: only the real positions of a window, as a 1x1 layer */
};

/* Error codes returned by every tnns_cuda_* function (0 = success). */
enum tnns_status {
    TNNS_OK = 0,
    TNNS_ERR_INVALID = 1,     /* NULL pointer, non-positive dimension, kernel larger than image .. */
    TNNS_ERR_CUDA = 2,        /* a CUDA runtime call failed; see tnns_cuda_error_detail           */
    TNNS_ERR_NOMEM = 3,       /* host or device allocation failed                                 */
    TNNS_ERR_UNSUPPORTED = 4, /* the forced algorithm cannot run this shape                       */
    TNNS_ERR_DEVICE_WAIT = 5  /* a bounded on-device wait expired (kernel returned early)         */
};

int tnns_cuda_create(int device, tnns_cuda_ctx** ctx);
void tnns_cuda_destroy(tnns_cuda_ctx* ctx);

/* Derived sizes.  K words are 64-bit words per plane and row. */
int tnns_out_dim(int in, int pad, int k, int stride); /* src/tnns/tnns_cpu_mm_p2.c:7-10 */
int tnns_k_words(int C, int KH, int KW);              /* Kw                              */
int tnns_k_padded(int C, int KH, int KW);             /* Kp                              */
/* Bytes of the packed im2row matrix for this type and shape. */
size_t tnns_packed_bytes(int type, const tnns_shape_t* s);

/* Copies packed weights (host or device memory; reference layout for `type`: packing-2 for TNN/BTN,
 * one-plane for TBN/BNN) to the device and prepares the per-kernel constants and the
 * operand images the GEMM kernels need.  Done once per layer. */
int tnns_cuda_upload_weights(tnns_cuda_ctx* ctx, int type, const int64_t* packed_host, int KN, int C, int KH,
                             int KW, tnns_cuda_weights** out);
/* Weight packing on the device: fp32 [KN][C][KH][KW] and one threshold per kernel, both in device
 * memory, -> packed rows in d_packed (KN * Kp * 8 bytes, doubled for ternary), the same bytes as
 * tnns_pack_weights_ternary / _binary produce on the host (src/utils.c:468-521, 634-675).
 * tnns_cuda_upload_weights accepts the result (its `packed` pointer may be host or device). */
int tnns_cuda_pack_weights(tnns_cuda_ctx* ctx, int ternary, const float* d_w, const float* d_thr, int64_t* d_packed, int KN, int C,
                           int KH, int KW, void* stream);

/* Same for callers that hold only a packed operand (the mm_* functions): KN rows of
 * K_words plane words (before the pad-to-four; the buffer is Kp wide), K_unpack =
 * number of elements per row before any padding (used by BNN only).  Weights uploaded
 * this way serve tnns_cuda_gemm; tnns_cuda_conv rejects them. */
int tnns_cuda_upload_weights_packed(tnns_cuda_ctx* ctx, int type, const int64_t* packed_host, int KN, int K_words,
                                    int K_unpack, tnns_cuda_weights** out);
void tnns_cuda_free_weights(tnns_cuda_ctx* ctx, tnns_cuda_weights* w);

/* Quantise + pack + im2row on the device.  ternary != 0: packing-2 rows (t2r_p2_opt
 * semantics), else one-plane rows (b2r semantics).  d_x: fp32 in `layout`; d_thr: N
 * floats; d_packed: tnns_packed_bytes() bytes, 16-byte aligned.  `stream` is a
 * cudaStream_t passed as void* (NULL = default stream).  Asynchronous. */
int tnns_cuda_pack(tnns_cuda_ctx* ctx, int ternary, const float* d_x, const float* d_thr, int64_t* d_packed,
                   const tnns_shape_t* s, int layout, int algo, void* stream);

/* Bitwise GEMM + PReLU on the device: d_a is the packed im2row matrix of N*OH*OW rows
 * in the layout the weights' type expects; d_y receives N*KN*OH*OW floats in `layout`
 * (NCHW: ((n*KN+kn)*OH+oh)*OW+ow as include/tnns/mm.h:30; NHWC: row-major rows x KN).
 * Asynchronous. */
int tnns_cuda_gemm(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const int64_t* d_a, float* d_y, int N, int OH,
                   int OW, float alpha, int layout, int algo, void* stream);

/* Whole layer on the device: pack into the context's workspace (grown with cudaMalloc
 * when too small), then GEMM + PReLU.  Asynchronous unless the workspace grows. */
int tnns_cuda_conv(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y,
                   const tnns_shape_t* s, float alpha, int layout, int pack_algo, int gemm_algo, void* stream);

/* Same with a caller-owned workspace.  Every route needs only what it writes there, and with
 * TNNS_PACK_AUTO / TNNS_GEMM_AUTO the call takes the best route the workspace holds: the
 * copy-engine routes keep a 4-bit image (tnns_fused_workspace_bytes, tnns_slab_workspace_bytes;
 * 128-byte aligned), the gathering route bit planes (tnns_packed_image_bytes), the explicit route --
 * the only one a forced pack or GEMM algorithm takes -- the packed im2row matrix
 * (tnns_packed_bytes).  A workspace of the largest of these that applies never limits the choice. */
int tnns_cuda_conv_ws(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr,
                      float* d_y, void* d_workspace, size_t workspace_bytes, const tnns_shape_t* s, float alpha,
                      int layout, int pack_algo, int gemm_algo, void* stream);

/* Chained layers without the fp32 round trip (the reference chains layers through fp32 host
 * buffers, src/timing_layers.c:188-201; every layer re-quantises its input).  Between two
 * layers only the quantised activations matter, so the GEMM can emit them directly:
 *
 *   "packed image" of an N x C x H x W activation tensor: bit planes [n][plane][pixel][ic] of
 *   64-bit words, pixel = ih*W + iw, ic = 64-channel group, plane 0 sign, plane 1 zero (ternary
 *   only), same bit meaning as the packed layouts above; tnns_packed_image_bytes() bytes.
 *
 * tnns_cuda_gemm_packed_out: GEMM + PReLU of the current layer whose epilogue quantises each
 * output with d_thr_next[n] (ternary: sign = y < -t, zero = !(y < -t || y > t); binary: y < t)
 * and writes the packed image of the N x KN x OH x OW result -- bit-identical to packing the fp32
 * output.  tnns_cuda_im2row_packed: packed image -> im2row matrix of the next layer (the same
 * bytes tnns_cuda_pack would produce from the fp32 tensor).  Both asynchronous. */
size_t tnns_packed_image_bytes(int ternary, int N, int C, int H, int W);
/* Quantise only: fp32 tensor in `layout` -> packed image (the first half of t2r_p2_opt / b2r,
 * src/tnns/ternarize2row_avx2.c:438-452, src/tnns/binarize2row_avx2.c:15-22, without the
 * im2row scatter).  d_image: tnns_packed_image_bytes() bytes, 32-byte aligned. */
int tnns_cuda_quantise(tnns_cuda_ctx* ctx, int ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                       int W, int layout, void* stream);
/* GEMM + PReLU that gathers the im2row rows of layer `s` itself from the packed image of the
 * layer's input (implicit im2row: the KH*KW-times larger im2row matrix is never materialised).
 * Same result as tnns_cuda_pack + tnns_cuda_gemm.  tnns_cuda_conv takes this route by default. */
int tnns_cuda_gemm_implicit(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const tnns_shape_t* s,
                            float alpha, int layout, void* stream);
/* The same route with the copy engine doing the gather (ternary activations; 64-channel groups per
 * pixel: 1, 2 or a multiple of 4; tnns_cuda_im2col_supported says whether a layer qualifies).  tnns_cuda_quantise_e2m1 writes the
 * quantised input as a 4-bit operand image, [n][pixel][C/2 bytes] with {-1,0,+1} as e2m1 nibbles
 * (tnns_e2m1_image_bytes() bytes, 32-byte aligned); tnns_cuda_gemm_im2col then receives every
 * 128-pixel activation tile of a filter tap (256, 128 or 64 channels) as one im2col tensor copy (zero fill
 * outside the image = the reference's padding value, src/tnns/ternarize2row_avx2.c:438-452)
 * straight into the layout the tensor core reads: no warp expands or gathers anything.  Same
 * result as tnns_cuda_pack + tnns_cuda_gemm; tnns_cuda_conv prefers this route where it applies.
 * pairs: 1 = one block per 128-row tile; 2 = block pairs (two SMs share a 256-row tile through
 * tcgen05.mma.cta_group::2, each holding half of the weight tile; layers with more than 128
 * kernels); 0 = pairs once there are enough 256-row tiles for every SM pair. */
size_t tnns_e2m1_image_bytes(int N, int C, int H, int W);
int tnns_cuda_im2col_supported(const tnns_cuda_weights* w, const tnns_shape_t* s);
int tnns_cuda_quantise_e2m1(tnns_cuda_ctx* ctx, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H, int W,
                            int layout, void* stream);
int tnns_cuda_gemm_im2col(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const tnns_shape_t* s,
                          float alpha, int layout, int pairs, void* stream);
/* The copy-engine route as ONE launch (t2r_p2_opt's thresholding, src/tnns/ternarize2row_avx2.c:438-452,
 * and mm_tnn / mm_tbn, src/tnns/mm_p2_final_tnn_avx2.c:384-387, in one kernel): beside the GEMM's
 * warps every block runs quantiser warps that turn the fp32 input into the 4-bit operand image,
 * 128 pixels x 64 channels at a time in image order, and count finished pieces per image in global
 * memory; a tile's tensor copies start once the images of its rows are complete, so the
 * HBM-bound quantisation runs underneath the tensor-bound MMAs of earlier tiles.  Needs what
 * tnns_cuda_gemm_im2col needs plus NCHW input with H*W a multiple of four and a 16-byte aligned
 * d_x (tnns_cuda_conv_fused_supported).  d_workspace: tnns_fused_workspace_bytes() bytes, 128-byte
 * aligned (image + synchronisation words).  The context owns a second set of synchronisation words,
 * bound to the first stream that makes such a call and left zeroed by every launch; calls on that
 * stream use them and may overlap their set-up with the previous such launch's tail, calls on any
 * other stream use the words in the workspace, which the call clears on `stream` first.  The first
 * call may allocate those words (and synchronise the device); keep it out of stream capture.  Same
 * result as every other route.  tnns_cuda_conv / _conv_ws take it with gemm_algo
 * TNNS_GEMM_F4_FUSED, and with TNNS_GEMM_AUTO where the layer has at least three tiles per SM. */
size_t tnns_fused_workspace_bytes(int N, int C, int H, int W);
int tnns_cuda_conv_fused_supported(const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout);
int tnns_cuda_conv_fused(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y,
                         void* d_workspace, size_t workspace_bytes, const tnns_shape_t* s, float alpha, int pairs, void* stream);
/* 1 where tnns_cuda_conv with TNNS_GEMM_AUTO takes that route by itself (the layer qualifies and
 * every SM has at least three 128-row tiles), else 0. */
int tnns_cuda_conv_fused_preferred(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout);
/* The same launch as the first layer of a chain (src/timing_layers.c:188-201 chains layers through fp32
 * buffers): fp32 input in, and instead of the fp32 output the next layer's quantised activations
 * (d_image_out, d_thr_next, next_format as for tnns_cuda_gemm_im2col_packed_out below). */
int tnns_cuda_conv_fused_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr,
                                    void* d_image_out, const float* d_thr_next, int next_format, void* d_workspace,
                                    size_t workspace_bytes, const tnns_shape_t* s, float alpha, int pairs, void* stream);
/* Stride-1 layers from a BORDERED 4-bit image (t2r_p2_opt / b2r scatter every packed pixel to the
 * KH*KW windows that use it, src/tnns/ternarize2row_avx2.c:285-313, src/tnns/binarize2row_avx2.c:131-199;
 * here no window is ever materialised).  The image keeps the layer's padding around every image:
 * [n][H + 2*PH][W + 2*PW][C/2 bytes] (tnns_e2m1_bordered_image_bytes), border pixels = the padding
 * value -- ternary 0, binary +1 (b2r pads with zero bits, src/tnns/binarize2row_avx2.c:146-151) -- so all
 * four network types qualify.  Output rows are laid over the padded lattice, and the 128 rows of a
 * tile read, for filter tap (kh, kw), 128 consecutive pixels of the image starting kh*(W+2*PW) + kw
 * further on: ONE tiled tensor copy of 128 + (KH-1)*(W+2*PW) + KW-1 pixels per tile and 256-channel
 * group serves every tap, the tensor core reading each tap as a row-shifted view of that slab
 * (rows on border positions are computed and not stored).  Needs stride 1 and 64, 128 or a multiple
 * of 256 channels (after rounding to 64): tnns_cuda_slab_supported.
 *   tnns_cuda_quantise_e2m1_bordered  fp32 NCHW (H*W a multiple of four) or NHWC (C a multiple of four, at least
 *                                     128 pixels in all) -> bordered image, 128-byte aligned
 *   tnns_cuda_gemm_slab               bordered image -> fp32 output (same result as every other route)
 *   tnns_cuda_gemm_slab_packed_out    the same with the quantising epilogue: next_format 0 / 1 bit planes
 *                                     (binary / ternary), 2 plain 4-bit image, 3 bordered 4-bit image for a
 *                                     ternary next layer with padding (next_PH, next_PW), 5 the same for a
 *                                     binary next layer.  Formats 3 / 5 need the next layer's padded size to
 *                                     equal this layer's (a same-size stride-1 chain); the rows on border
 *                                     positions then write the next image's border, so the whole image is
 *                                     rewritten by every launch.
 *   tnns_cuda_conv_slab(_packed_out)  ONE launch: quantiser warps write the bordered image inside the GEMM
 *                                     kernel (workspace: tnns_slab_workspace_bytes, 128-byte aligned; the
 *                                     synchronisation words follow the rules of tnns_cuda_conv_fused).
 * tnns_cuda_conv / _conv_ws take these routes with gemm_algo TNNS_GEMM_F4_SLAB / _SLAB_FUSED. */
size_t tnns_e2m1_bordered_image_bytes(int N, int C, int H, int W, int PH, int PW);
size_t tnns_slab_workspace_bytes(int N, int C, int H, int W, int PH, int PW);
int tnns_cuda_slab_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s);
/* 1 where the library's own rule (tnns_cuda_conv with TNNS_GEMM_AUTO) takes the slab-fed route for this layer. */
int tnns_cuda_slab_preferred(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s);
/* The tnns_gemm_algo that tnns_cuda_conv / _conv_ws resolve TNNS_GEMM_AUTO to for this layer and input
 * (workspace permitting): _F4_SLAB_FUSED, _F4_SLAB, _F4_FUSED, or _F4_TC for the two-launch forms. */
int tnns_cuda_conv_auto_algo(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout);
int tnns_cuda_conv_slab_one_launch_preferred(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout);
int tnns_cuda_conv_slab_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s, const float* d_x, int layout);
int tnns_cuda_quantise_e2m1_bordered(tnns_cuda_ctx* ctx, int ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                                     int W, int PH, int PW, int layout, void* stream);
int tnns_cuda_gemm_slab(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const tnns_shape_t* s, float alpha,
                        int layout, int pairs, void* stream);
int tnns_cuda_gemm_slab_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, void* d_image_out, const float* d_thr_next,
                                   int next_format, int next_PH, int next_PW, const tnns_shape_t* s, float alpha, int pairs, void* stream);
int tnns_cuda_conv_slab(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y, void* d_workspace,
                        size_t workspace_bytes, const tnns_shape_t* s, float alpha, int pairs, void* stream);
int tnns_cuda_conv_slab_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, void* d_image_out,
                                   const float* d_thr_next, int next_format, int next_PH, int next_PW, void* d_workspace, size_t workspace_bytes,
                                   const tnns_shape_t* s, float alpha, int pairs, void* stream);
/* Layers with few input channels (C <= 16: the first layer of an image network), no reference counterpart.
 * The reference pads every filter tap to 64 channels (src/tnns/ternarize2row_avx2.c:285-313); here the
 * window's KH*KW*C real positions form the row of a virtual 1x1 layer (rounded up to 64, 128 or a multiple
 * of 256 "channels"), whose packed kernel is derived once at upload: tnns_cuda_conv_dense quantises the
 * fp32 input (either layout) straight into that layer's 4-bit image -- tnns_dense_workspace_bytes, 128-byte
 * aligned -- and runs the copy-engine fed GEMM on it.  Same output bits as every other route.  Ternary
 * activations (TNN, TBN); tnns_cuda_dense_supported tells whether a layer qualifies.  _packed_out writes
 * the next layer's quantised activations instead (next_format 0 / 1 bit planes, 2 plain 4-bit image, 3 the 4-bit
 * image bordered by next_PH rows / next_PW columns for a slab-fed next layer).
 * tnns_cuda_conv / _conv_ws take this route by themselves (TNNS_GEMM_F4_DENSE asks for it). */
size_t tnns_dense_workspace_bytes(const tnns_shape_t* s);
int tnns_cuda_dense_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const tnns_shape_t* s);
int tnns_cuda_conv_dense(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, float* d_y, void* d_workspace,
                         size_t workspace_bytes, const tnns_shape_t* s, float alpha, int layout, void* stream);
int tnns_cuda_conv_dense_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* d_x, const float* d_thr, void* d_image_out,
                                    const float* d_thr_next, int next_format, int next_PH, int next_PW, void* d_workspace,
                                    size_t workspace_bytes, const tnns_shape_t* s, float alpha, int layout, void* stream);
/* Chaining on the copy-engine route: the same GEMM with the quantising epilogue of
 * tnns_cuda_gemm_packed_out.  next_format (also accepted as `next_ternary` by
 * tnns_cuda_gemm_packed_out): 0 = binary bit planes, 1 = ternary bit planes, 2 = ternary 4-bit
 * operand image (tnns_e2m1_image_bytes(N, KN, OH, OW) bytes) -- what tnns_cuda_gemm_im2col of the
 * next layer reads, so a stack of qualifying layers runs as one GEMM per layer with nothing but
 * 4-bit images in between. */
int tnns_cuda_gemm_im2col_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, void* d_image_out,
                                     const float* d_thr_next, int next_format, const tnns_shape_t* s, float alpha, int pairs,
                                     void* stream);
/* The same producer writing the 4-bit image BORDERED (tnns_e2m1_bordered_image_bytes(N, KN, OH, OW, next_PH, next_PW) bytes,
 * 128-byte aligned): what a slab-fed next layer with padding (next_PH, next_PW) reads.  Any layer the im2col GEMM
 * takes can produce it -- strided ones too -- each output pixel going to its place inside the border, and the
 * frame (zeros) written by the same launch. */
int tnns_cuda_gemm_im2col_bordered_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, void* d_image_out,
                                       const float* d_thr_next, int next_PH, int next_PW, const tnns_shape_t* s, float alpha, int pairs,
                                       void* stream);
int tnns_cuda_gemm_packed_out(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const int64_t* d_a, void* d_image,
                              const float* d_thr_next, int next_ternary, int N, int OH, int OW, float alpha, void* stream);
int tnns_cuda_im2row_packed(tnns_cuda_ctx* ctx, int ternary, const void* d_image, int64_t* d_packed, const tnns_shape_t* s,
                            void* stream);

/* Whole layer with HOST input / output buffers (the device-side half of tnns_conv,
 * src/tnns/tnns_cpu_mm_p2.c:83-120): the batch is cut into slices whose upload, kernels and
 * download overlap on three streams; page-locked buffers (tnns_cuda_malloc_host, cudaHostAlloc,
 * cudaHostRegister) give full PCIe speed.  Synchronous: returns when h_y is complete. */
int tnns_cuda_conv_host(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const float* h_x, const float* h_thr,
                        float* h_y, const tnns_shape_t* s, float alpha, int layout);

/* ---- One host batch over several GPUs ------------------------------------------------------
 * The reference's tnns_conv (src/tnns/tnns_cpu_mm_p2.c:83-120) receives ONE host batch and works
 * through its rows one after the other (include/tnns/mm.h:22-31: no state is carried from row to
 * row).  These entry points take the same host batch and spread it over G devices by image index:
 * shard g owns the images tnns_shard_range gives it -- contiguous slices of input and output --
 * the packed weights are uploaded to every device once, and no data moves between devices.
 * One host thread per device, all released together by a start barrier.
 *
 * Failure handling is per shard: a shard that fails does not stop the others.  The call returns
 * the first failing shard's status (TNNS_OK if none), shard_status[g] (may be NULL) receives every
 * shard's own, and tnns_cuda_error_detail() names the failed shards; the slices of h_y that belong
 * to successful shards are complete. */
typedef struct tnns_cuda_multi tnns_cuda_multi;                 /* a group of devices, one context each */
typedef struct tnns_cuda_multi_weights tnns_cuda_multi_weights; /* one layer's weights on every device  */
/* [n0, n1) = images of shard `shard` of `shards`; the first N % shards shards own one image more. */
void tnns_shard_range(int N, int shard, int shards, int* n0, int* n1);
/* The host-side engine by itself: runs fn(shard, shards, n0, n1, arg) on `shards` host threads (the
 * caller's thread is shard 0) behind a start barrier and collects the return values as statuses. */
typedef int (*tnns_shard_fn)(int shard, int shards, int n0, int n1, void* arg);
int tnns_shard_run(int shards, int N, tnns_shard_fn fn, void* arg, int* shard_status);
int tnns_cuda_multi_create(const int* devices, int count, tnns_cuda_multi** out);
void tnns_cuda_multi_destroy(tnns_cuda_multi* m);
int tnns_cuda_multi_device_count(const tnns_cuda_multi* m);
tnns_cuda_ctx* tnns_cuda_multi_context(const tnns_cuda_multi* m, int index); /* shard `index`'s context */
int tnns_cuda_multi_upload_weights(tnns_cuda_multi* m, int type, const int64_t* packed_host, int KN, int C, int KH, int KW,
                                   tnns_cuda_multi_weights** out);
void tnns_cuda_multi_free_weights(tnns_cuda_multi* m, tnns_cuda_multi_weights* w);
/* tnns_cuda_conv_host over the group: HOST buffers in and out (page-locked ones, allocated as
 * portable, move at full speed on every device), synchronous.  The drop-in tnns_conv takes this
 * path when the environment variable TNNS_B200_DEVICES lists more than one device ("0,1,2,3"). */
int tnns_cuda_multi_conv_host(tnns_cuda_multi* m, const tnns_cuda_multi_weights* w, const float* h_x, const float* h_thr, float* h_y,
                              const tnns_shape_t* s, float alpha, int layout, int* shard_status);

/* Whole layer for callers that must not allocate (no counterpart in the reference, which
 * has no device and no allocator constraints).  Meant for hosts that cannot call
 * cudaMalloc: servers that give all device memory to their own arena at start-up,
 * plug-ins living inside another framework's caching allocator, or latency-critical
 * loops where an allocation, which may synchronise the device, is forbidden.
 *
 * The packed im2row matrix is kept in a fixed array of TNNS_NOALLOC_SCRATCH_BYTES bytes
 * that is part of the library image: a GPU holds that much memory from the moment the
 * array's module is loaded on it until the process exits.  With CUDA's default lazy module
 * loading that is the first call of this function on the device, with
 * CUDA_MODULE_LOADING=EAGER the creation of the CUDA context.  So make one start-up call per
 * device -- an empty batch (s->N == 0) is enough and launches nothing -- BEFORE your arena
 * takes the device's memory; a first call that finds no room left returns TNNS_ERR_NOMEM.
 * After that call no later call changes the amount of free device memory.
 * A layer whose packed matrix
 * (tnns_packed_bytes) is larger is refused with TNNS_ERR_UNSUPPORTED and a message that
 * names both sizes; split the batch or use tnns_cuda_conv_ws.
 *
 * No context and no weights handle are needed: d_packed_weights is a device pointer to
 * the kernel rows in the reference layout for `type` (16-byte aligned), d_x / d_thr /
 * d_y are the caller's device buffers as for tnns_cuda_conv.  The work runs on the
 * CURRENT device, which must own all four pointers.  The call itself uses no cudaMalloc,
 * cudaFree or other allocating routine.  The first call on each device (empty batches
 * included) also looks up the device address of the scratch array and two device
 * attributes; make that first call outside of any stream capture.
 *
 * All calls on a device share the one scratch array.  Nothing in it needs to start at
 * zero (every call rewrites all of the rows it then reads), but two calls that can run
 * at the same time on the GPU -- different streams, or different host threads -- race on
 * it: order them on one stream or with events.  Asynchronous. */
#define TNNS_NOALLOC_SCRATCH_BYTES (32u << 20)
size_t tnns_cuda_noalloc_scratch_bytes(void);
int tnns_cuda_conv_noalloc(int type, const int64_t* d_packed_weights, const float* d_x, const float* d_thr, float* d_y,
                           const tnns_shape_t* s, float alpha, int layout, void* stream);

/* Blocks until all work submitted through ctx's own streams has finished and reports
 * any asynchronous error, including the on-device status word. */
int tnns_cuda_sync(tnns_cuda_ctx* ctx);

/* Self-test of the on-device failure detection: every mbarrier wait inside the kernels is bounded
 * (about one second); this launches a one-warp kernel whose wait can never be satisfied, so that
 * the following tnns_cuda_sync returns TNNS_ERR_DEVICE_WAIT.  The kernel returns normally and the
 * context remains usable. */
int tnns_cuda_selftest_wait_expiry(tnns_cuda_ctx* ctx);

/* The rule of the quantising epilogues, on the host (no GPU needed; no reference counterpart).  A layer
 * that writes the next layer's quantised activations applies, for 0 < alpha <= 1, thresholds to its raw
 * integer accumulator v instead of evaluating PReLU(v + bias) first:
 *     sign bit = (v + *n1 < 0)      above = (*t2 - v < 0)      ternary non-zero = sign | above
 * which equals the reference's PReLU (src/tnns/mm_p2_final_tnn_avx2.c:90-93) followed by its quantisers
 * (src/tnns/ternarize2row_avx2.c:438-452, src/tnns/binarize2row_avx2.c:19-21) for every integer v below
 * 2^22 in magnitude.  This returns the two constants the kernels derive from a next-layer threshold t,
 * so that the equivalence can be checked exhaustively on a CPU.  ternary = 0: *t2 is 0 and unused. */
int tnns_prelu_thresholds(float t, float alpha, float bias, int ternary, float* n1, float* t2);

/* Plain device-memory helpers so that C callers need no CUDA headers.  Synchronous. */
int tnns_cuda_malloc(tnns_cuda_ctx* ctx, size_t bytes, void** out);
/* Free and total bytes of device memory on the context's device (cudaMemGetInfo). */
int tnns_cuda_mem_info(tnns_cuda_ctx* ctx, size_t* free_bytes, size_t* total_bytes);
void tnns_cuda_free(tnns_cuda_ctx* ctx, void* p);
/* Page-locked host memory (cudaHostAlloc, portable + mapped): the buffers tnns_cuda_conv_host
 * moves at full PCIe speed. */
int tnns_cuda_malloc_host(tnns_cuda_ctx* ctx, size_t bytes, void** out);
void tnns_cuda_free_host(tnns_cuda_ctx* ctx, void* p);
int tnns_cuda_memcpy_h2d(tnns_cuda_ctx* ctx, void* dst, const void* src, size_t bytes);
int tnns_cuda_memcpy_d2h(tnns_cuda_ctx* ctx, void* dst, const void* src, size_t bytes);

/* Measurement utility: issue rate of one instruction kind over the whole GPU.
 * op 0 = LOP3, 1 = POPC, 2 = IADD: 1e9 thread-instructions per second, the denominator for
 * "fraction of the integer pipe" figures of the popcount GEMM.
 * op 3 = tcgen05.mma kind::i8, 4 = tcgen05.mma kind::mxf4: 1e9 operations (2*M*N*K) per second
 * of an issue-bound loop of 128 x 256 MMAs on operands resident in shared memory (no loads,
 * no epilogue): the tensor-pipe denominator for the tensor-core GEMMs. */
int tnns_cuda_pipe_rate(tnns_cuda_ctx* ctx, int op, double* giga_per_s);

/* Number of kernels this library has launched in the calling thread since load. */
unsigned long long tnns_cuda_launch_count(void);

/* Last error of the calling thread (sticky until the next failing call). */
int tnns_cuda_last_error(void);
const char* tnns_cuda_strerror(int status);
const char* tnns_cuda_error_detail(void);

#ifdef __cplusplus
}
#endif
#endif /* TNNS_B200_H */
