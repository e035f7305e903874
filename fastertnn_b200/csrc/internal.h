// Internal declarations shared by the CUDA translation units of libtnns_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "tnns_b200.h"

#define TNNS_WORD_BITS 64

// Everything a kernel needs to know about one layer's geometry.
struct TnnsGeom {
    int N, C, H, W;
    int KN, KH, KW;
    int PH, PW, SH, SW;
    int OH, OW;
    int Cp;  // 64-channel groups per pixel
    int Kw;  // plane words per row before padding
    int Kp;  // plane words per row, multiple of four
};

struct tnns_cuda_ctx {
    int device;
    int sm_count;
    size_t smem_optin;          // max dynamic shared memory per block
    void* workspace;            // packed im2row matrix for tnns_cuda_conv
    size_t workspace_bytes;
    unsigned int* d_status;     // device status word (bounded waits report here)
    unsigned int* h_status;     // pinned mirror
    cudaStream_t s_copy_in, s_compute, s_copy_out;  // used by tnns_cuda_conv_host
    cudaEvent_t ev_in[2], ev_done[2], ev_out[2];
    void* stage_in[2];          // device staging for host-buffer convs
    void* stage_out[2];
    void* stage_pack[2];
    float* stage_thr;
    size_t stage_in_bytes, stage_out_bytes, stage_pack_bytes, stage_thr_count;
    // synchronisation words of the one-launch layer kernel: zero between launches (the kernel clears
    // them on its way out), used by launches on the one stream they are bound to
    unsigned int* fused_sync;
    size_t fused_sync_words;
    cudaStream_t fused_sync_stream;
};

struct tnns_cuda_weights {
    int type;
    int KN, C, KH, KW;
    int Cp, Kw, Kp;
    int K_unpack;         // elements per row before any padding (BNN needs it)
    int device;
    uint64_t* d_packed;   // reference layout for `type`
    size_t packed_bytes;
    int8_t* d_i8;         // {-1,0,+1} operand image for the tensor-core GEMM (may be NULL)
    size_t i8_bytes;
    int i8_kchunks;       // number of 128-element K chunks in d_i8
    uint8_t* d_f4;        // e2m1 operand image for the 4-bit tensor-core GEMM (may be NULL)
    size_t f4_bytes;
    uint32_t* d_jtab;     // plane word j -> kh<<24 | kw<<16 | ic (implicit im2row), NULL without layer geometry
    // layers with few input channels: the same kernel as a 1x1 layer over only the real positions of a window
    // (dense.cu), NULL where that form does not apply
    tnns_cuda_weights* dense;
};

// error plumbing (thread local)
int tnns_fail(int status, const char* fmt, ...);
void tnns_count_launch(void);
#define TNNS_CUDA_TRY(expr)                                                                      \
    do {                                                                                         \
        cudaError_t err__ = (expr);                                                              \
        if (err__ != cudaSuccess)                                                                \
            return tnns_fail(err__ == cudaErrorMemoryAllocation ? TNNS_ERR_NOMEM : TNNS_ERR_CUDA, \
                             "%s failed: %s", #expr, cudaGetErrorString(err__));                 \
    } while (0)

int tnns_make_geom(const tnns_shape_t* s, TnnsGeom* g);

// kernel launchers (all asynchronous on `stream`)
int tnns_launch_pack(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_packed,
                     const TnnsGeom& g, int layout, int algo, cudaStream_t stream);
int tnns_launch_gemm_popc(tnns_cuda_ctx* ctx, int type, const void* d_a, const void* d_b, float* d_y, long long M,
                          int KN, int Kp, int OHW, int K_unpack, float alpha, int layout, bool tiled,
                          cudaStream_t stream);

// tensor-core path (gemm_i8_tc.cu)
int tnns_i8_tile_n(int KN);
int tnns_build_i8_weights(tnns_cuda_ctx* ctx, tnns_cuda_weights* w);
// d_pimg != NULL: write the next layer's quantised bit planes instead of fp32 (d_y unused)
int tnns_launch_gemm_tc(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_a, float* d_y, long long M, int OHW, float alpha,
                        int layout, bool f4, cudaStream_t stream, void* d_pimg = nullptr, const float* d_thr_next = nullptr,
                        int next_ternary = 1, const TnnsGeom* implicit_geom = nullptr);
// implicit_geom != NULL: d_a is the quantised image [n][plane][pixel][ic] of the layer input and
// the kernel gathers the im2row rows itself (4-bit form only)
#define TNNS_SRC_PACKED_IMAGE 2  // internal "layout" of tnns_launch_pack: input is already bit planes
// quantise only (no im2row): fp32 tensor -> packed image, in one of two formats
//   TNNS_IMG_PLANES  bit planes [n][plane][pixel][ic], one 64-bit word per 64 channels
//   TNNS_IMG_E2M1    4-bit operand image [n][pixel][ic][32 bytes]: the 64 channels of a group as the
//                    e2m1 nibbles tnns_expand32_f4 makes of the low and the high half of its plane
//                    words -- exactly the bytes the 4-bit GEMM keeps in shared memory, so a tensor
//                    copy can deliver im2row tiles without any expansion (ternary activations only)
#define TNNS_IMG_PLANES 1
#define TNNS_IMG_E2M1 2
int tnns_launch_quantise(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                         int W, int layout, cudaStream_t stream, int format = TNNS_IMG_PLANES);
// the same for NCHW input whose rows the copy engine can fetch (H*W a multiple of four floats,
// 16-byte aligned base): tensor copies into a shared-memory ring instead of register loads
bool tnns_quantise_tma_supported(const float* d_x, int H, int W, int layout);
// PH, PW (4-bit image only): store the image bordered, i.e. every image framed by PH rows / PW columns of
// the padding value (ternary 0, binary +1), [n][H + 2*PH][W + 2*PW][C/2 bytes]
// layout TNNS_NHWC: the input is (pixels) x (channels), fetched as 128-byte-swizzled boxes (tnns_quantise_tma_nhwc_supported)
bool tnns_quantise_tma_nhwc_supported(const float* d_x, int N, int C, int H, int W);
int tnns_launch_quantise_tma(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                             int W, cudaStream_t stream, int format, int PH = 0, int PW = 0, int layout = TNNS_NCHW);
// dense form of layers with few input channels (dense.cu): channels of the virtual 1x1 layer, whether a kernel
// qualifies, the repacked kernel of that layer, and the quantise kernel that writes its 4-bit image
int tnns_dense_channels(int C, int KH, int KW);
bool tnns_dense_eligible(int type, int C, int KH, int KW);
int tnns_launch_repack_weights_dense(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, uint64_t* d_out, int Kp_out);
int tnns_launch_dense_quantise(tnns_cuda_ctx* ctx, const float* d_x, const float* d_thr, void* d_img, const TnnsGeom& g, int Kd, int layout,
                               cudaStream_t stream);
// driver-encoded descriptor of a two-dimensional tensor for the copy engine (128 bytes at `map`)
int tnns_tensor_map_2d(void* map, int elem_bytes, const void* base, unsigned long long dim0, unsigned long long dim1,
                       unsigned long long stride1_bytes, unsigned box0, unsigned box1, int swizzle_bytes = 0);
// 4-bit GEMM + PReLU whose activation tiles the copy engine gathers (im2col tensor copies) from
// an e2m1 image; needs ternary activations and a channel count that fills 128-byte chunks
bool tnns_im2col_supported(const tnns_cuda_weights* w, const TnnsGeom& g);
// d_pimg != NULL: write the next layer's quantised activations instead of fp32 (next_format 0: binary
// bit planes, 1: ternary bit planes, 2: ternary 4-bit operand image)
// fused != NULL: the same launch also quantises the layer's fp32 input into d_image (quantiser
// warps beside the GEMM's, tiles wait for their images); d_sync = tnns_fused_sync_bytes(N) bytes
// of device memory, 128-byte aligned, cleared by the launcher on `stream`
struct TnnsFusedInput {
    const float* d_x;
    const float* d_thr;
    unsigned int* d_sync;
};
size_t tnns_fused_sync_bytes(int N);
bool tnns_fused_supported(const tnns_cuda_weights* w, const TnnsGeom& g, const float* d_x, int layout);
int tnns_launch_gemm_im2col(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const TnnsGeom& g,
                            float alpha, int layout, cudaStream_t stream, int pairs = 0, void* d_pimg = nullptr,
                            const float* d_thr_next = nullptr, int next_format = 1, const TnnsFusedInput* fused = nullptr, int next_PH = 0,
                            int next_PW = 0);

int tnns_fused_sync_prepare(tnns_cuda_ctx* ctx, int N, cudaStream_t stream, unsigned int* caller_words, unsigned int** words_out, int* self_clean);

// Slab-fed 4-bit GEMM + PReLU for stride-1 layers (gemm_slab.cu): d_image is the BORDERED 4-bit image of
// the layer input, [n][H + 2*PH][W + 2*PW][C/2 bytes] with the padding value in the border, and one
// slab of pixels per tile serves every filter tap.  All four network types (binary activations: the
// border holds +1).  d_pimg != NULL: quantised output for the next layer instead of fp32 --
// next_format 0 / 1 bit planes, 2 plain 4-bit image, 3 bordered 4-bit image for a next layer with
// padding (next_PH, next_PW) whose padded size equals this layer's; next_binary: that layer's
// activations are binary.  fused != NULL: the same launch quantises the fp32 input into d_image.
bool tnns_slab_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const TnnsGeom& g, bool fused);
size_t tnns_bordered_image_bytes(int N, int C, int H, int W, int PH, int PW);
int tnns_launch_gemm_slab(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const TnnsGeom& g, float alpha, int layout,
                          cudaStream_t stream, int pairs = 0, void* d_pimg = nullptr, const float* d_thr_next = nullptr, int next_format = 2,
                          int next_binary = 0, int next_PH = 0, int next_PW = 0, const TnnsFusedInput* fused = nullptr);

int tnns_launch_pack_weights(tnns_cuda_ctx* ctx, bool ternary, const float* d_w, const float* d_thr, void* d_packed, int KN, int C,
                             int KH, int KW, cudaStream_t stream);

int tnns_launch_mma_rate(tnns_cuda_ctx* ctx, bool f4, int iters, double* ops, cudaStream_t stream);
int tnns_launch_wait_selftest(tnns_cuda_ctx* ctx, cudaStream_t stream);

// Division by a runtime-constant divisor without the hardware divide sequence.
// Exact for every 32-bit unsigned numerator (Granlund-Montgomery round-up method).
struct FastDiv {
    uint32_t mul, sh1, sh2, d;
#ifdef __CUDACC__
    __device__ __forceinline__ uint32_t div(uint32_t n) const {
        uint32_t t = __umulhi(mul, n);
        return (t + ((n - t) >> sh1)) >> sh2;
    }
#endif
};
FastDiv tnns_fastdiv(uint32_t d);

#ifdef __CUDACC__
// 32 elements (one 32-bit lane of the sign plane, one of the zero plane) -> 32 e2m1 nibbles (four
// words) in a fixed permuted order: nibble = sign<<3 | nonzero<<1 (+1 = 0x2, -1 = 0xA, 0 = 0x0).
// x gathers, per nibble, the sign bits of elements 4i+3, 4i+2 (bits 3, 2) over their non-zero
// bits (bits 1, 0); masking x with 0xA gives the nibbles of the elements 4i+3, masking x<<1 those
// of the elements 4i+2; y does the same for 4i+1 and 4i.  Ten integer operations per 32 elements.
// Activations and weights go through this same routine, so the permutation cancels in the dot product.
// 32 channels of one pixel from a pixel-major (NHWC) tile that the copy engine wrote in the 128-byte swizzle
// pattern: `row` = the pixel's 128 bytes in shared memory; of its eight 16-byte chunks, chunk c sits where
// address bits 4..6 equal c XOR address bits 7..9 (the pattern is a function of the shared-memory address).
// Channel b ends at bit b (visit 31 .. 0 and shift left); the predicates are read off sign bits (v < -t <=>
// signbit(v + t); |v| > t <=> signbit(t - |v|); binary v < t <=> signbit(v - t)); channels at or past nch read
// as absent (sign 0, non-zero 0).  Lanes of a warp = neighbouring pixels: each load instruction spreads over
// all banks, where a plain [pixel][channel] tile would put every lane on the same one.
template <bool TERNARY>
__device__ __forceinline__ void tnns_quantise_row32_swz128(const unsigned char* row, int nch, float t, uint32_t& sg_out, uint32_t& nz_out) {
    const uint32_t x = (static_cast<uint32_t>(__cvta_generic_to_shared(row)) >> 7) & 7u;
    uint32_t sg = 0, nz = 0;
#pragma unroll
    for (int c = 7; c >= 0; c--) {
        const float4 v4 = *reinterpret_cast<const float4*>(row + ((static_cast<uint32_t>(c) ^ x) << 4));
#pragma unroll
        for (int e = 3; e >= 0; e--) {
            const float v = e == 3 ? v4.w : e == 2 ? v4.z : e == 1 ? v4.y : v4.x;
            if (4 * c + e < nch) {
                if (TERNARY) {
                    sg = __funnelshift_l(__float_as_uint(v + t), sg, 1);
                    nz = __funnelshift_l(__float_as_uint(t - fabsf(v)), nz, 1);
                } else {
                    sg = __funnelshift_l(__float_as_uint((v + 0.0f) - t), sg, 1);
                }
            } else {
                sg <<= 1;
                nz <<= 1;
            }
        }
    }
    sg_out = sg;
    nz_out = nz;
}

__device__ __forceinline__ void tnns_expand32_f4(uint32_t s, uint32_t z, uint32_t (&w)[4]) {
    const uint32_t x = (s & 0xCCCCCCCCu) | (~(z >> 2) & 0x33333333u);
    const uint32_t y = ((s << 2) & 0xCCCCCCCCu) | (~z & 0x33333333u);
    w[0] = x & 0xAAAAAAAAu;
    w[1] = (x << 1) & 0xAAAAAAAAu;
    w[2] = y & 0xAAAAAAAAu;
    w[3] = (y << 1) & 0xAAAAAAAAu;
}
#endif
