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
// quantise only: fp32 tensor -> packed image [n][plane][pixel][ic] (no im2row)
int tnns_launch_quantise(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                         int W, int layout, cudaStream_t stream);

int tnns_launch_pack_weights(tnns_cuda_ctx* ctx, bool ternary, const float* d_w, const float* d_thr, void* d_packed, int KN, int C,
                             int KH, int KW, cudaStream_t stream);

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
