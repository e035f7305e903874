// Bitwise GEMM + PReLU on the integer pipe (the device form of mm_tnn / mm_tbn / mm_btn /
// mm_bnn; reference: src/tnns/mm_p2_final_{tnn,tbn,btn,bnn}_avx2.c, include/tnns/mm.h:11-71).
//
// Arithmetic per 32-bit lane of an (activation row, kernel) pair:
//   TNN  z = az|bz ; n = (as^bs)&~z ; acc = 64*Kp - sum popc(z) - 2*sum popc(n)
//   TBN  n = (as^bs)&~az            ; acc = 64*Kp - sum popc(az) - 2*sum popc(n)
//   BTN  n = (as^bs)&~bz            ; acc = 64*Kp - sum popc(bz) - 2*sum popc(n)
//   BNN  n = as^bs                  ; acc = K_unpack - 2*sum popc(n)
// POPC is the scarce instruction, so the tiled kernel counts with bit-sliced carry-save
// adders (the GPU analogue of the reference's CSA256_custom3 + popcnt256,
// src/tnns/mm_p2_final_tnn_avx2.c:44-53,72-77): four lanes are compressed by LOP3 full
// adders and only the weight-8 (TNN) or weight-4 (others) carry word is popcounted.
#include <algorithm>

#include "internal.h"

namespace {

// The reference has two PReLU expressions, which differ in the sign of a zero sum under a negative
// alpha: mm_tnn scales every non-positive value (src/tnns/mm_p2_final_tnn_avx2.c:90-93, 204-208: 0*alpha),
// mm_tbn / mm_btn / mm_bnn pass zero through (result >= 0 ? result : alpha*result,
// src/tnns/mm_p2_final_tbn_avx2.c:73, _btn_:73, _bnn_:60).
template <int TYPE>
__device__ __forceinline__ float prelu_i(int acc, float alpha) {
    if (TYPE == TNN) return acc > 0 ? (float)acc : (float)acc * alpha;
    return acc >= 0 ? (float)acc : alpha * (float)acc;
}

__device__ __forceinline__ size_t out_index(long long r, int kn, int KN, int OHW, int layout) {
    if (layout == TNNS_NHWC) return (size_t)r * KN + kn;
    const long long n = r / OHW;
    return ((size_t)n * KN + kn) * OHW + (size_t)(r - n * OHW);  // include/tnns/mm.h:30
}

// ---------------------------------------------------------------------------------------
// Reference-shaped kernel: one thread per output, operands read from global memory.
// ---------------------------------------------------------------------------------------
template <int TYPE>
__global__ void __launch_bounds__(256) gemm_popc_simple_kernel(const uint32_t* __restrict__ A, const uint32_t* __restrict__ B,
                                                               float* __restrict__ y, long long M, int KN, int Kp, int OHW,
                                                               int K_unpack, float alpha, int layout) {
    constexpr bool A2 = (TYPE == TNN || TYPE == TBN), B2 = (TYPE == TNN || TYPE == BTN);
    const long long total = M * KN;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int groups = Kp / 4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int kn = (int)(i / M);
        const long long r = i - (long long)kn * M;
        const uint32_t* a = A + (size_t)r * Kp * (A2 ? 4 : 2);
        const uint32_t* b = B + (size_t)kn * Kp * (B2 ? 4 : 2);
        int cz = 0, cn = 0;
        for (int g = 0; g < groups; g++) {
            const uint32_t* ag = a + g * (A2 ? 16 : 8);
            const uint32_t* bg = b + g * (B2 ? 16 : 8);
#pragma unroll
            for (int l = 0; l < 8; l++) {
                const uint32_t as = ag[l], bs = bg[l];
                if (TYPE == TNN) {
                    const uint32_t z = ag[8 + l] | bg[8 + l];
                    cz += __popc(z);
                    cn += __popc((as ^ bs) & ~z);
                } else if (TYPE == TBN) {
                    cz += __popc(ag[8 + l]);
                    cn += __popc((as ^ bs) & ~ag[8 + l]);
                } else if (TYPE == BTN) {
                    cz += __popc(bg[8 + l]);
                    cn += __popc((as ^ bs) & ~bg[8 + l]);
                } else {
                    cn += __popc(as ^ bs);
                }
            }
        }
        const int acc = (TYPE == BNN) ? K_unpack - 2 * cn : 64 * Kp - cz - 2 * cn;
        y[out_index(r, kn, KN, OHW, layout)] = prelu_i<TYPE>(acc, alpha);
    }
}

// ---------------------------------------------------------------------------------------
// Tiled kernel: 64x64 outputs per block, 256 threads, 4x4 outputs per thread; operands
// staged through shared memory by a 4-deep cp.async ring, one 256-element K group (eight
// 32-bit lanes per plane) per stage.
// ---------------------------------------------------------------------------------------
constexpr int TM = 64, TN = 64, RM = 4, RN = 4, NTHREADS = 256, NSTAGE = 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ uint32_t maj3(uint32_t a, uint32_t b, uint32_t c) { return (a & b) | (c & (a ^ b)); }

struct Csa {
    uint32_t ones, twos, fours;
    int acc;
};

// TNN: four lanes of z (weight 1) and n (weight 2, disjoint from z); because n is a
// subset of ~z, (ones&z)|n is the exact weight-2 word of ones+z+2n.
__device__ __forceinline__ void csa_step_tnn(Csa& s, const uint4& as, const uint4& az, const uint4& bs, const uint4& bz) {
    uint32_t h0, h1, h2, h3, z, n;
    z = az.x | bz.x; n = (as.x ^ bs.x) & ~z; h0 = (s.ones & z) | n; s.ones ^= z;
    z = az.y | bz.y; n = (as.y ^ bs.y) & ~z; h1 = (s.ones & z) | n; s.ones ^= z;
    z = az.z | bz.z; n = (as.z ^ bs.z) & ~z; h2 = (s.ones & z) | n; s.ones ^= z;
    z = az.w | bz.w; n = (as.w ^ bs.w) & ~z; h3 = (s.ones & z) | n; s.ones ^= z;
    const uint32_t ca = maj3(s.twos, h0, h1); s.twos ^= h0 ^ h1;
    const uint32_t cb = maj3(s.twos, h2, h3); s.twos ^= h2 ^ h3;
    const uint32_t c8 = maj3(s.fours, ca, cb); s.fours ^= ca ^ cb;
    s.acc += __popc(c8);
}
__device__ __forceinline__ int csa_total_tnn(const Csa& s) {
    return __popc(s.ones) + 2 * __popc(s.twos) + 4 * __popc(s.fours) + 8 * s.acc;
}

// Single-weight stream (TBN/BTN/BNN): four words of weight 1.
__device__ __forceinline__ void csa_step_w1(Csa& s, uint32_t n0, uint32_t n1, uint32_t n2, uint32_t n3) {
    const uint32_t ca = maj3(s.ones, n0, n1); s.ones ^= n0 ^ n1;
    const uint32_t cb = maj3(s.ones, n2, n3); s.ones ^= n2 ^ n3;
    const uint32_t c4 = maj3(s.twos, ca, cb); s.twos ^= ca ^ cb;
    s.acc += __popc(c4);
}
__device__ __forceinline__ int csa_total_w1(const Csa& s) { return __popc(s.ones) + 2 * __popc(s.twos) + 4 * s.acc; }

template <int TYPE>
__global__ void __launch_bounds__(NTHREADS) gemm_popc_tiled_kernel(const uint32_t* __restrict__ A, const uint32_t* __restrict__ B,
                                                                   float* __restrict__ y, long long M, int KN, int Kp, int OHW,
                                                                   int K_unpack, float alpha, int layout) {
    constexpr bool A2 = (TYPE == TNN || TYPE == TBN), B2 = (TYPE == TNN || TYPE == BTN);
    constexpr int AW = A2 ? 16 : 8, BW = B2 ? 16 : 8;  // 32-bit words per row and K group
    constexpr int AP = AW + 4, BP = BW + 4;             // padded pitch: 16-byte units stay conflict free
    __shared__ __align__(16) uint32_t sA[NSTAGE][TM * AP];
    __shared__ __align__(16) uint32_t sB[NSTAGE][TN * BP];

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int lm = lane & 15, ln = lane >> 4;
    const long long m0 = (long long)blockIdx.x * TM;
    const int n0 = blockIdx.y * TN;
    const int groups = Kp / 4;
    const size_t a_pitch = (size_t)Kp * (A2 ? 4 : 2), b_pitch = (size_t)Kp * (B2 ? 4 : 2);  // 32-bit words per row

    // cp.async assignment: 16-byte chunk `tid` of each operand tile (rows clamped; results of
    // clamped rows are never stored)
    constexpr int ACH = AW / 4, BCH = BW / 4;  // chunks per row
    const bool a_active = tid < TM * ACH, b_active = tid < TN * BCH;
    const int a_row = tid / ACH, a_ch = tid % ACH, b_row = tid / BCH, b_ch = tid % BCH;
    const uint32_t* a_src = A + (size_t)min(m0 + (long long)a_row, M - 1) * a_pitch + a_ch * 4;
    const uint32_t* b_src = B + (size_t)min(n0 + b_row, KN - 1) * b_pitch + b_ch * 4;

    auto issue = [&](int g) {
        if (g < groups) {
            const int st = g % NSTAGE;
            if (a_active) cp_async16(&sA[st][a_row * AP + a_ch * 4], a_src + (size_t)g * AW);
            if (b_active) cp_async16(&sB[st][b_row * BP + b_ch * 4], b_src + (size_t)g * BW);
        }
        cp_async_commit();
    };

    Csa st[RM][RN];
#pragma unroll
    for (int i = 0; i < RM; i++)
#pragma unroll
        for (int j = 0; j < RN; j++) st[i][j] = Csa{0u, 0u, 0u, 0};
    int az_cnt[RM] = {0, 0, 0, 0}, bz_cnt[RN] = {0, 0, 0, 0};

#pragma unroll
    for (int g = 0; g < NSTAGE - 1; g++) issue(g);

    for (int g = 0; g < groups; g++) {
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();
        issue(g + NSTAGE - 1);  // refills the stage consumed in iteration g-1
        const uint32_t* a_s = sA[g % NSTAGE];
        const uint32_t* b_s = sB[g % NSTAGE];
#pragma unroll
        for (int half = 0; half < 2; half++) {
            uint4 as[RM], az[RM], bs[RN], bz[RN];
#pragma unroll
            for (int i = 0; i < RM; i++) {
                const uint32_t* p = a_s + (lm + 16 * i) * AP + half * 4;
                as[i] = *reinterpret_cast<const uint4*>(p);
                if (A2) az[i] = *reinterpret_cast<const uint4*>(p + 8);
            }
#pragma unroll
            for (int j = 0; j < RN; j++) {
                const uint32_t* p = b_s + (warp * 8 + ln * 4 + j) * BP + half * 4;
                bs[j] = *reinterpret_cast<const uint4*>(p);
                if (B2) bz[j] = *reinterpret_cast<const uint4*>(p + 8);
            }
            if (TYPE == TBN) {
#pragma unroll
                for (int i = 0; i < RM; i++) az_cnt[i] += __popc(az[i].x) + __popc(az[i].y) + __popc(az[i].z) + __popc(az[i].w);
            }
            if (TYPE == BTN) {
#pragma unroll
                for (int j = 0; j < RN; j++) bz_cnt[j] += __popc(bz[j].x) + __popc(bz[j].y) + __popc(bz[j].z) + __popc(bz[j].w);
            }
#pragma unroll
            for (int i = 0; i < RM; i++)
#pragma unroll
                for (int j = 0; j < RN; j++) {
                    if (TYPE == TNN) {
                        csa_step_tnn(st[i][j], as[i], az[i], bs[j], bz[j]);
                    } else if (TYPE == TBN) {
                        csa_step_w1(st[i][j], (as[i].x ^ bs[j].x) & ~az[i].x, (as[i].y ^ bs[j].y) & ~az[i].y,
                                    (as[i].z ^ bs[j].z) & ~az[i].z, (as[i].w ^ bs[j].w) & ~az[i].w);
                    } else if (TYPE == BTN) {
                        csa_step_w1(st[i][j], (as[i].x ^ bs[j].x) & ~bz[j].x, (as[i].y ^ bs[j].y) & ~bz[j].y,
                                    (as[i].z ^ bs[j].z) & ~bz[j].z, (as[i].w ^ bs[j].w) & ~bz[j].w);
                    } else {
                        csa_step_w1(st[i][j], as[i].x ^ bs[j].x, as[i].y ^ bs[j].y, as[i].z ^ bs[j].z, as[i].w ^ bs[j].w);
                    }
                }
        }
    }
    cp_async_wait<0>();

    // epilogue: integer result -> PReLU -> fp32 store
#pragma unroll
    for (int i = 0; i < RM; i++) {
        const long long r = m0 + lm + 16 * i;
        if (r >= M) continue;
        const long long n_img = r / OHW;
        const int rem = (int)(r - n_img * OHW);
        float v[RN];
#pragma unroll
        for (int j = 0; j < RN; j++) {
            int acc;
            if (TYPE == TNN) acc = 64 * Kp - csa_total_tnn(st[i][j]);
            else if (TYPE == TBN) acc = 64 * Kp - az_cnt[i] - 2 * csa_total_w1(st[i][j]);
            else if (TYPE == BTN) acc = 64 * Kp - bz_cnt[j] - 2 * csa_total_w1(st[i][j]);
            else acc = K_unpack - 2 * csa_total_w1(st[i][j]);
            v[j] = prelu_i<TYPE>(acc, alpha);
        }
        const int c0 = n0 + warp * 8 + ln * 4;
        if (layout == TNNS_NHWC) {
            float* dst = y + (size_t)r * KN + c0;
            if (c0 + 3 < KN && (KN & 3) == 0) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            else {
#pragma unroll
                for (int j = 0; j < RN; j++) if (c0 + j < KN) dst[j] = v[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < RN; j++)
                if (c0 + j < KN) y[((size_t)n_img * KN + c0 + j) * OHW + rem] = v[j];
        }
    }
}

template <int TYPE>
int launch_typed(tnns_cuda_ctx* ctx, const void* d_a, const void* d_b, float* d_y, long long M, int KN, int Kp, int OHW,
                 int K_unpack, float alpha, int layout, bool tiled, cudaStream_t stream) {
    const uint32_t* A = reinterpret_cast<const uint32_t*>(d_a);
    const uint32_t* B = reinterpret_cast<const uint32_t*>(d_b);
    if (tiled) {
        const long long gx = (M + TM - 1) / TM;
        if (gx > 0x7FFFFFFFLL) return tnns_fail(TNNS_ERR_UNSUPPORTED, "too many rows for one launch");
        dim3 grid((unsigned)gx, (unsigned)((KN + TN - 1) / TN));
        gemm_popc_tiled_kernel<TYPE><<<grid, NTHREADS, 0, stream>>>(A, B, d_y, M, KN, Kp, OHW, K_unpack, alpha, layout);
    } else {
        const long long total = M * KN;
        const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 64);
        gemm_popc_simple_kernel<TYPE><<<blocks, 256, 0, stream>>>(A, B, d_y, M, KN, Kp, OHW, K_unpack, alpha, layout);
    }
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}

}  // namespace

int tnns_launch_gemm_popc(tnns_cuda_ctx* ctx, int type, const void* d_a, const void* d_b, float* d_y, long long M,
                          int KN, int Kp, int OHW, int K_unpack, float alpha, int layout, bool tiled,
                          cudaStream_t stream) {
    if (M == 0 || KN == 0) return TNNS_OK;
    switch (type) {
        case TNN: return launch_typed<TNN>(ctx, d_a, d_b, d_y, M, KN, Kp, OHW, K_unpack, alpha, layout, tiled, stream);
        case TBN: return launch_typed<TBN>(ctx, d_a, d_b, d_y, M, KN, Kp, OHW, K_unpack, alpha, layout, tiled, stream);
        case BTN: return launch_typed<BTN>(ctx, d_a, d_b, d_y, M, KN, Kp, OHW, K_unpack, alpha, layout, tiled, stream);
        case BNN: return launch_typed<BNN>(ctx, d_a, d_b, d_y, M, KN, Kp, OHW, K_unpack, alpha, layout, tiled, stream);
        default: return tnns_fail(TNNS_ERR_INVALID, "unknown network type %d", type);
    }
}
