// Quantise-only kernel fed by the copy engine (the thresholding half of t2r_p2_opt / b2r,
// reference: src/tnns/ternarize2row_avx2.c:438-452, src/tnns/binarize2row_avx2.c:15-22, without
// the im2row scatter) for NCHW input.
//
// The input is read as a two-dimensional tensor: one row per (image, channel) with H*W floats.
// A persistent block walks work items (image, band of 128 pixels, group of 64 channels); the
// producer thread requests each item as ONE tensor copy -- a box of 128 pixels x 64 channels,
// 32 KB -- into a four-deep shared-memory ring, so about 128 KB per SM are in flight towards HBM
// at any time without holding a single register.  Two groups of four consumer warps take the
// stages alternately: thread = pixel, 64 conflict-free shared-memory reads (lanes read
// consecutive floats), the sign and non-zero bits pushed into the plane words branch-free, the
// stage handed back, then the pixel's 64 channels stored as one 64-bit word per plane or as
// 32 bytes of e2m1 operands.  The kernel is bound by HBM traffic: 4 bytes read per input value.
//
// NHWC input (NHWC_IN) is the tensor (pixels of all images) x (channels): an item arrives as two
// copies of 128 pixels x 32 channels, written in the 128-byte swizzle pattern, so that a thread
// reads its pixel's channels as eight 16-byte loads per half whose physical chunk is rotated by the
// pixel index: the 32 lanes of a warp then spread over all banks (a plain [pixel][channel] tile
// would put every lane on the same bank).
#include <cuda.h>

#include <algorithm>

#include "internal.h"
#include "mbar.cuh"

namespace {

constexpr int QL = 128;                      // pixels per band = threads per consumer group
constexpr int QC = 64;                       // channels per stage = one plane word
constexpr int QSTG = 4;                      // ring depth
constexpr int QGROUPS = 2;                   // consumer groups
// A stage must always go to the same group: a group works through its items in order, so its
// successive waits on one stage's barrier are successive phases.  With a ring depth that is not a
// multiple of the group count a group would meet a stage again two phases later, and a parity
// wait cannot tell phase p from phase p + 2.
static_assert(QSTG % QGROUPS == 0, "every stage of the ring belongs to one consumer group");
constexpr int QTHREADS = 32 + QGROUPS * QL;  // producer warp + consumers
constexpr int QSTAGE_BYTES = QL * QC * 4;
constexpr size_t QSMEM = 1024 + (size_t)QSTG * QSTAGE_BYTES + 128;

__device__ __forceinline__ uint32_t push_sign_bit(uint32_t acc, float d) { return __funnelshift_l(__float_as_uint(d), acc, 1); }

template <bool TERNARY, int IMG, bool NHWC_IN>
__global__ void __launch_bounds__(QTHREADS, 1)
quantise_tma_kernel(const __grid_constant__ CUtensorMap tmap, const float* __restrict__ thr, void* __restrict__ out, int N, int C, int HW,
                    int Cp, int nbands, unsigned int* status, int W, int Wp, int HpWp, int off0) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + QSTG * QSTAGE_BYTES);
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + QSTG);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * QSTG);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // NCHW: an item is (image, band of 128 pixels of that image, channel group).  NHWC: the pixels of all
    // images are the rows of one tensor, a band is 128 consecutive rows and may straddle images.
    const long long items = NHWC_IN ? (long long)nbands * Cp : (long long)N * nbands * Cp;
    const int rows_total = NHWC_IN ? N * HW : 0;
    // The GEMM that follows on the stream is launched as a programmatic dependent: its blocks may
    // take SMs as the blocks of this launch leave and set themselves up there; it waits for this
    // launch to complete before it reads the image.  All blocks of this launch are resident at once.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (tid == 0) {
        for (int s = 0; s < QSTG; s++) {
            mbar_init(bar_full + 8 * s, 1);   // the producer's arrive with the expected bytes
            mbar_init(bar_empty + 8 * s, 4);  // the four warps of the group that read the stage
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // launched as a programmatic dependent itself: the input may be the output of the launch before
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (IMG == TNNS_IMG_E2M1 && HpWp != HW && warp > 0) {
        // bordered image (4-bit form): pixel (y, x) of image n sits at n*HpWp + y*Wp + x + off0 and the
        // frame of PH rows / PW columns around every image holds the layer's padding value -- ternary 0,
        // binary +1 -- so that a consumer reads padding like any other pixel.  Written here, before the
        // items, by all consumer threads of the grid.
        const uint32_t padw = TERNARY ? 0u : 0x22222222u;
        const uint4 pad4 = make_uint4(padw, padw, padw, padw);
        const int PH = off0 / Wp, PW = off0 - PH * Wp, H = HW / W;
        const long long total = (long long)N * HpWp;
        for (long long t = (long long)blockIdx.x * (QGROUPS * QL) + (tid - 32); t < total; t += (long long)gridDim.x * (QGROUPS * QL)) {
            const int r = (int)(t % HpWp), y = r / Wp, x = r - y * Wp;
            if (y < PH || y >= PH + H || x < PW || x >= PW + W) {
                uint4* dst = reinterpret_cast<uint4*>(out) + (size_t)t * Cp * 2;
                for (int u = 0; u < 2 * Cp; u++) dst[u] = pad4;
            }
        }
    }
    if (warp == 0) {
        if (lane == 0) {
            long long k = 0;
            for (long long i = blockIdx.x; i < items; i += gridDim.x, k++) {
                const int s = (int)(k % QSTG);
                const int ic = (int)(i % Cp);
                const long long nb = i / Cp;
                const int band = (int)(nb % nbands), n = (int)(nb / nbands);
                if (!mbar_wait(bar_empty + 8 * s, (uint32_t)((k / QSTG) & 1) ^ 1, abort_flag, status, 0x21)) goto done;
                mbar_arrive_expect_tx(bar_full + 8 * s, QSTAGE_BYTES);  // the whole box(es), edges zero-filled
                if (NHWC_IN) {
                    const int row0 = (int)nb * QL;  // pixel row of the (pixels x channels) tensor
                    tma_tile2d_g2s(smem_u32(smem + s * QSTAGE_BYTES), &tmap, ic * QC, row0, bar_full + 8 * s);
                    tma_tile2d_g2s(smem_u32(smem + s * QSTAGE_BYTES + QSTAGE_BYTES / 2), &tmap, ic * QC + 32, row0, bar_full + 8 * s);
                } else {
                    tma_tile2d_g2s(smem_u32(smem + s * QSTAGE_BYTES), &tmap, band * QL, n * C + ic * QC, bar_full + 8 * s);
                }
            }
        }
    } else {
        const int grp = (warp - 1) >> 2;
        const int p = tid - 32 - grp * QL;  // pixel of the band
        long long k = grp;
        // The threshold of an item's image is loaded one item ahead and not touched until its turn: an
        // instruction that uses a just-issued load holds the (in-order) warp for the whole round trip.
        const long long step = (long long)QGROUPS * gridDim.x, first = blockIdx.x + (long long)grp * gridDim.x;
        auto threshold_of = [&](long long i) -> float {
            if (NHWC_IN) {
                const int row = (int)(i / Cp) * QL + p;
                return row < rows_total ? __ldg(thr + row / HW) : 0.f;
            }
            return __ldg(thr + i / ((long long)Cp * nbands));
        };
        float t_raw = first < items ? threshold_of(first) : 0.f;
        for (long long i = first; i < items; i += step, k += QGROUPS) {
            const int s = (int)(k % QSTG);
            const int ic = (int)(i % Cp);
            const long long nb = i / Cp;
            int band, n, pix;
            if (NHWC_IN) {
                const int row = (int)nb * QL + p;
                n = row / HW;
                pix = row < rows_total ? row - n * HW : HW;  // rows past the tensor's end were zero-filled and are not stored
                band = 0;
            } else {
                band = (int)(nb % nbands);
                n = (int)(nb / nbands);
                pix = band * QL + p;
            }
            const int nch = min(QC, C - ic * QC);  // channels present in this group
            const float t = t_raw + 0.0f;  // + 0.0f: a threshold of -0 behaves as +0 in every compare
            if (i + step < items) t_raw = threshold_of(i + step);
            if (!mbar_wait(bar_full + 8 * s, (uint32_t)((k / QSTG) & 1), abort_flag, status, 0x22)) goto done;
            const float* sp = reinterpret_cast<const float*>(smem + s * QSTAGE_BYTES) + p;
            uint32_t sg[2] = {0, 0}, nz[2] = {0, 0};
            // channel b of a half ends at bit b: visit 31 .. 0 and shift left; predicates read
            // off sign bits (v < -t <=> signbit(v + t); |v| > t <=> signbit(t - |v|); v < t <=> signbit(v - t))
            if (NHWC_IN) {
                const unsigned char* row = smem + s * QSTAGE_BYTES + p * 128;
                tnns_quantise_row32_swz128<TERNARY>(row, nch, t, sg[0], nz[0]);
                tnns_quantise_row32_swz128<TERNARY>(row + QSTAGE_BYTES / 2, nch - 32, t, sg[1], nz[1]);
            } else if (nch == QC) {
#pragma unroll
                for (int half = 0; half < 2; half++) {
#pragma unroll
                    for (int b = 31; b >= 0; b--) {
                        const float v = sp[(32 * half + b) * QL];
                        if (TERNARY) {
                            sg[half] = push_sign_bit(sg[half], v + t);
                            nz[half] = push_sign_bit(nz[half], t - fabsf(v));
                        } else {
                            sg[half] = push_sign_bit(sg[half], (v + 0.0f) - t);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = QC - 1; c >= 0; c--) {
                    const int half = c >> 5;
                    if (c < nch) {
                        const float v = sp[c * QL];
                        if (TERNARY) {
                            sg[half] = push_sign_bit(sg[half], v + t);
                            nz[half] = push_sign_bit(nz[half], t - fabsf(v));
                        } else {
                            sg[half] = push_sign_bit(sg[half], (v + 0.0f) - t);
                        }
                    } else {  // absent channel: sign 0, non-zero 0
                        sg[half] <<= 1;
                        nz[half] <<= 1;
                    }
                }
            }
            if (!TERNARY) nz[0] = nz[1] = 0xFFFFFFFFu;  // the binary alphabet has no zero; absent channels read +1
            // every value is in registers: hand the stage back before storing
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
            if (pix < HW) {
                if (IMG == TNNS_IMG_E2M1) {
                    uint32_t lo[4], hi[4];
                    tnns_expand32_f4(sg[0], ~nz[0], lo);
                    tnns_expand32_f4(sg[1], ~nz[1], hi);
                    const int y = pix / W, x = pix - y * W;
                    uint4* dst = reinterpret_cast<uint4*>(out) + (((size_t)n * HpWp + (size_t)y * Wp + x + off0) * Cp + ic) * 2;
                    dst[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    dst[1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                } else {
                    uint64_t* img = reinterpret_cast<uint64_t*>(out);
                    const size_t planes = TERNARY ? 2 : 1;
                    const size_t at = ((size_t)n * planes * HW + pix) * Cp + ic;
                    img[at] = ((uint64_t)sg[1] << 32) | sg[0];
                    if (TERNARY) img[at + (size_t)HW * Cp] = ~(((uint64_t)nz[1] << 32) | nz[0]);
                }
            }
        }
    }
done:
    __syncwarp();
    if (*abort_flag && warp == 0 && lane == 0) {
        // a wait gave up: give the copies already issued time to land before shared memory is released
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    __syncthreads();
}

}  // namespace

bool tnns_quantise_tma_supported(const float* d_x, int H, int W, int layout) {
    const long long HW = (long long)H * W;
    return layout == TNNS_NCHW && HW % 4 == 0 && HW >= 32 && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0;
}

// NHWC: rows of C floats must be 16-byte multiples and the tensor large enough for a box of 128 pixel rows
bool tnns_quantise_tma_nhwc_supported(const float* d_x, int N, int C, int H, int W) {
    return C % 4 == 0 && (long long)N * H * W >= 128 && (long long)N * H * W < 0x7FFFFFFFLL && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0;
}

int tnns_launch_quantise_tma(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                             int W, cudaStream_t stream, int format, int PH, int PW, int layout) {
    const int HW = H * W;
    if (N == 0) return TNNS_OK;
    if ((PH || PW) && format != TNNS_IMG_E2M1) return tnns_fail(TNNS_ERR_INVALID, "only the 4-bit image has a bordered form");
    const int Wp = W + 2 * PW, HpWp = (H + 2 * PH) * Wp, off0 = PH * Wp + PW;
    const int Cp = (C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS;
    const bool nhwc = layout == TNNS_NHWC;
    const int nbands = nhwc ? (int)(((long long)N * HW + QL - 1) / QL) : (HW + QL - 1) / QL;
    alignas(64) CUtensorMap map;
    int rc = nhwc ? tnns_tensor_map_2d(&map, 4, d_x, (unsigned long long)C, (unsigned long long)N * HW, (unsigned long long)C * 4, 32, QL, 128)
                  : tnns_tensor_map_2d(&map, 4, d_x, (unsigned long long)HW, (unsigned long long)N * C, (unsigned long long)HW * 4, QL, QC);
    if (rc) return rc;
    const long long items = nhwc ? (long long)nbands * Cp : (long long)N * nbands * Cp;
    const int grid = (int)std::min<long long>(items, ctx->sm_count);
    auto launch = [&](auto kern, bool* smem_set) -> int {
        if (!smem_set[ctx->device & 63]) {  // once per kernel and device
            TNNS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QSMEM));
            smem_set[ctx->device & 63] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(QTHREADS);
        cfg.dynamicSmemBytes = QSMEM;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        TNNS_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, map, d_thr, d_image, N, C, HW, Cp, nbands, ctx->d_status, W, Wp, HpWp, off0));
        tnns_count_launch();
        TNNS_CUDA_TRY(cudaGetLastError());
        return TNNS_OK;
    };
    static bool set_flags[8][64] = {};
    const int which = (format == TNNS_IMG_E2M1 ? 0 : 2) + (ternary ? 0 : 1) + (nhwc ? 4 : 0);
    switch (which) {
        case 0: return launch(quantise_tma_kernel<true, TNNS_IMG_E2M1, false>, set_flags[0]);
        case 1: return launch(quantise_tma_kernel<false, TNNS_IMG_E2M1, false>, set_flags[1]);
        case 2: return launch(quantise_tma_kernel<true, TNNS_IMG_PLANES, false>, set_flags[2]);
        case 3: return launch(quantise_tma_kernel<false, TNNS_IMG_PLANES, false>, set_flags[3]);
        case 4: return launch(quantise_tma_kernel<true, TNNS_IMG_E2M1, true>, set_flags[4]);
        case 5: return launch(quantise_tma_kernel<false, TNNS_IMG_E2M1, true>, set_flags[5]);
        case 6: return launch(quantise_tma_kernel<true, TNNS_IMG_PLANES, true>, set_flags[6]);
        default: return launch(quantise_tma_kernel<false, TNNS_IMG_PLANES, true>, set_flags[7]);
    }
}
