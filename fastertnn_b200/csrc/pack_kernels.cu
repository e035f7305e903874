// Fused quantise + bit-pack + im2row kernels (the device form of t2r_p2_opt and b2r,
// reference: src/tnns/ternarize2row_avx2.c:715-803, src/tnns/binarize2row_avx2.c:131-199).
//
// The reference scatters every packed pixel word to all (oh,ow,kh,kw) windows that use
// it.  Here the work is turned around: a thread block owns a band of output rows of one
// image, packs the input pixels that band needs ONCE into shared memory (phase 1, fully
// coalesced fp32 reads) and then streams out the band's im2row rows as contiguous 16-byte
// stores, gathering the plane words from shared memory (phase 2).  The kernel is bound by
// HBM traffic: 4 bytes read per input value plus 16*Kp (ternary) or 8*Kp (binary) bytes
// written per output row.
#include <algorithm>
#include <climits>
#include <cstdlib>

#include "internal.h"

namespace {

constexpr int kPackThreads = 256;
#ifndef TNNS_PACK_MINCTA
#define TNNS_PACK_MINCTA 4
#endif

// ---------------------------------------------------------------------------------------
// Reference-shaped kernel: one thread per plane word, channels fetched straight from
// global memory.  Slow (strided reads, every pixel re-quantised KH*KW times) but handles
// every geometry; used for cross-checks and for shapes the staged kernel cannot hold.
// ---------------------------------------------------------------------------------------
template <bool TERNARY, bool NHWC>
__global__ void __launch_bounds__(256) pack_gather_kernel(const float* __restrict__ x, const float* __restrict__ thr,
                                                         uint64_t* __restrict__ out, TnnsGeom g, long long total) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / g.Kp;
        const int j = (int)(i - r * g.Kp);
        const int ow = (int)(r % g.OW);
        const int oh = (int)((r / g.OW) % g.OH);
        const int n = (int)(r / ((long long)g.OW * g.OH));
        uint64_t sign = 0, nz = 0;
        if (j < g.Kw) {
            const int ic = j % g.Cp, kw = (j / g.Cp) % g.KW, kh = j / (g.Cp * g.KW);
            const int ih = oh * g.SH + kh - g.PH, iw = ow * g.SW + kw - g.PW;
            if (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) {
                const float t = thr[n], nt = -t;
                const int nch = min(TNNS_WORD_BITS, g.C - ic * TNNS_WORD_BITS);
                const float* px;
                size_t cs;
                if (NHWC) {
                    px = x + (((size_t)n * g.H + ih) * g.W + iw) * g.C + (size_t)ic * TNNS_WORD_BITS;
                    cs = 1;
                } else {
                    px = x + (((size_t)n * g.C + (size_t)ic * TNNS_WORD_BITS) * g.H + ih) * g.W + iw;
                    cs = (size_t)g.H * g.W;
                }
                for (int b = 0; b < nch; b++) {
                    const float v = px[b * cs];
                    if (TERNARY) {
                        if (v < nt) { sign |= 1ull << b; nz |= 1ull << b; }
                        else if (v > t) nz |= 1ull << b;
                    } else {
                        if (v < t) sign |= 1ull << b;
                    }
                }
            }
        }
        if (TERNARY) {
            uint64_t* row = out + (size_t)r * 2 * g.Kp + (size_t)(j >> 2) * 8 + (j & 3);
            row[0] = sign;
            row[4] = ~nz;
        } else {
            out[(size_t)r * g.Kp + j] = sign;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Staged kernel.
//   grid.x = N * nbands ; block = 256 threads ; dynamic smem:
//     planes * Lmax * Cp   uint64   packed pixels of the band, [pixel][ic] (plane 0 sign, 1 zero)
//     Kp                   int32    tap table: word offset of plane word j relative to the
//                                   window's first pixel, (kh*W + kw)*Cp + ic ; INT_MIN for the
//                                   words added by the pad-to-four
//     Kp                   uint32   tap table: kh<<16 | kw  (border windows only)
// LAYOUT 0: NCHW, one thread packs VEC neighbouring pixels over 64 channels (loads are
//           coalesced along W, channel stride H*W).
// LAYOUT 1: NHWC, one warp packs 32 neighbouring channels of a pixel with __ballot_sync.
// LAYOUT 2: the input is already quantised bit planes [n][plane][pixel][ic] (written by the GEMM
//           epilogue of the previous layer); phase 1 is a plain copy of the band's rows.
// PAIR:     C_pack is even, so plane words 2k and 2k+1 of a row are neighbours in shared
//           memory and move as one 128-bit load.
// ---------------------------------------------------------------------------------------
constexpr int kPadWord = INT_MIN;

// Branch-free quantisation.  For finite fp32 a, b the rounded difference a-b is negative
// exactly when a < b (gradual underflow keeps non-zero differences non-zero, and x-x is +0),
// so the predicates are read off sign bits:
//   ternary sign     v < -t   <=>  signbit(v + t)
//   ternary non-zero |v| > t  <=>  signbit(t - |v|)   (equals "v < -t or v > t" for every t)
//   binary  sign     v <  t   <=>  signbit(v - t)
// and pushed into the plane word with one funnel shift each: acc = (acc << 1) | signbit.
// Channels are therefore visited from 31 down to 0 so that channel b ends at bit b.
__device__ __forceinline__ uint32_t push_sign(uint32_t acc, float d) {
    return __funnelshift_l(__float_as_uint(d), acc, 1);
}

template <bool TERNARY, int VEC>
__device__ __forceinline__ void quantise_batch(const float* __restrict__ q, size_t HW, float t, uint32_t (&sg)[VEC],
                                               uint32_t (&nzb)[VEC]) {
    // channels q[7*HW] .. q[0] (descending), eight at a time: all loads first, then the pushes
    float vals[8][VEC];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const float* pk = q + (size_t)(7 - k) * HW;
        if (VEC == 4) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(pk));
            vals[k][0] = f.x; vals[k][1 % VEC] = f.y; vals[k][2 % VEC] = f.z; vals[k][3 % VEC] = f.w;
        } else {
            vals[k][0] = __ldg(pk);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; k++)
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            if (TERNARY) {
                sg[v] = push_sign(sg[v], vals[k][v] + t);
                nzb[v] = push_sign(nzb[v], t - fabsf(vals[k][v]));
            } else {
                sg[v] = push_sign(sg[v], (vals[k][v] + 0.0f) - t);  // + 0.0f turns -0 into +0: (-0) - (+0) would be -0
            }
        }
}

// IMG_OUT: stop after phase 1 and write the band's packed pixels out as they are (quantise only:
//           the packed image [n][plane][pixel][ic] that the implicit-im2row GEMM reads); the
//           geometry passed in is then that of a 1x1 stride-1 window, so bands have no halo.
// IMG_OUT = TNNS_IMG_E2M1 writes the same pixels as 4-bit operands instead (32 bytes per 64 channels).
template <bool TERNARY, int LAYOUT, int VEC, bool PAIR, int IMG_OUT>
__global__ void __launch_bounds__(kPackThreads, TNNS_PACK_MINCTA)
pack_staged_kernel(const float* __restrict__ x, const float* __restrict__ thr, uint4* __restrict__ out, TnnsGeom g,
                   int BOH, int nbands, int Lmax, FastDiv divU, FastDiv divOW, FastDiv divL) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int PLANES = TERNARY ? 2 : 1;
    uint64_t* sm_sign = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* sm_zero = sm_sign + (size_t)Lmax * g.Cp;  // only valid when TERNARY
    int* joff = reinterpret_cast<int*>(sm_sign + (size_t)PLANES * Lmax * g.Cp);
    uint32_t* jtap = reinterpret_cast<uint32_t*>(joff + g.Kp);

    const int tid = threadIdx.x;
    const int n = blockIdx.x / nbands;
    const int band = blockIdx.x - n * nbands;
    const int oh0 = band * BOH;
    const int boh = min(BOH, g.OH - oh0);
    const int ih_lo = max(oh0 * g.SH - g.PH, 0);
    const int ih_hi = min((oh0 + boh - 1) * g.SH - g.PH + g.KH, g.H);  // exclusive
    const int nrow = max(ih_hi - ih_lo, 0);                              // input rows held in smem
    const int L = nrow * g.W;                                            // pixels held in smem
    const float t = (LAYOUT == 2) ? 0.f : thr[n] + 0.0f, nt = -t;  // + 0.0f: a threshold of -0 behaves as +0 in every compare

    for (int j = tid; j < g.Kp; j += kPackThreads) {
        int off = kPadWord;
        uint32_t tap = 0;
        if (j < g.Kw) {
            const int ic = j % g.Cp, kw = (j / g.Cp) % g.KW, kh = j / (g.Cp * g.KW);
            off = (kh * g.W + kw) * g.Cp + ic;
            tap = ((uint32_t)kh << 16) | (uint32_t)kw;
        }
        joff[j] = off;
        jtap[j] = tap;
    }

    // ---------------- phase 1: quantise + pack the band's input pixels ----------------
    if (LAYOUT == 2) {
        const uint64_t* planes = reinterpret_cast<const uint64_t*>(x);
        const size_t HWC = (size_t)g.H * g.W * g.Cp;
        const uint64_t* src_s = planes + (size_t)n * PLANES * HWC + (size_t)ih_lo * g.W * g.Cp;
        const int words = L * g.Cp;
        for (int i = tid; i < words; i += kPackThreads) {
            sm_sign[i] = __ldg(src_s + i);
            if (TERNARY) sm_zero[i] = __ldg(src_s + HWC + i);
        }
    } else if (LAYOUT == 0) {
        const size_t HW = (size_t)g.H * g.W;
        const int LV = L / VEC;  // VEC divides L by construction (host checks W % VEC == 0)
        const int items = g.Cp * LV;
        for (int id = tid; id < items; id += kPackThreads) {
            const int ic = (LV == (int)divL.d) ? (int)divL.div((uint32_t)id) : id / LV;
            const int p = (id - ic * LV) * VEC;
            const int nch = min(TNNS_WORD_BITS, g.C - ic * TNNS_WORD_BITS);
            const float* src = x + ((size_t)n * g.C + (size_t)ic * TNNS_WORD_BITS) * HW + (size_t)ih_lo * g.W + p;
            uint32_t sg[2][VEC], nzb[2][VEC];
#pragma unroll
            for (int v = 0; v < VEC; v++) { sg[0][v] = sg[1][v] = 0; nzb[0][v] = nzb[1][v] = 0; }
#pragma unroll
            for (int half = 0; half < 2; half++) {
                if (nch >= 32 * half + 32) {
#pragma unroll 1
                    for (int b0 = 24; b0 >= 0; b0 -= 8)  // one batch of eight loads in flight per thread
                        quantise_batch<TERNARY, VEC>(src + (size_t)(32 * half + b0) * HW, HW, t, sg[half], nzb[half]);
                } else {
                    const int lim = nch - 32 * half;  // channels present in this half-word; may be <= 0
                    for (int b = 31; b >= 0; b--) {
                        const float* q = src + (size_t)(32 * half + b) * HW;
#pragma unroll
                        for (int v = 0; v < VEC; v++) {
                            if (b < lim) {
                                const float val = __ldg(q + v);
                                if (TERNARY) {
                                    sg[half][v] = push_sign(sg[half][v], val + t);
                                    nzb[half][v] = push_sign(nzb[half][v], t - fabsf(val));
                                } else {
                                    sg[half][v] = push_sign(sg[half][v], (val + 0.0f) - t);
                                }
                            } else {  // absent channel: sign 0, non-zero 0
                                sg[half][v] <<= 1;
                                if (TERNARY) nzb[half][v] <<= 1;
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < VEC; v++) {
                const int at = (p + v) * g.Cp + ic;
                sm_sign[at] = ((uint64_t)sg[1][v] << 32) | sg[0][v];
                if (TERNARY) sm_zero[at] = ~(((uint64_t)nzb[1][v] << 32) | nzb[0][v]);
            }
        }
    } else {
        // NHWC: the band's pixels are one contiguous run of L*C floats.
        const float* base = x + ((size_t)n * g.H + ih_lo) * g.W * g.C;
        const int lane = tid & 31, warp = tid >> 5;
        constexpr int NWARP = kPackThreads / 32;
        uint32_t* sm_sign32 = reinterpret_cast<uint32_t*>(sm_sign);
        uint32_t* sm_zero32 = reinterpret_cast<uint32_t*>(sm_zero);
        if ((g.C & 63) == 0) {
            // item i covers floats [32*i, 32*i+32) of the run: pixel i/(C/32), half-word i%(C/32);
            // the packed smem image [p][ic] viewed as uint32 is indexed by i itself.
            const int items = L * (g.C >> 5);
            constexpr int UNR = 8;
            for (int i0 = warp * UNR; i0 < items; i0 += NWARP * UNR) {
                float v[UNR];
#pragma unroll
                for (int u = 0; u < UNR; u++) v[u] = (i0 + u < items) ? __ldg(base + (size_t)(i0 + u) * 32 + lane) : 0.f;
#pragma unroll
                for (int u = 0; u < UNR; u++) {
                    if (TERNARY) {
                        const uint32_t s = __ballot_sync(0xFFFFFFFFu, v[u] < nt);
                        const uint32_t z = __ballot_sync(0xFFFFFFFFu, (v[u] < nt) || (v[u] > t));
                        if (lane == 0 && i0 + u < items) { sm_sign32[i0 + u] = s; sm_zero32[i0 + u] = ~z; }
                    } else {
                        const uint32_t s = __ballot_sync(0xFFFFFFFFu, v[u] < t);
                        if (lane == 0 && i0 + u < items) sm_sign32[i0 + u] = s;
                    }
                }
            }
        } else {
            // general channel count: item = (pixel, 32-channel half-word), tails predicated
            const int halves = 2 * g.Cp;
            const int items = L * halves;
            for (int i = warp; i < items; i += NWARP) {
                const int p = i / halves, h = i - p * halves;
                const int c = 32 * h + lane;
                const float v = (c < g.C) ? __ldg(base + (size_t)p * g.C + c) : 0.f;
                const bool ok = c < g.C;
                if (TERNARY) {
                    const uint32_t s = __ballot_sync(0xFFFFFFFFu, ok && v < nt);
                    const uint32_t z = __ballot_sync(0xFFFFFFFFu, ok && ((v < nt) || (v > t)));
                    if (lane == 0) { sm_sign32[i] = s; sm_zero32[i] = ~z; }
                } else {
                    const uint32_t s = __ballot_sync(0xFFFFFFFFu, ok && v < t);
                    if (lane == 0) sm_sign32[i] = s;
                }
            }
        }
    }
    __syncthreads();

    if (IMG_OUT == TNNS_IMG_E2M1) {
        // word i of the band = (pixel, channel group) -> 32 bytes at the same index
        uint4* dst = out + ((size_t)n * g.H * g.W + (size_t)ih_lo * g.W) * g.Cp * 2;
        const int words = L * g.Cp;
        for (int i = tid; i < words; i += kPackThreads) {
            const uint64_t s = sm_sign[i], z = TERNARY ? sm_zero[i] : 0ull;
            uint32_t lo[4], hi[4];
            tnns_expand32_f4((uint32_t)s, (uint32_t)z, lo);
            tnns_expand32_f4((uint32_t)(s >> 32), (uint32_t)(z >> 32), hi);
            dst[2 * (size_t)i] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            dst[2 * (size_t)i + 1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        }
        return;
    }
    if (IMG_OUT) {
        uint64_t* img = reinterpret_cast<uint64_t*>(out);
        const size_t HWC = (size_t)g.H * g.W * g.Cp;
        uint64_t* dst_s = img + (size_t)n * PLANES * HWC + (size_t)ih_lo * g.W * g.Cp;
        const int words = L * g.Cp;
        for (int i = tid; i < words; i += kPackThreads) {
            dst_s[i] = sm_sign[i];
            if (TERNARY) dst_s[HWC + i] = sm_zero[i];
        }
        return;
    }

    // ---------------- phase 2: emit the band's im2row rows ----------------
    // One unit = plane words (2k, 2k+1) of one output row: for a ternary row the sign pair and
    // the zero pair (two 16-byte stores 32 bytes apart), for a binary row one 16-byte store.
    const uint32_t UP = (uint32_t)g.Kp / 2;                              // units per row
    const uint32_t U = TERNARY ? (uint32_t)g.Kp : (uint32_t)g.Kp / 2;   // 16-byte chunks per row
    const uint32_t units = (uint32_t)(boh * g.OW) * UP;
    uint4* dst = out + ((size_t)n * g.OH + oh0) * g.OW * U;
    for (uint32_t q = tid; q < units; q += kPackThreads) {
        const uint32_t row = divU.div(q);
        const uint32_t k = q - row * UP;
        const uint32_t ohl = divOW.div(row);
        const int ow = (int)(row - ohl * g.OW);
        const int ih0 = (oh0 + (int)ohl) * g.SH - g.PH - ih_lo;  // window origin relative to the smem band
        const int iw0 = ow * g.SW - g.PW;
        const int base = (ih0 * g.W + iw0) * g.Cp;
        const bool interior = ih0 >= 0 && ih0 + g.KH <= nrow && iw0 >= 0 && iw0 + g.KW <= g.W;
        const int2 o = *reinterpret_cast<const int2*>(joff + 2 * k);
        uint64_t s0 = 0, s1 = 0, z0 = ~0ull, z1 = ~0ull;
        if (PAIR && interior && o.x != kPadWord) {
            // C_pack even: word 2k+1 follows word 2k in shared memory and both are real taps
            const uint4 sv = *reinterpret_cast<const uint4*>(sm_sign + base + o.x);
            s0 = ((uint64_t)sv.y << 32) | sv.x; s1 = ((uint64_t)sv.w << 32) | sv.z;
            if (TERNARY) {
                const uint4 zv = *reinterpret_cast<const uint4*>(sm_zero + base + o.x);
                z0 = ((uint64_t)zv.y << 32) | zv.x; z1 = ((uint64_t)zv.w << 32) | zv.z;
            }
        } else {
            const uint2 tp = *reinterpret_cast<const uint2*>(jtap + 2 * k);
            if (o.x != kPadWord) {
                const int ih = ih0 + (int)(tp.x >> 16), iw = iw0 + (int)(tp.x & 0xFFFF);
                if (ih >= 0 && ih < nrow && iw >= 0 && iw < g.W) { s0 = sm_sign[base + o.x]; if (TERNARY) z0 = sm_zero[base + o.x]; }
            }
            if (o.y != kPadWord) {
                const int ih = ih0 + (int)(tp.y >> 16), iw = iw0 + (int)(tp.y & 0xFFFF);
                if (ih >= 0 && ih < nrow && iw >= 0 && iw < g.W) { s1 = sm_sign[base + o.y]; if (TERNARY) z1 = sm_zero[base + o.y]; }
            }
        }
        if (TERNARY) {
            uint4* d = dst + (size_t)row * U + (k >> 1) * 4 + (k & 1);
            d[0] = make_uint4((uint32_t)s0, (uint32_t)(s0 >> 32), (uint32_t)s1, (uint32_t)(s1 >> 32));
            d[2] = make_uint4((uint32_t)z0, (uint32_t)(z0 >> 32), (uint32_t)z1, (uint32_t)(z1 >> 32));
        } else {
            dst[(size_t)row * U + k] = make_uint4((uint32_t)s0, (uint32_t)(s0 >> 32), (uint32_t)s1, (uint32_t)(s1 >> 32));
        }
    }
}

template <bool TERNARY, int LAYOUT, int VEC, int IMG_OUT = 0>
int launch_staged(tnns_cuda_ctx* ctx, const float* d_x, const float* d_thr, void* d_packed, const TnnsGeom& g, int BOH,
                  int Lmax, size_t smem, cudaStream_t stream) {
    const int nbands = (g.OH + BOH - 1) / BOH;
    const uint32_t UP = g.Kp / 2;
    const int LV = std::max(Lmax / VEC, 1);
    const bool pair = (g.Cp % 2) == 0;
    auto launch = [&](auto kern) -> int {
        // the attribute belongs to (function, device), not to a context: every caller sets the same
        // value, the device's opt-in maximum, so host threads packing layers of different band
        // sizes cannot lower each other's limit between this call and the launch
        if (smem > 48 * 1024)
            TNNS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, ctx->smem_optin)));
        kern<<<g.N * nbands, kPackThreads, smem, stream>>>(d_x, d_thr, reinterpret_cast<uint4*>(d_packed), g, BOH, nbands, Lmax,
                                                           tnns_fastdiv(UP), tnns_fastdiv(g.OW), tnns_fastdiv(LV));
        tnns_count_launch();
        TNNS_CUDA_TRY(cudaGetLastError());
        return TNNS_OK;
    };
    if (IMG_OUT) return launch(pack_staged_kernel<TERNARY, LAYOUT, VEC, false, IMG_OUT>);
    return pair ? launch(pack_staged_kernel<TERNARY, LAYOUT, VEC, true, 0>) : launch(pack_staged_kernel<TERNARY, LAYOUT, VEC, false, 0>);
}

}  // namespace

FastDiv tnns_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    if (d <= 1) { f.mul = 0; f.sh1 = 0; f.sh2 = 0; return f; }  // t=0 -> (0 + (n>>0)) >> 0 = n
    uint32_t l = 0;
    while ((1ull << l) < d) l++;
    const uint64_t m = ((1ull << 32) * ((1ull << l) - d)) / d + 1;
    f.mul = (uint32_t)m;
    f.sh1 = 1;
    f.sh2 = l - 1;
    return f;
}

// Rows of input a band of `boh` output rows touches, clipped to the image height.
static int band_input_rows(const TnnsGeom& g, int boh) { return std::min((boh - 1) * g.SH + g.KH, g.H); }

int tnns_launch_pack(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_packed,
                     const TnnsGeom& g, int layout, int algo, cudaStream_t stream) {
    const long long rows = (long long)g.N * g.OH * g.OW;
    if (rows == 0) return TNNS_OK;
    if (layout != TNNS_NCHW && layout != TNNS_NHWC && layout != TNNS_SRC_PACKED_IMAGE)
        return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    // An NCHW tensor with one pixel per image is bit-identical to its NHWC form; the
    // channel-contiguous kernel is the coalesced one for it (fully-connected layers).
    int eff_layout = layout;
    if (layout == TNNS_NCHW && g.H * g.W == 1) eff_layout = TNNS_NHWC;

    const int planes = ternary ? 2 : 1;
    // staged kernel limits: tap table fields and 32-bit chunk counters
    bool staged_ok = g.KH < 65536 && g.KW < 65536 &&
                     (long long)(g.KH * (long long)g.W + g.KW) * g.Cp < (1LL << 30);
    int BOH = 0, Lmax = 0;
    size_t smem = 0;
    if (staged_ok) {
        // bands small enough for four resident blocks per SM, and at least two blocks per SM
        const size_t budget_pref = 48 * 1024, budget_max = ctx->smem_optin;
        const int min_blk = 2;
        auto smem_for = [&](int boh) {
            return (size_t)planes * band_input_rows(g, boh) * g.W * g.Cp * 8 + (size_t)g.Kp * 8;
        };
        if (smem_for(1) > budget_max) staged_ok = false;
        else {
            BOH = g.OH;
            while (BOH > 1 && smem_for(BOH) > budget_pref) BOH = (BOH + 1) / 2;
            // enough thread blocks to fill the machine twice over, if the layer allows it
            while (BOH > 1 && (long long)g.N * ((g.OH + BOH - 1) / BOH) < (long long)min_blk * ctx->sm_count) BOH = (BOH + 1) / 2;
            Lmax = band_input_rows(g, BOH) * g.W;
            smem = smem_for(BOH);
            if ((unsigned long long)BOH * g.OW * g.Kp >= (1ull << 31)) staged_ok = false;
        }
    }
    if ((algo == TNNS_PACK_STAGED || layout == TNNS_SRC_PACKED_IMAGE) && !staged_ok)
        return tnns_fail(TNNS_ERR_UNSUPPORTED, "staged pack kernel cannot hold this geometry in shared memory");
    const bool use_staged = (algo == TNNS_PACK_STAGED) || (algo == TNNS_PACK_AUTO && staged_ok);

    if (!use_staged) {
        const long long total = rows * g.Kp;
        const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 32);
        uint64_t* o = reinterpret_cast<uint64_t*>(d_packed);
        if (ternary) {
            if (layout == TNNS_NHWC) pack_gather_kernel<true, true><<<blocks, 256, 0, stream>>>(d_x, d_thr, o, g, total);
            else pack_gather_kernel<true, false><<<blocks, 256, 0, stream>>>(d_x, d_thr, o, g, total);
        } else {
            if (layout == TNNS_NHWC) pack_gather_kernel<false, true><<<blocks, 256, 0, stream>>>(d_x, d_thr, o, g, total);
            else pack_gather_kernel<false, false><<<blocks, 256, 0, stream>>>(d_x, d_thr, o, g, total);
        }
        tnns_count_launch();
        TNNS_CUDA_TRY(cudaGetLastError());
        return TNNS_OK;
    }

    if (layout == TNNS_SRC_PACKED_IMAGE)
        return ternary ? launch_staged<true, 2, 1>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream)
                       : launch_staged<false, 2, 1>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream);
    if (eff_layout == TNNS_NHWC) {
        return ternary ? launch_staged<true, 1, 1>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream)
                       : launch_staged<false, 1, 1>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream);
    }
    // NCHW: 128-bit loads need every (channel plane, band start) to be 16-byte aligned
    const bool vec4 = (g.W % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_x) & 15) == 0);
    if (vec4)
        return ternary ? launch_staged<true, 0, 4>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream)
                       : launch_staged<false, 0, 4>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream);
    return ternary ? launch_staged<true, 0, 1>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream)
                   : launch_staged<false, 0, 1>(ctx, d_x, d_thr, d_packed, g, BOH, Lmax, smem, stream);
}

// Quantise only: fp32 tensor -> packed image.  Runs the staged kernel on the geometry of a 1x1
// stride-1 window (one band = BOH image rows, no halo) with the IMG_OUT tail.
int tnns_launch_quantise(tnns_cuda_ctx* ctx, bool ternary, const float* d_x, const float* d_thr, void* d_image, int N, int C, int H,
                         int W, int layout, cudaStream_t stream, int format) {
    if (N == 0) return TNNS_OK;
    if (format != TNNS_IMG_PLANES && format != TNNS_IMG_E2M1) return tnns_fail(TNNS_ERR_INVALID, "unknown image format %d", format);
    if (format == TNNS_IMG_E2M1 && !ternary) return tnns_fail(TNNS_ERR_UNSUPPORTED, "the 4-bit image holds ternary activations only");
    if (tnns_quantise_tma_supported(d_x, H, W, layout))
        return tnns_launch_quantise_tma(ctx, ternary, d_x, d_thr, d_image, N, C, H, W, stream, format);
    // (a 1x1 image is the same memory in both layouts: fully connected layers take this form too)
    if ((layout == TNNS_NHWC || H * W == 1) && tnns_quantise_tma_nhwc_supported(d_x, N, C, H, W))
        return tnns_launch_quantise_tma(ctx, ternary, d_x, d_thr, d_image, N, C, H, W, stream, format, 0, 0, TNNS_NHWC);
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    TnnsGeom g;
    g.N = N; g.C = C; g.H = H; g.W = W; g.KN = 1; g.KH = g.KW = 1; g.PH = g.PW = 0; g.SH = g.SW = 1;
    g.OH = H; g.OW = W;
    g.Cp = (C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS;
    g.Kw = g.Cp;
    g.Kp = 4 * ((g.Kw + 3) / 4);
    const int planes = ternary ? 2 : 1;
    auto smem_for = [&](int boh) { return (size_t)planes * boh * W * g.Cp * 8 + (size_t)g.Kp * 8; };
    if (smem_for(1) > ctx->smem_optin) return tnns_fail(TNNS_ERR_UNSUPPORTED, "one image row of %d x %d channels does not fit shared memory", W, C);
    int BOH = H;
    while (BOH > 1 && smem_for(BOH) > 48 * 1024) BOH = (BOH + 1) / 2;
    // at least two blocks per SM, but never bands so small that a block's 256 threads lack an
    // item each (an item = 4 pixels x 64 channels in the vector form)
    while (BOH > 1 && (long long)N * ((H + BOH - 1) / BOH) < 2LL * ctx->sm_count &&
           (long long)(BOH / 2) * W * g.Cp >= 4LL * kPackThreads)
        BOH = (BOH + 1) / 2;
    const int Lmax = BOH * W;
    const size_t smem = smem_for(BOH);
    int eff_layout = layout;
    if (layout == TNNS_NCHW && H * W == 1) eff_layout = TNNS_NHWC;
    const bool vec4 = (W % 4 == 0) && ((reinterpret_cast<uintptr_t>(d_x) & 15) == 0);
    if (format == TNNS_IMG_E2M1) {
        if (eff_layout == TNNS_NHWC) return launch_staged<true, 1, 1, TNNS_IMG_E2M1>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream);
        if (vec4) return launch_staged<true, 0, 4, TNNS_IMG_E2M1>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream);
        return launch_staged<true, 0, 1, TNNS_IMG_E2M1>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream);
    }
    if (eff_layout == TNNS_NHWC)
        return ternary ? launch_staged<true, 1, 1, TNNS_IMG_PLANES>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream)
                       : launch_staged<false, 1, 1, TNNS_IMG_PLANES>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream);
    if (vec4)
        return ternary ? launch_staged<true, 0, 4, TNNS_IMG_PLANES>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream)
                       : launch_staged<false, 0, 4, TNNS_IMG_PLANES>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream);
    return ternary ? launch_staged<true, 0, 1, TNNS_IMG_PLANES>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream)
                   : launch_staged<false, 0, 1, TNNS_IMG_PLANES>(ctx, d_x, d_thr, d_image, g, BOH, Lmax, smem, stream);
}

// ---------------------------------------------------------------------------------------
// Weight packing on the device (once per model): fp32 [KN][C][KH][KW] + one threshold per
// kernel -> packing-2 rows (ternary) or one-plane rows (binary), the layouts of
// ternarize_opt_avx2 / binarize_opt_avx2 (reference: src/utils.c:468-521, 634-675).  One thread
// per plane word.  Ternary decision order as in the reference: v > t is +1, else v < -t is -1,
// else 0; channels past C are quantised as the value 0.0.
// ---------------------------------------------------------------------------------------
namespace {
template <bool TERNARY>
__global__ void pack_weights_kernel(const float* __restrict__ w, const float* __restrict__ thr, uint64_t* __restrict__ out, int KN,
                                    int C, int KHW, int Cp, int Kw, int Kp) {
    const long long total = (long long)KN * Kp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int kn = (int)(i / Kp), j = (int)(i - (long long)kn * Kp);
        uint64_t sign = 0, zero = TERNARY ? ~0ull : 0ull;  // pad-to-four words are zeros of the alphabet
        if (j < Kw) {
            const int ic = j % Cp, tap = j / Cp;
            const float t = thr[kn];
            zero = 0;
            for (int b = 0; b < TNNS_WORD_BITS; b++) {
                const int c = ic * TNNS_WORD_BITS + b;
                if (TERNARY) {
                    const float v = c < C ? w[((size_t)kn * C + c) * KHW + tap] : 0.0f;
                    if (v > t) continue;
                    if (v < -t) sign |= 1ull << b;
                    else zero |= 1ull << b;
                } else if (c < C && w[((size_t)kn * C + c) * KHW + tap] < t) {
                    sign |= 1ull << b;
                }
            }
        }
        if (TERNARY) {
            uint64_t* row = out + (size_t)kn * 2 * Kp + (size_t)(j >> 2) * 8 + (j & 3);
            row[0] = sign;
            row[4] = zero;
        } else {
            out[(size_t)kn * Kp + j] = sign;
        }
    }
}
}  // namespace

int tnns_launch_pack_weights(tnns_cuda_ctx* ctx, bool ternary, const float* d_w, const float* d_thr, void* d_packed, int KN, int C,
                             int KH, int KW, cudaStream_t stream) {
    const int Cp = (C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS, Kw = KH * KW * Cp, Kp = 4 * ((Kw + 3) / 4);
    const long long total = (long long)KN * Kp;
    const int blocks = (int)std::min<long long>((total + 127) / 128, (long long)ctx->sm_count * 16);
    uint64_t* o = reinterpret_cast<uint64_t*>(d_packed);
    if (ternary) pack_weights_kernel<true><<<blocks, 128, 0, stream>>>(d_w, d_thr, o, KN, C, KH * KW, Cp, Kw, Kp);
    else pack_weights_kernel<false><<<blocks, 128, 0, stream>>>(d_w, d_thr, o, KN, C, KH * KW, Cp, Kw, Kp);
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}
