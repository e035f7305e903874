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

#include "internal.h"

namespace {

constexpr int kPackThreads = 256;

__device__ __forceinline__ void tern_accum(float v, float t, float nt, uint32_t bit, uint32_t& sign, uint32_t& nz) {
    // sign iff v < -t ; non-zero iff v < -t or v > t  (src/tnns/ternarize2row_avx2.c:444-449)
    const bool neg = v < nt;
    const bool pos = v > t;
    if (neg) sign |= bit;
    if (neg || pos) nz |= bit;
}

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
//     planes * Lmax * Cp   uint64   packed pixels of the band (plane 0 sign, plane 1 zero)
//     Kp                   uint32   tap table: j -> (kh<<24 | kw<<16 | ic)
// LAYOUT 0: NCHW, one thread packs VEC neighbouring pixels over 64 channels (loads are
//           coalesced along W, channel stride H*W).
// LAYOUT 1: NHWC, one warp packs 32 neighbouring channels of a pixel with __ballot_sync.
// ---------------------------------------------------------------------------------------
template <bool TERNARY, int LAYOUT, int VEC>
__global__ void __launch_bounds__(kPackThreads)
pack_staged_kernel(const float* __restrict__ x, const float* __restrict__ thr, uint4* __restrict__ out, TnnsGeom g,
                   int BOH, int nbands, int Lmax, FastDiv divU, FastDiv divOW, FastDiv divL) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int PLANES = TERNARY ? 2 : 1;
    uint64_t* sm_sign = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* sm_zero = sm_sign + (size_t)Lmax * g.Cp;  // only valid when TERNARY
    uint32_t* jtab = reinterpret_cast<uint32_t*>(sm_sign + (size_t)PLANES * Lmax * g.Cp);

    const int tid = threadIdx.x;
    const int n = blockIdx.x / nbands;
    const int band = blockIdx.x - n * nbands;
    const int oh0 = band * BOH;
    const int boh = min(BOH, g.OH - oh0);
    const int ih_lo = max(oh0 * g.SH - g.PH, 0);
    const int ih_hi = min((oh0 + boh - 1) * g.SH - g.PH + g.KH, g.H);  // exclusive
    const int L = max(ih_hi - ih_lo, 0) * g.W;                          // pixels held in smem
    const float t = thr[n], nt = -t;

    for (int j = tid; j < g.Kp; j += kPackThreads) {
        uint32_t e = 0xFFFFFFFFu;  // words added by the pad-to-four
        if (j < g.Kw) {
            const int ic = j % g.Cp, kw = (j / g.Cp) % g.KW, kh = j / (g.Cp * g.KW);
            e = ((uint32_t)kh << 24) | ((uint32_t)kw << 16) | (uint32_t)ic;
        }
        jtab[j] = e;
    }

    // ---------------- phase 1: quantise + pack the band's input pixels ----------------
    if (LAYOUT == 0) {
        const size_t HW = (size_t)g.H * g.W;
        const int LV = L / VEC;  // VEC divides L by construction (host checks W % VEC == 0)
        const int items = g.Cp * LV;
        for (int id = tid; id < items; id += kPackThreads) {
            const int ic = (LV == divL.d) ? (int)divL.div((uint32_t)id) : id / LV;
            const int p = (id - ic * LV) * VEC;
            const int nch = min(TNNS_WORD_BITS, g.C - ic * TNNS_WORD_BITS);
            const float* src = x + ((size_t)n * g.C + (size_t)ic * TNNS_WORD_BITS) * HW + (size_t)ih_lo * g.W + p;
            uint32_t sg[VEC][2], nzb[VEC][2];
#pragma unroll
            for (int v = 0; v < VEC; v++) { sg[v][0] = sg[v][1] = 0; nzb[v][0] = nzb[v][1] = 0; }
#pragma unroll
            for (int half = 0; half < 2; half++) {
                if (nch >= 32 * half + 32) {
#pragma unroll 16
                    for (int b = 0; b < 32; b++) {
                        const float* q = src + (size_t)(32 * half + b) * HW;
                        float vals[VEC];
                        if (VEC == 4) {
                            const float4 f = __ldg(reinterpret_cast<const float4*>(q));
                            vals[0] = f.x; vals[1 % VEC] = f.y; vals[2 % VEC] = f.z; vals[3 % VEC] = f.w;
                        } else {
                            vals[0] = __ldg(q);
                        }
#pragma unroll
                        for (int v = 0; v < VEC; v++) {
                            if (TERNARY) tern_accum(vals[v], t, nt, 1u << b, sg[v][half], nzb[v][half]);
                            else if (vals[v] < t) sg[v][half] |= 1u << b;
                        }
                    }
                } else {
                    const int lim = nch - 32 * half;  // may be <= 0
                    for (int b = 0; b < lim; b++) {
                        const float* q = src + (size_t)(32 * half + b) * HW;
#pragma unroll
                        for (int v = 0; v < VEC; v++) {
                            const float val = __ldg(q + v);
                            if (TERNARY) tern_accum(val, t, nt, 1u << b, sg[v][half], nzb[v][half]);
                            else if (val < t) sg[v][half] |= 1u << b;
                        }
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < VEC; v++) {
                const size_t at = (size_t)(p + v) * g.Cp + ic;
                sm_sign[at] = ((uint64_t)sg[v][1] << 32) | sg[v][0];
                if (TERNARY) sm_zero[at] = ~(((uint64_t)nzb[v][1] << 32) | nzb[v][0]);
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

    // ---------------- phase 2: emit the band's im2row rows ----------------
    const uint32_t U = TERNARY ? (uint32_t)g.Kp : (uint32_t)g.Kp / 2;  // 16-byte chunks per row
    const uint32_t chunks = (uint32_t)(boh * g.OW) * U;
    uint4* dst = out + ((size_t)n * g.OH + oh0) * g.OW * U;
    for (uint32_t q = tid; q < chunks; q += kPackThreads) {
        const uint32_t row = divU.div(q);
        const uint32_t u = q - row * U;
        const uint32_t ohl = divOW.div(row);
        const int ow = (int)(row - ohl * g.OW);
        const int ihb = (oh0 + (int)ohl) * g.SH - g.PH - ih_lo;  // relative to the smem band
        const int iwb = ow * g.SW - g.PW;
        int plane, j0;
        if (TERNARY) { plane = (u >> 1) & 1; j0 = (int)((u >> 2) * 4 + (u & 1) * 2); }
        else { plane = 0; j0 = (int)(2 * u); }
        const uint64_t* sm = plane ? sm_zero : sm_sign;
        const uint64_t padv = plane ? ~0ull : 0ull;
        uint64_t w[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const uint32_t e = jtab[j0 + k];
            uint64_t val = padv;
            if (e != 0xFFFFFFFFu) {
                const int ihr = ihb + (int)(e >> 24);
                const int iw = iwb + (int)((e >> 16) & 0xFF);
                const int ic = (int)(e & 0xFFFF);
                // ihr is relative to ih_lo; rows above/below the image fall outside [0, ih_hi-ih_lo)
                if (ihr >= 0 && ihr < ih_hi - ih_lo && iw >= 0 && iw < g.W) val = sm[(size_t)(ihr * g.W + iw) * g.Cp + ic];
            }
            w[k] = val;
        }
        dst[q] = make_uint4((uint32_t)w[0], (uint32_t)(w[0] >> 32), (uint32_t)w[1], (uint32_t)(w[1] >> 32));
    }
}

template <bool TERNARY, int LAYOUT, int VEC>
int launch_staged(tnns_cuda_ctx* ctx, const float* d_x, const float* d_thr, void* d_packed, const TnnsGeom& g, int BOH,
                  int Lmax, size_t smem, cudaStream_t stream) {
    auto kern = pack_staged_kernel<TERNARY, LAYOUT, VEC>;
    if (smem > 48 * 1024) TNNS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int nbands = (g.OH + BOH - 1) / BOH;
    const uint32_t U = TERNARY ? g.Kp : g.Kp / 2;
    const int LV = std::max(Lmax / VEC, 1);
    kern<<<g.N * nbands, kPackThreads, smem, stream>>>(d_x, d_thr, reinterpret_cast<uint4*>(d_packed), g, BOH, nbands, Lmax,
                                                       tnns_fastdiv(U), tnns_fastdiv(g.OW), tnns_fastdiv(LV));
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
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
    if (layout != TNNS_NCHW && layout != TNNS_NHWC) return tnns_fail(TNNS_ERR_INVALID, "unknown layout %d", layout);
    // An NCHW tensor with one pixel per image is bit-identical to its NHWC form; the
    // channel-contiguous kernel is the coalesced one for it (fully-connected layers).
    int eff_layout = layout;
    if (layout == TNNS_NCHW && g.H * g.W == 1) eff_layout = TNNS_NHWC;

    const int planes = ternary ? 2 : 1;
    // staged kernel limits: tap table fields and 32-bit chunk counters
    bool staged_ok = g.KH < 256 && g.KW < 256 && g.Cp < 65536;
    int BOH = 0, Lmax = 0;
    size_t smem = 0;
    if (staged_ok) {
        const size_t budget_pref = 64 * 1024, budget_max = ctx->smem_optin;
        auto smem_for = [&](int boh) {
            return (size_t)planes * band_input_rows(g, boh) * g.W * g.Cp * 8 + (size_t)g.Kp * 4;
        };
        if (smem_for(1) > budget_max) staged_ok = false;
        else {
            BOH = g.OH;
            while (BOH > 1 && smem_for(BOH) > budget_pref) BOH = (BOH + 1) / 2;
            // enough thread blocks to fill the machine twice over, if the layer allows it
            while (BOH > 1 && (long long)g.N * ((g.OH + BOH - 1) / BOH) < 2LL * ctx->sm_count) BOH = (BOH + 1) / 2;
            Lmax = band_input_rows(g, BOH) * g.W;
            smem = smem_for(BOH);
            if ((unsigned long long)BOH * g.OW * g.Kp >= (1ull << 31)) staged_ok = false;
        }
    }
    if (algo == TNNS_PACK_STAGED && !staged_ok)
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
