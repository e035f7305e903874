// Layers with few input channels (the first layer of an image network: C = 3) as a dense GEMM.
//
// The reference pads every filter tap to 64 channels (`C_pack = ceil(C/64)`, plane word
// `j = (kh*KW + kw)*C_pack + ic`, src/tnns/ternarize2row_avx2.c:285-313), so a 7x7 filter over 3 channels
// is a row of 49 plane words = 3136 positions of which 147 can be non-zero, and every route that follows
// that layout multiplies (and fetches) the 2989 zeros as well.  Zeros contribute nothing to the sum, so
// the same output comes from a row that holds only the real positions: element `e = (kh*KW + kw)*C + c`,
// K = KH*KW*C, rounded up to a channel count the tensor-core GEMM takes (64, 128 or a multiple of 256).
// Two small kernels make that a layer the existing GEMMs run unchanged:
//   * repack_weights_dense_kernel (once per weight upload) writes the packed kernel of a VIRTUAL layer
//     -- 1x1 filter, K' channels -- in the reference's own packed format; the ordinary upload path then
//     builds its operand images;
//   * dense_quantise_kernel (per call) quantises the fp32 input with the reference's rule
//     (src/tnns/ternarize2row_avx2.c:438-452) and writes, per output pixel, the K' positions of its window
//     as the 4-bit image of that virtual layer (positions outside the input or past K: zero).
// The GEMM is then the copy-engine fed one on a 1x1, stride-1 layer over N x OH x OW "pixels" of K'
// "channels", with every epilogue it has.  Ternary activations only (TNN, TBN): a binary window pads
// with +1, which the zero positions of this form cannot express.
#include <algorithm>

#include "internal.h"

namespace {

// bit `c` of plane word (tap, c / 64) of the parent row -> bit e % 64 of virtual plane word e / 64
__global__ void repack_weights_dense_kernel(const uint64_t* __restrict__ packed, uint64_t* __restrict__ out, int KN, int Kp, int Cp, int C,
                                            int T, int two_planes, int Kp_out) {
    const long long total = (long long)KN * Kp_out;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int kn = (int)(i / Kp_out), jo = (int)(i - (long long)kn * Kp_out);
        const uint64_t* row = packed + (size_t)kn * Kp * (two_planes ? 2 : 1);
        uint64_t sign = 0, zero = ~0ull;  // positions past K: ternary 0 (a binary plane reads +1 there; the activations are 0)
        for (int b = 0; b < 64; b++) {
            const int e = jo * 64 + b;
            if (e >= T * C) break;
            const int tap = e / C, c = e - tap * C;
            const int j = tap * Cp + (c >> 6), bit = c & 63;
            if (two_planes) {
                const uint64_t s = row[(j >> 2) * 8 + (j & 3)], z = row[(j >> 2) * 8 + 4 + (j & 3)];
                sign |= ((s >> bit) & 1ull) << b;
                zero = (zero & ~(1ull << b)) | (((z >> bit) & 1ull) << b);
            } else {
                sign |= ((row[j] >> bit) & 1ull) << b;
            }
        }
        if (two_planes) {
            uint64_t* orow = out + (size_t)kn * Kp_out * 2;
            orow[(jo >> 2) * 8 + (jo & 3)] = sign;
            orow[(jo >> 2) * 8 + 4 + (jo & 3)] = zero;
        } else {
            out[(size_t)kn * Kp_out + jo] = sign;
        }
    }
}

// One thread = one output pixel's 32 consecutive positions (one 16-byte piece of its row of the virtual image).
// Neighbouring threads take neighbouring output pixels of the same piece: for every position their loads are SW
// floats apart (coalesced along the input row), and their 16-byte stores one image row (K'/2 bytes) apart.
// Pieces that lie entirely past K are written as zeros (binary weights read +1 there, not 0).  The walk over
// (kh, kw, c) keeps a running pointer and a running "inside the input" flag, so a position costs its load, two
// additions, two funnel shifts and the flag.
template <bool NHWC>
__global__ void __launch_bounds__(256)
dense_quantise_kernel(const float* __restrict__ x, const float* __restrict__ thr, uint4* __restrict__ img, TnnsGeom g, int K, int groups32,
                      FastDiv div_rows, FastDiv div_ow, FastDiv div_ohw, FastDiv div_c, FastDiv div_kw, long long total) {
    const long long cstride = NHWC ? 1 : (long long)g.H * g.W;   // one channel further
    const long long pstride = NHWC ? g.C : 1;                    // one input pixel to the right
    const long long rstride = pstride * g.W;                     // one input row down
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int grp = (int)div_rows.div((uint32_t)i);
        const uint32_t row = (uint32_t)i - (uint32_t)grp * div_rows.d;
        const uint32_t n = div_ohw.div(row);
        const uint32_t rem = row - n * (uint32_t)(g.OH * g.OW);
        const int oh = (int)div_ow.div(rem), ow = (int)(rem - (uint32_t)oh * g.OW);
        const float t = __ldg(thr + n) + 0.0f;  // + 0.0f: a threshold of -0 behaves as +0 in every compare
        const int ih0 = oh * g.SH - g.PH, iw0 = ow * g.SW - g.PW;
        const int e0 = grp * 32;
        if (e0 >= K) {
            img[(size_t)row * groups32 + grp] = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        // position e = (kh*KW + kw)*C + c, walked from the piece's last position down so that position b ends at bit b
        int e = min(e0 + 31, K - 1);
        const int tap = (int)div_c.div((uint32_t)e);
        int c = e - tap * g.C;
        int kh = (int)div_kw.div((uint32_t)tap), kw = tap - kh * g.KW;
        const float* px = x + (size_t)n * g.C * g.H * g.W + (long long)c * cstride + (long long)(ih0 + kh) * rstride + (long long)(iw0 + kw) * pstride;
        bool ok = (unsigned)(ih0 + kh) < (unsigned)g.H && (unsigned)(iw0 + kw) < (unsigned)g.W;
        uint32_t sg = 0, nz = 0, ins = 0;
        for (; e >= e0; e--) {
            const float v = ok ? __ldg(px) : 0.0f;
            sg = __funnelshift_l(__float_as_uint(v + t), sg, 1);
            nz = __funnelshift_l(__float_as_uint(t - fabsf(v)), nz, 1);
            ins = (ins << 1) | (ok ? 1u : 0u);
            if (--c >= 0) {
                px -= cstride;
            } else {
                c = g.C - 1;
                if (--kw >= 0) {
                    px += (long long)(g.C - 1) * cstride - pstride;
                } else {
                    kw = g.KW - 1;
                    kh--;
                    px += (long long)(g.C - 1) * cstride - rstride + (long long)(g.KW - 1) * pstride;
                }
                ok = (unsigned)(ih0 + kh) < (unsigned)g.H && (unsigned)(iw0 + kw) < (unsigned)g.W;
            }
        }
        // positions outside the input are the reference's padding: zero whatever the threshold (a negative one
        // would otherwise call the 0 read there "non-zero"); positions past K sit in the high bits, which stay 0
        sg &= ins;
        nz &= ins;
        uint32_t w4[4];
        tnns_expand32_f4(sg, ~nz, w4);
        img[(size_t)row * groups32 + grp] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
}

}  // namespace

// K' of the virtual layer: the real positions rounded up to a pixel size the copy-engine fed GEMM takes
int tnns_dense_channels(int C, int KH, int KW) {
    const long long K = (long long)C * KH * KW;
    if (K <= 64) return 64;
    if (K <= 128) return 128;
    return (int)(((K + 255) / 256) * 256);
}

// Taken for ternary activations where at most a quarter of the padded row is real and the dense row stays short.
bool tnns_dense_eligible(int type, int C, int KH, int KW) {
    if (!(type == TNN || type == TBN) || C <= 0 || C > 16 || KH <= 0 || KW <= 0) return false;
    const long long K = (long long)C * KH * KW;
    return K <= 1024 && (long long)tnns_dense_channels(C, KH, KW) * 2 <= 64LL * KH * KW;
}

// Packed kernel of the virtual layer (device memory, the reference's layout for `w->type`, Kp_out plane words per row).
int tnns_launch_repack_weights_dense(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, uint64_t* d_out, int Kp_out) {
    (void)ctx;
    const bool two = (w->type == TNN || w->type == BTN);
    const long long total = (long long)w->KN * Kp_out;
    const int blocks = (int)std::min<long long>((total + 127) / 128, 4096);
    repack_weights_dense_kernel<<<blocks, 128>>>(w->d_packed, d_out, w->KN, w->Kp, w->Cp, w->C, w->KH * w->KW, two ? 1 : 0, Kp_out);
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}

int tnns_launch_dense_quantise(tnns_cuda_ctx* ctx, const float* d_x, const float* d_thr, void* d_img, const TnnsGeom& g, int Kd, int layout,
                               cudaStream_t stream) {
    const long long rows = (long long)g.N * g.OH * g.OW;
    if (rows == 0) return TNNS_OK;
    const int groups32 = Kd / 32;
    const int K = g.C * g.KH * g.KW;
    const long long total = rows * groups32;
    if (rows >= 0x7FFFFFFFLL || total >= 0xFFFFFFFFLL) return tnns_fail(TNNS_ERR_UNSUPPORTED, "too many output pixels for the dense first-layer form");
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 16);
    const FastDiv dg = tnns_fastdiv((uint32_t)rows), dow = tnns_fastdiv((uint32_t)g.OW), dohw = tnns_fastdiv((uint32_t)(g.OH * g.OW)),
                  dc = tnns_fastdiv((uint32_t)g.C), dkw = tnns_fastdiv((uint32_t)g.KW);
    if (layout == TNNS_NHWC)
        dense_quantise_kernel<true><<<blocks, 256, 0, stream>>>(d_x, d_thr, reinterpret_cast<uint4*>(d_img), g, K, groups32, dg, dow, dohw, dc, dkw, total);
    else
        dense_quantise_kernel<false><<<blocks, 256, 0, stream>>>(d_x, d_thr, reinterpret_cast<uint4*>(d_img), g, K, groups32, dg, dow, dohw, dc, dkw, total);
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}
