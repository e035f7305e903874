/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the FasterTNN "final" (packing-2)
 * ternary/binary conv + GEMM path.  Nothing in the shipped library links, loads or
 * calls this file; only the test-suite, the smoke check and the CPU-baseline leg of
 * the benchmark may.
 *
 * Parity pin: this restatement is compared word-for-word / bit-for-bit against the
 * reference's own objects (compiled by oracle/Makefile into oracle/_ref/) on the 12
 * shapes of the reference's test table (include/timing/shapes_test.h:6-17), for all
 * four network types, and against committed SHA-256 digests of those outputs
 * (tests/golden/).
 *
 * Every function is written in "gather" form (one output word / one output value at
 * a time) and is deliberately scalar: it is the specification, not a fast path.
 *
 * Citations are to files of the reference project (fpgasystems/FasterTNN).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define WORD_BITS 64 /* include/tnns/common.h:12  (cntbits) */

static int ceil_div(int a, int b) { return (a + b - 1) / b; }
static int pad4(int k) { return 4 * ((k + 3) / 4); }

/* Output extent of the convolution; integer division as in
 * src/tnns/tnns_cpu_mm_p2.c:7-10. */
int orc_out_dim(int in, int pad, int k, int stride) { return (in + 2 * pad - k) / stride + 1; }

/* 64-bit words per bit-plane and row before / after padding to a multiple of four
 * (src/tnns/ternarize2row_avx2.c:730-732, src/tnns/binarize2row_avx2.c:146). */
int orc_kw(int C, int KH, int KW) { return KH * KW * ceil_div(C, WORD_BITS); }
int orc_kp(int C, int KH, int KW) { return pad4(orc_kw(C, KH, KW)); }

/* Position of plane word j inside a packing-2 row: alternating groups of four sign
 * words and four zero words (src/tnns/ternarize2row_avx2.c:297-304). */
static inline size_t p2_sign_at(int j) { return (size_t)(j / 4) * 8 + (size_t)(j % 4); }

/* Pack the 64 channels [64*ic, 64*ic+64) of one pixel.  Ternary rule:
 * sign bit iff v < -t, zero bit iff neither v < -t nor v > t
 * (src/tnns/ternarize2row_avx2.c:438-452); channels past C read as zeros of the
 * ternary alphabet (zero bit set).  `cstride` is the distance between channels. */
static void pack_ternary_pixel(const float* px, size_t cstride, int nch, float t,
                               uint64_t* sign, uint64_t* zero) {
    uint64_t s = 0, z = ~(uint64_t)0;
    for (int b = 0; b < nch; b++) {
        float v = px[(size_t)b * cstride];
        if (v < -t) { s |= (uint64_t)1 << b; z &= ~((uint64_t)1 << b); }
        else if (v > t) { z &= ~((uint64_t)1 << b); }
    }
    *sign = s; *zero = z;
}

/* Binary rule: bit set (value -1) iff v < t, strictly
 * (src/tnns/binarize2row_avx2.c:15-22).  Missing channels stay 0 (= +1). */
static uint64_t pack_binary_pixel(const float* px, size_t cstride, int nch, float t) {
    uint64_t s = 0;
    for (int b = 0; b < nch; b++)
        if (px[(size_t)b * cstride] < t) s |= (uint64_t)1 << b;
    return s;
}

/*
 * Ternarize + bit-pack + im2row.  Follows t2r_p2_opt
 * (src/tnns/ternarize2row_avx2.c:715-803) including its prefill convention
 * (sign = 0 / zero = all-ones for padding pixels and for the words added by the
 * pad-to-4, :748-755).  x is NCHW, thr has one symmetric threshold per image.
 * Returns N*OH*OW rows of 2*Kp int64 (caller frees).
 */
int64_t* orc_t2r(const float* x, const float* thr, int N, int C, int H, int W, int PH, int PW,
                 int KH, int KW, int SH, int SW) {
    const int Cp = ceil_div(C, WORD_BITS), Kw = KH * KW * Cp, Kp = pad4(Kw);
    const int OH = orc_out_dim(H, PH, KH, SH), OW = orc_out_dim(W, PW, KW, SW);
    const size_t rows = (size_t)N * OH * OW, pitch = 2 * (size_t)Kp;
    uint64_t* out = (uint64_t*)aligned_alloc(64, ((rows * pitch * 8 + 63) / 64) * 64 + 64);
    if (!out) return NULL;
    for (size_t r = 0; r < rows; r++) {
        const int n = (int)(r / ((size_t)OH * OW));
        const int oh = (int)((r / OW) % OH), ow = (int)(r % OW);
        uint64_t* row = out + r * pitch;
        for (int j = 0; j < Kp; j++) {
            uint64_t s = 0, z = ~(uint64_t)0;
            if (j < Kw) {
                const int ic = j % Cp, kw = (j / Cp) % KW, kh = j / (Cp * KW);
                const int ih = oh * SH + kh - PH, iw = ow * SW + kw - PW;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                    int nch = C - ic * WORD_BITS;
                    if (nch > WORD_BITS) nch = WORD_BITS;
                    const float* px = x + (((size_t)n * C + (size_t)ic * WORD_BITS) * H + ih) * W + iw;
                    pack_ternary_pixel(px, (size_t)H * W, nch, thr[n], &s, &z);
                }
            }
            row[p2_sign_at(j)] = s;
            row[p2_sign_at(j) + 4] = z;
        }
    }
    return (int64_t*)out;
}

/*
 * Binarize + bit-pack + im2row.  Follows b2r (src/tnns/binarize2row_avx2.c:131-199):
 * one plane, Kp words per row, buffer zero-filled so padding pixels, channel tails
 * and pad-to-4 words all read as +1 (:151).
 */
int64_t* orc_b2r(const float* x, const float* thr, int N, int C, int H, int W, int PH, int PW,
                 int KH, int KW, int SH, int SW) {
    const int Cp = ceil_div(C, WORD_BITS), Kw = KH * KW * Cp, Kp = pad4(Kw);
    const int OH = orc_out_dim(H, PH, KH, SH), OW = orc_out_dim(W, PW, KW, SW);
    const size_t rows = (size_t)N * OH * OW;
    uint64_t* out = (uint64_t*)aligned_alloc(64, ((rows * Kp * 8 + 63) / 64) * 64 + 64);
    if (!out) return NULL;
    for (size_t r = 0; r < rows; r++) {
        const int n = (int)(r / ((size_t)OH * OW));
        const int oh = (int)((r / OW) % OH), ow = (int)(r % OW);
        for (int j = 0; j < Kp; j++) {
            uint64_t s = 0;
            if (j < Kw) {
                const int ic = j % Cp, kw = (j / Cp) % KW, kh = j / (Cp * KW);
                const int ih = oh * SH + kh - PH, iw = ow * SW + kw - PW;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                    int nch = C - ic * WORD_BITS;
                    if (nch > WORD_BITS) nch = WORD_BITS;
                    const float* px = x + (((size_t)n * C + (size_t)ic * WORD_BITS) * H + ih) * W + iw;
                    s = pack_binary_pixel(px, (size_t)H * W, nch, thr[n]);
                }
            }
            out[r * Kp + j] = s;
        }
    }
    return (int64_t*)out;
}

/*
 * Host weight packers.  Ternary follows ternarize_opt_avx2 (src/utils.c:468-521):
 * w is [KN][C][KH][KW]; plane word j = (kh*KW+kw)*C_pack + ic (:511) goes to the
 * packing-2 position of row kn (:512-514).  Its decision order differs from the
 * activation rule: v > t is tested first (:501-507), and channels past C are fed
 * the value 0.0 through the same test (:497-500).
 */
int64_t* orc_pack_w_ternary(const float* w, const float* thr, int KN, int C, int KH, int KW) {
    const int Cp = ceil_div(C, WORD_BITS), Kw = KH * KW * Cp, Kp = pad4(Kw);
    const size_t pitch = 2 * (size_t)Kp;
    uint64_t* out = (uint64_t*)aligned_alloc(64, (((size_t)KN * pitch * 8 + 63) / 64) * 64 + 64);
    if (!out) return NULL;
    for (int kn = 0; kn < KN; kn++) {
        uint64_t* row = out + (size_t)kn * pitch;
        for (int j = 0; j < Kp; j++) { row[p2_sign_at(j)] = 0; row[p2_sign_at(j) + 4] = ~(uint64_t)0; }
        for (int j = 0; j < Kw; j++) {
            const int ic = j % Cp, kw = (j / Cp) % KW, kh = j / (Cp * KW);
            uint64_t s = 0, z = 0;
            for (int b = 0; b < WORD_BITS; b++) {
                const int c = ic * WORD_BITS + b;
                const float v = c < C ? w[(((size_t)kn * C + c) * KH + kh) * KW + kw] : 0.0f;
                if (v > thr[kn]) { /* +1: both bits clear */ }
                else if (v < -thr[kn]) s |= (uint64_t)1 << b;
                else z |= (uint64_t)1 << b;
            }
            row[p2_sign_at(j)] = s;
            row[p2_sign_at(j) + 4] = z;
        }
    }
    return (int64_t*)out;
}

/* Binary weights follow binarize_opt_avx2 (src/utils.c:634-675): Kp words per
 * kernel, word j at kn*Kp + j, bit iff w < thr[kn]. */
int64_t* orc_pack_w_binary(const float* w, const float* thr, int KN, int C, int KH, int KW) {
    const int Cp = ceil_div(C, WORD_BITS), Kw = KH * KW * Cp, Kp = pad4(Kw);
    uint64_t* out = (uint64_t*)aligned_alloc(64, (((size_t)KN * Kp * 8 + 63) / 64) * 64 + 64);
    if (!out) return NULL;
    memset(out, 0, (size_t)KN * Kp * 8);
    for (int kn = 0; kn < KN; kn++)
        for (int j = 0; j < Kw; j++) {
            const int ic = j % Cp, kw = (j / Cp) % KW, kh = j / (Cp * KW);
            uint64_t s = 0;
            for (int b = 0; b < WORD_BITS; b++) {
                const int c = ic * WORD_BITS + b;
                if (c < C && w[(((size_t)kn * C + c) * KH + kh) * KW + kw] < thr[kn]) s |= (uint64_t)1 << b;
            }
            out[(size_t)kn * Kp + j] = s;
        }
    return (int64_t*)out;
}

/* PReLU as mm_tnn applies it to the integer accumulator: positive values pass, non-positive
 * are scaled (src/tnns/mm_p2_final_tnn_avx2.c:90-93, 204-208), so a zero sum is 0*alpha: +0 for
 * alpha >= 0, -0 for a negative alpha. */
static inline float prelu_i(int acc, float alpha) { return acc > 0 ? (float)acc : (float)acc * alpha; }
/* mm_tbn / mm_btn / mm_bnn write `result >= 0 ? (float) result : prelu_alpha * result`
 * (src/tnns/mm_p2_final_tbn_avx2.c:73, _btn_:73, _bnn_:60): a zero sum stays +0 whatever the sign
 * of alpha, whereas mm_tnn multiplies it (prelu_i above; src/tnns/mm_p2_final_tnn_avx2.c:90-93). */
static inline float prelu_i_ge(int acc, float alpha) { return acc >= 0 ? (float)acc : alpha * (float)acc; }

static inline size_t nchw_at(size_t r, int kn, int KN, size_t OHW) {
    return ((r / OHW) * KN + kn) * OHW + r % OHW; /* include/tnns/mm.h:30 */
}

/*
 * TNN GEMM: both operands packing-2.  acc = 64*Kp - sum popc(az|bz)
 *           - 2 * sum popc((as^bs) & ~(az|bz))
 * (src/tnns/mm_p2_final_tnn_avx2.c:72-77,87; K is padded to four first, :385).
 * K counts 64-bit words per plane before that padding.
 */
float* orc_mm_tnn(const int64_t* a, const int64_t* b, int N, int OH, int OW, int KN, int K, float alpha) {
    const int Kp = pad4(K);
    const size_t OHW = (size_t)OH * OW, M = (size_t)N * OHW, pitch = 2 * (size_t)Kp;
    float* y = (float*)calloc(M * KN + 1, sizeof(float));
    if (!y) return NULL;
    const uint64_t* A = (const uint64_t*)a; const uint64_t* B = (const uint64_t*)b;
    for (long long r = 0; r < (long long)M; r++)
        for (int kn = 0; kn < KN; kn++) {
            const uint64_t* ar = A + (size_t)r * pitch; const uint64_t* br = B + (size_t)kn * pitch;
            int cz = 0, cn = 0;
            for (int j = 0; j < Kp; j++) {
                const size_t p = p2_sign_at(j);
                const uint64_t z = ar[p + 4] | br[p + 4];
                cz += __builtin_popcountll(z);
                cn += __builtin_popcountll((ar[p] ^ br[p]) & ~z);
            }
            y[nchw_at((size_t)r, kn, KN, OHW)] = prelu_i(64 * Kp - cz - 2 * cn, alpha);
        }
    return y;
}

/* TBN GEMM: a packing-2, b one plane of Kp words per kernel
 * (src/tnns/mm_p2_final_tbn_avx2.c:34-80; b index :61). */
float* orc_mm_tbn(const int64_t* a, const int64_t* b, int N, int OH, int OW, int KN, int K, float alpha) {
    const int Kp = pad4(K);
    const size_t OHW = (size_t)OH * OW, M = (size_t)N * OHW, pitch = 2 * (size_t)Kp;
    float* y = (float*)calloc(M * KN + 1, sizeof(float));
    if (!y) return NULL;
    const uint64_t* A = (const uint64_t*)a; const uint64_t* B = (const uint64_t*)b;
    for (long long r = 0; r < (long long)M; r++) {
        const uint64_t* ar = A + (size_t)r * pitch;
        int cz = 0;
        for (int j = 0; j < Kp; j++) cz += __builtin_popcountll(ar[p2_sign_at(j) + 4]);
        for (int kn = 0; kn < KN; kn++) {
            const uint64_t* br = B + (size_t)kn * Kp;
            int cn = 0;
            for (int j = 0; j < Kp; j++) {
                const size_t p = p2_sign_at(j);
                cn += __builtin_popcountll((ar[p] ^ br[j]) & ~ar[p + 4]);
            }
            y[nchw_at((size_t)r, kn, KN, OHW)] = prelu_i_ge(64 * Kp - cz - 2 * cn, alpha);
        }
    }
    return y;
}

/* BTN GEMM: a one plane, b packing-2 (src/tnns/mm_p2_final_btn_avx2.c:34-80). */
float* orc_mm_btn(const int64_t* a, const int64_t* b, int N, int OH, int OW, int KN, int K, float alpha) {
    const int Kp = pad4(K);
    const size_t OHW = (size_t)OH * OW, M = (size_t)N * OHW, pitch = 2 * (size_t)Kp;
    float* y = (float*)calloc(M * KN + 1, sizeof(float));
    if (!y) return NULL;
    const uint64_t* A = (const uint64_t*)a; const uint64_t* B = (const uint64_t*)b;
    for (long long r = 0; r < (long long)M; r++) {
        const uint64_t* ar = A + (size_t)r * Kp;
        for (int kn = 0; kn < KN; kn++) {
            const uint64_t* br = B + (size_t)kn * pitch;
            int cz = 0, cn = 0;
            for (int j = 0; j < Kp; j++) {
                const size_t p = p2_sign_at(j);
                cz += __builtin_popcountll(br[p + 4]);
                cn += __builtin_popcountll((ar[j] ^ br[p]) & ~br[p + 4]);
            }
            y[nchw_at((size_t)r, kn, KN, OHW)] = prelu_i_ge(64 * Kp - cz - 2 * cn, alpha);
        }
    }
    return y;
}

/* BNN GEMM: both one plane; acc = K_unpack - 2*popc(a^b)
 * (src/tnns/mm_p2_final_bnn_avx2.c:34-67). */
float* orc_mm_bnn(const int64_t* a, const int64_t* b, int N, int OH, int OW, int KN, int K, int K_unpack,
                  float alpha) {
    const int Kp = pad4(K);
    const size_t OHW = (size_t)OH * OW, M = (size_t)N * OHW;
    float* y = (float*)calloc(M * KN + 1, sizeof(float));
    if (!y) return NULL;
    const uint64_t* A = (const uint64_t*)a; const uint64_t* B = (const uint64_t*)b;
    for (long long r = 0; r < (long long)M; r++)
        for (int kn = 0; kn < KN; kn++) {
            int cn = 0;
            for (int j = 0; j < Kp; j++)
                cn += __builtin_popcountll(A[(size_t)r * Kp + j] ^ B[(size_t)kn * Kp + j]);
            y[nchw_at((size_t)r, kn, KN, OHW)] = prelu_i_ge(K_unpack - 2 * cn, alpha);
        }
    return y;
}

/*
 * Whole layer, as tnns_conv dispatches it (src/tnns/tnns_cpu_mm_p2.c:6-120):
 * type 0 TNN, 1 TBN, 2 BTN, 3 BNN (include/tnns/common.h:16).  x NCHW fp32, thr per
 * image, w already packed in the layout the type expects.  Returns NCHW fp32.
 */
float* orc_conv(int type, const float* x, const float* thr, const int64_t* w, int N, int C, int H, int W,
                int KN, int KH, int KW, int PH, int PW, int SH, int SW, float alpha) {
    const int OH = orc_out_dim(H, PH, KH, SH), OW = orc_out_dim(W, PW, KW, SW);
    const int K = orc_kw(C, KH, KW);
    int64_t* a = (type == 0 || type == 1) ? orc_t2r(x, thr, N, C, H, W, PH, PW, KH, KW, SH, SW)
                                          : orc_b2r(x, thr, N, C, H, W, PH, PW, KH, KW, SH, SW);
    if (!a) return NULL;
    float* y = NULL;
    switch (type) {
        case 0: y = orc_mm_tnn(a, w, N, OH, OW, KN, K, alpha); break;
        case 1: y = orc_mm_tbn(a, w, N, OH, OW, KN, K, alpha); break;
        case 2: y = orc_mm_btn(a, w, N, OH, OW, KN, K, alpha); break;
        case 3: y = orc_mm_bnn(a, w, N, OH, OW, KN, K, C * KH * KW, alpha); break;
        default: break;
    }
    free(a);
    return y;
}

void orc_free(void* p) { free(p); }
