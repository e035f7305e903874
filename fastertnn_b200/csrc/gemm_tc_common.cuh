// Device helpers shared by the tensor-core GEMM kernels (gemm_tc.cu, gemm_slab.cu): PTX wrappers for the
// copy engine and tcgen05, shared-memory matrix descriptors, bounded waits on global counters, and the
// quantiser / publisher roles of the one-launch forms.
#pragma once
#include <cuda.h>  // CUtensorMap and the encode prototypes only; the entry points are looked up at run time

#include "internal.h"
#include "mbar.cuh"
#include "prelu_thresholds.cuh"

namespace {

constexpr int BM = 128;        // rows per accumulator (tensor-memory lanes)
constexpr int KCH = 128;       // K elements = bytes per row and stage (one swizzle atom)
constexpr int A_SUB = BM * KCH;  // bytes of one 128-row activation sub-tile per stage
constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_EXP0 = 2;
// fused quantisation (QF)
constexpr int Q_FLAG0 = 32;   // the per-image words start one 128-byte line after the item counter
constexpr int Q_PIX = 128;    // pixels per quantise item = quantiser threads per block
constexpr int Q_STG = 2;      // stages of the quantiser warps' ring
constexpr int Q_PUBN = 8;     // items the quantiser warps may be ahead of the publisher

__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// im2col tensor copy: `pixels per column` base pixels starting at (w, h, n), walking the layer's
// output lattice (stride, padding box are in the tensor map), each read at filter offset (kw, kh),
// channels from byte c on; outside the image the copy engine writes zeros.
__device__ __forceinline__ void tma_im2col_g2s(uint32_t dst_smem, const void* tmap, int c, int w, int h, int n, unsigned short kw,
                                               unsigned short kh, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(kw), "h"(kh)
        : "memory");
}
// Block-pair forms of the tensor copies: the data lands in the executing block's shared memory,
// the bytes are reported to `bar`, which may live in the other block of the pair (an address in
// the shared::cluster window).  No multicast: every block fetches its own tile.
__device__ __forceinline__ void tma_im2col_g2s_pair(uint32_t dst_smem, const void* tmap, int c, int w, int h, int n, unsigned short kw,
                                                    unsigned short kh, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(kw), "h"(kh)
        : "memory");
}
__device__ __forceinline__ void tma_tile2d_g2s_pair(uint32_t dst_smem, const void* tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
// Block-pair forms, issued by the first block of the pair for both: the commit arrives on the
// barrier at the same shared-memory offset in both blocks.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((unsigned short)3)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
// The same two with the descriptors given as (low word, high word): only a descriptor's low word -- the
// shared-memory address in 16-byte units -- changes from MMA to MMA, so the issuing thread does 32-bit adds on
// it and nothing else (its instruction stream paces the tensor pipe).
__device__ __forceinline__ void tc_mma_f4_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], da, db, %5, [%6], [%7], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_mma_f4_pair_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                  uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], da, db, %5, [%6], [%7], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 B apart, 8-row
// groups 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
// The same for a sub-tile whose rows are 64 or 32 bytes long (64- / 32-byte swizzle; eight-row
// groups 512 / 256 bytes apart): taps = 2 or 4 filter taps share a 128-byte stage row, each tap in
// a sub-tile of its own.  taps = 1 is the 128-byte form of make_desc.
__device__ __forceinline__ uint64_t make_desc_taps(uint32_t smem_addr, int taps) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((1024 / taps) >> 4) << 32;                       // stride byte offset
    d |= (uint64_t)1 << 46;                                          // version
    d |= (uint64_t)(taps == 1 ? 2 : (taps == 2 ? 4 : 6)) << 61;      // SWIZZLE_128B / _64B / _32B
    return d;
}
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;              // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset
    d |= (uint64_t)1 << 46;              // version
    d |= (uint64_t)2 << 61;              // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait for a counter in global memory that other blocks advance.
__device__ __forceinline__ bool counter_wait(const unsigned int* ctr, unsigned int target, volatile int* abort_flag, unsigned int* status,
                                             unsigned code) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++) {
            if (ld_acquire_gpu(ctr) >= target) return true;
            __nanosleep(40);
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) {
            *abort_flag = 1;
            atomicOr(status, STATUS_WAIT_EXPIRED | code);
            return false;
        }
    }
}
__device__ __forceinline__ uint32_t push_sign(uint32_t acc, float d) { return __funnelshift_l(__float_as_uint(d), acc, 1); }

// 32 layer outputs of one pixel -> one 32-bit lane of the next layer's sign plane and non-zero plane
// (element j at bit j; same rules as the quantise kernels: sign = f < -t, non-zero = |f| > t; binary:
// sign = f < t).  One shift chain per plane: splitting each into four chains joined at the end was
// measured slower on 64-kernel tiles (55 against 49 us per layer), where the epilogue's instruction
// count, not its dependency stalls, is what the tile rate hangs on.
__device__ __forceinline__ void quantise32_ternary(const float (&f)[32], float tq, uint32_t& sg, uint32_t& nz) {
    sg = 0;
    nz = 0;
#pragma unroll
    for (int j = 31; j >= 0; j--) {
        sg = push_sign(sg, f[j] + tq);
        nz = push_sign(nz, tq - fabsf(f[j]));
    }
}
__device__ __forceinline__ uint32_t quantise32_binary(const float (&f)[32], float tq) {
    uint32_t sg = 0;
#pragma unroll
    for (int j = 31; j >= 0; j--) sg = push_sign(sg, (f[j] + 0.0f) - tq);  // + 0.0f: -0 reads as +0
    return sg;
}

// PReLU of 32 fp32 accumulators (4-bit form), as the reference evaluates it on an integer sum
// (src/tnns/mm_p2_final_tnn_avx2.c:90-93; zero_passes: the tbn / btn / bnn forms pass a zero sum through).
// The run-time choices sit outside the unrolled loops: inside, every element pays for both sides of each.
__device__ __forceinline__ void prelu32_f4(const uint32_t (&v)[32], float (&f)[32], bool alpha_in_unit, int acc_bias, float bias_f, float alpha,
                                           int zero_passes) {
    if (alpha_in_unit && acc_bias) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float a = __uint_as_float(v[j]) + bias_f;
            f[j] = fmaxf(a, fmaf(a, alpha, 0.0f));
        }
    } else if (alpha_in_unit) {
        // 0 < alpha <= 1: PReLU(a) = max(a, alpha*a), two instructions per output.  The product is formed as
        // fma(a, alpha, +0): one rounding like the reference's acc*alpha, and a -0 sum (all products -0) gives
        // +0, which max(-0, +0) returns.
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float a = __uint_as_float(v[j]);
            f[j] = fmaxf(a, fmaf(a, alpha, 0.0f));
        }
    } else {
        // any alpha: the reference's expression on the canonical +0, a > 0 ? a : a*alpha
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float ac = (acc_bias ? __uint_as_float(v[j]) + bias_f : __uint_as_float(v[j])) + 0.0f;
            f[j] = ac * ((zero_passes ? ac >= 0.f : ac > 0.f) ? 1.0f : alpha);
        }
    }
}

// Tensor-memory load of 16 lanes x 32 columns in the 16x256b shape: thread t of the warp receives, for each
// group k of eight columns, w[4k], w[4k+1] = row t/4, columns 8k + 2(t%4) and + 1, and w[4k+2], w[4k+3] = the
// same columns of row t/4 + 8.  Four neighbouring lanes thus hold 32 contiguous bytes of one row: the shape
// for writing a pixel-major (NHWC) fp32 tile with full sectors per store.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t* w) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]), "=r"(w[8]), "=r"(w[9]),
          "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15])
        : "r"(taddr)
        : "memory");
}

// Stores what two such loads (lanes 0..15 and 16..31 of the warp's quadrant) delivered: f[16*hh + 4k + 2*b + {0,1}] is
// row 16*hh + 8*b + lane/4 of the quadrant, columns 8k + 2(lane%4) and + 1 of the slice.  y_quad = the quadrant's first
// row at the slice's first column; rows_left / cols_left = rows and columns that exist from there on; KN is even.
__device__ __forceinline__ void store_rows16(const float (&f)[32], float* y_quad, int KN, long long rows_left, int cols_left, int lane) {
    const int cc = 2 * (lane & 3);
#pragma unroll
    for (int h = 0; h < 4; h++) {
        const int r = 8 * h + (lane >> 2);
        if (r < rows_left) {
            float* yr = y_quad + (size_t)r * KN + cc;
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (8 * k + cc < cols_left)
                    __stcs(reinterpret_cast<float2*>(yr + 8 * k), make_float2(f[16 * (h >> 1) + 4 * k + 2 * (h & 1)], f[16 * (h >> 1) + 4 * k + 2 * (h & 1) + 1]));
        }
    }
}

// The same for rows that are not neighbours in memory (the slab-fed GEMM's rows are positions of the padded lattice):
// yrow[h] = where row 8*h + lane/4 of the quadrant starts at the slice's first column, or nullptr if that row is not stored.
__device__ __forceinline__ void store_rows16_at(const float (&f)[32], float* const (&yrow)[4], int cols_left, int lane) {
    const int cc = 2 * (lane & 3);
#pragma unroll
    for (int h = 0; h < 4; h++) {
        if (yrow[h]) {
            float* yr = yrow[h] + cc;
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (8 * k + cc < cols_left)
                    __stcs(reinterpret_cast<float2*>(yr + 8 * k), make_float2(f[16 * (h >> 1) + 4 * k + 2 * (h & 1)], f[16 * (h >> 1) + 4 * k + 2 * (h & 1) + 1]));
        }
    }
}

// Quantiser role of the fused form, called by the four quantiser warps together (thread = pixel).
// An item = 128 neighbouring pixels x 64 channels of one image (NCHW, a row of the 2-D tensor
// (image, channel) x pixels per channel).  The first lane claims items in image order from a
// global counter -- so the images the first tiles need are finished first, whichever blocks
// run -- and requests each as ONE tensor copy into a two-stage ring; every thread then reads its
// pixel's 64 channels from shared memory (conflict-free), pushes the sign bits of (v + t) and
// (t - |v|) into the plane words (src/tnns/ternarize2row_avx2.c:438-452 read off sign bits),
// hands the stage back and stores the pixel's 64 channels as 32 bytes of e2m1 operands.  A warp
// that has stored its part of item k sets its progress word to k + 1; the publisher (below) turns
// that into counts on the images' words in global memory.
struct QuantArgs {
    const float* qthr;
    uint4* qimg;
    unsigned int* q_sync;
    int qN, qC, q_nbands, Cp, HW;
    unsigned int* status;
    // Where pixel (y, x) of image n lands in the 4-bit image: pixel index n*HpWp + y*Wp + x + off0.
    // Plain image: Wp = W, HpWp = H*W, off0 = 0.  Bordered image (the layer's padding stored around
    // every image): Wp = W + 2*PW, HpWp = (H + 2*PH)*Wp, off0 = PH*Wp + PW; border != 0 then adds one
    // item per image, after its pixel items, that writes the border pixels (the padding value).
    int W, Wp, HpWp, off0, border;
    int binary;  // activations in {-1,+1} (x < t), absent channels and the border +1; else ternary, both 0
    int nhwc;    // the fp32 input is pixel-major: an item arrives as two 128-byte-swizzled boxes of 128 pixels x 32 channels
};
__device__ __forceinline__ QuantArgs plain_quant_args(const float* qthr, uint4* qimg, unsigned int* q_sync, int qN, int qC, int q_nbands, int Cp,
                                                      int H, int W, unsigned int* status, int nhwc = 0) {
    QuantArgs a;
    a.qthr = qthr; a.qimg = qimg; a.q_sync = q_sync; a.qN = qN; a.qC = qC; a.q_nbands = q_nbands; a.Cp = Cp; a.HW = H * W; a.status = status;
    a.W = W; a.Wp = W; a.HpWp = H * W; a.off0 = 0; a.border = 0; a.binary = 0; a.nhwc = nhwc;
    return a;
}
// Control words of the quantiser warps and the publisher, behind the quantiser ring's barriers.
struct QuantCtl {
    unsigned int item[Q_STG];   // item held by each stage (>= items: end mark)
    unsigned int done[4];        // per quantiser warp: items whose stores it has issued
    unsigned int published;      // items the publisher has counted
    unsigned int total;          // items this block processed, ~0u while the quantiser warps run
    int pub_n[Q_PUBN];           // image of item k at k % Q_PUBN
};
static_assert(sizeof(QuantCtl) + 2 * Q_STG * sizeof(uint64_t) <= 128, "control words behind the quantiser ring");
__device__ __noinline__ void quantise_items(const QuantArgs p, const CUtensorMap* tmap_q, unsigned char* stage0, uint64_t* qbars,
                                            volatile int* abort_flag, const int qtid) {
    constexpr int QSTG = Q_STG, Q_STAGE = Q_PIX * 64 * 4;
    const int lane = qtid & 31, qwarp = qtid >> 5;
    const uint32_t bar_full = smem_u32(qbars), bar_empty = smem_u32(qbars + QSTG);
    volatile QuantCtl* ctl = reinterpret_cast<volatile QuantCtl*>(qbars + 2 * QSTG);
    const unsigned int pix_items = (unsigned int)p.q_nbands * (unsigned int)p.Cp;  // pixel items per image
    const unsigned int per_img = pix_items + (p.border ? 1u : 0u);                 // + the image's border item
    const unsigned int items = (unsigned int)p.qN * per_img;
    // issue: the claimed item goes into stage s (a border item or the end mark complete the barrier without bytes)
    auto issue = [&](int s, unsigned int i) {
        ctl->item[s] = i;
        const unsigned int n = i / per_img, r = i - n * per_img;
        if (i < items && r < pix_items) {
            const int ic = (int)(r % (unsigned int)p.Cp), band = (int)(r / (unsigned int)p.Cp);
            mbar_arrive_expect_tx(bar_full + 8 * s, Q_STAGE);  // the whole box(es), edges zero-filled
            if (p.nhwc) {
                // rows of the (pixels of all images) x (channels) tensor; a band's last rows may belong to the next image and are not stored
                const int row0 = (int)n * p.HW + band * Q_PIX;
                tma_tile2d_g2s(smem_u32(stage0 + s * Q_STAGE), tmap_q, ic * 64, row0, bar_full + 8 * s);
                tma_tile2d_g2s(smem_u32(stage0 + s * Q_STAGE + Q_STAGE / 2), tmap_q, ic * 64 + 32, row0, bar_full + 8 * s);
            } else {
                tma_tile2d_g2s(smem_u32(stage0 + s * Q_STAGE), tmap_q, band * Q_PIX, (int)n * p.qC + ic * 64, bar_full + 8 * s);
            }
        } else {
            mbar_arrive(bar_full + 8 * s);
        }
    };
    unsigned int next = 0;  // issuer only: the item claimed ahead
    if (qtid == 0) {
#pragma unroll
        for (int s = 0; s < QSTG; s++) issue(s, atomicAdd(p.q_sync, 1u));
        next = atomicAdd(p.q_sync, 1u);
    }
    // the image's threshold is fetched one item ahead (a peek at the item the other stage holds,
    // checked when its turn comes), so its load latency is not paid in front of the first compare
    int pf_n = -1;
    float pf_t = 0.f;
    unsigned int k = 0;
    for (;; k++) {
        const int s = (int)(k % QSTG);
        const uint32_t ph = (k / QSTG) & 1;
        if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 7)) break;
        const unsigned int i = ctl->item[s];
        if (i >= items) break;  // every later claim is past the end as well
        const int n = (int)(i / per_img);
        const unsigned int r = i - (unsigned int)n * per_img;
        const bool border_item = r >= pix_items;
        const int ic = (int)(r % (unsigned int)p.Cp), band = (int)(r / (unsigned int)p.Cp);
        const int nch = border_item ? 0 : min(64, p.qC - ic * 64);
        const float t = ((n == pf_n) ? pf_t : __ldg(p.qthr + n)) + 0.0f;  // + 0.0f: a threshold of -0 behaves as +0
        {
            // the loaded value is not touched before the next iteration: an instruction that used it
            // here would hold this warp until the load returned
            const unsigned int i2 = ctl->item[(s + 1) % QSTG];  // may be stale: only ever used after the check above
            if (i2 < items) {
                pf_n = (int)(i2 / per_img);
                pf_t = __ldg(p.qthr + pf_n);
            }
        }
        const float* sp = reinterpret_cast<const float*>(stage0 + s * Q_STAGE) + qtid;
        uint32_t sg[2] = {0, 0}, nz[2] = {0, 0};
        // channel b of a half ends at bit b: visit 31 .. 0 and shift left (four independent chains)
        if (p.nhwc) {
            const unsigned char* row = stage0 + s * Q_STAGE + qtid * 128;
            if (p.binary) {
                tnns_quantise_row32_swz128<false>(row, nch, t, sg[0], nz[0]);
                tnns_quantise_row32_swz128<false>(row + Q_STAGE / 2, nch - 32, t, sg[1], nz[1]);
                nz[0] = nz[1] = 0xFFFFFFFFu;  // no zeros in the binary alphabet
            } else {
                tnns_quantise_row32_swz128<true>(row, nch, t, sg[0], nz[0]);
                tnns_quantise_row32_swz128<true>(row + Q_STAGE / 2, nch - 32, t, sg[1], nz[1]);
            }
        } else if (nch == 64 && !p.binary) {
#pragma unroll
            for (int b = 31; b >= 0; b--) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float v = sp[(32 * h + b) * Q_PIX];
                    sg[h] = push_sign(sg[h], v + t);
                    nz[h] = push_sign(nz[h], t - fabsf(v));
                }
            }
        } else if (p.binary) {
            // x < t reads -1 (src/tnns/binarize2row_avx2.c:19-21); absent channels are +1: sign 0
#pragma unroll
            for (int h = 0; h < 2; h++) {
#pragma unroll 4
                for (int b = 31; b >= 0; b--) {
                    if (32 * h + b < nch) sg[h] = push_sign(sg[h], (sp[(32 * h + b) * Q_PIX] + 0.0f) - t);
                    else sg[h] <<= 1;
                }
                nz[h] = 0xFFFFFFFFu;  // no zeros in the binary alphabet
            }
        } else {
#pragma unroll
            for (int h = 0; h < 2; h++) {
#pragma unroll 1
                for (int b = 31; b >= 0; b--) {
                    if (32 * h + b < nch) {
                        const float v = sp[(32 * h + b) * Q_PIX];
                        sg[h] = push_sign(sg[h], v + t);
                        nz[h] = push_sign(nz[h], t - fabsf(v));
                    } else {  // absent channel: sign 0, non-zero 0
                        sg[h] <<= 1;
                        nz[h] <<= 1;
                    }
                }
            }
        }
        // every value is in registers: hand the stage back; the issuer refills it at once
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        if (qtid == 0) {
            if (!mbar_wait(bar_empty + 8 * s, ph, abort_flag, p.status, 8)) break;
            issue(s, next);
            next = atomicAdd(p.q_sync, 1u);
            // the publisher's ring of image indices: never more than Q_PUBN items ahead of it
            if (k >= Q_PUBN && ctl->published + Q_PUBN <= k) {
                const long long t0 = clock64();
                while (ctl->published + Q_PUBN <= k && !*abort_flag) {
                    if (clock64() - t0 > 2000000000LL) {
                        *abort_flag = 1;
                        atomicOr(p.status, STATUS_WAIT_EXPIRED | 9);
                    }
                }
            }
            ctl->pub_n[k % Q_PUBN] = n;
        }
        const int pix = band * Q_PIX + qtid;
        if (border_item) {
            // the image's border pixels: the padding value in every channel group (ternary 0, binary +1)
            const uint32_t padw = p.binary ? 0x22222222u : 0u;
            const uint4 pad4 = make_uint4(padw, padw, padw, padw);
            const int PH = p.off0 / p.Wp, PW = p.off0 - PH * p.Wp, H = p.HW / p.W;
            for (int tpx = qtid; tpx < p.HpWp; tpx += Q_PIX) {
                const int y = tpx / p.Wp, x = tpx - y * p.Wp;
                if (y < PH || y >= PH + H || x < PW || x >= PW + p.W) {
                    uint4* dst = p.qimg + ((size_t)n * p.HpWp + tpx) * p.Cp * 2;
                    for (int u = 0; u < 2 * p.Cp; u++) dst[u] = pad4;
                }
            }
        } else if (pix < p.HW) {
            uint32_t lo[4], hi[4];
            tnns_expand32_f4(sg[0], ~nz[0], lo);
            tnns_expand32_f4(sg[1], ~nz[1], hi);
            const int y = pix / p.W, x = pix - y * p.W;
            uint4* dst = p.qimg + (((size_t)n * p.HpWp + (size_t)y * p.Wp + x + p.off0) * p.Cp + ic) * 2;
            dst[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            dst[1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        }
        // progress word of this warp: release at block scope, so that the publisher, having read it,
        // may publish the warp's stores (and, for the first warp, the image index) further
        __syncwarp();
        if (lane == 0) {
            __threadfence_block();
            ctl->done[qwarp] = k + 1;
        }
    }
    __syncwarp();
    if (qtid == 0) ctl->total = k;
}

// Publisher of the fused form (one thread).  Counting a finished item on its image's word needs a
// gpu-scope release fence in front -- the item's plain stores must be visible to whoever sees the
// count -- and under the GEMM's store traffic that fence takes longer than quantising the item.
// So the quantiser warps never fence at gpu scope: this thread watches their progress words,
// and whenever all four have moved on it issues ONE fence and counts every newly finished item
// (four warps per item) with relaxed adds.  The producer threads of all blocks poll those counts.
__device__ __noinline__ void publish_items(unsigned int* q_sync, unsigned int* status, uint64_t* qbars, volatile int* abort_flag) {
    volatile QuantCtl* ctl = reinterpret_cast<volatile QuantCtl*>(qbars + 2 * Q_STG);
    unsigned int published = 0;
    long long t0 = clock64();
    for (;;) {
        const unsigned int m = min(min(ctl->done[0], ctl->done[1]), min(ctl->done[2], ctl->done[3]));
        if (m > published) {
            __threadfence();  // acquire of the progress words at block scope, release of the warps' stores at gpu scope
            for (unsigned int j = published; j < m; j++)
                asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(q_sync + Q_FLAG0 + ctl->pub_n[j % Q_PUBN]), "r"(4u) : "memory");
            published = m;
            ctl->published = m;
            t0 = clock64();
        } else {
            if (ctl->total == published || *abort_flag) break;
            if (clock64() - t0 > 4000000000LL) {
                *abort_flag = 1;
                atomicOr(status, STATUS_WAIT_EXPIRED | 10);
                break;
            }
            __nanosleep(64);
        }
    }
}

}  // namespace
