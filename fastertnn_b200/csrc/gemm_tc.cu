// Bitwise GEMM + PReLU on the 5th-generation tensor cores (reference: mm_tnn / mm_tbn / mm_btn /
// mm_bnn, src/tnns/mm_p2_final_*_avx2.c).  The packed {-1,0,+1} / {-1,+1} operands are expanded
// on the fly and multiplied by tcgen05.mma with the accumulators in tensor memory, in one of
// two forms:
//   int8  (F4 = false)  kind::i8, int32 accumulators, 128 K elements per 128-byte row and stage
//   4-bit (F4 = true)   kind::mxf4 on e2m1 nibbles with every block scale = 1, fp32
//                       accumulators, 256 K elements per row and stage (default: half the
//                       shared-memory bytes per multiply-accumulate, twice the tensor rate)
// Both are exact: |acc| <= 64*Kp < 2^22, so the int32 and the fp32 sums are the same integers
// and the fp32 output is bit-identical to the popcount kernels.
//
// The activation operand reaches shared memory in one of two ways:
//   expander-fed (ATMA = false)  warps gather the packed planes (an explicit im2row matrix or, for the
//                       implicit form, the bit-plane image of the layer input) and expand them
//   tensor-copy fed (ATMA = true)  the layer input was quantised straight into 4-bit operands and
//                       the copy engine delivers each stage as im2col tensor copies; no expander
//                       warps, optionally on block pairs (CG = 2, tcgen05.mma.cta_group::2), and
//                       optionally with the quantise step itself in the same launch (QF = true:
//                       four quantiser warps and a publisher thread beside the GEMM's roles; a
//                       tile's copies start once the images of its rows are complete)
//
// Expander-fed form: one persistent block per SM, 22 warps in four roles (the tensor-copy form
// keeps warps 0, 1 and eight epilogue warps):
//   warp 0      weight producer: one bulk async copy (TMA engine, no multicast, no tensor map)
//               per stage of a pre-expanded, pre-swizzled weight tile (built once per layer)
//   warp 1      MMA issuer: one thread issues four tcgen05.mma per stage and commits to the
//               stage's "empty" barrier; owns the tensor-memory allocation
//   12-16 warps activation expanders in NG groups: thread = row; group k fills stages k, k+NG, ...
//               so NG stages are expanded at once; packed planes come from global memory through
//               a register prefetch ring and are stored in the 128-byte-swizzled K-major layout
//               the MMA descriptor expects
//   4-8 warps   epilogue: tcgen05.ld the finished accumulator, apply the BNN constant and PReLU,
//               store fp32 (NCHW: 32 consecutive pixels per warp and kernel -> 128-byte stores)
// Every mbarrier wait is bounded; on expiry the kernel raises a status word, all roles leave
// their loops, tensor memory is freed and the kernel returns.
//
// The order of the K elements inside a stage is whatever the expansion routine produces;
// activations and weights go through the same routine, so the permutation cancels in the dot
// product.
#include <cuda.h>  // CUtensorMap and the encode prototypes only; the entry point is looked up at run time

#include <algorithm>
#include <type_traits>
#include <vector>

#include "gemm_tc_common.cuh"



namespace {

// A block owns MT stacked 128-row sub-tiles (MT*128 rows) and BN kernels: every weight stage
// that arrives from L2 feeds MT MMAs, which is what keeps the L2 -> SM weight traffic below
// the tensor pipe's appetite.  Roles: warp 0 weight producer, warp 1 MMA issuer, NG groups of
// 4*MT expander warps, 4*MT epilogue warps.
// F4 selects the 4-bit form: operands as e2m1 nibbles (+1 = 0x2, -1 = 0xA, 0 = 0x0), multiplied by
// tcgen05.mma.kind::mxf4 with every block scale equal to 1 (ue8m0 0x7F) and fp32 accumulators --
// sums of at most 2^22 products of +-1 are exact in fp32.  A stage then covers 256 K elements in
// the same 128 bytes per row, which halves the shared-memory traffic per multiply-accumulate and
// doubles the tensor rate.  The block scales occupy the top 32 tensor-memory columns (480..511),
// which leaves 480 columns for two accumulator sets.  With BN = 256 the two sets overlap in 32
// columns (set 0 = columns 0..255, set 1 = columns 224..479): the epilogue drains the shared
// columns first and hands them back, so the next tile's MMAs run while the rest is drained.
// ATMA: the activation stage is not expanded by warps but delivered by the copy engine as one
// im2col tensor copy from a 4-bit (e2m1) image of the layer input -- 128 output pixels x 128 bytes
// (256 channels of one filter tap), zero-filled outside the image, written in the swizzled layout
// the MMA reads.  No expander warps then: producer warp, MMA warp, eight epilogue warps.
// CG = 2 (tensor-copy form only) pairs two blocks -- a cluster of two, on the two SMs of one TPC --
// on one 256-row tile: tcgen05.mma.cta_group::2, issued by the first block for both, multiplies
// each block's own 128 activation rows with the whole weight tile, of which each block holds
// half.  A block then receives 32 KB instead of 48 KB per stage from L2 and the ring is six deep.
// Both blocks' tensor copies report to the first block's "full" barrier; its commits release the
// stage and publish the accumulator in both blocks (multicast arrive).
// QF (tensor-copy form only) fuses the quantise step into the same launch: four more warps turn the
// layer's fp32 input into the 4-bit image, item by item (128 pixels x 64 channels, claimed from a
// global counter, fetched as one 32 KB tensor copy into a two-stage ring of their own -- the GEMM
// ring is one or two stages shallower to make room), and count every finished item on its image's
// word in global memory; the producer thread starts a tile's tensor copies once the images its
// rows belong to are complete.  The quantisation (HBM-bound) then runs underneath the MMAs
// (tensor-bound) of earlier tiles.
template <int BN, int MT, bool F4, bool ATMA = false, int CG = 1, int TAPS = 1, bool QF = false>
struct TcCfg {
    static_assert(!QF || ATMA, "fused quantisation: tensor-copy form only");
    static constexpr int NQ = QF ? 5 : 0;  // four quantiser warps (thread = pixel of a 128-pixel item) and the publisher's warp
    static_assert(TAPS == 1 || (ATMA && (TAPS == 2 || TAPS == 4)), "taps per stage row: tensor-copy form only");
    static_assert(!ATMA || (F4 && MT == 1), "tensor-copy activations: 4-bit form, one accumulator per block");
    static_assert(CG == 1 || (CG == 2 && ATMA), "block pairs: tensor-copy form only");
    static constexpr int QSTG = Q_STG, Q_STAGE = 128 * 64 * 4;  // quantiser ring: stages, bytes per stage
    // smem ring depth
    static constexpr int NSTG_QF = (CG == 2) ? 5 : (BN == 256 ? 3 : 4);
    static constexpr int NSTG = QF ? NSTG_QF : ((CG == 2) ? 6 : ((MT == 1) ? 4 : 3));
    static constexpr int A_STAGE = MT * A_SUB, B_STAGE = (BN / CG) * KCH;
    static constexpr bool OVL = F4 && MT == 1 && BN == 256;        // overlapping accumulator sets
    static constexpr int NBUF = (OVL || MT * BN <= (F4 ? 128 : 256)) ? 2 : 1;  // accumulator sets in tensor memory
    static constexpr int ACC_OFF = OVL ? BN - 32 : MT * BN;        // column distance between the sets
    // epilogue warps per lane quadrant: two share each quadrant's columns where the drain is
    // not (or only partly) hidden behind the next tile's MMAs
    static constexpr int EPW = ATMA ? 2 : (((NBUF == 1 || OVL) && MT == 1) ? 2 : 1);
    // expander groups (stages expanded concurrently); 22 warps per block in every MT = 1 form
    static constexpr int NG = ATMA ? 0 : ((MT == 1) ? (EPW == 2 ? 3 : 4) : 2);
    static constexpr int WARP_EPI0 = WARP_EXP0 + 4 * MT * NG;
    static constexpr int WARP_Q0 = WARP_EPI0 + 4 * MT * EPW;
    static constexpr int NTHREADS = 32 * (2 + 4 * MT * NG + 4 * MT * EPW + NQ);
    static constexpr int TAPMAX = QF ? 192 : 1024;  // entries of the tap table kept in shared memory (QF: 192 entries + the 256 bytes of barriers = 1 KB, see Q_OFF)
    static constexpr size_t Q_OFF = (size_t)NSTG * (A_STAGE + B_STAGE) + 256 + TAPMAX * sizeof(uint32_t);  // quantiser ring, then its barriers
    static_assert(!QF || Q_OFF % 1024 == 0, "the quantiser ring receives 128-byte-swizzled boxes: its stages start on 1024-byte boundaries");
    static constexpr size_t SMEM = 1024 + Q_OFF + (QF ? QSTG * Q_STAGE + 128 : 0);
    static_assert(SMEM <= 232448, "shared memory per block");
};


// 32 elements (one 32-bit lane per plane) -> 32 int8 in a fixed permuted order, as eight words.
// code = zero<<1 | sign : 0 -> +1, 1 -> -1, 2 or 3 -> 0 (a set zero bit wins, as az|bz does).
__device__ __forceinline__ void expand32(uint32_t s, uint32_t z, uint32_t (&w)[8]) {
    constexpr uint32_t TAB = 0x0000FF01u;
    const uint32_t x = (s & 0x55555555u) | ((z << 1) & 0xAAAAAAAAu);   // codes of even elements
    const uint32_t y = ((s >> 1) & 0x55555555u) | (z & 0xAAAAAAAAu);   // codes of odd elements
    const uint32_t e0 = x & 0x33333333u, e1 = (x >> 2) & 0x33333333u;
    const uint32_t e2 = y & 0x33333333u, e3 = (y >> 2) & 0x33333333u;
    w[0] = __byte_perm(TAB, 0, e0); w[1] = __byte_perm(TAB, 0, e0 >> 16);
    w[2] = __byte_perm(TAB, 0, e1); w[3] = __byte_perm(TAB, 0, e1 >> 16);
    w[4] = __byte_perm(TAB, 0, e2); w[5] = __byte_perm(TAB, 0, e2 >> 16);
    w[6] = __byte_perm(TAB, 0, e3); w[7] = __byte_perm(TAB, 0, e3 >> 16);
}

// Writes the 128 int8 of one row and chunk (four lanes) into a swizzled tile image.
// `tile` points at row 0 of a 1024-byte aligned tile; generic pointer (smem or global).
__device__ __forceinline__ void store_row_chunk(unsigned char* tile, int r, const uint4& s, const uint4& z) {
    const uint32_t sl[4] = {s.x, s.y, s.z, s.w}, zl[4] = {z.x, z.y, z.z, z.w};
    unsigned char* row = tile + (size_t)r * KCH;
#pragma unroll
    for (int l = 0; l < 4; l++) {
        uint32_t w[8];
        expand32(sl[l], zl[l], w);
        *reinterpret_cast<uint4*>(row + (((2 * l) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(row + (((2 * l + 1) ^ (r & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
    }
}


// 4-bit form: one row and stage = 256 elements = eight lanes per plane -> 128 bytes.
__device__ __forceinline__ void store_row_stage_f4(unsigned char* tile, int r, const uint4 (&s)[2], const uint4 (&z)[2]) {
    const uint32_t sl[8] = {s[0].x, s[0].y, s[0].z, s[0].w, s[1].x, s[1].y, s[1].z, s[1].w};
    const uint32_t zl[8] = {z[0].x, z[0].y, z[0].z, z[0].w, z[1].x, z[1].y, z[1].z, z[1].w};
    unsigned char* row = tile + (size_t)r * KCH;
#pragma unroll
    for (int l = 0; l < 8; l++) {
        uint32_t w[4];
        tnns_expand32_f4(sl[l], zl[l], w);
        *reinterpret_cast<uint4*>(row + ((l ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// ---------------------------------------------------------------------------------------
// One-time weight expansion: packed rows -> int8 tile images, [n_tile][chunk][BN rows][128 B],
// swizzled exactly as the MMA reads them, rows past KN left zero.
// ---------------------------------------------------------------------------------------
// zero_from >= 0 (4-bit form): plane words from that index on -- the words added by the pad-to-four --
// are written as zeros whatever the row holds there (binary rows read +1), so that an activation
// operand may leave those K positions undefined.
__global__ void expand_weights_kernel(const uint4* __restrict__ packed, unsigned char* __restrict__ img, int KN, int Kp, int BN,
                                      int two_planes, int f4, int zero_from) {
    const int nch = f4 ? Kp / 4 : Kp / 2;
    const long long total = (long long)KN * nch;
    const size_t pitch = two_planes ? (size_t)Kp : (size_t)Kp / 2;  // uint4 per row
    const int gsz = two_planes ? 4 : 2;                              // uint4 per 256-element group
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int kn = (int)(i / nch), c = (int)(i - (long long)kn * nch);
        unsigned char* tile = img + ((size_t)(kn / BN) * nch + c) * (size_t)BN * KCH;
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        if (f4) {
            const uint4* grp = packed + (size_t)kn * pitch + (size_t)c * gsz;
            uint4 s[2] = {grp[0], grp[1]};
            uint4 z[2] = {two_planes ? grp[2] : zero4, two_planes ? grp[3] : zero4};
            if (zero_from >= 0 && 4 * c + 4 > zero_from) {
                uint32_t* sw = reinterpret_cast<uint32_t*>(s);
                uint32_t* zw = reinterpret_cast<uint32_t*>(z);
                for (int q = 0; q < 4; q++)
                    if (4 * c + q >= zero_from) {
                        sw[2 * q] = sw[2 * q + 1] = 0u;
                        zw[2 * q] = zw[2 * q + 1] = 0xFFFFFFFFu;
                    }
            }
            store_row_stage_f4(tile, kn % BN, s, z);
        } else {
            const uint4* grp = packed + (size_t)kn * pitch + (size_t)(c >> 1) * gsz;
            store_row_chunk(tile, kn % BN, grp[c & 1], two_planes ? grp[2 + (c & 1)] : zero4);
        }
    }
}

struct GemmArgs {
    const uint4* A;             // packed activations
    const unsigned char* Bimg;  // expanded weights
    float* y;
    long long M;
    int KN, Kp, OHW, layout;
    int a_two_planes;
    int acc_bias;               // added to the integer dot product (BNN: K_unpack - 64*Kp)
    float alpha;
    unsigned int* status;
    // optional quantised output for a following layer (instead of y): bit planes [n][plane][pixel][ic]
    uint32_t* pimg;
    const float* thr_next;      // one threshold per image for that quantisation
    int next_ternary, cp_next;  // planes of the next layer's activations, its 64-channel groups
    int pimg_e2m1;              // write that output as a 4-bit operand image [n][pixel][ic][32 B] instead of bit planes
    // that image bordered for a slab-fed next layer: pixel (oh, ow) of image n at n*o_HpWp + (oh + o_PH)*o_Wp + ow + o_PW,
    // the frame of o_PH rows / o_PW columns around every image written (zeros) by this launch; o_HpWp = 0: plain image
    int o_Wp, o_HpWp, o_PH, o_PW;
    // PReLU of a zero sum: mm_tnn scales it (0*alpha, -0 for a negative alpha), mm_tbn / mm_btn / mm_bnn pass
    // +0 through (src/tnns/mm_p2_final_tnn_avx2.c:90-93 against mm_p2_final_tbn_avx2.c:73)
    int zero_passes;
    // optional implicit im2row (4-bit form): A is not a packed im2row matrix but the quantised
    // image [n][plane][pixel][ic] of the layer input; row r, plane word j are gathered on the fly
    const uint64_t* img;
    const uint32_t* jtab;       // per plane word j: kh<<24 | kw<<16 | ic, 0xFFFFFFFF for pad words
    int H, W, OW, Cp, SH, SW, PH, PW;
    // fused quantisation (QF): the layer's fp32 NCHW input and per-image thresholds, the 4-bit image
    // the quantiser warps write (the tensor the activation copies read), and the launch's
    // synchronisation words, zero when the launch starts: q_sync[0] = next item to claim,
    // q_sync[1] = blocks that have left, q_sync[Q_FLAG0 + n] = finished items of image n
    const float* qx;
    const float* qthr;
    uint4* qimg;
    unsigned int* q_sync;
    int qN, qC, q_nbands;
    int q_nhwc;        // that input is pixel-major (NHWC)
    int q_self_clean;  // the last block to leave zeroes the words again (q_sync[1] counts the blocks that left)
};



// Bordered output image (quantising epilogue, next_format 3): the frame around every image holds the next layer's padding
// value (ternary 0).  Written by the epilogue threads of all blocks after the wait for the launch before, which may still
// read this buffer.  Kept out of line: inlined, its registers cost the fp32 path of the large layer a percent.
__device__ __noinline__ void fill_output_border(uint4* img, int cp_next, int H, int W, int nimg, int o_Wp, int o_HpWp, int o_PH, int o_PW,
                                                long long first, long long step) {
    const long long total = (long long)nimg * o_HpWp;
    const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
    for (long long i = first; i < total; i += step) {
        const int r = (int)(i % o_HpWp), y = r / o_Wp, x = r - y * o_Wp;
        if (y < o_PH || y >= o_PH + H || x < o_PW || x >= o_PW + W) {
            uint4* dst = img + (size_t)i * cp_next * 2;
            for (int u = 0; u < 2 * cp_next; u++) dst[u] = z4;
        }
    }
}

// TAPS (tensor-copy form): filter taps per 128-byte stage row -- 1: a tap's 256 channels fill the
// row (C_pack % 4 == 0); 2: C_pack = 2, two taps of 128 channels in two 64-byte-swizzled sub-tiles;
// 4: C_pack = 1, four taps of 64 channels in four 32-byte-swizzled sub-tiles.
template <int BN, int MT, bool F4, bool ATMA, int CG, int TAPS, bool QF>
__global__ void __launch_bounds__(TcCfg<BN, MT, F4, ATMA, CG, TAPS, QF>::NTHREADS, 1)
gemm_tc_kernel(GemmArgs p, const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_q) {
    using Cfg = TcCfg<BN, MT, F4, ATMA, CG, TAPS, QF>;
    constexpr int NSTG = Cfg::NSTG, A_STAGE = Cfg::A_STAGE, B_STAGE = Cfg::B_STAGE, NBUF = Cfg::NBUF, WARP_EPI0 = Cfg::WARP_EPI0, NG = Cfg::NG, EPW = Cfg::EPW;
    constexpr int BMT = MT * BM;      // rows per block
    constexpr int TILE_M = CG * BMT;  // rows per tile (a block pair shares one 256-row tile)
    // instruction descriptor: i8 -- s32 accumulate (2<<4), signed 8-bit A and B (1<<7, 1<<10);
    // mxf4 -- e2m1 A and B (1<<7, 1<<10), ue8m0 scales (1<<23); both K-major, N>>3 at bit 17, M>>4 at bit 24
    constexpr uint32_t IDESC = (F4 ? (1u << 23) : (2u << 4)) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                               ((uint32_t)((CG * BM) >> 4) << 24);
    constexpr bool OVL = Cfg::OVL;
    constexpr int ACC_OFF = Cfg::ACC_OFF;
    constexpr uint32_t SF_COL = 480;  // first tensor-memory column of the (all-ones) block scales
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + NSTG * A_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + NSTG * B_STAGE);
    // barriers: full[NSTG], empty[NSTG], tmem_full[2], tmem_empty[2]
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + NSTG), bar_tfull = smem_u32(bars + 2 * NSTG),
                   bar_tempty = smem_u32(bars + 2 * NSTG + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NSTG + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // The tap table (plane word -> kh, kw, ic) sits on the producer's critical path once per stage,
    // so its first TAPMAX entries are copied to shared memory; longer tables fall back to global loads.
    uint32_t* s_taps = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(bars) + 256);
    auto tap_at = [&](int j) -> uint32_t { return j < Cfg::TAPMAX ? s_taps[j] : __ldg(p.jtab + j); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Programmatic dependent launch: a following launch of this kind may place its
    // blocks on SMs as the blocks of this one leave, run its set-up there, and wait (below, before
    // it touches any global data) until this launch has completed.  All blocks of a launch are
    // resident at once, so letting the dependents in early cannot starve this launch of SMs.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int nchunks = F4 ? p.Kp / 4 : p.Kp / 2;  // stages per tile
    const int ntn = (p.KN + BN - 1) / BN;
    const long long ntm = (p.M + TILE_M - 1) / TILE_M;
    const long long ntiles = ntm * ntn;
    // a unit = the block (CG = 1) or the block pair (CG = 2) that walks one tile sequence
    const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
    const long long unit = blockIdx.x / CG, nunits = gridDim.x / CG;

    if (p.jtab)
        for (int j = threadIdx.x; j < min(p.Kp, Cfg::TAPMAX); j += blockDim.x) s_taps[j] = __ldg(p.jtab + j);
    if (tid == 0) {
        for (int s = 0; s < NSTG; s++) {
            mbar_init(bar_full + 8 * s, ATMA ? 1 : 1 + 4 * MT);  // weight producer + the expander warps
            mbar_init(bar_empty + 8 * s, 1);  // tcgen05.commit
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, CG * 4 * MT * EPW);  // the epilogue warps (of both blocks of a pair)
        }
        if (QF) {
            uint64_t* qbars = reinterpret_cast<uint64_t*>(smem + Cfg::Q_OFF + Cfg::QSTG * Cfg::Q_STAGE);
            for (int s = 0; s < Cfg::QSTG; s++) {
                mbar_init(smem_u32(qbars + s), 1);               // the issuer's arrive with the expected bytes
                mbar_init(smem_u32(qbars + Cfg::QSTG + s), 4);   // the four quantiser warps
            }
            volatile QuantCtl* ctl = reinterpret_cast<volatile QuantCtl*>(qbars + 2 * Cfg::QSTG);
            ctl->done[0] = ctl->done[1] = ctl->done[2] = ctl->done[3] = 0;
            ctl->published = 0;
            ctl->total = 0xFFFFFFFFu;
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == WARP_MMA) {
        if (CG == 2) {
            // both blocks of the pair allocate, from the same warp index, the same columns
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    // pair: no remote arrive, copy completion or multicast commit may reach a barrier before its block initialised it
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (F4) {
        // block scales: ue8m0 0x7F = 2^0 in every byte of columns 480..511 (16 columns for the
        // row scales, 16 for the column scales; one MMA reads at most four of each), so whatever
        // bytes the MMA picks as scale of a row block or column block, it reads 1.0
        if (warp >= WARP_EPI0 && warp < WARP_EPI0 + 4) {
            const uint32_t one = 0x7F7F7F7Fu;
#pragma unroll 1
            for (uint32_t c = 0; c < 32; c += 8) {
                const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SF_COL + c;
                asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(one)
                             : "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        tc_fence_before();
        if (CG == 2) cluster_sync_all(); else __syncthreads();  // pair: the first block's MMAs read both blocks' scales
        tc_fence_after();
    }

    // everything above touched only on-chip state and the layer's constant tables; what follows reads
    // and writes tensors that the previous launch on the stream may still be working on
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == WARP_TMA) {
        if (lane == 0) {
            uint32_t s = 0, ph = 1;  // ring slot and the parity its "empty" barrier is waited with
            // pair: both blocks' copies report to the first block's barrier
            const uint32_t bar_full_lead = (CG == 2) ? mapa_shared(bar_full, 0) : bar_full;
            for (long long t = unit; t < ntiles; t += nunits) {
                const int n_tile = (int)(t % ntn);
                const unsigned char* src = p.Bimg + (size_t)n_tile * nchunks * B_STAGE;
                // tensor-copy activations: base pixel of the block's first output pixel
                int a_n = 0, a_h = 0, a_w = 0;
                if (ATMA) {
                    long long row0 = (t / ntn) * TILE_M + (long long)rank * BMT;
                    if (row0 >= p.M) row0 = 0;  // second block of a pair past the last row: any valid pixels, never stored
                    // 32-bit divisions where the row index allows it (64-bit ones cost this thread hundreds of cycles per tile)
                    a_n = row0 < 0x7FFFFFFFLL ? (int)((uint32_t)row0 / (uint32_t)p.OHW) : (int)(row0 / p.OHW);
                    const int rem = (int)(row0 - (long long)a_n * p.OHW);
                    const int oh = rem / p.OW;
                    a_h = oh * p.SH - p.PH;
                    a_w = (rem - oh * p.OW) * p.SW - p.PW;
                    if (QF) {
                        // the copies of this tile read the images of its rows: wait until the
                        // quantiser warps (of any block) have finished them
                        const long long last = min(row0 + BMT, p.M) - 1;
                        const int n_last = (int)(last / p.OHW);
                        const unsigned int per_image = (unsigned int)(p.q_nbands * p.Cp) * 4u;  // every quantiser warp counts itself
                        for (int n = a_n; n <= n_last; n++)
                            if (!counter_wait(p.q_sync + Q_FLAG0 + n, per_image, abort_flag, p.status, 6)) goto done;
                        // their plain stores, now visible to this thread, before the copy engine's reads
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    }
                }
                for (int c = 0; c < nchunks; c++, s = (s + 1 == NSTG) ? 0 : s + 1, ph ^= (s == 0)) {
                    if (!mbar_wait(bar_empty + 8 * s, ph, abort_flag, p.status, 1)) goto done;
                    // tensor-copy activations: the stage's four plane words are TAPS filter taps
                    // (TAPS: one tap of 256 channels, two of 128 or four of 64), one copy and one sub-tile
                    // each; words added by the pad-to-four have no tap: their sub-tile keeps what
                    // it held (any nibble is a finite e2m1 value) and meets zero weights
                    uint32_t tap[4];
                    int a_bytes = 0;
                    constexpr int wpt = 4 / TAPS, sub = A_STAGE / TAPS;  // plane words and bytes per tap
                    if (ATMA) {
#pragma unroll
                        for (int q = 0; q < TAPS; q++) {
                            tap[q] = tap_at(4 * c + q * wpt);
                            if (tap[q] != 0xFFFFFFFFu) a_bytes += sub;
                        }
                    }
                    if (CG == 2) {
                        if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * s, CG * (B_STAGE + a_bytes));
                        tma_tile2d_g2s_pair(smem_u32(sB + s * B_STAGE), &tmap_b, 0, (n_tile * nchunks + c) * BN + (int)rank * (BN / CG),
                                            bar_full_lead + 8 * s);
#pragma unroll
                        for (int q = 0; q < TAPS; q++)
                            if (tap[q] != 0xFFFFFFFFu)
                                tma_im2col_g2s_pair(smem_u32(sA + s * A_STAGE + q * sub), &tmap_a, (int)(tap[q] & 0xFFFF) * 32, a_w, a_h, a_n,
                                                    (unsigned short)((tap[q] >> 16) & 0xFF), (unsigned short)(tap[q] >> 24), bar_full_lead + 8 * s);
                        continue;
                    }
                    mbar_arrive_expect_tx(bar_full + 8 * s, B_STAGE + a_bytes);
                    bulk_g2s(smem_u32(sB + s * B_STAGE), src + (size_t)c * B_STAGE, B_STAGE, bar_full + 8 * s);
                    if (ATMA) {
#pragma unroll
                        for (int q = 0; q < TAPS; q++)
                            if (tap[q] != 0xFFFFFFFFu)
                                tma_im2col_g2s(smem_u32(sA + s * A_STAGE + q * sub), &tmap_a, (int)(tap[q] & 0xFFFF) * 32, a_w, a_h, a_n,
                                               (unsigned short)((tap[q] >> 16) & 0xFF), (unsigned short)(tap[q] >> 24), bar_full + 8 * s);
                    }
                }
            }
        }
    } else if (warp == WARP_MMA) {
        if (lane == 0 && rank == 0) {  // pair: the first block issues for both
            // This one thread's instruction stream paces the tensor pipe, so it is kept short: the
            // ring slot and its phase are running counters, the descriptors of slot s are those of
            // slot 0 plus s stage sizes (the address field counts 16-byte units and cannot carry
            // out of its 14 bits for shared-memory addresses), K steps add constants.
            uint32_t lt = 0, s = 0, ph = 0;
            constexpr int KPS = 4 / TAPS;                       // 32-byte K steps per sub-tile
            const uint64_t da0 = make_desc_taps(smem_u32(sA), TAPS), db0 = make_desc(smem_u32(sB));
            // Only a descriptor's low word (the address, in 16-byte units) changes from stage to stage and from K
            // step to K step: the loop does 32-bit adds on running low words and nothing else between two MMAs.
            // Measured on the slab-fed twin of this loop: every dependent instruction in front of an MMA costs
            // this thread, which shares its scheduler with two epilogue warps, about ten clocks of issue time.
            const uint32_t a_lo0 = (uint32_t)da0, a_hi = (uint32_t)(da0 >> 32), b_lo0 = (uint32_t)db0, b_hi = (uint32_t)(db0 >> 32);
            const uint32_t sfa = tmem_base + SF_COL, sfb = tmem_base + SF_COL + 16;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;                // descriptors of ring slot s
            for (long long t = unit; t < ntiles; t += nunits, lt++) {
                const int buf = lt % NBUF;
                // overlapping sets: one barrier, completed once per tile when the columns shared
                // with the previous tile's set have been drained; otherwise one barrier per set
                if (!mbar_wait(OVL ? bar_tempty : bar_tempty + 8 * buf, (OVL ? (lt & 1) : ((lt / NBUF) & 1)) ^ 1, abort_flag, p.status, 2)) goto done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * ACC_OFF;
                uint32_t acc = 0;
                for (int c = 0; c < nchunks; c++) {
                    if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, 3)) goto done;
                    tc_fence_after();
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
                        for (int k = 0; k < KCH / 32; k++) {
                            // K step k: sub-tile k / KPS, 32 bytes x (k % KPS) into its rows
                            constexpr int SUB16 = (A_STAGE / TAPS) >> 4;
                            const uint32_t ak = a_lo + (uint32_t)(mt * (A_SUB >> 4) + (k / KPS) * SUB16 + 2 * (k % KPS));
                            if (CG == 2) tc_mma_f4_pair_lh(d_tmem, ak, a_hi, b_lo + 2 * k, b_hi, IDESC, sfa, sfb, acc | (uint32_t)k);
                            else if (F4) tc_mma_f4_lh(d_tmem + mt * BN, ak, a_hi, b_lo + 2 * k, b_hi, IDESC, sfa, sfb, acc | (uint32_t)k);
                            else tc_mma_i8(d_tmem + mt * BN, ((uint64_t)a_hi << 32) | ak, ((uint64_t)b_hi << 32) | (b_lo + 2 * k), IDESC, (c | k) ? 1u : 0u);
                        }
                    }
                    acc = 1;
                    // stage reusable once these MMAs have read it (pair: in both blocks)
                    if (CG == 2) tc_commit_pair(bar_empty + 8 * s); else tc_commit(bar_empty + 8 * s);
                    if (++s == NSTG) { s = 0; ph ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                    else { a_lo += A_STAGE >> 4; b_lo += B_STAGE >> 4; }
                }
                // accumulator complete (pair: each block's epilogue drains its own 128 rows)
                if (CG == 2) tc_commit_pair(bar_tfull + 8 * buf); else tc_commit(bar_tfull + 8 * buf);
            }
        }
    } else if (!ATMA && warp < WARP_EPI0) {
        // ---------------- activation expanders ----------------
        // NG groups of MT*128 threads; thread = row.  Group k expands the stages it = k, k+NG,
        // k+2*NG, ... of the block's flat (tile, chunk) sequence, so NG stages are being
        // expanded at the same time and one slow dependency chain never starves the MMA.
        // The packed planes of a row come straight from global memory (L2); a register ring keeps
        // PF of this group's stages of loads in flight, running ahead across tile boundaries.
        const int e = tid - WARP_EXP0 * 32;
        const int grp = e / BMT;
        const int r = e - grp * BMT;  // row of the block tile, 0 .. MT*128-1
        constexpr int PF = F4 ? 2 : 4;
        const size_t pitch = p.a_two_planes ? (size_t)p.Kp : (size_t)p.Kp / 2;  // uint4 per row
        const int gsz = p.a_two_planes ? 4 : 2;                                    // uint4 per 256-element group
        constexpr int RW = F4 ? 2 : 1;  // uint4 per plane and stage
        uint4 ring_s[PF][RW], ring_z[PF][RW];
        // prefetch cursor: (tile, chunk) of the next load of this group
        long long pf_t = blockIdx.x;
        int pf_c = grp;
        while (pf_c >= nchunks) { pf_c -= nchunks; pf_t += gridDim.x; }
        // implicit im2row: window origin of this thread's row in the prefetch cursor's tile
        int im_n = 0, im_ih0 = 0, im_iw0 = 0;
        long long im_tile = -1;
        const size_t img_plane = (size_t)p.H * p.W * p.Cp;  // words per image and plane
        const int img_planes = p.a_two_planes ? 2 : 1;
        auto fetch = [&](uint4 (&ds)[RW], uint4 (&dz)[RW]) {
            if (pf_t < ntiles) {
                if (F4 && p.img) {
                    if (im_tile != pf_t) {
                        im_tile = pf_t;
                        const long long row = min((pf_t / ntn) * BMT + r, p.M - 1);
                        const long long n_img = row / p.OHW;
                        const int rem = (int)(row - n_img * p.OHW);
                        const int oh = rem / p.OW;
                        im_n = (int)n_img;
                        im_ih0 = oh * p.SH - p.PH;
                        im_iw0 = (rem - oh * p.OW) * p.SW - p.PW;
                    }
                    const uint64_t* base = p.img + (size_t)im_n * img_planes * img_plane;
                    uint64_t sw[4], zw[4];
                    if ((p.Cp & 3) == 0) {
                        // the four words of a stage are four neighbouring channel groups of one tap
                        const uint32_t e = tap_at(4 * pf_c);
                        const int ih = im_ih0 + (int)(e >> 24), iw = im_iw0 + (int)((e >> 16) & 0xFF);
                        if (ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) {
                            const uint4* src = reinterpret_cast<const uint4*>(base + ((size_t)ih * p.W + iw) * p.Cp + (e & 0xFFFF));
                            const uint4 a0 = __ldg(src), a1 = __ldg(src + 1);
                            ds[0] = a0; ds[1 % RW] = a1;
                            if (p.a_two_planes) {
                                const uint4* zsrc = reinterpret_cast<const uint4*>(reinterpret_cast<const uint64_t*>(src) + img_plane);
                                dz[0] = __ldg(zsrc); dz[1 % RW] = __ldg(zsrc + 1);
                            } else {
                                dz[0] = dz[1 % RW] = make_uint4(0, 0, 0, 0);
                            }
                        } else {
                            const uint32_t zf = p.a_two_planes ? 0xFFFFFFFFu : 0u;  // padding: ternary zero, binary +1
                            ds[0] = ds[1 % RW] = make_uint4(0, 0, 0, 0);
                            dz[0] = dz[1 % RW] = make_uint4(zf, zf, zf, zf);
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const uint32_t e = tap_at(4 * pf_c + q);
                            const int ih = im_ih0 + (int)(e >> 24), iw = im_iw0 + (int)((e >> 16) & 0xFF);
                            sw[q] = 0;
                            zw[q] = p.a_two_planes ? ~0ull : 0ull;
                            if (e != 0xFFFFFFFFu && ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) {
                                const uint64_t* src = base + ((size_t)ih * p.W + iw) * p.Cp + (e & 0xFFFF);
                                sw[q] = __ldg(src);
                                if (p.a_two_planes) zw[q] = __ldg(src + img_plane);
                            }
                        }
                        ds[0] = make_uint4((uint32_t)sw[0], (uint32_t)(sw[0] >> 32), (uint32_t)sw[1], (uint32_t)(sw[1] >> 32));
                        ds[1 % RW] = make_uint4((uint32_t)sw[2], (uint32_t)(sw[2] >> 32), (uint32_t)sw[3], (uint32_t)(sw[3] >> 32));
                        dz[0] = make_uint4((uint32_t)zw[0], (uint32_t)(zw[0] >> 32), (uint32_t)zw[1], (uint32_t)(zw[1] >> 32));
                        dz[1 % RW] = make_uint4((uint32_t)zw[2], (uint32_t)(zw[2] >> 32), (uint32_t)zw[3], (uint32_t)(zw[3] >> 32));
                    }
                    pf_c += NG;
                    while (pf_c >= nchunks) { pf_c -= nchunks; pf_t += gridDim.x; }
                    return;
                }
                const uint4* rowp = p.A + (size_t)min((pf_t / ntn) * BMT + r, p.M - 1) * pitch;
                if (F4) {
                    const uint4* row = rowp + (size_t)pf_c * gsz;
#pragma unroll
                    for (int q = 0; q < RW; q++) {
                        ds[q] = __ldg(row + q);
                        dz[q] = p.a_two_planes ? __ldg(row + 2 + q) : make_uint4(0, 0, 0, 0);
                    }
                } else {
                    const uint4* row = rowp + (size_t)(pf_c >> 1) * gsz + (pf_c & 1);
                    ds[0] = __ldg(row);
                    dz[0] = p.a_two_planes ? __ldg(row + 2) : make_uint4(0, 0, 0, 0);
                }
                pf_c += NG;
                while (pf_c >= nchunks) { pf_c -= nchunks; pf_t += gridDim.x; }
            }
        };
#pragma unroll
        for (int i = 0; i < PF; i++) fetch(ring_s[i], ring_z[i]);
        long long my_tiles = (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
        if (blockIdx.x >= ntiles) my_tiles = 0;
        const long long total_it = my_tiles * nchunks;
        for (long long it0 = grp; it0 < total_it; it0 += (long long)NG * PF) {
#pragma unroll
            for (int i = 0; i < PF; i++) {
                const long long it = it0 + (long long)i * NG;
                if (it < total_it) {
                    const int s = (int)(it % NSTG);
                    if (!mbar_wait(bar_empty + 8 * s, (uint32_t)((it / NSTG) & 1) ^ 1, abort_flag, p.status, 4)) goto done;
                    {
                        unsigned char* tile = sA + s * A_STAGE + (r >> 7) * A_SUB;
                        if constexpr (F4) store_row_stage_f4(tile, r & 127, ring_s[i], ring_z[i]);
                        else store_row_chunk(tile, r & 127, ring_s[i][0], ring_z[i][0]);
                    }
                    fence_proxy_async();  // generic-proxy smem writes -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * s);
                    fetch(ring_s[i], ring_z[i]);
                }
            }
        }
    } else if (QF && warp >= Cfg::WARP_Q0) {
        uint64_t* qbars = reinterpret_cast<uint64_t*>(smem + Cfg::Q_OFF + Cfg::QSTG * Cfg::Q_STAGE);
        if (warp < Cfg::WARP_Q0 + 4)
            quantise_items(plain_quant_args(p.qthr, p.qimg, p.q_sync, p.qN, p.qC, p.q_nbands, p.Cp, p.H, p.W, p.status, p.q_nhwc), &tmap_q, smem + Cfg::Q_OFF, qbars,
                           abort_flag, tid - Cfg::WARP_Q0 * 32);
        else if (lane == 0)
            publish_items(p.q_sync, p.status, qbars, abort_flag);
    } else {
        // ---------------- epilogue ----------------
        const int q = warp & 3;                 // tensor-memory lane quadrant this warp may access
        const int sub = ((warp - WARP_EPI0) >> 2) % MT;   // which 128-row sub-tile (accumulator) it drains
        const int ecol = ((warp - WARP_EPI0) >> 2) / MT;  // which share of the columns
        constexpr int ECOLS = BN / EPW;
        const bool alpha_in_unit = p.alpha > 0.f && p.alpha <= 1.f;
        const int bias_magic = 0x4B400000 + p.acc_bias;
        const float bias_f = (float)p.acc_bias;  // +0.0f when there is none: a + 0.0f also turns a -0 sum into +0
        uint32_t lt = 0;
        const uint32_t bar_release = (CG == 2 && rank != 0) ? mapa_shared(bar_tempty, 0) : 0u;  // pair: the first block's barrier
        // quantised output with 0 < alpha <= 1: PReLU and the next layer's rule collapse into thresholds on
        // the accumulator (two instructions per output and plane instead of evaluating the PReLU first)
        const bool by_thr = F4 && p.pimg != nullptr && alpha_in_unit;
        // (not in the one-launch form, whose producers write plain images only: the code is compiled out there, where
        // its mere presence measured one percent of the large layer)
        if (F4 && !QF && p.pimg && p.pimg_e2m1 && p.o_HpWp)
            fill_output_border(reinterpret_cast<uint4*>(p.pimg), p.cp_next, p.OHW / p.OW, p.OW, (int)(p.M / p.OHW), p.o_Wp, p.o_HpWp, p.o_PH, p.o_PW,
                               (long long)blockIdx.x * (32 * 4 * MT * EPW) + (tid - 32 * WARP_EPI0), (long long)gridDim.x * (32 * 4 * MT * EPW));
        const bool rows16 = F4 && p.pimg == nullptr && p.layout == TNNS_NHWC && (p.KN & 1) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 7) == 0;
        tnns_thr::Pair qt = {0.f, 0.f};
        long long qt_img = -1;
        for (long long t = unit; t < ntiles; t += nunits, lt++) {
            const int buf = lt % NBUF;
            const long long m0 = (t / ntn) * TILE_M + (long long)rank * BMT + sub * BM;
            const int n0 = (int)(t % ntn) * BN;
            // the row's image (a 64-bit division) and threshold: worked out while the tile's MMAs run
            const long long row = m0 + q * 32 + lane;
            const bool row_ok = row < p.M;
            const long long n_img = row_ok ? row / p.OHW : 0;
            const int rem = (int)(row - n_img * p.OHW);
            float* ybase = (p.layout == TNNS_NHWC) ? p.y + (size_t)row * p.KN : p.y + (size_t)n_img * p.KN * p.OHW + rem;
            const float tq = (p.pimg && row_ok) ? __ldg(p.thr_next + n_img) + 0.0f : 0.f;  // + 0.0f: -0 acts as +0
            if (by_thr && row_ok && n_img != qt_img) {
                // the next layer's rule as thresholds on the raw accumulator, once per image this thread meets
                qt = tnns_thr::make(tq, p.alpha, bias_f, p.next_ternary != 0);
                qt_img = n_img;
            }
            if (!mbar_wait(bar_tfull + 8 * buf, (lt / NBUF) & 1, abort_flag, p.status, 5)) goto done;
            tc_fence_after();
            // overlapping sets: start with the 32 columns shared with the other set (the last of
            // set 0, the first of set 1) if this warp owns them, and release after the first slice
            constexpr int NSL = ECOLS / 32;
            int start = 0;
            if (OVL && buf == 0 && ecol == EPW - 1) start = NSL - 1;
#pragma unroll 1
            for (int i = 0; i < NSL; i++) {
                const int cb = ecol * ECOLS + ((i + start) % NSL) * 32;
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * ACC_OFF + sub * BN + cb);
                if (rows16) {
                    // pixel-major fp32 output: fetched in the shape that gives four lanes one 32-byte piece of a row
                    tmem_ld_16x256b_x4(taddr, v);
                    tmem_ld_16x256b_x4(taddr + (16u << 16), v + 16);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (OVL ? (i == 0) : (i == NSL - 1)) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (CG == 2 && rank != 0) mbar_arrive_cluster(bar_release + (OVL ? 0 : 8 * buf));
                            else mbar_arrive(OVL ? bar_tempty : bar_tempty + 8 * buf);
                        }
                    }
                    const long long row0 = m0 + q * 32;
                    if (row0 < p.M) {
                        float f[32];
                        prelu32_f4(v, f, alpha_in_unit, p.acc_bias, bias_f, p.alpha, p.zero_passes);
                        store_rows16(f, p.y + (size_t)row0 * p.KN + (n0 + cb), p.KN, p.M - row0, p.KN - (n0 + cb), lane);
                    }
                    continue;
                }
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                      "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                      "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (OVL ? (i == 0) : (i == NSL - 1)) {
                    // the last slice (overlapping sets: the shared slice) is in registers: hand
                    // the columns back before storing it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2 && rank != 0) mbar_arrive_cluster(bar_release + (OVL ? 0 : 8 * buf));
                        else mbar_arrive(OVL ? bar_tempty : bar_tempty + 8 * buf);
                    }
                }
                if (row_ok) {
                    float f[32];
                    uint32_t sg = 0, nz = 0;
                    if (by_thr) {
                        if (p.next_ternary) {
                            uint32_t above = 0;
#pragma unroll
                            for (int j = 31; j >= 0; j--) {
                                sg = push_sign(sg, __uint_as_float(v[j]) + qt.n1);
                                above = push_sign(above, qt.t2 - __uint_as_float(v[j]));
                            }
                            nz = sg | above;
                        } else {
#pragma unroll
                            for (int j = 31; j >= 0; j--) sg = push_sign(sg, __uint_as_float(v[j]) + qt.n1);
                        }
                    } else if (F4) {
                        prelu32_f4(v, f, alpha_in_unit, p.acc_bias, bias_f, p.alpha, p.zero_passes);
                    } else {
                        // int -> float without the conversion unit: for |a| < 2^22 the float with bit
                        // pattern 0x4B400000 + a is 1.5*2^23 + a exactly, so subtracting 1.5*2^23 gives a.
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float a = __int_as_float((int)v[j] + bias_magic) - 12582912.0f;
                            f[j] = a * ((p.zero_passes ? a >= 0.f : a > 0.f) ? 1.0f : p.alpha);  // a == 0 is +0 here
                        }
                    }
                    const int c0 = n0 + cb;
                    const bool full = c0 + 32 <= p.KN;
                    if (p.pimg) {
                        // Quantise the 32 channels this thread holds for its pixel straight into one
                        // 32-bit lane of the next layer's bit planes (same rules as the pack kernel:
                        // sign = f < -t, non-zero = |f| > t; binary: f < t), channels past KN absent.
                        if (c0 < p.cp_next * 64) {
                            if (!by_thr) {
                                if (p.next_ternary) quantise32_ternary(f, tq, sg, nz);
                                else sg = quantise32_binary(f, tq);
                            }
                            const int have = p.KN - c0;
                            const uint32_t valid = have >= 32 ? 0xFFFFFFFFu : (have > 0 ? (1u << have) - 1u : 0u);
                            if (p.pimg_e2m1) {
                                // the 32 channels as 16 bytes of e2m1 operands, where the copy-engine GEMM
                                // of the next layer expects them (same expansion routine as everywhere)
                                uint32_t w4[4];
                                tnns_expand32_f4(sg & valid, ~(nz & valid), w4);
                                // the row's pixel in the next layer's image: plain, or inside its border (worked out here, in the
                                // branch that stores it: as a value kept across the slices it cost the fp32 path 3 % on the large layer)
                                long long opix = n_img * p.OHW + rem;
                                if (!QF && p.o_HpWp) {
                                    const int oh = rem / p.OW;
                                    opix = n_img * p.o_HpWp + (long long)(oh + p.o_PH) * p.o_Wp + (rem - oh * p.OW) + p.o_PW;
                                }
                                uint4* px = reinterpret_cast<uint4*>(p.pimg) + (size_t)opix * ((size_t)p.cp_next * 2) + (c0 >> 5);
                                *px = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                            } else {
                                const int planes = p.next_ternary ? 2 : 1;
                                const size_t lanes = (size_t)p.cp_next * 2;  // 32-bit lanes per pixel and plane
                                uint32_t* px = p.pimg + ((size_t)n_img * planes * p.OHW + rem) * lanes + (c0 >> 5);
                                px[0] = sg & valid;
                                if (p.next_ternary) px[(size_t)p.OHW * lanes] = ~(nz & valid);
                            }
                        }
                    } else if (p.layout == TNNS_NHWC) {
                        if (full && (p.KN & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                __stcs(reinterpret_cast<float4*>(ybase + c0 + j), make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (c0 + j < p.KN) __stcs(ybase + c0 + j, f[j]);
                        }
                    } else {
                        float* yc = ybase + (size_t)c0 * p.OHW;
                        if (full) {
#pragma unroll
                            for (int j = 0; j < 32; j++, yc += p.OHW) __stcs(yc, f[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++, yc += p.OHW)
                                if (c0 + j < p.KN) __stcs(yc, f[j]);
                        }
                    }
                }
            }
        }
    }

done:
    __syncwarp();
    if (*abort_flag && warp == WARP_TMA && lane == 0) {
        // a wait gave up: give the bulk copies already issued time to land before smem is released
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    tc_fence_before();
    // pair: neither block may leave (and release its shared and tensor memory) while the other can
    // still arrive on its barriers or the first block's MMAs still use them
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    if (warp == WARP_MMA) {
        tc_fence_after();
        if (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if (QF && p.q_self_clean && warp == WARP_TMA) {
        // Every role of this block is past its last use of the synchronisation words.  The block
        // that leaves last zeroes them, so the next launch on the stream finds them clean without
        // a clearing operation in between (also after a wait that gave up: every block comes here).
        unsigned int left = 0;
        if (lane == 0) {
            __threadfence();
            left = atomicAdd(p.q_sync + 1, 1u);
        }
        left = __shfl_sync(0xFFFFFFFFu, left, 0);
        if (left == gridDim.x - 1) {
            __threadfence();
            for (int i = lane; i < Q_FLAG0 + p.qN; i += 32) p.q_sync[i] = 0;
        }
    }
}

// Self-test of the bounded wait: one warp waits on an mbarrier that nothing ever completes.  The
// wait gives up after its limit, raises the status word and the kernel returns normally.
__global__ void wait_expiry_selftest_kernel(unsigned int* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 0x7F);
}

// Issue-bound tensor-pipe rate: one block per SM keeps one 128 x 256 operand pair (pseudo-random
// {-1,0,+1} values) in shared memory and issues `iters` groups of four MMAs on it back to back,
// with no loads, expansion or epilogue.  What the GEMM kernel's 2*M*N*K / t is compared with.
template <bool F4>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, unsigned int* status) {
    constexpr int BN = 256;
    constexpr uint32_t IDESC = (F4 ? (1u << 23) : (2u << 4)) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + A_SUB;
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int r = tid; r < BM + BN; r += blockDim.x) {
        uint32_t h = (uint32_t)r * 2654435761u + blockIdx.x * 40503u + 12345u;
        uint4 sg[2], zr[2];
        uint32_t* ps = reinterpret_cast<uint32_t*>(sg);
        uint32_t* pz = reinterpret_cast<uint32_t*>(zr);
        for (int i = 0; i < 8; i++) {
            h = h * 1664525u + 1013904223u; ps[i] = h;
            h = h * 1664525u + 1013904223u; pz[i] = h & (h >> 7);  // about a quarter zeros
        }
        unsigned char* tile = r < BM ? sA : sB;
        const int rr = r < BM ? r : r - BM;
        if (F4) store_row_stage_f4(tile, rr, sg, zr);
        else store_row_chunk(tile, rr, sg[0], zr[0]);
    }
    if (tid == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (F4) {
        const uint32_t one = 0x7F7F7F7Fu;
        for (uint32_t c = 0; c < 32; c += 8) {
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + 480 + c;
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(one) : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }
    if (tid == 0) {
        const uint64_t da = make_desc(smem_u32(sA)), db = make_desc(smem_u32(sB));
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int k = 0; k < KCH / 32; k++) {
                if (F4) tc_mma_f4(tmem_base, da + 2 * k, db + 2 * k, IDESC, tmem_base + 480, tmem_base + 496, (it | k) ? 1u : 0u);
                else tc_mma_i8(tmem_base, da + 2 * k, db + 2 * k, IDESC, (it | k) ? 1u : 0u);
            }
        }
        tc_commit(smem_u32(&bar));
        mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 8);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int BN, int MT, bool F4, bool ATMA = false, int CG = 1, int TAPS = 1, bool QF = false>
int launch_cfg(tnns_cuda_ctx* ctx, const GemmArgs& a, cudaStream_t stream, const CUtensorMap* tmap_a = nullptr,
               const CUtensorMap* tmap_b = nullptr, const CUtensorMap* tmap_q = nullptr) {
    using Cfg = TcCfg<BN, MT, F4, ATMA, CG, TAPS, QF>;
    auto kern = gemm_tc_kernel<BN, MT, F4, ATMA, CG, TAPS, QF>;
    static const CUtensorMap no_map = {};
    // once per kernel and device: the attribute belongs to (function, device), and the call costs a microsecond per launch
    static bool smem_set[64] = {false};
    if (!smem_set[ctx->device & 63]) {
        TNNS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
        smem_set[ctx->device & 63] = true;
    }
    const long long tiles = ((a.M + CG * MT * BM - 1) / (CG * MT * BM)) * ((a.KN + BN - 1) / BN);
    // the launch may be scheduled while its predecessor on the stream drains (the kernel
    // waits for it, griddepcontrol.wait, before it touches global data)
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    nattr++;
    if (CG == 1) {
        const int grid = (int)std::min<long long>(tiles, ctx->sm_count);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(Cfg::NTHREADS);
        cfg.dynamicSmemBytes = Cfg::SMEM;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = nattr;
        TNNS_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a, tmap_a ? *tmap_a : no_map, no_map, tmap_q ? *tmap_q : no_map));
    } else {
        // block pairs: clusters of two consecutive blocks, as many as can be resident at once (the
        // kernel is persistent; a pair that had to wait for a free TPC would start its whole tile
        // sequence after the others finished)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CG * (ctx->sm_count / CG));
        cfg.blockDim = dim3(Cfg::NTHREADS);
        cfg.dynamicSmemBytes = Cfg::SMEM;
        cfg.stream = stream;
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = CG;
        attr[nattr].val.clusterDim.y = 1;
        attr[nattr].val.clusterDim.z = 1;
        nattr++;
        cfg.attrs = attr;
        cfg.numAttrs = nattr;
        static int max_pairs[64] = {0};  // per device
        int& mp = max_pairs[ctx->device & 63];
        if (mp == 0) {
            int n = 0;
            TNNS_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
            if (n <= 0) return tnns_fail(TNNS_ERR_CUDA, "no block pair of the tensor-core GEMM fits this device");
            mp = std::min(n, ctx->sm_count / CG);
        }
        cfg.gridDim = dim3(CG * (int)std::min<long long>(tiles, mp));
        TNNS_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a, tmap_a ? *tmap_a : no_map, tmap_b ? *tmap_b : no_map, tmap_q ? *tmap_q : no_map));
    }
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}

// One 128-row accumulator per block (MT = 1) measured fastest on every layer shape tried: more
// blocks in flight and a deeper ring; MT = 2 (two stacked accumulators, half the weight traffic
// per MMA) was 10-70 % slower and is not instantiated.
template <int BN, bool F4>
int launch_bn(tnns_cuda_ctx* ctx, const GemmArgs& a, cudaStream_t stream) {
    return launch_cfg<BN, 1, F4>(ctx, a, stream);
}

}  // namespace

int tnns_i8_tile_n(int KN) { return KN <= 64 ? 64 : (KN <= 128 ? 128 : 256); }

// Builds both operand images of a layer's weights: int8 (128 K elements per 128-byte row and
// stage) and e2m1 (256 K elements per row and stage).
int tnns_build_i8_weights(tnns_cuda_ctx* ctx, tnns_cuda_weights* w) {
    const int BN = tnns_i8_tile_n(w->KN);
    const int ntn = (w->KN + BN - 1) / BN;
    const bool two = (w->type == TNN || w->type == BTN);
    for (int f4 = 0; f4 < 2; f4++) {
        const int nch = f4 ? w->Kp / 4 : w->Kp / 2;
        const size_t bytes = (size_t)ntn * nch * BN * KCH;
        void* img = nullptr;
        TNNS_CUDA_TRY(cudaMalloc(&img, bytes));
        if (f4) { w->d_f4 = (uint8_t*)img; w->f4_bytes = bytes; }
        else { w->d_i8 = (int8_t*)img; w->i8_bytes = bytes; w->i8_kchunks = nch; }
        TNNS_CUDA_TRY(cudaMemset(img, 0, bytes));
        const long long total = (long long)w->KN * nch;
        const int blocks = (int)std::min<long long>((total + 127) / 128, 4096);
        // TBN: ternary activations meet binary weights, whose pad words read +1; the products there are
        // zero only because the activation pad words are zeros -- writing zero weights instead changes
        // nothing and lets the tensor-copy form skip those K positions.  (BNN keeps +1: its epilogue
        // constant counts the padded +1 x +1 products.)
        const int zero_from = (f4 && w->type == TBN) ? w->Kw : -1;
        expand_weights_kernel<<<blocks, 128>>>(reinterpret_cast<const uint4*>(w->d_packed), reinterpret_cast<unsigned char*>(img), w->KN,
                                                w->Kp, BN, two ? 1 : 0, f4, zero_from);
        tnns_count_launch();
        TNNS_CUDA_TRY(cudaGetLastError());
    }
    // tap table for the implicit-im2row form: plane word j -> kh<<24 | kw<<16 | ic
    if (w->C > 0 && w->KH < 256 && w->KW < 256 && w->Cp < 65536) {
        std::vector<uint32_t> tab(w->Kp, 0xFFFFFFFFu);
        for (int j = 0; j < w->Kw; j++) {
            const int ic = j % w->Cp, kw = (j / w->Cp) % w->KW, kh = j / (w->Cp * w->KW);
            tab[j] = ((uint32_t)kh << 24) | ((uint32_t)kw << 16) | (uint32_t)ic;
        }
        TNNS_CUDA_TRY(cudaMalloc(&w->d_jtab, tab.size() * sizeof(uint32_t)));
        TNNS_CUDA_TRY(cudaMemcpy(w->d_jtab, tab.data(), tab.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
    }
    TNNS_CUDA_TRY(cudaDeviceSynchronize());
    return TNNS_OK;
}

int tnns_launch_gemm_tc(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_a, float* d_y, long long M, int OHW, float alpha,
                        int layout, bool f4, cudaStream_t stream, void* d_pimg, const float* d_thr_next, int next_ternary,
                        const TnnsGeom* implicit_geom) {
    if (M == 0) return TNNS_OK;
    const void* img = f4 ? (const void*)w->d_f4 : (const void*)w->d_i8;
    if (!img) return tnns_fail(TNNS_ERR_UNSUPPORTED, "weights carry no tensor-core operand image");
    if (w->Kp >= 65536) return tnns_fail(TNNS_ERR_UNSUPPORTED, "rows of %d plane words exceed the tensor-core path's exact range", w->Kp);
    GemmArgs a;
    a.A = reinterpret_cast<const uint4*>(d_a);
    a.Bimg = reinterpret_cast<const unsigned char*>(img);
    a.y = d_y;
    a.M = M;
    a.KN = w->KN;
    a.Kp = w->Kp;
    a.OHW = OHW;
    // one output pixel per image (fully connected layers): both layouts are the same memory, and the pixel-major
    // epilogue writes 16 bytes per lane where the channel-major one would write 4 (rows are KN floats apart either way)
    a.layout = OHW == 1 ? TNNS_NHWC : layout;
    a.a_two_planes = (w->type == TNN || w->type == TBN) ? 1 : 0;
    a.acc_bias = (w->type == BNN) ? w->K_unpack - 64 * w->Kp : 0;
    a.zero_passes = w->type != TNN;
    a.alpha = alpha;
    a.status = ctx->d_status;
    a.pimg = reinterpret_cast<uint32_t*>(d_pimg);
    a.thr_next = d_thr_next;
    a.next_ternary = next_ternary != 0;
    a.pimg_e2m1 = next_ternary == 2;
    a.o_Wp = a.o_HpWp = a.o_PH = a.o_PW = 0;
    a.cp_next = (w->KN + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS;
    a.img = nullptr;
    a.jtab = nullptr;
    a.H = a.W = a.OW = a.Cp = a.SH = a.SW = a.PH = a.PW = 0;
    a.qx = a.qthr = nullptr; a.qimg = nullptr; a.q_sync = nullptr; a.qN = a.qC = a.q_nbands = a.q_self_clean = a.q_nhwc = 0;
    if (implicit_geom) {
        // d_a is the quantised image of the layer input, not an im2row matrix
        if (!f4 || !w->d_jtab) return tnns_fail(TNNS_ERR_UNSUPPORTED, "implicit im2row needs the 4-bit tensor-core GEMM and layer geometry");
        const TnnsGeom& g = *implicit_geom;
        a.img = reinterpret_cast<const uint64_t*>(d_a);
        a.jtab = w->d_jtab;
        a.H = g.H; a.W = g.W; a.OW = g.OW; a.Cp = g.Cp; a.SH = g.SH; a.SW = g.SW; a.PH = g.PH; a.PW = g.PW;
    }
    const int bn = tnns_i8_tile_n(w->KN);
    if (f4) {
        switch (bn) {
            case 64: return launch_bn<64, true>(ctx, a, stream);
            case 128: return launch_bn<128, true>(ctx, a, stream);
            default: return launch_bn<256, true>(ctx, a, stream);
        }
    }
    switch (bn) {
        case 64: return launch_bn<64, false>(ctx, a, stream);
        case 128: return launch_bn<128, false>(ctx, a, stream);
        default: return launch_bn<256, false>(ctx, a, stream);
    }
}

// ---------------------------------------------------------------------------------------
// Tensor-copy activations: the tensor map of the e2m1 image and the launch
// ---------------------------------------------------------------------------------------
bool tnns_im2col_supported(const tnns_cuda_weights* w, const TnnsGeom& g) {
    if (!(w->type == TNN || w->type == TBN)) return false;   // outside the image the copy engine writes 0, a ternary zero
    if (!w->d_f4 || !w->d_jtab || w->Kp >= 65536) return false;
    if (tnns_i8_tile_n(w->KN) != 256 && tnns_i8_tile_n(w->KN) != 128 && tnns_i8_tile_n(w->KN) != 64) return false;
    if (g.Cp != 1 && g.Cp != 2 && g.Cp % 4 != 0) return false;  // a 128-byte stage row = 1 tap of 256 channels, 2 of 128 or 4 of 64
    if (g.KH > 255 || g.KW > 255 || g.SH > 8 || g.SW > 8) return false;          // filter offsets are 8 bits, traversal strides <= 8
    if (g.PH > 128 || g.PW > 128 || g.PH - (g.KH - 1) < -128 || g.PW - (g.KW - 1) < -128) return false;  // box corners are 8 bits
    return true;
}

namespace {
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const int*,
                                   const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_im2col_map(CUtensorMap* map, const void* d_image, const TnnsGeom& g) {
    static EncodeIm2colFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        TNNS_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !fn) return tnns_fail(TNNS_ERR_UNSUPPORTED, "the driver offers no cuTensorMapEncodeIm2col");
        encode = reinterpret_cast<EncodeIm2colFn>(fn);
    }
    // the image as a (bytes-of-channels, W, H, N) tensor of bytes; a box = 128 bytes x 128 base pixels
    const cuuint64_t cbytes = (cuuint64_t)g.Cp * 32;
    const cuuint64_t dims[4] = {cbytes, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.N};
    const cuuint64_t strides[3] = {cbytes, cbytes * g.W, cbytes * g.W * g.H};
    // the base pixel (top-left of the filter window) moves over [-pad, size + pad - kernel]
    const int lower[2] = {-g.PW, -g.PH};
    const int upper[2] = {g.PW - (g.KW - 1), g.PH - (g.KH - 1)};
    const cuuint32_t estr[4] = {1, (cuuint32_t)g.SW, (cuuint32_t)g.SH, 1};
    // channels per pixel and copy: 128 bytes (256 channels), or the whole pixel when it has 64 or 32 bytes
    const int taps = g.Cp == 1 ? 4 : (g.Cp == 2 ? 2 : 1);
    const CUtensorMapSwizzle swz = taps == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : (taps == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(d_image), dims, strides, lower, upper, 128 / taps, BM, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tnns_fail(TNNS_ERR_CUDA, "cuTensorMapEncodeIm2col failed with driver error %d", (int)r);
    // Drivers up to 13.1 set a flag in im2col maps of tensors below 128 KiB that must be clear
    // (the correction CUTLASS applies to its im2col descriptors, cute/atom/copy_traits_sm90_im2col.hpp).
    int driver = 0;
    TNNS_CUDA_TRY(cudaDriverGetVersion(&driver));
    if (driver <= 13010 && cbytes * g.W * g.H * g.N < 131072) reinterpret_cast<uint64_t*>(map)[1] &= ~(1ull << 21);
    return TNNS_OK;
}
}  // namespace

namespace {
// The expanded weight image as rows of 128 bytes; a box = the 128 rows one block of a pair holds
// of one stage.  The image is stored swizzled already, so the copy itself does not swizzle.
int encode_weight_map(CUtensorMap* map, const tnns_cuda_weights* w, int BN) {
    return tnns_tensor_map_2d(map, 1, w->d_f4, KCH, w->f4_bytes / KCH, KCH, KCH, BN / 2);
}
}  // namespace

// pairs: 0 = decide by size, 1 = single blocks, 2 = block pairs (kernel tile of 256 only)
size_t tnns_fused_sync_bytes(int N) { return ((size_t)(Q_FLAG0 + N) * sizeof(unsigned int) + 127) & ~(size_t)127; }

bool tnns_fused_supported(const tnns_cuda_weights* w, const TnnsGeom& g, const float* d_x, int layout) {
    if (!tnns_im2col_supported(w, g)) return false;
    const long long HW = (long long)g.H * g.W;
    // the quantiser warps receive 128 pixels x 64 channels per item: NCHW as one tensor copy (rows of H*W floats, 16-byte pitch
    // and base), NHWC as two swizzled boxes of 32 channels (rows of C floats, 16-byte pitch and base)
    if (layout == TNNS_NHWC ? !tnns_quantise_tma_nhwc_supported(d_x, g.N, g.C, g.H, g.W) : !tnns_quantise_tma_supported(d_x, g.H, g.W, layout)) return false;
    const long long items = (long long)g.N * ((HW + Q_PIX - 1) / Q_PIX) * g.Cp;
    return items < 0x7FFFFFFFLL;
}

// Synchronisation words of a one-launch layer (item counter, count of blocks that have left, one word
// per image).  The context keeps one set of its own, bound to the first stream that launches a fused
// form: every launch leaves them zeroed (the last block out clears them), so launches on that stream
// need no clearing operation, and consecutive launches can overlap their set-up with the
// predecessor's tail (programmatic dependent launch).  Launches on any other stream use the words
// in the caller's workspace, cleared here on `stream`.
int tnns_fused_sync_prepare(tnns_cuda_ctx* ctx, int N, cudaStream_t stream, unsigned int* caller_words, unsigned int** words_out, int* self_clean) {
    const size_t words = (size_t)Q_FLAG0 + (size_t)N;
    if (ctx->fused_sync_words < words && (!ctx->fused_sync || ctx->fused_sync_stream == stream)) {
        TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
        TNNS_CUDA_TRY(cudaDeviceSynchronize());  // earlier launches may still use the old words
        if (ctx->fused_sync) cudaFree(ctx->fused_sync);
        ctx->fused_sync = nullptr;
        ctx->fused_sync_words = 0;
        const size_t cap = std::max<size_t>(words, 4096);
        TNNS_CUDA_TRY(cudaMalloc(&ctx->fused_sync, cap * sizeof(unsigned int)));
        TNNS_CUDA_TRY(cudaMemset(ctx->fused_sync, 0, cap * sizeof(unsigned int)));
        ctx->fused_sync_words = cap;
        ctx->fused_sync_stream = stream;
    }
    const bool own = ctx->fused_sync && ctx->fused_sync_words >= words && ctx->fused_sync_stream == stream;
    if (!own) TNNS_CUDA_TRY(cudaMemsetAsync(caller_words, 0, tnns_fused_sync_bytes(N), stream));
    *words_out = own ? ctx->fused_sync : caller_words;
    *self_clean = own ? 1 : 0;
    return TNNS_OK;
}

int tnns_launch_gemm_im2col(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const TnnsGeom& g, float alpha,
                            int layout, cudaStream_t stream, int pairs, void* d_pimg, const float* d_thr_next, int next_format,
                            const TnnsFusedInput* fused, int next_PH, int next_PW) {
    const long long M = (long long)g.N * g.OH * g.OW;
    if (M == 0) return TNNS_OK;
    if (!tnns_im2col_supported(w, g)) return tnns_fail(TNNS_ERR_UNSUPPORTED, "layer shape or type outside the tensor-copy activation path");
    if (reinterpret_cast<uintptr_t>(d_image) & 15) return tnns_fail(TNNS_ERR_INVALID, "image must be 16-byte aligned");
    unsigned int* fused_words = nullptr;
    int fused_self_clean = 0;
    if (fused) {
        if (!fused->d_x || !fused->d_thr || !fused->d_sync) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
        if (!tnns_fused_supported(w, g, fused->d_x, layout))
            return tnns_fail(TNNS_ERR_UNSUPPORTED, "fused quantisation needs a 16-byte aligned input: NCHW with H*W a multiple of four, or NHWC with C a multiple of four");
        if (reinterpret_cast<uintptr_t>(fused->d_sync) & 127) return tnns_fail(TNNS_ERR_INVALID, "synchronisation words must be 128-byte aligned");
        int rc0 = tnns_fused_sync_prepare(ctx, g.N, stream, fused->d_sync, &fused_words, &fused_self_clean);
        if (rc0) return rc0;
    }
    CUtensorMap map;
    int rc = encode_im2col_map(&map, d_image, g);
    if (rc) return rc;
    GemmArgs a;
    a.A = nullptr;
    a.Bimg = reinterpret_cast<const unsigned char*>(w->d_f4);
    a.y = d_y;
    a.M = M;
    a.KN = w->KN;
    a.Kp = w->Kp;
    a.OHW = g.OH * g.OW;
    a.layout = a.OHW == 1 ? TNNS_NHWC : layout;  // one pixel per image: same memory, wider stores (see above)
    a.a_two_planes = 1;
    a.acc_bias = 0;
    a.zero_passes = w->type != TNN;
    a.alpha = alpha;
    a.status = ctx->d_status;
    a.pimg = reinterpret_cast<uint32_t*>(d_pimg);
    a.thr_next = d_thr_next;
    a.next_ternary = next_format != 0;
    a.pimg_e2m1 = next_format == 2 || next_format == 3;
    a.o_Wp = a.o_HpWp = a.o_PH = a.o_PW = 0;
    if (next_format == 3) {
        // bordered 4-bit image for a slab-fed next layer with padding (next_PH, next_PW)
        if (fused) return tnns_fail(TNNS_ERR_UNSUPPORTED, "the one-launch form writes plain output images only");
        if (!d_pimg || next_PH < 0 || next_PW < 0) return tnns_fail(TNNS_ERR_INVALID, "bordered output needs an output image and a non-negative border");
        a.o_PH = next_PH; a.o_PW = next_PW;
        a.o_Wp = g.OW + 2 * next_PW;
        a.o_HpWp = (g.OH + 2 * next_PH) * a.o_Wp;
        if ((long long)g.N * a.o_HpWp >= 0x7FFFFFFFLL) return tnns_fail(TNNS_ERR_UNSUPPORTED, "bordered output image too large");
    }
    a.cp_next = (w->KN + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS;
    a.img = nullptr;
    a.jtab = w->d_jtab;
    a.qx = a.qthr = nullptr; a.qimg = nullptr; a.q_sync = nullptr; a.qN = a.qC = a.q_nbands = a.q_self_clean = a.q_nhwc = 0;
    a.H = g.H; a.W = g.W; a.OW = g.OW; a.Cp = g.Cp; a.SH = g.SH; a.SW = g.SW; a.PH = g.PH; a.PW = g.PW;
    alignas(64) CUtensorMap map_q;
    if (fused) {
        // the fp32 input as a 2-D tensor: one row of H*W floats per (image, channel); box = 128 pixels x 64 channels
        const unsigned long long HW = (unsigned long long)g.H * g.W;
        // (pixel-major input: one row of C floats per pixel of any image; box = 128 pixels x 32 channels, 128-byte swizzle)
        if (layout == TNNS_NHWC)
            rc = tnns_tensor_map_2d(&map_q, 4, fused->d_x, (unsigned long long)g.C, (unsigned long long)g.N * HW, (unsigned long long)g.C * 4, 32, Q_PIX, 128);
        else
            rc = tnns_tensor_map_2d(&map_q, 4, fused->d_x, HW, (unsigned long long)g.N * g.C, HW * 4, Q_PIX, 64);
        if (rc) return rc;
        a.q_nhwc = layout == TNNS_NHWC;
        a.qx = fused->d_x;
        a.qthr = fused->d_thr;
        a.qimg = reinterpret_cast<uint4*>(const_cast<void*>(d_image));
        a.q_sync = fused_words;
        a.q_self_clean = fused_self_clean;
        a.qN = g.N;
        a.qC = g.C;
        a.q_nbands = (g.H * g.W + Q_PIX - 1) / Q_PIX;
    }
    const int taps = g.Cp == 1 ? 4 : (g.Cp == 2 ? 2 : 1);
    const int bn = tnns_i8_tile_n(w->KN);
    if (pairs == 2 && bn != 256) return tnns_fail(TNNS_ERR_UNSUPPORTED, "block pairs need more than 128 kernels");
    // Block pairs once there are enough 256-row tiles to occupy every SM pair.
    const long long pair_tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((w->KN + bn - 1) / bn);
    const bool use_pairs = bn == 256 && (pairs == 2 || (pairs == 0 && pair_tiles >= ctx->sm_count / 2));
    CUtensorMap map_b;
    if (use_pairs && (rc = encode_weight_map(&map_b, w, bn))) return rc;
    auto go = [&](auto taps_c) -> int {
        constexpr int T = decltype(taps_c)::value;
        if (fused) {
            if (use_pairs) return launch_cfg<256, 1, true, true, 2, T, true>(ctx, a, stream, &map, &map_b, &map_q);
            switch (bn) {
                case 64: return launch_cfg<64, 1, true, true, 1, T, true>(ctx, a, stream, &map, nullptr, &map_q);
                case 128: return launch_cfg<128, 1, true, true, 1, T, true>(ctx, a, stream, &map, nullptr, &map_q);
                default: return launch_cfg<256, 1, true, true, 1, T, true>(ctx, a, stream, &map, nullptr, &map_q);
            }
        }
        if (use_pairs) return launch_cfg<256, 1, true, true, 2, T>(ctx, a, stream, &map, &map_b);
        switch (bn) {
            case 64: return launch_cfg<64, 1, true, true, 1, T>(ctx, a, stream, &map);
            case 128: return launch_cfg<128, 1, true, true, 1, T>(ctx, a, stream, &map);
            default: return launch_cfg<256, 1, true, true, 1, T>(ctx, a, stream, &map);
        }
    };
    if (taps == 4) return go(std::integral_constant<int, 4>());
    if (taps == 2) return go(std::integral_constant<int, 2>());
    return go(std::integral_constant<int, 1>());
}

// Launches the issue-bound MMA loop on every SM; `ops` receives the 2*M*N*K operations it performs.
int tnns_launch_mma_rate(tnns_cuda_ctx* ctx, bool f4, int iters, double* ops, cudaStream_t stream) {
    const size_t smem = 1024 + A_SUB + 256 * KCH;
    auto kern = f4 ? mma_rate_kernel<true> : mma_rate_kernel<false>;
    TNNS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<ctx->sm_count, 128, smem, stream>>>(iters, ctx->d_status);
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    *ops = (double)ctx->sm_count * iters * (KCH / 32) * 2.0 * BM * 256 * (f4 ? 64 : 32);
    return TNNS_OK;
}

int tnns_launch_wait_selftest(tnns_cuda_ctx* ctx, cudaStream_t stream) {
    wait_expiry_selftest_kernel<<<1, 32, 0, stream>>>(ctx->d_status);
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}
