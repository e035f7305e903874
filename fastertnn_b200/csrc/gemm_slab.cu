// Bitwise GEMM + PReLU on the tensor cores for stride-1 layers, fed from a BORDERED 4-bit image: one
// slab of pixels per tile serves every filter tap (reference: mm_tnn / mm_tbn / mm_btn / mm_bnn,
// src/tnns/mm_p2_final_*_avx2.c, on the rows t2r_p2_opt / b2r would have scattered,
// src/tnns/ternarize2row_avx2.c:285-313).
//
// The layer input is stored as e2m1 operands with its padding around every image:
// [n][Hp = H + 2*PH][Wp = W + 2*PW][C/2 bytes], border pixels = the padding value (ternary 0, binary
// +1).  Output rows are laid over that same padded lattice: virtual row q = (n*Hp + y)*Wp + x is the
// window whose top-left corner is padded pixel (y, x); it is a real output pixel (oh, ow) = (y, x)
// when y < OH and x < OW, and is computed but never stored otherwise ((Hp*Wp)/(OH*OW) - 1 more
// MMAs: 13 % at 32x32, 7 % at 56x56).  Filter tap (kh, kw) of 128 consecutive virtual rows then
// reads the 128 consecutive pixels q0 + kh*Wp + kw ..., so ALL taps of a tile are row-shifted views of
// ONE slab of 128 + (KH-1)*Wp + (KW-1) pixels: one tiled tensor copy per tile and 128-byte channel
// group instead of one im2col copy per tap -- 25 KB instead of 144 KB per 512-channel tile at 32x32,
// and one request instead of twelve per 64-channel tile.  The tensor core reads a shifted view by
// starting its shared-memory descriptor at the slab's row kh*Wp + kw: the swizzle pattern is a
// function of the absolute shared-memory address, which the copy engine and the MMA share.
//
// A pixel's bytes per slab row follow the channel count as in the im2col form: 128 bytes (256
// channels; more channels = several slabs per tile, one after the other), 64 or 32 (128 / 64
// channels; 64- / 32-byte swizzle), and a weight stage is the same pre-expanded 128-byte-row image
// (four plane words), so K steps that only exist because rows are padded to four words are skipped.
// Weights that fit the ring entirely are fetched once per block and stay (64-kernel layers).
//
// Roles per block: producer warp (slabs and weight stages), MMA warp, eight epilogue warps; with QF
// four quantiser warps and a publisher as in the im2col form (gemm_tc.cu).  Block pairs
// (tcgen05.mma.cta_group::2) share a 256-row tile, each block with its own slab and half of the
// weight stage.  Every wait is bounded.
#include <algorithm>
#include <type_traits>

#include "gemm_tc_common.cuh"

namespace {

constexpr int SL_MAXSLAB = 4;    // slab buffers at most
constexpr int SL_MAXSTG = 12;    // weight ring depth at most
constexpr int SL_TAPMAX = 4096;  // filter taps at most
constexpr int SL_BAR_BYTES = 512;

struct SlabArgs {
    const unsigned char* Bimg;  // expanded weights [n_tile][stage][BN rows][128 B]
    float* y;
    int Mv;                     // virtual rows: N * Hp * Wp
    int KN, nchunks;            // kernels, weight stages per kernel tile
    int OH, OW, Wp, HpWp;       // output size, padded input lattice
    int KW, T;                  // filter width, taps KH*KW
    int G;                      // 128-byte channel groups per pixel (one slab each); 1 for 64 / 128 channels
    int slab_bytes, copy_rows, ncopies;  // slab buffer size; rows per tensor copy and copies per slab
    int nslab, nstg;            // ring depths
    int b_resident;             // the kernel tile's weight stages all fit the ring: fetched once per block
    int layout, zero_passes, acc_bias;
    float alpha;
    unsigned int* status;
    // optional quantised output for a following layer (instead of y)
    uint32_t* pimg;
    const float* thr_next;
    int next_format;            // 0 binary bit planes, 1 ternary bit planes, 2 plain 4-bit image, 3 bordered 4-bit image
    int next_binary;            // formats 2 / 3: the next layer's activations are binary
    int cp_next;
    int o_Wp, o_Hp, o_PH, o_PW; // format 3: the next image's padded lattice (== this layer's) and its border
    // fused quantisation
    const float* qthr;
    uint4* qimg;
    unsigned int* q_sync;
    int qN, qC, q_nbands, q_H, q_W, q_PH, q_PW, q_binary, q_self_clean, Cp;
    FastDiv div_hpwp, div_wp;
};

template <int BN, int CG, int TAPS, bool QF>
struct SlabCfg {
    static constexpr int RB = 128 / TAPS;             // bytes of a pixel in a slab row
    static constexpr int B_STAGE = (BN / CG) * KCH;   // bytes of a weight stage in one block
    static constexpr bool OVL = BN == 256;            // overlapping accumulator sets (scales leave 480 columns)
    static constexpr int ACC_OFF = OVL ? BN - 32 : BN;
    static constexpr int EPW = 2;                     // epilogue warps per lane quadrant
    static constexpr int WARP_EPI0 = 2, WARP_Q0 = 2 + 4 * EPW;
    // Two separate accumulator sets and single blocks: a second warp issues the MMAs of every other tile, so that one
    // issuer's barrier waits and descriptor arithmetic run under the other's MMAs (see the MMA role).
    static constexpr bool DUAL = !OVL && CG == 1;
    static constexpr int WARP_MMA2 = 2 + 4 * EPW + (QF ? 5 : 0);
    static constexpr int NTHREADS = 32 * (2 + 4 * EPW + (QF ? 5 : 0) + (DUAL ? 1 : 0));
    static constexpr int Q_STAGE = Q_PIX * 64 * 4;
    static constexpr int SMEM_MAX = 232448;
};

template <int BN, int CG, int TAPS, bool QF>
__global__ void __launch_bounds__(SlabCfg<BN, CG, TAPS, QF>::NTHREADS, 1)
gemm_slab_kernel(SlabArgs p, const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_q) {
    using Cfg = SlabCfg<BN, CG, TAPS, QF>;
    constexpr int RB = Cfg::RB, B_STAGE = Cfg::B_STAGE, WARP_EPI0 = Cfg::WARP_EPI0, EPW = Cfg::EPW, ACC_OFF = Cfg::ACC_OFF;
    constexpr bool OVL = Cfg::OVL;
    constexpr int TILE_M = CG * BM;
    // e2m1 A and B (1<<7, 1<<10), ue8m0 scales (1<<23), K-major, N>>3 at bit 17, M>>4 at bit 24
    constexpr uint32_t IDESC = (1u << 23) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((CG * BM) >> 4) << 24);
    constexpr uint32_t SF_COL = 480;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;
    unsigned char* sB = smem + p.nslab * p.slab_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + p.nstg * B_STAGE);
    const uint32_t bar_sfull = smem_u32(bars), bar_sempty = smem_u32(bars + SL_MAXSLAB), bar_bfull = smem_u32(bars + 2 * SL_MAXSLAB),
                   bar_bempty = smem_u32(bars + 2 * SL_MAXSLAB + SL_MAXSTG), bar_tfull = smem_u32(bars + 2 * SL_MAXSLAB + 2 * SL_MAXSTG),
                   bar_tempty = smem_u32(bars + 2 * SL_MAXSLAB + 2 * SL_MAXSTG + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SL_MAXSLAB + 2 * SL_MAXSTG + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    unsigned char* q_ring = reinterpret_cast<unsigned char*>(bars) + SL_BAR_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int ntn = (p.KN + BN - 1) / BN;
    const int ntm = (p.Mv + TILE_M - 1) / TILE_M;
    const int ntiles = ntm * ntn;
    const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
    const int unit = blockIdx.x / CG, nunits = gridDim.x / CG;
    const int SPG = (TAPS == 1) ? p.T : p.nchunks;  // weight stages per slab

    if (tid == 0) {
        for (int s = 0; s < SL_MAXSLAB; s++) {
            mbar_init(bar_sfull + 8 * s, 1);
            mbar_init(bar_sempty + 8 * s, 1);
        }
        for (int s = 0; s < SL_MAXSTG; s++) {
            mbar_init(bar_bfull + 8 * s, 1);
            mbar_init(bar_bempty + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, CG * 4 * EPW);
        }
        if (QF) {
            uint64_t* qbars = reinterpret_cast<uint64_t*>(q_ring + Q_STG * Cfg::Q_STAGE);
            for (int s = 0; s < Q_STG; s++) {
                mbar_init(smem_u32(qbars + s), 1);
                mbar_init(smem_u32(qbars + Q_STG + s), 4);
            }
            volatile QuantCtl* ctl = reinterpret_cast<volatile QuantCtl*>(qbars + 2 * Q_STG);
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
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // unit block scales (ue8m0 0x7F) in columns 480..511, as in the im2col form
    if (warp >= WARP_EPI0 && warp < WARP_EPI0 + 4) {
        const uint32_t one = 0x7F7F7F7Fu;
#pragma unroll 1
        for (uint32_t c = 0; c < 32; c += 8) {
            const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SF_COL + c;
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(one) : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after();

    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == WARP_TMA) {
        if (lane == 0) {
            uint32_t sl = 0, slph = 1, s = 0, ph = 1;
            bool first_tile = true;
            const uint32_t sfull_lead = (CG == 2) ? mapa_shared(bar_sfull, 0) : bar_sfull;
            const uint32_t bfull_lead = (CG == 2) ? mapa_shared(bar_bfull, 0) : bar_bfull;
            const uint32_t copy_bytes = (uint32_t)(p.ncopies * p.copy_rows * RB);
            for (int t = unit; t < ntiles; t += nunits, first_tile = false) {
                const int n_tile = t % ntn;
                const int q0 = (t / ntn) * TILE_M + (int)rank * BM;  // first virtual row = first pixel of the block's slab
                if (QF && q0 < p.Mv) {
                    // the slab reads the images its pixels belong to: wait until the quantiser warps (of any
                    // block) have finished them, border item included
                    const int q_last = min(q0 + p.ncopies * p.copy_rows, p.Mv) - 1;
                    const int n_first = (int)p.div_hpwp.div((uint32_t)q0), n_last = (int)p.div_hpwp.div((uint32_t)q_last);
                    const unsigned int per_image = (unsigned int)(p.q_nbands * p.Cp + 1) * 4u;
                    for (int n = n_first; n <= n_last; n++)
                        if (!counter_wait(p.q_sync + Q_FLAG0 + n, per_image, abort_flag, p.status, 6)) goto done;
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                for (int cg = 0; cg < p.G; cg++) {
                    if (!mbar_wait(bar_sempty + 8 * sl, slph, abort_flag, p.status, 0x11)) goto done;
                    const uint32_t dst = smem_u32(sA + sl * p.slab_bytes);
                    if (CG == 2) {
                        if (rank == 0) mbar_arrive_expect_tx(bar_sfull + 8 * sl, CG * copy_bytes);
                        for (int i = 0; i < p.ncopies; i++)
                            tma_tile2d_g2s_pair(dst + i * p.copy_rows * RB, &tmap_a, cg * KCH, q0 + i * p.copy_rows, sfull_lead + 8 * sl);
                    } else {
                        mbar_arrive_expect_tx(bar_sfull + 8 * sl, copy_bytes);
                        for (int i = 0; i < p.ncopies; i++)
                            tma_tile2d_g2s(dst + i * p.copy_rows * RB, &tmap_a, cg * KCH, q0 + i * p.copy_rows, bar_sfull + 8 * sl);
                    }
                    if (++sl == (uint32_t)p.nslab) { sl = 0; slph ^= 1; }
                    if (p.b_resident && !first_tile) continue;
                    for (int j = 0; j < SPG; j++) {
                        const int c = (TAPS == 1) ? j * p.G + cg : j;
                        const uint32_t slot = p.b_resident ? (uint32_t)c : s;
                        if (!p.b_resident && !mbar_wait(bar_bempty + 8 * slot, ph, abort_flag, p.status, 1)) goto done;
                        if (CG == 2) {
                            if (rank == 0) mbar_arrive_expect_tx(bar_bfull + 8 * slot, CG * B_STAGE);
                            tma_tile2d_g2s_pair(smem_u32(sB + slot * B_STAGE), &tmap_b, 0, (n_tile * p.nchunks + c) * BN + (int)rank * (BN / CG),
                                                bfull_lead + 8 * slot);
                        } else {
                            mbar_arrive_expect_tx(bar_bfull + 8 * slot, B_STAGE);
                            bulk_g2s(smem_u32(sB + slot * B_STAGE), p.Bimg + ((size_t)n_tile * p.nchunks + c) * B_STAGE, B_STAGE, bar_bfull + 8 * slot);
                        }
                        if (!p.b_resident && ++s == (uint32_t)p.nstg) { s = 0; ph ^= 1; }
                    }
                }
            }
        }
    } else if (warp == WARP_MMA || (Cfg::DUAL && warp == Cfg::WARP_MMA2)) {
        if (lane == 0 && rank == 0) {  // pair: the first block issues for both
            // This one thread's instruction stream paces the tensor pipe.  Two things measured on this loop:
            // nothing that touches shared memory may stand between two MMAs (a table look-up per tap, queued
            // behind the MMAs just issued, cost 60 clocks per MMA: tap offsets are running counters), and the
            // MMAs of a tile must sit in ONE divergent region (issued one by one from `if (leader)` branches of
            // a warp-wide loop, every reconvergence waited for the MMA before it: three times slower).
            uint32_t lt = 0, sl = 0, slph = 0, s = 0, ph = 0;
            bool first_tile = true;
            const uint64_t da0 = make_desc_taps(smem_u32(sA), TAPS), db0 = make_desc(smem_u32(sB));
            const uint32_t slab16 = (uint32_t)(p.slab_bytes >> 4);
            const uint32_t row16 = (uint32_t)(p.Wp * (RB / 16));  // one image row further down the slab, in descriptor units
            const uint32_t a_lo0 = (uint32_t)da0, a_hi = (uint32_t)(da0 >> 32), b_lo0 = (uint32_t)db0, b_hi = (uint32_t)(db0 >> 32);
            const uint32_t sfa = tmem_base + SF_COL, sfb = tmem_base + SF_COL + 16;
            const bool fast3x3 = p.T == 9 && p.KW == 3;
            if (warp != WARP_MMA && !fast3x3) goto done;  // the generic loop has one issuer
            if (fast3x3) {
                // 3x3 filters: the nine tap offsets live in registers and every MMA of a slab is issued from straight-line
                // code -- one 32-bit add per operand and MMA.  (The generic loop below spends a dozen dependent
                // instructions between two MMAs; with the epilogue warps competing for the same scheduler that cost
                // 250 clocks per MMA on 64-kernel tiles against 85 for the instruction alone.)
                //
                // Two issuers (DUAL): this thread takes every other tile of the block's sequence -- its accumulator set is
                // always the same one -- and steps its ring positions over the other issuer's tiles.  Measured on
                // 256 x 64x56x56 -> 64 with one issuer: 1560 clocks per tile of which 550 were this thread's two barrier
                // waits with the tensor pipe idle, and 1010 the issue of nine MMAs that execute in 770.
                uint32_t aoff[9];
#pragma unroll
                for (int j = 0; j < 9; j++) aoff[j] = (uint32_t)((j / 3) * p.Wp + (j % 3)) * (RB / 16);
                constexpr int KPT = 4 / TAPS;               // K steps (32 bytes) per tap: 1, 2 or 4
                constexpr int NISSUE = Cfg::DUAL ? 2 : 1;
                const int me = (warp == WARP_MMA) ? 0 : 1;
                const int stages_per_tile = p.G * ((9 * KPT + 3) / 4);
                auto skip_tile = [&]() {  // ring positions over a tile the other issuer takes
                    for (int i = 0; i < p.G; i++)
                        if (++sl == (uint32_t)p.nslab) { sl = 0; slph ^= 1; }
                    if (!p.b_resident)
                        for (int i = 0; i < stages_per_tile; i++)
                            if (++s == (uint32_t)p.nstg) { s = 0; ph ^= 1; }
                };
                if (me == 1) { skip_tile(); lt = 1; }
                for (int t = unit + me * nunits; t < ntiles; t += NISSUE * nunits, lt += NISSUE, first_tile = false) {
                    const int buf = lt & 1;
                    if (!mbar_wait(OVL ? bar_tempty : bar_tempty + 8 * buf, (OVL ? (lt & 1) : ((lt >> 1) & 1)) ^ 1, abort_flag, p.status, 2)) goto done;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * ACC_OFF;
                    uint32_t acc = 0;
                    for (int cg = 0; cg < p.G; cg++) {
                        if (!mbar_wait(bar_sfull + 8 * sl, slph, abort_flag, p.status, 0x13)) goto done;
                        tc_fence_after();
                        const uint32_t slab_lo = a_lo0 + sl * slab16;
                        uint32_t b_lo = 0;
#pragma unroll
                        for (int q = 0; q < 9 * KPT; q++) {   // K step q: tap q / KPT, stage q / 4
                            const int k = q & 3;
                            if (k == 0) {
                                const int j = q >> 2;
                                const int c = (TAPS == 1) ? j * p.G + cg : j;
                                const uint32_t slot = p.b_resident ? (uint32_t)c : s;
                                if (!p.b_resident || first_tile) {
                                    if (!mbar_wait(bar_bfull + 8 * slot, p.b_resident ? 0u : ph, abort_flag, p.status, 3)) goto done;
                                    tc_fence_after();
                                }
                                b_lo = b_lo0 + slot * (uint32_t)(B_STAGE >> 4);
                            }
                            const uint32_t a_lo = slab_lo + aoff[q / KPT] + 2u * (uint32_t)(q % KPT);
                            if (CG == 2) tc_mma_f4_pair_lh(d_tmem, a_lo, a_hi, b_lo + 2u * k, b_hi, IDESC, sfa, sfb, acc);
                            else tc_mma_f4_lh(d_tmem, a_lo, a_hi, b_lo + 2u * k, b_hi, IDESC, sfa, sfb, acc);
                            acc = 1;
                            if ((k == 3 || q == 9 * KPT - 1) && !p.b_resident) {
                                if (CG == 2) tc_commit_pair(bar_bempty + 8 * s); else tc_commit(bar_bempty + 8 * s);
                                if (++s == (uint32_t)p.nstg) { s = 0; ph ^= 1; }
                            }
                        }
                        if (CG == 2) tc_commit_pair(bar_sempty + 8 * sl); else tc_commit(bar_sempty + 8 * sl);
                        if (++sl == (uint32_t)p.nslab) { sl = 0; slph ^= 1; }
                    }
                    if (CG == 2) tc_commit_pair(bar_tfull + 8 * buf); else tc_commit(bar_tfull + 8 * buf);
                    if (NISSUE == 2) skip_tile();
                }
            } else
            for (int t = unit; t < ntiles; t += nunits, lt++, first_tile = false) {
                const int buf = lt & 1;
                if (!mbar_wait(OVL ? bar_tempty : bar_tempty + 8 * buf, (OVL ? (lt & 1) : ((lt >> 1) & 1)) ^ 1, abort_flag, p.status, 2))
                    goto done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * ACC_OFF;
                uint32_t acc = 0;
                for (int cg = 0; cg < p.G; cg++) {
                    if (!mbar_wait(bar_sfull + 8 * sl, slph, abort_flag, p.status, 0x13)) goto done;
                    tc_fence_after();
                    const uint64_t da = da0 + (uint64_t)(sl * slab16);
                    // tap (kh, kw) starts kh*Wp + kw rows into the slab: kept as running counters -- a table in
                    // shared memory would put a load, queued behind the MMAs just issued, in front of every MMA
                    uint32_t kwc = 0, rowoff = 0, tapoff = 0;
                    int tap = 0;
                    for (int j = 0; j < SPG; j++) {
                        const int c = (TAPS == 1) ? j * p.G + cg : j;
                        const uint32_t slot = p.b_resident ? (uint32_t)c : s;
                        if (!p.b_resident || first_tile) {
                            if (!mbar_wait(bar_bfull + 8 * slot, p.b_resident ? 0u : ph, abort_flag, p.status, 3)) goto done;
                            tc_fence_after();
                        }
                        const uint64_t db = db0 + (uint64_t)(slot * (B_STAGE >> 4));
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            // K step k of the stage = 64 elements = 32 bytes of one tap's pixel row
                            const uint32_t koff = (TAPS == 1) ? 2u * k : (TAPS == 2 ? 2u * (k & 1) : 0u);
                            if (TAPS == 1 || tap < p.T) {
                                const uint64_t dak = da + (uint64_t)(tapoff + koff);
                                if (CG == 2) tc_mma_f4_pair(d_tmem, dak, db + 2 * k, IDESC, tmem_base + SF_COL, tmem_base + SF_COL + 16, acc);
                                else tc_mma_f4(d_tmem, dak, db + 2 * k, IDESC, tmem_base + SF_COL, tmem_base + SF_COL + 16, acc);
                                acc = 1;
                            }
                            // the next K step belongs to the next tap: after every step (32-byte pixels), every second
                            // (64-byte pixels) or the stage's last (128-byte pixels)
                            if (TAPS == 4 || (TAPS == 2 && (k & 1)) || (TAPS == 1 && k == 3)) {
                                tap++;
                                if (++kwc == (uint32_t)p.KW) { kwc = 0; rowoff += row16; tapoff = rowoff; }
                                else tapoff += RB / 16;
                            }
                        }
                        if (!p.b_resident) {
                            if (CG == 2) tc_commit_pair(bar_bempty + 8 * s); else tc_commit(bar_bempty + 8 * s);
                            if (++s == (uint32_t)p.nstg) { s = 0; ph ^= 1; }
                        }
                    }
                    if (CG == 2) tc_commit_pair(bar_sempty + 8 * sl); else tc_commit(bar_sempty + 8 * sl);
                    if (++sl == (uint32_t)p.nslab) { sl = 0; slph ^= 1; }
                }
                if (CG == 2) tc_commit_pair(bar_tfull + 8 * buf); else tc_commit(bar_tfull + 8 * buf);
            }
        }
    } else if (QF && warp >= Cfg::WARP_Q0) {
        uint64_t* qbars = reinterpret_cast<uint64_t*>(q_ring + Q_STG * Cfg::Q_STAGE);
        if (warp < Cfg::WARP_Q0 + 4) {
            QuantArgs qa;
            qa.qthr = p.qthr; qa.qimg = p.qimg; qa.q_sync = p.q_sync; qa.qN = p.qN; qa.qC = p.qC; qa.q_nbands = p.q_nbands; qa.Cp = p.Cp;
            qa.HW = p.q_H * p.q_W; qa.status = p.status;
            qa.W = p.q_W; qa.Wp = p.Wp; qa.HpWp = p.HpWp; qa.off0 = p.q_PH * p.Wp + p.q_PW; qa.border = 1; qa.binary = p.q_binary; qa.nhwc = 0;
            quantise_items(qa, &tmap_q, q_ring, qbars, abort_flag, tid - Cfg::WARP_Q0 * 32);
        } else if (lane == 0) {
            publish_items(p.q_sync, p.status, qbars, abort_flag);
        }
    } else if (warp >= WARP_EPI0 && warp < WARP_EPI0 + 4 * EPW) {
        // ---------------- epilogue ----------------
        const int q = warp & 3;                        // tensor-memory lane quadrant this warp may access
        const int ecol = (warp - WARP_EPI0) >> 2;      // which share of the columns
        constexpr int ECOLS = BN / EPW;
        constexpr int NSL = ECOLS / 32;
        const bool alpha_in_unit = p.alpha > 0.f && p.alpha <= 1.f;
        const float bias_f = (float)p.acc_bias;
        const int OHW = p.OH * p.OW;
        uint32_t lt = 0;
        const uint32_t bar_release = (CG == 2 && rank != 0) ? mapa_shared(bar_tempty, 0) : 0u;
        // quantised output with 0 < alpha <= 1: PReLU and the next layer's rule collapse into thresholds on
        // the accumulator (two instructions per output and plane instead of evaluating the PReLU first).
        // Taken on 256-kernel tiles only: on narrower tiles, where the epilogue of one tile runs beside the few
        // MMAs of the next, the shorter but denser instruction stream slowed the tensor pipe more than it
        // saved (256 x 64x56x56 -> 64 with a bordered image out: 60 us against 49).
        const bool next_tern = !p.next_binary && p.next_format != 0;
        const bool by_thr = BN == 256 && p.pimg != nullptr && alpha_in_unit;
        tnns_thr::Pair qt = {0.f, 0.f};
        int qt_img = -1;
        // pixel-major fp32 output: the accumulator is fetched in the 16x256b shape (four lanes = 32 contiguous bytes of a row)
        const bool rows16 = p.pimg == nullptr && p.layout == TNNS_NHWC && (p.KN & 1) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 7) == 0;
        for (int t = unit; t < ntiles; t += nunits, lt++) {
            const int buf = lt & 1;
            const int n0 = (t % ntn) * BN;
            // where this thread's row sits in the lattice, and its image's threshold: worked out while the tile's MMAs run
            const int row = (t / ntn) * TILE_M + (int)rank * BM + q * 32 + lane;  // virtual row
            const bool row_ok = row < p.Mv;
            const int n_img = row_ok ? (int)p.div_hpwp.div((uint32_t)row) : 0;
            const int rem = row - n_img * p.HpWp;
            const int yy = (int)p.div_wp.div((uint32_t)max(rem, 0)), xx = rem - yy * p.Wp;
            const bool valid = row_ok && yy < p.OH && xx < p.OW;   // a real output pixel (oh, ow) = (yy, xx)
            const int opix = yy * p.OW + xx;
            float* ybase = (p.layout == TNNS_NHWC) ? p.y + ((size_t)n_img * OHW + opix) * p.KN : p.y + (size_t)n_img * p.KN * OHW + opix;
            const float tq = (p.pimg && valid) ? __ldg(p.thr_next + n_img) + 0.0f : 0.f;
            if (by_thr && valid && n_img != qt_img) {
                // the next layer's rule as thresholds on the raw accumulator, once per image this thread meets
                qt = tnns_thr::make(tq, p.alpha, bias_f, next_tern);
                qt_img = n_img;
            }
            // rows16: the four rows of the quadrant this thread stores (8*h + lane/4), each mapped to its output pixel
            float* yrow0[4] = {nullptr, nullptr, nullptr, nullptr};
            if (rows16) {
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    const int r = (t / ntn) * TILE_M + (int)rank * BM + q * 32 + 8 * h + (lane >> 2);
                    if (r < p.Mv) {
                        const int ni = (int)p.div_hpwp.div((uint32_t)r);
                        const int rm = r - ni * p.HpWp;
                        const int y2 = (int)p.div_wp.div((uint32_t)rm), x2 = rm - y2 * p.Wp;
                        if (y2 < p.OH && x2 < p.OW) yrow0[h] = p.y + ((size_t)ni * OHW + (size_t)(y2 * p.OW + x2)) * p.KN;
                    }
                }
            }
            if (!mbar_wait(bar_tfull + 8 * buf, (lt >> 1) & 1, abort_flag, p.status, 5)) goto done;
            tc_fence_after();
            int start = 0;
            if (OVL && buf == 0 && ecol == EPW - 1) start = NSL - 1;
#pragma unroll 1
            for (int i = 0; i < NSL; i++) {
                const int cb = ecol * ECOLS + ((i + start) % NSL) * 32;
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * ACC_OFF + cb);
                if (rows16) {
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
                    float f[32];
                    prelu32_f4(v, f, alpha_in_unit, p.acc_bias, bias_f, p.alpha, p.zero_passes);
                    const int c0 = n0 + cb;
                    float* const yrow[4] = {yrow0[0] ? yrow0[0] + c0 : nullptr, yrow0[1] ? yrow0[1] + c0 : nullptr,
                                            yrow0[2] ? yrow0[2] + c0 : nullptr, yrow0[3] ? yrow0[3] + c0 : nullptr};
                    store_rows16_at(f, yrow, p.KN - c0, lane);
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
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2 && rank != 0) mbar_arrive_cluster(bar_release + (OVL ? 0 : 8 * buf));
                        else mbar_arrive(OVL ? bar_tempty : bar_tempty + 8 * buf);
                    }
                }
                const int c0 = n0 + cb;
                if (valid) {
                    float f[32];
                    uint32_t sg = 0, nz = 0;
                    if (by_thr) {
                        if (next_tern) {
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
                    } else
                    // (the run-time choices are taken outside the unrolled loops: left inside, every element pays for
                    // both sides of each -- the epilogue warps share their schedulers with the MMA-issuing threads)
                    if (alpha_in_unit && p.acc_bias) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float a = __uint_as_float(v[j]) + bias_f;
                            f[j] = fmaxf(a, fmaf(a, p.alpha, 0.0f));
                        }
                    } else if (alpha_in_unit) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float a = __uint_as_float(v[j]);
                            f[j] = fmaxf(a, fmaf(a, p.alpha, 0.0f));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float ac = (p.acc_bias ? __uint_as_float(v[j]) + bias_f : __uint_as_float(v[j])) + 0.0f;
                            f[j] = ac * ((p.zero_passes ? ac >= 0.f : ac > 0.f) ? 1.0f : p.alpha);
                        }
                    }
                    const bool full = c0 + 32 <= p.KN;
                    if (p.pimg) {
                        if (c0 < p.cp_next * 64) {
                            const bool tern = next_tern;
                            if (!by_thr) {
                                if (tern) quantise32_ternary(f, tq, sg, nz);
                                else sg = quantise32_binary(f, tq);
                            }
                            const int have = p.KN - c0;
                            const uint32_t vmask = have >= 32 ? 0xFFFFFFFFu : (have > 0 ? (1u << have) - 1u : 0u);
                            if (p.next_format >= 2) {
                                // the 32 channels as 16 bytes of e2m1 operands; channels past KN: ternary 0, binary +1
                                uint32_t w4[4];
                                tnns_expand32_f4(sg & vmask, tern ? ~(nz & vmask) : 0u, w4);
                                size_t px;
                                if (p.next_format == 3) {
                                    int y2 = yy + p.o_PH, x2 = xx + p.o_PW;
                                    px = (size_t)n_img * ((size_t)p.o_Hp * p.o_Wp) + (size_t)y2 * p.o_Wp + x2;
                                } else {
                                    px = (size_t)n_img * OHW + opix;
                                }
                                *(reinterpret_cast<uint4*>(p.pimg) + px * ((size_t)p.cp_next * 2) + (c0 >> 5)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                            } else {
                                const int planes = tern ? 2 : 1;
                                const size_t lanes = (size_t)p.cp_next * 2;
                                uint32_t* px = p.pimg + ((size_t)n_img * planes * OHW + opix) * lanes + (c0 >> 5);
                                px[0] = sg & vmask;
                                if (tern) px[(size_t)OHW * lanes] = ~(nz & vmask);
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
                        float* yc = ybase + (size_t)c0 * OHW;
                        if (full) {
#pragma unroll
                            for (int j = 0; j < 32; j++, yc += OHW) __stcs(yc, f[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++, yc += OHW)
                                if (c0 + j < p.KN) __stcs(yc, f[j]);
                        }
                    }
                } else if (row_ok && p.pimg && p.next_format == 3 && c0 < p.cp_next * 64) {
                    // A virtual row that is no output pixel (yy >= OH or xx >= OW) stands for one border
                    // pixel of the next layer's image, whose padded lattice is this layer's: shifted by the
                    // border and wrapped, the rows that are output pixels cover the interior and these
                    // rows exactly the frame.  They write the padding value, so every launch rewrites the
                    // whole image and nothing has to be cleared beforehand.
                    int y2 = yy + p.o_PH, x2 = xx + p.o_PW;
                    if (y2 >= p.o_Hp) y2 -= p.o_Hp;
                    if (x2 >= p.o_Wp) x2 -= p.o_Wp;
                    const uint32_t padw = p.next_binary ? 0x22222222u : 0u;
                    const size_t px = (size_t)n_img * ((size_t)p.o_Hp * p.o_Wp) + (size_t)y2 * p.o_Wp + x2;
                    *(reinterpret_cast<uint4*>(p.pimg) + px * ((size_t)p.cp_next * 2) + (c0 >> 5)) = make_uint4(padw, padw, padw, padw);
                }
            }
        }
    }

done:
    __syncwarp();
    if (*abort_flag && warp == WARP_TMA && lane == 0) {
        // a wait gave up: give the copies already issued time to land before shared memory is released
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
    tc_fence_before();
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    if (warp == WARP_MMA) {
        tc_fence_after();
        if (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if (QF && p.q_self_clean && warp == WARP_TMA) {
        // the block that leaves last zeroes the synchronisation words for the next launch on the stream
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

template <int BN, int CG, int TAPS, bool QF>
int launch_slab(tnns_cuda_ctx* ctx, const SlabArgs& a, size_t smem, cudaStream_t stream, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b,
                const CUtensorMap* tmap_q) {
    using Cfg = SlabCfg<BN, CG, TAPS, QF>;
    auto kern = gemm_slab_kernel<BN, CG, TAPS, QF>;
    static const CUtensorMap no_map = {};
    static bool smem_set[64] = {false};  // once per kernel and device
    if (!smem_set[ctx->device & 63]) {
        TNNS_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_MAX));
        smem_set[ctx->device & 63] = true;
    }
    const long long tiles = (long long)((a.Mv + CG * BM - 1) / (CG * BM)) * ((a.KN + BN - 1) / BN);
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    nattr++;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(Cfg::NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    if (CG == 1) {
        cfg.gridDim = dim3((int)std::min<long long>(tiles, ctx->sm_count));
    } else {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = CG;
        attr[nattr].val.clusterDim.y = 1;
        attr[nattr].val.clusterDim.z = 1;
        nattr++;
        static int max_pairs[64] = {0};  // per device; measured with the largest shared-memory request
        int& mp = max_pairs[ctx->device & 63];
        if (mp == 0) {
            cfg.gridDim = dim3(CG * (ctx->sm_count / CG));
            cfg.dynamicSmemBytes = Cfg::SMEM_MAX;
            cfg.attrs = attr;
            cfg.numAttrs = nattr;
            int n = 0;
            TNNS_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
            if (n <= 0) return tnns_fail(TNNS_ERR_CUDA, "no block pair of the slab-fed GEMM fits this device");
            mp = std::min(n, ctx->sm_count / CG);
            cfg.dynamicSmemBytes = smem;
        }
        cfg.gridDim = dim3(CG * (int)std::min<long long>(tiles, mp));
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    TNNS_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, a, tmap_a ? *tmap_a : no_map, tmap_b ? *tmap_b : no_map, tmap_q ? *tmap_q : no_map));
    tnns_count_launch();
    TNNS_CUDA_TRY(cudaGetLastError());
    return TNNS_OK;
}

struct SlabPlan {
    int taps, rb, G, T, Wp, Hp, slab_rows, ncopies, copy_rows, slab_bytes, bn;
};

bool make_plan(const tnns_cuda_weights* w, const TnnsGeom& g, SlabPlan* pl) {
    if (!w->d_f4 || w->Kp >= 65536) return false;
    if (g.SH != 1 || g.SW != 1) return false;                      // the virtual lattice is the padded input lattice
    if (g.Cp != 1 && g.Cp != 2 && g.Cp % 4 != 0) return false;     // a pixel = 32, 64 or a multiple of 128 bytes
    pl->taps = g.Cp == 1 ? 4 : (g.Cp == 2 ? 2 : 1);
    pl->rb = 128 / pl->taps;
    pl->G = g.Cp >= 4 ? g.Cp / 4 : 1;
    pl->T = g.KH * g.KW;
    if (pl->T > SL_TAPMAX) return false;
    pl->Wp = g.W + 2 * g.PW;
    pl->Hp = g.H + 2 * g.PH;
    if ((long long)g.N * pl->Hp * pl->Wp >= 0x7FFFFFFFLL - 4096) return false;  // virtual rows are 32-bit
    pl->slab_rows = BM + (g.KH - 1) * pl->Wp + (g.KW - 1);
    pl->ncopies = (pl->slab_rows + 255) / 256;                     // a tensor copy moves at most 256 rows
    if (pl->ncopies > 4) return false;
    // every copy starts on a whole swizzle atom (eight rows) of the slab buffer
    pl->copy_rows = (((pl->slab_rows + pl->ncopies - 1) / pl->ncopies) + 7) & ~7;
    pl->slab_bytes = (pl->ncopies * pl->copy_rows * pl->rb + 1023) & ~1023;
    pl->bn = tnns_i8_tile_n(w->KN);
    return true;
}

// ring depths for a configuration; false when not even two slabs and three weight stages fit
bool ring_depths(const SlabPlan& pl, int b_stage, int fixed, int nchunks, bool one_kernel_tile, int* nslab, int* nstg, int* resident) {
    const int avail = 232448 - fixed;
    int ns = pl.slab_bytes <= 16384 ? 4 : (pl.slab_bytes <= 32768 ? 3 : 2);
    for (; ns >= 2; ns--) {
        const int rest = avail - ns * pl.slab_bytes;
        if (rest < 3 * b_stage) continue;
        int nb = std::min(SL_MAXSTG, rest / b_stage);
        *resident = (one_kernel_tile && nchunks <= nb) ? 1 : 0;
        if (*resident) nb = nchunks;
        *nslab = ns;
        *nstg = nb;
        return true;
    }
    return false;
}

}  // namespace

namespace {
struct SlabChoice {
    SlabPlan pl;
    bool pairs;
    int b_stage, fixed, nslab, nstg, resident, Mv, ntn;
    size_t smem;
};
// The form a launch takes: single blocks or block pairs (pairs_req 0 = by size, 1, 2), ring depths.
bool choose_form(int sm_count, const tnns_cuda_weights* w, const TnnsGeom& g, int pairs_req, bool fused, SlabChoice* ch) {
    if (!make_plan(w, g, &ch->pl)) return false;
    const SlabPlan& pl = ch->pl;
    ch->Mv = g.N * pl.Hp * pl.Wp;
    ch->ntn = (w->KN + pl.bn - 1) / pl.bn;
    const long long pair_tiles = (long long)((ch->Mv + 2 * BM - 1) / (2 * BM)) * ch->ntn;
    if (pairs_req == 2 && pl.bn != 256) return false;
    ch->pairs = pl.bn == 256 && (pairs_req == 2 || (pairs_req == 0 && pair_tiles >= sm_count / 2));
    ch->b_stage = (pl.bn / (ch->pairs ? 2 : 1)) * KCH;
    ch->fixed = 1024 + SL_BAR_BYTES + (fused ? Q_STG * Q_PIX * 64 * 4 + 128 : 0);
    if (!ring_depths(pl, ch->b_stage, ch->fixed, w->Kp / 4, ch->ntn == 1, &ch->nslab, &ch->nstg, &ch->resident)) return false;
    ch->smem = (size_t)ch->fixed + (size_t)ch->nslab * pl.slab_bytes + (size_t)ch->nstg * ch->b_stage;
    return true;
}
}  // namespace

bool tnns_slab_supported(const tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const TnnsGeom& g, bool fused) {
    SlabChoice ch;
    return choose_form(ctx->sm_count, w, g, 0, fused, &ch);
}

size_t tnns_bordered_image_bytes(int N, int C, int H, int W, int PH, int PW) {
    if (N < 0 || C <= 0 || H <= 0 || W <= 0 || PH < 0 || PW < 0) return 0;
    return (size_t)N * (H + 2 * PH) * (W + 2 * PW) * ((C + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS) * 32;
}

int tnns_launch_gemm_slab(tnns_cuda_ctx* ctx, const tnns_cuda_weights* w, const void* d_image, float* d_y, const TnnsGeom& g, float alpha, int layout,
                          cudaStream_t stream, int pairs, void* d_pimg, const float* d_thr_next, int next_format, int next_binary, int next_PH,
                          int next_PW, const TnnsFusedInput* fused) {
    if (g.N == 0) return TNNS_OK;
    SlabChoice ch;
    if (!choose_form(ctx->sm_count, w, g, pairs, fused != nullptr, &ch))
        return tnns_fail(TNNS_ERR_UNSUPPORTED, "layer outside the slab-fed GEMM (stride 1; 64, 128 or 256*k channels; slab and weight ring within shared memory)");
    const SlabPlan& pl = ch.pl;
    if (reinterpret_cast<uintptr_t>(d_image) & 127) return tnns_fail(TNNS_ERR_INVALID, "bordered image must be 128-byte aligned");
    const bool act_binary = w->type == BTN || w->type == BNN;
    const int Mv = ch.Mv;
    const bool use_pairs = ch.pairs;
    const size_t smem = ch.smem;
    SlabArgs a = {};
    a.nslab = ch.nslab; a.nstg = ch.nstg; a.b_resident = ch.resident;
    a.Bimg = reinterpret_cast<const unsigned char*>(w->d_f4);
    a.y = d_y;
    a.Mv = Mv;
    a.KN = w->KN;
    a.nchunks = w->Kp / 4;
    a.OH = g.OH; a.OW = g.OW; a.Wp = pl.Wp; a.HpWp = pl.Hp * pl.Wp;
    a.KW = g.KW; a.T = pl.T; a.G = pl.G;
    a.slab_bytes = pl.slab_bytes; a.copy_rows = pl.copy_rows; a.ncopies = pl.ncopies;
    a.layout = (g.OH * g.OW == 1) ? TNNS_NHWC : layout;  // one pixel per image: both layouts are the same memory, the pixel-major epilogue stores 16 bytes per lane
    a.zero_passes = w->type != TNN;
    // BNN counts its products: pad words are never multiplied here, absent channels (+1 x +1) are
    a.acc_bias = (w->type == BNN) ? w->K_unpack - 64 * w->Kw : 0;
    a.alpha = alpha;
    a.status = ctx->d_status;
    a.pimg = reinterpret_cast<uint32_t*>(d_pimg);
    a.thr_next = d_thr_next;
    a.next_format = next_format;
    a.next_binary = next_binary;
    a.cp_next = (w->KN + TNNS_WORD_BITS - 1) / TNNS_WORD_BITS;
    a.o_PH = next_PH; a.o_PW = next_PW; a.o_Hp = g.OH + 2 * next_PH; a.o_Wp = g.OW + 2 * next_PW;
    if (d_pimg && next_format == 3 && (a.o_Hp != pl.Hp || a.o_Wp != pl.Wp))
        return tnns_fail(TNNS_ERR_UNSUPPORTED, "a bordered output image needs the next layer's padded size (%d x %d) to equal this layer's (%d x %d)",
                         a.o_Hp, a.o_Wp, pl.Hp, pl.Wp);
    a.Cp = g.Cp;
    a.div_hpwp = tnns_fastdiv((uint32_t)a.HpWp);
    a.div_wp = tnns_fastdiv((uint32_t)pl.Wp);
    // the bordered image as rows of pixels: (bytes of a pixel) x (all padded pixels of the batch)
    alignas(64) CUtensorMap map_a, map_b, map_q;
    int rc = tnns_tensor_map_2d(&map_a, 1, d_image, (unsigned long long)g.Cp * 32, (unsigned long long)Mv, (unsigned long long)g.Cp * 32, pl.rb,
                                pl.copy_rows, pl.rb);
    if (rc) return rc;
    if (use_pairs && (rc = tnns_tensor_map_2d(&map_b, 1, w->d_f4, KCH, w->f4_bytes / KCH, KCH, KCH, pl.bn / 2))) return rc;
    if (fused) {
        if (!fused->d_x || !fused->d_thr || !fused->d_sync) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
        if (!tnns_quantise_tma_supported(fused->d_x, g.H, g.W, layout))
            return tnns_fail(TNNS_ERR_UNSUPPORTED, "fused quantisation needs NCHW input with H*W a multiple of four and a 16-byte aligned base");
        const unsigned long long HW = (unsigned long long)g.H * g.W;
        if ((rc = tnns_tensor_map_2d(&map_q, 4, fused->d_x, HW, (unsigned long long)g.N * g.C, HW * 4, Q_PIX, 64))) return rc;
        unsigned int* words = nullptr;
        int self_clean = 0;
        if ((rc = tnns_fused_sync_prepare(ctx, g.N, stream, fused->d_sync, &words, &self_clean))) return rc;
        a.qthr = fused->d_thr;
        a.qimg = reinterpret_cast<uint4*>(const_cast<void*>(d_image));
        a.q_sync = words;
        a.q_self_clean = self_clean;
        a.qN = g.N; a.qC = g.C; a.q_H = g.H; a.q_W = g.W; a.q_PH = g.PH; a.q_PW = g.PW;
        a.q_nbands = (g.H * g.W + Q_PIX - 1) / Q_PIX;
        a.q_binary = act_binary ? 1 : 0;
    }
    auto go = [&](auto taps_c) -> int {
        constexpr int T = decltype(taps_c)::value;
        if (fused) {
            if (use_pairs) return launch_slab<256, 2, T, true>(ctx, a, smem, stream, &map_a, &map_b, &map_q);
            switch (pl.bn) {
                case 64: return launch_slab<64, 1, T, true>(ctx, a, smem, stream, &map_a, nullptr, &map_q);
                case 128: return launch_slab<128, 1, T, true>(ctx, a, smem, stream, &map_a, nullptr, &map_q);
                default: return launch_slab<256, 1, T, true>(ctx, a, smem, stream, &map_a, nullptr, &map_q);
            }
        }
        if (use_pairs) return launch_slab<256, 2, T, false>(ctx, a, smem, stream, &map_a, &map_b, nullptr);
        switch (pl.bn) {
            case 64: return launch_slab<64, 1, T, false>(ctx, a, smem, stream, &map_a, nullptr, nullptr);
            case 128: return launch_slab<128, 1, T, false>(ctx, a, smem, stream, &map_a, nullptr, nullptr);
            default: return launch_slab<256, 1, T, false>(ctx, a, smem, stream, &map_a, nullptr, nullptr);
        }
    };
    if (pl.taps == 4) return go(std::integral_constant<int, 4>());
    if (pl.taps == 2) return go(std::integral_constant<int, 2>());
    return go(std::integral_constant<int, 1>());
}
