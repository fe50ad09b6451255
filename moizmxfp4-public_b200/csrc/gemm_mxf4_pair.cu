// quant_matmul for large M on CTA pairs: tcgen05.mma.cta_group::2 (one instruction spans two SMs).
//
// Same arithmetic, operand formats and pipeline roles as gemm_mxf4.cu.  Here two CTAs of a cluster work on one
// 256 (weight rows) x BN (activation rows) tile of out^T: each CTA holds its own 128 weight rows and HALF of the
// activation tile in shared memory, and the tensor cores of both SMs read both halves.  Per accumulator column
// each SM therefore reads half as many activation bytes from its shared memory as the one-CTA kernel does, which
// is what bounds that kernel in EXACT mode.
//
// CTA 0 of the pair (the leader) issues every tcgen05.mma and tcgen05.commit; the instructions execute in both SMs,
// each on its own shared and tensor memory at the same addresses, so both CTAs keep identical layouts.  Completion
// (stage free, correction tile free, scale columns free, accumulator full) is multicast to the same barrier in both CTAs.
//
// What differs from the one-CTA kernel, each point measured:
//  * Scale factors do not pass through shared memory or tcgen05.cp.  A tcgen05.cp sits in the same in-order pipe as
//    the MMAs and cost over a hundred cycles each here; four warps per CTA (one per tensor-memory lane quarter) load
//    the prepared scale tiles from global memory one stage ahead and write them with tcgen05.st into a ring of column
//    sets that is deeper than the operand pipeline.
//  * The operand tiles of BOTH CTAs complete their bytes on the leader's barrier (TMA with .cta_group::2), so the MMA
//    thread learns of the peer's tiles without any thread of the peer in between.
//  * What threads of the peer do produce per stage (scales written, correction tile built) and per tile (accumulator
//    drained) reaches the leader as remote mbarrier arrives with CTA-scope release.  With cluster-scope release each
//    arrive cost the sender a fence of more than a thousand cycles and the kernel ran 40 % slower.
//  * One 256-column accumulator fills half of tensor memory and the scale ring the other half, so the epilogue cannot
//    overlap the next tile.  Eight warps therefore drain the accumulator into registers (as bf16 pairs) first, hand it
//    back, and only then transpose through shared memory and store, as TMA tile stores when the output is aligned.
// Every wait is bounded as in the one-CTA kernel; both CTAs meet at a cluster barrier before they exit, so no
// remote arrival can target a CTA that has gone.
#include <atomic>
#include "gemm_mxf4_tc.cuh"

namespace mxfp4 {
namespace {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
// Arrive on a barrier of the other CTA.  Default semantics (release at CTA scope), as is customary for signalling
// inside a cluster: a release at cluster scope costs the arriving thread a fence of well over a thousand cycles, which
// put every report of the peer CTA on the critical path.  What the reports order is already complete when they are
// sent: tensor-memory stores after tcgen05.wait::st, shared-memory writes after fence.proxy.async.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// per-stage report of the peer CTA to the leader's ready barrier
__device__ __forceinline__ void mbar_report_remote(uint32_t cluster_addr) {
    mbar_arrive_remote(cluster_addr);
}
// bounded wait on a barrier that the other CTA of the pair may signal (a local barrier all the same)
__device__ __forceinline__ bool mbar_wait_cl(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return mbar_wait(bar, parity, abort_flag);
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {     // arrives on the same barrier of both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc2_mma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// TMA tile load whose completion bytes go to a barrier of either CTA of the pair (a shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
                 : "memory");
}
// instruction descriptor as make_idesc, with M = 256 (128 rows in each CTA)
__device__ __forceinline__ uint32_t make_idesc_pair(int n, uint32_t sf_id) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(256 >> 4) << 24) | (sf_id << 29) | (sf_id << 4);
}

// warps: 0 TMA producer, 1 and kMma2Warp MMA issuers (leader CTA), 2-5 scale-factor writers (one per tensor-memory lane
// quarter), 6-9 and kEpi2Warp.. epilogue (two warps per lane quarter, half of the columns each), 10..10+kTransformWarps-1
// correction transform (EXACT mode)
// Measured on the 8192 x 11008 x 4096 problem, sustained: the second MMA issuer on warp 18 instead of warp 15 (another
// warp scheduler than before: the two issuers and the producer now sit on three different schedulers) +2.5 %; 4
// transform warps instead of 8 -1 %; 16 epilogue warps (64 columns each) -2 % at equal ring depths; two correction tiles
// instead of three -3.5 %, four tiles with four operand slots instead of three with five +3 % (kept), five or six tiles
// with four or three slots -1.5 % / -4 %; 32-column tensor-memory loads in the epilogue -1 % (spills); a suspend-time
// hint on mbarrier.try_wait (fewer polling instructions) -1 %.
constexpr int kTransformWarps = 8;
constexpr int kEpiWarps = 8;                         // two per lane quarter
constexpr int kEpiGroups = kEpiWarps / 4;            // column groups of the accumulator, one warp per lane quarter each
constexpr int kMma2Warp = 10 + kTransformWarps;
constexpr int kEpi2Warp = kMma2Warp + 1;
constexpr int kPairThreads = (kEpi2Warp + kEpiWarps - 4) * 32;
static_assert(kEpiWarps == 8 || kEpiWarps == 16, "epilogue warps");
static_assert(kTransformWarps == 4 || kTransformWarps == 8, "transform warps");
static_assert((kEpi2Warp & 3) != ((kEpi2Warp + 1) & 3), "lane quarters");

// 32 lanes x 32 bits, N consecutive columns, registers -> tensor memory
__device__ __forceinline__ void tc_st_x16(uint32_t taddr, const uint4& a, const uint4& b, const uint4& c, const uint4& d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(a.x),
                 "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w), "r"(c.x), "r"(c.y), "r"(c.z), "r"(c.w), "r"(d.x), "r"(d.y),
                 "r"(d.z), "r"(d.w)
                 : "memory");
}
__device__ __forceinline__ void tc_st_x8(uint32_t taddr, const uint4& a, const uint4& b) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// 32 lanes x 16 columns, loaded and waited for
__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                   "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]),
                      "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]));
}

template <int BN>
struct PairCfg {
    static constexpr int kHalf = BN / 2;                           // activation rows each CTA stages
    static constexpr int kXT = BN <= 128 ? 1 : 2;                  // 128-row groups of activation scales a tile can touch
    static constexpr int kWBytes = kTileW * kStageKBytes;          // 16 KB
    static constexpr int kXBytes = kHalf * kStageKBytes;
    static constexpr int kOffX = kWBytes;
    static constexpr int kStageBytes = kWBytes + kXBytes;          // a pipeline slot holds the two operand tiles only
    static constexpr int kCorrBufs = 4;                            // ring of correction tiles (EXACT mode)
    static constexpr int kCorrBytes = kCorrBufs * kWBytes;
    static constexpr int kEpiBytes = kEpiWarps * 2048;             // per epilogue warp: 32 x 32 bf16 for the transpose
    static constexpr int kEpiCols = BN / kEpiGroups;               // accumulator columns one epilogue warp drains
    static constexpr int kAccBufs = BN <= 192 ? 2 : 1;
    static constexpr int kAccStride = BN <= 128 ? 128 : (BN <= 192 ? 192 : 256);
    // tensor memory: the accumulators, then a ring of scale-factor column sets
    static constexpr int kColSf = kAccBufs * kAccStride;
    static constexpr int kSfSetCols = 32;
    static constexpr int kColSfw = kColSf;         // 2 K-tiles x 4 columns (pass 1)
    static constexpr int kColSfw2 = kColSf + 8;    // same for pass 2
    static constexpr int kColSfx = kColSf + 16;    // 2 K-tiles x 4*kXT columns
    static constexpr int kBudget = 227 * 1024 - 1024 - 1024 - kEpiBytes - kCorrBytes;
    static constexpr int kBySmem = kBudget / kStageBytes;
    // four operand slots and four correction tiles: measured 3 % faster than five slots and three tiles (same shared memory)
    static constexpr int kStages = kBySmem < 4 ? kBySmem : 4;
    static constexpr int kByTmem = (512 - kColSf) / kSfSetCols;
    static constexpr int kSfSets = kByTmem < 8 ? kByTmem : 8;      // a deeper ring than the operand pipeline: the peer's reports get a head start
    static constexpr int kSmemBytes = kStages * kStageBytes + kCorrBytes + kEpiBytes + 1024 + 1024;
    static constexpr uint32_t kTxBytes = kWBytes + kXBytes;
    static constexpr int kSfRegs = 4 + 2 * kXT;    // 128-bit words of scale factors a thread moves per stage
    static constexpr int kTmemCols = 512;
    static_assert(BN % 32 == 0 && BN <= 256 && kHalf % 8 == 0 && (BN / kEpiGroups) % 32 == 0, "tile width");
    static_assert(kStages >= 2 && kSfSets >= 2 && 16 + 8 * kXT <= kSfSetCols && kStageBytes % 1024 == 0, "pipeline depth / tensor memory");
};

// Work units of the pair kernel: (pair of weight tiles, activation tile); no K split (large M only).
struct PairUnit {
    int n_pair, m_tile;
};
__device__ __forceinline__ PairUnit get_pair_unit(const GemmParams& p, int n_pairs, int u) {
    PairUnit w;
    w.n_pair = u % n_pairs;
    w.m_tile = u / n_pairs;
    return w;
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    gemm_mxf4_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
    using C = PairCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t corr_base = base + C::kStages * C::kStageBytes;
    uint8_t* corr_ptr = base_ptr + C::kStages * C::kStageBytes;
    uint8_t* epi_ptr = corr_ptr + C::kCorrBytes;
    const uint32_t bars = corr_base + C::kCorrBytes + C::kEpiBytes;
    // in every CTA, signalled locally or by the leader's multicast commits
    auto full_bar = [&](int s) { return bars + 8u * s; };                        // EXACT mode: this CTA's weight tile has landed (the transform waits for it)
    auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };        // MMAs have finished with the stage (both CTAs)
    // used in the leader only; the peer's arrivals come in remotely
    auto ready_bar = [&](int s) { return bars + 8u * (3 * C::kStages + s); };    // EXACT mode: both CTAs have built their correction tiles
    auto tiles_bar = [&](int s) { return bars + 8u * (2 * C::kStages + s); };    // TMA bytes of BOTH CTAs: activation halves, in FAST mode also the weight tiles
    auto sfe_bar = [&](int k) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 6 + k); };   // in every CTA: MMAs have finished with scale column set k
    auto corr_empty_bar = [&](int c) { return bars + 8u * (5 * C::kStages + c); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 2 + b); };   // leader: 8 epilogue warps of the pair
    auto unit_started_bar = [&](int i) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 4 + (i & 1)); };
    auto sfr_bar = [&](int k) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 6 + C::kSfSets + k); };   // leader: both CTAs have written set k
    uint8_t* tail = epi_ptr + C::kEpiBytes + 8 * (5 * C::kStages + C::kCorrBufs + 6 + 2 * C::kSfSets);
    static_assert(8 * (5 * C::kStages + C::kCorrBufs + 6 + 2 * C::kSfSets) + 8 <= 1024, "barrier area");
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;
    const int n_pairs = (p.n_tiles + 1) / 2;
    const int total_units = n_pairs * p.m_tiles;
    const int first_unit = blockIdx.x >> 1, unit_step = gridDim.x >> 1;

    if (threadIdx.x == 64) {
        // fetch the TMA descriptors now: the first loads and stores would otherwise pay for it
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        if (p.tma_store) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(tiles_bar(s), 1);
            mbar_init(ready_bar(s), 2 * kTransformWarps);   // the transform warps of both CTAs
        }
        for (int c = 0; c < C::kCorrBufs; ++c) mbar_init(corr_empty_bar(c), 1);
        for (int k = 0; k < C::kSfSets; ++k) {
            mbar_init(sfe_bar(k), 1);
            mbar_init(sfr_bar(k), 8);             // 4 + 4 scale-factor warps
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 2);        // both MMA issuers commit (multicast to both CTAs)
            mbar_init(acc_empty_bar(b), 2 * kEpiWarps);      // the epilogue warps of both CTAs
        }
        mbar_init(unit_started_bar(0), 1);
        mbar_init(unit_started_bar(1), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        // each CTA takes all 512 columns of its own SM, so both allocations start at the same address
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(C::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                               // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (each CTA loads its own tiles)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const uint32_t tiles0 = map_to_cta(tiles_bar(0), 0);
            // launched behind the activation quantiser with programmatic stream serialisation: everything up to here
            // (barriers, tensor memory, descriptors) overlapped its tail; its results are needed from here on
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int u = first_unit; u < total_units && ok; u += unit_step) {
                const PairUnit w = get_pair_unit(p, n_pairs, u);
                const int m0 = w.m_tile * BN;
                const int n_tile = w.n_pair * 2 + (int)rank;
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!mbar_wait_cl(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t st = base + s * C::kStageBytes;
                    // The leader's barrier counts the bytes of both CTAs (its own expect_tx may come after the peer's
                    // bytes: the count goes negative for a moment, the phase cannot complete before the arrive).
                    const uint32_t tb = tiles0 + 8u * s;
                    if (p.exact) {
                        if (leader) mbar_expect_tx(tiles_bar(s), 2 * C::kXBytes);
                        mbar_expect_tx(full_bar(s), C::kWBytes);
                        tma_load_2d(st, &map_w, full_bar(s), ks * kStageKBytes, n_tile * kTileW);
                    } else {
                        if (leader) mbar_expect_tx(tiles_bar(s), 2 * C::kTxBytes);
                        tma_load_2d_pair(st, &map_w, tb, ks * kStageKBytes, n_tile * kTileW);
                    }
                    tma_load_2d_pair(st + C::kOffX, &map_x, tb, ks * kStageKBytes, m0 + (int)rank * C::kHalf);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == kMma2Warp) {
        // ------------------------------------------------------------------ MMA issuers (leader CTA only), alternate stages
        if (leader && lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            const uint32_t idesc0 = make_idesc_pair(BN, 0), idesc2 = make_idesc_pair(BN, 2);
            uint32_t it = 0;
            int i = 0;
            bool ok = true;
            for (int u = first_unit; u < total_units && ok; u += unit_step, ++i) {
                const PairUnit w = get_pair_unit(p, n_pairs, u);
                const int buf = i % C::kAccBufs;
                const uint32_t acc_ph = (i / C::kAccBufs) & 1;
                const uint32_t acc = tmem + buf * C::kAccStride;
                const uint32_t sfx_off = ((w.m_tile * BN) % 128) / 32;
                ok = mbar_wait_cl(acc_empty_bar(buf), acc_ph ^ 1u, abort_flag);   // both CTAs' epilogues have drained this buffer
                if (!ok) break;
                tc_fence_after();
                bool order_ok = ((it & 1u) == me);
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    if ((it & 1u) != me) continue;
                    if (!order_ok) {
                        ok = mbar_wait(unit_started_bar(i), ((uint32_t)i >> 1) & 1u, abort_flag);
                        if (!ok) break;
                        order_ok = true;
                    }
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    ok = mbar_wait_cl(tiles_bar(s), ph, abort_flag);
                    ok = ok && mbar_wait_cl(sfr_bar(it % C::kSfSets), (it / C::kSfSets) & 1, abort_flag);
                    ok = ok && (!p.exact || mbar_wait_cl(ready_bar(s), ph, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = base + s * C::kStageBytes;
                    const uint32_t sft = tmem + (it % C::kSfSets) * C::kSfSetCols;       // this stage's scale-factor columns
                    const uint32_t sfx_col = sft + C::kColSfx + sfx_off;
                    const int cb = it % C::kCorrBufs;
                    const uint64_t wdesc = desc_sw128(st), cdesc = desc_sw128(corr_base + cb * C::kWBytes), xdesc = desc_sw128(st + C::kOffX);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const int g = kb >> 1;
                        const uint32_t idesc = (kb & 1) ? idesc2 : idesc0;
                        const uint64_t adv = (uint64_t)(kb * 32 >> 4);
                        const uint32_t sfb = sfx_col + 4 * C::kXT * g;
                        tc2_mma_mxf4(acc, wdesc + adv, xdesc + adv, idesc, sft + C::kColSfw + 4 * g, sfb, (ks > 0 || kb > 0) ? 1u : 0u);
                        if (ks == 0 && kb == 0) mbar_arrive(unit_started_bar(i));
                        if (p.exact) tc2_mma_mxf4(acc, cdesc + adv, xdesc + adv, idesc, sft + C::kColSfw2 + 4 * g, sfb, 1u);
                    }
                    tc2_commit_both(empty_bar(s));
                    tc2_commit_both(sfe_bar(it % C::kSfSets));
                    if (p.exact) tc2_commit_both(corr_empty_bar(cb));
                }
                tc2_commit_both(acc_full_bar(buf));
            }
        }
        __syncwarp();
    } else if (warp >= 10 && warp < kMma2Warp) {
        // ------------------------------------------------------------------ correction transform (EXACT mode)
        if (p.exact) {
            constexpr int kTT = kTransformWarps * 32;                             // transform threads
            const int t = (warp - 10) * 32 + lane;
            uint32_t it = 0;
            bool ok = true;
            for (int u = first_unit; u < total_units && ok; u += unit_step) {
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    const int cb = it % C::kCorrBufs;
                    const uint32_t cph = (it / C::kCorrBufs) & 1;
                    ok = __all_sync(0xFFFFFFFFu, mbar_wait_cl(corr_empty_bar(cb), cph ^ 1u, abort_flag) && mbar_wait(full_bar(s), ph, abort_flag));
                    if (!ok) break;
                    const uint4* src = reinterpret_cast<const uint4*>(base_ptr + s * C::kStageBytes);
                    uint4* dst = reinterpret_cast<uint4*>(corr_ptr + cb * C::kWBytes);
                    uint4 v[C::kWBytes / 16 / kTT];
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / kTT; ++j) v[j] = src[j * kTT + t];
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / kTT; ++j) {
                        v[j].x = corr_word(v[j].x); v[j].y = corr_word(v[j].y); v[j].z = corr_word(v[j].z); v[j].w = corr_word(v[j].w);
                    }
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / kTT; ++j) dst[j * kTT + t] = v[j];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(ready_bar(s));
                        else mbar_report_remote(map_to_cta(ready_bar(s), 0));
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ scale factors: global -> registers -> tensor memory
        // tcgen05.cp would put these copies into the same in-order pipe as the MMAs, where each one costs more than
        // a hundred cycles.  Four warps (one per lane quarter: the layout wants the 32 rows of a scale tile
        // replicated in all four) load the prepared tiles straight from global memory, one stage ahead, and write
        // them with tcgen05.st, beside the MMAs and independent of the operand pipeline.  Thread l owns row l of
        // every 32 x 16-byte scale tile: one 128-bit load per tile, four columns of its lane.
        {
            const uint32_t lane_base = ((uint32_t)(warp & 3) * 32u) << 16;
            const uint32_t sfr0 = leader ? 0u : map_to_cta(sfr_bar(0), 0);
            const int64_t m_groups_end = ((int64_t)p.M + 127) / 128 * 128;
            auto load_sf = [&](int u, int ks, uint4 (&r)[C::kSfRegs]) {
                const PairUnit w = get_pair_unit(p, n_pairs, u);
                const int n_tile = w.n_pair * 2 + (int)rank;
                const int sf_tile = n_tile < p.n_tiles ? n_tile : p.n_tiles - 1;     // a tile past the end reads a valid one; nothing of it is stored
                const uint8_t* wp = p.sfw + ((int64_t)sf_tile * p.kstages + ks) * 2048 + lane * 16;
#pragma unroll
                for (int j = 0; j < 4; ++j) r[j] = __ldg(reinterpret_cast<const uint4*>(wp + 512 * j));      // pass 1: K halves 0, 1; pass 2: K halves 0, 1
                const int m0 = w.m_tile * BN;
#pragma unroll
                for (int t = 0; t < C::kXT; ++t) {
                    int64_t grp = m0 / 128 + t;
                    if (grp * 128 >= m_groups_end) grp = m0 / 128;      // a group past the end: its rows are beyond M and never stored
                    const uint8_t* xp = p.sfx + (grp * p.kstages + ks) * 1024 + lane * 16;
#pragma unroll
                    for (int g = 0; g < 2; ++g) r[4 + C::kXT * g + t] = __ldg(reinterpret_cast<const uint4*>(xp + 512 * g));   // column order: K half, then group
                }
            };
            uint4 cur[C::kSfRegs], nxt[C::kSfRegs];
            if (p.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");     // the activation scales come from the kernel in front
            if (first_unit < total_units) load_sf(first_unit, 0, cur);
            uint32_t it = 0;
            bool ok = true;
            for (int u = first_unit; u < total_units && ok; u += unit_step) {
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    // the MMAs that read this column set (kSfSets stages ago) must have completed
                    ok = __all_sync(0xFFFFFFFFu, mbar_wait_cl(sfe_bar(it % C::kSfSets), ((it / C::kSfSets) & 1) ^ 1u, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sft = tmem + lane_base + (it % C::kSfSets) * C::kSfSetCols;
                    tc_st_x16(sft + C::kColSfw, cur[0], cur[1], cur[2], cur[3]);
                    if constexpr (C::kXT == 2) tc_st_x16(sft + C::kColSfx, cur[4], cur[5], cur[6], cur[7]);
                    else tc_st_x8(sft + C::kColSfx, cur[4], cur[5]);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        const int k = it % C::kSfSets;
                        if (leader) mbar_arrive(sfr_bar(k));
                        else mbar_report_remote(sfr0 + 8u * k);
                    }
                    // Fetch the next stage's scales only now: a release-arrive waits for the thread's outstanding
                    // loads, so a prefetch issued before it would delay the report by a trip to L2.  The loads
                    // complete while this warp waits for the next column set to become free.
                    int nu = u, nks = ks + 1;
                    if (nks == p.kstages) { nks = 0; nu = u + unit_step; }
                    if (nu < total_units) load_sf(nu, nks, nxt);
#pragma unroll
                    for (int j = 0; j < C::kSfRegs; ++j) cur[j] = nxt[j];
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (each CTA stores its own 128 weight rows)
        // Eight warps: lane quarter q = warp % 4 (the quarter a warp may read), column half h.  The tensor-memory load
        // of the next 32-column block is in flight while the current one is converted, transposed through shared memory
        // (so that 32 consecutive n of a row go out as 16-byte stores) and stored.
        const int e = warp < 10 ? warp - 6 : 4 + warp - kEpi2Warp;       // 0..kEpiWarps-1
        const int q = warp & 3;
        const int h = e >> 2;                                            // column group
        __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(epi_ptr + e * 2048);
        const bool has_bias = p.bias != nullptr;
        const bool vec_ok = (p.ldo % 8 == 0) && (((uintptr_t)p.out) % 16 == 0);
        int i = 0;
        bool ok = true;
        for (int u = first_unit; u < total_units && ok; u += unit_step, ++i) {
            const PairUnit w = get_pair_unit(p, n_pairs, u);
            const int buf = i % C::kAccBufs;
            ok = mbar_wait_cl(acc_full_bar(buf), (i / C::kAccBufs) & 1, abort_flag);
            ok = __all_sync(0xFFFFFFFFu, ok && !*abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int n0 = (w.n_pair * 2 + (int)rank) * kTileW + q * 32;
            const int n = n0 + lane;
            const float bias = (has_bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
            const bool vec = vec_ok && (n0 + 32 <= p.N);
            const int mbeg = w.m_tile * BN + h * C::kEpiCols;               // first activation row of this warp's columns
            const int rows_left = p.M - mbeg;
            const int nchunk = rows_left <= 0 ? 0 : (rows_left >= C::kEpiCols ? C::kEpiCols / 32 : (rows_left + 31) / 32);
            const uint32_t taddr0 = tmem + buf * C::kAccStride + ((uint32_t)(q * 32) << 16) + h * C::kEpiCols;
            auto release = [&]() {                                           // every load of this warp has completed
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(acc_empty_bar(buf));
                    else mbar_arrive_remote(map_to_cta(acc_empty_bar(buf), 0));
                }
            };
            // Phase 1: the warp's BN/2 columns leave tensor memory 16 at a time and stay in registers as bf16 pairs
            // (m, m+1); the accumulator is handed back as soon as the last load has completed.
            constexpr int kBlocks = C::kEpiCols / 32;              // 32-column blocks per warp
            uint32_t pk[kBlocks * 16];
#pragma unroll
            for (int c = 0; c < kBlocks * 2; ++c) {
                if (c * 16 < nchunk * 32) {                        // warp-uniform
                    uint32_t v[16];
                    tc_ld_32x16(taddr0 + c * 16, v);
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        if (has_bias) {
                            // `output += bias` in bf16: round the product, add, round again
                            const float a = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j]))) + bias;
                            const float b = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j + 1]))) + bias;
                            const __nv_bfloat162 y = __floats2bfloat162_rn(a, b);
                            pk[c * 8 + (j >> 1)] = *reinterpret_cast<const uint32_t*>(&y);
                        } else {
                            const __nv_bfloat162 y = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                            pk[c * 8 + (j >> 1)] = *reinterpret_cast<const uint32_t*>(&y);
                        }
                    }
                }
            }
            release();
            // Phase 2: block by block through the warp's 32 x 32 staging tile (transpose: 32 consecutive n per row) and out
            unsigned short* t16u = reinterpret_cast<unsigned short*>(t16);
#pragma unroll
            for (int c = 0; c < kBlocks; ++c) {
                if (c < nchunk) {
                    const int m0 = mbeg + c * 32;
                    if (p.tma_store) {
                        // the previous tile must have been read out of shared memory before it is overwritten
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        __syncwarp();
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint32_t w2 = pk[c * 16 + j];
                        t16u[(2 * j) * 32 + lane] = (unsigned short)(w2 & 0xFFFFu);
                        t16u[(2 * j + 1) * 32 + lane] = (unsigned short)(w2 >> 16);
                    }
                    if (p.tma_store) {
                        // the 32 (m) x 32 (n) bf16 tile leaves as one TMA store; rows and columns past M, N are clipped
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0 && n0 < p.N) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_out), "r"(smem_u32(t16)),
                                         "r"(n0), "r"(m0)
                                         : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    } else {
                        __syncwarp();
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            const int row = r * 8 + (lane >> 2), seg = lane & 3;
                            const int m = m0 + row;
                            if (m < p.M) {
                                if (vec) {
                                    *reinterpret_cast<uint4*>(p.out + (int64_t)m * p.ldo + n0 + seg * 8) = *reinterpret_cast<const uint4*>(t16 + row * 32 + seg * 8);
                                } else {
                                    for (int x = 0; x < 8; ++x)
                                        if (n0 + seg * 8 + x < p.N) p.out[(int64_t)m * p.ldo + n0 + seg * 8 + x] = t16[row * 32 + seg * 8 + x];
                                }
                            }
                        }
                        __syncwarp();
                    }
                }
            }
        }
        if (p.tma_store && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // all tile stores of this warp are complete
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (p.status) atomicExch(p.status, MXFP4_E_TIMEOUT);
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        __syncthreads();
    }
    cluster_sync_all();          // neither CTA leaves while the other may still signal it or have MMAs reading its tiles
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
    }
}

template <int BN>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, GemmParams& p, cudaStream_t st) {
    using C = PairCfg<BN>;
    static std::atomic<int> clusters[64];       // co-resident CTA pairs per device, 0 = not configured yet
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) { set_error("mxfp4_gemm: device index out of range"); return MXFP4_E_CUDA; }
    if (!clusters[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxf4_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm: cudaFuncSetAttribute (pair kernel)");
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * num_sms(), 1, 1);
        cfg.blockDim = dim3(kPairThreads, 1, 1);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_mxf4_pair_kernel<BN>, &cfg);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm: cudaOccupancyMaxActiveClusters");
        if (n < 1) { set_error("mxfp4_gemm: no CTA pair of the cta_group::2 kernel fits on this device"); return MXFP4_E_CUDA; }
        clusters[dev] = n;
    }
    p.m_tiles = (p.M + BN - 1) / BN;
    const int64_t units = (int64_t)((p.n_tiles + 1) / 2) * p.m_tiles;
    const int64_t resident = clusters[dev].load();
    const int pairs = (int)(units < resident ? units : resident);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = p.pdl ? 1 : 0;           // may start its set-up while the activation quantiser in front is still running
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_mxf4_pair_kernel<BN>, mw, mx, mo, p);
    if (le != cudaSuccess) return cuda_fail(le, "mxfp4_gemm (tcgen05 cta_group::2 kernel)");
    return MXFP4_OK;
}

}  // namespace

int launch_gemm_pair(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mo, GemmParams& p, cudaStream_t st) {
    switch (bn) {
        case 128: return launch_pair<128>(mw, mx, mo, p, st);
        case 192: return launch_pair<192>(mw, mx, mo, p, st);
        case 256: return launch_pair<256>(mw, mx, mo, p, st);
    }
    set_error("mxfp4_gemm: no cta_group::2 kernel for tile width %d", bn);
    return MXFP4_E_BADARG;
}

}  // namespace mxfp4
