// quant_matmul for large M on CTA pairs: tcgen05.mma.cta_group::2 (one instruction spans two SMs).
//
// Same arithmetic, operand formats and pipeline roles as gemm_mxf4.cu.  Here two CTAs of a cluster work on one
// 256 (weight rows) x BN (activation rows) tile of out^T: each CTA holds its own 128 weight rows and HALF of the
// activation tile in shared memory, and the tensor cores of both SMs read both halves.  Per accumulator column
// each SM therefore reads half as many activation bytes from its shared memory as the one-CTA kernel does, which
// is what bounds that kernel in EXACT mode.
//
// CTA 0 of the pair (the leader) issues every tcgen05.mma / tcgen05.cp / tcgen05.commit; the instructions execute
// in both SMs, each on its own shared and tensor memory at the same addresses, so both CTAs keep identical
// layouts.  Completion is multicast to the same barrier in both CTAs.  What the peer CTA produces (tiles landed,
// correction tile built, accumulator drained) reaches the leader as remote mbarrier arrivals.
// Every wait is bounded as in the one-CTA kernel; both CTAs meet at a cluster barrier before they exit, so no
// remote arrival can target a CTA that has gone.
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
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cl(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait on a barrier that the other CTA of the pair may signal
__device__ __forceinline__ bool mbar_wait_cl(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_cl(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) break;
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc2_commit(uint32_t bar) {          // arrives on this CTA's barrier
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {     // arrives on the same barrier of both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void tc2_cp_sf(uint32_t tmem_addr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
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
// instruction descriptor as make_idesc, with M = 256 (128 rows in each CTA)
__device__ __forceinline__ uint32_t make_idesc_pair(int n, uint32_t sf_id) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(256 >> 4) << 24) | (sf_id << 29) | (sf_id << 4);
}

template <int BN>
struct PairCfg {
    static constexpr int kHalf = BN / 2;                           // activation rows each CTA stages
    static constexpr int kXT = BN <= 128 ? 1 : 2;                  // 128-row groups of activation scales a tile can touch
    static constexpr int kWBytes = kTileW * kStageKBytes;          // 16 KB
    static constexpr int kXBytes = kHalf * kStageKBytes;
    static constexpr int kSfwBytes = 2048;
    static constexpr int kSfxBytes = 1024 * kXT;                   // scales of the WHOLE activation tile, in both CTAs
    static constexpr int kOffX = kWBytes;
    static constexpr int kOffSfw = kOffX + kXBytes;
    static constexpr int kOffSfx = kOffSfw + kSfwBytes;
    static constexpr int kStageBytes = (kOffSfx + kSfxBytes + 1023) / 1024 * 1024;
    static constexpr int kCorrBufs = 2;
    static constexpr int kCorrBytes = kCorrBufs * kWBytes;
    static constexpr int kEpiBytes = 4 * 4096;
    static constexpr int kAccBufs = BN <= 192 ? 2 : 1;
    static constexpr int kAccStride = BN <= 128 ? 128 : (BN <= 192 ? 192 : 256);
    // tensor memory: the accumulators, then one set of scale-factor columns per MMA-issuing thread
    static constexpr int kColSf = kAccBufs * kAccStride;
    static constexpr int kSfSetCols = 32;
    static constexpr int kColSfw = kColSf;         // 2 K-tiles x 4 columns (pass 1)
    static constexpr int kColSfw2 = kColSf + 8;    // same for pass 2
    static constexpr int kColSfx = kColSf + 16;    // 2 K-tiles x 4*kXT columns
    static constexpr int kBudget = 227 * 1024 - 1024 - 512 - kEpiBytes - kCorrBytes;
    static constexpr int kBySmem = kBudget / kStageBytes;
    static constexpr int kStages = kBySmem < 8 ? kBySmem : 8;
    static constexpr int kSmemBytes = kStages * kStageBytes + kCorrBytes + kEpiBytes + 1024 + 512;
    static constexpr uint32_t kTxBytes = kWBytes + kXBytes + kSfwBytes + kSfxBytes;   // everything a CTA loads for a stage
    static constexpr int kTmemCols = 512;
    static_assert(BN % 32 == 0 && BN <= 256 && kHalf % 8 == 0, "tile width");
    static_assert(kStages >= 2 && 16 + 8 * kXT <= kSfSetCols && kColSf + 2 * kSfSetCols <= 512, "pipeline depth / tensor memory");
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
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_mxf4_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
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
    auto full_bar = [&](int s) { return bars + 8u * s; };                        // this CTA's operand and scale tiles have landed
    auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };        // MMAs have finished with the stage (both CTAs)
    // used in the leader only; the peer's arrivals come in remotely
    auto ready_bar = [&](int s) { return bars + 8u * (3 * C::kStages + s); };    // both CTAs: tiles landed, correction built
    auto corr_empty_bar = [&](int c) { return bars + 8u * (5 * C::kStages + c); };
    auto acc_full_bar = [&](int b) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 2 + b); };   // leader: 8 epilogue warps of the pair
    auto unit_started_bar = [&](int i) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 4 + (i & 1)); };
    uint8_t* tail = epi_ptr + C::kEpiBytes + 8 * (5 * C::kStages + C::kCorrBufs + 6);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const bool leader = rank == 0;
    const int n_pairs = (p.n_tiles + 1) / 2;
    const int total_units = n_pairs * p.m_tiles;
    const int first_unit = blockIdx.x >> 1, unit_step = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            // one "tiles landed" report per CTA; in EXACT mode also the 8 + 8 transform warps
            mbar_init(ready_bar(s), p.exact ? 18 : 2);
        }
        for (int c = 0; c < C::kCorrBufs; ++c) mbar_init(corr_empty_bar(c), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 2);        // both MMA issuers commit (multicast to both CTAs)
            mbar_init(acc_empty_bar(b), 8);       // 4 epilogue warps in each CTA
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
            for (int u = first_unit; u < total_units && ok; u += unit_step) {
                const PairUnit w = get_pair_unit(p, n_pairs, u);
                const int m0 = w.m_tile * BN;
                const int n_tile = w.n_pair * 2 + (int)rank;
                const int sf_tile = n_tile < p.n_tiles ? n_tile : p.n_tiles - 1;     // a tile past the end reads a valid one; nothing of it is stored
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
#ifdef MXFP4_PAIR_PROF
                    const long long pt0 = clock64();
#endif
                    if (!mbar_wait_cl(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
#ifdef MXFP4_PAIR_PROF
                    reinterpret_cast<long long*>(p.status)[1024 + blockIdx.x * 8 + 4] += clock64() - pt0;
#endif
                    const uint32_t st = base + s * C::kStageBytes;
                    mbar_expect_tx(full_bar(s), C::kTxBytes);
                    tma_load_2d(st, &map_w, full_bar(s), ks * kStageKBytes, n_tile * kTileW);
                    tma_load_2d(st + C::kOffX, &map_x, full_bar(s), ks * kStageKBytes, m0 + (int)rank * C::kHalf);
                    bulk_load(st + C::kOffSfw, p.sfw + ((int64_t)sf_tile * p.kstages + ks) * 2048, 2048, full_bar(s));
#pragma unroll
                    for (int t = 0; t < C::kXT; ++t) {
                        int64_t grp = m0 / 128 + t;
                        if (grp * 128 >= ((int64_t)p.M + 127) / 128 * 128) grp = m0 / 128;
                        bulk_load(st + C::kOffSfx + t * 1024, p.sfx + (grp * p.kstages + ks) * 1024, 1024, full_bar(s));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 15) {
        // ------------------------------------------------------------------ MMA issuers (leader CTA only), alternate stages
        if (leader && lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            const uint32_t idesc0 = make_idesc_pair(BN, 0), idesc2 = make_idesc_pair(BN, 2);
            uint32_t it = 0;
            int i = 0;
            bool ok = true;
#ifdef MXFP4_PAIR_PROF
            long long pf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long pstart = clock64();
#define PROF_T(var) const long long var = clock64()
#define PROF_ADD(i, v) pf[i] += (v)
#else
#define PROF_T(var)
#define PROF_ADD(i, v)
#endif
            for (int u = first_unit; u < total_units && ok; u += unit_step, ++i) {
                const PairUnit w = get_pair_unit(p, n_pairs, u);
                const int buf = i % C::kAccBufs;
                const uint32_t acc_ph = (i / C::kAccBufs) & 1;
                const uint32_t acc = tmem + buf * C::kAccStride;
                const uint32_t sfx_off = ((w.m_tile * BN) % 128) / 32;
                PROF_T(ta0);
                ok = mbar_wait_cl(acc_empty_bar(buf), acc_ph ^ 1u, abort_flag);   // both CTAs' epilogues have drained this buffer
                if (!ok) break;
                PROF_T(ta1);
                PROF_ADD(3, ta1 - ta0);
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
                    PROF_T(tr0);
#ifdef MXFP4_PAIR_PROF
                    if (!mbar_try_wait_cl(ready_bar(s), ph)) pf[2] += 1;
#endif
                    ok = mbar_wait_cl(ready_bar(s), ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    PROF_T(tr1);
                    PROF_ADD(1, tr1 - tr0);
                    PROF_ADD(7, 1);
                    const uint32_t st = base + s * C::kStageBytes;
                    // Scale factors, shared -> tensor memory in both SMs, into this thread's own column set.  Copies
                    // and MMAs of one thread execute in issue order, so the MMAs below see them and the copies of
                    // this thread's next stage cannot overtake these MMAs.
                    const uint32_t sft = tmem + me * C::kSfSetCols;
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        tc2_cp_sf(sft + C::kColSfw + 4 * g, desc_sf(st + C::kOffSfw + 512 * g));
                        if (p.exact) tc2_cp_sf(sft + C::kColSfw2 + 4 * g, desc_sf(st + C::kOffSfw + 1024 + 512 * g));
#pragma unroll
                        for (int t = 0; t < C::kXT; ++t)
                            tc2_cp_sf(sft + C::kColSfx + 4 * C::kXT * g + 4 * t, desc_sf(st + C::kOffSfx + 1024 * t + 512 * g));
                    }
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
                    PROF_T(ti1);
                    PROF_ADD(5, ti1 - tr1);
                    tc2_commit_both(empty_bar(s));
                    if (p.exact) tc2_commit_both(corr_empty_bar(cb));
                    PROF_T(tc1);
                    PROF_ADD(6, tc1 - ti1);
                }
                tc2_commit_both(acc_full_bar(buf));
            }
#ifdef MXFP4_PAIR_PROF
            if (me == 0) {
                pf[0] = clock64() - pstart;
                long long* dstp = reinterpret_cast<long long*>(p.status) + 1024 + blockIdx.x * 8;
                for (int j = 0; j < 8; ++j)
                    if (j != 4) dstp[j] = pf[j];
            }
#endif
        }
        __syncwarp();
    } else if (warp < 6 || (warp > 10 && warp < 15)) {
        // ------------------------------------------------------------------ correction transform (EXACT mode), 8 warps per CTA
        if (p.exact) {
            const int t = (warp < 6 ? warp - 2 : warp - 7) * 32 + lane;
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
                    uint4 v[C::kWBytes / 16 / 256];
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / 256; ++j) v[j] = src[j * 256 + t];
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / 256; ++j) {
                        v[j].x = corr_word(v[j].x); v[j].y = corr_word(v[j].y); v[j].z = corr_word(v[j].z); v[j].w = corr_word(v[j].w);
                    }
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / 256; ++j) dst[j * 256 + t] = v[j];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(ready_bar(s));
                        else mbar_arrive_remote(map_to_cta(ready_bar(s), 0));
                    }
                }
            }
        }
    } else if (warp == 10 || warp == 16) {
        // ------------------------------------------------------------------ "tiles landed" report to the leader's ready barrier
        if (warp == 10 && lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const uint32_t ready0 = leader ? 0u : map_to_cta(ready_bar(0), 0);
            for (int u = first_unit; u < total_units && ok; u += unit_step) {
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    ok = mbar_wait(full_bar(s), ph, abort_flag);
                    if (!ok) break;
                    if (leader) mbar_arrive(ready_bar(s));
                    else mbar_arrive_remote(ready0 + 8u * s);
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (each CTA stores its own 128 weight rows)
        const int q = warp & 3;
        uint32_t* tile = reinterpret_cast<uint32_t*>(epi_ptr + (warp - 6) * 4096);
        const bool has_bias = p.bias != nullptr;
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
            bool released = false;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const int m0 = w.m_tile * BN + c0;
                if (m0 >= p.M) break;
                uint32_t v[32];
                tc_ld_32x32(tmem + buf * C::kAccStride + ((uint32_t)(q * 32) << 16) + c0, v);
                if (c0 + 32 >= BN || m0 + 32 >= p.M) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(acc_empty_bar(buf));
                        else mbar_arrive_remote(map_to_cta(acc_empty_bar(buf), 0));
                    }
                    released = true;
                }
                __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(tile);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    __nv_bfloat16 y = __float2bfloat16_rn(__uint_as_float(v[j]));
                    if (has_bias) y = __float2bfloat16_rn(__bfloat162float(y) + bias);
                    t16[j * 32 + lane] = y;
                }
                __syncwarp();
                const bool vec = (p.ldo % 8 == 0) && (((uintptr_t)p.out) % 16 == 0) && (n0 + 32 <= p.N);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int row = r * 8 + (lane >> 2), seg = lane & 3;
                    const int m = m0 + row;
                    if (m < p.M) {
                        if (vec) {
                            *reinterpret_cast<uint4*>(p.out + (int64_t)m * p.ldo + n0 + seg * 8) = *reinterpret_cast<const uint4*>(t16 + row * 32 + seg * 8);
                        } else {
                            for (int e = 0; e < 8; ++e)
                                if (n0 + seg * 8 + e < p.N) p.out[(int64_t)m * p.ldo + n0 + seg * 8 + e] = t16[row * 32 + seg * 8 + e];
                        }
                    }
                }
                __syncwarp();
            }
            (void)released;
        }
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
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams& p, cudaStream_t st) {
    using C = PairCfg<BN>;
    static int clusters[64] = {0};       // co-resident CTA pairs per device, 0 = not configured yet
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) { set_error("mxfp4_gemm: device index out of range"); return MXFP4_E_CUDA; }
    if (!clusters[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxf4_pair_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm: cudaFuncSetAttribute (pair kernel)");
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * num_sms(), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
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
    const int pairs = (int)(units < clusters[dev] ? units : clusters[dev]);
    gemm_mxf4_pair_kernel<BN><<<2 * pairs, kThreads, C::kSmemBytes, st>>>(mw, mx, p);
    MXFP4_CHECK_LAUNCH("mxfp4_gemm (tcgen05 cta_group::2 kernel)");
    return MXFP4_OK;
}

}  // namespace

int launch_gemm_pair(int bn, const CUtensorMap& mw, const CUtensorMap& mx, GemmParams& p, cudaStream_t st) {
    switch (bn) {
        case 128: return launch_pair<128>(mw, mx, p, st);
        case 192: return launch_pair<192>(mw, mx, p, st);
        case 256: return launch_pair<256>(mw, mx, p, st);
    }
    set_error("mxfp4_gemm: no cta_group::2 kernel for tile width %d", bn);
    return MXFP4_E_BADARG;
}

}  // namespace mxfp4
