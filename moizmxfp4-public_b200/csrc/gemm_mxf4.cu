// quant_matmul on Blackwell's block-scaled FP4 tensor cores (sm_100a, tcgen05 / TMEM / TMA).
//
//   out[M,N] (bf16) = Xq[M,K] . Wref[N,K]^T (+ bias)
//
// Xq   : activations after mxfp4_act_quantize (hardware E2M1 codes, E8M0 scales);
// Wref : the weight exactly as the reference dequantises it (src/mxfp4/quantizer.py:143-198), i.e.
//        magnitudes {0.5,.75,1,1.5,2,3,4,6} * 2^(b-127).  Hardware E2M1 decodes codes 0 and 1 as 0 and
//        0.5 instead of 0.5 and 0.75, so in EXACT mode every K step issues two MMAs into the same
//        accumulator:   Wref = HW(codes) * 2^(b-127)  +  HW(corr) * 2^(b-128),
//        corr = sign | (code==0 ? 2 : code==1 ? 1 : 0), built in shared memory by the transform warps
//        from the tile TMA just delivered.  The reference bytes are consumed as they are (the "even
//        element in the high nibble" order is shared by both operands, so dot products are unchanged).
//        FAST mode skips the correction pass (weights then decode as hardware E2M1; not parity).
//
// Tiling: one CTA computes a 128 (weight rows, the MMA's M / TMEM lanes) x BN (activation rows, the
// MMA's N / TMEM columns) tile of out^T.  K advances in stages of 256 elements (128 bytes per row,
// one 128-byte swizzle span), 4 MMAs of K=64 per stage and pass.  The grid is persistent (one CTA per SM)
// and walks a list of work units (K range, weight tile, activation tile).
// Warps (17): 0 = TMA producer, 1 and 15 = MMA issuers (1 owns TMEM), 2..5 and 11..14 = correction transform,
// 6..9 = epilogue, 10 and 16 = scale-factor copiers.
// Every wait is bounded; a wait that runs out records MXFP4_E_TIMEOUT in the status word and the
// CTA drains and exits.
#include <atomic>
#include <cstdlib>

#include "gemm_mxf4_tc.cuh"

namespace mxfp4 {
namespace {

template <int BN>
struct Cfg {
    static constexpr int kXT = BN <= 128 ? 1 : 2;                  // 128-row groups of activation scales a tile can touch
    static constexpr int kWBytes = kTileW * kStageKBytes;          // 16 KB
    static constexpr int kXBytes = BN * kStageKBytes;
    static constexpr int kSfwBytes = 2048;
    static constexpr int kSfxBytes = 1024 * kXT;
    static constexpr int kOffX = kWBytes;
    // decode-sized tiles have room for four correction tiles beside four pipeline slots (4-5 % on [128, 12288..22016, 4096])
    static constexpr int kCorrBufs = BN <= 128 ? 4 : 2;            // correction tiles live in a small ring of their own, so that a
    static constexpr int kCorrBytes = kCorrBufs * kWBytes;         // pipeline slot only holds what TMA delivers (more slots in flight)
    static constexpr int kOffSfw = kOffX + kXBytes;
    static constexpr int kOffSfx = kOffSfw + kSfwBytes;
    static constexpr int kStageBytes = (kOffSfx + kSfxBytes + 1023) / 1024 * 1024;
    static constexpr int kEpiBytes = 4 * 4096;                     // per epilogue warp: 32 x 32 words for the transpose
    static constexpr int kBudget = 227 * 1024 - 1024 /*alignment*/ - 512 /*barriers*/ - kEpiBytes - kCorrBytes;
    static constexpr int kStages = (kBudget / kStageBytes) < 8 ? (kBudget / kStageBytes) : 8;
    static constexpr int kSmemBytes = kStages * kStageBytes + kCorrBytes + kEpiBytes + 1024 + 512;
    static constexpr uint32_t kTxBytes = kWBytes + kXBytes;          // operand tiles (full barrier)
    static constexpr uint32_t kSfTxBytes = kSfwBytes + kSfxBytes;    // scale tiles (their own barrier: they land sooner)
    // tensor-memory columns: two accumulators, then scale factors
    // two accumulators (epilogue of one unit overlaps the MMAs of the next) when they fit beside the scale factors
    static constexpr int kAccBufs = BN <= 192 ? 2 : 1;
    static constexpr int kAccStride = BN <= 128 ? 128 : (BN <= 192 ? 192 : 256);
    static constexpr int kColSf = kAccBufs * kAccStride;
    static constexpr int kColSfw = kColSf;         // 2 K-tiles x 4 columns (pass 1)
    static constexpr int kColSfw2 = kColSf + 8;    // same for pass 2
    static constexpr int kColSfx = kColSf + 16;    // 2 K-tiles x 4*kXT columns
    static constexpr int kTmemCols = 512;
    static_assert(BN % 32 == 0 && BN <= 256, "tile width");
    static constexpr int kSfSetCols = 32;          // one set of scale-factor columns per pipeline stage
    static_assert(kColSf + kStages * kSfSetCols <= 512 && 16 + 8 * kXT <= kSfSetCols, "tensor memory budget");
    static_assert(kStages >= 2, "pipeline depth");
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1) gemm_mxf4_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // stages need 1024-byte alignment (128-byte swizzle)
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t corr_base = base + C::kStages * C::kStageBytes;                 // ring of correction tiles
    uint8_t* corr_ptr = base_ptr + C::kStages * C::kStageBytes;
    uint8_t* epi_ptr = corr_ptr + C::kCorrBytes;
    const uint32_t bars = corr_base + C::kCorrBytes + C::kEpiBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
    // everything the MMA thread needs for a stage: correction tile built (4 transform warps, EXACT mode) and scale
    // factors in tensor memory (copier's commit).  One wait per stage: under load every mbarrier round trip costs the
    // issuing thread a few hundred cycles.
    auto ready_bar = [&](int s) { return bars + 8u * (2 * C::kStages + s); };
    auto sfld_bar = [&](int s) { return bars + 8u * (4 * C::kStages + s); };     // scale tiles have landed in shared memory
    auto corr_empty_bar = [&](int c) { return bars + 8u * (5 * C::kStages + c); };   // MMAs have finished with a correction tile
    auto acc_full_bar = [&](int b) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 2 + b); };
    // "the overwriting MMA of unit i has been issued", one barrier per unit parity (the issuers are never more than
    // one unit apart, so a barrier is never two phases ahead of a waiter)
    auto unit_started_bar = [&](int i) { return bars + 8u * (5 * C::kStages + C::kCorrBufs + 4 + (i & 1)); };
    uint8_t* tail = epi_ptr + C::kEpiBytes + 8 * (5 * C::kStages + C::kCorrBufs + 6);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_units = p.n_tiles * p.m_tiles * p.ksplit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(ready_bar(s), p.exact ? 10 : 2);       // 8 transform warps (EXACT) + the two copiers' commits
            mbar_init(sfld_bar(s), 1);
        }
        for (int c = 0; c < C::kCorrBufs; ++c) mbar_init(corr_empty_bar(c), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 2);        // both MMA issuers commit
            mbar_init(acc_empty_bar(b), 4);
        }
        mbar_init(unit_started_bar(0), 1);
        mbar_init(unit_started_bar(1), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(C::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // a split-K reduction launched behind this kernel may be scheduled as soon as SMs have room (it waits for this grid)
    if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // what = 1: weight tile and weight scales, 2: activation tile and activation scales, 3: both
            auto issue = [&](const Unit& w, int ks, uint32_t it, int what) -> bool {
                const int s = it % C::kStages;
                const uint32_t st = base + s * C::kStageBytes;
                const int m0 = w.m_tile * BN;
                if (what & 1) {
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) return false;
                    mbar_expect_tx(full_bar(s), C::kTxBytes);
                    mbar_expect_tx(sfld_bar(s), C::kSfTxBytes);
                    tma_load_2d(st, &map_w, full_bar(s), ks * kStageKBytes, w.n_tile * kTileW);
                    bulk_load(st + C::kOffSfw, p.sfw + ((int64_t)w.n_tile * p.kstages + ks) * 2048, 2048, sfld_bar(s));
                }
                if (what & 2) {
                    tma_load_2d(st + C::kOffX, &map_x, full_bar(s), ks * kStageKBytes, m0);
#pragma unroll
                    for (int t = 0; t < C::kXT; ++t) {
                        // 128-row scale groups the tile touches; a second group past the end of the buffer is
                        // replaced by the first (its rows are beyond M and never stored)
                        int64_t grp = m0 / 128 + t;
                        if (grp * 128 >= ((int64_t)p.M + 127) / 128 * 128) grp = m0 / 128;
                        bulk_load(st + C::kOffSfx + t * 1024, p.sfx + (grp * p.kstages + ks) * 1024, 1024, sfld_bar(s));
                    }
                }
                return true;
            };
            uint32_t it = 0;          // running stage counter across units
            bool ok = true;
            int u_start = blockIdx.x, ks_start = -1;       // where the main loop begins (-1: at the unit's first stage)
            if (p.pdl) {
                // The activations come from the kernel in front of this one, which may still be running: fill the
                // pipeline with the weight side first (it depends on nothing), then wait for that kernel, then add
                // the activation side of the same stages.
                int u = blockIdx.x, ks = 0, npre = 0;
                Unit w = {};
                if (u < total_units) { w = get_unit(p, u); ks = w.ks0; }
                auto advance = [&]() {
                    if (++ks >= w.ks1) {
                        u += gridDim.x;
                        if (u < total_units) { w = get_unit(p, u); ks = w.ks0; }
                    }
                };
                while (ok && npre < C::kStages && u < total_units) {
                    ok = issue(w, ks, (uint32_t)npre, 1);
                    advance();
                    ++npre;
                }
                u_start = u; ks_start = ks;
                asm volatile("griddepcontrol.wait;" ::: "memory");
                u = blockIdx.x;
                if (u < total_units) { w = get_unit(p, u); ks = w.ks0; }
                for (int j = 0; j < npre && ok; ++j) {
                    issue(w, ks, (uint32_t)j, 2);
                    advance();
                }
                it = (uint32_t)npre;
            }
            for (int u = u_start; u < total_units && ok; u += gridDim.x) {
                const Unit w = get_unit(p, u);
                const int m0 = w.m_tile * BN;
                for (int ks = (u == u_start && ks_start >= 0) ? ks_start : w.ks0; ks < w.ks1; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t st = base + s * C::kStageBytes;
                    mbar_expect_tx(full_bar(s), C::kTxBytes);
                    mbar_expect_tx(sfld_bar(s), C::kSfTxBytes);
                    tma_load_2d(st, &map_w, full_bar(s), ks * kStageKBytes, w.n_tile * kTileW);
                    tma_load_2d(st + C::kOffX, &map_x, full_bar(s), ks * kStageKBytes, m0);
                    bulk_load(st + C::kOffSfw, p.sfw + ((int64_t)w.n_tile * p.kstages + ks) * 2048, 2048, sfld_bar(s));
#pragma unroll
                    for (int t = 0; t < C::kXT; ++t) {
                        int64_t grp = m0 / 128 + t;
                        if (grp * 128 >= ((int64_t)p.M + 127) / 128 * 128) grp = m0 / 128;
                        bulk_load(st + C::kOffSfx + t * 1024, p.sfx + (grp * p.kstages + ks) * 1024, 1024, sfld_bar(s));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 15) {
        // ------------------------------------------------------------------ MMA issuers
        // Issuing a tcgen05.mma blocks while earlier MMAs execute (the queue is shallow), so whatever one thread does
        // between two stages -- barrier wait, fence, commits -- would leave the tensor pipe idle.  Two threads
        // therefore take alternate stages: while one is blocked issuing, the other has already done its waiting.
        // Only the MMA that overwrites the accumulator (first of a unit) has to be issued before the others of
        // its unit; the thread that owns it signals `unit_started`, the other one waits for that once per unit.
        if (lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            const uint32_t idesc0 = make_idesc(BN, 0), idesc2 = make_idesc(BN, 2);
            uint32_t it = 0;
            int i = 0;                // units done by this CTA
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
                const Unit w = get_unit(p, u);
                const int buf = i % C::kAccBufs;
                const uint32_t acc_ph = (i / C::kAccBufs) & 1;
                const uint32_t acc = tmem + buf * C::kAccStride;
                // activation scales of a tile that starts inside a 128-row group sit at a column offset
                const uint32_t sfx_off = ((w.m_tile * BN) % 128) / 32;
                ok = mbar_wait(acc_empty_bar(buf), acc_ph ^ 1u, abort_flag);   // epilogue has drained this buffer
                if (!ok) break;
                tc_fence_after();
                bool order_ok = ((it & 1u) == me);          // this thread owns the unit's first stage: nothing to wait for
                for (int ks = w.ks0; ks < w.ks1; ++ks, ++it) {
                    if ((it & 1u) != me) continue;           // the other issuer's stage
                    if (!order_ok) {
                        ok = mbar_wait(unit_started_bar(i), ((uint32_t)i >> 1) & 1u, abort_flag);
                        if (!ok) break;
                        order_ok = true;
                    }
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    ok = mbar_wait(ready_bar(s), ph, abort_flag);   // tiles landed, correction built, scales in tensor memory
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = base + s * C::kStageBytes;
                    const uint32_t sft = tmem + s * C::kSfSetCols;       // this stage's scale-factor columns
                    const uint32_t sfx_col = sft + C::kColSfx + sfx_off;
                    const int cb = it % C::kCorrBufs;                    // correction tile of this stage
                    const uint64_t wdesc = desc_sw128(st), cdesc = desc_sw128(corr_base + cb * C::kWBytes), xdesc = desc_sw128(st + C::kOffX);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const int g = kb >> 1;
                        const uint32_t idesc = (kb & 1) ? idesc2 : idesc0;
                        const uint64_t adv = (uint64_t)(kb * 32 >> 4);             // 64 elements = 32 bytes along K
                        const uint32_t sfb = sfx_col + 4 * C::kXT * g;
                        tc_mma_mxf4(acc, wdesc + adv, xdesc + adv, idesc, sft + C::kColSfw + 4 * g, sfb, (ks > w.ks0 || kb > 0) ? 1u : 0u);
                        if (ks == w.ks0 && kb == 0) mbar_arrive(unit_started_bar(i));
                        if (p.exact) tc_mma_mxf4(acc, cdesc + adv, xdesc + adv, idesc, sft + C::kColSfw2 + 4 * g, sfb, 1u);
                    }
                    tc_commit(empty_bar(s));                      // frees the stage once these MMAs have read it
                    if (p.exact) tc_commit(corr_empty_bar(cb));   // and the correction tile
                }
                tc_commit(acc_full_bar(buf));     // accumulator of this unit complete (or abandoned)
            }
        }
        __syncwarp();
    } else if (warp < 6 || (warp > 10 && warp < 15)) {
        // ------------------------------------------------------------------ correction transform (EXACT mode), 8 warps
        if (p.exact) {
            const int t = (warp < 6 ? warp - 2 : warp - 7) * 32 + lane;       // 0..255
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                const Unit w = get_unit(p, u);
                for (int ks = w.ks0; ks < w.ks1; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    const int cb = it % C::kCorrBufs;
                    const uint32_t cph = (it / C::kCorrBufs) & 1;
                    ok = __all_sync(0xFFFFFFFFu, mbar_wait(corr_empty_bar(cb), cph ^ 1u, abort_flag) && mbar_wait(full_bar(s), ph, abort_flag));
                    if (!ok) break;
                    const uint4* src = reinterpret_cast<const uint4*>(base_ptr + s * C::kStageBytes);
                    uint4* dst = reinterpret_cast<uint4*>(corr_ptr + cb * C::kWBytes);
                    // all loads first, then the bit work, then all stores: eight independent chains per thread
                    uint4 v[C::kWBytes / 16 / 256];
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / 256; ++j) v[j] = src[j * 256 + t];
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / 256; ++j) {
                        v[j].x = corr_word(v[j].x); v[j].y = corr_word(v[j].y); v[j].z = corr_word(v[j].z); v[j].w = corr_word(v[j].w);
                    }
#pragma unroll
                    for (int j = 0; j < C::kWBytes / 16 / 256; ++j) dst[j * 256 + t] = v[j];   // same offset in and out: the swizzle is preserved
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make the writes visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ready_bar(s));
                }
            }
        }
    } else if (warp == 10 || warp == 16) {
        // ------------------------------------------------------------------ scale-factor copier
        // Shared memory -> tensor memory with tcgen05.cp, one column set per pipeline stage.  Issuing these
        // copies costs the issuing thread a few hundred cycles per stage, so they live here and not in the MMA
        // thread; tcgen05.commit tells the MMA thread when a stage's scales are in place.  A set is reused only
        // after its stage has been refilled, i.e. after the MMAs that read it have completed.
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                const Unit w = get_unit(p, u);
                for (int ks = w.ks0; ks < w.ks1; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    ok = mbar_wait(sfld_bar(s), ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = base + s * C::kStageBytes;
                    const uint32_t sft = tmem + s * C::kSfSetCols;
                    if (warp == 10) {
                        // weight scales (both passes); this copier also vouches for the operand tiles
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            tc_cp_sf(sft + C::kColSfw + 4 * g, desc_sf(st + C::kOffSfw + 512 * g));
                            if (p.exact) tc_cp_sf(sft + C::kColSfw2 + 4 * g, desc_sf(st + C::kOffSfw + 1024 + 512 * g));
                        }
                        // the copies are under way; "ready" must also imply that the operand tiles have landed
                        ok = mbar_wait(full_bar(s), ph, abort_flag);
                        if (!ok) break;
                    } else {
                        // activation scales
#pragma unroll
                        for (int g = 0; g < 2; ++g)
#pragma unroll
                            for (int t = 0; t < C::kXT; ++t)
                                tc_cp_sf(sft + C::kColSfx + 4 * C::kXT * g + 4 * t, desc_sf(st + C::kOffSfx + 1024 * t + 512 * g));
                    }
                    tc_commit(ready_bar(s));
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;                               // TMEM lane quarter this warp may read
        uint32_t* tile = reinterpret_cast<uint32_t*>(epi_ptr + (warp - 6) * 4096);
        const bool split = p.ksplit > 1;
        int i = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
            const Unit w = get_unit(p, u);
            const int buf = i % C::kAccBufs;
            ok = mbar_wait(acc_full_bar(buf), (i / C::kAccBufs) & 1, abort_flag);
            ok = __all_sync(0xFFFFFFFFu, ok && !*abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int n0 = w.n_tile * kTileW + q * 32;        // first output column of this warp
            const int n = n0 + lane;
            const float bias = (!split && p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
            const bool has_bias = !split && p.bias != nullptr;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const int m0 = w.m_tile * BN + c0;
                if (m0 >= p.M) break;                             // uniform across the warp
                uint32_t v[32];
                tc_ld_32x32(tmem + buf * C::kAccStride + ((uint32_t)(q * 32) << 16) + c0, v);
                if (c0 + 32 >= BN || m0 + 32 >= p.M) {            // last read of this accumulator: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
                if (split) {
                    // float32 partial sums, [ksp][m][n]
                    float* dstp = p.partial + ((int64_t)w.ksp * p.M) * p.N;
#pragma unroll
                    for (int j = 0; j < 32; ++j) tile[j * 32 + lane] = v[j];
                    __syncwarp();
                    const bool vec = (p.N % 4 == 0) && (n0 + 32 <= p.N);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int row = r * 8 + (lane >> 2), seg = lane & 3;
                        const int m = m0 + row;
                        if (m < p.M) {
                            if (vec) {
#pragma unroll
                                for (int h = 0; h < 2; ++h)
                                    *reinterpret_cast<uint4*>(dstp + (int64_t)m * p.N + n0 + seg * 8 + h * 4) =
                                        *reinterpret_cast<const uint4*>(tile + row * 32 + seg * 8 + h * 4);
                            } else {
                                for (int e = 0; e < 8; ++e)
                                    if (n0 + seg * 8 + e < p.N) dstp[(int64_t)m * p.N + n0 + seg * 8 + e] = __uint_as_float(tile[row * 32 + seg * 8 + e]);
                            }
                        }
                    }
                    __syncwarp();
                } else {
                    // bf16 output: transpose a 32(m) x 32(n) block through shared memory so that each row of 32
                    // consecutive n (64 bytes) is written with 16-byte stores
                    __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(tile);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        __nv_bfloat16 y = __float2bfloat16_rn(__uint_as_float(v[j]));
                        if (has_bias) y = __float2bfloat16_rn(__bfloat162float(y) + bias);   // `output += bias` in bf16
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
                                *reinterpret_cast<uint4*>(p.out + (int64_t)m * p.ldo + n0 + seg * 8) =
                                    *reinterpret_cast<const uint4*>(t16 + row * 32 + seg * 8);
                            } else {
                                for (int e = 0; e < 8; ++e)
                                    if (n0 + seg * 8 + e < p.N) p.out[(int64_t)m * p.ldo + n0 + seg * 8 + e] = t16[row * 32 + seg * 8 + e];
                            }
                        }
                    }
                    __syncwarp();
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (p.status) atomicExch(p.status, MXFP4_E_TIMEOUT);
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);     // let copies and MMAs in flight retire before freeing
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
    }
}

// Sums the K-split partials, rounds to bf16, adds the bias: out[m][n] = bf16(bf16(sum_s partial[s][m][n]) + bias[n]).
// The order of the sum is fixed, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int ksplit, int64_t M, int64_t N,
                                                            const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int64_t ldo) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the partial sums come from the GEMM grid in front
    const int64_t total = M * N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < ksplit; ++s) acc += partial[(int64_t)s * total + i];
        const int64_t m = i / N, n = i - m * N;
        __nv_bfloat16 y = __float2bfloat16_rn(acc);
        if (bias) y = __float2bfloat16_rn(__bfloat162float(y) + __bfloat162float(bias[n]));
        out[m * ldo + n] = y;
    }
}

// Same sum, four consecutive columns per thread (128-bit loads of the partials, one 64-bit store); needs N % 4 == 0,
// ldo % 4 == 0 and an 8-byte-aligned output.
__global__ void __launch_bounds__(256) splitk_reduce4_kernel(const float4* __restrict__ partial, int ksplit, int64_t M, int64_t N,
                                                             const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int64_t ldo) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the partial sums come from the GEMM grid in front
    const int64_t total4 = M * N / 4;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total4; i += (int64_t)gridDim.x * blockDim.x) {
        float4 acc = __ldcs(partial + i);
        for (int s = 1; s < ksplit; ++s) {
            const float4 v = __ldcs(partial + (int64_t)s * total4 + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int64_t e = i * 4, m = e / N, n = e - m * N;
        float r[4] = {acc.x, acc.y, acc.z, acc.w};
        __nv_bfloat16 y[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            y[j] = __float2bfloat16_rn(r[j]);
            if (bias) y[j] = __float2bfloat16_rn(__bfloat162float(y[j]) + __bfloat162float(bias[n + j]));
        }
        uint2 o;
        o.x = (uint32_t)__bfloat16_as_ushort(y[0]) | ((uint32_t)__bfloat16_as_ushort(y[1]) << 16);
        o.y = (uint32_t)__bfloat16_as_ushort(y[2]) | ((uint32_t)__bfloat16_as_ushort(y[3]) << 16);
        *reinterpret_cast<uint2*>(out + m * ldo + n) = o;
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::atomic<EncodeTiledFn> fn{nullptr};
    if (!fn.load()) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn.store((EncodeTiledFn)ptr);
    }
    return fn.load();
}

// Byte matrix [rows, row_bytes] (row pitch = row_bytes), box = 128 bytes x box_rows, 128-byte swizzle,
// out-of-range parts of a box read as zero.
int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t row_bytes, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MXFP4_E_CUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)kStageKBytes, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld, row_bytes=%lld)", (int)r, (long long)rows, (long long)row_bytes); return MXFP4_E_CUDA; }
    return MXFP4_OK;
}

// bf16 matrix [rows, cols] with row pitch ld elements, boxes of 32 x 32, no swizzle (the epilogue's TMA stores).
// Needs a 16-byte aligned base and a pitch that is a multiple of 16 bytes; returns MXFP4_E_ALIGN otherwise.
int make_out_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MXFP4_E_CUDA; }
    if ((uintptr_t)ptr % 16 || (ld * 2) % 16) return MXFP4_E_ALIGN;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r); return MXFP4_E_CUDA; }
    return MXFP4_OK;
}

template <int BN>
int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams& p, cudaStream_t st) {
    using C = Cfg<BN>;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxf4_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm: cudaFuncSetAttribute");
        configured[dev] = true;
    }
    p.m_tiles = (p.M + BN - 1) / BN;
    const int64_t units = (int64_t)p.n_tiles * p.m_tiles * p.ksplit;
    const int grid = (int)(units < num_sms() ? units : num_sms());      // persistent: at most one CTA per SM
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = p.pdl ? 1 : 0;           // may start while the activation quantiser in front is still running
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_mxf4_kernel<BN>, mw, mx, p);
    if (le != cudaSuccess) return cuda_fail(le, "mxfp4_gemm (tcgen05 kernel)");
    return MXFP4_OK;
}

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// Tile width (the MMA's N = activation rows per tile) and number of K ranges of the one-CTA kernel, chosen together
// from a cost model in units of one 128-wide pipeline stage:
//     rounds * (stages per unit + fixed cost per unit) * t(bn)  [+ reduction: fixed cost + traffic of the partials]
// with rounds = ceil(tiles * ksplit / SMs) and t(128, 192, 256) = 1, 1.19, 1.375 (shared-memory bytes per stage); a
// 256-wide tile has a single accumulator, so its epilogue is not hidden and costs six more stages per unit.
// Problems with fewer tiles than SMs leave most of the chip idle; narrower tiles or a cut along K spread the weight
// stream over it.  The model was fitted to the measured grid M in {192..1024} x {4096^2, 11008x4096, 4096x11008} and is
// within ~10 % of the best measured (bn, ksplit) everywhere there.  MXFP4_GEMM_BN / MXFP4_GEMM_KSPLIT override.
//
// swap: the kernel of gemm_mxf4_swap.cu (activations on the MMA's M side, 256 weight rows per tile) instead.  With at
// most 128 activation rows a 128-row weight tile costs the same MMA time as a 256-row one there, so it is taken where
// the 128-row tiles need two rounds over the SMs and the 256-row tiles one (e.g. [128, 22016, 4096]: 172 tiles on 148
// SMs).  MXFP4_GEMM_SWAP=1 takes it for every M <= 128, MXFP4_GEMM_SWAP=0 never.
struct TilePlan {
    int bn, ksplit;
    bool swap;
};
TilePlan pick_plan(int64_t M, int64_t N, int64_t K) {
    const int64_t nks = (K + kStageK - 1) / kStageK;
    const int64_t sms = num_sms();
    const int64_t n_tiles = (N + kTileW - 1) / kTileW;
    int force_bn = 0, force_ks = 0;
    if (const char* e = getenv("MXFP4_GEMM_BN")) {
        const int v = atoi(e);
        if (v == 32 || v == 64 || v == 128 || v == 192 || v == 256) force_bn = v;
    }
    if (const char* e = getenv("MXFP4_GEMM_KSPLIT")) {
        const int v = atoi(e);
        if (v >= 1 && v <= 32) force_ks = v <= nks ? v : (int)nks;
    }
    if (M <= 128) {
        const int64_t wide = (N + 255) / 256;
        const char* e = getenv("MXFP4_GEMM_SWAP");
        const int forced = e ? atoi(e) : -1;
        if (forced == 1 || (forced < 0 && n_tiles > sms && wide <= sms)) {
            int64_t ks = force_ks ? force_ks : sms / wide;          // K ranges only while they fit the same round
            if (ks > 8) ks = 8;
            if (ks > nks) ks = nks;
            if (ks < 1) ks = 1;
            return {256, (int)ks, true};
        }
    }
    static const int kWidths[5] = {32, 64, 128, 192, 256};
    static const int kT1000[5] = {700, 800, 1000, 1190, 1375};     // t(bn) x 1000 (narrow tiles: measured, latency-dominated)
    TilePlan best = {128, 1, false};
    int64_t best_cost = -1;
    for (int i = 0; i < 5; ++i) {
        const int bn = kWidths[i];
        if (force_bn ? bn != force_bn : (M <= 128 ? bn != (M <= 32 ? 32 : M <= 64 ? 64 : 128) : bn < 128)) continue;
        const int64_t tiles = n_tiles * ((M + bn - 1) / bn);
        const int64_t unit_fixed = bn == 256 ? 8 : 2;
        for (int ks = 1; ks <= 32 && ks <= nks; ++ks) {
            if (force_ks ? ks != force_ks : (ks > 1 && (M > 1024 || tiles * 4 >= sms * 3))) continue;
            const int64_t rounds = (tiles * ks + sms - 1) / sms;
            int64_t cost = rounds * ((nks + ks - 1) / ks + unit_fixed) * kT1000[i];
            if (ks > 1) cost += 3000 + (int64_t)ks * M * N * 8 / 5000;       // reduction: launch + partials written and read (~5 MB per stage time)
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = {bn, ks, false}; }
        }
    }
    return best;
}
int pick_ksplit(int64_t M, int64_t N, int64_t K) { return pick_plan(M, N, K).ksplit; }

// Tile width of the cta_group::2 kernel (gemm_mxf4_pair.cu), or 0 for the one-CTA kernel.  Measured on B200 against the
// one-CTA kernel over M in {512..16384} x (N, K) in {4096^2, 11008x4096, 4096x11008, 12288x4096, 22016x4096}: in EXACT mode
// the pair kernel is 5-20 % faster from M = 768 up (from 512 for very wide weights); in FAST mode it wins only for
// M = 1024..2048 with N <= 12288.  MXFP4_GEMM_PAIR=0 forces the one-CTA kernel, MXFP4_GEMM_PAIR=1 the pair kernel wherever
// it can run (M >= 512, N >= 256); MXFP4_GEMM_PAIR_BN picks the width (128, 192, 256).
int pick_pair_bn(int64_t M, int64_t N, bool exact) {
    const char* e = getenv("MXFP4_GEMM_PAIR");
    const int forced = e ? atoi(e) : -1;
    if (forced == 0 || M < 512 || N < 256) return 0;
    if (forced < 0) {
        const bool use = exact ? (M >= 768 || N >= 16384) : (M >= 1024 && M <= 2048 && N <= 12288);
        if (!use) return 0;
    }
    const char* b = getenv("MXFP4_GEMM_PAIR_BN");
    const int bn = b ? atoi(b) : 0;
    return (bn == 128 || bn == 192 || bn == 256) ? bn : 256;
}

}  // namespace
}  // namespace mxfp4

extern "C" int64_t mxfp4_gemm_splitk_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int ks = mxfp4::pick_ksplit(M, N, K);
    return ks > 1 ? (int64_t)ks * M * N * 4 : 0;
}

extern "C" int64_t mxfp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int mode) {
    (void)mode;
    if (M <= 0 || K <= 0) return 0;
    // [control block, 4 KB: status word + reserved] [packed activations M*K/2] [blocked activation scales] [K-split partial sums]
    return 4096 + mxfp4::align_up(M * (K / 2), 256) + mxfp4::align_up(mxfp4_act_scales_bytes(M, K), 256) + mxfp4_gemm_splitk_bytes(M, N, K);
}

namespace mxfp4 {
namespace {
constexpr int kControlBytes = 4096;     // control block: int[0] = status word, the rest is reserved

int gemm_run(const uint8_t* a_packed, const uint8_t* a_sf_blocked, const uint8_t* w_packed, const uint8_t* w_sf_prepared,
             const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M, int64_t N, int64_t K, int mode, void* splitk_workspace,
             int64_t splitk_bytes, int* status_dev, void* stream, bool behind_act_quantize = false, bool keep_partials = false) {
    if (M < 0 || N < 0 || K < 0) { set_error("mxfp4_gemm: negative size"); return MXFP4_E_SHAPE; }
    if (M == 0 || N == 0) return MXFP4_OK;
    if (K == 0 || K % 32) { set_error("mxfp4_gemm: K=%lld must be a positive multiple of 32", (long long)K); return MXFP4_E_SHAPE; }
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) { set_error("mxfp4_gemm: dimension too large"); return MXFP4_E_SHAPE; }
    if (!a_packed || !a_sf_blocked || !w_packed || !w_sf_prepared || !out_bf16) { set_error("mxfp4_gemm: null pointer"); return MXFP4_E_BADARG; }
    if (mode != MXFP4_GEMM_EXACT && mode != MXFP4_GEMM_FAST) { set_error("mxfp4_gemm: unknown mode %d", mode); return MXFP4_E_BADARG; }
    if (ldo < N) { set_error("mxfp4_gemm: ldo < N"); return MXFP4_E_SHAPE; }
    if ((uintptr_t)a_packed % 16 || (uintptr_t)w_packed % 16 || (uintptr_t)a_sf_blocked % 16 || (uintptr_t)w_sf_prepared % 16) {
        set_error("mxfp4_gemm: packed operands and scale buffers must be 16-byte aligned");
        return MXFP4_E_ALIGN;
    }
    CUtensorMap mw, mx;
    const int pair_bn = pick_pair_bn(M, N, mode == MXFP4_GEMM_EXACT);            // 0: one-CTA kernel
    const TilePlan plan = pick_plan(M, N, K);
    const bool swap = !pair_bn && plan.swap;                                     // activations on the MMA's M side
    const int bn = pair_bn ? pair_bn : plan.bn;
    int rc = make_map(&mw, w_packed, N, K / 2, swap ? 256 : kTileW);
    if (rc) return rc;
    rc = make_map(&mx, a_packed, M, K / 2, swap ? 128 : (pair_bn ? pair_bn / 2 : bn));
    if (rc) return rc;
    GemmParams p;
    p.sfw = w_sf_prepared; p.sfx = a_sf_blocked; p.bias = (const __nv_bfloat16*)bias_bf16; p.out = (__nv_bfloat16*)out_bf16;
    p.partial = nullptr;
    p.ldo = ldo; p.M = (int)M; p.N = (int)N; p.K = (int)K; p.kstages = (int)((K + kStageK - 1) / kStageK);
    p.n_tiles = swap ? (int)((N + 255) / 256) : (int)((N + kTileW - 1) / kTileW); p.m_tiles = 0;
    p.ksplit = 1;
    const int want = pair_bn ? 1 : plan.ksplit;
    if (want > 1 && splitk_workspace != nullptr && splitk_bytes >= (int64_t)want * M * N * 4 && (uintptr_t)splitk_workspace % 16 == 0) {
        p.ksplit = want;
        p.partial = (float*)splitk_workspace;
    } else if (want > 1 && keep_partials) {
        // the caller will read [ksplit][M][N] partial sums as mxfp4_gemm_plan announced them: they must exist
        set_error("mxfp4_gemm: MXFP4_GEMM_KEEP_PARTIALS needs a 16-byte aligned split-K workspace of %lld bytes", (long long)want * M * N * 4);
        return MXFP4_E_WORKSPACE;
    }
    p.exact = mode == MXFP4_GEMM_EXACT; p.status = status_dev;
    p.pdl = behind_act_quantize;
    cudaStream_t st = (cudaStream_t)stream;
    p.tma_store = 0;
    if (pair_bn) {
        CUtensorMap mo;
        const int orc = make_out_map(&mo, out_bf16, M, N, ldo);
        if (orc == MXFP4_E_CUDA) return orc;
        p.tma_store = orc == MXFP4_OK;          // an unaligned output keeps the plain stores
        if (!p.tma_store) mo = mw;              // any valid map: the kernel does not touch it
        return launch_gemm_pair(pair_bn, mw, mx, mo, p, st);
    }
    if (swap) rc = launch_gemm_swap(mw, mx, p, st);
    else switch (bn) {
        case 32: rc = launch_gemm<32>(mw, mx, p, st); break;
        case 64: rc = launch_gemm<64>(mw, mx, p, st); break;
        case 128: rc = launch_gemm<128>(mw, mx, p, st); break;
        case 192: rc = launch_gemm<192>(mw, mx, p, st); break;
        default: rc = launch_gemm<256>(mw, mx, p, st); break;
    }
    if (rc) return rc;
    if (p.ksplit > 1 && !keep_partials) {
        const bool vec = N % 4 == 0 && ldo % 4 == 0 && (uintptr_t)p.out % 8 == 0;
        const int64_t total = vec ? M * N / 4 : M * N;
        int64_t grid = (total + 255) / 256;
        const int64_t cap = (int64_t)num_sms() * 16;
        if (grid > cap) grid = cap;
        // launched with programmatic stream serialisation: the grid is scheduled while the GEMM drains and waits for it inside
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid, 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        cudaError_t le;
        if (vec) le = cudaLaunchKernelEx(&cfg, splitk_reduce4_kernel, (const float4*)p.partial, p.ksplit, M, N, p.bias, p.out, ldo);
        else le = cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, (const float*)p.partial, p.ksplit, M, N, p.bias, p.out, ldo);
        if (le != cudaSuccess) return cuda_fail(le, "mxfp4_gemm (split-K reduction)");
    }
    return MXFP4_OK;
}
}  // namespace
}  // namespace mxfp4

extern "C" int mxfp4_gemm_prequantized(const uint8_t* a_packed, const uint8_t* a_sf_blocked, const uint8_t* w_packed,
                                       const uint8_t* w_sf_prepared, const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M,
                                       int64_t N, int64_t K, int mode, void* splitk_workspace, int64_t splitk_bytes, int* control_block,
                                       void* stream) {
    return mxfp4::gemm_run(a_packed, a_sf_blocked, w_packed, w_sf_prepared, bias_bf16, out_bf16, ldo, M, N, K, mode, splitk_workspace,
                           splitk_bytes, control_block, stream);
}

extern "C" int mxfp4_gemm_plan(int64_t M, int64_t N, int64_t K, int mode, int* ksplit, int* cta_pairs) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 32) { mxfp4::set_error("mxfp4_gemm_plan: bad shape"); return MXFP4_E_SHAPE; }
    const int pair_bn = mxfp4::pick_pair_bn(M, N, mode == MXFP4_GEMM_EXACT);
    if (ksplit) *ksplit = pair_bn ? 1 : mxfp4::pick_ksplit(M, N, K);
    if (cta_pairs) *cta_pairs = pair_bn ? 1 : 0;
    return MXFP4_OK;
}

extern "C" int mxfp4_gemm_prequantized_ex(const uint8_t* a_packed, const uint8_t* a_sf_blocked, const uint8_t* w_packed,
                                          const uint8_t* w_sf_prepared, const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M,
                                          int64_t N, int64_t K, int mode, void* splitk_workspace, int64_t splitk_bytes, int* control_block,
                                          int flags, void* stream) {
    return mxfp4::gemm_run(a_packed, a_sf_blocked, w_packed, w_sf_prepared, bias_bf16, out_bf16, ldo, M, N, K, mode, splitk_workspace,
                           splitk_bytes, control_block, stream, (flags & MXFP4_GEMM_CHAINED) != 0, (flags & MXFP4_GEMM_KEEP_PARTIALS) != 0);
}

extern "C" int mxfp4_gemm(const void* x_bf16, int64_t ldx, const uint8_t* w_packed, const uint8_t* w_sf_prepared, const void* bias_bf16,
                          void* out_bf16, int64_t ldo, int64_t M, int64_t N, int64_t K, int mode, void* workspace,
                          int64_t workspace_bytes, void* stream) {
    using namespace mxfp4;
    if (M < 0 || N < 0 || K < 0) { set_error("mxfp4_gemm: negative size"); return MXFP4_E_SHAPE; }
    if (M == 0 || N == 0) return MXFP4_OK;
    if (K == 0 || K % 32) { set_error("mxfp4_gemm: K=%lld must be a positive multiple of 32", (long long)K); return MXFP4_E_SHAPE; }
    if (!x_bf16 || !workspace) { set_error("mxfp4_gemm: null pointer"); return MXFP4_E_BADARG; }
    if (workspace_bytes < mxfp4_gemm_workspace_bytes(M, N, K, mode)) {
        set_error("mxfp4_gemm: workspace of %lld bytes, need %lld", (long long)workspace_bytes, (long long)mxfp4_gemm_workspace_bytes(M, N, K, mode));
        return MXFP4_E_WORKSPACE;
    }
    if ((uintptr_t)workspace % 256) { set_error("mxfp4_gemm: workspace must be 256-byte aligned"); return MXFP4_E_ALIGN; }
    uint8_t* ws = (uint8_t*)workspace;
    int* status = (int*)ws;
    uint8_t* a_packed = ws + kControlBytes;
    uint8_t* a_sf = a_packed + align_up(M * (K / 2), 256);
    uint8_t* partial = a_sf + align_up(mxfp4_act_scales_bytes(M, K), 256);
    int rc = mxfp4_act_quantize(x_bf16, M, K, ldx, a_packed, a_sf, stream);
    if (rc) return rc;
    return gemm_run(a_packed, a_sf, w_packed, w_sf_prepared, bias_bf16, out_bf16, ldo, M, N, K, mode, partial,
                    mxfp4_gemm_splitk_bytes(M, N, K), status, stream, /*behind_act_quantize=*/true);
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some hosts of this library may not allocate device memory at the point where they need a matmul: a
// serving process that handed the whole GPU to its own memory pool at start-up and forbids cudaMalloc
// afterwards, a plugin loaded into such a process, or code on a latency-critical path where an allocation
// would synchronise the device.  For them the scratch that mxfp4_gemm takes as `workspace` (quantised
// activations, their scale tiles, split-K partial sums) lives in the fixed array below instead.
// Every GPU that loads the library holds these 16 MiB until the process exits.
// ------------------------------------------------------------------------------------------------
namespace mxfp4 {
namespace {
constexpr int64_t kNoAllocScratchBytes = 16ll << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace
}  // namespace mxfp4

extern "C" int mxfp4_gemm_noalloc(const void* x_bf16, int64_t ldx, const uint8_t* w_packed, const uint8_t* w_sf_prepared,
                                  const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M, int64_t N, int64_t K, int mode,
                                  int* status_dev, void* stream) {
    using namespace mxfp4;
    if (M < 0 || N < 0 || K < 0) { set_error("mxfp4_gemm_noalloc: negative size"); return MXFP4_E_SHAPE; }
    if (M == 0 || N == 0) return MXFP4_OK;
    if (K == 0 || K % 32) { set_error("mxfp4_gemm_noalloc: K=%lld must be a positive multiple of 32", (long long)K); return MXFP4_E_SHAPE; }
    if (!x_bf16) { set_error("mxfp4_gemm_noalloc: null pointer"); return MXFP4_E_BADARG; }
    const int64_t act_bytes = align_up(M * (K / 2), 256);
    const int64_t sf_bytes = align_up(mxfp4_act_scales_bytes(M, K), 256);
    const int64_t split_bytes = mxfp4_gemm_splitk_bytes(M, N, K);
    const int64_t need = kControlBytes + act_bytes + sf_bytes + split_bytes;
    if (need > kNoAllocScratchBytes) {
        set_error("mxfp4_gemm_noalloc: M=%lld N=%lld K=%lld needs %lld bytes of scratch, the built-in array holds %lld; "
                  "use mxfp4_gemm with a caller-provided workspace for this size",
                  (long long)M, (long long)N, (long long)K, (long long)need, (long long)kNoAllocScratchBytes);
        return MXFP4_E_WORKSPACE;
    }
    // The array's name is only a host-side handle; the kernels need its device address, which differs per
    // device.  Looked up once per device, with that device current (it is: the caller made it current).
    static std::atomic<unsigned char*> scratch_addr[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm_noalloc: cudaGetDevice");
    if (dev < 0 || dev >= 64) { set_error("mxfp4_gemm_noalloc: device index %d out of range", dev); return MXFP4_E_UNSUPPORTED; }
    if (scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm_noalloc: cudaGetSymbolAddress");
        scratch_addr[dev] = (unsigned char*)ptr;
    }
    uint8_t* a_packed = scratch_addr[dev] + kControlBytes;
    uint8_t* a_sf = a_packed + act_bytes;
    uint8_t* partial = a_sf + sf_bytes;
    int rc = mxfp4_act_quantize(x_bf16, M, K, ldx, a_packed, a_sf, stream);
    if (rc) return rc;
    return gemm_run(a_packed, a_sf, w_packed, w_sf_prepared, bias_bf16, out_bf16, ldo, M, N, K, mode,
                    split_bytes ? partial : nullptr, split_bytes, status_dev, stream, /*behind_act_quantize=*/true);
}
