// quant_matmul for at most 128 activation rows with the operand roles of gemm_mxf4.cu exchanged.
//
// A tcgen05.mma whose M side holds 128 rows takes about 128 cycles however few rows its N side has, so the kernel of
// gemm_mxf4.cu (128 weight rows on the M side, the batch on the N side) pays the full-width time for every 128 weight
// rows at decode sizes.  Here the activations (up to 128 rows, zero-filled by TMA beyond M) sit on the M side / the
// lanes of tensor memory and 256 weight rows on the N side / its columns: half as many MMAs for the same weight, and
// the accumulator comes out row-major (a lane is an output row), so the epilogue stores without a transpose.
//
// Numerics are those of gemm_mxf4.cu: EXACT mode issues a second MMA per K step on a correction tile (now the B
// operand, 256 rows) with the "scale - 1" bytes; FAST mode skips it.  Same K stages of 256 elements, same scale-factor
// tiles (a 128-row tile of prepared weight scales is the same 512-byte atom whether it feeds the A or the B side), same
// K split with float32 partial sums [ksplit][M][N], same bounded waits and programmatic dependent launch.
// Warps (17): 0 = TMA producer, 1 and 15 = MMA issuers (1 owns tensor memory), 2..5 and 11..14 = correction transform,
// 6..9 = epilogue, 10 and 16 = scale-factor copiers.
#include <atomic>

#include "gemm_mxf4_tc.cuh"

namespace mxfp4 {
namespace {

constexpr int kBW = 256;                                       // weight rows per tile (the MMA's N)
struct SCfg {
    static constexpr int kWBytes = kBW * kStageKBytes;         // 32 KB
    static constexpr int kXBytes = 128 * kStageKBytes;         // 16 KB: always a 128-row box, rows past M arrive as zeros
    static constexpr int kSfwBytes = 2 * 2048;                 // two 128-row tiles of prepared weight scales (both passes each)
    static constexpr int kSfxBytes = 1024;
    static constexpr int kOffX = kWBytes;
    static constexpr int kOffSfw = kOffX + kXBytes;
    static constexpr int kOffSfx = kOffSfw + kSfwBytes;
    static constexpr int kStageBytes = (kOffSfx + kSfxBytes + 1023) / 1024 * 1024;
    static constexpr int kStages = 3;
    static constexpr int kCorrBufs = 2;
    static constexpr int kCorrBytes = kCorrBufs * kWBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kCorrBytes + 1024 + 512;
    static constexpr uint32_t kTxBytes = kWBytes + kXBytes;
    static constexpr uint32_t kSfTxBytes = kSfwBytes + kSfxBytes;
    // tensor memory: one 256-column accumulator, then one set of scale-factor columns per pipeline stage
    static constexpr int kColSf = 256;
    static constexpr int kSfSetCols = 48;
    static constexpr int kColSfa = 0;       // activations: 2 K-tiles x 4 columns
    static constexpr int kColSfb = 8;       // weights, pass 1: 2 K-tiles x (2 row tiles x 4 columns)
    static constexpr int kColSfb2 = 24;     // weights, pass 2
    static constexpr int kTmemCols = 512;
    static_assert(kSmemBytes <= 227 * 1024 && kColSf + kStages * kSfSetCols <= 512, "shared / tensor memory budget");
};

__global__ void __launch_bounds__(kThreads, 1) gemm_mxf4_swap_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    using C = SCfg;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // stages need 1024-byte alignment (128-byte swizzle)
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t corr_base = base + C::kStages * C::kStageBytes;                 // ring of correction tiles
    uint8_t* corr_ptr = base_ptr + C::kStages * C::kStageBytes;
    const uint32_t bars = corr_base + C::kCorrBytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };                          // operand tiles have landed
    auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };          // the MMAs have finished with the stage
    auto ready_bar = [&](int s) { return bars + 8u * (2 * C::kStages + s); };      // correction built, scales in tensor memory
    auto sfld_bar = [&](int s) { return bars + 8u * (3 * C::kStages + s); };       // scale tiles have landed in shared memory
    auto corr_empty_bar = [&](int c) { return bars + 8u * (4 * C::kStages + c); };
    const uint32_t acc_full_bar = bars + 8u * (4 * C::kStages + C::kCorrBufs);
    const uint32_t acc_empty_bar = acc_full_bar + 8u;
    auto unit_started_bar = [&](int i) { return acc_full_bar + 16u + 8u * (i & 1); };
    uint8_t* tail = corr_ptr + C::kCorrBytes + 8 * (4 * C::kStages + C::kCorrBufs + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_units = p.n_tiles * p.ksplit;          // n_tiles counts 256-row weight tiles here; one activation tile
    const int w_tiles128 = (p.N + 127) / 128;               // prepared weight scales come in 128-row tiles

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(ready_bar(s), p.exact ? 10 : 2);       // 8 transform warps (EXACT) + the two copiers' commits
            mbar_init(sfld_bar(s), 1);
        }
        for (int c = 0; c < C::kCorrBufs; ++c) mbar_init(corr_empty_bar(c), 1);
        mbar_init(acc_full_bar, 2);             // both MMA issuers commit
        mbar_init(acc_empty_bar, 4);
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
                if (what & 1) {
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) return false;
                    mbar_expect_tx(full_bar(s), C::kTxBytes);
                    mbar_expect_tx(sfld_bar(s), C::kSfTxBytes);
                    tma_load_2d(st, &map_w, full_bar(s), ks * kStageKBytes, w.n_tile * kBW);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        // a second 128-row tile past the end of the weight is replaced by the first (its rows are
                        // beyond N and never stored)
                        int64_t t128 = (int64_t)w.n_tile * 2 + t;
                        if (t128 >= w_tiles128) t128 = (int64_t)w.n_tile * 2;
                        bulk_load(st + C::kOffSfw + t * 2048, p.sfw + (t128 * p.kstages + ks) * 2048, 2048, sfld_bar(s));
                    }
                }
                if (what & 2) {
                    tma_load_2d(st + C::kOffX, &map_x, full_bar(s), ks * kStageKBytes, 0);
                    bulk_load(st + C::kOffSfx, p.sfx + (int64_t)ks * 1024, 1024, sfld_bar(s));
                }
                return true;
            };
            // The activations may come from a kernel that is still running (programmatic dependent launch): fill the
            // pipeline with the weight side first, wait for that kernel, then add the activation side of the same stages.
            uint32_t it = 0;
            bool ok = true;
            int u = blockIdx.x, ks = 0, npre = 0;
            Unit w = {};
            if (u < total_units) { w = get_unit(p, u); ks = w.ks0; }
            auto advance = [&]() {
                if (++ks >= w.ks1) {
                    u += gridDim.x;
                    if (u < total_units) { w = get_unit(p, u); ks = w.ks0; }
                }
            };
            if (p.pdl) {
                while (ok && npre < C::kStages && u < total_units) {
                    ok = issue(w, ks, (uint32_t)npre, 1);
                    advance();
                    ++npre;
                }
                const int u_next = u, ks_next = ks;
                const Unit w_next = w;
                asm volatile("griddepcontrol.wait;" ::: "memory");
                u = blockIdx.x;
                if (u < total_units) { w = get_unit(p, u); ks = w.ks0; }
                for (int j = 0; j < npre && ok; ++j) {
                    issue(w, ks, (uint32_t)j, 2);
                    advance();
                }
                it = (uint32_t)npre;
                u = u_next; ks = ks_next; w = w_next;
            }
            while (ok && u < total_units) {
                ok = issue(w, ks, it, 3);
                advance();
                ++it;
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 15) {
        // ------------------------------------------------------------------ MMA issuers (alternate stages, as in gemm_mxf4.cu)
        if (lane == 0) {
            const uint32_t me = warp == 1 ? 0u : 1u;
            const uint32_t idesc0 = make_idesc(kBW, 0), idesc2 = make_idesc(kBW, 2);
            uint32_t it = 0;
            int i = 0;                // units done by this CTA
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
                const Unit w = get_unit(p, u);
                ok = mbar_wait(acc_empty_bar, ((uint32_t)i & 1u) ^ 1u, abort_flag);   // epilogue has drained the accumulator
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
                    const uint32_t sft = tmem + C::kColSf + s * C::kSfSetCols;       // this stage's scale-factor columns
                    const int cb = it % C::kCorrBufs;                                // correction tile of this stage
                    const uint64_t wdesc = desc_sw128(st), cdesc = desc_sw128(corr_base + cb * C::kWBytes), xdesc = desc_sw128(st + C::kOffX);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const int g = kb >> 1;
                        const uint32_t idesc = (kb & 1) ? idesc2 : idesc0;
                        const uint64_t adv = (uint64_t)(kb * 32 >> 4);             // 64 elements = 32 bytes along K
                        const uint32_t sfa = sft + C::kColSfa + 4 * g;
                        tc_mma_mxf4(tmem, xdesc + adv, wdesc + adv, idesc, sfa, sft + C::kColSfb + 8 * g, (ks > w.ks0 || kb > 0) ? 1u : 0u);
                        if (ks == w.ks0 && kb == 0) mbar_arrive(unit_started_bar(i));
                        if (p.exact) tc_mma_mxf4(tmem, xdesc + adv, cdesc + adv, idesc, sfa, sft + C::kColSfb2 + 8 * g, 1u);
                    }
                    tc_commit(empty_bar(s));                      // frees the stage once these MMAs have read it
                    if (p.exact) tc_commit(corr_empty_bar(cb));   // and the correction tile
                }
                tc_commit(acc_full_bar);          // accumulator of this unit complete (or abandoned)
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
        // ------------------------------------------------------------------ scale-factor copiers: shared -> tensor memory
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
                    const uint32_t sft = tmem + C::kColSf + s * C::kSfSetCols;
                    if (warp == 10) {
                        // weight scales of both 128-row tiles (both passes); this copier also vouches for the operand tiles
#pragma unroll
                        for (int g = 0; g < 2; ++g)
#pragma unroll
                            for (int t = 0; t < 2; ++t) {
                                tc_cp_sf(sft + C::kColSfb + 8 * g + 4 * t, desc_sf(st + C::kOffSfw + 2048 * t + 512 * g));
                                if (p.exact) tc_cp_sf(sft + C::kColSfb2 + 8 * g + 4 * t, desc_sf(st + C::kOffSfw + 2048 * t + 1024 + 512 * g));
                            }
                        ok = mbar_wait(full_bar(s), ph, abort_flag);
                        if (!ok) break;
                    } else {
#pragma unroll
                        for (int g = 0; g < 2; ++g) tc_cp_sf(sft + C::kColSfa + 4 * g, desc_sf(st + C::kOffSfx + 512 * g));
                    }
                    tc_commit(ready_bar(s));
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue: a lane is an output row
        const int q = warp & 3;                               // TMEM lane quarter this warp may read
        const int m = q * 32 + lane;
        const bool split = p.ksplit > 1;
        const bool has_bias = !split && p.bias != nullptr;
        int i = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
            const Unit w = get_unit(p, u);
            ok = mbar_wait(acc_full_bar, (uint32_t)i & 1u, abort_flag);
            ok = __all_sync(0xFFFFFFFFu, ok && !*abort_flag);
            if (!ok) break;
            tc_fence_after();
            float* prow = split ? p.partial + ((int64_t)w.ksp * p.M + m) * p.N : nullptr;
            __nv_bfloat16* orow = p.out + (int64_t)m * p.ldo;
            const bool pvec = p.N % 4 == 0, ovec = p.ldo % 8 == 0 && ((uintptr_t)p.out) % 16 == 0;
#pragma unroll 1
            for (int c0 = 0; c0 < kBW; c0 += 32) {
                const int n0 = w.n_tile * kBW + c0;               // < N: the loop ends behind the chunk that reaches N
                uint32_t v[32];
                tc_ld_32x32(tmem + ((uint32_t)(q * 32) << 16) + c0, v);
                const bool last = c0 + 32 >= kBW || n0 + 32 >= p.N;
                if (last) {                                       // last read of the accumulator: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar);
                }
                if (m < p.M) {
                    const bool full = n0 + 32 <= p.N;
                    if (split) {
                        // float32 partial sums, [ksp][m][n]
                        if (full && pvec) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(prow + n0 + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (n0 + j < p.N) prow[n0 + j] = __uint_as_float(v[j]);
                        }
                    } else {
                        uint32_t o[16];
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            __nv_bfloat16 y0 = __float2bfloat16_rn(__uint_as_float(v[j])), y1 = __float2bfloat16_rn(__uint_as_float(v[j + 1]));
                            if (has_bias) {                       // `output += bias` in bf16
                                if (n0 + j < p.N) y0 = __float2bfloat16_rn(__bfloat162float(y0) + __bfloat162float(p.bias[n0 + j]));
                                if (n0 + j + 1 < p.N) y1 = __float2bfloat16_rn(__bfloat162float(y1) + __bfloat162float(p.bias[n0 + j + 1]));
                            }
                            o[j >> 1] = (uint32_t)__bfloat16_as_ushort(y0) | ((uint32_t)__bfloat16_as_ushort(y1) << 16);
                        }
                        if (full && ovec) {
#pragma unroll
                            for (int j = 0; j < 16; j += 4) *reinterpret_cast<uint4*>(orow + n0 + 2 * j) = make_uint4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (n0 + j < p.N) orow[n0 + j] = __ushort_as_bfloat16((unsigned short)((o[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
                        }
                    }
                }
                if (last) break;
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

}  // namespace

// map_w: packed weight with 256-row boxes; map_x: packed activations with 128-row boxes.  p.n_tiles must count 256-row
// weight tiles, p.M <= 128.
int launch_gemm_swap(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams& p, cudaStream_t st) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxf4_swap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SCfg::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm: cudaFuncSetAttribute");
        configured[dev] = true;
    }
    p.m_tiles = 1;
    const int64_t units = (int64_t)p.n_tiles * p.ksplit;
    const int grid = (int)(units < num_sms() ? units : num_sms());      // persistent: at most one CTA per SM
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = SCfg::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = p.pdl ? 1 : 0;           // may start while the kernel that makes the activations is still running
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_mxf4_swap_kernel, mw, mx, p);
    if (le != cudaSuccess) return cuda_fail(le, "mxfp4_gemm (tcgen05 kernel, activations on the M side)");
    return MXFP4_OK;
}

}  // namespace mxfp4
