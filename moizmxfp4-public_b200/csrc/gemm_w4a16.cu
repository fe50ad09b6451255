// W4A16 quant_matmul on the bf16 tensor cores (tcgen05.mma kind::f16): the reference's own GEMM semantics.
//
//   out[M,N] (bf16) = X[M,K] (bf16, NOT quantised) . Wd[N,K]^T (+ bias),   Wd = bf16(level[code] * scale)
//
// which is what FallbackBackend.matmul (src/mxfp4/backends.py:295-312) and the Triton kernel
// (src/mxfp4/fused_kernels.py:141-158, :174-178) compute: dequantise the weight, cast it to the activations' dtype,
// multiply with float32 accumulation, round to bf16, add the bias in bf16.  Two uses:
//   * weights quantised with scale_format="bf16" (src/mxfp4/quantizer.py:137-139): their scales are not powers of two, so
//     they cannot feed the block-scaled FP4 tensor cores;
//   * E8M0 weights when the caller wants the reference's literal numerics (no activation quantisation) at the price of
//     the bf16 tensor rate (a quarter of the FP4 rate).
// The weight never exists in dequantised form in global memory: two groups of eight decoder warps take alternate K
// stages, so that one group's waits (copies, barriers, the proxy fence) overlap the other's arithmetic.  A thread fetches
// the packed codes and scales of its (row, 32-element block) with cp.async into a private ring in shared memory, kAhead
// of its group's stages ahead, builds its part of the bf16 tile in shared memory in the 128-byte-swizzled layout the
// tensor core reads (integer assembly of the levels, one bf16x2 multiply by the scale), and the group hands the tile to
// the MMA thread through an mbarrier.  Activations arrive by TMA.  Accumulators are double-buffered in tensor memory (no
// scale factors live there for kind::f16), so the epilogue of a tile overlaps the next tile's MMAs.
// Tile: 128 weight rows (MMA M) x BN activation rows (MMA N) x 64 elements of K per stage (one 128-byte swizzle span of
// bf16), 4 MMAs of K = 16 per stage.  Persistent grid, one CTA per SM.  Every wait is bounded as in the FP4 kernels.
#include <atomic>
#include "gemm_mxf4_tc.cuh"

namespace mxfp4 {
namespace {

constexpr int kWThreads = 704;      // warps: 0 TMA producer, 1 MMA issuer (owns tensor memory), 2-17 weight decoders, 18-21 epilogue
constexpr int kWStageK = 64;        // elements of K per stage

constexpr int kGroups = 2;          // decoder groups: group g decodes the K stages with index = g (mod kGroups)
constexpr int kGroupThreads = 256;  // per group: (weight row of the tile, which 32-element block of the stage)
constexpr int kDecoders = kGroups * kGroupThreads;
constexpr int kAhead = 2;           // stages OF ITS GROUP between a thread's request for its scales and their use

// (Two 128-row weight tiles against one 128-row activation tile would need a third less L2 traffic than 128 x 256, but
// measured 527 against 891 TFLOP/s on [8192, 11008, 4096]: MMAs of 128 columns read their operands from shared memory at
// twice the rate per flop.)
template <int BN>
struct WCfg {
    static constexpr int kABytes = kTileW * 128;                 // decoded weight tile: 128 rows x 64 bf16
    static constexpr int kBBytes = BN * 128;                     // activation tile: BN rows x 64 bf16
    static constexpr int kCBytes = kTileW * (kWStageK / 2);      // packed codes of the weight tile: 128 rows x 32 bytes
    static constexpr int kStageBytes = kABytes + kBBytes + kCBytes;
    static constexpr int kFetchBytes = kAhead * kDecoders * 8;   // per thread and stage in flight: two words of scales
    static constexpr int kBudget = 227 * 1024 - 1024 - 512 - kFetchBytes;
    static constexpr int kStages = (kBudget / kStageBytes) < 6 ? (kBudget / kStageBytes) : 6;
    static constexpr int kSmemBytes = kStages * kStageBytes + kFetchBytes + 1024 + 512;
    static constexpr int kAccStride = 256;                       // two accumulators of up to 256 columns
    static_assert(BN % 32 == 0 && BN <= 256 && kStages >= 2 && kStageBytes % 1024 == 0, "tile width");
};

struct W4A16Params {
    const uint8_t* w_packed;    // [N, K/2]
    const void* w_scales;       // [N, K/block] uint8 (E8M0) or bf16
    int scale_fmt, block;
    const __nv_bfloat16* bias;
    __nv_bfloat16* out;
    int64_t ldo;
    int M, N, K;
    int kstages, n_tiles, m_tiles;
    int* status;
};

// Instruction descriptor of kind::f16 with bf16 operands and float32 accumulation: accumulator format F32 (=1) at [4,6),
// A and B format BF16 (=1) at [7,10) / [10,13), both K-major, N>>3 at [17,23), M>>4 at [24,29).
__device__ __forceinline__ uint32_t make_idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileW >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// A scale as a bf16 pair from its stored form (the E8M0 byte or the bf16 bit pattern).  Exact: a bf16 scale is taken as
// it is, 2^(byte-127) is a bf16 value for every byte (a subnormal one for byte 0, +inf for byte 255, as the reference's
// float32 scale cast to bf16 would be).
__device__ __forceinline__ __nv_bfloat162 scale_pair(int scale_fmt, uint32_t raw) {
    uint32_t bits = raw;
    if (scale_fmt == MXFP4_SF_E8M0) bits = raw == 0 ? 0x0040u : raw << 7;
    bits |= bits << 16;
    return *reinterpret_cast<const __nv_bfloat162*>(&bits);
}

__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

// Four code bytes (8 elements, even element in the high nibble) -> four bf16 pairs: bf16(level * scale), as the
// reference's dequantize() followed by the cast to the activations' dtype gives them.  The level of a code c = e<<1 | m
// is (1 + m/2) * 2^(e-1), whose bf16 pattern is 0x3F00 + (c << 6) with the nibble's sign bit moved to bit 15.  Two
// nibbles sit in the two 16-bit lanes of a word; one multiply by 0x1040 places copies at bit 6 and at bit 12 of each
// lane, a mask keeps magnitude and sign.  The product with the scale is one bf16x2 multiply: level and scale have at
// most 2 and 8 significant bits, so rounding the exact product once to bf16 is the float32 multiply followed by the
// cast.  The lanes hold elements (0,4), (1,5), (2,6), (3,7); byte permutes put neighbours side by side again.
__device__ __forceinline__ uint32_t levels_times_scale(uint32_t lanes, __nv_bfloat162 s2) {
    const uint32_t lv = ((lanes * 0x1040u) & 0x81C081C0u) + 0x3F003F00u;
    const __nv_bfloat162 y = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&lv), s2);
    return *reinterpret_cast<const uint32_t*>(&y);
}
__device__ __forceinline__ uint4 decode8(uint32_t w, __nv_bfloat162 s2) {
    const uint32_t r04 = levels_times_scale((w >> 4) & 0x000F000Fu, s2);
    const uint32_t r15 = levels_times_scale(w & 0x000F000Fu, s2);
    const uint32_t r26 = levels_times_scale((w >> 12) & 0x000F000Fu, s2);
    const uint32_t r37 = levels_times_scale((w >> 8) & 0x000F000Fu, s2);
    return make_uint4(__byte_perm(r04, r15, 0x5410), __byte_perm(r26, r37, 0x5410), __byte_perm(r04, r15, 0x7632), __byte_perm(r26, r37, 0x7632));
}

template <int BN>
__global__ void __launch_bounds__(kWThreads, 1) gemm_w4a16_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                                                                  const W4A16Params p) {
    using C = WCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // 128-byte swizzle wants 1024-byte aligned tiles
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t fetch = base + C::kStages * C::kStageBytes;    // [kAhead][512] x 8 bytes of scale words
    const uint32_t bars = fetch + C::kFetchBytes;
    auto x_full_bar = [&](int s) { return bars + 8u * s; };                        // the activation tile and the packed codes have landed (TMA bytes)
    auto w_ready_bar = [&](int s) { return bars + 8u * (C::kStages + s); };        // the eight decoder warps of the stage's group have written the weight tile
    auto empty_bar = [&](int s) { return bars + 8u * (2 * C::kStages + s); };      // the MMAs have finished with the stage
    auto acc_full_bar = [&](int b) { return bars + 8u * (3 * C::kStages + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (3 * C::kStages + 2 + b); };
    uint8_t* tail = base_ptr + C::kStages * C::kStageBytes + C::kFetchBytes + 8 * (3 * C::kStages + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_units = p.n_tiles * p.m_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(x_full_bar(s), 1);
            mbar_init(w_ready_bar(s), kGroupThreads / 32);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer: activation tiles
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
                const int m0 = (u / p.n_tiles) * BN, n0 = (u % p.n_tiles) * kTileW;
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(x_full_bar(s), C::kBBytes + C::kCBytes);
                    tma_load_2d(base + s * C::kStageBytes + C::kABytes + C::kBBytes, &map_w, x_full_bar(s), ks * (kWStageK / 2), n0);
                    tma_load_2d(base + s * C::kStageBytes + C::kABytes, &map_x, x_full_bar(s), ks * kWStageK, m0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16(BN);
            uint32_t it = 0;
            int i = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
                const int buf = i & 1;
                const uint32_t acc = tmem + buf * C::kAccStride;
                ok = mbar_wait(acc_empty_bar(buf), (((uint32_t)i >> 1) & 1u) ^ 1u, abort_flag);     // the epilogue has drained this accumulator
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    ok = mbar_wait(x_full_bar(s), ph, abort_flag) && mbar_wait(w_ready_bar(s), ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = base + s * C::kStageBytes;
                    const uint64_t adesc = desc_sw128(st), bdesc = desc_sw128(st + C::kABytes);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint64_t adv = (uint64_t)(kb * 32 >> 4);            // 16 bf16 = 32 bytes along K
                        tc_mma_bf16(acc, adesc + adv, bdesc + adv, idesc, (ks > 0 || kb > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));
                }
                tc_commit(acc_full_bar(buf));
            }
        }
        __syncwarp();
    } else if (warp < 2 + kDecoders / 32) {
        // ------------------------------------------------------------------ weight decoders: packed codes + scales -> bf16 tile
        const int group = (warp - 2) / (kGroupThreads / 32);
        const int t = (warp - 2) * 32 + lane;                                      // 0..511: slot in the fetch rings
        const int tg = t - group * kGroupThreads;
        const int row = tg >> 1, half = tg & 1;        // which weight row of the tile, which 32-element block of the stage
        const int block_shift = p.block == 16 ? 4 : (p.block == 32 ? 5 : 6);
        const int sbytes = p.scale_fmt == MXFP4_SF_E8M0 ? 1 : 2;
        const int slen = (block_shift == 4 ? 2 : 1) * sbytes;                      // bytes of scales per thread and stage: 1, 2 or 4
        const uint32_t scale_ring = fetch + (uint32_t)t * 8u;
        auto scale_slot = [&](int j) { return scale_ring + (uint32_t)(j * kDecoders * 8); };
        // weight row of unit u this thread decodes, p.N (outside) when the CTA has no such unit
        auto unit_row = [&](int u) { return u < total_units ? (u % p.n_tiles) * kTileW + row : p.N; };
        // byte offset of the first scale of element k0 within the row's scales
        auto scale_off = [&](int k0) { return (uint32_t)((k0 >> block_shift) * sbytes); };
        const uintptr_t sbase = reinterpret_cast<uintptr_t>(p.w_scales);
        const int64_t srow = (int64_t)(p.K >> block_shift) * sbytes;              // bytes of scales per weight row

        // A cursor over this group's stages: (unit, stage of the unit), kGroups stages of the CTA's sequence per step.
        struct Cursor { int u, ks, row; };
        auto advance = [&](Cursor& c) {
            c.ks += kGroups;
            while (c.ks >= p.kstages && c.u < total_units) {
                c.ks -= p.kstages;
                c.u += gridDim.x;
                c.row = unit_row(c.u);
            }
        };
        Cursor rq{(int)blockIdx.x, 0, unit_row(blockIdx.x)};       // request cursor, kAhead steps ahead of the decode cursor
        rq.ks = group - kGroups;
        advance(rq);
        Cursor dc = rq;                                             // decode cursor
        // The packed codes of a stage arrive by TMA with the activations; a thread fetches its own scales with cp.async,
        // kAhead steps ahead.  One copy group per step, empty for blocks outside the matrix, so that "all but the newest
        // kAhead-1 groups are complete" always means "the scales of the stage to decode are here".
        auto request = [&](int j) {
            const int k0 = rq.ks * kWStageK + half * 32;
            if (rq.row < p.N && k0 < p.K) {
                // the aligned word holding the first scale byte, and the next one only where the bytes run into it
                const uintptr_t a = sbase + (uintptr_t)(rq.row * srow) + scale_off(k0), a0 = a & ~(uintptr_t)3;
                cp_async_4(scale_slot(j), reinterpret_cast<const void*>(a0));
                if ((a & 3) + slen > 4) cp_async_4(scale_slot(j) + 4, reinterpret_cast<const void*>(a0 + 4));
            }
            cp_async_commit();
            advance(rq);
        };
#pragma unroll
        for (int j = 0; j < kAhead; ++j) request(j);

        const int my_units = blockIdx.x < total_units ? (total_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const uint32_t my_stages = (uint32_t)my_units * (uint32_t)p.kstages;       // of the whole CTA; this group takes every kGroups-th
        bool ok = true;
        for (uint32_t it0 = group; it0 < my_stages && ok; it0 += kGroups * kAhead) {
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const uint32_t it = it0 + j * kGroups;
                if (it >= my_stages) break;
                cp_async_wait<kAhead - 1>();
                const int k0 = dc.ks * kWStageK + half * 32;
                const bool valid = dc.row < p.N && k0 < p.K;        // rows past N and blocks past K decode to zero
                uint32_t raw0 = 0, raw1 = 0;
                if (valid) {
                    uint32_t w0, w1;
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(scale_slot(j)) : "memory");
                    const uint32_t a_lo = (uint32_t)(sbase + (uintptr_t)(dc.row * srow)) + scale_off(k0);
                    // this thread's scale bytes, first one lowest (w1 is only meaningful where the bytes run into it)
                    const uint32_t v = __funnelshift_r(w0, w1, (a_lo & 3u) * 8u);
                    raw0 = sbytes == 1 ? (v & 0xFFu) : (v & 0xFFFFu);
                    raw1 = block_shift != 4 ? raw0 : (sbytes == 1 ? ((v >> 8) & 0xFFu) : (v >> 16));
                }
                __nv_bfloat162 s0 = scale_pair(p.scale_fmt, raw0), s1 = scale_pair(p.scale_fmt, raw1);
                if (!valid) s0 = s1 = __float2bfloat162_rn(0.0f);
                advance(dc);
                const int s = it % C::kStages;
                const uint32_t ph = (it / C::kStages) & 1;
                // the stage's TMA loads are issued only after its previous MMAs have finished (the producer waits for
                // that), so once the codes are here the decoded tile may be overwritten too
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(x_full_bar(s), ph, abort_flag));
                if (!ok) break;
                uint4 codes;        // [128 rows][32 bytes], as the TMA wrote them (rows past N and bytes past K/2 are zero)
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(codes.x), "=r"(codes.y), "=r"(codes.z), "=r"(codes.w)
                             : "r"(base + s * C::kStageBytes + C::kABytes + C::kBBytes + tg * 16) : "memory");
                uint8_t* dst = base_ptr + s * C::kStageBytes + row * 128;
                const uint32_t cw[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
                for (int c = 0; c < 4; ++c)     // 16-byte chunk index within the 128-byte row, swizzled with the row's position in its group of eight
                    *reinterpret_cast<uint4*>(dst + (((half * 4 + c) ^ (row & 7)) << 4)) = decode8(cw[c], c < 2 ? s0 : s1);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(w_ready_bar(s));
                request(j);                             // the scale slot just read takes the step kAhead further on
            }
        }
        cp_async_wait<0>();
    } else {
        // ------------------------------------------------------------------ epilogue
        // A thread holds weight row n (its lane of tensor memory) for 32 activation rows: out[m][n0 + lane] makes every
        // store of a warp one 64-byte run.
        const int q = warp & 3;                               // tensor-memory lane quarter this warp may read
        const bool has_bias = p.bias != nullptr;
        int i = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
            const int buf = i & 1;
            ok = mbar_wait(acc_full_bar(buf), ((uint32_t)i >> 1) & 1u, abort_flag);
            ok = __all_sync(0xFFFFFFFFu, ok && !*abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int n = (u % p.n_tiles) * kTileW + q * 32 + lane;
            const int mt = (u / p.n_tiles) * BN;
            const float bias = (has_bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const int m0 = mt + c0;
                if (m0 >= p.M) {
                    if (c0 == 0) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(acc_empty_bar(buf)); }
                    break;
                }
                uint32_t v[32];
                tc_ld_32x32(tmem + buf * C::kAccStride + ((uint32_t)(q * 32) << 16) + c0, v);
                if (c0 + 32 >= BN || m0 + 32 >= p.M) {            // last read of this accumulator: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
                if (n < p.N) {
                    __nv_bfloat16* o = p.out + (int64_t)m0 * p.ldo + n;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (m0 + j < p.M) {
                            __nv_bfloat16 y = __float2bfloat16_rn(__uint_as_float(v[j]));
                            if (has_bias) y = __float2bfloat16_rn(__bfloat162float(y) + bias);   // `output += bias` in bf16
                            o[(int64_t)j * p.ldo] = y;
                        }
                    }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static std::atomic<EncodeTiledFn> fn{nullptr};
    if (!fn.load()) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn.store((EncodeTiledFn)f);
    }
    return fn.load();
}

// bf16 matrix [rows, cols] with row pitch ld elements, boxes of 64 elements (128 bytes) x box_rows, 128-byte swizzle,
// out-of-range parts of a box read as zero
int make_x_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MXFP4_E_CUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)kWStageK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (bf16 activations) failed with CUresult %d", (int)r); return MXFP4_E_CUDA; }
    return MXFP4_OK;
}

// packed codes [rows, row_bytes] uint8, boxes of 32 bytes (64 codes) x 128 rows, no swizzle, out-of-range parts read as zero
int make_w_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t row_bytes) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from this driver"); return MXFP4_E_CUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(kWStageK / 2), (cuuint32_t)kTileW};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (packed codes) failed with CUresult %d", (int)r); return MXFP4_E_CUDA; }
    return MXFP4_OK;
}

template <int BN>
int launch_w4a16(const CUtensorMap& mx, const CUtensorMap& mw, W4A16Params& p, cudaStream_t st) {
    using C = WCfg<BN>;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm_w4a16: cudaFuncSetAttribute");
        configured[dev] = true;
    }
    p.m_tiles = (p.M + BN - 1) / BN;
    const int64_t units = (int64_t)p.n_tiles * p.m_tiles;
    const int grid = (int)(units < num_sms() ? units : num_sms());
    gemm_w4a16_kernel<BN><<<grid, kWThreads, C::kSmemBytes, st>>>(mx, mw, p);
    MXFP4_CHECK_LAUNCH("mxfp4_gemm_w4a16");
    return MXFP4_OK;
}

}  // namespace
}  // namespace mxfp4

extern "C" int mxfp4_gemm_w4a16(const void* x_bf16, int64_t ldx, const uint8_t* w_packed, const void* w_scales, int scale_fmt, int block_size,
                                const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M, int64_t N, int64_t K, int* status_dev,
                                void* stream) {
    using namespace mxfp4;
    if (M < 0 || N < 0 || K < 0) { set_error("mxfp4_gemm_w4a16: negative size"); return MXFP4_E_SHAPE; }
    if (M == 0 || N == 0) return MXFP4_OK;
    if (block_size != 16 && block_size != 32 && block_size != 64) { set_error("mxfp4_gemm_w4a16: block_size %d (16, 32 or 64)", block_size); return MXFP4_E_UNSUPPORTED; }
    if (K == 0 || K % 32 || K % block_size) { set_error("mxfp4_gemm_w4a16: K=%lld must be a positive multiple of 32 and of the block size", (long long)K); return MXFP4_E_SHAPE; }
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) { set_error("mxfp4_gemm_w4a16: dimension too large"); return MXFP4_E_SHAPE; }
    if (scale_fmt != MXFP4_SF_E8M0 && scale_fmt != MXFP4_SF_BF16) { set_error("mxfp4_gemm_w4a16: unknown scale format %d", scale_fmt); return MXFP4_E_BADARG; }
    if (!x_bf16 || !w_packed || !w_scales || !out_bf16) { set_error("mxfp4_gemm_w4a16: null pointer"); return MXFP4_E_BADARG; }
    if (ldx < K || ldo < N) { set_error("mxfp4_gemm_w4a16: ldx < K or ldo < N"); return MXFP4_E_SHAPE; }
    if ((uintptr_t)x_bf16 % 16 || (ldx * 2) % 16 || (uintptr_t)w_packed % 16 || (scale_fmt == MXFP4_SF_BF16 && (uintptr_t)w_scales % 2)) {
        set_error("mxfp4_gemm_w4a16: x and w_packed must be 16-byte aligned, the activations' row pitch a multiple of 16 bytes");
        return MXFP4_E_ALIGN;
    }
    W4A16Params p;
    p.w_packed = w_packed; p.w_scales = w_scales; p.scale_fmt = scale_fmt; p.block = block_size;
    p.bias = (const __nv_bfloat16*)bias_bf16; p.out = (__nv_bfloat16*)out_bf16; p.ldo = ldo;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.kstages = (int)((K + kWStageK - 1) / kWStageK);
    p.n_tiles = (int)((N + kTileW - 1) / kTileW); p.m_tiles = 0;
    p.status = status_dev;
    const int bn = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
    CUtensorMap mx;
    CUtensorMap mw;
    int rc = make_x_map(&mx, x_bf16, M, K, ldx, bn);
    if (rc) return rc;
    rc = make_w_map(&mw, w_packed, N, K / 2);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (bn) {
        case 32: return launch_w4a16<32>(mx, mw, p, st);
        case 64: return launch_w4a16<64>(mx, mw, p, st);
        case 128: return launch_w4a16<128>(mx, mw, p, st);
        default: return launch_w4a16<256>(mx, mw, p, st);
    }
}
