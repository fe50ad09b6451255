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
// The weight never exists in dequantised form in global memory: eight transform warps read the packed codes and scales
// straight from global memory (one 32-element block per thread and K stage, the next stage's loads in flight while the
// current one is decoded), build the bf16 tile in shared memory in the 128-byte-swizzled layout the tensor core reads, and
// hand it to the MMA thread through an mbarrier.  Activations arrive by TMA.  Accumulators are double-buffered in tensor
// memory (no scale factors live there for kind::f16), so the epilogue of a tile overlaps the next tile's MMAs.
// Tile: WT x 128 weight rows (MMA M = 128 each) x BN activation rows (MMA N) x 64 elements of K per stage (one 128-byte
// swizzle span of bf16), 4 x WT MMAs of K = 16 per stage.  Persistent grid, one CTA per SM.  Every wait is bounded as in the FP4 kernels.
#include <atomic>
#include "gemm_mxf4_tc.cuh"

namespace mxfp4 {
namespace {

constexpr int kWThreads = 448;      // warps: 0 TMA producer, 1 MMA issuer (owns tensor memory), 2-9 weight decoders, 10-13 epilogue
constexpr int kWStageK = 64;        // elements of K per stage

// WT weight tiles of 128 rows share one activation tile.  Only WT = 1 is instantiated: two weight tiles against a
// 128-row activation tile need a third less L2 traffic than one against 256 rows, but measured 527 against 891 TFLOP/s
// on [8192, 11008, 4096] (MMAs of 128 columns read their operands from shared memory at twice the rate per flop).
template <int BN, int WT>
struct WCfg {
    static constexpr int kABytes = kTileW * 128;                 // one decoded weight tile: 128 rows x 64 bf16
    static constexpr int kBBytes = BN * 128;                     // activation tile: BN rows x 64 bf16
    static constexpr int kStageBytes = WT * kABytes + kBBytes;
    static constexpr int kEpiBytes = 4 * 4096;
    static constexpr int kBudget = 227 * 1024 - 1024 - 512 - kEpiBytes;
    static constexpr int kStages = (kBudget / kStageBytes) < 6 ? (kBudget / kStageBytes) : 6;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + 512;
    static constexpr int kAccStride = 256;                       // two accumulators of up to 256 columns
    static_assert(BN % 32 == 0 && WT * BN <= 256 && kStages >= 2 && kStageBytes % 1024 == 0, "tile width");
};

struct W4A16Params {
    const uint8_t* w_packed;    // [N, K/2]
    const void* w_scales;       // [N, K/block] uint8 (E8M0) or bf16
    int scale_fmt, block;
    const __nv_bfloat16* bias;
    __nv_bfloat16* out;
    int64_t ldo;
    int M, N, K;
    int kstages, n_tiles, n_supers, m_tiles;      // n_supers: groups of WT weight tiles
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

// what one decoder thread needs for one (row, 32-element block) of a stage
struct WBlock {
    uint4 codes;               // 16 bytes = 32 codes
    __nv_bfloat162 s0, s1;     // scale of elements 0-15 and 16-31 in both halves (they differ only for block_size 16)
};

// A scale as a bf16 pair.  Exact: a bf16 scale is taken as it is, 2^(byte-127) is a bf16 value for every byte (a
// subnormal one for byte 0).
__device__ __forceinline__ __nv_bfloat162 scale_pair(const W4A16Params& p, int64_t idx) {
    if (p.scale_fmt == MXFP4_SF_E8M0) return __float2bfloat162_rn(e8m0_value(__ldg(reinterpret_cast<const uint8_t*>(p.w_scales) + idx)));
    return __bfloat162bfloat162(__ldg(reinterpret_cast<const __nv_bfloat16*>(p.w_scales) + idx));
}

// k0: first element of the block, a multiple of 32; block_shift = log2(block size)
__device__ __forceinline__ WBlock load_wblock(const W4A16Params& p, int block_shift, int n, int k0) {
    WBlock b;
    b.codes = make_uint4(0, 0, 0, 0);
    b.s0 = b.s1 = __float2bfloat162_rn(0.0f);             // rows past N and blocks past K decode to zero
    if (n < p.N && k0 < p.K) {
        b.codes = __ldg(reinterpret_cast<const uint4*>(p.w_packed + (int64_t)n * (p.K >> 1) + (k0 >> 1)));
        const int64_t first = (int64_t)n * (p.K >> block_shift) + (k0 >> block_shift);
        b.s0 = scale_pair(p, first);
        b.s1 = block_shift == 4 ? scale_pair(p, first + 1) : b.s0;
    }
    return b;
}

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

template <int BN, int WT>
__global__ void __launch_bounds__(kWThreads, 1) gemm_w4a16_kernel(const __grid_constant__ CUtensorMap map_x, const W4A16Params p) {
    using C = WCfg<BN, WT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // 128-byte swizzle wants 1024-byte aligned tiles
    uint8_t* base_ptr = smem_raw + (base - raw);
    uint8_t* epi_ptr = base_ptr + C::kStages * C::kStageBytes;
    const uint32_t bars = base + C::kStages * C::kStageBytes + C::kEpiBytes;
    auto x_full_bar = [&](int s) { return bars + 8u * s; };                        // the activation tile has landed (TMA bytes)
    auto w_ready_bar = [&](int s) { return bars + 8u * (C::kStages + s); };        // the eight decoder warps have written the weight tile
    auto empty_bar = [&](int s) { return bars + 8u * (2 * C::kStages + s); };      // the MMAs have finished with the stage
    auto acc_full_bar = [&](int b) { return bars + 8u * (3 * C::kStages + b); };
    auto acc_empty_bar = [&](int b) { return bars + 8u * (3 * C::kStages + 2 + b); };
    uint8_t* tail = epi_ptr + C::kEpiBytes + 8 * (3 * C::kStages + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(tail);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_units = p.n_supers * p.m_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(x_full_bar(s), 1);
            mbar_init(w_ready_bar(s), 8);
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
                const int m0 = (u / p.n_supers) * BN;
                for (int ks = 0; ks < p.kstages; ++ks, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(x_full_bar(s), C::kBBytes);
                    tma_load_2d(base + s * C::kStageBytes + WT * C::kABytes, &map_x, x_full_bar(s), ks * kWStageK, m0);
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
                    const uint64_t bdesc = desc_sw128(st + WT * C::kABytes);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint64_t adv = (uint64_t)(kb * 32 >> 4);            // 16 bf16 = 32 bytes along K
#pragma unroll
                        for (int w = 0; w < WT; ++w)                              // weight tile w accumulates into columns [w*BN, (w+1)*BN)
                            tc_mma_bf16(acc + w * BN, desc_sw128(st + w * C::kABytes) + adv, bdesc + adv, idesc, (ks > 0 || kb > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));
                }
                tc_commit(acc_full_bar(buf));
            }
        }
        __syncwarp();
    } else if (warp < 10) {
        // ------------------------------------------------------------------ weight decoders: packed codes + scales -> bf16 tile
        const int t = (warp - 2) * 32 + lane;          // 0..255
        const int row = t >> 1, half = t & 1;          // which weight row of the tile, which 32-element block of the stage
        const int block_shift = p.block == 16 ? 4 : (p.block == 32 ? 5 : 6);
        // Codes and scales are requested kAhead stages before they are decoded (a ring in registers): one stage of
        // decoding is far shorter than the latency of these 16-byte loads with a row pitch of K/2 bytes.
        constexpr int kAhead = 4;
        WBlock ring[kAhead][WT];
        int pu = blockIdx.x, pks = 0;                  // unit and stage the next request is for
        int prow0 = pu < total_units ? (pu % p.n_supers) * WT * kTileW + row : p.N;      // this thread's row in that unit's first weight tile
        auto request = [&](WBlock (&dst)[WT]) {
#pragma unroll
            for (int w = 0; w < WT; ++w) dst[w] = load_wblock(p, block_shift, prow0 < p.N ? prow0 + w * kTileW : p.N, pks * kWStageK + half * 32);
            if (++pks == p.kstages) {
                pks = 0;
                pu += gridDim.x;
                prow0 = pu < total_units ? (pu % p.n_supers) * WT * kTileW + row : p.N;
            }
        };
#pragma unroll
        for (int j = 0; j < kAhead; ++j) request(ring[j]);
        const int my_units = blockIdx.x < total_units ? (total_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const uint32_t my_stages = (uint32_t)my_units * (uint32_t)p.kstages;
        bool ok = true;
        for (uint32_t it0 = 0; it0 < my_stages && ok; it0 += kAhead) {
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const uint32_t it = it0 + j;
                if (it >= my_stages) break;
                const int s = it % C::kStages;
                const uint32_t ph = (it / C::kStages) & 1;
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(empty_bar(s), ph ^ 1u, abort_flag));
                if (!ok) break;
#pragma unroll
                for (int w = 0; w < WT; ++w) {
                    uint8_t* tile = base_ptr + s * C::kStageBytes + w * C::kABytes;
                    const WBlock& blk = ring[j][w];
                    const uint32_t cw[4] = {blk.codes.x, blk.codes.y, blk.codes.z, blk.codes.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        // 16-byte chunk index within the 128-byte row, swizzled with the row's position in its group of eight
                        const int chunk = half * 4 + c;
                        *reinterpret_cast<uint4*>(tile + row * 128 + ((chunk ^ (row & 7)) << 4)) = decode8(cw[c], c < 2 ? blk.s0 : blk.s1);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(w_ready_bar(s));
                request(ring[j]);                       // the slot just decoded takes the stage kAhead further on
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;                               // tensor-memory lane quarter this warp may read
        uint32_t* tile = reinterpret_cast<uint32_t*>(epi_ptr + (warp - 10) * 4096);
        const bool has_bias = p.bias != nullptr;
        int i = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++i) {
            const int buf = i & 1;
            ok = mbar_wait(acc_full_bar(buf), ((uint32_t)i >> 1) & 1u, abort_flag);
            ok = __all_sync(0xFFFFFFFFu, ok && !*abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int mt = (u / p.n_supers) * BN;
#pragma unroll 1
            for (int cc = 0; cc < WT * BN; cc += 32) {
                const int w = cc / BN, c0 = cc - w * BN;          // weight tile and column inside its accumulator
                const int n0 = ((u % p.n_supers) * WT + w) * kTileW + q * 32;
                const int n = n0 + lane;
                const float bias = (has_bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
                const int m0 = mt + c0;
                const bool last = cc + 32 >= WT * BN;             // last read of this accumulator: hand it back
                if (m0 >= p.M) {                                   // activation rows past M: nothing to store
                    if (last) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(acc_empty_bar(buf)); }
                    continue;
                }
                uint32_t v[32];
                tc_ld_32x32(tmem + buf * C::kAccStride + ((uint32_t)(q * 32) << 16) + cc, v);
                if (last) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar(buf));
                }
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
                    const int rw = r * 8 + (lane >> 2), seg = lane & 3;
                    const int m = m0 + rw;
                    if (m < p.M) {
                        if (vec) {
                            *reinterpret_cast<uint4*>(p.out + (int64_t)m * p.ldo + n0 + seg * 8) = *reinterpret_cast<const uint4*>(t16 + rw * 32 + seg * 8);
                        } else {
                            for (int e = 0; e < 8; ++e)
                                if (n0 + seg * 8 + e < p.N) p.out[(int64_t)m * p.ldo + n0 + seg * 8 + e] = t16[rw * 32 + seg * 8 + e];
                        }
                    }
                }
                __syncwarp();
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

// bf16 matrix [rows, cols] with row pitch ld elements, boxes of 64 elements (128 bytes) x box_rows, 128-byte swizzle,
// out-of-range parts of a box read as zero
int make_x_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    static std::atomic<EncodeTiledFn> fn{nullptr};
    if (!fn.load()) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn.store((EncodeTiledFn)f);
    }
    EncodeTiledFn enc = fn.load();
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

template <int BN, int WT>
int launch_w4a16(const CUtensorMap& mx, W4A16Params& p, cudaStream_t st) {
    using C = WCfg<BN, WT>;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_w4a16_kernel<BN, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(e, "mxfp4_gemm_w4a16: cudaFuncSetAttribute");
        configured[dev] = true;
    }
    p.m_tiles = (p.M + BN - 1) / BN;
    p.n_supers = (p.n_tiles + WT - 1) / WT;
    const int64_t units = (int64_t)p.n_supers * p.m_tiles;
    const int grid = (int)(units < num_sms() ? units : num_sms());
    gemm_w4a16_kernel<BN, WT><<<grid, kWThreads, C::kSmemBytes, st>>>(mx, p);
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
    p.n_tiles = (int)((N + kTileW - 1) / kTileW); p.m_tiles = 0; p.n_supers = 0;
    p.status = status_dev;
    const int bn = M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256));
    CUtensorMap mx;
    int rc = make_x_map(&mx, x_bf16, M, K, ldx, bn);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (bn) {
        case 32: return launch_w4a16<32, 1>(mx, p, st);
        case 64: return launch_w4a16<64, 1>(mx, p, st);
        case 128: return launch_w4a16<128, 1>(mx, p, st);
        default: return launch_w4a16<256, 1>(mx, p, st);
    }
}
