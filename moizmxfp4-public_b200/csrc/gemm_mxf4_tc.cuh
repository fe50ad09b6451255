// Shared pieces of the tcgen05 GEMM kernels: PTX wrappers (mbarrier, TMA, tcgen05), operand and instruction
// descriptors, the correction-code transform, kernel parameters and the work-unit walk.
#pragma once
#include <cuda.h>

#include "mxfp4_common.cuh"

namespace mxfp4 {

struct GemmParams {
    const uint8_t* sfw;     // prepared weight scales
    const uint8_t* sfx;     // blocked activation scales
    const __nv_bfloat16* bias;
    __nv_bfloat16* out;     // [M, ldo] bf16 (ksplit == 1)
    float* partial;         // [ksplit, M, N] float32 (ksplit > 1)
    int64_t ldo;
    int M, N, K;
    int kstages;            // ceil(K / 256)
    int ksplit;             // K is cut into this many ranges of whole stages, one work unit each
    int n_tiles, m_tiles;
    int exact;
    int pdl;                // launched behind the activation quantiser with programmatic stream serialisation
    int* status;
    int tma_store;          // cta_group::2 kernel: the output goes out as TMA tile stores (map_out is valid)
};

// cta_group::2 kernel (gemm_mxf4_pair.cu): tile widths 128, 192, 256; the activation map's box holds bn/2 rows
// map_out: bf16 [M, ldo] with 32 x 32 boxes; used when p.tma_store is set
int launch_gemm_pair(int bn, const CUtensorMap& map_w, const CUtensorMap& map_x, const CUtensorMap& map_out, GemmParams& p, cudaStream_t stream);

// kernel with the activations on the MMA's M side (gemm_mxf4_swap.cu), for M <= 128: map_w holds 256-row boxes, map_x
// 128-row boxes, p.n_tiles counts 256-row weight tiles
int launch_gemm_swap(const CUtensorMap& map_w, const CUtensorMap& map_x, GemmParams& p, cudaStream_t stream);

namespace {

constexpr int kTileW = 128;         // weight rows per CTA (MMA M)
constexpr int kStageK = 256;        // elements of K per pipeline stage
constexpr int kStageKBytes = 128;   // bytes per row per stage
constexpr long long kWaitLimitCycles = 2000000000ll;   // about one second: a wait that long has failed

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA's abort flag) when the limit is reached or another
// role has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    // try_wait suspends the thread in hardware until the phase completes or a short time limit passes, so a plain
    // retry loop wakes up with the lowest latency; the abort flag and the bound are looked at every 64 retries.
    // (An explicit, longer suspend-time hint cut the polling instructions but cost 1 % on large problems.)
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) break;
        }
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t tmem_addr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
        "%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major operand tile whose rows are 128 bytes, 128-byte swizzle:
// 8-row groups 1024 bytes apart.  Fields: start>>4 [0,14) | LBO>>4 [16,30) | SBO>>4 [32,46) |
// version=1 [46,48) | layout [61,64) with 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Descriptor of one 512-byte scale tile (32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor for kind::mxf4 (block-scaled): A/B format E2M1 (=1) at [7,10)/[10,13), both
// K-major, N>>3 at [17,23), scale format UE8M0 (=1) at bit 23, M>>4 at [24,29), scale-factor byte
// selectors for B at [4,6) and A at [29,31) (0 or 2: which half of the 4 scale bytes per row), K=64.
__device__ __forceinline__ uint32_t make_idesc(int n, uint32_t sf_id) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(kTileW >> 4) << 24) | (sf_id << 29) | (sf_id << 4);
}

// corr nibble = sign | (code==0 ? 2 : code==1 ? 1 : 0), eight nibbles at a time
__device__ __forceinline__ uint32_t corr_word(uint32_t w) {
    const uint32_t e0 = ~((w >> 2) | (w >> 1)) & 0x11111111u;      // bit 0 of each nibble: exponent field is zero
    return (w & (e0 << 3)) | ((e0 & ~w) << 1) | (e0 & w);
}


constexpr int kThreads = 544;   // warps: 0 producer, 1 and 15 MMA issuers, 2-5 and 11-14 transform, 6-9 epilogue, 10 and 16 scale-factor copiers

// A work unit is (k-range, weight tile, activation tile); units are dealt round-robin to the CTAs of
// a persistent grid.  All roles walk the same unit sequence.
struct Unit {
    int n_tile, m_tile, ksp, ks0, ks1;
};
__device__ __forceinline__ Unit get_unit(const GemmParams& p, int u) {
    Unit w;
    w.ksp = u % p.ksplit;
    const int t = u / p.ksplit;
    w.n_tile = t % p.n_tiles;
    w.m_tile = t / p.n_tiles;
    w.ks0 = (int)((int64_t)p.kstages * w.ksp / p.ksplit);
    w.ks1 = (int)((int64_t)p.kstages * (w.ksp + 1) / p.ksplit);
    return w;
}

}  // namespace
}  // namespace mxfp4
