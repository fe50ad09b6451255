// Operand preparation for the block-scaled FP4 GEMM on sm_100a:
//   * mxfp4_act_quantize         bf16 activations -> packed hardware-E2M1 codes + E8M0 scales, the scales
//                                written directly in the tile order the tensor core's scale loader wants;
//   * mxfp4_prepare_weight_scales  re-tiles a weight's row-major E8M0 scale bytes into the same order and
//                                adds the "minus one" copy used by the correction pass.
//
// Scale tile order ("blocked"): the [rows, K/32] scale matrix is cut into tiles of 128 rows x 4 blocks
// (= 128 elements of K).  One tile is 512 contiguous bytes, byte offset (r%32)*16 + (r/32)*4 + c for row
// r and block c of the tile: exactly the 32-lane x 128-bit image that `tcgen05.cp.32x128b.warpx4`
// copies into tensor memory.  Tiles of one 128-row group are stored K-stage by K-stage (a stage is 256
// elements of K = 2 tiles = 1 KB); K is padded to whole stages and rows to whole groups with zero bytes
// (2^-127: finite, and multiplied by zero codes).
#include "mxfp4_common.cuh"

namespace mxfp4 {
namespace {

__device__ __forceinline__ void ld_256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Two floats -> one byte of hardware E2M1 (round to nearest even, saturating); `hi` lands in the high nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
    uint16_t o;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(o) : "f"(hi), "f"(lo));
    return o;
}

__device__ __forceinline__ int64_t blocked_offset(int64_t row, int64_t kb, int64_t kstages, int64_t stage_bytes) {
    return ((row >> 7) * kstages + (kb >> 3)) * stage_bytes + ((kb >> 2) & 1) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3);
}

// One thread per (row, 32-element block) of the padded [m_pad, kstages*8] block grid.
__global__ void __launch_bounds__(256) act_quantize_kernel(const uint8_t* __restrict__ x, int64_t M, int64_t kblocks, int64_t ld_bytes,
                                                           int64_t m_pad, int64_t kstages, uint8_t* __restrict__ packed,
                                                           uint8_t* __restrict__ sf) {
    // a GEMM launched behind this kernel with programmatic stream serialisation may start its set-up and weight loads now
    // (it waits for this grid's results with griddepcontrol.wait before it touches them)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t kb_pad = kstages * 8;
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= m_pad * kb_pad) return;
    int64_t row, kb;
    if (m_pad * kb_pad < 0x7FFFFFFFll) {
        // 32-bit index arithmetic whenever the block grid allows it: a 64-bit division per thread costs about as many
        // instructions as the rest of the kernel
        const uint32_t r32 = (uint32_t)idx / (uint32_t)kb_pad;
        row = r32;
        kb = (uint32_t)idx - r32 * (uint32_t)kb_pad;
    } else {
        row = idx / kb_pad;
        kb = idx - row * kb_pad;
    }
    uint32_t byte = 0;
    if (row < M && kb < kblocks) {
        uint32_t w[16];
        {
            uint32_t lo[8], hi[8];
            const uint8_t* p = x + row * ld_bytes + kb * 64;
            ld_256(p, lo);
            ld_256(p + 32, hi);
#pragma unroll
            for (int i = 0; i < 8; ++i) { w[i] = lo[i]; w[8 + i] = hi[i]; }
        }
        __nv_bfloat162 m2 = __habs2(as_bf162(w[0]));
#pragma unroll
        for (int i = 1; i < 16; ++i) m2 = __hmax2(m2, __habs2(as_bf162(w[i])));
        const uint32_t mb = as_u32(m2);
        const uint32_t amax16 = max(mb & 0xFFFFu, mb >> 16);
        // scale = 2^ceil(log2(amax/6)): exponent E-2, plus one when the mantissa exceeds 1.5
        int b = (int)(amax16 >> 7) - 2 + ((amax16 & 0x7Fu) > 0x40u ? 1 : 0);
        b = b < 0 ? 0 : (b > 254 ? 254 : b);
        byte = (uint32_t)b;
        const float inv = b == 0 ? __uint_as_float(0x7F000000u) : (b == 254 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(254 - b) << 23));
        uint32_t out[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t v = w[4 * g + j];
                const float even = __uint_as_float(v << 16) * inv;           // element 2i   (low half of the register)
                const float odd = __uint_as_float(v & 0xFFFF0000u) * inv;    // element 2i+1
                word |= cvt_e2m1x2(even, odd) << (8 * j);                    // even element in the high nibble
            }
            out[g] = word;
        }
        *reinterpret_cast<uint4*>(packed + row * (kblocks * 16) + kb * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    }
    sf[blocked_offset(row, kb, kstages, 1024)] = (uint8_t)byte;
}

// One thread per (row, block) of the padded grid of a weight's scales.
__global__ void __launch_bounds__(256) prepare_weight_scales_kernel(const uint8_t* __restrict__ scales, int64_t N, int64_t kblocks,
                                                                    int64_t n_pad, int64_t kstages, uint8_t* __restrict__ out) {
    const int64_t kb_pad = kstages * 8;
    const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (idx >= n_pad * kb_pad) return;
    const int64_t row = idx / kb_pad, kb = idx - row * kb_pad;
    uint32_t b = 0;
    if (row < N && kb < kblocks) b = scales[row * kblocks + kb];
    const int64_t off = blocked_offset(row, kb, kstages, 2048);
    out[off] = (uint8_t)b;                             // pass 1: the stored scale
    out[off + 1024] = (uint8_t)(b > 0 ? b - 1 : 0);    // pass 2: half of it
}

}  // namespace
}  // namespace mxfp4

extern "C" int64_t mxfp4_act_scales_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0) return 0;
    return ((M + 127) / 128) * ((K + 255) / 256) * 1024;
}

extern "C" int64_t mxfp4_prepared_scales_bytes(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0) return 0;
    return ((N + 127) / 128) * ((K + 255) / 256) * 2048;
}

extern "C" int mxfp4_act_quantize(const void* x_bf16, int64_t M, int64_t K, int64_t ld, uint8_t* a_packed, uint8_t* a_sf_blocked,
                                  void* stream) {
    using namespace mxfp4;
    if (M < 0 || K < 0) { set_error("mxfp4_act_quantize: negative size"); return MXFP4_E_SHAPE; }
    if (M == 0 || K == 0) return MXFP4_OK;
    if (K % 32) { set_error("mxfp4_act_quantize: K=%lld is not a multiple of 32", (long long)K); return MXFP4_E_SHAPE; }
    if (!x_bf16 || !a_packed || !a_sf_blocked) { set_error("mxfp4_act_quantize: null pointer"); return MXFP4_E_BADARG; }
    if (ld < K) { set_error("mxfp4_act_quantize: ld < K"); return MXFP4_E_SHAPE; }
    if ((uintptr_t)x_bf16 % 32 || (ld * 2) % 32 || (uintptr_t)a_packed % 16) {
        set_error("mxfp4_act_quantize: x must be 32-byte aligned with a row pitch that is a multiple of 32 bytes, a_packed 16-byte aligned");
        return MXFP4_E_ALIGN;
    }
    const int64_t m_pad = (M + 127) / 128 * 128, kstages = (K + 255) / 256;
    const int64_t total = m_pad * kstages * 8;
    const int threads = 256;
    const int64_t grid = (total + threads - 1) / threads;
    if (grid > 0x7FFFFFFF) { set_error("mxfp4_act_quantize: too large"); return MXFP4_E_SHAPE; }
    act_quantize_kernel<<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>((const uint8_t*)x_bf16, M, K / 32, ld * 2, m_pad, kstages,
                                                                               a_packed, a_sf_blocked);
    MXFP4_CHECK_LAUNCH("mxfp4_act_quantize");
    return MXFP4_OK;
}

extern "C" int mxfp4_prepare_weight_scales(const uint8_t* scales, int64_t N, int64_t K, uint8_t* prepared, void* stream) {
    using namespace mxfp4;
    if (N < 0 || K < 0) { set_error("mxfp4_prepare_weight_scales: negative size"); return MXFP4_E_SHAPE; }
    if (N == 0 || K == 0) return MXFP4_OK;
    if (K % 32) { set_error("mxfp4_prepare_weight_scales: K=%lld is not a multiple of 32", (long long)K); return MXFP4_E_SHAPE; }
    if (!scales || !prepared) { set_error("mxfp4_prepare_weight_scales: null pointer"); return MXFP4_E_BADARG; }
    const int64_t n_pad = (N + 127) / 128 * 128, kstages = (K + 255) / 256;
    const int64_t total = n_pad * kstages * 8;
    const int threads = 256;
    const int64_t grid = (total + threads - 1) / threads;
    if (grid > 0x7FFFFFFF) { set_error("mxfp4_prepare_weight_scales: too large"); return MXFP4_E_SHAPE; }
    prepare_weight_scales_kernel<<<(unsigned)grid, threads, 0, (cudaStream_t)stream>>>(scales, N, K / 32, n_pad, kstages, prepared);
    MXFP4_CHECK_LAUNCH("mxfp4_prepare_weight_scales");
    return MXFP4_OK;
}
