// BF16/FP16/FP32 -> MXFP4 block quantiser for sm_100a.
//
// Reproduces MXFP4Quantizer.quantize (reference: src/mxfp4/quantizer.py:71-141) bit for bit.
//
// Streaming kernel (bf16 input, 32-element blocks, contiguous rows): one thread owns one block.
// It reads its 64 bytes with two 256-bit loads (a warp covers 2 KB of contiguous input, every 32-byte
// sector fully used), keeps the block in registers, and writes one 128-bit word of codes (a warp
// writes 512 contiguous bytes) plus one scale byte (a warp writes one 32-byte sector).  There is no
// per-element division: the reference's decision "fl(|x|/s) > midpoint" is turned into "|x| > T" with
// two per-block thresholds computed exactly in double precision; the other five thresholds are those
// two times powers of two, i.e. a fixed offset of the bf16 bit pattern, so the code index is obtained
// with 16-bit SIMD-within-a-register arithmetic on pairs of elements.
//
// General kernel: any float dtype, block size, row stride and ragged row length; it restates the
// reference's arithmetic literally (IEEE division per element).
#include "mxfp4_common.cuh"

namespace mxfp4 {
namespace {

// ------------------------------------------------------------------------------------------------
// Literal restatement for one block (also the slow path of the streaming kernel).
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned exact_nibble(float v, float s) {
    const float n = __fdiv_rn(v, s);                       // quantizer.py:97
    const float a = fabsf(n);
    // argmin over the 8 levels with the first minimum winning (quantizer.py:112-114) == number of
    // midpoints strictly below a; the differences the reference forms are exact next to a midpoint.
    const unsigned idx = (a > 0.625f) + (a > 0.875f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    return (n < 0.0f ? 8u : 0u) | idx;                     // quantizer.py:119-122
}

template <typename T>
__device__ __noinline__ void quantize_block_exact(const T* __restrict__ src, int valid, int block, int scale_fmt,
                                                  uint8_t* __restrict__ packed_out, void* __restrict__ scale_out) {
    float amax = 0.0f;
    for (int i = 0; i < valid; ++i) amax = fmaxf(amax, fabsf(to_f32<T>(src[i])));
    amax = fmaxf(amax, 1e-8f);                             // quantizer.py:90-91
    const float s = __fdiv_rn(amax, 6.0f);                 // quantizer.py:95-96
    for (int i = 0; i < block; i += 2) {
        const float v0 = i < valid ? to_f32<T>(src[i]) : 0.0f;          // zero padding, quantizer.py:63-69
        const float v1 = i + 1 < valid ? to_f32<T>(src[i + 1]) : 0.0f;
        packed_out[i >> 1] = (uint8_t)((exact_nibble(v0, s) << 4) | exact_nibble(v1, s));   // quantizer.py:124-128
    }
    if (scale_fmt == MXFP4_SF_E8M0) *(uint8_t*)scale_out = (uint8_t)e8m0_byte(s);           // quantizer.py:100-102
    else *(__nv_bfloat16*)scale_out = __float2bfloat16_rn(s);                               // quantizer.py:137-139
}

template <typename T>
__global__ void __launch_bounds__(128) quantize_general_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                                                               int block, int64_t nblk, int scale_fmt,
                                                               uint8_t* __restrict__ packed, void* __restrict__ scales) {
    const int64_t total = rows * nblk;
    const int scale_bytes = scale_fmt == MXFP4_SF_E8M0 ? 1 : 2;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nblk, b = i - r * nblk;
        const int64_t c0 = b * block;
        const int64_t left = cols - c0;
        const int valid = left < block ? (int)left : block;
        quantize_block_exact<T>(x + r * ld + c0, valid, block, scale_fmt, packed + i * (block / 2),
                                (uint8_t*)scales + i * scale_bytes);
    }
}

// Quantise and dequantise in one pass (MXLinear.simulate_quantization, src/mxfp4/modules.py:144-150: the reference runs
// quantize() and dequantize() back to back on the whole weight in every forward).  Same arithmetic as the two kernels,
// nothing packed in between: out = +-level[code] * stored_scale, float32, of the padded width.
template <typename T>
__global__ void __launch_bounds__(128) fake_quantize_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, int64_t ld, int block,
                                                            int64_t nblk, int scale_fmt, float* __restrict__ out) {
    const int64_t total = rows * nblk;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nblk, b = i - r * nblk;
        const int64_t c0 = b * block;
        const int64_t left = cols - c0;
        const int valid = left < block ? (int)left : block;
        const T* src = x + r * ld + c0;
        float amax = 0.0f;
        for (int j = 0; j < valid; ++j) amax = fmaxf(amax, fabsf(to_f32<T>(src[j])));
        amax = fmaxf(amax, 1e-8f);                             // quantizer.py:90-91
        const float s = __fdiv_rn(amax, 6.0f);                 // quantizer.py:95-96
        const float stored = scale_fmt == MXFP4_SF_E8M0 ? e8m0_value(e8m0_byte(s)) : __bfloat162float(__float2bfloat16_rn(s));
        float* dst = out + r * (nblk * block) + c0;
        for (int j = 0; j < block; ++j) {
            const unsigned nib = exact_nibble(j < valid ? to_f32<T>(src[j]) : 0.0f, s);
            dst[j] = (ref_level(nib & 7u) * ((nib & 8u) ? -1.0f : 1.0f)) * stored;      // quantizer.py:171-193
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Streaming kernel.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ld_256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// thresholds: midpoint + half an ulp of the midpoint (float32), for the two midpoints in [0.5, 1)
#define MXFP4_CP (0.625 + 0x1p-25)
#define MXFP4_CQ (0.875 + 0x1p-25)

// One 32-element block held in registers as 16 bf16 pairs -> 16 code bytes and one scale.
__device__ __forceinline__ void quantize_one_block(const uint32_t (&w)[16], int64_t blk, int scale_fmt, uint4* __restrict__ packed,
                                                   void* __restrict__ scales) {
    // amax over the 32 elements, as bf16 bit patterns (quantizer.py:90)
    __nv_bfloat162 m2 = __habs2(as_bf162(w[0]));
#pragma unroll
    for (int i = 1; i < 16; ++i) m2 = __hmax2(m2, __habs2(as_bf162(w[i])));
    const uint32_t mb = as_u32(m2);
    const uint32_t amax16 = max(mb & 0xFFFFu, mb >> 16);
    const float amax = fmaxf(__uint_as_float(amax16 << 16), 1e-8f);     // quantizer.py:91
    const float s = __fdiv_rn(amax, 6.0f);                              // quantizer.py:95-96

    if (__float_as_uint(s) >= 0x47800000u) {
        // s >= 2^16 (or inf/NaN): a quotient could underflow to zero and lose its sign, and the
        // scaled thresholds could overflow; take the literal path.
        uint8_t bytes[16];
        __nv_bfloat16 tmp[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) *reinterpret_cast<uint32_t*>(&tmp[2 * i]) = w[i];
        uint16_t sc = 0;
        quantize_block_exact<__nv_bfloat16>(tmp, 32, 32, scale_fmt, bytes, &sc);
        uint4 o;
        o.x = bytes[0] | bytes[1] << 8 | bytes[2] << 16 | (uint32_t)bytes[3] << 24;
        o.y = bytes[4] | bytes[5] << 8 | bytes[6] << 16 | (uint32_t)bytes[7] << 24;
        o.z = bytes[8] | bytes[9] << 8 | bytes[10] << 16 | (uint32_t)bytes[11] << 24;
        o.w = bytes[12] | bytes[13] << 8 | bytes[14] << 16 | (uint32_t)bytes[15] << 24;
        packed[blk] = o;
        if (scale_fmt == MXFP4_SF_E8M0) ((uint8_t*)scales)[blk] = (uint8_t)sc;
        else ((uint16_t*)scales)[blk] = sc;
        return;
    }

    // fl32(|x|/s) > t  <=>  |x| > s*(t + ulp(t)/2)  <=>  |x| > round_down_f32(s*(t + ulp(t)/2)); the
    // product has at most 49 significant bits, so it is exact in double.  For bf16 |x| only the upper
    // 16 bits of the threshold matter:  |x| > T  <=>  bits16(|x|) > bits32(T) >> 16.
    const uint32_t p16 = __float_as_uint(__double2float_rd((double)s * MXFP4_CP)) >> 16;   // 0.625 s
    const uint32_t q16 = __float_as_uint(__double2float_rd((double)s * MXFP4_CQ)) >> 16;   // 0.875 s
    // The thresholds are p, q, 2p, 2q, 4p, 4q, 8p: +128 per doubling in bf16 bit space.  With
    // u' = max(u, q16-127):  #{j: u > p16 + 128 j} = (u' - (p16-127)) >> 7, same for q.
    const uint32_t plow2 = (p16 - 127u) * 0x00010001u;
    const uint32_t qlow2 = (q16 - 127u) * 0x00010001u;
    const __nv_bfloat162 qclamp = as_bf162(qlow2);
    const __nv_bfloat162 zero2 = as_bf162(0u);

    uint32_t out[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t nib[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 v = as_bf162(w[4 * g + j]);
            const uint32_t u = as_u32(__hmax2(__habs2(v), qclamp));
            const uint32_t a = (u - plow2) & 0xFF80FF80u;
            const uint32_t b = (u - qlow2) & 0xFF80FF80u;
            const uint32_t idx2 = (a + b) >> 7;                               // code of the even element at bit 0, odd at bit 16
            nib[j] = idx2 | (__hlt2_mask(v, zero2) & 0x00080008u);           // sign bit only for x < 0 (not for -0.0)
        }
        const uint32_t X = prmt(nib[0], nib[1], 0x6240u);   // [e0, e2, e1, e3]
        const uint32_t Y = prmt(nib[2], nib[3], 0x6240u);   // [e4, e6, e5, e7]
        out[g] = (prmt(X, Y, 0x5410u) << 4) | prmt(X, Y, 0x7632u);           // even element in the high nibble
    }
    packed[blk] = make_uint4(out[0], out[1], out[2], out[3]);
    if (scale_fmt == MXFP4_SF_E8M0) ((uint8_t*)scales)[blk] = (uint8_t)e8m0_byte(s);
    else ((__nv_bfloat16*)scales)[blk] = __float2bfloat16_rn(s);
}

// One thread per block, one CTA per 128 blocks.  (Measured alternatives on 4096 x 4096 and on one Llama-2-7B layer: a
// persistent grid of 2-4 CTAs per SM with a grid stride, with or without the next block's loads in flight, and two or
// four blocks per thread all lost 4-15 % against this plain mapping, whose many small CTAs keep more bytes in flight
// per SM; chaining consecutive launches, below, gained 4-6 %.)
__global__ void __launch_bounds__(128) quantize_bf16_b32_kernel(const uint8_t* __restrict__ x, int64_t nblocks, int scale_fmt,
                                                                uint4* __restrict__ packed, void* __restrict__ scales) {
    MXFP4_CHAIN_PROLOGUE();
    const int64_t blk = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (blk >= nblocks) return;
    uint32_t w[16];
    {
        uint32_t lo[8], hi[8];
        ld_256(x + blk * 64, lo);
        ld_256(x + blk * 64 + 32, hi);
#pragma unroll
        for (int i = 0; i < 8; ++i) { w[i] = lo[i]; w[8 + i] = hi[i]; }
    }
    quantize_one_block(w, blk, scale_fmt, packed, scales);
}

template <typename T>
int launch_general(const void* x, int64_t rows, int64_t cols, int64_t ld, int block, int scale_fmt, uint8_t* packed,
                   void* scales, cudaStream_t st) {
    const int64_t nblk = (cols + block - 1) / block;
    const int64_t total = rows * nblk;
    const int threads = 128;
    int64_t grid = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)num_sms() * 64;
    if (grid > cap) grid = cap;
    quantize_general_kernel<T><<<(unsigned)grid, threads, 0, st>>>((const T*)x, rows, cols, ld, block, nblk, scale_fmt, packed, scales);
    MXFP4_CHECK_LAUNCH("mxfp4_quantize (general kernel)");
    return MXFP4_OK;
}

}  // namespace
}  // namespace mxfp4

extern "C" int mxfp4_quantize(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int block_size,
                              int scale_fmt, uint8_t* packed, void* scales, void* stream) {
    using namespace mxfp4;
    if (rows < 0 || cols < 0) { set_error("mxfp4_quantize: negative size"); return MXFP4_E_SHAPE; }
    if (block_size <= 0 || (block_size & 1) || block_size > 1024) {
        set_error("mxfp4_quantize: block_size %d must be even and in [2, 1024]", block_size);
        return MXFP4_E_SHAPE;
    }
    if (scale_fmt != MXFP4_SF_E8M0 && scale_fmt != MXFP4_SF_BF16) { set_error("mxfp4_quantize: unknown scale format %d", scale_fmt); return MXFP4_E_BADARG; }
    if (x_dtype != MXFP4_DT_BF16 && x_dtype != MXFP4_DT_F16 && x_dtype != MXFP4_DT_F32) { set_error("mxfp4_quantize: unknown dtype %d", x_dtype); return MXFP4_E_BADARG; }
    if (rows == 0 || cols == 0) return MXFP4_OK;
    if (!x || !packed || !scales) { set_error("mxfp4_quantize: null pointer"); return MXFP4_E_BADARG; }
    if (ld < cols) { set_error("mxfp4_quantize: ld %lld < cols %lld", (long long)ld, (long long)cols); return MXFP4_E_SHAPE; }
    cudaStream_t st = (cudaStream_t)stream;

    const bool streaming = x_dtype == MXFP4_DT_BF16 && block_size == 32 && cols % 32 == 0 && ld == cols &&
                           ((uintptr_t)x % 32 == 0) && ((uintptr_t)packed % 16 == 0) && ((uintptr_t)scales % 2 == 0);
    if (streaming) {
        const int64_t nblocks = rows * (cols / 32);
        const int threads = 128;           // 128-thread CTAs: 2-3 % over 256 on layer-sized tensors, 64 and 512 lose 10 %
        const int64_t ctas = (nblocks + threads - 1) / threads;
        if (ctas > 0x7FFFFFFF) { set_error("mxfp4_quantize: tensor too large for one launch"); return MXFP4_E_SHAPE; }
        // chained to the kernel in front: a stream of quantise calls (a whole model) loses the launch gap between them
        cudaError_t le = launch_chained(quantize_bf16_b32_kernel, (unsigned)ctas, threads, st, (const uint8_t*)x, nblocks, scale_fmt,
                                        (uint4*)packed, scales);
        if (le != cudaSuccess) return cuda_fail(le, "mxfp4_quantize (streaming kernel)");
        return MXFP4_OK;
    }
    switch (x_dtype) {
        case MXFP4_DT_BF16: return launch_general<__nv_bfloat16>(x, rows, cols, ld, block_size, scale_fmt, packed, scales, st);
        case MXFP4_DT_F16: return launch_general<__half>(x, rows, cols, ld, block_size, scale_fmt, packed, scales, st);
        default: return launch_general<float>(x, rows, cols, ld, block_size, scale_fmt, packed, scales, st);
    }
}

extern "C" int mxfp4_fake_quantize(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int block_size, int scale_fmt,
                                   float* out, void* stream) {
    using namespace mxfp4;
    if (rows < 0 || cols < 0) { set_error("mxfp4_fake_quantize: negative size"); return MXFP4_E_SHAPE; }
    if (block_size <= 0 || (block_size & 1) || block_size > 1024) { set_error("mxfp4_fake_quantize: block_size %d must be even and in [2, 1024]", block_size); return MXFP4_E_SHAPE; }
    if (scale_fmt != MXFP4_SF_E8M0 && scale_fmt != MXFP4_SF_BF16) { set_error("mxfp4_fake_quantize: unknown scale format %d", scale_fmt); return MXFP4_E_BADARG; }
    if (rows == 0 || cols == 0) return MXFP4_OK;
    if (!x || !out) { set_error("mxfp4_fake_quantize: null pointer"); return MXFP4_E_BADARG; }
    if (ld < cols) { set_error("mxfp4_fake_quantize: ld < cols"); return MXFP4_E_SHAPE; }
    const int64_t nblk = (cols + block_size - 1) / block_size;
    const int64_t total = rows * nblk;
    int64_t grid = (total + 127) / 128;
    const int64_t cap = (int64_t)num_sms() * 64;
    if (grid > cap) grid = cap;
    cudaStream_t st = (cudaStream_t)stream;
    switch (x_dtype) {
        case MXFP4_DT_BF16: fake_quantize_kernel<__nv_bfloat16><<<(unsigned)grid, 128, 0, st>>>((const __nv_bfloat16*)x, rows, cols, ld, block_size, nblk, scale_fmt, out); break;
        case MXFP4_DT_F16: fake_quantize_kernel<__half><<<(unsigned)grid, 128, 0, st>>>((const __half*)x, rows, cols, ld, block_size, nblk, scale_fmt, out); break;
        case MXFP4_DT_F32: fake_quantize_kernel<float><<<(unsigned)grid, 128, 0, st>>>((const float*)x, rows, cols, ld, block_size, nblk, scale_fmt, out); break;
        default: set_error("mxfp4_fake_quantize: unknown dtype %d", x_dtype); return MXFP4_E_BADARG;
    }
    MXFP4_CHECK_LAUNCH("mxfp4_fake_quantize");
    return MXFP4_OK;
}
