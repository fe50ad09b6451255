// MXFP4 -> float32 / bfloat16 block dequantiser for sm_100a.
//
// Reproduces MXFP4Quantizer.dequantize (reference: src/mxfp4/quantizer.py:143-198) bit for bit.
//
// Streaming kernel (E8M0 scales, 32-element blocks): each thread turns one 32-bit word of codes
// (8 elements) into 32 bytes of float32 (or 16 bytes of bf16) with one 256-bit (128-bit) store, so a
// warp reads 128 contiguous bytes and writes 1 KB contiguous.  No multiply: level * 2^(b-127) is
// assembled directly as sign | (b - 1 + e) << 23 | m << 22 with code = e<<1 | m.  Scale bytes for which
// that exponent would leave the normal range (b < 2 or b > 251) take a true multiplication.
//
// General kernel: any block size, bf16 scales; literal level * scale in float32.
#include "mxfp4_common.cuh"

namespace mxfp4 {
namespace {

__device__ __forceinline__ float decode_mul(unsigned nib, float scale) {
    const float v = ref_level(nib & 7u) * ((nib & 8u) ? -1.0f : 1.0f);    // quantizer.py:171-181
    return v * scale;                                                     // quantizer.py:193
}

template <bool kBf16Out>
__global__ void __launch_bounds__(256) dequantize_e8m0_b32_kernel(const uint32_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                                                   int64_t nwords, void* __restrict__ out) {
    MXFP4_CHAIN_PROLOGUE();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nwords; i += stride) {
        const uint32_t w = __ldg(packed + i);
        const uint32_t sc = __ldg(scales + (i >> 2));
        uint32_t o[8];
        if (sc >= 2u && sc <= 251u) {
            const uint32_t base = (sc - 1u) << 23;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // byte j holds element 2j in its high nibble and 2j+1 in its low nibble (quantizer.py:163-168)
                const uint32_t hi = w << (24 - 8 * j);        // high nibble of byte j in bits 31..28
                const uint32_t lo = w << (28 - 8 * j);        // low nibble of byte j in bits 31..28
                o[2 * j] = (hi & 0x80000000u) | (((hi >> 6) & 0x01C00000u) + base);
                o[2 * j + 1] = (lo & 0x80000000u) | (((lo >> 6) & 0x01C00000u) + base);
            }
        } else {
            const float s = e8m0_value(sc);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t b = (w >> (8 * j)) & 0xFFu;
                o[2 * j] = __float_as_uint(decode_mul(b >> 4, s));
                o[2 * j + 1] = __float_as_uint(decode_mul(b & 15u, s));
            }
        }
        if (kBf16Out) {
            uint32_t h[4];
            if (sc >= 2u && sc <= 251u) {
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = (o[2 * j] >> 16) | (o[2 * j + 1] & 0xFFFF0000u);   // low mantissa bits are zero
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(o[2 * j]), __uint_as_float(o[2 * j + 1]));
                    h[j] = *reinterpret_cast<const uint32_t*>(&t);
                }
            }
            reinterpret_cast<uint4*>(out)[i] = make_uint4(h[0], h[1], h[2], h[3]);
        } else {
            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(reinterpret_cast<uint8_t*>(out) + i * 32),
                         "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                         : "memory");
        }
    }
}

template <bool kBf16Out>
__global__ void __launch_bounds__(256) dequantize_general_kernel(const uint8_t* __restrict__ packed, const void* __restrict__ scales,
                                                                  int scale_fmt, int64_t nbytes, int block, void* __restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nbytes; i += stride) {
        const uint32_t b = packed[i];
        const int64_t blk = (2 * i) / block;          // rows are whole numbers of blocks, so the flat index works
        const float s = scale_fmt == MXFP4_SF_E8M0 ? e8m0_value(((const uint8_t*)scales)[blk])            // quantizer.py:155-157
                                                   : __bfloat162float(((const __nv_bfloat16*)scales)[blk]);  // quantizer.py:160
        const float v0 = decode_mul(b >> 4, s), v1 = decode_mul(b & 15u, s);
        if (kBf16Out) reinterpret_cast<__nv_bfloat162*>(out)[i] = __floats2bfloat162_rn(v0, v1);
        else reinterpret_cast<float2*>(out)[i] = make_float2(v0, v1);
    }
}

}  // namespace
}  // namespace mxfp4

extern "C" int mxfp4_dequantize(const uint8_t* packed, const void* scales, int scale_fmt, int64_t rows, int64_t cols_pad,
                                int block_size, void* out, int out_dtype, void* stream) {
    using namespace mxfp4;
    if (rows < 0 || cols_pad < 0) { set_error("mxfp4_dequantize: negative size"); return MXFP4_E_SHAPE; }
    if (block_size <= 0 || (block_size & 1)) { set_error("mxfp4_dequantize: block_size %d must be even", block_size); return MXFP4_E_SHAPE; }
    if (cols_pad % block_size) {
        set_error("mxfp4_dequantize: width %lld is not a multiple of block_size %d", (long long)cols_pad, block_size);
        return MXFP4_E_SHAPE;
    }
    if (scale_fmt != MXFP4_SF_E8M0 && scale_fmt != MXFP4_SF_BF16) { set_error("mxfp4_dequantize: unknown scale format %d", scale_fmt); return MXFP4_E_BADARG; }
    if (out_dtype != MXFP4_DT_F32 && out_dtype != MXFP4_DT_BF16) { set_error("mxfp4_dequantize: output dtype must be f32 or bf16"); return MXFP4_E_UNSUPPORTED; }
    if (rows == 0 || cols_pad == 0) return MXFP4_OK;
    if (!packed || !scales || !out) { set_error("mxfp4_dequantize: null pointer"); return MXFP4_E_BADARG; }
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t nbytes = rows * (cols_pad / 2);
    const int threads = 256;
    const int64_t cap = (int64_t)num_sms() * 32;

    const bool streaming = scale_fmt == MXFP4_SF_E8M0 && block_size == 32 && ((uintptr_t)packed % 4 == 0) && ((uintptr_t)out % 32 == 0);
    if (streaming) {
        const int64_t nwords = nbytes / 4;
        int64_t grid = (nwords + threads - 1) / threads;
        if (grid > cap) grid = cap;
        // chained to the kernel in front (see launch_chained): consecutive launches lose the gap between them
        cudaError_t le;
        if (out_dtype == MXFP4_DT_F32)
            le = launch_chained(dequantize_e8m0_b32_kernel<false>, (unsigned)grid, threads, st, (const uint32_t*)packed, (const uint8_t*)scales, nwords, out);
        else
            le = launch_chained(dequantize_e8m0_b32_kernel<true>, (unsigned)grid, threads, st, (const uint32_t*)packed, (const uint8_t*)scales, nwords, out);
        if (le != cudaSuccess) return cuda_fail(le, "mxfp4_dequantize (streaming kernel)");
        return MXFP4_OK;
    }
    int64_t grid = (nbytes + threads - 1) / threads;
    if (grid > cap) grid = cap;
    if (out_dtype == MXFP4_DT_F32)
        dequantize_general_kernel<false><<<(unsigned)grid, threads, 0, st>>>(packed, scales, scale_fmt, nbytes, block_size, out);
    else
        dequantize_general_kernel<true><<<(unsigned)grid, threads, 0, st>>>(packed, scales, scale_fmt, nbytes, block_size, out);
    MXFP4_CHECK_LAUNCH("mxfp4_dequantize (general kernel)");
    return MXFP4_OK;
}
