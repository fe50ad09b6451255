// Shared definitions for the sm_100a MXFP4 kernels and their C-ABI wrappers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/mxfp4_b200.h"

namespace mxfp4 {

// Thread-local message for mxfp4_last_error().
void set_error(const char* fmt, ...);

inline int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return MXFP4_E_CUDA;
}

#define MXFP4_CHECK_LAUNCH(what)                                        \
    do {                                                                \
        cudaError_t e__ = cudaGetLastError();                           \
        if (e__ != cudaSuccess) return ::mxfp4::cuda_fail(e__, what);   \
    } while (0)

int num_sms();  // SM count of the current device (cached per device)

// Launch with programmatic stream serialisation: the grid may be scheduled while the kernel in front of it on the
// stream is still draining.  Kernels launched this way execute griddepcontrol.wait in every thread before they touch
// global memory, so results are those of a plain launch; what overlaps is only the scheduling of their CTAs with the
// tail of the kernel in front (a few microseconds per launch, which is a third of a 4096 x 4096 quantise).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// first statements of a kernel launched with launch_chained: let the next launch be scheduled, then wait for the
// kernel in front (both are no-ops when there is nothing to chain to)
#define MXFP4_CHAIN_PROLOGUE()                                              \
    do {                                                                    \
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     \
        asm volatile("griddepcontrol.wait;" ::: "memory");                  \
    } while (0)

// ---------------------------------------------------------------------------------------------
// The reference codebook (quantizer.py:28-33): magnitudes {0.5,.75,1,1.5,2,3,4,6} for codes 0..7,
// i.e. (1 + m/2) * 2^(e-1) with e = code>>1, m = code&1 -- no zero, unlike hardware E2M1.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float ref_level(int code) {
    return __uint_as_float(((126u + (unsigned)(code >> 1)) << 23) | ((unsigned)(code & 1) << 22));
}

// E8M0 byte of a positive finite float32 scale s: round(log2(s)) + 127 (quantizer.py:45-48).
// log2(s) = E-127 + log2(1.m); it rounds up exactly when 1.m > sqrt(2), and 0x3504F3 is the mantissa
// of the largest float32 below sqrt(2).
__device__ __forceinline__ unsigned e8m0_byte(float s) {
    s = fmaxf(s, 1e-10f);
    const unsigned u = __float_as_uint(s);
    const unsigned b = (u >> 23) + ((u & 0x7FFFFFu) > 0x3504F3u ? 1u : 0u);
    return b > 255u ? 255u : b;
}

// 2^(b-127) as float32 for every byte (quantizer.py:50-61): b = 0 is the subnormal 2^-127, b = 255 is +inf.
__device__ __forceinline__ float e8m0_value(unsigned b) {
    return b == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(b << 23);   // 255<<23 is +inf
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

}  // namespace mxfp4
