/*
 * C ABI of libmxfp4_b200.so -- the sm_100a (NVIDIA B200) backend for the MXFP4 hot path of
 * moizyousufi/MoizMXFP4-public.  Plain pointers and sizes only; every pointer named "device" must be
 * device memory of the current CUDA device.  Nothing here allocates device memory, synchronises the
 * stream, or touches the host copy of any buffer: each call enqueues kernels on `stream` (a
 * cudaStream_t passed as void*; NULL is the legacy default stream) and returns.
 *
 * Every function returns 0 on success or one of the negative MXFP4_E_* codes; mxfp4_last_error()
 * then holds a message for the calling thread.
 *
 * Citations "replaces ..." name the reference interface each entry point stands in for
 * (file:line inside the reference project).
 */
#ifndef MXFP4_B200_H_
#define MXFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MXFP4_API __attribute__((visibility("default")))
#else
#define MXFP4_API
#endif

#define MXFP4_OK 0
#define MXFP4_E_BADARG (-1)      /* null pointer, unknown enum value */
#define MXFP4_E_SHAPE (-2)       /* sizes the kernels cannot take (odd block, K not a multiple of 32, ...) */
#define MXFP4_E_ALIGN (-3)       /* pointer or leading dimension not aligned as documented */
#define MXFP4_E_UNSUPPORTED (-4) /* valid request outside what this backend implements */
#define MXFP4_E_CUDA (-5)        /* a CUDA runtime/driver call failed; message has the CUDA error */
#define MXFP4_E_TIMEOUT (-6)     /* a bounded device-side wait ran out (reported through a status word) */
#define MXFP4_E_WORKSPACE (-7)   /* workspace smaller than mxfp4_gemm_workspace_bytes() */

/* element types */
#define MXFP4_DT_BF16 0
#define MXFP4_DT_F16 1
#define MXFP4_DT_F32 2
/* scale formats of MXFP4Quantizer(scale_format=...) -- src/mxfp4/quantizer.py:12-23 */
#define MXFP4_SF_E8M0 0 /* uint8, value 2^(b-127) */
#define MXFP4_SF_BF16 1 /* bfloat16 */

/* Library/ABI version (major*10000 + minor*100 + patch). */
MXFP4_API int mxfp4_version(void);

/* Copies the calling thread's last error message into buf (NUL-terminated, truncated to n). */
MXFP4_API void mxfp4_last_error(char* buf, size_t n);

/* Compute capability and SM count of the current device.  The backend only runs on sm_100
 * (replaces detect_architecture(), src/mxfp4/backends.py:34-131, which picks among three backends). */
MXFP4_API int mxfp4_device_info(int* sm_major, int* sm_minor, int* num_sms);

/*
 * Block quantiser.  Replaces MXFP4Quantizer.quantize, src/mxfp4/quantizer.py:71-141, bit for bit on
 * finite inputs: per block of `block_size` consecutive elements of a row (rows zero-padded to a
 * multiple of block_size), amax = max|x| clamped to 1e-8, s = amax/6, codes = index of the nearest of
 * {0.5,.75,1,1.5,2,3,4,6} to |x/s| (ties to the smaller), nibble = sign<<3 | code, even element in the
 * HIGH nibble; scale = uint8(round(log2 s) + 127) for E8M0 or bfloat16(s).
 *
 *   x        device, [rows, cols] of x_dtype, row r starts at x + r*ld elements (ld >= cols)
 *   packed   device, [rows, cols_pad/2] uint8, contiguous, cols_pad = ceil(cols/block_size)*block_size
 *   scales   device, [rows, cols_pad/block_size] uint8 (E8M0) or bfloat16 (BF16), contiguous
 * block_size must be even and <= 1024.  bf16 input, block_size 32, cols % 32 == 0, ld == cols and a
 * 32-byte-aligned x take the streaming kernel; everything else takes a general kernel.
 */
MXFP4_API int mxfp4_quantize(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int block_size,
                   int scale_fmt, uint8_t* packed, void* scales, void* stream);

/*
 * Block dequantiser.  Replaces MXFP4Quantizer.dequantize, src/mxfp4/quantizer.py:143-198, bit for
 * bit: out = +-level[code] * scale, float32, of the PADDED width cols_pad.
 *
 *   packed  device, [rows, cols_pad/2] uint8, contiguous
 *   scales  device, [rows, cols_pad/block_size] uint8 (E8M0) or bfloat16, contiguous
 *   out     device, [rows, cols_pad] of out_dtype: MXFP4_DT_F32 (what the reference returns) or
 *           MXFP4_DT_BF16 (the cast MXLinear.forward applies next, src/mxfp4/modules.py:135-136, fused in;
 *           exact whenever the float32 value is representable in bf16, i.e. for all E8M0 scales)
 */
MXFP4_API int mxfp4_dequantize(const uint8_t* packed, const void* scales, int scale_fmt, int64_t rows, int64_t cols_pad,
                     int block_size, void* out, int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MXFP4_B200_H_ */
