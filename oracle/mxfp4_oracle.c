/*
 * CPU oracle for the MXFP4 hot path.  TEST INFRASTRUCTURE ONLY: this file is the checker that the
 * CUDA kernels are compared against (and the timed "port" CPU baseline); nothing in the shipped
 * package links, loads or calls it.
 *
 * Every function restates, operation for operation, what the reference's PyTorch code computes on
 * CPU tensors; citations are file:line inside the reference project (moizyousufi/MoizMXFP4-public).
 * Parity is pinned: tests/test_oracle_golden.py checks this file against fixtures produced by
 * running the reference itself (tests/golden/make_golden.py).
 *
 * All arithmetic is IEEE binary32, round-to-nearest-even, no flush-to-zero, no contraction
 * (compile with -O2 -ffp-contract=off and without -ffast-math).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DT_BF16 0
#define DT_F16 1
#define DT_F32 2
#define SF_E8M0 0
#define SF_BF16 1

/* src/mxfp4/quantizer.py:28-33 -- the reference codebook: no zero, 0.75 present. */
static const float kLevels[8] = {0.5f, 0.75f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0) {
        if (m == 0) return bits_to_f32(sign);
        float v = ldexpf((float)m, -24);                 /* subnormal: m * 2^-24 */
        return sign ? -v : v;
    }
    if (e == 31) return bits_to_f32(sign | 0x7F800000u | (m << 13));
    return bits_to_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* torch `.to(torch.bfloat16)` on a float32 tensor: round-to-nearest-even on the upper 16 bits. */
static inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0;  /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float load_as_f32(const void* x, int dtype, int64_t i) {
    /* src/mxfp4/quantizer.py:83 -- `tensor.float()`: exact upcast. */
    switch (dtype) {
        case DT_BF16: return bf16_to_f32(((const uint16_t*)x)[i]);
        case DT_F16:  return f16_to_f32(((const uint16_t*)x)[i]);
        default:      return ((const float*)x)[i];
    }
}

/* src/mxfp4/quantizer.py:35-48 -- _to_e8m0: round(log2(clamp(s, 1e-10))) + 127, clamped to [0,255]. */
static inline uint8_t to_e8m0(float s) {
    float c = s < 1e-10f ? 1e-10f : s;
    float e = rintf(log2f(c)) + 127.0f;
    if (e < 0.0f) e = 0.0f;
    if (e > 255.0f) e = 255.0f;
    return (uint8_t)e;
}

/* src/mxfp4/quantizer.py:50-61 -- _from_e8m0: pow(2, b - 127) in float32 (b = 0 gives the subnormal
 * 2^-127, b = 255 overflows to +inf). */
static inline float from_e8m0(uint8_t b) {
    if (b == 255) return INFINITY;
    return ldexpf(1.0f, (int)b - 127);
}

/*
 * src/mxfp4/quantizer.py:71-141 -- MXFP4Quantizer.quantize on a [rows, cols] matrix (leading
 * dimensions flattened by the caller).  The last dimension is zero-padded to a multiple of `block`
 * (:63-69, :84).  packed is [rows, cols_pad/2]; scales is [rows, cols_pad/block], uint8 (e8m0) or
 * bf16 bit patterns.
 */
int mxfp4_oracle_quantize(const void* x, int dtype, int64_t rows, int64_t cols, int block, int scale_fmt,
                          uint8_t* packed, void* scales) {
    if (block <= 0 || (block & 1) || block > 4096) return -1;
    const int64_t nblk = (cols + block - 1) / block;
    const int64_t cols_pad = nblk * block;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float v[4096];
        uint8_t nib[4096];
        for (int64_t b = 0; b < nblk; ++b) {
            float amax = 0.0f;
            for (int i = 0; i < block; ++i) {
                int64_t c = b * block + i;
                v[i] = c < cols ? load_as_f32(x, dtype, r * cols + c) : 0.0f;     /* :84 zero pad */
                float a = fabsf(v[i]);
                if (a > amax) amax = a;                                           /* :90 amax(abs) */
            }
            if (amax < 1e-8f) amax = 1e-8f;                                       /* :91 clamp */
            const float s = amax / 6.0f;                                          /* :95-96 */
            for (int i = 0; i < block; ++i) {
                const float n = v[i] / s;                                         /* :97 */
                const float a = fabsf(n);
                int idx = 0;
                float best = fabsf(a - kLevels[0]);
                for (int j = 1; j < 8; ++j) {                                     /* :112-114 argmin: */
                    float d = fabsf(a - kLevels[j]);                              /* first minimum wins */
                    if (d < best) { best = d; idx = j; }
                }
                nib[i] = (uint8_t)(((n < 0.0f) ? 8 : 0) | idx);                   /* :119-122 */
            }
            uint8_t* prow = packed + r * (cols_pad / 2) + b * (block / 2);
            for (int i = 0; i < block; i += 2)                                    /* :124-128 even -> high */
                prow[i / 2] = (uint8_t)((nib[i] << 4) | nib[i + 1]);
            if (scale_fmt == SF_E8M0)
                ((uint8_t*)scales)[r * nblk + b] = to_e8m0(s);                    /* :100-102 */
            else
                ((uint16_t*)scales)[r * nblk + b] = f32_to_bf16_rne(s);           /* :137-139 */
        }
    }
    return 0;
}

/*
 * src/mxfp4/quantizer.py:143-198 -- MXFP4Quantizer.dequantize: float32 output of the PADDED width.
 */
int mxfp4_oracle_dequantize(const uint8_t* packed, const void* scales, int scale_fmt, int64_t rows,
                            int64_t cols_pad, int block, float* out) {
    if (block <= 0 || (block & 1) || cols_pad % block) return -1;
    const int64_t nblk = cols_pad / block;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t b = 0; b < nblk; ++b) {
            const float s = scale_fmt == SF_E8M0 ? from_e8m0(((const uint8_t*)scales)[r * nblk + b])   /* :155-160 */
                                                 : bf16_to_f32(((const uint16_t*)scales)[r * nblk + b]);
            for (int i = 0; i < block; ++i) {
                const int64_t c = b * block + i;
                const uint8_t byte = packed[r * (cols_pad / 2) + c / 2];
                const uint8_t nibv = (c & 1) ? (byte & 0x0F) : (byte >> 4);      /* :163-168 */
                const float val = kLevels[nibv & 7] * ((nibv & 8) ? -1.0f : 1.0f);  /* :171-181 */
                out[r * cols_pad + c] = val * s;                                  /* :193 */
            }
        }
    }
    return 0;
}

/*
 * Activation quantiser of the new GEMM (there is no counterpart in the reference's own quantiser:
 * its tensor-core path, src/mxfp4/backends.py:162-183, hands activations to a third-party kernel).
 * Definition, in exact arithmetic on bf16 inputs, block = 32 along K:
 *   amax = max |x_i|  (bits E = biased exponent, m7 = mantissa)
 *   byte = clamp(E - 2 + [m7 > 0x40], 0, 254)   i.e. scale 2^(byte-127) = 2^ceil(log2(amax/6))
 *   q_i  = x_i * 2^(127-byte) in float32, rounded to hardware E2M1 {0,.5,1,1.5,2,3,4,6}
 *          (round-to-nearest, ties to the even mantissa, saturating at 6)
 *   nibble = sign<<3 | e<<1 | m ; even element -> HIGH nibble (the reference's byte order,
 *   src/mxfp4/quantizer.py:124-128).  amax = 0 gives byte 0 and all-zero codes; -0.0 keeps its sign
 *   bit, which decodes to -0.0.
 */
static inline uint8_t e2m1_rne(float q) {
    const uint32_t sign = (f32_to_bits(q) >> 31) << 3;
    const float a = fabsf(q);
    uint32_t code;
    if (a <= 0.25f) code = 0;          /* tie 0.25 -> 0 (even) */
    else if (a < 0.75f) code = 1;      /* 0.5 */
    else if (a <= 1.25f) code = 2;     /* ties 0.75, 1.25 -> 1.0 (even) */
    else if (a < 1.75f) code = 3;      /* 1.5 */
    else if (a <= 2.5f) code = 4;      /* ties 1.75, 2.5 -> 2.0 */
    else if (a < 3.5f) code = 5;       /* 3.0 */
    else if (a <= 5.0f) code = 6;      /* ties 3.5, 5.0 -> 4.0 */
    else code = 7;                     /* 6.0, saturating */
    return (uint8_t)(sign | code);
}

int mxfp4_oracle_act_quantize(const uint16_t* x, int64_t M, int64_t K, uint8_t* packed, uint8_t* scales) {
    if (K % 32) return -1;
    const int64_t nblk = K / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; ++r) {
        for (int64_t b = 0; b < nblk; ++b) {
            const uint16_t* p = x + r * K + b * 32;
            uint16_t amax = 0;
            for (int i = 0; i < 32; ++i) {
                uint16_t a = p[i] & 0x7FFFu;
                if (a > amax) amax = a;
            }
            int byte = (int)(amax >> 7) - 2 + ((amax & 0x7Fu) > 0x40u ? 1 : 0);
            if (byte < 0) byte = 0;
            if (byte > 254) byte = 254;
            const float inv = byte == 0 ? bits_to_f32(0x7F000000u) /* 2^127 */
                                        : (byte == 254 ? bits_to_f32(0x00400000u) /* 2^-127 */
                                                       : bits_to_f32((uint32_t)(254 - byte) << 23));
            uint8_t nib[32];
            for (int i = 0; i < 32; ++i) nib[i] = e2m1_rne(bf16_to_f32(p[i]) * inv);
            for (int i = 0; i < 32; i += 2)
                packed[r * (K / 2) + b * 16 + i / 2] = (uint8_t)((nib[i] << 4) | nib[i + 1]);
            scales[r * nblk + b] = (uint8_t)byte;
        }
    }
    return 0;
}

/* Decode of the activation format above (hardware E2M1: code 0 is zero, code 1 is 0.5). */
int mxfp4_oracle_act_dequantize(const uint8_t* packed, const uint8_t* scales, int64_t M, int64_t K, float* out) {
    static const float hw[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    if (K % 32) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; ++r)
        for (int64_t c = 0; c < K; ++c) {
            const uint8_t byte = packed[r * (K / 2) + c / 2];
            const uint8_t nibv = (c & 1) ? (byte & 0x0F) : (byte >> 4);
            const float v = hw[nibv & 7] * from_e8m0(scales[r * (K / 32) + c / 32]);
            out[r * K + c] = (nibv & 8) ? -v : v;
        }
    return 0;
}

/*
 * out[M,N] = a[M,K] . w[N,K]^T (+ bias[N]) with float32 inputs and double accumulation: the
 * arithmetic core of src/mxfp4/backends.py:307-310 (`torch.matmul(input, W.T)`, `output += bias`)
 * once the caller has dequantised.  Output is float32; callers round to bf16 as the reference does.
 */
int mxfp4_oracle_matmul_nt(const float* a, const float* w, const float* bias, int64_t M, int64_t N, int64_t K,
                           float* out) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
            double acc = 0.0;
            const float* ar = a + i * K;
            const float* wr = w + j * K;
            for (int64_t k = 0; k < K; ++k) acc += (double)ar[k] * (double)wr[k];
            out[i * N + j] = (float)acc + (bias ? bias[j] : 0.0f);
        }
    return 0;
}

int mxfp4_oracle_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
