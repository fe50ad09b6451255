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

/*
 * Quantise and dequantise in one pass: out[rows, cols_pad] float32 = dequantize(quantize(x)), bit for bit, without
 * the packed intermediate.  Replaces the fake-quantisation forward of MXLinear.simulate_quantization,
 * src/mxfp4/modules.py:144-150 (quantize() + dequantize() of the whole weight per forward).  Arguments as mxfp4_quantize.
 */
MXFP4_API int mxfp4_fake_quantize(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int block_size,
                                  int scale_fmt, float* out, void* stream);

/* GEMM modes */
#define MXFP4_GEMM_EXACT 0 /* weights decode exactly as the reference dequantises them (two MMAs per K step) */
#define MXFP4_GEMM_FAST 1  /* single pass: weight codes 0 and 1 decode as hardware E2M1 (0, 0.5); NOT parity */

/*
 * Bytes of the tensor-core scale layouts ("blocked": tiles of 128 rows x 4 blocks, 512 bytes each,
 * byte (r%32)*16 + (r/32)*4 + c; rows padded to 128, K padded to 256).
 *   activation scales: ceil(M/128) * ceil(K/256) * 1024
 *   prepared weight scales: ceil(N/128) * ceil(K/256) * 2048  (the scale bytes and a copy decremented by one)
 */
MXFP4_API int64_t mxfp4_act_scales_bytes(int64_t M, int64_t K);
MXFP4_API int64_t mxfp4_prepared_scales_bytes(int64_t N, int64_t K);

/*
 * Activation quantiser of the GEMM (the job QuTLASSBackend.quantize hands to a third-party kernel,
 * src/mxfp4/backends.py:162-183): bf16 [M, K] (row pitch ld elements, K % 32 == 0) ->
 *   a_packed      device, [M, K/2] uint8: hardware E2M1 codes {0,.5,1,1.5,2,3,4,6}, round-to-nearest-even,
 *                 even element in the high nibble (the reference's byte order)
 *   a_sf_blocked  device, mxfp4_act_scales_bytes(M, K): E8M0 byte = exponent of 2^ceil(log2(amax/6)) per 32-block
 * x must be 32-byte aligned and ld*2 a multiple of 32; a_packed 16-byte aligned.
 */
MXFP4_API int mxfp4_act_quantize(const void* x_bf16, int64_t M, int64_t K, int64_t ld, uint8_t* a_packed,
                                 uint8_t* a_sf_blocked, void* stream);

/*
 * Re-tiles a weight's E8M0 scales [N, K/32] (as mxfp4_quantize / the reference produce them) into the
 * tensor-core layout, mxfp4_prepared_scales_bytes(N, K) bytes.  Done once per weight; the result is a
 * cache, not part of the checkpoint (the reference's to_blocked() call per matmul, src/mxfp4/backends.py:227-228).
 */
MXFP4_API int mxfp4_prepare_weight_scales(const uint8_t* scales, int64_t N, int64_t K, uint8_t* prepared, void* stream);

/* Workspace of mxfp4_gemm: 4 KB control block (status word; rest reserved) + packed activations + blocked activation scales + the
 * float32 partial sums of a K-split (mxfp4_gemm_splitk_bytes; problems with fewer tiles than SMs, M <= 1024, may be
 * cut along K so that every SM streams part of the weight; the partials are summed in a fixed order by a second kernel). */
MXFP4_API int64_t mxfp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int mode);
MXFP4_API int64_t mxfp4_gemm_splitk_bytes(int64_t M, int64_t N, int64_t K);

/*
 * out[M,N] (bf16, row pitch ldo) = act_quantize(x)[M,K] . Wref[N,K]^T (+ bias[N], bf16), float32 accumulation on
 * the block-scaled FP4 tensor cores.  Replaces quant_matmul / backend.matmul, src/mxfp4/kernel_dispatcher.py:163-198
 * and src/mxfp4/backends.py:191-312.
 *   x_bf16         device, [M, K] bf16, row pitch ldx elements
 *   w_packed       device, [N, K/2] uint8, the reference's packed weight, unchanged
 *   w_sf_prepared  device, from mxfp4_prepare_weight_scales
 *   workspace      device, >= mxfp4_gemm_workspace_bytes, 256-byte aligned.  Its first 4 KB are a control block that the
 *                  caller zeroes once (not per call): int[0] is a status word -- a kernel whose bounded wait ran out stores
 *                  MXFP4_E_TIMEOUT there -- and the rest is reserved.
 * K % 32 == 0.  Launches two or three kernels on `stream` (activation quantiser, GEMM, split-K reduction), chained by
 * programmatic dependent launch: each starts its set-up while the one in front drains and waits for its results on the
 * device.  Work enqueued on the stream before and after the call is ordered as with plain launches.  Large M in EXACT
 * mode runs on CTA pairs (tcgen05 cta_group::2, clusters of two); results are bit-identical to the one-CTA kernel.
 */
MXFP4_API int mxfp4_gemm(const void* x_bf16, int64_t ldx, const uint8_t* w_packed, const uint8_t* w_sf_prepared,
                         const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M, int64_t N, int64_t K, int mode,
                         void* workspace, int64_t workspace_bytes, void* stream);

/* The GEMM alone, on activations already quantised by mxfp4_act_quantize.  splitk_workspace (16-byte aligned,
 * >= mxfp4_gemm_splitk_bytes) may be NULL: the K-split is then not used.  control_block: NULL, or 4 KB of device memory
 * zeroed once, laid out like the first 4 KB of mxfp4_gemm's workspace (int[0] receives MXFP4_E_TIMEOUT). */
MXFP4_API int mxfp4_gemm_prequantized(const uint8_t* a_packed, const uint8_t* a_sf_blocked, const uint8_t* w_packed,
                                      const uint8_t* w_sf_prepared, const void* bias_bf16, void* out_bf16, int64_t ldo,
                                      int64_t M, int64_t N, int64_t K, int mode, void* splitk_workspace,
                                      int64_t splitk_bytes, int* control_block, void* stream);

/*
 * mxfp4_gemm_prequantized with two options for chains of kernels (no counterpart in the reference):
 *   MXFP4_GEMM_CHAINED        the kernel that produced the activations sits directly in front on the stream and signals
 *                             griddepcontrol.launch_dependents (mxfp4_act_quantize and mxfp4_act_fused do): the GEMM is
 *                             launched with programmatic stream serialisation, loads weights while that kernel drains and
 *                             waits for it on the device before it touches the activations;
 *   MXFP4_GEMM_KEEP_PARTIALS  when the problem is cut along K (mxfp4_gemm_plan says into how many ranges) the float32
 *                             partial sums stay in splitk_workspace as [ksplit][M][N] and no reduction kernel runs:
 *                             the consumer sums them (mxfp4_act_fused does); the bias is then NOT applied and out_bf16 is
 *                             not written.  Without a K-split the flag changes nothing.
 * mxfp4_gemm_plan: the number of K ranges mxfp4_gemm* uses for a shape (1: no split) and whether CTA pairs run it.
 */
#define MXFP4_GEMM_CHAINED 1
#define MXFP4_GEMM_KEEP_PARTIALS 2
MXFP4_API int mxfp4_gemm_plan(int64_t M, int64_t N, int64_t K, int mode, int* ksplit, int* cta_pairs);
MXFP4_API int mxfp4_gemm_prequantized_ex(const uint8_t* a_packed, const uint8_t* a_sf_blocked, const uint8_t* w_packed,
                                         const uint8_t* w_sf_prepared, const void* bias_bf16, void* out_bf16, int64_t ldo,
                                         int64_t M, int64_t N, int64_t K, int mode, void* splitk_workspace,
                                         int64_t splitk_bytes, int* control_block, int flags, void* stream);

/*
 * W4A16: out[M,N] (bf16) = x[M,K] (bf16, not quantised) . bf16(dequantize(w))[N,K]^T (+ bias), float32 accumulation on the bf16
 * tensor cores.  The literal arithmetic of the reference's own GEMM paths (FallbackBackend.matmul,
 * src/mxfp4/backends.py:295-312; Triton quant_matmul, src/mxfp4/fused_kernels.py:141-207): weights decoded inside the
 * kernel (never materialised in global memory), activations untouched.  Used for scale_format="bf16" weights (their scales
 * are not powers of two) and, on request, for E8M0 weights when the reference's numerics without activation quantisation
 * are wanted at a quarter of the FP4 rate.
 *   w_scales  device, [N, K/block_size] uint8 (MXFP4_SF_E8M0) or bfloat16 (MXFP4_SF_BF16), row-major as the quantiser wrote them
 *   block_size 16, 32 or 64; K a multiple of 32 and of block_size; x and w_packed 16-byte aligned, ldx*2 a multiple of 16
 *   status_dev optional device int: receives MXFP4_E_TIMEOUT if a bounded wait ran out
 */
MXFP4_API int mxfp4_gemm_w4a16(const void* x_bf16, int64_t ldx, const uint8_t* w_packed, const void* w_scales, int scale_fmt,
                               int block_size, const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M, int64_t N,
                               int64_t K, int* status_dev, void* stream);

/*
 * mxfp4_gemm without any workspace argument and without any device allocation.  It has no counterpart in the
 * reference.  It is for callers that cannot allocate device memory when the matmul is due: a process whose
 * own pool owns the whole GPU and which bans cudaMalloc after start-up, a plugin living inside such a process,
 * or a latency-critical loop where an allocation would stall the device.  The scratch mxfp4_gemm takes as
 * `workspace` is a fixed 16 MiB array inside the library instead (held by every GPU that loads the library, until
 * the process exits).  Inputs and outputs are still the caller's.
 *   - Problems whose scratch (packed activations M*K/2 + activation scale tiles + split-K partials, see
 *     mxfp4_gemm_workspace_bytes) exceeds 16 MiB are rejected with MXFP4_E_WORKSPACE; typical decode shapes
 *     (M <= 128 with Llama-2-7B/70B layer sizes) fit.
 *   - The first call on each device looks up the array's device address; make that first call outside any stream
 *     capture, with the device current.
 *   - All calls share the one array and it keeps whatever the last call left there (nothing in it has to start
 *     at zero).  Two calls that overlap on the GPU -- different streams, or several host threads -- race on it;
 *     serialise them or use mxfp4_gemm with separate workspaces.
 *   - status_dev: optional device int, zeroed by the caller; receives MXFP4_E_TIMEOUT if a bounded wait ran out.
 * Other arguments as for mxfp4_gemm.
 */
MXFP4_API int mxfp4_gemm_noalloc(const void* x_bf16, int64_t ldx, const uint8_t* w_packed, const uint8_t* w_sf_prepared,
                                 const void* bias_bf16, void* out_bf16, int64_t ldo, int64_t M, int64_t N, int64_t K, int mode,
                                 int* status_dev, void* stream);

/*
 * Tensor parallelism on one NVSwitch box (no counterpart in the reference, which has no distributed code): sum of the
 * bf16 partial products [M, N] of a row-parallel layer over `world` ranks, one process per GPU, as ONE kernel over peer
 * memory (P2P loads and stores; no NCCL call, no multimem).  Every rank adds all partials in float32 in rank order, so
 * all ranks get the same bits; the bias is added once, after the sum.
 *   blocks     host array [world] of device pointers: every rank's peer-visible block for this call site (blocks[rank] is
 *              this rank's own; the others are the peers' blocks as mapped into this process, e.g. torch symmetric
 *              memory or CUDA IPC).  Layout of a block: mxfp4_peer_partial_offset() bytes of flags, zeroed once before
 *              the first call on every rank, then the rank's partial, [M, ld] bf16.  The GEMM writes the partial there.
 *   epoch      local device uint32[2], zeroed once: the call counter of this call site (device-side, so a launch
 *              captured in a CUDA graph works on every replay).
 *   status_dev optional local device int: receives MXFP4_E_TIMEOUT if a peer did not show up within the wait bound (ten
 *              seconds; MXFP4_PEER_WAIT_MS in the environment sets another).  The launch then writes NaN to `out` instead of a sum.
 * All ranks must make the same sequence of calls per call site.  N, ld, ldo multiples of 8; world <= 8.
 */
MXFP4_API int64_t mxfp4_peer_block_bytes(int64_t M, int64_t ld);
MXFP4_API int64_t mxfp4_peer_partial_offset(void);
MXFP4_API int mxfp4_peer_allreduce(void* const* blocks, int world, int rank, uint32_t* epoch, const void* bias_bf16, void* out_bf16,
                                   int64_t ldo, int64_t M, int64_t N, int64_t ld, int* status_dev, void* stream);

/*
 * What lies between two GEMMs of a transformer block, as ONE kernel that ends in the GEMM's activation format.  The
 * reference has no counterpart: it leaves these steps to the model's PyTorch code (what it does own is the layer on
 * either side, MXLinear.forward, src/mxfp4/modules.py:114-140).  One launch
 *   1. gathers the result of the GEMM in front: a bf16 matrix (in_bf16), the float32 partial sums of a K-split
 *      (in_f32, `splits` of them `split_stride` elements apart; they are summed here in fixed order, so no separate
 *      reduction kernel runs), or -- tensor parallelism -- the bf16 partial products of all `world` ranks of a
 *      row-parallel layer in peer-visible blocks laid out as for mxfp4_peer_allreduce (flag handshake included: this
 *      IS the all-reduce);
 *   2. applies   MXFP4_ACT_RMSNORM   hidden = residual + (value + bias);  x = gamma * (hidden * rsqrt(mean(hidden^2) + eps))
 *                MXFP4_ACT_SILU_MUL  x = silu(value[:, 0:K]) * value[:, K:2K]
 *                MXFP4_ACT_SUM3      x = value[:, 0:K] + value[:, K:2K] + value[:, 2K:3K]
 *                MXFP4_ACT_IDENTITY  x = value
 *      rounding to bf16 after every step where the separate PyTorch operations would;
 *   3. quantises x as mxfp4_act_quantize does: packed [M, K/2] and blocked scales (mxfp4_act_scales_bytes(M, K)).
 * RMSNORM may also store `hidden` (the new residual stream; may alias `residual`), and with packed == NULL only that.
 * With all three sources absent RMSNORM takes value = 0 (the first layer of a stack).
 * peer_wait_done = 0 skips the second handshake ("everybody has finished reading"): allowed when every rank runs
 * another peer call site between two uses of this one, as the alternating attention / MLP layers of a model do.
 * Pointers 16-byte aligned, row pitches multiples of 8 elements, K a multiple of 32 and at most 32768.
 */
#define MXFP4_ACT_RMSNORM 1
#define MXFP4_ACT_SILU_MUL 2
#define MXFP4_ACT_SUM3 3
#define MXFP4_ACT_IDENTITY 4
typedef struct mxfp4_act_fused_args {
    int op;
    const void* in_bf16;       /* device bf16 [M, ld_in] or NULL */
    const void* in_f32;        /* device float32 [splits][M][ld_in] or NULL */
    int splits;
    int64_t split_stride;      /* elements between two partial sums */
    int64_t ld_in;
    void* const* peer_blocks;  /* host array [world] of device pointers, or NULL */
    int world, rank;
    uint32_t* epoch;           /* device uint32[2], zeroed once (call counter of this call site) */
    int peer_wait_done;
    int* status_dev;           /* optional device int: receives MXFP4_E_TIMEOUT; hidden_out is then NaN, codes zero */
    const void* bias;          /* bf16 [K] or NULL */
    const void* residual;      /* bf16 [M, ld_res] or NULL */
    int64_t ld_res;
    void* hidden_out;          /* bf16 [M, ld_hid] or NULL */
    int64_t ld_hid;
    float eps;
    int64_t M, K;
    uint8_t* packed;           /* [M, K/2] or NULL */
    uint8_t* sf;               /* blocked scales */
    const void* gamma;         /* bf16 [K] or NULL: the norm's learned weight (RMSNORM) */
    void* const* peer_results; /* host array [world] of device pointers or NULL: two-shot mode (see below) */
    uint32_t* owner_count;     /* device uint32, zeroed once (two-shot mode) */
} mxfp4_act_fused_args;
/* Two-shot mode of the peer sum (peer_results != NULL, M >= world): the rows are split over the ranks in contiguous chunks of
 * ceil(M / world); every rank sums, normalises and quantises only ITS rows (reading 1/world of every partial), leaves hidden
 * state, codes and scales in its peer-visible result block (ceil(M / world) rows of mxfp4_act_fused_result_row_bytes(K) bytes)
 * and copies the other rows from their owners' blocks: (world-1)/world * 2.3 units of NVLink traffic per rank instead of
 * world-1, which pays from four ranks up and for prefill-sized M.  No call-site interleaving is assumed in this mode. */
MXFP4_API int64_t mxfp4_act_fused_result_row_bytes(int64_t K);
MXFP4_API int mxfp4_act_fused(const mxfp4_act_fused_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MXFP4_B200_H_ */
