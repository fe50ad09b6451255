// Everything between two GEMMs of a transformer block, as ONE row-wise kernel that ends in the GEMM's own MXFP4
// activation format (mxfp4_act_fused).
//
// The reference runs each linear layer as dequantise + F.linear (src/mxfp4/modules.py:114-140) and leaves what lies
// between two layers (residual add, normalisation, SwiGLU) to the model's own PyTorch code.  With an FP4 GEMM every such
// gap would cost several small launches plus the activation quantiser; here one kernel per gap
//   1. gathers the previous GEMM's result: a bf16 matrix, the float32 partial sums of a K-split (summed here, in fixed
//      order, so the separate reduction kernel disappears), or -- tensor parallelism -- the bf16 partial products of
//      all ranks of a row-parallel layer, read over NVLink peer memory after a flag handshake (the all-reduce);
//   2. applies the step in between:
//        RMSNORM   hidden = residual + value (+ bias);  x = hidden * rsqrt(mean(hidden^2) + eps) (* gamma)
//        SILU_MUL  x = silu(value[:, :K]) * value[:, K:2K]
//        SUM3      x = value[:, :K] + value[:, K:2K] + value[:, 2K:3K]
//        IDENTITY  x = value
//      with the bf16 roundings the unfused PyTorch operations would make after each step;
//   3. quantises x exactly as mxfp4_act_quantize does and writes packed codes + blocked scales.
// One CTA per activation row; a thread owns a few 8-element chunks and keeps them in registers between the two passes
// of the normalisation; the four lanes of a 32-element block find its maximum with two warp shuffles.
#include <cstdlib>

#include "mxfp4_common.cuh"

namespace mxfp4 {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxChunksPerThread = 8;      // 512 threads x 8 chunks x 8 elements: K <= 32768

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
    uint16_t o;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(o) : "f"(hi), "f"(lo));
    return o;
}
__device__ __forceinline__ int64_t blocked_offset(int64_t row, int64_t kb, int64_t kstages) {
    return ((row >> 7) * kstages + (kb >> 3)) * 1024 + ((kb >> 2) & 1) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kb & 3);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct FusedParams {
    int op;
    // source of the value
    const __nv_bfloat16* in_bf16;     // [M, ld_in]                       (splits == 0, world == 1)
    const float* in_f32;              // [splits][M][ld_in] partial sums  (splits >= 1)
    int splits;
    int64_t split_stride, ld_in;
    const uint8_t* peer[kMaxWorld];   // every rank's peer-visible block: flags, then the bf16 partial [M, ld_in]   (world > 1)
    int world, rank;
    uint32_t* epoch;
    long long wait_cycles;
    int wait_done;                    // also wait for the "done" handshake (call sites that are reused back to back)
    uint8_t* result[kMaxWorld];       // two-shot mode: every rank's peer-visible result block (rows it owns: hidden | codes | scales)
    int two_shot;                     // rows are split over the ranks; every rank reduces its own rows and fetches the others' results
    int64_t rows_per;                 // rows a rank owns (the last rank may own fewer)
    int64_t res_row_bytes;
    uint32_t* owner_count;            // local device counter of this rank's finished owned rows
    int* status;
    const __nv_bfloat16* bias;        // [K] or null, added to the value
    const __nv_bfloat16* gamma;       // [K] or null (RMSNORM): the norm's learned weight
    const __nv_bfloat16* residual;    // [M, ld_res] or null (RMSNORM)
    int64_t ld_res;
    __nv_bfloat16* hidden_out;        // [M, ld_hid] or null (RMSNORM): residual + value
    int64_t ld_hid;
    float eps;
    int64_t M, K;
    uint8_t* packed;                  // [M, K/2] or null (then only hidden_out is produced)
    uint8_t* sf;
    int64_t kstages, m_pad;
};

constexpr int kPeerFlagBytes = 2 * kMaxWorld * 4;

__device__ __forceinline__ void unpack8(const uint4& w, float (&v)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) { v[2 * t] = __uint_as_float(u[t] << 16); v[2 * t + 1] = __uint_as_float(u[t] & 0xFFFF0000u); }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {      // values exactly representable in bf16
    uint32_t u[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) u[t] = (__float_as_uint(v[2 * t]) >> 16) | (__float_as_uint(v[2 * t + 1]) & 0xFFFF0000u);
    return make_uint4(u[0], u[1], u[2], u[3]);
}

// 8 consecutive values of one row, starting at column c, from whichever source the call uses, rounded to bf16 as the
// GEMM's own output / the split-K reduction / the peer reduction would have left them
__device__ __forceinline__ void load_value8(const FusedParams& p, int64_t m, int64_t c, float (&v)[8]) {
    if (p.world > 1) {
        uint4 w[kMaxWorld];
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)        // all ranks' loads in flight together; at most L2 (the data changes between launches)
            if (r < p.world) w[r] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.peer[r] + kPeerFlagBytes) + m * p.ld_in + c));
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r) {
            if (r < p.world) {
                float t[8];
                unpack8(w[r], t);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += t[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bf16_round(acc[i]);      // rank order, float32, rounded once: same bits on every rank
    } else if (p.splits >= 1) {
        const float* src = p.in_f32 + m * p.ld_in + c;
        float4 a = __ldcs(reinterpret_cast<const float4*>(src)), b = __ldcs(reinterpret_cast<const float4*>(src) + 1);
#pragma unroll 4
        for (int s = 1; s < p.splits; ++s) {
            const float4 a2 = __ldcs(reinterpret_cast<const float4*>(src + s * p.split_stride));
            const float4 b2 = __ldcs(reinterpret_cast<const float4*>(src + s * p.split_stride) + 1);
            a.x += a2.x; a.y += a2.y; a.z += a2.z; a.w += a2.w;
            b.x += b2.x; b.y += b2.y; b.z += b2.z; b.w += b2.w;
        }
        v[0] = bf16_round(a.x); v[1] = bf16_round(a.y); v[2] = bf16_round(a.z); v[3] = bf16_round(a.w);
        v[4] = bf16_round(b.x); v[5] = bf16_round(b.y); v[6] = bf16_round(b.z); v[7] = bf16_round(b.w);
    } else if (p.in_bf16 != nullptr) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.in_bf16 + m * p.ld_in + c)), v);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;                    // no GEMM in front (first layer): hidden = residual
    }
}

// One CTA per activation row; a thread owns NB chunks of 8 consecutive elements (one 128-bit access each) and parks them
// as bf16 pairs between the two passes of the normalisation; the four lanes of a 32-element block share its maximum with
// two shuffles.  Many small chunks instead of whole blocks per thread: the code stays short (these kernels run for a few
// microseconds, so instruction fetch counts) and a row's loads are all in flight together.
template <int NB>
__global__ void __launch_bounds__(512) act_fused_kernel(const FusedParams p) {
    __shared__ float s_red[16];
    __shared__ int s_ok;
    // chained launches: the GEMM behind this kernel may be scheduled now; this kernel touches no global memory before the
    // kernel in front of it has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t kblocks = p.K / 32, chunks = p.K / 8;
    const int tid = threadIdx.x, T = blockDim.x;
    // Row of this CTA.  In two-shot mode the rows this rank owns come first in launch order: they never wait for another
    // rank's results, so the CTAs that do wait (for rows other ranks own) cannot keep them off the SMs.
    int64_t m = blockIdx.x;
    int owner = p.rank;
    int64_t own_lo = 0, own_n = 0;
    if (p.two_shot) {
        own_lo = p.rows_per * p.rank;
        own_n = own_lo >= p.M ? 0 : (p.M - own_lo < p.rows_per ? p.M - own_lo : p.rows_per);
        if ((int64_t)blockIdx.x < own_n) m = own_lo + blockIdx.x;
        else { m = blockIdx.x - own_n; if (m >= own_lo) m += own_n; }
        owner = m < p.M ? (int)(m / p.rows_per) : p.rank;
    }
    const bool fetch = p.two_shot && m < p.M && owner != p.rank;      // this row's results come from the rank that owns it

    uint32_t n = 0;
    if (p.world > 1) {
        // ---- all-reduce handshake: this rank's partial is complete (earlier kernels of this stream wrote it); tell the
        // peers, then wait until theirs are
        n = p.epoch[0] + 1;                       // stable during the launch: only its last CTA advances it, at its end
        uint32_t* my_flags = reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(p.peer[p.rank]));
        if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
            __threadfence_system();
            st_release_sys(reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(p.peer[tid])) + p.rank, n);     // ready[rank] in the peer's block
        }
        if (tid == 0) {
            int ok = 1;
            const long long t0 = clock64();
            if (fetch) {
                // the owner's "my rows of call n are in my result block"
                while ((int32_t)(ld_acquire_sys(my_flags + kMaxWorld + owner) - n) < 0) {
                    if (clock64() - t0 > p.wait_cycles) { ok = 0; break; }
                }
            } else {
                for (int r = 0; r < p.world && ok; ++r) {
                    if (r == p.rank) continue;
                    while ((int32_t)(ld_acquire_sys(my_flags + r) - n) < 0) {
                        if (clock64() - t0 > p.wait_cycles) { ok = 0; break; }
                    }
                }
            }
            s_ok = ok;
        }
        __syncthreads();
        if (!s_ok) {
            // a peer did not show up: no sum exists.  hidden_out becomes NaN so that nothing downstream mistakes stale
            // memory for activations; the codes become zeros; the status word says why.
            if (tid == 0 && p.status) atomicExch(p.status, MXFP4_E_TIMEOUT);
            if (m < p.M) {
                // (two-shot: the rows this rank owns go to its result block as NaN too, so the peers that fetch them see it)
                uint8_t* res = (p.two_shot && !fetch) ? p.result[p.rank] + (m - own_lo) * p.res_row_bytes : nullptr;
                for (int64_t ci = tid; ci < chunks; ci += T) {
                    if (p.hidden_out) *reinterpret_cast<uint4*>(p.hidden_out + m * p.ld_hid + ci * 8) = make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u);
                    if (p.packed) *reinterpret_cast<uint32_t*>(p.packed + m * (kblocks * 16) + ci * 4) = 0u;
                    if (res) {
                        *reinterpret_cast<uint4*>(res + ci * 16) = make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u);
                        *reinterpret_cast<uint32_t*>(res + p.K * 2 + ci * 4) = 0u;
                    }
                }
            }
        }
    }

    if (fetch && s_ok) {
        // ---- second shot: copy the row's hidden state, codes and scales from the owner's result block over NVLink
        const uint8_t* src = p.result[owner] + (m - p.rows_per * owner) * p.res_row_bytes;
        for (int64_t ci = tid; ci < chunks; ci += T) {
            if (p.hidden_out) *reinterpret_cast<uint4*>(p.hidden_out + m * p.ld_hid + ci * 8) = __ldcg(reinterpret_cast<const uint4*>(src) + ci);
            if (p.packed) *reinterpret_cast<uint32_t*>(p.packed + m * (kblocks * 16) + ci * 4) = __ldcg(reinterpret_cast<const uint32_t*>(src + p.K * 2) + ci);
        }
        if (p.packed)
            for (int64_t kb = tid; kb < kblocks; kb += T) p.sf[blocked_offset(m, kb, p.kstages)] = __ldcg(src + p.K * 2 + p.K / 2 + kb);
    }
    const bool row_ok = m < p.M && !fetch && (p.world == 1 || s_ok);
    uint8_t* res_row = (p.two_shot && row_ok) ? p.result[p.rank] + (m - own_lo) * p.res_row_bytes : nullptr;
    if (row_ok) {
        uint4 xp[NB];
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < NB; ++it) {
            const int64_t ci = tid + (int64_t)it * T;
            if (ci < chunks) {
                const int64_t c = ci * 8;
                float x[8];
                load_value8(p, m, c, x);
                if (p.op == MXFP4_ACT_RMSNORM) {
                    if (p.bias) {
                        float bv[8];
                        unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + c)), bv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) x[i] = bf16_round(x[i] + bv[i]);
                    }
                    if (p.residual) {
                        float rv[8];
                        unpack8(__ldg(reinterpret_cast<const uint4*>(p.residual + m * p.ld_res + c)), rv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) x[i] = bf16_round(rv[i] + x[i]);
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
                    xp[it] = pack8(x);
                    if (p.hidden_out) *reinterpret_cast<uint4*>(p.hidden_out + m * p.ld_hid + c) = xp[it];
                    if (res_row) *reinterpret_cast<uint4*>(res_row + c * 2) = xp[it];
                } else if (p.op == MXFP4_ACT_SILU_MUL) {
                    float u[8];
                    load_value8(p, m, p.K + c, u);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float sl = bf16_round(x[i] / (1.0f + expf(-x[i])));     // silu in float32, rounded as the bf16 op would
                        x[i] = bf16_round(sl * u[i]);
                    }
                    xp[it] = pack8(x);
                } else if (p.op == MXFP4_ACT_IDENTITY) {
                    xp[it] = pack8(x);
                } else {   // MXFP4_ACT_SUM3
                    float a[8];
                    load_value8(p, m, p.K + c, a);
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = bf16_round(x[i] + a[i]);
                    load_value8(p, m, 2 * p.K + c, a);
#pragma unroll
                    for (int i = 0; i < 8; ++i) x[i] = bf16_round(x[i] + a[i]);
                    xp[it] = pack8(x);
                }
            }
        }
        float r = 1.0f;
        if (p.op == MXFP4_ACT_RMSNORM && p.packed) {
            // sum of squares over the row: warp shuffle, then across the warps of the CTA
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            if ((tid & 31) == 0) s_red[tid >> 5] = ss;
            __syncthreads();
            float tot = 0.0f;
            for (int w = 0; w < (T >> 5); ++w) tot += s_red[w];
            r = rsqrtf(tot / (float)p.K + p.eps);
        }
        if (p.packed) {
#pragma unroll
            for (int it = 0; it < NB; ++it) {
                const int64_t ci = tid + (int64_t)it * T;
                // whole warps go through the shuffles (chunks is a multiple of 4, so a block's four lanes are in or out together)
                float x[8];
                float amax = 0.0f;
                if (ci < chunks) {
                    unpack8(xp[it], x);
                    float gm[8];
                    const bool scaled = p.op == MXFP4_ACT_RMSNORM && p.gamma != nullptr;
                    if (scaled) unpack8(__ldg(reinterpret_cast<const uint4*>(p.gamma + ci * 8)), gm);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (p.op == MXFP4_ACT_RMSNORM) x[i] = bf16_round(x[i] * r);
                        if (scaled) x[i] = bf16_round(gm[i] * x[i]);          // weight * normalised, both bf16
                        amax = fmaxf(amax, fabsf(x[i]));
                    }
                }
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
                if (ci < chunks) {
                    // the arithmetic of act_quantize_kernel: scale 2^ceil(log2(amax/6)), codes by cvt.rn.satfinite.e2m1x2
                    const uint32_t amax16 = __float_as_uint(amax) >> 16;                     // the values are bf16: the low half is zero
                    int b = (int)(amax16 >> 7) - 2 + ((amax16 & 0x7Fu) > 0x40u ? 1 : 0);
                    b = b < 0 ? 0 : (b > 254 ? 254 : b);
                    const float inv = b == 0 ? __uint_as_float(0x7F000000u) : (b == 254 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(254 - b) << 23));
                    uint32_t word = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) word |= cvt_e2m1x2(x[2 * j] * inv, x[2 * j + 1] * inv) << (8 * j);   // even element in the high nibble
                    *reinterpret_cast<uint32_t*>(p.packed + m * (kblocks * 16) + ci * 4) = word;
                    if ((ci & 3) == 0) p.sf[blocked_offset(m, ci >> 2, p.kstages)] = (uint8_t)b;
                    if (res_row) {
                        *reinterpret_cast<uint32_t*>(res_row + p.K * 2 + ci * 4) = word;
                        if ((ci & 3) == 0) res_row[p.K * 2 + p.K / 2 + (ci >> 2)] = (uint8_t)b;
                    }
                }
            }
        }
    }
    // scale bytes of the padding (rows up to a multiple of 128, blocks up to a whole K stage) are zero
    if (p.packed) {
        const int64_t kb_pad = p.kstages * 8;
        if (m < p.M) {
            for (int64_t kb = kblocks + tid; kb < kb_pad; kb += T) p.sf[blocked_offset(m, kb, p.kstages)] = 0;
        } else {
            for (int64_t kb = tid; kb < kb_pad; kb += T) p.sf[blocked_offset(m, kb, p.kstages)] = 0;
        }
    }

    if (p.two_shot && p.world > 1) {
        // first shot complete for this row; the last of this rank's owned rows tells every peer that the result block is ready
        __syncthreads();
        if (tid == 0 && !fetch && m < p.M) {
            __threadfence_system();
            const uint32_t done_rows = atomicAdd(p.owner_count, 1u);
            if ((int64_t)done_rows == own_n - 1) {
                *p.owner_count = 0;
                for (int rr = 0; rr < p.world; ++rr)
                    if (rr != p.rank) st_release_sys(reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(p.peer[rr])) + kMaxWorld + p.rank, n);
            }
        }
    }
    if (p.world > 1) {
        // the last CTA to get here closes the call: tells the peers that this rank has finished reading, optionally waits
        // for the same from them, then advances the call number
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const uint32_t ticket = atomicAdd(p.epoch + 1, 1u);
            if (ticket == gridDim.x - 1) {
                // "this rank has finished reading call n" is always published (a plain store per peer), so that the call
                // site stays usable by launches that do wait for it; the wait itself is optional
                uint32_t* my_flags = reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(p.peer[p.rank]));
                if (!p.two_shot)
                    for (int rr = 0; rr < p.world; ++rr)
                        if (rr != p.rank) st_release_sys(reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(p.peer[rr])) + kMaxWorld + p.rank, n);
                if (p.wait_done && !p.two_shot) {
                    const long long t0 = clock64();
                    bool ok = true;
                    for (int rr = 0; rr < p.world && ok; ++rr) {
                        if (rr == p.rank) continue;
                        while ((int32_t)(ld_acquire_sys(my_flags + kMaxWorld + rr) - n) < 0) {
                            if (clock64() - t0 > p.wait_cycles) { ok = false; break; }
                        }
                    }
                    if (!ok && p.status) atomicExch(p.status, MXFP4_E_TIMEOUT);
                }
                p.epoch[1] = 0;
                __threadfence();
                p.epoch[0] = n;
            }
        }
    }
}

}  // namespace
}  // namespace mxfp4

extern "C" int64_t mxfp4_act_fused_result_row_bytes(int64_t K) {
    if (K <= 0) return 0;
    return K * 2 + K / 2 + (K / 32 + 15) / 16 * 16;          // hidden (bf16) | codes | scale bytes, 16-byte aligned rows
}

extern "C" int mxfp4_act_fused(const mxfp4_act_fused_args* a, void* stream) {
    using namespace mxfp4;
    if (!a) { set_error("mxfp4_act_fused: null argument block"); return MXFP4_E_BADARG; }
    if (a->op != MXFP4_ACT_RMSNORM && a->op != MXFP4_ACT_SILU_MUL && a->op != MXFP4_ACT_SUM3 && a->op != MXFP4_ACT_IDENTITY) {
        set_error("mxfp4_act_fused: unknown op %d", a->op);
        return MXFP4_E_BADARG;
    }
    if (a->M < 0 || a->K < 0) { set_error("mxfp4_act_fused: negative size"); return MXFP4_E_SHAPE; }
    if (a->M == 0 || a->K == 0) return MXFP4_OK;
    if (a->K % 32) { set_error("mxfp4_act_fused: K=%lld is not a multiple of 32", (long long)a->K); return MXFP4_E_SHAPE; }
    if (a->K > (int64_t)512 * kMaxChunksPerThread * 8) {
        set_error("mxfp4_act_fused: K=%lld beyond %d (a row is held in registers)", (long long)a->K, 512 * kMaxChunksPerThread * 8);
        return MXFP4_E_UNSUPPORTED;
    }
    if (a->M > 0x7FFFFFFF) { set_error("mxfp4_act_fused: too many rows"); return MXFP4_E_SHAPE; }
    const int width = a->op == MXFP4_ACT_SILU_MUL ? 2 : (a->op == MXFP4_ACT_SUM3 ? 3 : 1);
    const int sources = (a->in_bf16 != nullptr) + (a->in_f32 != nullptr) + (a->world > 1);
    if (sources > 1) { set_error("mxfp4_act_fused: give one source (in_bf16, in_f32 partial sums, or peer blocks)"); return MXFP4_E_BADARG; }
    if (sources == 0 && !(a->op == MXFP4_ACT_RMSNORM && a->residual)) { set_error("mxfp4_act_fused: no input"); return MXFP4_E_BADARG; }
    if (sources == 1 && a->ld_in < width * a->K) { set_error("mxfp4_act_fused: ld_in %lld < %d * K", (long long)a->ld_in, width); return MXFP4_E_SHAPE; }
    if (a->in_f32 && (a->splits < 1 || a->splits > 64)) { set_error("mxfp4_act_fused: splits=%d", a->splits); return MXFP4_E_BADARG; }
    if (a->op != MXFP4_ACT_RMSNORM && (a->residual || a->hidden_out || a->bias || a->gamma || a->world > 1)) {
        set_error("mxfp4_act_fused: residual, hidden_out, bias, gamma and peer input belong to the RMSNORM op");
        return MXFP4_E_BADARG;
    }
    if (!a->packed && !a->hidden_out) { set_error("mxfp4_act_fused: nothing to produce"); return MXFP4_E_BADARG; }
    if (a->packed && !a->sf) { set_error("mxfp4_act_fused: packed without scale buffer"); return MXFP4_E_BADARG; }
    // 16-byte vector accesses everywhere
    if ((uintptr_t)a->in_bf16 % 16 || (uintptr_t)a->in_f32 % 16 || (uintptr_t)a->residual % 16 || (uintptr_t)a->hidden_out % 16 ||
        (uintptr_t)a->packed % 16 || (uintptr_t)a->bias % 16 || (uintptr_t)a->gamma % 16 || a->ld_in % 8 || a->ld_res % 8 || a->ld_hid % 8 || a->split_stride % 4) {
        set_error("mxfp4_act_fused: pointers must be 16-byte aligned and row pitches multiples of 8 elements");
        return MXFP4_E_ALIGN;
    }
    FusedParams p = {};
    p.op = a->op;
    p.in_bf16 = (const __nv_bfloat16*)a->in_bf16; p.in_f32 = (const float*)a->in_f32;
    p.splits = a->in_f32 ? a->splits : 0; p.split_stride = a->split_stride; p.ld_in = a->ld_in;
    p.world = a->world > 1 ? a->world : 1; p.rank = a->rank;
    if (p.world > 1) {
        if (p.world > kMaxWorld || a->rank < 0 || a->rank >= p.world || !a->peer_blocks || !a->epoch) {
            set_error("mxfp4_act_fused: world=%d rank=%d (at most %d ranks; peer_blocks and epoch are required)", a->world, a->rank, kMaxWorld);
            return MXFP4_E_BADARG;
        }
        for (int r = 0; r < p.world; ++r) {
            if (!a->peer_blocks[r] || (uintptr_t)a->peer_blocks[r] % 16) { set_error("mxfp4_act_fused: peer block %d is null or misaligned", r); return MXFP4_E_ALIGN; }
            p.peer[r] = (const uint8_t*)a->peer_blocks[r];
        }
        p.epoch = a->epoch;
        long long ms = 10000;
        if (const char* e = getenv("MXFP4_PEER_WAIT_MS")) { const long long v = atoll(e); if (v > 0 && v <= 600000) ms = v; }
        p.wait_cycles = ms * 2000000ll;
        p.wait_done = a->peer_wait_done ? 1 : 0;
        if (a->peer_results) {
            // two-shot: needs at least one row per rank and a counter
            if (!a->owner_count || a->M < p.world) { set_error("mxfp4_act_fused: two-shot mode needs owner_count and M >= world"); return MXFP4_E_BADARG; }
            for (int r = 0; r < p.world; ++r) {
                if (!a->peer_results[r] || (uintptr_t)a->peer_results[r] % 16) { set_error("mxfp4_act_fused: result block %d is null or misaligned", r); return MXFP4_E_ALIGN; }
                p.result[r] = (uint8_t*)a->peer_results[r];
            }
            p.two_shot = 1;
            p.rows_per = (a->M + p.world - 1) / p.world;
            p.res_row_bytes = mxfp4_act_fused_result_row_bytes(a->K);
            p.owner_count = a->owner_count;
        }
    }
    p.status = a->status_dev;
    p.bias = (const __nv_bfloat16*)a->bias; p.gamma = (const __nv_bfloat16*)a->gamma; p.residual = (const __nv_bfloat16*)a->residual; p.ld_res = a->ld_res;
    p.hidden_out = (__nv_bfloat16*)a->hidden_out; p.ld_hid = a->ld_hid;
    p.eps = a->eps; p.M = a->M; p.K = a->K;
    p.packed = a->packed; p.sf = a->sf;
    p.kstages = (a->K + 255) / 256; p.m_pad = (a->M + 127) / 128 * 128;
    const unsigned grid = (unsigned)(a->packed ? p.m_pad : a->M);      // padding rows only zero their scale bytes
    const int64_t chunks = a->K / 8;
    const unsigned threads = (unsigned)(chunks >= 512 ? 512 : (chunks + 31) / 32 * 32);
    const int nb = (int)((chunks + threads - 1) / threads);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t le;
    switch (nb) {
        case 1: le = launch_chained(act_fused_kernel<1>, grid, threads, st, p); break;
        case 2: le = launch_chained(act_fused_kernel<2>, grid, threads, st, p); break;
        case 3: le = launch_chained(act_fused_kernel<3>, grid, threads, st, p); break;
        case 4: le = launch_chained(act_fused_kernel<4>, grid, threads, st, p); break;
        case 5: case 6: le = launch_chained(act_fused_kernel<6>, grid, threads, st, p); break;
        default: le = launch_chained(act_fused_kernel<8>, grid, threads, st, p); break;
    }
    if (le != cudaSuccess) return cuda_fail(le, "mxfp4_act_fused");
    return MXFP4_OK;
}
