// Sum of the partial products of a row-parallel MXLinear over the ranks of one NVSwitch box, as one kernel over peer
// memory (plain P2P loads and stores, no NCCL, no multimem): every rank reads every rank's bf16 partial [M, N] from
// peer-visible buffers, adds them in float32 in rank order (so all ranks produce the same bits), adds the bias and
// writes its own bf16 result.
//
// Each rank owns one peer-visible block per call site:  [ flags: 2 * kMaxWorld uint32 | partial: M x ld bf16 ].
//   ready[r] (in MY block)  the number of the call for which rank r's partial is complete   (written by rank r)
//   done[r]  (in MY block)  the number of the call whose partials rank r has finished reading (written by rank r)
// Call numbers live on the device (epoch word, advanced by the last block of each launch), so a launch captured
// in a CUDA graph does the right thing on every replay.  A launch
//   1. publishes ready = n to every peer (the partial was written by earlier kernels on this stream),
//   2. waits until every peer's ready >= n,
//   3. sums,
//   4. publishes done = n and waits until every peer's done >= n: only then may the next GEMM at this call site
//      overwrite this rank's partial.
// Every wait is bounded (about ten seconds of clock64: ranks of a job may be seconds apart, a lost rank must not hang the
// others); a wait that runs out sets the status word, the launch writes NaN instead of a sum and finishes.
#include <cstdlib>

#include "mxfp4_common.cuh"

namespace mxfp4 {
namespace {

constexpr int kMaxWorld = 8;
constexpr long long kPeerWaitDefaultMs = 10000;   // ranks of one job can be seconds apart; MXFP4_PEER_WAIT_MS overrides

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 16 bytes from (possibly peer) memory, cached at most in L2 (the data changes between launches; L1 could be stale).
// Not volatile: the compiler is free to put many of these loads in flight before the first use.
__device__ __forceinline__ uint4 ld_cg_16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

struct PeerParams {
    uint8_t* block[kMaxWorld];   // every rank's peer-visible block (block[rank] is local)
    int world, rank;
    uint32_t* epoch;             // local: [0] calls completed at this call site, [1] block ticket of the running launch
    const __nv_bfloat16* bias;
    __nv_bfloat16* out;
    int64_t ldo, M, N, ld;       // ld: row pitch of the partials, elements
    int* status;
    long long wait_cycles;       // bound of each wait
};

// waits until every peer's counter in `mine[0..world)` has reached n; false when the bound ran out
__device__ __forceinline__ bool wait_all(const uint32_t* mine, int world, int rank, uint32_t n, long long limit) {
    const long long t0 = clock64();
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        while ((int32_t)(ld_acquire_sys(mine + r) - n) < 0) {
            if (clock64() - t0 > limit) return false;
        }
    }
    return true;
}

// U vectors of 8 bf16 per thread and iteration, all loads of all ranks issued before the first add
template <int U>
__global__ void __launch_bounds__(256) peer_allreduce_kernel(const PeerParams p) {
    __shared__ int s_ok;
    const uint32_t n = p.epoch[0] + 1;                          // stable: only the last block of a launch advances it, at its end
    uint32_t* my_flags = reinterpret_cast<uint32_t*>(p.block[p.rank]);
    if (blockIdx.x == 0 && threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(p.block[threadIdx.x]) + p.rank, n);     // ready[rank] in the peer's block
    }
    if (threadIdx.x == 0) s_ok = wait_all(my_flags, p.world, p.rank, n, p.wait_cycles) ? 1 : 0;
    __syncthreads();
    if (s_ok) {
        const int64_t vec_per_row = p.N / 8;
        const int64_t total = p.M * vec_per_row;
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
            uint4 v[U][kMaxWorld];
            int64_t off_in[U], off_out[U];
            int col[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t i = i0 + u * stride;
                const int64_t m = i / vec_per_row, c = (i - m * vec_per_row) * 8;
                off_in[u] = m * p.ld + c; off_out[u] = m * p.ldo + c; col[u] = (int)c;
                if (i < total) {
#pragma unroll
                    for (int r = 0; r < kMaxWorld; ++r)
                        if (r < p.world) v[u][r] = ld_cg_16(reinterpret_cast<const __nv_bfloat16*>(p.block[r] + 2 * kMaxWorld * 4) + off_in[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (i0 + u * stride >= total) break;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int r = 0; r < kMaxWorld; ++r) {
                    if (r < p.world) {
                        const uint32_t w[4] = {v[u][r].x, v[u][r].y, v[u][r].z, v[u][r].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[2 * j] += __uint_as_float(w[j] << 16);
                            acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
                        }
                    }
                }
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat16 a = __float2bfloat16_rn(acc[2 * j]), b = __float2bfloat16_rn(acc[2 * j + 1]);
                    if (p.bias) {
                        a = __float2bfloat16_rn(__bfloat162float(a) + __bfloat162float(p.bias[col[u] + 2 * j]));
                        b = __float2bfloat16_rn(__bfloat162float(b) + __bfloat162float(p.bias[col[u] + 2 * j + 1]));
                    }
                    o[j] = (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
                }
                *reinterpret_cast<uint4*>(p.out + off_out[u]) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    } else {
        // a peer did not show up: no sum exists.  The output becomes NaN, so that nothing downstream mistakes stale
        // memory for activations, and the status word says why.
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, MXFP4_E_TIMEOUT);
        const int64_t vec_per_row = p.N / 8;
        const int64_t total = p.M * vec_per_row;
        const uint4 nan4 = make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u);
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t m = i / vec_per_row, c = (i - m * vec_per_row) * 8;
            *reinterpret_cast<uint4*>(p.out + m * p.ldo + c) = nan4;
        }
    }
    // the last block to get here tells the peers that this rank has finished reading, waits for theirs and closes the call
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t ticket = atomicAdd(p.epoch + 1, 1u);
        if (ticket == gridDim.x - 1) {
            for (int r = 0; r < p.world; ++r)
                if (r != p.rank) st_release_sys(reinterpret_cast<uint32_t*>(p.block[r]) + kMaxWorld + p.rank, n);   // done[rank] in the peer's block
            if (!wait_all(my_flags + kMaxWorld, p.world, p.rank, n, p.wait_cycles) && p.status) atomicExch(p.status, MXFP4_E_TIMEOUT);
            p.epoch[1] = 0;
            __threadfence();
            p.epoch[0] = n;
        }
    }
}

}  // namespace
}  // namespace mxfp4

extern "C" int64_t mxfp4_peer_block_bytes(int64_t M, int64_t ld) {
    if (M <= 0 || ld <= 0) return 0;
    return 2 * mxfp4::kMaxWorld * 4 + M * ld * 2;
}

extern "C" int64_t mxfp4_peer_partial_offset(void) { return 2 * mxfp4::kMaxWorld * 4; }

extern "C" int mxfp4_peer_allreduce(void* const* blocks, int world, int rank, uint32_t* epoch, const void* bias_bf16, void* out_bf16,
                                    int64_t ldo, int64_t M, int64_t N, int64_t ld, int* status_dev, void* stream) {
    using namespace mxfp4;
    if (!blocks || !epoch || !out_bf16) { set_error("mxfp4_peer_allreduce: null pointer"); return MXFP4_E_BADARG; }
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) { set_error("mxfp4_peer_allreduce: world=%d rank=%d (at most %d ranks)", world, rank, kMaxWorld); return MXFP4_E_BADARG; }
    if (M < 0 || N < 0) { set_error("mxfp4_peer_allreduce: negative size"); return MXFP4_E_SHAPE; }
    if (M == 0 || N == 0) return MXFP4_OK;
    if (N % 8 || ld % 8 || ldo % 8 || ld < N || ldo < N) { set_error("mxfp4_peer_allreduce: N, ld and ldo must be multiples of 8 with ld, ldo >= N"); return MXFP4_E_SHAPE; }
    if ((uintptr_t)out_bf16 % 16) { set_error("mxfp4_peer_allreduce: out must be 16-byte aligned"); return MXFP4_E_ALIGN; }
    PeerParams p;
    for (int r = 0; r < kMaxWorld; ++r) p.block[r] = nullptr;
    for (int r = 0; r < world; ++r) {
        if (!blocks[r] || (uintptr_t)blocks[r] % 16) { set_error("mxfp4_peer_allreduce: block %d is null or not 16-byte aligned", r); return MXFP4_E_ALIGN; }
        p.block[r] = (uint8_t*)blocks[r];
    }
    p.world = world; p.rank = rank; p.epoch = epoch; p.bias = (const __nv_bfloat16*)bias_bf16; p.out = (__nv_bfloat16*)out_bf16;
    p.ldo = ldo; p.M = M; p.N = N; p.ld = ld; p.status = status_dev;
    long long ms = kPeerWaitDefaultMs;
    if (const char* e = getenv("MXFP4_PEER_WAIT_MS")) { const long long v = atoll(e); if (v > 0 && v <= 600000) ms = v; }
    p.wait_cycles = ms * 2000000ll;          // clock64 ticks at about 2 GHz
    const int64_t total = M * (N / 8);
    int64_t grid = (total + 255) / 256;
    const int64_t cap = (int64_t)num_sms() * 4;
    if (grid > cap) grid = cap;
    // more vectors per thread while few ranks leave registers for them
    if (world <= 2) peer_allreduce_kernel<4><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(p);
    else if (world <= 4) peer_allreduce_kernel<2><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(p);
    else peer_allreduce_kernel<1><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(p);
    MXFP4_CHECK_LAUNCH("mxfp4_peer_allreduce");
    return MXFP4_OK;
}
