// All-gather of column shards over NVLink peer memory, one kernel per rank.
//
// A row-sharded linear leaves every rank with local[rows, cols] = its columns
// r*cols .. (r+1)*cols of the full activation. This kernel writes that shard
// straight into the full[rows, world*cols] buffer of EVERY rank (its own
// included) with plain peer stores, publishes a per-rank epoch in each peer's
// flag array once all of its stores are fenced, and returns when the local flag
// array shows the same epoch from every rank - so the next kernel in the stream
// sees the complete activation. No library collective, no staging copy. Optionally
// the shard is also stored rounded to bf16 into a second buffer of every rank, the
// form the tensor-core linears read.
//
// Every rank runs the same sequence of gathers, so "epoch" is simply the number
// of gathers a rank has done; it lives in device memory, which keeps the kernel
// replayable from a CUDA graph. The wait is bounded by a wall-clock budget: when
// it runs out the kernel sets a status bit and returns instead of spinning.
//
// Buffer reuse: a peer may only overwrite full[] of call k+1 after this rank has
// consumed call k. Callers guarantee it by giving consecutive gathers different
// buffers (the decode step rotates through four per layer): a peer reaches its
// next use of a buffer only after this rank has joined the gathers in between,
// which it issues, in stream order, after the consumer of the earlier one.
#include "b2_common.cuh"
#include "b2_kernels.h"

#include <cuda_bf16.h>

namespace b2 {
namespace {

constexpr int kThreads = 256;
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;   // 2 s

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct PeerGatherArgs {
    const float* local;           // [rows, cols]
    const uint64_t* peer_full;    // device array [world]: address of every rank's full[rows, world*cols]
    const uint64_t* peer_full16;  // nullable, same for every rank's bf16 copy of full (same shape)
    const uint64_t* peer_flags;   // device array [world]: address of every rank's flag array uint32[world]
    uint32_t* state;              // local: [0] epoch of the last gather, [1] CTAs done in this launch
    uint32_t* status;             // local status word (B2_PEER_STATUS_TIMEOUT: wait budget ran out)
    uint32_t rows, cols, rank, world;
};

__global__ void __launch_bounds__(kThreads)
peer_gather_kernel(const PeerGatherArgs a) {
    const uint32_t epoch = a.state[0] + 1u;   // read by every CTA before the last one bumps it
    const uint64_t full_cols = static_cast<uint64_t>(a.cols) * a.world;
    const uint64_t n4 = static_cast<uint64_t>(a.rows) * a.cols / 4;   // cols is a multiple of 4
    const uint32_t cols4 = a.cols / 4;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n4; i += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(a.local) + i);
        const uint64_t r = i / cols4, c4 = i % cols4;
        const uint64_t dst = r * full_cols + static_cast<uint64_t>(a.rank) * a.cols + c4 * 4;
        for (uint32_t p = 0; p < a.world; ++p) {
            float* full = reinterpret_cast<float*>(a.peer_full[p]);
            *reinterpret_cast<float4*>(full + dst) = v;
        }
        if (a.peer_full16 != nullptr) {   // the form the tensor-core linears read: no conversion pass after the gather
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            for (uint32_t p = 0; p < a.world; ++p) {
                __nv_bfloat16* full16 = reinterpret_cast<__nv_bfloat16*>(a.peer_full16[p]);
                *reinterpret_cast<uint2*>(full16 + dst) = packed;
            }
        }
    }
    // One system-scope fence per CTA, by the thread that then counts the CTA in: the barrier orders
    // every thread's stores before it, and the fence is cumulative over what the barrier ordered.
    __syncthreads();
    __shared__ uint32_t s_last;
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t done = atomicAdd(&a.state[1], 1u) + 1u;
        s_last = done == gridDim.x ? 1u : 0u;
    }
    __syncthreads();
    if (s_last == 0u) return;

    // Last CTA of this rank: every store of the launch is fenced. Publish, then wait for the peers.
    if (threadIdx.x < a.world) {
        uint32_t* flags = reinterpret_cast<uint32_t*>(a.peer_flags[threadIdx.x]);
        st_release_sys(flags + a.rank, epoch);
    }
    if (threadIdx.x < a.world) {
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(a.peer_flags[a.rank]) + threadIdx.x;
        const unsigned long long t0 = global_ns();
        uint32_t polls = 0;
        // epochs compare modulo 2^32: "reached" means not behind
        while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
            if ((++polls & 1023u) == 0u && global_ns() - t0 > kWaitBudgetNs) {
                atomicOr(a.status, B2_PEER_STATUS_TIMEOUT);
                break;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        a.state[1] = 0u;
        a.state[0] = epoch;
        __threadfence();
    }
}

}  // namespace

int32_t launch_peer_gather(const DeviceContext& ctx, const float* local, uint64_t rows, uint64_t cols,
                           const uint64_t* peer_full, const uint64_t* peer_full_bf16, const uint64_t* peer_flags,
                           uint32_t rank, uint32_t world, uint32_t* state, uint32_t* status, cudaStream_t stream) {
    PeerGatherArgs a;
    a.local = local;
    a.peer_full = peer_full;
    a.peer_full16 = peer_full_bf16;
    a.peer_flags = peer_flags;
    a.state = state;
    a.status = status;
    a.rows = static_cast<uint32_t>(rows);
    a.cols = static_cast<uint32_t>(cols);
    a.rank = rank;
    a.world = world;
    const uint64_t n4 = rows * cols / 4;
    uint64_t blocks = (n4 + kThreads - 1) / kThreads;
    // A few CTAs saturate the NVLink stores of a decode-sized shard; all of them must be resident
    // together (the last one to finish publishes), so stay far below the SM count.
    const uint64_t cap = static_cast<uint64_t>(ctx.sm_count > 8 ? ctx.sm_count / 4 : 2);
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    peer_gather_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(a);
    B2_CUDA_TRY(cudaGetLastError());
    return B2_STATUS_OK;
}

}  // namespace b2
