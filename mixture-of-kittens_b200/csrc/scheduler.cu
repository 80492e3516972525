// Slot-table scheduler: router top-k ids of all ranks -> per-expert padded row ranges and the
// (peer rank, peer route) tables of this rank.  Integer-only, bit-exact with the reference
// scheduler (csrc/scheduler.cuh:35-147 in Mixture-of-Kittens): routes of one peer are ordered
// "thread-major" over 1024 virtual threads, peers are interleaved round-robin inside an expert,
// experts are padded to 256 rows.
//
// The reference rescans every peer's routes 2*El times.  Here every route is read exactly twice:
//   pass 1  one warp per chunk (4 virtual threads of one peer) histograms its routes per local
//           expert in shared memory                        -> chunk_hist[peer][chunk][expert]
//   pass 2  one warp per (expert, peer) turns the 256 chunk counts into exclusive offsets and
//           the total                                      -> cnt[expert][peer]
//   pass 3  every block rebuilds expert bases from cnt; one warp per chunk walks its routes in
//           order, ranks equal experts inside the warp with match.any, and writes the slots.
// Algorithmic traffic: 2 * W*T*K*4 B of route reads + 2 * capacity * 4 B of table writes.
#include <atomic>

#include "common.cuh"
#include "profile.cuh"

namespace mok {
namespace {

constexpr int kVThreads = 1024;           // virtual threads of the reference ordering
constexpr int kChunkVts = 4;              // virtual threads per warp-chunk
constexpr int kChunks = kVThreads / kChunkVts;   // 256 chunks per peer
constexpr int kWarpsPerBlock = 8;
constexpr int kBlockThreads = kWarpsPerBlock * 32;
constexpr int kPad = 256;                 // expert row padding

struct SchedParams {
    const int* topk;        // [W, R]
    int W, R, El, rank, capacity;
    int* peer_rank;         // [capacity]
    int* peer_token_idx;    // [capacity]
    int* num_tokens;        // [1]
    int* tokens_per_expert; // [El]
    int* chunk_hist;        // [W, kChunks, El]
    int* cnt;               // [El, W]
    int* status;
};

// Position `idx` of a chunk's route list -> route index r (or -1 past the end).  Virtual thread
// vt owns routes vt, vt+1024, ...; a chunk is the concatenation of its 4 virtual threads' lists.
__device__ __forceinline__ int chunk_route(int v0, int idx, int q, int rem) {
#pragma unroll
    for (int j = 0; j < kChunkVts; ++j) {
        const int vt = v0 + j;
        const int n = q + (vt < rem ? 1 : 0);
        if (idx < n) return vt + idx * kVThreads;
        idx -= n;
    }
    return -1;
}
__device__ __forceinline__ int chunk_len(int v0, int q, int rem) {
    int n = 0;
#pragma unroll
    for (int j = 0; j < kChunkVts; ++j) n += q + ((v0 + j) < rem ? 1 : 0);
    return n;
}

__global__ void __launch_bounds__(kBlockThreads) sched_count_kernel(SchedParams p) {
    extern __shared__ int smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int* hist = smem + warp * p.El;

    // fill both tables with -1 (unwritten slots), grid-stride
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.capacity; i += gridDim.x * blockDim.x) {
        p.peer_rank[i] = -1;
        p.peer_token_idx[i] = -1;
    }

    const int gchunk = blockIdx.x * kWarpsPerBlock + warp;     // over W * kChunks
    if (gchunk >= p.W * kChunks) return;
    const int peer = gchunk / kChunks, chunk = gchunk % kChunks;
    for (int e = lane; e < p.El; e += 32) hist[e] = 0;
    __syncwarp();

    const int q = p.R / kVThreads, rem = p.R % kVThreads;
    const int v0 = chunk * kChunkVts;
    const int len = chunk_len(v0, q, rem);
    const int first = p.rank * p.El;
    const int* routes = p.topk + static_cast<size_t>(peer) * p.R;
    for (int base = 0; base < len; base += 32) {
        const int r = chunk_route(v0, base + lane, q, rem);
        if (r >= 0) {
            const int e = routes[r] - first;
            if (e >= 0 && e < p.El) atomicAdd(&hist[e], 1);
        }
    }
    __syncwarp();
    int* out = p.chunk_hist + static_cast<size_t>(gchunk) * p.El;
    for (int e = lane; e < p.El; e += 32) out[e] = hist[e];
}

// one warp per (expert, peer): exclusive scan over the 256 chunks, in place
__global__ void __launch_bounds__(kBlockThreads) sched_scan_kernel(SchedParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x * kWarpsPerBlock + warp;       // e * W + peer
    if (pair >= p.El * p.W) return;
    const int e = pair / p.W, peer = pair % p.W;
    constexpr int kPerLane = kChunks / 32;                      // 8 consecutive chunks per lane
    int v[kPerLane];
    int sum = 0;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        v[j] = p.chunk_hist[(static_cast<size_t>(peer) * kChunks + lane * kPerLane + j) * p.El + e];
        sum += v[j];
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
    }
    int run = incl - sum;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
        p.chunk_hist[(static_cast<size_t>(peer) * kChunks + lane * kPerLane + j) * p.El + e] = run;
        run += v[j];
    }
    if (lane == 31) p.cnt[pair] = incl;
}

__global__ void __launch_bounds__(kBlockThreads) sched_place_kernel(SchedParams p) {
    extern __shared__ int smem[];
    int* s_cnt = smem;                        // [El * W]
    int* s_base = s_cnt + p.El * p.W;         // [El]
    int* s_run = s_base + p.El;               // [warps][El]
    __shared__ int s_warp_tot[kWarpsPerBlock];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int i = threadIdx.x; i < p.El * p.W; i += blockDim.x) s_cnt[i] = p.cnt[i];
    __syncthreads();
    // padded rows per expert -> exclusive scan over experts (block-wide, El <= 1024)
    int carry = 0;
    for (int e0 = 0; e0 < p.El; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        int padded = 0;
        if (e < p.El) {
            int tot = 0;
            for (int r = 0; r < p.W; ++r) tot += s_cnt[e * p.W + r];
            padded = (tot + kPad - 1) / kPad * kPad;
            if (blockIdx.x == 0) p.tokens_per_expert[e] = padded;
        }
        int incl = padded;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += n;
        }
        if (lane == 31) s_warp_tot[warp] = incl;
        __syncthreads();
        int warp_off = 0, block_tot = 0;
        for (int w = 0; w < kWarpsPerBlock; ++w) {
            if (w < warp) warp_off += s_warp_tot[w];
            block_tot += s_warp_tot[w];
        }
        if (e < p.El) s_base[e] = carry + warp_off + incl - padded;
        carry += block_tot;
        __syncthreads();
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        p.num_tokens[0] = carry;
        if (carry > p.capacity) report_status(p.status, MOK_STATUS_SCHEDULE_OVERFLOW, carry);
    }

    const int gchunk = blockIdx.x * kWarpsPerBlock + warp;
    if (gchunk >= p.W * kChunks) return;
    const int peer = gchunk / kChunks, chunk = gchunk % kChunks;
    int* run = s_run + warp * p.El;
    const int* start = p.chunk_hist + static_cast<size_t>(gchunk) * p.El;
    for (int e = lane; e < p.El; e += 32) run[e] = start[e];
    __syncwarp();

    const int q = p.R / kVThreads, rem = p.R % kVThreads;
    const int v0 = chunk * kChunkVts;
    const int len = chunk_len(v0, q, rem);
    const int first = p.rank * p.El;
    const int* routes = p.topk + static_cast<size_t>(peer) * p.R;
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int base = 0; base < len; base += 32) {
        const int r = chunk_route(v0, base + lane, q, rem);
        int e = -1;
        if (r >= 0) {
            e = routes[r] - first;
            if (e < 0 || e >= p.El) e = -1;
        }
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (e >= 0) {
            const int j = run[e] + __popc(same & lt_mask);
            int dst = s_base[e];
            for (int rr = 0; rr < p.W; ++rr) {
                const int c = s_cnt[e * p.W + rr];
                dst += min(c, j) + ((rr < peer && c > j) ? 1 : 0);
            }
            if (dst < p.capacity) {
                p.peer_rank[dst] = peer;
                p.peer_token_idx[dst] = r;
            }
        }
        __syncwarp();
        if (e >= 0 && (same & lt_mask) == 0) run[e] += __popc(same);   // lowest lane of each group
        __syncwarp();
    }
}

}  // namespace
}  // namespace mok

extern "C" size_t mok_schedule_scratch_bytes(int ep_size, int num_local_experts) {
    if (ep_size <= 0 || num_local_experts <= 0) return 0;
    return (static_cast<size_t>(ep_size) * mok::kChunks * num_local_experts +
            static_cast<size_t>(ep_size) * num_local_experts) * sizeof(int);
}

namespace mok {
// shared by the caller-scratch entry point; `scratch` is a device pointer
int launch_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                    int num_local_experts, int schedule_capacity, int rank,
                    int32_t* schedule_peer_rank, int32_t* schedule_peer_token_idx,
                    int32_t* num_tokens, int32_t* tokens_per_expert,
                    void* scratch, int32_t* status, cudaStream_t stream) {
    SchedParams p;
    p.topk = topk_all;
    p.W = ep_size;
    p.R = num_local_tokens * topk;
    p.El = num_local_experts;
    p.rank = rank;
    p.capacity = schedule_capacity;
    p.peer_rank = schedule_peer_rank;
    p.peer_token_idx = schedule_peer_token_idx;
    p.num_tokens = num_tokens;
    p.tokens_per_expert = tokens_per_expert;
    p.chunk_hist = static_cast<int*>(scratch);
    p.cnt = p.chunk_hist + static_cast<size_t>(ep_size) * kChunks * num_local_experts;
    p.status = status;

    const int chunk_blocks = (ep_size * kChunks + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const size_t smem_count = static_cast<size_t>(kWarpsPerBlock) * p.El * sizeof(int);
    const size_t smem_place = (static_cast<size_t>(p.El) * p.W + p.El + static_cast<size_t>(kWarpsPerBlock) * p.El) * sizeof(int);
    // The dynamic shared-memory ceiling is a sticky per-device attribute: set it once to what the largest accepted
    // problem needs, so that concurrent calls with different expert counts cannot lower it under one another.
    static std::atomic<bool> configured[64];
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        constexpr size_t kMaxCount = static_cast<size_t>(kWarpsPerBlock) * MOK_MAX_LOCAL_EXPERTS * sizeof(int);
        constexpr size_t kMaxPlace = (static_cast<size_t>(MOK_MAX_LOCAL_EXPERTS) * MOK_MAX_PEERS + MOK_MAX_LOCAL_EXPERTS +
                                      static_cast<size_t>(kWarpsPerBlock) * MOK_MAX_LOCAL_EXPERTS) * sizeof(int);
        MOK_CUDA_CHECK(cudaFuncSetAttribute(sched_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMaxCount)));
        MOK_CUDA_CHECK(cudaFuncSetAttribute(sched_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kMaxPlace)));
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    ProfScope prof(kSlotScheduler, stream, 3);
    sched_count_kernel<<<chunk_blocks, kBlockThreads, smem_count, stream>>>(p);
    const int pair_blocks = (p.El * p.W + kWarpsPerBlock - 1) / kWarpsPerBlock;
    sched_scan_kernel<<<pair_blocks, kBlockThreads, 0, stream>>>(p);
    sched_place_kernel<<<chunk_blocks, kBlockThreads, smem_place, stream>>>(p);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
}  // namespace mok

extern "C" int mok_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                            int num_local_experts, int schedule_capacity, int rank,
                            int32_t* schedule_peer_rank, int32_t* schedule_peer_token_idx,
                            int32_t* num_tokens, int32_t* tokens_per_expert,
                            void* scratch, size_t scratch_bytes, int32_t* status, void* stream) {
    if (!topk_all || !schedule_peer_rank || !schedule_peer_token_idx || !num_tokens || !tokens_per_expert || !scratch)
        return MOK_ERR_INVALID;
    if (ep_size < 1 || ep_size > MOK_MAX_PEERS || rank < 0 || rank >= ep_size) return MOK_ERR_INVALID;
    if (num_local_tokens <= 0 || topk <= 0 || schedule_capacity <= 0) return MOK_ERR_INVALID;
    if (num_local_experts < 1 || num_local_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_INVALID;
    if (scratch_bytes < mok_schedule_scratch_bytes(ep_size, num_local_experts)) return MOK_ERR_INVALID;
    return mok::launch_schedule(topk_all, ep_size, num_local_tokens, topk, num_local_experts, schedule_capacity, rank,
                                schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                                scratch, status, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Scheduler variant for callers that must not allocate device memory.
//
// Some hosts of this library run under a fixed memory plan: an inference server that sized its
// arena at start-up, a real-time loop where cudaMalloc's implicit device synchronisation is not
// acceptable, or a plug-in boundary that hands out no allocator at all.  Such a caller cannot
// provide the chunk-histogram scratch mok_schedule() asks for.  This entry point keeps that
// scratch in a fixed array inside the library image instead, so the call needs nothing beyond the
// caller's inputs and outputs.
//
// The array is a file-scope __device__ object: every GPU that loads the library carries it
// (kStaticScratchBytes) until the process exits.  In host code its name is only a handle, not a
// device address, so the address is looked up with cudaGetSymbolAddress once per device, with that
// device current, on the first call made on that device; later calls reuse the cached address.
// That first call should therefore be made outside any stream capture.
//
// All calls on one GPU share the array.  The kernels overwrite every element they later read, so
// nothing has to be cleared between calls, but two calls whose kernels overlap on the GPU (two
// streams, or two threads) race on it: run them one after the other.
// ---------------------------------------------------------------------------------------------
namespace mok {
namespace {
constexpr size_t kStaticScratchBytes = 4u << 20;   // enough for ep_size * num_local_experts <= 4080
static __device__ __align__(256) unsigned char g_static_sched_scratch[kStaticScratchBytes];
std::atomic<void*> g_static_scratch_addr[64];    // per device; two threads that race on the first call store the same address

int static_scratch_for_current_device(void** out) {
    int dev = -1;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MOK_ERR_UNSUPPORTED;
    void* ptr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_sched_scratch);
        if (err != cudaSuccess || ptr == nullptr) { note_cuda_error(err, __FILE__, __LINE__); return MOK_ERR_CUDA; }
        g_static_scratch_addr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return MOK_OK;
}
}  // namespace
}  // namespace mok

extern "C" size_t mok_schedule_static_max_scratch_bytes(void) { return mok::kStaticScratchBytes; }

extern "C" int mok_schedule_static(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                                   int num_local_experts, int schedule_capacity, int rank,
                                   int32_t* schedule_peer_rank, int32_t* schedule_peer_token_idx,
                                   int32_t* num_tokens, int32_t* tokens_per_expert, int32_t* status, void* stream) {
    if (!topk_all || !schedule_peer_rank || !schedule_peer_token_idx || !num_tokens || !tokens_per_expert)
        return MOK_ERR_INVALID;
    if (ep_size < 1 || ep_size > MOK_MAX_PEERS || rank < 0 || rank >= ep_size) return MOK_ERR_INVALID;
    if (num_local_tokens <= 0 || topk <= 0 || schedule_capacity <= 0) return MOK_ERR_INVALID;
    if (num_local_experts < 1 || num_local_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_INVALID;
    if (mok_schedule_scratch_bytes(ep_size, num_local_experts) > mok::kStaticScratchBytes) return MOK_ERR_TOO_LARGE;
    void* scratch = nullptr;
    const int rc = mok::static_scratch_for_current_device(&scratch);
    if (rc != MOK_OK) return rc;
    return mok::launch_schedule(topk_all, ep_size, num_local_tokens, topk, num_local_experts, schedule_capacity, rank,
                                schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                                scratch, status, static_cast<cudaStream_t>(stream));
}
