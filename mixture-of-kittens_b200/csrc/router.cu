// Router in front of the layer: logits -> softmax -> top-K -> renormalise, and its backward.
//
// The reference leaves routing to the caller (mok/functional.py:354-430 takes int64 top_experts and
// casts them to int32 before the all-gather); its tests build the routes with torch.topk on the
// logits and a softmax over the K selected values (tests/utils.py:82-84).  This kernel does the same
// in one pass over the logits and can write the int32 routes straight into every rank's all-gather
// buffer, which removes the cast and the separate all-gather launch.
//
// One warp per token.  Renormalised top-K probabilities do not depend on the other experts:
//   w_k = p_k / sum_{j in S} p_j = exp(l_k - m) / sum_{j in S} exp(l_j - m),   m = max logit,
// so only the K selected logits enter the arithmetic.  Selection is K rounds of a warp-wide argmax
// (value descending, index ascending on ties), which also gives torch.topk's sorted order.
// HBM-bound: reads T*E*4 bytes, writes T*K*(4+4[+8]) bytes.
#include <algorithm>

#include "common.cuh"
#include "gemm.cuh"
#include "profile.cuh"

namespace mok {
namespace {

constexpr int kRouterWarps = 8;

template <int kPerLane>
__global__ void __launch_bounds__(kRouterWarps * 32) router_topk_kernel(const float* __restrict__ logits, int T, int E, int K,
                                                                        int* __restrict__ top_i32, long long* __restrict__ top_i64,
                                                                        float* __restrict__ weights, PeerPtrs gather, int W,
                                                                        int rank) {
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
    const int warps_total = gridDim.x * kRouterWarps;
    for (int t = warp_global; t < T; t += warps_total) {
        const float* row = logits + static_cast<size_t>(t) * E;
        float v[kPerLane];
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            const int e = lane + 32 * j;
            const float lv = e < E ? row[e] : -INFINITY;
            v[j] = lv == lv ? lv : -INFINITY;       // a NaN logit ranks with -inf: it wins only when nothing else is left
        }
        unsigned taken = 0;                // bit j: this lane's j-th value has been selected
        float my_val = -INFINITY;          // lane k keeps the k-th selected (value, expert)
        int my_idx = 0;
        for (int k = 0; k < K; ++k) {
            float best = -INFINITY;
            int best_e = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < kPerLane; ++j) {
                const int e = lane + 32 * j;
                const bool free_slot = e < E && !((taken >> j) & 1u);
                // among equal values the lower expert index wins; the first free slot seeds the search
                if (free_slot && (v[j] > best || (v[j] == best && e < best_e) || best_e == 0x7fffffff)) { best = v[j]; best_e = e; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, off);
                const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
                if (oe != 0x7fffffff && (best_e == 0x7fffffff || ov > best || (ov == best && oe < best_e))) { best = ov; best_e = oe; }
            }
            if (best_e != 0x7fffffff && (best_e & 31) == lane) taken |= 1u << (best_e >> 5);
            if (lane == k) { my_val = best; my_idx = best_e == 0x7fffffff ? 0 : best_e; }
        }
        const float top = __shfl_sync(0xffffffffu, my_val, 0);
        float ex = lane < K ? __expf(my_val - top) : 0.0f;
        float sum = ex;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (lane < K) {
            const size_t o = static_cast<size_t>(t) * K + lane;
            weights[o] = ex / sum;
            if (top_i32) top_i32[o] = my_idx;
            if (top_i64) top_i64[o] = my_idx;
            for (int p = 0; p < W; ++p)
                static_cast<int*>(gather.p[p])[static_cast<size_t>(rank) * T * K + o] = my_idx;
        }
    }
}

// d_logits[t, e_k] = w_k * (d_w_k - sum_j w_j d_w_j) for the selected experts, 0 elsewhere
__global__ void __launch_bounds__(kRouterWarps * 32) router_topk_bwd_kernel(const int* __restrict__ top_i32, const float* __restrict__ weights,
                                                                            const float* __restrict__ d_weights, float* __restrict__ d_logits,
                                                                            int T, int E, int K) {
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
    const int warps_total = gridDim.x * kRouterWarps;
    for (int t = warp_global; t < T; t += warps_total) {
        float* row = d_logits + static_cast<size_t>(t) * E;
        for (int e = lane; e < E; e += 32) row[e] = 0.0f;
        __syncwarp();
        const size_t o = static_cast<size_t>(t) * K + lane;
        const float w = lane < K ? weights[o] : 0.0f;
        const float dw = lane < K ? d_weights[o] : 0.0f;
        float dot = w * dw;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        if (lane < K) {
            const int e = top_i32[o];
            if (e >= 0 && e < E) row[e] = w * (dw - dot);
        }
    }
}

template <int kPerLane>
void launch_topk(const float* logits, int T, int E, int K, int* i32, long long* i64, float* w, const PeerPtrs& gather, int W, int rank,
                 int blocks, cudaStream_t s) {
    router_topk_kernel<kPerLane><<<blocks, kRouterWarps * 32, 0, s>>>(logits, T, E, K, i32, i64, w, gather, W, rank);
}

}  // namespace
}  // namespace mok

using namespace mok;

extern "C" int mok_router_topk(const float* logits, int num_tokens, int num_experts, int topk, int32_t* top_experts_i32,
                               int64_t* top_experts_i64, float* router_weights, const uint64_t* all_gather_ptrs, int ep_size,
                               int ep_rank, void* stream) {
    if (!logits || !router_weights || (!top_experts_i32 && !top_experts_i64 && !all_gather_ptrs)) return MOK_ERR_INVALID;
    if (num_tokens <= 0 || num_experts <= 0 || topk <= 0 || topk > 32 || topk > num_experts) return MOK_ERR_INVALID;
    if (num_experts > 1024) return MOK_ERR_UNSUPPORTED;
    PeerPtrs gather{};
    int W = 0;
    if (all_gather_ptrs) {
        if (ep_size < 1 || ep_size > MOK_MAX_PEERS || ep_rank < 0 || ep_rank >= ep_size) return MOK_ERR_INVALID;
        for (int i = 0; i < ep_size; ++i) {
            if (!all_gather_ptrs[i]) return MOK_ERR_INVALID;
            gather.p[i] = reinterpret_cast<void*>(all_gather_ptrs[i]);
        }
        W = ep_size;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = std::min((num_tokens + kRouterWarps - 1) / kRouterWarps, device_sm_count() * 8);
    long long* i64 = reinterpret_cast<long long*>(top_experts_i64);
    ProfScope prof(kSlotOther, s);
    const int per_lane = (num_experts + 31) / 32;
    if (per_lane <= 1) launch_topk<1>(logits, num_tokens, num_experts, topk, top_experts_i32, i64, router_weights, gather, W, ep_rank, blocks, s);
    else if (per_lane <= 2) launch_topk<2>(logits, num_tokens, num_experts, topk, top_experts_i32, i64, router_weights, gather, W, ep_rank, blocks, s);
    else if (per_lane <= 4) launch_topk<4>(logits, num_tokens, num_experts, topk, top_experts_i32, i64, router_weights, gather, W, ep_rank, blocks, s);
    else if (per_lane <= 8) launch_topk<8>(logits, num_tokens, num_experts, topk, top_experts_i32, i64, router_weights, gather, W, ep_rank, blocks, s);
    else if (per_lane <= 16) launch_topk<16>(logits, num_tokens, num_experts, topk, top_experts_i32, i64, router_weights, gather, W, ep_rank, blocks, s);
    else launch_topk<32>(logits, num_tokens, num_experts, topk, top_experts_i32, i64, router_weights, gather, W, ep_rank, blocks, s);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

extern "C" int mok_router_topk_bwd(const int32_t* top_experts_i32, const float* router_weights, const float* d_router_weights,
                                   float* d_logits, int num_tokens, int num_experts, int topk, void* stream) {
    if (!top_experts_i32 || !router_weights || !d_router_weights || !d_logits) return MOK_ERR_INVALID;
    if (num_tokens <= 0 || num_experts <= 0 || topk <= 0 || topk > 32 || topk > num_experts) return MOK_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = std::min((num_tokens + kRouterWarps - 1) / kRouterWarps, device_sm_count() * 8);
    ProfScope prof(kSlotOther, s);
    router_topk_bwd_kernel<<<blocks, kRouterWarps * 32, 0, s>>>(top_experts_i32, router_weights, d_router_weights, d_logits, num_tokens,
                                                                num_experts, topk);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
