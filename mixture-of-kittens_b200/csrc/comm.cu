// Memory-movement kernels of the MoE layer: top-k all-gather, device barrier, token dispatch
// (pull rows from peers' buffers over NVLink), combine (push rows into peers' buffers), and the
// two HBM-bound epilogues.  All peer traffic is plain unicast ld/st on peer-mapped addresses;
// there is no cluster multicast and no library collective on this path.
#include "comm.cuh"
#include "mxfp8.cuh"
#include "profile.cuh"

namespace mok {
namespace {

// ---------------------------------------------------------------------------------------
// all-gather of int32 top-k ids: every rank stores its block into slot `rank` of each peer
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) all_gather_kernel(const int4* __restrict__ src, int64_t n_vec, int64_t numel,
                                                         PeerPtrs peers, int W, int rank) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        const int4 v = src[i];
        for (int p = 0; p < W; ++p) {
            int4* dst = reinterpret_cast<int4*>(static_cast<int*>(peers.p[p]) + static_cast<int64_t>(rank) * numel);
            dst[i] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------
// device barrier: target += W; add 1 to every peer's counter; wait (bounded) on the own one
// ---------------------------------------------------------------------------------------
__global__ void barrier_kernel(uint32_t* local_counter, PeerPtrs peers, int W, uint32_t* target_ptr, int* status,
                               uint64_t timeout_ns) {
    __shared__ uint32_t s_target;
    if (threadIdx.x == 0) s_target = atomicAdd(target_ptr, static_cast<uint32_t>(W)) + static_cast<uint32_t>(W);
    __syncthreads();
    if (threadIdx.x < W) {
        // release at system scope: everything this stream wrote before the barrier is visible to a
        // peer that observes the increment
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peers.p[threadIdx.x]) : "memory");
    }
    if (threadIdx.x == 0) {
        const uint32_t target = s_target;
        const uint64_t t0 = global_timer_ns();
        uint32_t value;
        uint32_t spins = 0;
        while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(local_counter) : "memory");
            if (static_cast<int32_t>(value - target) >= 0) break;
            if ((++spins & 0x3F) == 0 && global_timer_ns() - t0 > timeout_ns) {
                report_status(status, MOK_STATUS_BARRIER_TIMEOUT, static_cast<int>(value));
                break;
            }
            __nanosleep(64);
        }
    }
}

// ---------------------------------------------------------------------------------------
// epilogues: 8 bf16 (16 B) per thread, fp32 accumulation in k order
// ---------------------------------------------------------------------------------------
template <bool kWeighted>
__global__ void __launch_bounds__(256) epilogue_kernel(const uint4* __restrict__ shared_rows, const uint4* __restrict__ routed_rows,
                                                       const float* __restrict__ weights, uint4* __restrict__ out,
                                                       int64_t T, int vec_per_row, int K) {
    const int64_t total = T * vec_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t t = i / vec_per_row;
        const int v = static_cast<int>(i - t * vec_per_row);
        const uint4 s = shared_rows[i];
        float acc[8];
        {
            const uint32_t w[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = unpack_bf16(w[j]);
                acc[2 * j] = f.x; acc[2 * j + 1] = f.y;
            }
        }
        const uint4* r = routed_rows + (t * K) * vec_per_row + v;
        for (int k = 0; k < K; ++k) {
            const uint4 q = r[static_cast<int64_t>(k) * vec_per_row];
            const float wk = kWeighted ? weights[t * K + k] : 1.0f;
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = unpack_bf16(w[j]);
                if (kWeighted) {
                    acc[2 * j] += __fmul_rn(f.x, wk);
                    acc[2 * j + 1] += __fmul_rn(f.y, wk);
                } else {
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        out[i] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                            pack_bf16(acc[6], acc[7]));
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------
// dispatch: local row i <- peer[peer_rank[i]] row (peer_token_idx[i] / row_divisor); padding rows
// (peer_rank < 0) become zeros.  Optionally scales the row by a per-row float and re-rounds to bf16
// (backward "reverse combine").  One warp per row, 16-byte vectors, several loads in flight.
// ---------------------------------------------------------------------------------------
template <bool kScale>
__global__ void __launch_bounds__(256) dispatch_rows_kernel(RowMoveParams p) {
    const int n_total = min(*p.num_tokens, p.capacity);
    const int win_rows = max(0, min(n_total - p.row_offset, p.row_limit));
    int row_lo, rows;
    chunk_range(win_rows, p.chunk, row_lo, rows);
    const int warps_per_block = blockDim.x >> 5;
    const int warp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int n_warps = gridDim.x * warps_per_block;
    const int vec_per_row = p.hidden >> 3;
    for (int row = row_lo + warp; row < rows; row += n_warps) {
        const int g = p.row_offset + row;
        const int pr = p.peer_rank[g];
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.local) + static_cast<size_t>(row) * p.hidden);
        if (pr < 0) {
            for (int v = lane; v < vec_per_row; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
            if (kScale && lane == 0) p.row_scale_out[row] = 0.0f;
            continue;
        }
        const int tok = p.peer_token_idx[g];
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.peers.p[pr]) +
                                                           static_cast<size_t>(tok / p.row_divisor) * p.hidden);
        float w = 1.0f;
        if (kScale) {
            w = static_cast<const float*>(p.scale_peers.p[pr])[tok];
            if (lane == 0) p.row_scale_out[row] = w;
        }
        for (int v0 = lane; v0 < vec_per_row; v0 += 128) {
            uint4 buf[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + j * 32 < vec_per_row) buf[j] = src[v0 + j * 32];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (v0 + j * 32 < vec_per_row) {
                    uint4 o = buf[j];
                    if (kScale) {
                        uint32_t* w32 = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 f = unpack_bf16(w32[q]);
                            w32[q] = pack_bf16(f.x * w, f.y * w);
                        }
                    }
                    dst[v0 + j * 32] = o;
                }
            }
        }
    }
}

// combine: peer[peer_rank[i]] row peer_token_idx[i] <- local row i (padding rows skipped).  With
// `partials` set it also sums the router-gradient partials of the row in column order and stores
// the float at peer[...]'s d_router_weight[peer_token_idx[i]].
__global__ void __launch_bounds__(256) combine_rows_kernel(RowMoveParams p) {
    const int n_total = min(*p.num_tokens, p.capacity);
    const int win_rows = max(0, min(n_total - p.row_offset, p.row_limit));
    int row_lo, rows;
    chunk_range(win_rows, p.chunk, row_lo, rows);
    const int warps_per_block = blockDim.x >> 5;
    const int warp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int n_warps = gridDim.x * warps_per_block;
    const int vec_per_row = p.hidden >> 3;
    for (int row = row_lo + warp; row < rows; row += n_warps) {
        const int g = p.row_offset + row;
        const int pr = p.peer_rank[g];
        if (pr < 0) continue;
        const int tok = p.peer_token_idx[g];
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.local) + static_cast<size_t>(row) * p.hidden);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.peers.p[pr]) + static_cast<size_t>(tok) * p.hidden);
        for (int v0 = lane; v0 < vec_per_row; v0 += 128) {
            uint4 buf[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + j * 32 < vec_per_row) buf[j] = src[v0 + j * 32];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (v0 + j * 32 < vec_per_row) dst[v0 + j * 32] = buf[j];
        }
        if (p.partials != nullptr && lane == 0) {
            float s = 0.0f;
            for (int c = 0; c < p.partial_cols; ++c) s += p.partials[static_cast<size_t>(row) * p.partial_cols + c];
            static_cast<float*>(p.scale_peers.p[pr])[tok] = s;
        }
    }
}

// dispatch + MXFP8 quantisation.  Work unit = 32 consecutive rows (one MX block along the token axis)
// x 256 columns, staged in shared memory: coalesced row gathers in, then one normal block and one
// transposed block per thread out.  Padding rows are zeros (scale byte 88, as the reference's
// device code produces for an all-zero block).
template <bool kScale>
__global__ void __launch_bounds__(256) dispatch_quant_kernel(RowMoveParams p, QuantOut o) {
    constexpr int kCols = 256, kStride = kCols + 8;
    __shared__ __align__(16) __nv_bfloat16 tile[32 * kStride];
    const int n_total = min(*p.num_tokens, p.capacity);
    const int win_rows = max(0, min(n_total - p.row_offset, p.row_limit));
    int row_lo, row_hi;
    chunk_range(win_rows, p.chunk, row_lo, row_hi);
    const int col_chunks = p.hidden / kCols;
    const int units = ((row_hi - row_lo) / 32) * col_chunks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const int rb = unit / col_chunks, cc = unit - rb * col_chunks;
        const int row0 = row_lo + rb * 32, col0 = cc * kCols;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = warp * 4 + i;
            const int g = p.row_offset + row0 + r;
            const int pr = p.peer_rank[g];
            uint4 v = make_uint4(0, 0, 0, 0);
            float w = 0.0f;
            if (pr >= 0) {
                const int tok = p.peer_token_idx[g];
                const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.peers.p[pr]) +
                                                                   static_cast<size_t>(tok / p.row_divisor) * p.hidden + col0);
                v = src[lane];
                if (kScale) {
                    w = static_cast<const float*>(p.scale_peers.p[pr])[tok];
                    uint32_t* w32 = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = unpack_bf16(w32[q]);
                        w32[q] = pack_bf16(f.x * w, f.y * w);
                    }
                }
            }
            if (kScale && cc == 0 && lane == 0) p.row_scale_out[row0 + r] = w;
            *reinterpret_cast<uint4*>(&tile[r * kStride + lane * 8]) = v;
        }
        __syncthreads();
        {   // normal: thread -> (row, 32-wide block)
            const int r = threadIdx.x >> 3, kb = threadIdx.x & 7;
            uint32_t in[16], out[8], sb;
            const uint4* src = reinterpret_cast<const uint4*>(&tile[r * kStride + kb * 32]);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const uint4 v = src[j]; in[4 * j] = v.x; in[4 * j + 1] = v.y; in[4 * j + 2] = v.z; in[4 * j + 3] = v.w; }
            mx_quantize_block(in, out, sb);
            uint4* dst = reinterpret_cast<uint4*>(o.q + static_cast<size_t>(row0 + r) * p.hidden + col0 + kb * 32);
            dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
            dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
            o.sc[mx_scale_offset(row0 + r, (col0 >> 5) + kb, p.hidden >> 7)] = static_cast<uint8_t>(sb);
        }
        {   // transposed: thread -> column, block = the 32 rows
            const int c = threadIdx.x;
            uint32_t in[16], out[8], sb;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint16_t lo = *reinterpret_cast<const uint16_t*>(&tile[(2 * j) * kStride + c]);
                const uint16_t hi = *reinterpret_cast<const uint16_t*>(&tile[(2 * j + 1) * kStride + c]);
                in[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
            }
            mx_quantize_block(in, out, sb);
            uint4* dst = reinterpret_cast<uint4*>(o.qt + static_cast<size_t>(col0 + c) * o.t_rows + row0);
            dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
            dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
            o.sct[mx_scale_offset(col0 + c, row0 >> 5, o.t_rows >> 7)] = static_cast<uint8_t>(sb);
        }
        __syncthreads();
    }
}

int launch_dispatch_quant(const RowMoveParams& p, const QuantOut& out, bool scale, int num_blocks, cudaStream_t stream) {
    ProfScope prof(kSlotDispatch, stream);
    if (scale) dispatch_quant_kernel<true><<<num_blocks, 256, 0, stream>>>(p, out);
    else dispatch_quant_kernel<false><<<num_blocks, 256, 0, stream>>>(p, out);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

int launch_dispatch_rows(const RowMoveParams& p, bool scale, int num_blocks, cudaStream_t stream) {
    ProfScope prof(kSlotDispatch, stream);
    if (scale) dispatch_rows_kernel<true><<<num_blocks, 256, 0, stream>>>(p);
    else dispatch_rows_kernel<false><<<num_blocks, 256, 0, stream>>>(p);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
int launch_combine_rows(const RowMoveParams& p, int num_blocks, cudaStream_t stream) {
    ProfScope prof(kSlotCombine, stream);
    combine_rows_kernel<<<num_blocks, 256, 0, stream>>>(p);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

}  // namespace mok

using namespace mok;

extern "C" int mok_all_gather_top_experts(const int32_t* top_experts, int64_t numel, const uint64_t* peer_buffer_ptrs,
                                          int ep_size, int rank, void* stream) {
    if (!top_experts || !peer_buffer_ptrs || numel <= 0 || numel % 4 != 0) return MOK_ERR_INVALID;
    if (ep_size < 1 || ep_size > MOK_MAX_PEERS || rank < 0 || rank >= ep_size) return MOK_ERR_INVALID;
    PeerPtrs peers{};
    for (int i = 0; i < ep_size; ++i) {
        if (!peer_buffer_ptrs[i]) return MOK_ERR_INVALID;
        peers.p[i] = reinterpret_cast<void*>(peer_buffer_ptrs[i]);
    }
    const int64_t n_vec = numel / 4;
    const int blocks = static_cast<int>(std::min<int64_t>((n_vec + 255) / 256, 296));
    ProfScope prof(kSlotAllGather, static_cast<cudaStream_t>(stream));
    all_gather_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const int4*>(top_experts), n_vec,
                                                                             numel, peers, ep_size, rank);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

extern "C" int mok_barrier_all(uint32_t* local_counter, const uint64_t* peer_counter_ptrs, int ep_size, uint32_t* target,
                               int32_t* status, uint64_t timeout_ns, void* stream) {
    if (!local_counter || !peer_counter_ptrs || !target) return MOK_ERR_INVALID;
    if (ep_size < 1 || ep_size > MOK_MAX_PEERS) return MOK_ERR_INVALID;
    PeerPtrs peers{};
    for (int i = 0; i < ep_size; ++i) {
        if (!peer_counter_ptrs[i]) return MOK_ERR_INVALID;
        peers.p[i] = reinterpret_cast<void*>(peer_counter_ptrs[i]);
    }
    ProfScope prof(kSlotBarrier, static_cast<cudaStream_t>(stream));
    barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(local_counter, peers, ep_size, target, status,
                                                                    timeout_ns ? timeout_ns : kWaitLimitNs);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

static int epilogue_grid(int64_t total_vec) {
    return static_cast<int>(std::min<int64_t>((total_vec + 255) / 256, 148 * 16));
}

extern "C" int mok_fwd_epilogue(const void* y_shared, const void* combine_buffer, const float* topk_weights, void* output,
                                int num_local_tokens, int hidden, int topk, void* stream) {
    if (!y_shared || !combine_buffer || !topk_weights || !output) return MOK_ERR_INVALID;
    if (num_local_tokens <= 0 || hidden <= 0 || hidden % 8 || topk <= 0) return MOK_ERR_INVALID;
    const int vpr = hidden / 8;
    ProfScope prof(kSlotEpilogue, static_cast<cudaStream_t>(stream));
    epilogue_kernel<true><<<epilogue_grid(static_cast<int64_t>(num_local_tokens) * vpr), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(y_shared), static_cast<const uint4*>(combine_buffer), topk_weights,
        static_cast<uint4*>(output), num_local_tokens, vpr, topk);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

extern "C" int mok_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* d_x, int num_local_tokens,
                                int hidden, int topk, void* stream) {
    if (!d_x_shared || !d_x_routed_buffer || !d_x) return MOK_ERR_INVALID;
    if (num_local_tokens <= 0 || hidden <= 0 || hidden % 8 || topk <= 0) return MOK_ERR_INVALID;
    const int vpr = hidden / 8;
    ProfScope prof(kSlotEpilogue, static_cast<cudaStream_t>(stream));
    epilogue_kernel<false><<<epilogue_grid(static_cast<int64_t>(num_local_tokens) * vpr), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(d_x_shared), static_cast<const uint4*>(d_x_routed_buffer), nullptr,
        static_cast<uint4*>(d_x), num_local_tokens, vpr, topk);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
