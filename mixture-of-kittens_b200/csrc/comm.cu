// Memory-movement kernels of the MoE layer: top-k all-gather, device barrier, token dispatch
// (pull rows from peers' buffers over NVLink), combine (push rows into peers' buffers), and the
// two HBM-bound epilogues.  All peer traffic is plain unicast ld/st on peer-mapped addresses;
// there is no cluster multicast and no library collective on this path.
#include "comm.cuh"

#include <cstdlib>
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

// route -> schedule row, for the epilogues that gather routed rows straight from the GEMM output
__global__ void __launch_bounds__(256) invert_rows_kernel(const int* __restrict__ peer_rank, const int* __restrict__ peer_token_idx,
                                                          const int* __restrict__ num_tokens, int row_limit, int routes,
                                                          int* __restrict__ route_row) {
    const int n = min(*num_tokens, row_limit);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        if (peer_rank[i] < 0) continue;
        const int r = peer_token_idx[i];
        if (r >= 0 && r < routes) route_row[r] = i;
    }
}

// same arithmetic as epilogue_kernel, but the k-th routed row of token t is rows[route_row[t*K+k]]
// (a route without a row adds nothing); kWeighted = forward, else backward, which also sums each
// route's router-gradient partials in column order.  `out` may be `shared_rows` itself (the backward pass
// sums in place: every element is read by the thread that writes it, before it writes), so neither is restrict.
template <bool kWeighted>
__global__ void __launch_bounds__(256) epilogue_rows_kernel(const uint4* shared_rows, const uint4* __restrict__ rows,
                                                            const int* __restrict__ route_row, const float* __restrict__ weights,
                                                            const float* __restrict__ partials, int partial_cols,
                                                            float* __restrict__ d_router_weights, uint4* out,
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
        for (int k = 0; k < K; ++k) {
            const int row = route_row[t * K + k];
            if (!kWeighted && v == 0) {
                float sum = 0.0f;
                if (row >= 0)
                    for (int c = 0; c < partial_cols; ++c) sum += partials[static_cast<size_t>(row) * partial_cols + c];
                d_router_weights[t * K + k] = sum;
            }
            if (row < 0) continue;
            const uint4 q = rows[static_cast<int64_t>(row) * vec_per_row + v];
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
// Row movement with the bulk-copy engine.  dispatch: local row i <- peer[peer_rank[i]] row
// (peer_token_idx[i] / row_divisor), padding rows (peer_rank < 0) become zeros, optionally scaled by
// the route's router weight and re-rounded to bf16 (backward "reverse combine").  combine:
// peer[peer_rank[i]] row peer_token_idx[i] <- local row i (padding rows skipped); with `partials` set it
// also sums the row's router-gradient partials in column order and stores the float at the peer.
//
// A row is cut into pieces of at most 4 KB.  Each warp owns two 4 KB shared-memory slots and runs a
// two-deep pipeline: cp.async.bulk global(peer) -> shared, completion on an mbarrier, then
// cp.async.bulk shared -> global(peer).  Only one lane issues the copies, so the kernel puts almost no
// load on the SM's load/store path and can share SMs with the GEMM CTAs; bytes in flight per SM are
// set by the slots (24 KB per CTA), not by registers.  Remote addresses are plain unicast peer
// mappings; no multicast.
enum : int { kMoveDispatch = 0, kMoveDispatchScale = 1, kMoveCombine = 2 };
constexpr int kMoveMaxWarps = 8;

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// (compiled for at most 32 registers per thread: beside a 640-thread MXFP8 GEMM CTA each of the SM's four register
// files has room for exactly one such warp)
template <int kMode>
__global__ void __launch_bounds__(kMoveMaxWarps * 32, 8) move_rows_kernel(RowMoveParams p) {
    extern __shared__ __align__(128) uint8_t slot_mem[];      // [warps][2][piece]
    __shared__ __align__(8) uint64_t bars[kMoveMaxWarps][2];
    const int kMoveWarps = static_cast<int>(blockDim.x >> 5);
    const int kMovePiece = p.piece_bytes;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_word = 0;
        for (int w = 0; w < kMoveWarps; ++w) { mbar_init(&bars[w][0], 1); mbar_init(&bars[w][1], 1); }
        mbar_fence_init();
    }
    __syncthreads();

    const int n_total = min(*p.num_tokens, p.capacity);
    const int win_rows = max(0, min(n_total - p.row_offset, p.row_limit));
    int row_lo, row_hi;
    chunk_range(win_rows, p.chunk, row_lo, row_hi);
    const int row_bytes = p.hidden * 2;
    const int pieces = (row_bytes + kMovePiece - 1) / kMovePiece;
    const long long units = static_cast<long long>(row_hi - row_lo) * pieces;
    const long long gwarp = static_cast<long long>(blockIdx.x) * kMoveWarps + warp;
    const long long nwarps = static_cast<long long>(gridDim.x) * kMoveWarps;

    // resolve unit -> (source, destination, bytes); returns false for rows that move nothing
    auto resolve = [&](long long unit, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes, float& w, int& row, int& piece) {
        row = row_lo + static_cast<int>(unit / pieces);
        piece = static_cast<int>(unit % pieces);
        const int g = p.row_offset + row;
        const int pr = p.peer_rank[g];
        const int off = piece * kMovePiece;
        bytes = static_cast<uint32_t>(min(kMovePiece, row_bytes - off));
        w = 0.0f;
        uint8_t* local = static_cast<uint8_t*>(p.local) + static_cast<size_t>(row) * row_bytes + off;
        if (pr < 0) { src = nullptr; dst = local; return false; }
        const int tok = p.peer_token_idx[g];
        if (kMode == kMoveCombine) {
            src = local;
            dst = static_cast<uint8_t*>(p.peers.p[pr]) + static_cast<size_t>(tok) * row_bytes + off;
        } else {
            src = static_cast<const uint8_t*>(p.peers.p[pr]) + static_cast<size_t>(tok / p.row_divisor) * row_bytes + off;
            dst = local;
            if (kMode == kMoveDispatchScale) w = static_cast<const float*>(p.scale_peers.p[pr])[tok];
        }
        return true;
    };

    uint32_t phase[2] = {0, 0};
    long long issued = 0;        // copies this warp has put in flight (slot = issued & 1)
    bool ok = true;
    // software pipeline: the load of unit u+1 is in flight while unit u is stored
    const uint8_t* src_n = nullptr; uint8_t* dst_n = nullptr; uint32_t bytes_n = 0; float w_n = 0.f; int row_n = 0, piece_n = 0;
    bool live_n = false, have_n = false;
    long long u = gwarp;
    auto start_load = [&](long long unit) {
        have_n = unit < units;
        if (!have_n) return;
        live_n = resolve(unit, src_n, dst_n, bytes_n, w_n, row_n, piece_n);
        if (live_n && lane == 0) {
            const int slot = static_cast<int>(issued & 1);
            // the slot was last read by the store committed in the previous iteration
            if (issued >= 2) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            mbar_arrive_expect_tx(&bars[warp][slot], bytes_n);
            bulk_g2s((slot_mem + (static_cast<size_t>(warp) * 2 + slot) * kMovePiece), src_n, bytes_n, &bars[warp][slot]);
        }
        if (live_n) ++issued;
    };
    start_load(u);
    while (have_n && ok) {
        const uint8_t* src = src_n; uint8_t* dst = dst_n; const uint32_t bytes = bytes_n; const float w = w_n;
        const int row = row_n, piece = piece_n; const bool live = live_n;
        const int slot = static_cast<int>((issued - 1) & 1);
        (void)src;
        u += nwarps;
        start_load(u);                                  // may bump `issued`; `slot` above was taken before
        if (!live) {
            if (kMode != kMoveCombine) {                // padding row of a dispatch: zeros
                uint4* d4 = reinterpret_cast<uint4*>(dst);
                for (uint32_t v = lane; v < bytes / 16; v += 32) d4[v] = make_uint4(0, 0, 0, 0);
                if (kMode == kMoveDispatchScale && piece == 0 && lane == 0) p.row_scale_out[row] = 0.0f;
            }
            continue;
        }
        if (!mbar_wait(&bars[warp][slot], phase[slot], abort_flag)) { ok = false; break; }
        phase[slot] ^= 1;
        if (kMode == kMoveDispatchScale) {
            uint4* s4 = reinterpret_cast<uint4*>((slot_mem + (static_cast<size_t>(warp) * 2 + slot) * kMovePiece));
            for (uint32_t v = lane; v < bytes / 16; v += 32) {
                uint4 q = s4[v];
                uint32_t* w32 = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
                for (int k = 0; k < 4; ++k) { const float2 f = unpack_bf16(w32[k]); w32[k] = pack_bf16(f.x * w, f.y * w); }
                s4[v] = q;
            }
            if (piece == 0 && lane == 0) p.row_scale_out[row] = w;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
        }
        if (lane == 0) bulk_s2g(dst, (slot_mem + (static_cast<size_t>(warp) * 2 + slot) * kMovePiece), bytes);
        if (kMode == kMoveCombine && p.partials != nullptr && piece == 0 && lane == 0) {
            float s = 0.0f;
            for (int c = 0; c < p.partial_cols; ++c) s += p.partials[static_cast<size_t>(row) * p.partial_cols + c];
            const int g = p.row_offset + row;
            static_cast<float*>(p.scale_peers.p[p.peer_rank[g]])[p.peer_token_idx[g]] = s;
        }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
    if (!ok && lane == 0) report_status(p.status, MOK_STATUS_PIPELINE_TIMEOUT, 200 + kMode);
}

// dispatch + MXFP8 quantisation.  Work unit = 32 consecutive rows (one MX block along the token axis)
// x kCols columns.  Warp 0 fetches the 32 row pieces (from whichever peer owns the row) with
// cp.async.bulk into one of two shared-memory tiles while all warps quantise the other tile: 1x32
// blocks along the rows and 32x1 blocks along the tokens.  Padding rows are zeros
// (scale byte 88, as the reference's device code produces for an all-zero block).  kScale multiplies
// every row by its route's router weight and re-rounds to bf16 first (backward "reverse combine").
// Two shapes: 256 threads on 32 x 256 tiles (33 KB; one block of each kind per thread), and a lean one of 64 threads
// on 32 x 128 tiles (17 KB, at most 64 registers per thread) that fits in what an MXFP8 GEMM CTA leaves of an SM.
template <bool kScale, int kThreads, int kCols>
__global__ void __launch_bounds__(kThreads, 1024 / kThreads) dispatch_quant_kernel(RowMoveParams p, QuantOut o) {
    constexpr int kRowBytes = kCols * 2, kRowBlocks = kCols / 32;
    __shared__ __align__(128) uint8_t tiles[2][32 * kRowBytes];
    __shared__ float s_w[2][32];
    __shared__ __align__(8) uint64_t bars[2];
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { abort_word = 0; mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_fence_init(); }
    __syncthreads();

    const int n_total = min(*p.num_tokens, p.capacity);
    const int win_rows = max(0, min(n_total - p.row_offset, p.row_limit));
    int row_lo, row_hi;
    chunk_range(win_rows, p.chunk, row_lo, row_hi);
    const int col_chunks = p.hidden / kCols;
    const int units = ((row_hi - row_lo) / 32) * col_chunks;

    auto fetch = [&](int unit, int buf) {           // warp 0 only
        const int rb = unit / col_chunks, cc = unit - rb * col_chunks;
        const int row = row_lo + rb * 32 + lane, col0 = cc * kCols;
        const int g = p.row_offset + row;
        const int pr = p.peer_rank[g];
        const uint8_t* src = nullptr;
        float w = 0.0f;
        if (pr >= 0) {
            const int tok = p.peer_token_idx[g];
            src = static_cast<const uint8_t*>(p.peers.p[pr]) + (static_cast<size_t>(tok / p.row_divisor) * p.hidden + col0) * 2;
            w = kScale ? static_cast<const float*>(p.scale_peers.p[pr])[tok] : 1.0f;
        } else {
            uint4* z = reinterpret_cast<uint4*>(&tiles[buf][lane * kRowBytes]);
#pragma unroll
            for (int v = 0; v < kRowBytes / 16; ++v) z[v] = make_uint4(0, 0, 0, 0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // later bulk copies reuse this row
        }
        s_w[buf][lane] = w;
        if (kScale && cc == 0) p.row_scale_out[row] = w;
        const unsigned live = __ballot_sync(0xffffffffu, pr >= 0);
        __syncwarp();
        if (lane == 0) mbar_arrive_expect_tx(&bars[buf], __popc(live) * kRowBytes);
        __syncwarp();
        if (pr >= 0) bulk_g2s(&tiles[buf][lane * kRowBytes], src, kRowBytes, &bars[buf]);
    };

    uint32_t phase[2] = {0, 0};
    int buf = 0;
    if (warp == 0 && blockIdx.x < units) fetch(blockIdx.x, 0);
    for (int unit = blockIdx.x; unit < units; unit += gridDim.x, buf ^= 1) {
        const int next = unit + gridDim.x;
        if (warp == 0 && next < units) fetch(next, buf ^ 1);      // the other tile was released by the barrier below
        if (!mbar_wait(&bars[buf], phase[buf], abort_flag)) break;
        phase[buf] ^= 1;
        const int rb = unit / col_chunks, cc = unit - rb * col_chunks;
        const int row0 = row_lo + rb * 32, col0 = cc * kCols;
        const __nv_bfloat16* tile = reinterpret_cast<const __nv_bfloat16*>(tiles[buf]);
#pragma unroll 1
        for (int b = threadIdx.x; b < 32 * kRowBlocks; b += kThreads) {   // normal: (row, 32-wide block)
            const int r = b / kRowBlocks, kb = b - r * kRowBlocks;
            uint32_t in[16], out[8], sb;
            const uint4* src = reinterpret_cast<const uint4*>(&tile[r * kCols + kb * 32]);
            const float w = s_w[buf][r];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const uint4 v = src[j]; in[4 * j] = v.x; in[4 * j + 1] = v.y; in[4 * j + 2] = v.z; in[4 * j + 3] = v.w; }
            if (kScale) {
#pragma unroll
                for (int j = 0; j < 16; ++j) { const float2 f = unpack_bf16(in[j]); in[j] = pack_bf16(f.x * w, f.y * w); }
            }
            mx_quantize_block(in, out, sb);
            st_global_256(o.q + static_cast<size_t>(row0 + r) * p.hidden + col0 + kb * 32, out[0], out[1], out[2], out[3], out[4],
                          out[5], out[6], out[7]);
            o.sc[mx_scale_offset(row0 + r, (col0 >> 5) + kb, p.hidden >> 7)] = static_cast<uint8_t>(sb);
        }
#pragma unroll 1
        for (int c = threadIdx.x; c < kCols; c += kThreads) {   // transposed: a column, block = the 32 rows
            uint32_t in[16], out[8], sb;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float lo = __bfloat162float(tile[(2 * j) * kCols + c]), hi = __bfloat162float(tile[(2 * j + 1) * kCols + c]);
                if (kScale) { lo *= s_w[buf][2 * j]; hi *= s_w[buf][2 * j + 1]; }
                in[j] = pack_bf16(lo, hi);
            }
            mx_quantize_block(in, out, sb);
            st_global_256(o.qt + static_cast<size_t>(col0 + c) * o.t_rows + row0, out[0], out[1], out[2], out[3], out[4], out[5],
                          out[6], out[7]);
            o.sct[mx_scale_offset(col0 + c, row0 >> 5, o.t_rows >> 7)] = static_cast<uint8_t>(sb);
        }
        __syncthreads();                              // tile `buf` may be refilled
    }
    if (threadIdx.x == 0 && *abort_flag) report_status(p.status, MOK_STATUS_PIPELINE_TIMEOUT, 210);
}

int launch_dispatch_quant(const RowMoveParams& p, const QuantOut& out, bool scale, int num_blocks, cudaStream_t stream) {
    ProfScope prof(kSlotDispatch, stream);
    if (p.lean) {
        if (scale) dispatch_quant_kernel<true, 64, 128><<<num_blocks, 64, 0, stream>>>(p, out);
        else dispatch_quant_kernel<false, 64, 128><<<num_blocks, 64, 0, stream>>>(p, out);
    } else {
        if (scale) dispatch_quant_kernel<true, 256, 256><<<num_blocks, 256, 0, stream>>>(p, out);
        else dispatch_quant_kernel<false, 256, 256><<<num_blocks, 256, 0, stream>>>(p, out);
    }
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

// Three shapes of mover CTA: "thin" (3 warps x 2 x 4 KB = 24 KB, many CTAs, fits beside a BF16 GEMM CTA), "lean"
// (2 warps, 16 KB: what the MXFP8 GEMM CTAs leave free) and "fat" (8 warps x 2 x 8 KB = 128 KB, a few CTAs that
// each take an SM of their own).
template <int kMode>
int launch_move(RowMoveParams p, int num_blocks, cudaStream_t stream) {
    const bool fat = p.fat_ctas != 0;
    const int warps = fat ? 8 : (p.lean ? 2 : 3);
    p.piece_bytes = fat ? 8192 : 4096;
    const int smem = warps * 2 * p.piece_bytes;
    static bool configured[64] = {false};
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(move_rows_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 2 * 8192));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    move_rows_kernel<kMode><<<num_blocks, warps * 32, smem, stream>>>(p);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

int launch_dispatch_rows(const RowMoveParams& p, bool scale, int num_blocks, cudaStream_t stream) {
    ProfScope prof(kSlotDispatch, stream);
    if (scale) return launch_move<kMoveDispatchScale>(p, num_blocks, stream);
    return launch_move<kMoveDispatch>(p, num_blocks, stream);
}
int launch_combine_rows(const RowMoveParams& p, int num_blocks, cudaStream_t stream) {
    ProfScope prof(kSlotCombine, stream);
    return launch_move<kMoveCombine>(p, num_blocks, stream);
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
    const int blocks = static_cast<int>(std::min<int64_t>((n_vec + 255) / 256, 2 * device_sm_count()));
    ProfScope prof(kSlotAllGather, static_cast<cudaStream_t>(stream));
    all_gather_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const int4*>(top_experts), n_vec,
                                                                             numel, peers, ep_size, rank);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

// Ranks reach a barrier with whatever skew their hosts have (a checkpoint being written, a data loader that
// stalls), so the default limit is minutes, not the seconds of the in-kernel pipeline waits.
// MOK_B200_BARRIER_TIMEOUT_MS overrides it.
static uint64_t default_barrier_timeout_ns() {
    static const uint64_t configured = [] {
        const char* e = std::getenv("MOK_B200_BARRIER_TIMEOUT_MS");
        const long long ms = e ? std::atoll(e) : 0;
        return static_cast<uint64_t>(ms > 0 ? ms : 120000) * 1000000ull;
    }();
    return configured;
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
                                                                    timeout_ns ? timeout_ns : default_barrier_timeout_ns());
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

static int epilogue_grid(int64_t total_vec) {
    return static_cast<int>(std::min<int64_t>((total_vec + 255) / 256, 16 * device_sm_count()));
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

namespace {
int invert_rows(const int32_t* peer_rank, const int32_t* peer_token_idx, const int32_t* num_tokens, int32_t* route_row,
                int routes, int row_limit, cudaStream_t s) {
    MOK_CUDA_CHECK(cudaMemsetAsync(route_row, 0xFF, static_cast<size_t>(routes) * sizeof(int32_t), s));
    mok::invert_rows_kernel<<<std::min(1024, (row_limit + 255) / 256), 256, 0, s>>>(peer_rank, peer_token_idx, num_tokens, row_limit,
                                                                                    routes, route_row);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
}  // namespace

extern "C" int mok_fwd_epilogue_rows(const void* y_shared, const void* y_routed, const int32_t* schedule_peer_rank,
                                     const int32_t* schedule_peer_token_idx, const int32_t* num_tokens,
                                     const float* topk_weights, int32_t* route_row, void* output, int num_local_tokens,
                                     int hidden, int topk, int row_limit, void* stream) {
    if (!y_shared || !y_routed || !schedule_peer_rank || !schedule_peer_token_idx || !num_tokens || !topk_weights ||
        !route_row || !output)
        return MOK_ERR_INVALID;
    if (num_local_tokens <= 0 || hidden <= 0 || hidden % 8 || topk <= 0 || row_limit <= 0) return MOK_ERR_INVALID;
    if (static_cast<int64_t>(num_local_tokens) * topk > INT32_MAX) return MOK_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vpr = hidden / 8;
    ProfScope prof(kSlotEpilogue, s, 2);
    MOK_TRY(invert_rows(schedule_peer_rank, schedule_peer_token_idx, num_tokens, route_row, num_local_tokens * topk, row_limit, s));
    mok::epilogue_rows_kernel<true><<<epilogue_grid(static_cast<int64_t>(num_local_tokens) * vpr), 256, 0, s>>>(
        static_cast<const uint4*>(y_shared), static_cast<const uint4*>(y_routed), route_row, topk_weights, nullptr, 0, nullptr,
        static_cast<uint4*>(output), num_local_tokens, vpr, topk);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

extern "C" int mok_bwd_epilogue_rows(const void* d_x_shared, const void* d_x_routed, const float* partials, int partial_cols,
                                     const int32_t* schedule_peer_rank, const int32_t* schedule_peer_token_idx,
                                     const int32_t* num_tokens, int32_t* route_row, void* d_x, float* d_router_weights,
                                     int num_local_tokens, int hidden, int topk, int row_limit, void* stream) {
    if (!d_x_shared || !d_x_routed || !partials || !schedule_peer_rank || !schedule_peer_token_idx || !num_tokens ||
        !route_row || !d_x || !d_router_weights)
        return MOK_ERR_INVALID;
    if (num_local_tokens <= 0 || hidden <= 0 || hidden % 8 || topk <= 0 || row_limit <= 0 || partial_cols <= 0)
        return MOK_ERR_INVALID;
    if (static_cast<int64_t>(num_local_tokens) * topk > INT32_MAX) return MOK_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vpr = hidden / 8;
    ProfScope prof(kSlotEpilogue, s, 2);
    MOK_TRY(invert_rows(schedule_peer_rank, schedule_peer_token_idx, num_tokens, route_row, num_local_tokens * topk, row_limit, s));
    mok::epilogue_rows_kernel<false><<<epilogue_grid(static_cast<int64_t>(num_local_tokens) * vpr), 256, 0, s>>>(
        static_cast<const uint4*>(d_x_shared), static_cast<const uint4*>(d_x_routed), route_row, nullptr, partials, partial_cols,
        d_router_weights, static_cast<uint4*>(d_x), num_local_tokens, vpr, topk);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
