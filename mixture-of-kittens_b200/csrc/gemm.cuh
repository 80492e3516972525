// Persistent grouped GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   - operands are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no
//     cluster multicast), 4 stages of 128x64 (A) + 256x64 (B) bf16 = 48 KB each;
//   - one elected thread issues tcgen05.mma (M=128, N=256, K=16 per instruction), fp32
//     accumulators live in tensor memory, double-buffered (2 x 256 columns) so the epilogue of
//     tile i overlaps the main loop of tile i+1;
//   - eight epilogue warps (two per TMEM lane quarter, each taking half of the tile's columns) read
//     the accumulator with tcgen05.ld and apply the fused epilogue:
//     plain bf16 store (optionally accumulating), SwiGLU forward (gate|up halves of one tile),
//     or SwiGLU backward with the router-gradient partial sums.
//
// Warp roles in a 320-thread CTA: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..9 = epilogue (TMEM lane quarter = warp id % 4, column half = (warp id - 2) / 4).  One CTA per SM; tiles are assigned
// round-robin (tile = blockIdx.x + i * gridDim.x), so results do not depend on timing.
//
// Row counts come from device memory (num_tokens / tokens_per_expert): nothing here needs a
// host synchronisation.  Every wait is bounded; on expiry the CTA drains, frees its tensor
// memory and reports MOK_STATUS_PIPELINE_TIMEOUT.
#pragma once

#include "common.cuh"
#include "profile.cuh"

namespace mok {

enum : int { kMajorK = 0, kMajorMN = 1 };
enum : int { kEpiStore = 0, kEpiSwigluFwd = 1, kEpiSwigluBwd = 2 };

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kBlockK * 2;   // 16 KB
constexpr int kBBytes = kBlockN * kBlockK * 2;   // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiSplit = 2;                      // epilogue warps per TMEM lane quarter
constexpr int kGemmThreads = 64 + 128 * kEpiSplit;
constexpr int kTmemCols = 512;
constexpr int kMaxExperts = MOK_MAX_LOCAL_EXPERTS;
constexpr int kGemmSmemBytes = kStages * kStageBytes + 256 + kMaxExperts * 4 + 1024;   // also 6 x 32 KB stages of the two-CTA form

struct GemmParams {
    // row domain
    const int* num_tokens;         // device row count (schedule rows); nullptr -> rows_host
    int rows_host;
    int capacity;
    int row_offset;                // first schedule row of the window (macrobatch) this launch covers
    int row_limit;                 // window size in rows; buffers are indexed relative to the window
    const int* tokens_per_expert;  // nullptr -> one group covering every row
    int num_experts;
    ChunkSpec chunk;               // row sub-range of the window this launch covers (not used by weight gradients)
    // tiling
    int n_tiles;                   // output tiles along N
    int m_tiles_w;                 // weight-gradient mode: output tiles along M
    int k_blocks_per_seg;          // K / 64 per segment (ignored in weight-gradient mode)
    int num_segs;                  // 1, or 2 for the two-GEMM accumulation d_gate*Wg + d_up*Wu
    int b_rows_per_expert;         // rows between experts in B's tensor map
    // epilogue
    __nv_bfloat16* out0;           // store: C; swiglu fwd: gate; swiglu bwd: d_hidden
    __nv_bfloat16* out1;           // swiglu fwd: up;   swiglu bwd: d_gate
    __nv_bfloat16* out2;           // swiglu fwd: hidden; swiglu bwd: d_up
    const __nv_bfloat16* in0;      // swiglu bwd: saved gate
    const __nv_bfloat16* in1;      // swiglu bwd: saved up
    int ld_out;
    long long out_expert_stride;   // weight-gradient mode: elements between experts in out0
    int accumulate;                // weight-gradient mode: add to the bf16 value already stored
    const float* row_scale;        // swiglu bwd: router weight per routed row (nullptr for the shared expert)
    float* partials;               // swiglu bwd: [rows, n_tiles * kEpiSplit] router-gradient partial sums (one per 128 columns)
    float limit;
    int has_limit;
    int* status;
};

// sigmoid through one tanh.approx (a single special-function op instead of exp + reciprocal):
// sigmoid(x) = 0.5 * tanh(0.5 x) + 0.5, absolute error about 2^-12, far below the bf16 rounding that follows
__device__ __forceinline__ float sigmoid_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(t, 0.5f, 0.5f);
}
__device__ __forceinline__ float silu_mul(float g, float u) {
    return g * sigmoid_fast(g) * u;
}

template <int kAMajor, int kBMajor, int kEpi, bool kWgrad, bool k2>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                    const GemmParams p) {
    // k2: a pair of CTAs (cluster of 2) shares one 256 x 256 tile; each CTA stages its own 128 rows of A and
    // its own 128 rows/columns of B, so a stage is 32 KB and six stages fit
    constexpr int kS = k2 ? 6 : kStages;
    constexpr int kBTile = k2 ? kBBytes / 2 : kBBytes;
    constexpr int kStg = kABytes + kBTile;
    constexpr int kTileM = k2 ? 2 * kBlockM : kBlockM;
    const uint32_t cta_rank = k2 ? cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    const int tile_first = k2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = k2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kS * kStg);
    uint64_t* empty_bar = full_bar + kS;
    uint64_t* tfull_bar = empty_bar + kS;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_end = reinterpret_cast<int*>(smem + kS * kStg + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int E = p.tokens_per_expert ? p.num_experts : 1;

    // inclusive prefix of padded rows per expert
    if (p.tokens_per_expert) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) s_end[e] = p.tokens_per_expert[e];
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kS; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], (k2 ? 8 : 4) * kEpiSplit); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 0 && p.tokens_per_expert) {
        const int per = (E + 31) / 32;
        int sum = 0;
        for (int j = 0; j < per; ++j) { const int e = lane * per + j; if (e < E) sum += s_end[e]; }
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) { const int n = __shfl_up_sync(0xffffffffu, incl, off); if (lane >= off) incl += n; }
        int run = incl - sum;
        for (int j = 0; j < per; ++j) { const int e = lane * per + j; if (e < E) { run += s_end[e]; s_end[e] = run; } }
    }
    if (warp == 1) {
        if (k2) { tmem_alloc_pair(tmem_slot, kTmemCols); tmem_relinquish_pair(); }
        else { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if (k2) cluster_sync_all();        // the partner's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_total = p.num_tokens ? min(*p.num_tokens, p.capacity) : p.rows_host;
    const int win_rows = max(0, min(n_total - p.row_offset, p.row_limit));
    // a weight-gradient launch that only accumulates has nothing to do on an empty window
    int chunk_lo = 0, chunk_hi = win_rows;
    if (!kWgrad) chunk_range(win_rows, p.chunk, chunk_lo, chunk_hi);
    const int m_tile0 = chunk_lo / kTileM;
    const int m_tiles_w = k2 ? p.m_tiles_w >> 1 : p.m_tiles_w;
    const int num_tiles = kWgrad ? ((p.accumulate && win_rows == 0) ? 0 : E * m_tiles_w * p.n_tiles)
                                 : ((chunk_hi - chunk_lo) / kTileM) * p.n_tiles;

    // tile -> coordinates.  a_row: first A/C row (window-relative); k_row0/k_blocks: contraction range
    auto decode = [&](int tile, int& m_idx, int& n_idx, int& expert, int& k_row0, int& k_blocks) {
        if constexpr (kWgrad) {
            const int per_e = m_tiles_w * p.n_tiles;
            expert = tile / per_e;
            const int r = tile - expert * per_e;
            m_idx = r / p.n_tiles;
            n_idx = r - m_idx * p.n_tiles;
            int s = 0, e_end = n_total;
            if (p.tokens_per_expert) { s = expert ? s_end[expert - 1] : 0; e_end = min(s_end[expert], n_total); }
            const int lo = max(s, p.row_offset), hi = min(e_end, p.row_offset + win_rows);
            k_row0 = lo - p.row_offset;
            k_blocks = hi > lo ? (hi - lo) / kBlockK : 0;
        } else {
            const int m_rel = tile / p.n_tiles;
            n_idx = tile - m_rel * p.n_tiles;
            m_idx = m_tile0 + m_rel;
            expert = 0;
            if (p.tokens_per_expert) {
                const int g = p.row_offset + m_idx * kTileM;
                int lo = 0, hi = E - 1;
                while (lo < hi) { const int mid = (lo + hi) >> 1; if (s_end[mid] > g) hi = mid; else lo = mid + 1; }
                expert = lo;
            }
            k_row0 = 0;
            k_blocks = p.k_blocks_per_seg * p.num_segs;
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmA0); tma_prefetch_desc(&tmB0);
            if (p.num_segs > 1) { tma_prefetch_desc(&tmA1); }
            if (p.num_segs > 1 || kEpi == kEpiSwigluFwd) { tma_prefetch_desc(&tmB1); }
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step) {
                int m_idx, n_idx, expert, k_row0, k_blocks;
                decode(tile, m_idx, n_idx, expert, k_row0, k_blocks);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* sa = smem + stage * kStg;
                    uint8_t* sb = sa + kABytes;
                    if (leader) mbar_arrive_expect_tx(&full_bar[stage], k2 ? 2 * kStg : kStg);
                    const int row_a = m_idx * kTileM + static_cast<int>(cta_rank) * kBlockM;   // this CTA's 128 rows / columns of A
                    const int col_b = n_idx * kBlockN + static_cast<int>(cta_rank) * (kBlockN / 2);
                    auto load = [&](void* dst, const CUtensorMap* map, int x, int y) {
                        if (k2) tma_load_2d_pair(dst, map, &full_bar[stage], x, y);
                        else tma_load_2d(dst, map, &full_bar[stage], x, y);
                    };
                    const int seg = (!kWgrad && kb >= p.k_blocks_per_seg) ? 1 : 0;
                    const int kk = (kWgrad ? kb : kb - seg * p.k_blocks_per_seg) * kBlockK;
                    const CUtensorMap* ma = seg ? &tmA1 : &tmA0;
                    const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
                    // A
                    if constexpr (kAMajor == kMajorK) {
                        load(sa, ma, kk, row_a);
                    } else {
#pragma unroll
                        for (int j = 0; j < kBlockM / 64; ++j)
                            load(sa + j * (kBlockK * 128), ma, row_a + j * 64, k_row0 + kk);
                    }
                    // B
                    if constexpr (kBMajor == kMajorK) {
                        if constexpr (kEpi == kEpiSwigluFwd) {
                            const int y = expert * p.b_rows_per_expert + n_idx * (kBlockN / 2);
                            if (k2) {                       // the leader holds the gate rows, its partner the up rows
                                load(sb, leader ? &tmB0 : &tmB1, kk, y);
                            } else {
                                load(sb, &tmB0, kk, y);
                                load(sb + kBBytes / 2, &tmB1, kk, y);
                            }
                        } else {
                            load(sb, mb, kk, expert * p.b_rows_per_expert + (k2 ? col_b : n_idx * kBlockN));
                        }
                    } else {
                        const int y = kWgrad ? (k_row0 + kk) : (expert * p.b_rows_per_expert + kk);
#pragma unroll
                        for (int j = 0; j < (k2 ? kBlockN / 128 : kBlockN / 64); ++j)
                            load(sb + j * (kBlockK * 128), mb, (k2 ? col_b : n_idx * kBlockN) + j * 64, y);
                    }
                    if (++stage == kS) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc_bf16(kTileM, kBlockN, kAMajor, kBMajor);
            constexpr uint32_t a_lbo = kAMajor == kMajorK ? 16 : kBlockK * 128;
            constexpr uint32_t b_lbo = kBMajor == kMajorK ? 16 : kBlockK * 128;
            constexpr uint32_t a_kstep = kAMajor == kMajorK ? 32 : 2048;   // bytes per K=16 step
            constexpr uint32_t b_kstep = kBMajor == kMajorK ? 32 : 2048;
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++it) {
                int m_idx, n_idx, expert, k_row0, k_blocks;
                decode(tile, m_idx, n_idx, expert, k_row0, k_blocks);
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * kBlockN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * kStg);
                    const uint32_t sb = sa + kABytes;
                    const uint64_t adesc = make_smem_desc(sa, a_lbo, 1024);
                    const uint64_t bdesc = make_smem_desc(sb, b_lbo, 1024);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k) {
                        if (k2) umma_f16_pair(d_tmem, adesc + ((k * a_kstep) >> 4), bdesc + ((k * b_kstep) >> 4), idesc,
                                              (kb > 0 || k > 0) ? 1u : 0u);
                        else umma_f16(d_tmem, adesc + ((k * a_kstep) >> 4), bdesc + ((k * b_kstep) >> 4), idesc,
                                      (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    if (k2) umma_commit_pair(&empty_bar[stage]); else umma_commit(&empty_bar[stage]);
                    if (++stage == kS) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (k_blocks > 0) { if (k2) umma_commit_pair(&tfull_bar[buf]); else umma_commit(&tfull_bar[buf]); }
                else { mbar_arrive(&tfull_bar[buf]); if (k2) mbar_arrive_cta(&tfull_bar[buf], 1); }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;            // which share of the tile's columns this warp handles
        const int r_in_tile = quarter * 32 + lane;
        int it = 0;
        bool ok = true;
        for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++it) {
            int m_idx, n_idx, expert, k_row0, k_blocks;
            decode(tile, m_idx, n_idx, expert, k_row0, k_blocks);
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!mbar_wait(&tfull_bar[buf], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBlockN;
            const size_t row = static_cast<size_t>(m_idx) * kTileM + cta_rank * kBlockM + r_in_tile;

            if constexpr (kEpi == kEpiStore) {
                __nv_bfloat16* dst = p.out0 + (kWgrad ? static_cast<size_t>(expert) * p.out_expert_stride : 0) +
                                     row * p.ld_out + static_cast<size_t>(n_idx) * kBlockN;
                const bool skip_store = kWgrad && p.accumulate && k_blocks == 0;   // adding zero: leave as is
                constexpr int kPer = kBlockN / 32 / kEpiSplit;
#pragma unroll 1
                for (int c = half * kPer; c < (skip_store ? 0 : (half + 1) * kPer); ++c) {
                    uint32_t acc[32];
                    if (k_blocks > 0) { tmem_ld_32x32(t_addr + c * 32, acc); tmem_ld_wait(); }
                    else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[i] = 0u;
                    }
                    __nv_bfloat16* d16 = dst + c * 32;
#pragma unroll
                    for (int v = 0; v < 2; ++v) {            // 16 columns = 32 bytes per 256-bit store
                        float f[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(acc[v * 16 + i]);
                        if (kWgrad && p.accumulate) {
                            uint32_t o[8];
                            ld_global_256(d16 + v * 16, o);
#pragma unroll
                            for (int i = 0; i < 8; ++i) { const float2 q = unpack_bf16(o[i]); f[2 * i] += q.x; f[2 * i + 1] += q.y; }
                        }
                        st_global_256(d16 + v * 16, pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                                      pack_bf16(f[6], f[7]), pack_bf16(f[8], f[9]), pack_bf16(f[10], f[11]),
                                      pack_bf16(f[12], f[13]), pack_bf16(f[14], f[15]));
                    }
                }
            } else if constexpr (kEpi == kEpiSwigluFwd) {
                const size_t off = row * p.ld_out + static_cast<size_t>(n_idx) * (kBlockN / 2);
                constexpr int kPer = kBlockN / 64 / kEpiSplit;
#pragma unroll 1
                for (int c = half * kPer; c < (half + 1) * kPer; ++c) {
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(t_addr + c * 32, g);
                    tmem_ld_32x32(t_addr + kBlockN / 2 + c * 32, u);
                    tmem_ld_wait();
                    __nv_bfloat16* dg = p.out0 + off + c * 32;
                    __nv_bfloat16* du = p.out1 + off + c * 32;
                    __nv_bfloat16* dh = p.out2 + off + c * 32;
#pragma unroll
                    for (int v = 0; v < 2; ++v) {            // 16 columns = 32 bytes per 256-bit store
                        uint32_t gw[8], uw[8], hw[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            gw[i] = pack_bf16(__uint_as_float(g[v * 16 + 2 * i]), __uint_as_float(g[v * 16 + 2 * i + 1]));
                            uw[i] = pack_bf16(__uint_as_float(u[v * 16 + 2 * i]), __uint_as_float(u[v * 16 + 2 * i + 1]));
                            float2 gf = unpack_bf16(gw[i]), uf = unpack_bf16(uw[i]);
                            if (p.has_limit) {
                                gf.x = fminf(gf.x, p.limit); gf.y = fminf(gf.y, p.limit);
                                uf.x = fminf(fmaxf(uf.x, -p.limit), p.limit); uf.y = fminf(fmaxf(uf.y, -p.limit), p.limit);
                            }
                            hw[i] = pack_bf16(silu_mul(gf.x, uf.x), silu_mul(gf.y, uf.y));
                        }
                        st_global_256(dg + v * 16, gw[0], gw[1], gw[2], gw[3], gw[4], gw[5], gw[6], gw[7]);
                        st_global_256(du + v * 16, uw[0], uw[1], uw[2], uw[3], uw[4], uw[5], uw[6], uw[7]);
                        st_global_256(dh + v * 16, hw[0], hw[1], hw[2], hw[3], hw[4], hw[5], hw[6], hw[7]);
                    }
                }
            } else {
                // SwiGLU backward on the d_hidden tile just computed
                const size_t off = row * p.ld_out + static_cast<size_t>(n_idx) * kBlockN;
                float inv_w = 0.0f;
                if (p.row_scale) { const float w = p.row_scale[row]; inv_w = w > 0.0f ? 1.0f / w : 0.0f; }
                float partial = 0.0f;
                constexpr int kPer = kBlockN / 32 / kEpiSplit;
#pragma unroll 1
                for (int c = half * kPer; c < (half + 1) * kPer; ++c) {
                    uint32_t acc[32];
                    tmem_ld_32x32(t_addr + c * 32, acc);
                    uint32_t gv[2][8], uv[2][8];             // saved gate / up: two 256-bit loads each
#pragma unroll
                    for (int v = 0; v < 2; ++v) {
                        ld_global_256(p.in0 + off + c * 32 + v * 16, gv[v]);
                        ld_global_256(p.in1 + off + c * 32 + v * 16, uv[v]);
                    }
                    tmem_ld_wait();
                    __nv_bfloat16* dh = p.out0 + off + c * 32;
                    __nv_bfloat16* dg = p.out1 + off + c * 32;
                    __nv_bfloat16* du = p.out2 + off + c * 32;
#pragma unroll
                    for (int v = 0; v < 2; ++v) {            // 16 columns = 32 bytes per 256-bit access
                        uint32_t hw[8], gw[8], uw[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            hw[i] = pack_bf16(__uint_as_float(acc[v * 16 + 2 * i]), __uint_as_float(acc[v * 16 + 2 * i + 1]));
                            const float2 dhf = unpack_bf16(hw[i]);
                            float2 gf = unpack_bf16(gv[v][i]), uf = unpack_bf16(uv[v][i]);
                            bool gm0 = true, gm1 = true, um0 = true, um1 = true;
                            if (p.has_limit) {
                                gm0 = gf.x <= p.limit; gm1 = gf.y <= p.limit;
                                um0 = uf.x >= -p.limit && uf.x <= p.limit; um1 = uf.y >= -p.limit && uf.y <= p.limit;
                                gf.x = fminf(gf.x, p.limit); gf.y = fminf(gf.y, p.limit);
                                uf.x = fminf(fmaxf(uf.x, -p.limit), p.limit); uf.y = fminf(fmaxf(uf.y, -p.limit), p.limit);
                            }
                            const float s0 = sigmoid_fast(gf.x), s1 = sigmoid_fast(gf.y);
                            const float silu0 = gf.x * s0, silu1 = gf.y * s1;
                            const float ds0 = (1.0f - silu0) * s0 + silu0, ds1 = (1.0f - silu1) * s1 + silu1;
                            gw[i] = pack_bf16(gm0 ? ds0 * uf.x * dhf.x : 0.0f, gm1 ? ds1 * uf.y * dhf.y : 0.0f);
                            uw[i] = pack_bf16(um0 ? silu0 * dhf.x : 0.0f, um1 ? silu1 * dhf.y : 0.0f);
                            partial += dhf.x * inv_w * (silu0 * uf.x) + dhf.y * inv_w * (silu1 * uf.y);
                        }
                        st_global_256(dh + v * 16, hw[0], hw[1], hw[2], hw[3], hw[4], hw[5], hw[6], hw[7]);
                        st_global_256(dg + v * 16, gw[0], gw[1], gw[2], gw[3], gw[4], gw[5], gw[6], gw[7]);
                        st_global_256(du + v * 16, uw[0], uw[1], uw[2], uw[3], uw[4], uw[5], uw[6], uw[7]);
                    }
                }
                if (p.partials) p.partials[(row * p.n_tiles + n_idx) * kEpiSplit + half] = partial;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (k2) mbar_arrive_leader(&tempty_bar[buf]); else mbar_arrive(&tempty_bar[buf]); }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (k2) cluster_sync_all();        // neither CTA frees tensor memory or exits while its partner may still signal it
    if (warp == 1) { tc_fence_after(); if (k2) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols); }
    if (threadIdx.x == 0 && *abort_flag) report_status(p.status, MOK_STATUS_PIPELINE_TIMEOUT, warp);
}

// host side ---------------------------------------------------------------------------------
// elem_bytes 1 or 2: 128-byte-swizzled operand tiles; elem_bytes 4: unswizzled rows of 32-bit words (scale tiles)
int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                 uint32_t box_inner, uint32_t box_outer, int elem_bytes);
bool use_pairs();

struct GemmOperands {
    const void* a0; const void* b0; const void* a1; const void* b1;   // a1/b1: second segment or "up" weights
    uint64_t a_inner, a_outer;   // tensor-map extents of A (elements, rows)
    uint64_t b_inner, b_outer;
};
// a_major/b_major/epi/wgrad select the instantiation; `max_ctas` caps the grid (0 = all SMs)
int launch_grouped_gemm(int a_major, int b_major, int epi, bool wgrad, const GemmOperands& ops, const GemmParams& p,
                        int max_tiles, int max_ctas, int prof_slot, cudaStream_t stream);

}  // namespace mok
