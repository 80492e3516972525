// Persistent grouped GEMM for MXFP8 operands on tcgen05: E4M3 data, one E8M0 scale per 32
// elements along K (tcgen05.mma kind::mxf8f6f4.block_scale), fp32 accumulation in tensor memory.
//
// Both operands are always K-major (the layer keeps transposed-quantised copies where the
// contraction runs over tokens), so one shared-memory layout serves every GEMM of the layer:
//   A tile 128 rows x 128 B, B tile 256 rows x 128 B, 128-byte swizzle, loaded by TMA;
//   scale tiles (512 B per 128 rows x 128 K, already in the tcgen05 [32][16] layout in global
//   memory) are fetched by TMA through an unswizzled [tiles, 512 B] tensor map and copied shared ->
//   tensor memory by tcgen05.cp (32x128b, replicated over the four lane quarters) right before the
//   four K=32 MMAs of a stage.
// Two-CTA form (k2, the default): a pair of CTAs on neighbouring SMs shares one 256 x 256 tile
// (tcgen05.mma.cta_group::2).  Each CTA stages its own 128 rows of A with their scales, 128 of the
// tile's 256 B rows, and the scales of all 256 B rows (every CTA's tensor memory needs them), so a
// stage is 33.5 KB instead of 49.5 KB and the shared-memory fill per flop drops by a third.  The
// leader CTA issues tcgen05.cp and tcgen05.mma for both; loads are plain (no cluster multicast).
// Tensor memory: accumulator columns [0,256), then a ring of four 16-column scale slots (A scales 4
// columns, B scales 8) used by consecutive k-tiles.  There is no room for a second 256-column
// accumulator beside the scales, so the epilogue warps first pull
// the whole accumulator into registers as packed bf16 (the layer rounds GEMM outputs to bf16
// before any further use anyway), release it, and only then run the fused epilogue — the next
// tile's main loop overlaps everything but that read-out.
//
// Fused epilogues:
//   Store      bf16 C (optionally accumulating onto the stored bf16 value: weight gradients)
//   GateUp     tile = (gate | up) halves -> saved gate/up as MXFP8, hidden = SwiGLU as MXFP8 in
//              both layouts (normal for the down GEMM, transposed for the down weight gradient)
//   DgradDown  d_hidden bf16 + SwiGLU backward from the saved MXFP8 gate/up -> d_gate, d_up as
//              MXFP8 in both layouts + router-gradient partial sums
// A warp's 32 lanes own 32 consecutive rows, i.e. exactly one MX block along the token axis, so
// the transposed quantisation needs only a warp-wide max (redux.sync) per column.
#pragma once

#include "gemm.cuh"
#include "mxfp8.cuh"

namespace mok {

enum : int { kMxEpiStore = 0, kMxEpiGateUp = 1, kMxEpiDgradDown = 2 };

constexpr int kMxBlockK = 128;                        // bytes (= elements) of K per stage
constexpr int kMxABytes = kBlockM * kMxBlockK;        // 16 KB
constexpr int kMxBBytes = kBlockN * kMxBlockK;        // 32 KB
constexpr int kMxTileBytes = kMxABytes + kMxBBytes;
constexpr int kMxSfBytes = 512 + 1024;                // A scales + B scales per stage
// pipeline depth: one-CTA 4 stages of 49.5 KB for the plain-store epilogue, 3 where the epilogue needs transpose
// tiles in shared memory; two-CTA 6 and 5 stages of 33.5 KB
__host__ __device__ constexpr int mx_stages(int epi, bool k2) { return k2 ? (epi == 0 ? 6 : 5) : (epi == 0 ? 4 : 3); }
__host__ __device__ constexpr int mx_tile_bytes(bool k2) { return kMxABytes + (k2 ? kMxBBytes / 2 : kMxBBytes); }
constexpr int kMxEpiGroups = 4;                       // epilogue warps per TMEM lane quarter (each takes 64 of the 256 columns)
constexpr int kMxEpiWarps = 4 * kMxEpiGroups;
constexpr int kMxThreads = 128 + 32 * kMxEpiWarps;    // warps 0-3: producer, MMA issuer, two spare; warps 4-19: epilogue
// Registers are re-balanced between the roles with setmaxnreg (it works on groups of four warps, hence the two spare
// warps).  A CTA can only redistribute what it was given: 640 threads x 96 registers (five warps share each of the SM's
// four register files, which caps a thread at 96 at launch).  The first group gives up a third of its share and the
// sixteen epilogue warps grow to 104; the fused epilogues of the one-CTA form (leaner producer and issuer loops) run with
// 32 and 112 instead.  The launcher checks the sum against the kernel's actual allocation.
constexpr int kMxLaunchRegs = 96;
__host__ __device__ constexpr int mx_light_regs(int epi, bool k2) { return (k2 || epi == 0) ? 64 : 32; }
__host__ __device__ constexpr int mx_epi_regs(int epi, bool k2) { return (k2 || epi == 0) ? 104 : 112; }
static_assert(128 * mx_light_regs(0, true) + 512 * mx_epi_regs(0, true) <= 640 * kMxLaunchRegs, "register budget");
static_assert(128 * mx_light_regs(1, false) + 512 * mx_epi_regs(1, false) <= 640 * kMxLaunchRegs, "register budget");
constexpr int kMxTrBytes = kMxEpiWarps * 32 * 17 * 4; // per-epilogue-warp transpose tiles
__host__ __device__ constexpr int mx_smem_bytes(int epi, bool k2) {
    return mx_stages(epi, k2) * (mx_tile_bytes(k2) + kMxSfBytes) + 256 + kMaxExperts * 4 + (epi == 0 ? 0 : kMxTrBytes) + 1024;
}
// tensor-memory columns: accumulator [0,256); then four scale slots of 16 columns (A scales 4, B scales 8, 4 spare)
constexpr int kMxAccCols = 256, kMxSfaCol = 256, kMxSfSlots = 4, kMxSfSlotCols = 16;

struct MxGemmParams {
    // row domain (same meaning as GemmParams)
    const int* num_tokens;
    int rows_host, capacity, row_offset, row_limit;
    const int* tokens_per_expert;
    int num_experts;
    ChunkSpec chunk;               // row sub-range of the window this launch covers (not used by weight gradients)
    // tiling
    int n_tiles, m_tiles_w, k_tiles_per_seg, num_segs, b_rows_per_expert;
    // scales: [row_tiles, k_tiles, 512 B]; the kernel reads them through the four scale tensor maps the launcher
    // builds from these pointers
    const uint8_t* sfa0; const uint8_t* sfa1; int sfa_k_tiles;
    const uint8_t* sfb0; const uint8_t* sfb1; int sfb_k_tiles;
    // Store / DgradDown: bf16 output
    __nv_bfloat16* out_bf16;
    int ld_out;
    long long out_expert_stride;
    int accumulate;
    // quantised outputs: index 0 = gate or d_gate, 1 = up or d_up, 2 = hidden
    uint8_t* q[3]; uint8_t* sc[3];          // normal layout [rows, cols], scales [rows/128, cols/128, 512]
    uint8_t* qt[3]; uint8_t* sct[3];        // transposed layout [cols, t_rows], scales [cols/128, t_rows/128, 512]
    int q_cols;                             // intermediate size I
    int t_rows;                             // macrobatch size (row length of the transposed tensors)
    // DgradDown inputs: saved gate / up
    const uint8_t* in_q[2]; const uint8_t* in_sc[2];
    const float* row_scale;
    float* partials;
    float limit;
    int has_limit;
    int* status;
};

struct MxScaleMaps {               // unswizzled tensor maps over [tiles, 512 B] scale arrays
    CUtensorMap sfa0, sfa1, sfb0, sfb1;
};
// descriptor of a dense 32 x 16-byte scale block for tcgen05.cp (no swizzle, 8-row groups 128 B apart)
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= 1ull << 46;
    return d;
}

// quantise one 32-wide chunk of a row (16 packed bf16 words) along the row and store bytes + scale
__device__ __forceinline__ void mx_store_normal(const uint32_t (&w)[16], uint8_t* q, uint8_t* sc, size_t row, int col0, int cols) {
    uint32_t out[8], sb;
    mx_quantize_block(w, out, sb);
    st_global_256(q + row * cols + col0, out[0], out[1], out[2], out[3], out[4], out[5], out[6], out[7]);
    sc[mx_scale_offset(static_cast<int>(row), col0 >> 5, cols >> 7)] = static_cast<uint8_t>(sb);
}
// quantise the same chunk along the token axis.  The warp's 32 lanes hold rows row0..row0+31 (one MX
// block) of 32 columns; the chunk is transposed through a padded per-warp shared-memory tile so that
// lane j ends up with column j's 32 values and writes its 32 bytes to qt[col0+j][row0..row0+31].
constexpr int kMxTrWords = 32 * 17;
__device__ __forceinline__ void mx_store_transposed(const uint32_t (&w)[16], uint32_t* tr, uint8_t* qt, uint8_t* sct, size_t row,
                                                    int col0, int t_rows, int lane) {
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 16; ++i) tr[lane * 17 + i] = w[i];
    __syncwarp();
    uint32_t in[16], out[8], sb;
    const int wsel = lane >> 1, hsel = (lane & 1) * 16;
#pragma unroll
    for (int r2 = 0; r2 < 16; ++r2) {
        const uint32_t lo = (tr[(2 * r2) * 17 + wsel] >> hsel) & 0xFFFFu;
        const uint32_t hi = (tr[(2 * r2 + 1) * 17 + wsel] >> hsel) & 0xFFFFu;
        in[r2] = lo | (hi << 16);
    }
    mx_quantize_block(in, out, sb);
    const size_t row0 = row - lane;
    st_global_256(qt + static_cast<size_t>(col0 + lane) * t_rows + row0, out[0], out[1], out[2], out[3], out[4], out[5], out[6],
                  out[7]);
    sct[mx_scale_offset(col0 + lane, static_cast<int>(row0 >> 5), t_rows >> 7)] = static_cast<uint8_t>(sb);
}

template <int kEpi, bool kWgrad, bool k2>
__global__ void __launch_bounds__(kMxThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
               const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
               const __grid_constant__ MxScaleMaps sfm, const MxGemmParams p) {
    constexpr int kMxStages = mx_stages(kEpi, k2);
    constexpr int kTile = mx_tile_bytes(k2);
    constexpr int kTileM = k2 ? 2 * kBlockM : kBlockM;
    const uint32_t cta_rank = k2 ? cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    const int tile_first = k2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = k2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* sf_smem = smem + kMxStages * kTile;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(sf_smem + kMxStages * kMxSfBytes);
    uint64_t* empty_bar = full_bar + kMxStages;
    uint64_t* tfull_bar = empty_bar + kMxStages;
    uint64_t* tempty_bar = tfull_bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_end = reinterpret_cast<int*>(sf_smem + kMxStages * kMxSfBytes + 256);
    uint32_t* tr_smem = reinterpret_cast<uint32_t*>(sf_smem + kMxStages * kMxSfBytes + 256 + kMaxExperts * 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int E = p.tokens_per_expert ? p.num_experts : 1;
    if (p.tokens_per_expert) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) s_end[e] = p.tokens_per_expert[e];
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kMxStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(tfull_bar, 1);
        mbar_init(tempty_bar, k2 ? 2 * kMxEpiWarps : kMxEpiWarps);   // the leader's copy collects both CTAs' warps
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
    int chunk_lo = 0, chunk_hi = win_rows;
    if (!kWgrad) chunk_range(win_rows, p.chunk, chunk_lo, chunk_hi);
    const int m_tile0 = chunk_lo / kTileM;
    const int m_tiles_w = k2 ? p.m_tiles_w >> 1 : p.m_tiles_w;
    const int num_tiles = kWgrad ? ((p.accumulate && win_rows == 0) ? 0 : E * m_tiles_w * p.n_tiles)
                                 : ((chunk_hi - chunk_lo) / kTileM) * p.n_tiles;

    auto decode = [&](int tile, int& m_idx, int& n_idx, int& expert, int& k_row0, int& k_tiles) {
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
            k_tiles = hi > lo ? (hi - lo) / kMxBlockK : 0;
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
            k_tiles = p.k_tiles_per_seg * p.num_segs;
        }
    };

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(mx_light_regs(kEpi, k2)));
    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            tma_prefetch_desc(&tmA0); tma_prefetch_desc(&tmB0);
            tma_prefetch_desc(&sfm.sfa0); tma_prefetch_desc(&sfm.sfb0);
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step) {
                int m_idx, n_idx, expert, k_row0, k_tiles;
                decode(tile, m_idx, n_idx, expert, k_row0, k_tiles);
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* sa = smem + stage * kTile;
                    uint8_t* sb = sa + kMxABytes;
                    uint8_t* ssfa = sf_smem + stage * kMxSfBytes;
                    uint8_t* ssfb = ssfa + 512;
                    if (leader) mbar_arrive_expect_tx(&full_bar[stage], (k2 ? 2 : 1) * (kTile + kMxSfBytes));
                    auto load = [&](void* dst, const CUtensorMap* map, int x, int y) {
                        if (k2) tma_load_2d_pair(dst, map, &full_bar[stage], x, y);
                        else tma_load_2d(dst, map, &full_bar[stage], x, y);
                    };
                    const int seg = (!kWgrad && kt >= p.k_tiles_per_seg) ? 1 : 0;
                    const int kt_seg = kWgrad ? kt : kt - seg * p.k_tiles_per_seg;
                    const int k_tile_abs = (kWgrad ? k_row0 / kMxBlockK : 0) + kt_seg;      // k-tile index in the tensors
                    const CUtensorMap* ma = seg ? &tmA1 : &tmA0;
                    const CUtensorMap* mb = seg ? &tmB1 : &tmB0;
                    const CUtensorMap* msa = seg ? &sfm.sfa1 : &sfm.sfa0;
                    const CUtensorMap* msb = seg ? &sfm.sfb1 : &sfm.sfb0;
                    // A and its scales: this CTA's 128 rows of the tile
                    const int a_tile = m_idx * (kTileM / kBlockM) + static_cast<int>(cta_rank);
                    load(sa, ma, k_tile_abs * kMxBlockK, a_tile * kBlockM);
                    load(ssfa, msa, 0, a_tile * p.sfa_k_tiles + k_tile_abs);
                    // B: the whole 256 rows (one CTA) or this CTA's 128 (pair); scales of all 256 rows either way
                    if constexpr (kEpi == kMxEpiGateUp) {
                        const int y = expert * p.b_rows_per_expert + n_idx * (kBlockN / 2);
                        if (k2) {                           // the leader holds the gate rows, its partner the up rows
                            load(sb, leader ? &tmB0 : &tmB1, k_tile_abs * kMxBlockK, y);
                        } else {
                            load(sb, &tmB0, k_tile_abs * kMxBlockK, y);
                            load(sb + kMxBBytes / 2, &tmB1, k_tile_abs * kMxBlockK, y);
                        }
                        const int so = (y >> 7) * p.sfb_k_tiles + k_tile_abs;
                        load(ssfb, &sfm.sfb0, 0, so);
                        load(ssfb + 512, &sfm.sfb1, 0, so);
                    } else {
                        const int y = (kWgrad ? 0 : expert * p.b_rows_per_expert) + n_idx * kBlockN;
                        if (k2) {
                            load(sb, mb, k_tile_abs * kMxBlockK, y + static_cast<int>(cta_rank) * (kBlockN / 2));
                        } else {
                            load(sb, mb, k_tile_abs * kMxBlockK, y);
                        }
                        const int so = (y >> 7) * p.sfb_k_tiles + k_tile_abs;
                        load(ssfb, msb, 0, so);
                        load(ssfb + 512, msb, 0, so + p.sfb_k_tiles);
                    }
                    if (++stage == kMxStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc_mxf8(kTileM, kBlockN, 0, 0);
            int stage = 0; uint32_t phase = 0;
            uint32_t sf_slot = 0;
            int it = 0;
            bool ok = true;
            for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++it) {
                int m_idx, n_idx, expert, k_row0, k_tiles;
                decode(tile, m_idx, n_idx, expert, k_row0, k_tiles);
                if (!mbar_wait(tempty_bar, (it & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * kTile);
                    const uint32_t sb = sa + kMxABytes;
                    const uint32_t ssf = smem_u32(sf_smem + stage * kMxSfBytes);
                    // the scales of consecutive k-tiles go to different tensor-memory columns, so this copy does not
                    // have to wait for the previous k-tile's MMAs to finish reading theirs
                    const uint32_t sfa_t = tmem_base + kMxSfaCol + sf_slot * kMxSfSlotCols;
                    const uint32_t sfb_t = sfa_t + 4;
                    sf_slot = (sf_slot + 1) & (kMxSfSlots - 1);
                    if (k2) {
                        tmem_cp_32x128b_warpx4_pair(sfa_t, make_sf_desc(ssf));
                        tmem_cp_32x128b_warpx4_pair(sfb_t, make_sf_desc(ssf + 512));
                        tmem_cp_32x128b_warpx4_pair(sfb_t + 4, make_sf_desc(ssf + 1024));
                    } else {
                        tmem_cp_32x128b_warpx4(sfa_t, make_sf_desc(ssf));
                        tmem_cp_32x128b_warpx4(sfb_t, make_sf_desc(ssf + 512));
                        tmem_cp_32x128b_warpx4(sfb_t + 4, make_sf_desc(ssf + 1024));
                    }
                    const uint64_t adesc = make_smem_desc(sa, 16, 1024);
                    const uint64_t bdesc = make_smem_desc(sb, 16, 1024);
#pragma unroll
                    for (int k = 0; k < kMxBlockK / 32; ++k) {
                        const uint32_t id = idesc | (static_cast<uint32_t>(k) << 29) | (static_cast<uint32_t>(k) << 4);
                        if (k2) umma_mxf8_pair(tmem_base, adesc + ((k * 32) >> 4), bdesc + ((k * 32) >> 4), id, sfa_t, sfb_t,
                                               (kt > 0 || k > 0) ? 1u : 0u);
                        else umma_mxf8(tmem_base, adesc + ((k * 32) >> 4), bdesc + ((k * 32) >> 4), id, sfa_t, sfb_t,
                                       (kt > 0 || k > 0) ? 1u : 0u);
                    }
                    if (k2) umma_commit_pair(&empty_bar[stage]); else umma_commit(&empty_bar[stage]);
                    if (++stage == kMxStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (k_tiles > 0) { if (k2) umma_commit_pair(tfull_bar); else umma_commit(tfull_bar); }
                else { mbar_arrive(tfull_bar); if (k2) mbar_arrive_cta(tfull_bar, 1); }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(mx_epi_regs(kEpi, k2)));
        // ------------------------------------------------------------------ epilogue warps
        // Sixteen warps: four per TMEM lane quarter (a warp may only read lanes 32*(warp%4)...), each taking
        // 64 of the tile's 256 columns, so a thread holds its share of the accumulator as 32 packed words.
        // More resident warps also hide the latency of the epilogue's loads and stores.
        const int quarter = warp & 3;
        const int sub = (warp - 4) >> 2;                 // 0..3
        const int r_in_tile = quarter * 32 + lane;
        uint32_t* tr = tr_smem + (warp - 4) * kMxTrWords;
        int it = 0;
        bool ok = true;
        for (int tile = tile_first; tile < num_tiles && ok; tile += tile_step, ++it) {
            int m_idx, n_idx, expert, k_row0, k_tiles;
            decode(tile, m_idx, n_idx, expert, k_row0, k_tiles);
            if (!mbar_wait(tfull_bar, it & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            const size_t row = static_cast<size_t>(m_idx) * kTileM + cta_rank * kBlockM + r_in_tile;
            uint32_t pk[kEpi == kMxEpiDgradDown ? 1 : 32];
            if constexpr (kEpi == kMxEpiDgradDown) {
                // d_hidden is an output of its own: each 32-column chunk goes from tensor memory straight to global
                // memory as bf16 and is read back (this thread's own 64 bytes) when the SwiGLU backward needs it
                __nv_bfloat16* dh16 = p.out_bf16 + row * p.ld_out + n_idx * kBlockN + sub * 64;
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t acc[32];
                    tmem_ld_32x32(t_addr + (sub * 2 + c) * 32, acc);
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 2; ++v)
                        st_global_256(dh16 + c * 32 + v * 16,
                                      pack_bf16(__uint_as_float(acc[16 * v + 0]), __uint_as_float(acc[16 * v + 1])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 2]), __uint_as_float(acc[16 * v + 3])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 4]), __uint_as_float(acc[16 * v + 5])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 6]), __uint_as_float(acc[16 * v + 7])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 8]), __uint_as_float(acc[16 * v + 9])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 10]), __uint_as_float(acc[16 * v + 11])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 12]), __uint_as_float(acc[16 * v + 13])),
                                      pack_bf16(__uint_as_float(acc[16 * v + 14]), __uint_as_float(acc[16 * v + 15])));
                }
            } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                // GateUp: chunk `sub` of the gate half and chunk `sub` of the up half; otherwise two adjacent chunks
                const int col = (kEpi == kMxEpiGateUp) ? (c * (kBlockN / 2) + sub * 32) : (sub * 2 + c) * 32;
                uint32_t acc[32];
                if (k_tiles > 0) { tmem_ld_32x32(t_addr + col, acc); tmem_ld_wait(); }
                else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = 0u;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) pk[c * 16 + i] = pack_bf16(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1]));
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (k2) mbar_arrive_leader(tempty_bar); else mbar_arrive(tempty_bar); }   // accumulator is free

            if constexpr (kEpi == kMxEpiStore) {
                if (!(kWgrad && p.accumulate && k_tiles == 0)) {
                    __nv_bfloat16* dst = p.out_bf16 + (kWgrad ? static_cast<size_t>(expert) * p.out_expert_stride : 0) +
                                         row * p.ld_out + static_cast<size_t>(n_idx) * kBlockN + sub * 64;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {            // 16 columns = 32 bytes per 256-bit access
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = pk[8 * v + i];
                        if (kWgrad && p.accumulate) {
                            uint32_t q[8];
                            ld_global_256(dst + v * 16, q);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float2 a = unpack_bf16(o[i]), b = unpack_bf16(q[i]);
                                o[i] = pack_bf16(a.x + b.x, a.y + b.y);
                            }
                        }
                        st_global_256(dst + v * 16, o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]);
                    }
                }
            } else if constexpr (kEpi == kMxEpiGateUp) {
                const int col0 = n_idx * (kBlockN / 2) + sub * 32;
                // saved gate and up go out first; the hidden chunk is formed only after their temporaries are dead
                {
                    uint32_t g[16], u[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) { g[i] = pk[i]; u[i] = pk[16 + i]; }
                    mx_store_normal(g, p.q[0], p.sc[0], row, col0, p.q_cols);
                    mx_store_normal(u, p.q[1], p.sc[1], row, col0, p.q_cols);
                }
                uint32_t h[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 gf = unpack_bf16(pk[i]), uf = unpack_bf16(pk[16 + i]);
                    if (p.has_limit) {
                        gf.x = fminf(gf.x, p.limit); gf.y = fminf(gf.y, p.limit);
                        uf.x = fminf(fmaxf(uf.x, -p.limit), p.limit); uf.y = fminf(fmaxf(uf.y, -p.limit), p.limit);
                    }
                    h[i] = pack_bf16(silu_mul(gf.x, uf.x), silu_mul(gf.y, uf.y));
                }
                mx_store_normal(h, p.q[2], p.sc[2], row, col0, p.q_cols);
                mx_store_transposed(h, tr, p.qt[2], p.sct[2], row, col0, p.t_rows, lane);
            } else {
                // d_hidden was stored above; it comes back 32 columns at a time (from L1/L2), so no copy of the
                // accumulator stays in registers beside the SwiGLU temporaries
                float inv_w = 0.0f;
                if (p.row_scale) { const float w = p.row_scale[row]; inv_w = w > 0.0f ? 1.0f / w : 0.0f; }
                float partial = 0.0f;
                const int colbase = n_idx * kBlockN + sub * 64;
                const __nv_bfloat16* dh16 = p.out_bf16 + row * p.ld_out + colbase;
                const size_t so0 = mx_scale_offset(static_cast<int>(row), colbase >> 5, p.q_cols >> 7);   // 2 consecutive bytes
                const uint32_t gsc2 = *reinterpret_cast<const uint16_t*>(p.in_sc[0] + so0);
                const uint32_t usc2 = *reinterpret_cast<const uint16_t*>(p.in_sc[1] + so0);
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    const int col0 = colbase + c * 32;
                    const float gs = mx_scale_value((gsc2 >> (8 * c)) & 0xFFu), us = mx_scale_value((usc2 >> (8 * c)) & 0xFFu);
                    uint32_t gb[8], ub[8], dh[2][8];         // 32 saved fp8 gate / up values, 32 bf16 d_hidden values
                    ld_global_256(p.in_q[0] + row * p.q_cols + col0, gb);
                    ld_global_256(p.in_q[1] + row * p.q_cols + col0, ub);
                    ld_global_256(dh16 + c * 32, dh[0]);
                    ld_global_256(dh16 + c * 32 + 16, dh[1]);
                    uint32_t dg[16], du[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint16_t g2 = static_cast<uint16_t>(gb[i >> 1] >> ((i & 1) * 16));
                        const uint16_t u2 = static_cast<uint16_t>(ub[i >> 1] >> ((i & 1) * 16));
                        float2 gf = mx_unpack2(g2, gs), uf = mx_unpack2(u2, us);
                        const float2 dhf = unpack_bf16(dh[i >> 3][i & 7]);
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
                        dg[i] = pack_bf16(gm0 ? ds0 * uf.x * dhf.x : 0.0f, gm1 ? ds1 * uf.y * dhf.y : 0.0f);
                        du[i] = pack_bf16(um0 ? silu0 * dhf.x : 0.0f, um1 ? silu1 * dhf.y : 0.0f);
                        partial += dhf.x * inv_w * (silu0 * uf.x) + dhf.y * inv_w * (silu1 * uf.y);
                    }
                    mx_store_normal(dg, p.q[0], p.sc[0], row, col0, p.q_cols);
                    mx_store_transposed(dg, tr, p.qt[0], p.sct[0], row, col0, p.t_rows, lane);
                    mx_store_normal(du, p.q[1], p.sc[1], row, col0, p.q_cols);
                    mx_store_transposed(du, tr, p.qt[1], p.sct[1], row, col0, p.t_rows, lane);
                }
                if (p.partials) p.partials[row * (4 * p.n_tiles) + 4 * n_idx + sub] = partial;   // four column slices per tile
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (k2) cluster_sync_all();        // neither CTA frees tensor memory or exits while its partner may still signal it
    if (warp == 1) { tc_fence_after(); if (k2) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols); }
    if (threadIdx.x == 0 && *abort_flag) report_status(p.status, MOK_STATUS_PIPELINE_TIMEOUT, 100 + warp);
}

struct MxGemmOperands {
    const void* a0; const void* b0; const void* a1; const void* b1;
    uint64_t a_inner, a_outer, b_inner, b_outer;      // bytes of K per row, rows
};
int launch_mx_gemm(int epi, bool wgrad, const MxGemmOperands& ops, const MxGemmParams& p, int max_tiles, int max_ctas,
                   int prof_slot, cudaStream_t stream, bool allow_pairs = true);

}  // namespace mok
