// Parameters and launchers of the row-movement kernels (dispatch / combine), shared between
// comm.cu and the layer orchestration in layer.cu.
#pragma once

#include <algorithm>

#include "common.cuh"

namespace mok {

struct RowMoveParams {
    PeerPtrs peers;            // per-rank base of the remote [*, hidden] bf16 buffer
    PeerPtrs scale_peers;      // dispatch<scale>: per-rank router weights [T*K] f32 (read)
                               // combine+partials: per-rank d_router_weight [T*K] f32 (written)
    void* local;               // local [row_limit, hidden] bf16 buffer (dispatch: out, combine: in)
    const int* peer_rank;      // [capacity]
    const int* peer_token_idx; // [capacity] = token * topk + k
    const int* num_tokens;     // [1]
    int capacity;
    int row_offset;            // first schedule row of this macrobatch
    int row_limit;             // macrobatch size
    ChunkSpec chunk;           // row sub-range of the window this launch covers
    int hidden;
    int row_divisor;           // dispatch: topk (route -> token row); 1 otherwise
    float* row_scale_out;      // dispatch<scale>: [row_limit] router weight of every routed row
    const float* partials;     // combine: [row_limit, partial_cols] router-gradient partial sums
    int partial_cols;
    int* status;               // device status word (bounded waits report here)
    int fat_ctas;              // 1: few CTAs with 128 KB of copy slots each (dedicated SMs); 0: many thin CTAs
    int lean;                  // thin CTAs of two warps and 16 KB (what fits beside an MXFP8 GEMM CTA) instead of three and 24 KB
    int piece_bytes;           // set by the launcher
};

int launch_dispatch_rows(const RowMoveParams& p, bool scale, int num_blocks, cudaStream_t stream);

// dispatch with fused MXFP8 quantisation: gathered rows are written as E4M3 in both layouts
// (normal [rows, hidden] with scales along hidden; transposed [hidden, t_rows] with scales along
// rows) instead of bf16.  `p.local` is unused.
struct QuantOut {
    uint8_t* q; uint8_t* sc;      // [row_limit, hidden], [row_limit/128, hidden/128, 512]
    uint8_t* qt; uint8_t* sct;    // [hidden, t_rows],    [hidden/128, t_rows/128, 512]
    int t_rows;
};
int launch_dispatch_quant(const RowMoveParams& p, const QuantOut& out, bool scale, int num_blocks, cudaStream_t stream);
int launch_combine_rows(const RowMoveParams& p, int num_blocks, cudaStream_t stream);

}  // namespace mok
