/* C ABI of libmok_b200: the B200 (sm_100a) implementation of the Mixture-of-Kittens MoE
 * hot path (schedule -> dispatch -> grouped SwiGLU expert FFN -> combine, forward and
 * backward).  Plain pointers and sizes only; no torch or C++ types cross this boundary.
 *
 * Conventions
 *  - Every entry point launches on `stream` (a cudaStream_t passed as void*) and returns
 *    immediately: 0 on success, a negative MOK_ERR_* for errors the host can detect.
 *  - Errors only the device can detect (schedule overflow, a wait that ran out) are written
 *    to the caller's status word: int32[4] in device memory = {code, detail, block, 0},
 *    first error wins.  The library never traps and never waits without a limit.
 *  - The library allocates no device memory.  Callers own inputs, outputs and scratch.  (Its image
 *    carries one fixed 4 MiB __device__ array, resident on every GPU that loads the library: the
 *    scratch of mok_schedule_static, see there.)
 *  - "Reference" citations give the file:line of the interface in the Mixture-of-Kittens
 *    project that the entry point stands in for.
 */
#ifndef MOK_B200_H_
#define MOK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOK_MAX_PEERS 8          /* expert-parallel ranks on one NVSwitch box */
#define MOK_MAX_LOCAL_EXPERTS 1024

/* host-detected errors (return values) */
#define MOK_OK 0
#define MOK_ERR_INVALID (-1)     /* argument outside the documented domain */
#define MOK_ERR_CUDA (-2)        /* a CUDA runtime / driver call failed */
#define MOK_ERR_UNSUPPORTED (-3) /* shape or mode this build does not implement */
#define MOK_ERR_TOO_LARGE (-4)   /* problem exceeds a fixed, documented size limit of the entry point */

/* device-detected errors (status word code) */
#define MOK_STATUS_OK 0
#define MOK_STATUS_SCHEDULE_OVERFLOW 1 /* padded routes exceed schedule_capacity; detail = needed rows */
#define MOK_STATUS_BARRIER_TIMEOUT 2   /* a peer never arrived at mok_barrier_all; detail = counter seen */
#define MOK_STATUS_PIPELINE_TIMEOUT 3  /* an in-kernel producer/consumer wait ran out; detail = role */

int mok_version(void);
const char* mok_error_string(int code);
/* Name, text and source position of the last CUDA runtime call that failed inside this library on the calling
 * host thread ("" if none): the detail behind a MOK_ERR_CUDA return.  No reference counterpart. */
const char* mok_last_cuda_error(void);

/* Sizes, in bytes, of everything a caller has to allocate around the layer for one problem shape: the eight
 * rank-visible buffers of a workspace (each rank allocates the same sizes and exchanges the addresses), the
 * barrier state, the status word, the four schedule tables together, and the scheduler's scratch.
 * schedule_capacity = T * topk * max(2, ceil(ep_size * multiplier)) rows.
 * Reference: mok/functional.py:160-281 (create_workspace: the same buffers and the same capacity formula,
 * :196,206), csrc/scheduler.cuh:149-183 (the tables scheduler::schedule allocates). */
typedef struct mok_workspace_bytes {
    int64_t schedule_capacity;               /* rows */
    size_t x_buffer, combine_buffer;         /* bf16 [T, H], [T*K, H] */
    size_t d_y_buffer, d_x_routed_buffer;    /* bf16 [T, H], [T*K, H] */
    size_t router_weight_buffer, d_router_weight_buffer;   /* f32 [T, K] */
    size_t all_gather_top_experts_buffer;    /* i32 [ep_size, T, K] */
    size_t barrier_buffer, barrier_target;   /* u32 [1] each; both start at zero */
    size_t status_word;                      /* i32 [4], starts at zero */
    size_t schedule_tables;                  /* peer_rank + peer_token_idx [cap] + num_tokens [1] + tokens_per_expert [El] */
    size_t schedule_scratch;                 /* = mok_schedule_scratch_bytes(ep_size, El) */
} mok_workspace_bytes;
int mok_query_workspace_bytes(int ep_size, int num_local_tokens, int hidden, int topk, int num_local_experts,
                              double schedule_capacity_multiplier, mok_workspace_bytes* out);

/* Reads the caller's status word back to the host: copies the four int32 {code, detail, block, 0} from
 * `status_device` into `out_host`, optionally zeroes the word afterwards, and waits for `stream` (so it also
 * waits for the layer calls enqueued there).  The layer entry points never synchronise; call this at step
 * boundaries, where a host synchronisation is acceptable.
 * Reference: none as a function; it stands where the reference would have trapped (csrc/scheduler.cuh:86) or
 * spun without limit (csrc/utils.cuh:291-293, csrc/mok_megakernel.cuh:298-302). */
int mok_last_status(int32_t* status_device, int32_t* out_host, int clear, void* stream);

/* All-gather of the int32 top-k expert ids: rank `rank` stores its `numel` ids into slot `rank`
 * of every peer's [ep_size, numel] buffer with plain peer stores over NVLink.
 * Reference: mok/ops.py:6-58 (all_gather_top_experts), csrc/utils.cuh:230-263. */
int mok_all_gather_top_experts(const int32_t* top_experts, int64_t numel,
                               const uint64_t* peer_buffer_ptrs, int ep_size, int rank, void* stream);

/* Device-side barrier over the expert-parallel ranks: target += ep_size, every rank adds 1 to
 * each peer's counter, then waits until its own counter reaches the target.  The wait is bounded by
 * `timeout_ns`; 0 selects the default of two minutes (MOK_B200_BARRIER_TIMEOUT_MS in the environment
 * overrides the default).  On expiry the status word gets MOK_STATUS_BARRIER_TIMEOUT and the stream carries
 * on, so the data a later kernel reads from a peer may not be there yet: check the status word at every step
 * boundary (mok_last_status) and discard the step when it is set.
 * Reference: mok/ops.py:61-100 (barrier_all), csrc/utils.cuh:283-313. */
int mok_barrier_all(uint32_t* local_counter, const uint64_t* peer_counter_ptrs, int ep_size,
                    uint32_t* target, int32_t* status, uint64_t timeout_ns, void* stream);

/* Slot tables of this rank from the gathered top-k ids.  Bit-exact with the reference:
 * thread-major route order over 1024 virtual threads, round-robin interleave of peers, each
 * expert padded to 256 rows; unwritten slots hold -1 in both tables.
 * `scratch` must hold mok_schedule_scratch_bytes() bytes; contents need no initialisation.
 * Reference: mok/ops.py:103-150 (schedule), csrc/scheduler.cuh:35-183. */
size_t mok_schedule_scratch_bytes(int ep_size, int num_local_experts);
int mok_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                 int num_local_experts, int schedule_capacity, int rank,
                 int32_t* schedule_peer_rank, int32_t* schedule_peer_token_idx,
                 int32_t* num_tokens, int32_t* tokens_per_expert,
                 void* scratch, size_t scratch_bytes, int32_t* status, void* stream);

/* The same scheduler for callers that cannot allocate device memory (a server with a fixed
 * memory plan, a latency-critical loop that must not hit cudaMalloc's device synchronisation, a
 * plug-in host that exposes no allocator): the scratch lives in a fixed 4 MiB __device__ array
 * inside the library, resident on every GPU that loads it, so only inputs and outputs are passed.
 * Limit: mok_schedule_scratch_bytes(ep_size, num_local_experts) must not exceed
 * mok_schedule_static_max_scratch_bytes() (ep_size * num_local_experts <= 4080); larger problems
 * return MOK_ERR_TOO_LARGE and launch nothing.  The first call on a device looks up the array's
 * address; make that call outside any stream capture.  Calls on one GPU share the array: calls
 * that overlap on the GPU race, so issue them one after another.  Results are identical to
 * mok_schedule.  This entry point has no counterpart in the reference. */
size_t mok_schedule_static_max_scratch_bytes(void);
int mok_schedule_static(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                        int num_local_experts, int schedule_capacity, int rank,
                        int32_t* schedule_peer_rank, int32_t* schedule_peer_token_idx,
                        int32_t* num_tokens, int32_t* tokens_per_expert, int32_t* status, void* stream);

/* BF16 [E, M, N] -> MXFP8: E4M3 bytes plus one E8M0 scale per 1x32 block along the last
 * dimension, normal and/or transposed; scales in the [rows/128, cols/128, 32, 16] tcgen05
 * block-scale layout.  Pass NULL for a layout that is not wanted.
 * Reference: mok/ops.py:153-191 (mxfp8_quantize), csrc/mxfp8.cuh:45-72,184-278. */
int mok_mxfp8_quantize(const void* x_bf16, int num_matrices, int rows, int cols,
                       void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, void* stream);

/* out[t] = bf16(y_shared[t] + sum_k w[t,k] * combine[t*K+k]) in fp32, k ascending.
 * Reference: mok/ops.py:1011-1045 (fwd_epilogue), csrc/utils.cuh:65-133. */
int mok_fwd_epilogue(const void* y_shared, const void* combine_buffer, const float* topk_weights,
                     void* output, int num_local_tokens, int hidden, int topk, void* stream);

/* d_x[t] = bf16(d_x_shared[t] + sum_k d_x_routed_buffer[t*K+k]) in fp32, k ascending.
 * Reference: mok/ops.py:1048-1081 (bwd_epilogue), csrc/utils.cuh:158-205. */
int mok_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* d_x,
                     int num_local_tokens, int hidden, int topk, void* stream);

/* Router in front of the path: for every token the K largest logits (descending, lower expert index first among
 * equal values) and the softmax over those K values = softmax over all experts, top-K, renormalise.
 * logits f32 [num_tokens, num_experts] (num_experts <= 1024, topk <= 32).  Outputs, each optional except the
 * weights: top_experts_i32 [T,K], top_experts_i64 [T,K] (the dtype build_schedule takes), router_weights f32 [T,K];
 * with all_gather_ptrs (ep_size addresses of the [ep_size, T, K] int32 all-gather buffers) the int32 routes are also
 * written into slot ep_rank of every rank's buffer, which replaces the cast + mok_all_gather_top_experts of
 * build_schedule (a barrier must still follow before mok_schedule reads the buffer).
 * mok_router_topk_bwd: d_logits f32 [T, E] (fully written) from d_router_weights.
 * No reference counterpart: the reference takes finished routes (mok/functional.py:354-430); its tests build them
 * with torch.topk + softmax (tests/utils.py:82-84), which is the law implemented here. */
int mok_router_topk(const float* logits, int num_tokens, int num_experts, int topk, int32_t* top_experts_i32,
                    int64_t* top_experts_i64, float* router_weights, const uint64_t* all_gather_ptrs, int ep_size,
                    int ep_rank, void* stream);
int mok_router_topk_bwd(const int32_t* top_experts_i32, const float* router_weights, const float* d_router_weights,
                        float* d_logits, int num_tokens, int num_experts, int topk, void* stream);

/* Single-rank epilogues that gather the routed rows through the schedule instead of reading a combine buffer:
 *   out[t] = bf16(y_shared[t] + sum_k w[t,k] * y_routed[row(t,k)])            (forward)
 *   d_x[t] = bf16(d_x_shared[t] + sum_k d_x_routed[row(t,k)]),
 *   d_router_weights[t,k] = sum over columns of partials[row(t,k), :]          (backward)
 * where row(t,k) is the schedule row whose peer_token_idx is t*K+k, the same fp32 sums in the same k order as
 * mok_fwd_epilogue / mok_bwd_epilogue after a combine, so results are bit-identical to the two-step path.  They
 * follow a layer call made with defer_combine = 1 and save the combine pass over [T*K, hidden] (one write and
 * one read of it).  `route_row` is caller-provided scratch of T*K int32.  A route without a row (capacity
 * overflow, flagged in the status word by the scheduler) contributes zero.
 * No reference counterpart: the reference always combines into the symmetric buffer and then runs
 * fwd_epilogue / bwd_epilogue (mok/functional.py:569-571, 698-700). */
int mok_fwd_epilogue_rows(const void* y_shared, const void* y_routed, const int32_t* schedule_peer_rank,
                          const int32_t* schedule_peer_token_idx, const int32_t* num_tokens,
                          const float* topk_weights, int32_t* route_row, void* output, int num_local_tokens,
                          int hidden, int topk, int row_limit, void* stream);
int mok_bwd_epilogue_rows(const void* d_x_shared, const void* d_x_routed, const float* partials, int partial_cols,
                          const int32_t* schedule_peer_rank, const int32_t* schedule_peer_token_idx,
                          const int32_t* num_tokens, int32_t* route_row, void* d_x, float* d_router_weights,
                          int num_local_tokens, int hidden, int topk, int row_limit, void* stream);

/* ---- the fused layer passes -------------------------------------------------------------
 * All tensors are row-major and contiguous.  T = num_local_tokens, H = hidden, I = intermediate,
 * El = num_local_experts, K = topk, MB = macrobatch_size, cap = schedule_capacity.  Pointer
 * arrays `*_ptrs` hold ep_size device addresses, one per rank (own rank included).
 * Every tensor address must be 32-byte aligned (the kernels use 256-bit accesses and TMA); allocations of the CUDA
 * runtime and of PyTorch are. */

typedef struct mok_layer_common {
    int ep_size, ep_rank;
    int num_local_tokens, hidden, intermediate, num_local_experts, topk;
    int schedule_capacity, macrobatch_size, minibatch_size;
    int num_comm_sms;                       /* SM budget of the row movement, as the reference's fwd/bwd_num_comm_sms
                                               (mok/functional.py:22-29).  Used with ep_size > 1 while a window is cut into
                                               chunks (at least two minibatches): dispatch and combine run as 16 thin
                                               bulk-copy CTAs per budgeted SM beside the GEMM CTAs (default), or, with
                                               MOK_B200_DEDICATED_COMM_SMS=1, as one fat CTA on each of that many SMs of
                                               their own while the routed GEMM grids shrink by the same number (capped at
                                               half the GPU).  Results never depend on it.  MOK_B200_COMM_SMS in the
                                               environment overrides the value of every call. */
    int has_swiglu_limit;
    float swiglu_limit;
    int defer_combine;                      /* 1: leave the routed results in their rows (y_routed, or d_x_routed and the
                                               router-gradient partials) for mok_*_epilogue_rows instead of moving them
                                               to the combine buffers; accepted only with ep_size 1 and
                                               schedule_capacity <= macrobatch_size, else MOK_ERR_INVALID */
    const int32_t* schedule_peer_rank;      /* [cap] */
    const int32_t* schedule_peer_token_idx; /* [cap] */
    const int32_t* num_tokens;              /* [1]   */
    const int32_t* tokens_per_expert;       /* [El]  */
    int32_t* status;                        /* [4] or NULL */
} mok_layer_common;

/* Forward, BF16 routed experts.
 * Reference: mok/ops.py:371-514 (dispatch_mlp_swiglu_combine_fwd_bf16),
 * csrc/mok_megakernel.cuh:1561-1851,1990-2100. */
typedef struct mok_fwd_bf16_args {
    mok_layer_common c;
    const uint64_t* x_ptrs;              /* per-rank x buffers [T, H] bf16 */
    const uint64_t* combine_buffer_ptrs; /* per-rank combine buffers [T*K, H] bf16 */
    const void *w_shared_gate, *w_shared_up, *w_shared_down; /* [I,H] [I,H] [H,I] bf16 */
    const void *w_routed_gate, *w_routed_up, *w_routed_down; /* [El,I,H] [El,I,H] [El,H,I] bf16 */
    /* outputs */
    void *x_routed;                               /* [MB, H] */
    void *gate_shared, *up_shared, *hidden_shared; /* [T, I]  */
    void *gate_routed, *up_routed, *hidden_routed; /* [MB, I] */
    void *y_shared;                               /* [T, H]  */
    void *y_routed;                               /* [MB, H] */
} mok_fwd_bf16_args;
int mok_fwd_bf16(const mok_fwd_bf16_args* args, void* stream);

/* Backward, BF16 routed experts.  Mutates the saved routed activations when the schedule
 * spans more than one macrobatch (forward replay), as the reference does.
 * Reference: mok/ops.py:811-1008 (dispatch_mlp_swiglu_combine_bwd_bf16),
 * csrc/mok_megakernel.cuh:2102-2544,2779-2967. */
typedef struct mok_bwd_bf16_args {
    mok_layer_common c;
    const uint64_t* d_y_ptrs;                    /* per-rank upstream grads [T, H] bf16 */
    const uint64_t* d_x_routed_buffer_ptrs;      /* per-rank [T*K, H] bf16 */
    const uint64_t* router_weight_ptrs;          /* per-rank [T, K] f32 */
    const uint64_t* d_router_weight_ptrs;        /* per-rank [T, K] f32 */
    const uint64_t* x_ptrs;                      /* per-rank x [T, H] bf16 */
    const void *w_shared_gate, *w_shared_up, *w_shared_down;
    const void *w_routed_gate, *w_routed_up, *w_routed_down;
    /* saved forward activations (routed ones are overwritten by replay) */
    void *x_routed, *gate_routed, *up_routed, *hidden_routed;
    const void *gate_shared, *up_shared, *hidden_shared;
    /* outputs */
    void *d_x_shared;                                     /* [T, H]  */
    void *d_x_routed;                                     /* [MB, H] */
    void *d_gate_shared, *d_up_shared, *d_hidden_shared;  /* [T, I]  */
    void *d_gate_routed, *d_up_routed, *d_hidden_routed;  /* [MB, I] */
    void *d_y_routed;                                     /* [MB, H] */
    void *d_w_shared_gate, *d_w_shared_up, *d_w_shared_down;
    void *d_w_routed_gate, *d_w_routed_up, *d_w_routed_down;
    /* scratch: router weights per routed row [MB] f32, router-grad partials [MB, I/128] f32 */
    float* router_weights_routed;
    float* d_router_weight_partials;
} mok_bwd_bf16_args;
int mok_bwd_bf16(const mok_bwd_bf16_args* args, void* stream);

/* Forward, MXFP8 routed experts (E4M3 + E8M0 scale per 32 along K; shared expert stays BF16).
 * `*_q` are E4M3 bytes, `*_sc` scale tensors [rows/128, cols/128, 32, 16].  The four "work" tensors
 * are caller-provided scratch: x_q [MB,H], x_sc, hidden_q [MB,I], hidden_sc.
 * Reference: mok/ops.py:194-368 (dispatch_mlp_swiglu_combine_fwd_mxfp8),
 * csrc/mok_megakernel.cuh:1853-1988. */
typedef struct mok_fwd_mxfp8_args {
    mok_layer_common c;
    const uint64_t* x_ptrs;
    const uint64_t* combine_buffer_ptrs;
    const void *w_shared_gate, *w_shared_up, *w_shared_down;                 /* bf16 */
    const void *w_routed_gate_q, *w_routed_gate_sc;                          /* [El,I,H] */
    const void *w_routed_up_q, *w_routed_up_sc;                              /* [El,I,H] */
    const void *w_routed_down_q, *w_routed_down_sc;                          /* [El,H,I] */
    /* outputs */
    void *x_qt, *x_sct;                                                      /* [H, MB] */
    void *gate_shared, *up_shared, *hidden_shared;                           /* bf16 [T, I] */
    void *gate_q, *gate_sc, *up_q, *up_sc;                                   /* [MB, I] */
    void *hidden_qt, *hidden_sct;                                            /* [I, MB] */
    void *y_shared, *y_routed;                                               /* bf16 */
    /* scratch */
    void *work_x_q, *work_x_sc, *work_hidden_q, *work_hidden_sc;
} mok_fwd_mxfp8_args;
int mok_fwd_mxfp8(const mok_fwd_mxfp8_args* args, void* stream);

/* Backward, MXFP8 routed experts.  Weights come pre-transposed for the data gradients
 * (w_*_T: gate/up as [El,H,I], down as [El,I,H]); the untransposed gate/up weights are only read
 * when a later macrobatch has to be replayed.
 * Reference: mok/ops.py:517-808 (dispatch_mlp_swiglu_combine_bwd_mxfp8),
 * csrc/mok_megakernel.cuh:2546-2777. */
typedef struct mok_bwd_mxfp8_args {
    mok_layer_common c;
    const uint64_t* d_y_ptrs;
    const uint64_t* d_x_routed_buffer_ptrs;
    const uint64_t* router_weight_ptrs;
    const uint64_t* d_router_weight_ptrs;
    const uint64_t* x_ptrs;
    const void *w_shared_gate, *w_shared_up, *w_shared_down;
    const void *w_routed_gate_T_q, *w_routed_gate_T_sc, *w_routed_up_T_q, *w_routed_up_T_sc;
    const void *w_routed_down_T_q, *w_routed_down_T_sc;
    const void *w_routed_gate_q, *w_routed_gate_sc, *w_routed_up_q, *w_routed_up_sc;   /* replay */
    /* saved forward activations (routed ones are overwritten by replay) */
    void *x_qt, *x_sct, *gate_q, *gate_sc, *up_q, *up_sc, *hidden_qt, *hidden_sct;
    const void *gate_shared, *up_shared, *hidden_shared;
    /* outputs */
    void *d_x_shared, *d_x_routed;
    void *d_gate_shared, *d_gate_q, *d_gate_sc;
    void *d_up_shared, *d_up_q, *d_up_sc;
    void *d_hidden_shared, *d_hidden_routed;
    void *d_y_q, *d_y_sc;
    void *d_w_shared_gate, *d_w_shared_up, *d_w_shared_down;
    void *d_w_routed_gate, *d_w_routed_up, *d_w_routed_down;
    /* scratch */
    void *work_x_q, *work_x_sc, *work_hidden_q, *work_hidden_sc;           /* replay */
    void *work_d_y_qt, *work_d_y_sct, *work_d_gate_qt, *work_d_gate_sct, *work_d_up_qt, *work_d_up_sct;
    float* router_weights_routed;                                          /* [MB] */
    float* d_router_weight_partials;                                       /* [MB, I/64] */
} mok_bwd_mxfp8_args;
int mok_bwd_mxfp8(const mok_bwd_mxfp8_args* args, void* stream);

/* Launch accounting for benchmarks.  mok_launch_count(): kernels launched by this library since it
 * was loaded.  With mok_profile_enable(1) every launch is bracketed by CUDA events on its stream;
 * mok_profile_collect() waits for them and adds device milliseconds and launch counts per slot
 * (slot names from mok_profile_slot_name) into arrays of mok_profile_num_slots() entries.
 * No counterpart in the reference (its benchmarks time whole passes only,
 * benchmarks/utils.py:66-110). */
long long mok_launch_count(void);
int mok_profile_enable(int on);
int mok_profile_num_slots(void);
const char* mok_profile_slot_name(int slot);
int mok_profile_collect(double* ms_per_slot, long long* launches_per_slot);

/* Building block exposed for tests and tuning: C[M,N] (bf16) = A * B with fp32 accumulation on
 * tcgen05.  a_mn_major / b_mn_major select the memory layout of the operands:
 *   A: 0 = [M, K] row-major (K-major), 1 = [K, M] row-major (M-major)
 *   B: 0 = [N, K] row-major (K-major), 1 = [K, N] row-major (N-major)
 * M % 256 == 0, N % 256 == 0, K % 64 == 0. */
int mok_gemm_bf16(const void* a, const void* b, void* c, int m, int n, int k,
                  int a_mn_major, int b_mn_major, int32_t* status, void* stream);

/* The same for MXFP8 operands: A [M,K] and B [N,K] as E4M3 bytes with their scale tensors
 * ([rows/128, K/128, 32, 16]), C bf16.  M % 128 == 0, N % 256 == 0, K % 128 == 0. */
int mok_gemm_mxfp8(const void* a_fp8, const void* a_sc, const void* b_fp8, const void* b_sc, void* c,
                   int m, int n, int k, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOK_B200_H_ */
