// Layer passes: forward and backward of the expert-parallel MoE layer with BF16 routed experts.
// Each pass is a short, fixed sequence of launches on the caller's stream; all row counts are
// read on the device (num_tokens, tokens_per_expert), so nothing here synchronises with the host.
//
// Forward, per macrobatch window (last window first, so window 0's activations are the ones
// left in the buffers for backward — same contract as the reference megakernel):
//   dispatch rows  ->  [gate|up GEMM + SwiGLU]  ->  down GEMM  ->  combine rows
// plus the dense shared expert on the local tokens.
// Backward, per window (first window first; later windows replay dispatch + gate/up):
//   reverse-combine (w * d_y)  ->  [dgrad down + SwiGLU backward + router-grad partials]
//   ->  dgrad gate+up (one accumulator)  ->  reverse-dispatch (+ router grads)  ->  3 wgrads
#include <climits>
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "comm.cuh"
#include "gemm.cuh"
#include "mxgemm.cuh"

namespace mok {
namespace {

struct Dims {
    int W, rank, T, H, I, El, K, cap, MB;
};

int check_common(const mok_layer_common& c, Dims& d) {
    d = Dims{c.ep_size, c.ep_rank, c.num_local_tokens, c.hidden, c.intermediate, c.num_local_experts, c.topk,
             c.schedule_capacity, c.macrobatch_size};
    if (d.W < 1 || d.W > MOK_MAX_PEERS || d.rank < 0 || d.rank >= d.W) return MOK_ERR_INVALID;
    if (d.T <= 0 || d.T % 256 || d.H <= 0 || d.H % 256 || d.I <= 0 || d.I % 256) return MOK_ERR_INVALID;
    if (d.El < 1 || d.El > MOK_MAX_LOCAL_EXPERTS || d.K < 1 || d.K > 255) return MOK_ERR_INVALID;
    if (d.cap <= 0 || d.cap % 256 || d.MB <= 0 || d.MB % 256) return MOK_ERR_INVALID;
    if (c.minibatch_size <= 0 || c.minibatch_size % 256 || d.MB % c.minibatch_size) return MOK_ERR_INVALID;
    if (!c.schedule_peer_rank || !c.schedule_peer_token_idx || !c.num_tokens || !c.tokens_per_expert) return MOK_ERR_INVALID;
    // results may stay in their rows only when every row is local and one window holds the whole schedule
    if (c.defer_combine && (d.W != 1 || d.cap > d.MB)) return MOK_ERR_INVALID;
    return MOK_OK;
}

int fill_peers(PeerPtrs& out, const uint64_t* ptrs, int W) {
    if (!ptrs) return MOK_ERR_INVALID;
    for (int i = 0; i < W; ++i) {
        if (!ptrs[i]) return MOK_ERR_INVALID;
        out.p[i] = reinterpret_cast<void*>(ptrs[i]);
    }
    return MOK_OK;
}

// How the routed launches of one pipeline step are shaped; the pipeline hands one of these to every launch
// helper, so nothing about a call lives outside its own stack frame.
struct PassCtx {
    ChunkSpec chunk = {0, 1, 0};   // row sub-range of the window the launch covers
    int gemm_ctas = 0;             // cap on the CTAs of routed GEMM launches (0 = all SMs)
    int comm_sms = 0;              // > 0: the call's communication-SM budget applies to the row movers of this launch
    bool dedicated = false;        // the budget is SMs of the movers' own (fat CTAs), not mover CTAs beside the GEMM CTAs
};

GemmParams base_params(const mok_layer_common& c, const PassCtx& x, bool routed, int off, int limit) {
    GemmParams p{};
    if (routed) p.chunk = x.chunk;
    if (routed) {
        p.num_tokens = c.num_tokens;
        p.capacity = c.schedule_capacity;
        p.tokens_per_expert = c.tokens_per_expert;
        p.num_experts = c.num_local_experts;
        p.row_offset = off;
        p.row_limit = limit;
    } else {
        p.rows_host = c.num_local_tokens;
        p.row_limit = c.num_local_tokens;
        p.num_experts = 1;
    }
    p.num_segs = 1;
    p.limit = c.swiglu_limit;
    p.has_limit = c.has_swiglu_limit;
    p.status = c.status;
    return p;
}


// gate|up GEMM with fused SwiGLU: A [rows, H] K-major, B = (Wg, Wu) [E*I, H] K-major
int run_gate_up(const mok_layer_common& c, const PassCtx& x, const Dims& d, bool routed, int off, int limit, const void* a, int a_rows,
                const void* wg, const void* wu, void* gate, void* up, void* hidden, cudaStream_t s) {
    GemmParams p = base_params(c, x, routed, off, limit);
    p.n_tiles = d.I / (kBlockN / 2);
    p.k_blocks_per_seg = d.H / kBlockK;
    p.b_rows_per_expert = d.I;
    p.out0 = static_cast<__nv_bfloat16*>(gate);
    p.out1 = static_cast<__nv_bfloat16*>(up);
    p.out2 = static_cast<__nv_bfloat16*>(hidden);
    p.ld_out = d.I;
    GemmOperands o{};
    o.a0 = a; o.b0 = wg; o.b1 = wu;
    o.a_inner = d.H; o.a_outer = a_rows;
    o.b_inner = d.H; o.b_outer = static_cast<uint64_t>(routed ? d.El : 1) * d.I;
    return launch_grouped_gemm(kMajorK, kMajorK, kEpiSwigluFwd, false, o, p, (limit / kBlockM) * p.n_tiles, routed ? x.gemm_ctas : 0,
                               routed ? kSlotGateUpRouted : kSlotGateUpShared, s);
}

// down GEMM: A = hidden [rows, I] K-major, B = Wd [E*H, I] K-major
int run_down(const mok_layer_common& c, const PassCtx& x, const Dims& d, bool routed, int off, int limit, const void* hidden, int a_rows,
             const void* wd, void* y, cudaStream_t s) {
    GemmParams p = base_params(c, x, routed, off, limit);
    p.n_tiles = d.H / kBlockN;
    p.k_blocks_per_seg = d.I / kBlockK;
    p.b_rows_per_expert = d.H;
    p.out0 = static_cast<__nv_bfloat16*>(y);
    p.ld_out = d.H;
    GemmOperands o{};
    o.a0 = hidden; o.b0 = wd;
    o.a_inner = d.I; o.a_outer = a_rows;
    o.b_inner = d.I; o.b_outer = static_cast<uint64_t>(routed ? d.El : 1) * d.H;
    return launch_grouped_gemm(kMajorK, kMajorK, kEpiStore, false, o, p, (limit / kBlockM) * p.n_tiles, routed ? x.gemm_ctas : 0,
                               routed ? kSlotDownRouted : kSlotDownShared, s);
}

// d_hidden = d_y @ Wd (B is [E*H, I] read N-major), fused SwiGLU backward
int run_dgrad_down(const mok_layer_common& c, const PassCtx& x, const Dims& d, bool routed, int off, int limit, const void* d_y, int a_rows,
                   const void* wd, const void* gate, const void* up, void* d_hidden, void* d_gate, void* d_up,
                   const float* row_scale, float* partials, cudaStream_t s) {
    GemmParams p = base_params(c, x, routed, off, limit);
    p.n_tiles = d.I / kBlockN;
    p.k_blocks_per_seg = d.H / kBlockK;
    p.b_rows_per_expert = d.H;
    p.out0 = static_cast<__nv_bfloat16*>(d_hidden);
    p.out1 = static_cast<__nv_bfloat16*>(d_gate);
    p.out2 = static_cast<__nv_bfloat16*>(d_up);
    p.in0 = static_cast<const __nv_bfloat16*>(gate);
    p.in1 = static_cast<const __nv_bfloat16*>(up);
    p.ld_out = d.I;
    p.row_scale = row_scale;
    p.partials = partials;
    GemmOperands o{};
    o.a0 = d_y; o.b0 = wd;
    o.a_inner = d.H; o.a_outer = a_rows;
    o.b_inner = d.I; o.b_outer = static_cast<uint64_t>(routed ? d.El : 1) * d.H;
    return launch_grouped_gemm(kMajorK, kMajorMN, kEpiSwigluBwd, false, o, p, (limit / kBlockM) * p.n_tiles, routed ? x.gemm_ctas : 0,
                               routed ? kSlotDgradDownRouted : kSlotDgradDownShared, s);
}

// d_x = d_gate @ Wg + d_up @ Wu in one accumulator (B = [E*I, H] read N-major)
int run_dgrad_gate_up(const mok_layer_common& c, const PassCtx& x, const Dims& d, bool routed, int off, int limit, const void* d_gate,
                      const void* d_up, int a_rows, const void* wg, const void* wu, void* d_x, cudaStream_t s) {
    GemmParams p = base_params(c, x, routed, off, limit);
    p.n_tiles = d.H / kBlockN;
    p.k_blocks_per_seg = d.I / kBlockK;
    p.num_segs = 2;
    p.b_rows_per_expert = d.I;
    p.out0 = static_cast<__nv_bfloat16*>(d_x);
    p.ld_out = d.H;
    GemmOperands o{};
    o.a0 = d_gate; o.a1 = d_up; o.b0 = wg; o.b1 = wu;
    o.a_inner = d.I; o.a_outer = a_rows;
    o.b_inner = d.H; o.b_outer = static_cast<uint64_t>(routed ? d.El : 1) * d.I;
    return launch_grouped_gemm(kMajorK, kMajorMN, kEpiStore, false, o, p, (limit / kBlockM) * p.n_tiles, routed ? x.gemm_ctas : 0,
                               routed ? kSlotDgradGateUpRouted : kSlotDgradGateUpShared, s);
}

// dW[e] [m, n] = A[rows_e, m]^T @ B[rows_e, n]; both operands are read MN-major straight from the
// row-major activations
int run_wgrad(const mok_layer_common& c, const PassCtx& x, bool routed, int off, int limit, const void* a, int m, const void* b, int n,
              int rows, void* dw, int accumulate, cudaStream_t s) {
    GemmParams p = base_params(c, x, routed, off, limit);
    p.m_tiles_w = m / kBlockM;
    p.n_tiles = n / kBlockN;
    p.out0 = static_cast<__nv_bfloat16*>(dw);
    p.ld_out = n;
    p.out_expert_stride = static_cast<long long>(m) * n;
    p.accumulate = accumulate;
    GemmOperands o{};
    o.a0 = a; o.b0 = b;
    o.a_inner = m; o.a_outer = rows;
    o.b_inner = n; o.b_outer = rows;
    const int experts = routed ? c.num_local_experts : 1;
    return launch_grouped_gemm(kMajorMN, kMajorMN, kEpiStore, true, o, p, experts * p.m_tiles_w * p.n_tiles, 0,
                               routed ? kSlotWgradRouted : kSlotWgradShared, s);
}

RowMoveParams row_move(const mok_layer_common& c, const PassCtx& x, const Dims& d, int off, int limit, void* local) {
    RowMoveParams r{};
    r.local = local;
    r.peer_rank = c.schedule_peer_rank;
    r.peer_token_idx = c.schedule_peer_token_idx;
    r.num_tokens = c.num_tokens;
    r.capacity = d.cap;
    r.row_offset = off;
    r.row_limit = limit;
    r.hidden = d.H;
    r.row_divisor = 1;
    r.status = c.status;
    r.fat_ctas = (x.comm_sms > 0 && x.dedicated) ? 1 : 0;
    r.chunk = x.chunk;
    return r;
}

}  // namespace
}  // namespace mok

// -------------------------------------------------------------------------------------------------
// Two-stream pipeline.  A window is cut into `chunks` row ranges (derived on the device from
// num_tokens, see chunk_range); the row movement of a chunk runs on a side stream while the GEMMs
// of its neighbours run on the caller's stream:
//     side:  load(0) load(1)        store(0) load(2)        store(1) ...
//     main:          compute(0)              compute(1)              ...
// Dependencies are CUDA events only (no kernel waits on another kernel), the side stream forks from
// and joins back into the caller's stream inside the call, and results do not depend on timing.
// `comm_sms` (the reference's fwd/bwd_num_comm_sms) is the SM budget of the row movement while a chunked window runs.
// Shared form (default): the movers are thin bulk-copy CTAs, sixteen per budgeted SM, that sit beside the persistent
// GEMM CTAs (24 KB of shared memory and three warps fit next to one) and fill an SM whenever no GEMM CTA holds it, so
// the GEMMs keep every SM and the budget sets how many copy pipelines exist (the reference's defaults, 40 and 28 SMs,
// give 640 and 448 mover CTAs; measured on two B200s the step gets shorter up to about 600 CTAs and stays flat beyond).
// Dedicated form (MOK_B200_DEDICATED_COMM_SMS=1): that many SMs run fat mover CTAs of their own and the routed GEMM
// grids shrink by the same number, as in the reference's megakernel.  Measured on two B200s the shared form is 5-6 %
// faster than the best dedicated split, which is why it is the default.
// With MOK_B200_OVERLAP_SHARED=1 even an unchunked window puts its load on the side stream, so that it runs beside
// whatever the caller's stream holds since the last fork (the dense shared expert).  Off by default: measured on one
// B200 the two kernels slow each other down by what the overlap saves (step within 1 % either way).
// -------------------------------------------------------------------------------------------------
namespace mok {
namespace {

// Side streams and events are pooled per device and lent to one call at a time, so two host threads
// driving the same device never record or wait on each other's events.
struct DevicePool {
    std::vector<cudaStream_t> streams;
    std::vector<cudaEvent_t> events;
};
DevicePool g_pool[64];
std::mutex g_pool_mu;

int env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : fallback;
}

// MOK_B200_COMM_SMS: -1 / unset = take the budget from the call's num_comm_sms; 0 = no budget (four thin mover CTAs
// per SM of the GPU whatever the call says); n > 0 = n SMs whatever the call says
int comm_sm_override() {
    static const int configured = env_int("MOK_B200_COMM_SMS", -1);
    return configured;
}
bool dedicated_comm_sms() {
    static const bool on = env_int("MOK_B200_DEDICATED_COMM_SMS", 0) != 0;
    return on;
}
// Later windows hold rows only when the schedule exceeds one macrobatch (skewed routing: the busiest rank).  Cutting
// them into chunks as well lets their row movement overlap their GEMMs, at the price of a few empty launches on the
// ranks whose later windows are empty.  Measured on two B200s with Zipf(1.2) routing: BF16 passes 3 % faster, MXFP8
// passes no faster (their quantising dispatch cannot run beside a GEMM CTA), so the default is BF16 only;
// MOK_B200_CHUNK_ALL_WINDOWS=1 / 0 forces it on / off for both.
bool chunk_all_windows(bool mxfp8) {
    static const int configured = env_int("MOK_B200_CHUNK_ALL_WINDOWS", -1);
    return configured < 0 ? !mxfp8 : configured != 0;
}
// MOK_B200_LEAN_QUANT=1 gives the quantising dispatch of the MXFP8 passes its lean shape (64 threads, 17 KB), the one that
// fits beside an MXFP8 GEMM CTA.  Off by default: measured on two B200s (H=7168, 256 experts, top-8) the step is 3.5 %
// longer with it (35.0 against 33.8 ms) - the 256-thread shape, which runs whenever GEMM CTAs leave an SM, moves the
// rows faster than one lean CTA per SM gains by running beside them.
bool lean_quant(const PassCtx&) {
    static const bool on = env_int("MOK_B200_LEAN_QUANT", 0) > 0;
    return on;
}
bool overlap_shared_expert() {
    static const bool on = env_int("MOK_B200_OVERLAP_SHARED", 0) != 0;
    return on;
}

class Pipeline {
public:
    Pipeline(cudaStream_t main, int chunks, int min_rows, int comm_sms)
        : main_(main), chunks_(chunks), min_rows_(min_rows), comm_sms_(comm_sms) {
        if (cudaGetDevice(&dev_) != cudaSuccess || dev_ < 0 || dev_ >= 64) {
            note_error_text("cudaGetDevice failed or device index >= 64");
            rc_ = MOK_ERR_CUDA;
            return;
        }
        use_side_ = chunks_ > 1 || overlap_shared_expert();
        if (!use_side_) return;
        std::lock_guard<std::mutex> lock(g_pool_mu);
        DevicePool& pool = g_pool[dev_];
        if (!pool.streams.empty()) { side_ = pool.streams.back(); pool.streams.pop_back(); return; }
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        if (cudaStreamCreateWithPriority(&side_, cudaStreamNonBlocking, hi) != cudaSuccess) { side_ = nullptr; rc_ = MOK_ERR_CUDA; }
    }
    // Every exit path of a layer call ends here: the side stream is joined back into the caller's stream
    // (an open stream capture stays well-formed after an error) and the borrowed objects return to the pool.
    ~Pipeline() {
        if (side_ && forked_) order(side_, main_);
        std::lock_guard<std::mutex> lock(g_pool_mu);
        DevicePool& pool = g_pool[dev_ >= 0 && dev_ < 64 ? dev_ : 0];
        if (side_) pool.streams.push_back(side_);
        for (cudaEvent_t e : held_) pool.events.push_back(e);
    }
    Pipeline(const Pipeline&) = delete;
    Pipeline& operator=(const Pipeline&) = delete;
    int error() const { return rc_; }

    // side stream continues after everything enqueued on main so far / main after side
    int fork() { if (!use_side_) return MOK_OK; forked_ = true; return order(main_, side_); }
    int join() { if (!use_side_ || !forked_) return MOK_OK; forked_ = false; return order(side_, main_); }

    // load(stream, ctx) and store(stream, ctx) go to the side stream, compute(stream, ctx) to the caller's.
    template <class Load, class Compute, class Store>
    int run(bool chunked, Load load, Compute compute, Store store) {
        if (rc_ != MOK_OK) return rc_;
        int rc = MOK_OK;
        if (chunks_ <= 1 || !chunked) {
            PassCtx x;
            if (use_side_ && forked_) {
                if ((rc = load(side_, x))) return rc;
                if ((rc = join())) return rc;
            } else if ((rc = load(main_, x))) {
                return rc;
            }
            if ((rc = compute(main_, x))) return rc;
            return store(main_, x);
        }
        if (!forked_ && (rc = fork())) return rc;
        std::vector<cudaEvent_t> loaded(chunks_);
        if ((rc = load(side_, ctx(0)))) return rc;
        if ((rc = record(side_, loaded[0]))) return rc;
        for (int c = 0; c < chunks_; ++c) {
            if (c + 1 < chunks_) {
                if ((rc = load(side_, ctx(c + 1)))) return rc;
                if ((rc = record(side_, loaded[c + 1]))) return rc;
            }
            if (cudaStreamWaitEvent(main_, loaded[c], 0) != cudaSuccess) return MOK_ERR_CUDA;
            if ((rc = compute(main_, ctx(c)))) return rc;
            cudaEvent_t computed;
            if ((rc = record(main_, computed))) return rc;
            if (cudaStreamWaitEvent(side_, computed, 0) != cudaSuccess) return MOK_ERR_CUDA;
            if ((rc = store(side_, ctx(c)))) return rc;
        }
        return MOK_OK;
    }

private:
    PassCtx ctx(int c) const {
        PassCtx x;
        x.chunk = ChunkSpec{c, chunks_, min_rows_};
        if (comm_sms_ > 0) {
            x.comm_sms = comm_sms_;
            x.dedicated = dedicated_comm_sms();
            if (x.dedicated) x.gemm_ctas = device_sm_count() - comm_sms_;
        }
        return x;
    }
    int record(cudaStream_t s, cudaEvent_t& out) {
        {
            std::lock_guard<std::mutex> lock(g_pool_mu);
            DevicePool& pool = g_pool[dev_];
            if (!pool.events.empty()) { out = pool.events.back(); pool.events.pop_back(); }
            else if (cudaEventCreateWithFlags(&out, cudaEventDisableTiming) != cudaSuccess) return MOK_ERR_CUDA;
        }
        held_.push_back(out);
        return cudaEventRecord(out, s) == cudaSuccess ? MOK_OK : MOK_ERR_CUDA;
    }
    int order(cudaStream_t first, cudaStream_t then) {
        cudaEvent_t e;
        int rc = record(first, e);
        if (rc) return rc;
        return cudaStreamWaitEvent(then, e, 0) == cudaSuccess ? MOK_OK : MOK_ERR_CUDA;
    }
    cudaStream_t main_;
    cudaStream_t side_ = nullptr;
    int chunks_, min_rows_, comm_sms_;
    int dev_ = -1;
    bool use_side_ = false, forked_ = false;
    std::vector<cudaEvent_t> held_;
    int rc_ = MOK_OK;
};

// CTAs of a row-movement launch: sixteen thin CTAs per budgeted SM beside the GEMM CTAs, or one fat CTA per dedicated
// SM; without a budget (one rank, or a window moved in one piece) four thin CTAs per SM of the GPU
// (MOK_B200_COMM_BLOCKS overrides that default)
constexpr int kThinCtasPerBudgetedSm = 16;
int move_grid(const PassCtx& x) {
    if (x.comm_sms > 0) return x.dedicated ? x.comm_sms : kThinCtasPerBudgetedSm * x.comm_sms;
    static const int configured = env_int("MOK_B200_COMM_BLOCKS", 0);
    return configured > 0 ? configured : device_sm_count() * 4;
}

// the quantising dispatch is arithmetic-heavy and its CTAs are small (33 KB of shared memory, 256 threads): six of
// them fill a dedicated SM; in the shared form they take whatever SMs the GEMM launches leave free
int quant_grid(const PassCtx& x) {
    if (x.comm_sms > 0) return x.dedicated ? x.comm_sms * 6 : std::max(kThinCtasPerBudgetedSm * x.comm_sms, 2 * device_sm_count());
    return move_grid(x);
}

int pipeline_chunks(const mok_layer_common& c, int limit) {
    static const int configured = [] { const int v = env_int("MOK_B200_CHUNKS", 0); return v < 0 ? 0 : (v > 32 ? 32 : v); }();
    // default: no chunking on a single rank (movement and GEMMs compete for HBM there), four chunks
    // when rows cross NVLink (measured at 2 and 8 ranks: 2, 4, 8 and 16 chunks are within 4 % of each
    // other, 4 the shortest)
    const int want = configured > 0 ? configured : (c.ep_size > 1 ? 4 : 1);
    const int by_minibatch = limit / c.minibatch_size;
    return std::max(1, std::min(want, by_minibatch));
}

// SM budget of the row movers of this call: the caller's num_comm_sms when rows cross NVLink and the window is
// processed in chunks, unless the environment overrides it; dedicated SMs are capped at half of the GPU
int pipeline_comm_sms(const mok_layer_common& c, int chunks) {
    if (chunks <= 1) return 0;
    const int forced = comm_sm_override();
    int n = forced >= 0 ? forced : (c.ep_size > 1 ? c.num_comm_sms : 0);
    n = std::max(0, std::min(n, dedicated_comm_sms() ? device_sm_count() / 2 : device_sm_count()));
    return n & ~1;
}

}  // namespace
}  // namespace mok

using namespace mok;

extern "C" int mok_fwd_bf16(const mok_fwd_bf16_args* a, void* stream) {
    if (!a) return MOK_ERR_INVALID;
    Dims d;
    MOK_TRY(check_common(a->c, d));
    const mok_layer_common& c = a->c;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PeerPtrs x_peers{}, combine_peers{};
    MOK_TRY(fill_peers(x_peers, a->x_ptrs, d.W));
    MOK_TRY(fill_peers(combine_peers, a->combine_buffer_ptrs, d.W));
    const void* x_local = x_peers.p[d.rank];
    const int chunks = pipeline_chunks(c, std::min(d.MB, d.cap));
    Pipeline pipe(s, chunks, c.minibatch_size, pipeline_comm_sms(c, chunks));
    const PassCtx whole;       // launches outside the chunked pipeline cover their whole window on all SMs
    MOK_TRY(pipe.error());
    MOK_TRY(pipe.fork());

    // shared expert on the local tokens: its gate|up GEMM runs beside the first dispatch; its down projection beside
    // the first dispatch too when the window is moved in one piece, beside the last combine chunk when it is chunked
    MOK_TRY(run_gate_up(c, whole, d, false, 0, d.T, x_local, d.T, a->w_shared_gate, a->w_shared_up, a->gate_shared, a->up_shared,
                        a->hidden_shared, s));
    const bool shared_down_last = chunks > 1;
    if (!shared_down_last) MOK_TRY(run_down(c, whole, d, false, 0, d.T, a->hidden_shared, d.T, a->w_shared_down, a->y_shared, s));

    const int n_macro = (d.cap + d.MB - 1) / d.MB;
    for (int m = n_macro - 1; m >= 0; --m) {
        const int off = m * d.MB;
        const int limit = std::min(d.MB, d.cap - off);
        MOK_TRY(pipe.run(m == 0 || chunk_all_windows(false),
            [&](cudaStream_t st, const PassCtx& x) {
                RowMoveParams disp = row_move(c, x, d, off, limit, a->x_routed);
                disp.peers = x_peers;
                disp.row_divisor = d.K;
                return launch_dispatch_rows(disp, false, move_grid(x), st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                MOK_TRY(run_gate_up(c, x, d, true, off, limit, a->x_routed, d.MB, a->w_routed_gate, a->w_routed_up,
                                    a->gate_routed, a->up_routed, a->hidden_routed, st));
                return run_down(c, x, d, true, off, limit, a->hidden_routed, d.MB, a->w_routed_down, a->y_routed, st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                if (c.defer_combine) return static_cast<int>(MOK_OK);   // mok_fwd_epilogue_rows reads y_routed in place
                RowMoveParams comb = row_move(c, x, d, off, limit, a->y_routed);
                comb.peers = combine_peers;
                return launch_combine_rows(comb, move_grid(x), st);
            }));
        if (m == 0 && shared_down_last)
            MOK_TRY(run_down(c, whole, d, false, 0, d.T, a->hidden_shared, d.T, a->w_shared_down, a->y_shared, s));
        MOK_TRY(pipe.join());      // the next window reuses the buffers
        if (m > 0) MOK_TRY(pipe.fork());
    }
    return MOK_OK;
}

extern "C" int mok_bwd_bf16(const mok_bwd_bf16_args* a, void* stream) {
    if (!a) return MOK_ERR_INVALID;
    Dims d;
    MOK_TRY(check_common(a->c, d));
    const mok_layer_common& c = a->c;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PeerPtrs dy_peers{}, dxr_peers{}, rw_peers{}, drw_peers{}, x_peers{};
    MOK_TRY(fill_peers(dy_peers, a->d_y_ptrs, d.W));
    MOK_TRY(fill_peers(dxr_peers, a->d_x_routed_buffer_ptrs, d.W));
    MOK_TRY(fill_peers(rw_peers, a->router_weight_ptrs, d.W));
    MOK_TRY(fill_peers(drw_peers, a->d_router_weight_ptrs, d.W));
    MOK_TRY(fill_peers(x_peers, a->x_ptrs, d.W));
    if (!a->router_weights_routed || !a->d_router_weight_partials) return MOK_ERR_INVALID;
    const void* dy_local = dy_peers.p[d.rank];
    const void* x_local = x_peers.p[d.rank];
    const int partial_cols = d.I / kBlockN * kEpiSplit;
    const int chunks = pipeline_chunks(c, std::min(d.MB, d.cap));
    Pipeline pipe(s, chunks, c.minibatch_size, pipeline_comm_sms(c, chunks));
    const PassCtx whole;       // launches outside the chunked pipeline cover their whole window on all SMs
    MOK_TRY(pipe.error());
    MOK_TRY(pipe.fork());

    // shared expert (overlaps the first reverse-combine chunk)
    MOK_TRY(run_dgrad_down(c, whole, d, false, 0, d.T, dy_local, d.T, a->w_shared_down, a->gate_shared, a->up_shared,
                           a->d_hidden_shared, a->d_gate_shared, a->d_up_shared, nullptr, nullptr, s));
    MOK_TRY(run_dgrad_gate_up(c, whole, d, false, 0, d.T, a->d_gate_shared, a->d_up_shared, d.T, a->w_shared_gate, a->w_shared_up,
                              a->d_x_shared, s));
    MOK_TRY(run_wgrad(c, whole, false, 0, d.T, dy_local, d.H, a->hidden_shared, d.I, d.T, a->d_w_shared_down, 0, s));
    MOK_TRY(run_wgrad(c, whole, false, 0, d.T, a->d_gate_shared, d.I, x_local, d.H, d.T, a->d_w_shared_gate, 0, s));
    MOK_TRY(run_wgrad(c, whole, false, 0, d.T, a->d_up_shared, d.I, x_local, d.H, d.T, a->d_w_shared_up, 0, s));

    const int n_macro = (d.cap + d.MB - 1) / d.MB;
    for (int m = 0; m < n_macro; ++m) {
        const int off = m * d.MB;
        const int limit = std::min(d.MB, d.cap - off);
        if (m > 0) {   // replay the forward of this window into the saved-activation buffers
            RowMoveParams disp = row_move(c, whole, d, off, limit, a->x_routed);
            disp.peers = x_peers;
            disp.row_divisor = d.K;
            MOK_TRY(launch_dispatch_rows(disp, false, move_grid(whole), s));
            MOK_TRY(run_gate_up(c, whole, d, true, off, limit, a->x_routed, d.MB, a->w_routed_gate, a->w_routed_up, a->gate_routed,
                                a->up_routed, a->hidden_routed, s));
            MOK_TRY(pipe.fork());
        }
        MOK_TRY(pipe.run(m == 0 || chunk_all_windows(false),
            [&](cudaStream_t st, const PassCtx& x) {
                RowMoveParams rc = row_move(c, x, d, off, limit, a->d_y_routed);
                rc.peers = dy_peers;
                rc.scale_peers = rw_peers;
                rc.row_divisor = d.K;
                rc.row_scale_out = a->router_weights_routed;
                return launch_dispatch_rows(rc, true, move_grid(x), st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                MOK_TRY(run_dgrad_down(c, x, d, true, off, limit, a->d_y_routed, d.MB, a->w_routed_down, a->gate_routed,
                                       a->up_routed, a->d_hidden_routed, a->d_gate_routed, a->d_up_routed,
                                       a->router_weights_routed, a->d_router_weight_partials, st));
                return run_dgrad_gate_up(c, x, d, true, off, limit, a->d_gate_routed, a->d_up_routed, d.MB, a->w_routed_gate,
                                         a->w_routed_up, a->d_x_routed, st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                RowMoveParams rd = row_move(c, x, d, off, limit, a->d_x_routed);
                if (c.defer_combine) return static_cast<int>(MOK_OK);   // mok_bwd_epilogue_rows reads the rows in place
                rd.peers = dxr_peers;
                rd.scale_peers = drw_peers;
                rd.partials = a->d_router_weight_partials;
                rd.partial_cols = partial_cols;
                return launch_combine_rows(rd, move_grid(x), st);
            }));
        // the weight gradients read what the loads and the GEMMs of this window produced, all ordered before this
        // point of the caller's stream; the last reverse-dispatch chunk, still running on the side stream, reads
        // d_x_routed and the partials, which they do not touch: they overlap, and the join comes after them
        const int acc = m > 0 ? 1 : 0;
        MOK_TRY(run_wgrad(c, whole, true, off, limit, a->d_y_routed, d.H, a->hidden_routed, d.I, d.MB, a->d_w_routed_down, acc, s));
        MOK_TRY(run_wgrad(c, whole, true, off, limit, a->d_gate_routed, d.I, a->x_routed, d.H, d.MB, a->d_w_routed_gate, acc, s));
        MOK_TRY(run_wgrad(c, whole, true, off, limit, a->d_up_routed, d.I, a->x_routed, d.H, d.MB, a->d_w_routed_up, acc, s));
        MOK_TRY(pipe.join());      // the next window replays into the buffers the stores read
    }
    return MOK_OK;
}

extern "C" int mok_version(void) { return 101; }

extern "C" int mok_query_workspace_bytes(int ep_size, int num_local_tokens, int hidden, int topk, int num_local_experts,
                                         double schedule_capacity_multiplier, mok_workspace_bytes* out) {
    if (!out) return MOK_ERR_INVALID;
    if (ep_size < 1 || ep_size > MOK_MAX_PEERS || num_local_tokens <= 0 || num_local_tokens % 256 || hidden <= 0 || hidden % 256)
        return MOK_ERR_INVALID;
    if (topk < 1 || topk > 255 || num_local_experts < 1 || num_local_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_INVALID;
    if (!(schedule_capacity_multiplier > 0.0) || schedule_capacity_multiplier > 1e6) return MOK_ERR_INVALID;
    const long long routes = static_cast<long long>(num_local_tokens) * topk;
    long long factor = static_cast<long long>(std::ceil(ep_size * schedule_capacity_multiplier));
    if (factor < 2) factor = 2;
    const long long capacity = routes * factor;
    if (capacity > INT32_MAX) return MOK_ERR_TOO_LARGE;
    const size_t T = static_cast<size_t>(num_local_tokens), H = static_cast<size_t>(hidden), R = static_cast<size_t>(routes);
    out->schedule_capacity = capacity;
    out->x_buffer = T * H * 2;
    out->combine_buffer = R * H * 2;
    out->d_y_buffer = T * H * 2;
    out->d_x_routed_buffer = R * H * 2;
    out->router_weight_buffer = R * 4;
    out->d_router_weight_buffer = R * 4;
    out->all_gather_top_experts_buffer = static_cast<size_t>(ep_size) * R * 4;
    out->barrier_buffer = 4;
    out->barrier_target = 4;
    out->status_word = 16;
    out->schedule_tables = static_cast<size_t>(capacity) * 4 * 2 + 4 + static_cast<size_t>(num_local_experts) * 4;
    out->schedule_scratch = mok_schedule_scratch_bytes(ep_size, num_local_experts);
    return MOK_OK;
}

extern "C" int mok_last_status(int32_t* status_device, int32_t* out_host, int clear, void* stream) {
    if (!status_device || !out_host) return MOK_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MOK_CUDA_CHECK(cudaMemcpyAsync(out_host, status_device, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    if (clear) MOK_CUDA_CHECK(cudaMemsetAsync(status_device, 0, 4 * sizeof(int32_t), s));
    MOK_CUDA_CHECK(cudaStreamSynchronize(s));
    return MOK_OK;
}

extern "C" const char* mok_error_string(int code) {
    switch (code) {
        case MOK_OK: return "ok";
        case MOK_ERR_INVALID: return "invalid argument";
        case MOK_ERR_CUDA: return "CUDA call failed";
        case MOK_ERR_UNSUPPORTED: return "unsupported shape or mode";
        case MOK_ERR_TOO_LARGE: return "problem exceeds the fixed size limit of this entry point";
        case MOK_STATUS_SCHEDULE_OVERFLOW: return "schedule capacity exceeded";
        case MOK_STATUS_BARRIER_TIMEOUT: return "device barrier timed out";
        case MOK_STATUS_PIPELINE_TIMEOUT: return "kernel pipeline wait timed out";
        default: return "unknown";
    }
}

// =================================================================================================
// MXFP8 routed experts.  Same launch sequence as the BF16 passes; the routed GEMMs run block-scaled
// on E4M3 data, and every producer writes its output already quantised in the layout(s) its
// consumers contract over: dispatch -> x (normal for gate|up, transposed for the gate/up weight
// gradients); gate|up epilogue -> saved gate/up, hidden (normal for down, transposed for the down
// weight gradient); reverse-combine -> w*d_y (normal + transposed); dgrad-down epilogue -> d_gate,
// d_up (normal + transposed).  The shared expert stays BF16 (as in the reference, ops.py:240-246).
// =================================================================================================
namespace mok {
namespace {

MxGemmParams mx_base(const mok_layer_common& c, const PassCtx& x, int off, int limit) {
    MxGemmParams p{};
    p.chunk = x.chunk;
    p.num_tokens = c.num_tokens;
    p.capacity = c.schedule_capacity;
    p.tokens_per_expert = c.tokens_per_expert;
    p.num_experts = c.num_local_experts;
    p.row_offset = off;
    p.row_limit = limit;
    p.num_segs = 1;
    p.limit = c.swiglu_limit;
    p.has_limit = c.has_swiglu_limit;
    p.status = c.status;
    p.q_cols = c.intermediate;
    p.t_rows = c.macrobatch_size;
    return p;
}
inline uint8_t* u8(void* p) { return static_cast<uint8_t*>(p); }
inline const uint8_t* cu8(const void* p) { return static_cast<const uint8_t*>(p); }

int mx_gate_up(const mok_layer_common& c, const PassCtx& x, const Dims& d, int off, int limit, const void* x_q, const void* x_sc,
               const void* wg_q, const void* wg_sc, const void* wu_q, const void* wu_sc, void* gate_q, void* gate_sc,
               void* up_q, void* up_sc, void* hid_q, void* hid_sc, void* hid_qt, void* hid_sct, cudaStream_t s) {
    MxGemmParams p = mx_base(c, x, off, limit);
    p.n_tiles = d.I / (kBlockN / 2);
    p.k_tiles_per_seg = d.H / kMxBlockK;
    p.b_rows_per_expert = d.I;
    p.sfa0 = cu8(x_sc); p.sfa_k_tiles = d.H / 128;
    p.sfb0 = cu8(wg_sc); p.sfb1 = cu8(wu_sc); p.sfb_k_tiles = d.H / 128;
    p.q[0] = u8(gate_q); p.sc[0] = u8(gate_sc);
    p.q[1] = u8(up_q); p.sc[1] = u8(up_sc);
    p.q[2] = u8(hid_q); p.sc[2] = u8(hid_sc);
    p.qt[2] = u8(hid_qt); p.sct[2] = u8(hid_sct);
    MxGemmOperands o{};
    o.a0 = x_q; o.b0 = wg_q; o.b1 = wu_q;
    o.a_inner = d.H; o.a_outer = d.MB;
    o.b_inner = d.H; o.b_outer = static_cast<uint64_t>(d.El) * d.I;
    return launch_mx_gemm(kMxEpiGateUp, false, o, p, (limit / kBlockM) * p.n_tiles, x.gemm_ctas, kSlotGateUpRouted, s);
}

int mx_down(const mok_layer_common& c, const PassCtx& x, const Dims& d, int off, int limit, const void* hid_q, const void* hid_sc,
            const void* wd_q, const void* wd_sc, void* y, cudaStream_t s) {
    MxGemmParams p = mx_base(c, x, off, limit);
    p.n_tiles = d.H / kBlockN;
    p.k_tiles_per_seg = d.I / kMxBlockK;
    p.b_rows_per_expert = d.H;
    p.sfa0 = cu8(hid_sc); p.sfa_k_tiles = d.I / 128;
    p.sfb0 = cu8(wd_sc); p.sfb_k_tiles = d.I / 128;
    p.out_bf16 = static_cast<__nv_bfloat16*>(y);
    p.ld_out = d.H;
    MxGemmOperands o{};
    o.a0 = hid_q; o.b0 = wd_q;
    o.a_inner = d.I; o.a_outer = d.MB;
    o.b_inner = d.I; o.b_outer = static_cast<uint64_t>(d.El) * d.H;
    return launch_mx_gemm(kMxEpiStore, false, o, p, (limit / kBlockM) * p.n_tiles, x.gemm_ctas, kSlotDownRouted, s);
}

int mx_wgrad(const mok_layer_common& c, const PassCtx& x, const Dims& d, int off, int limit, const void* a_qt, const void* a_sct, int m,
             const void* b_qt, const void* b_sct, int n, void* dw, int accumulate, cudaStream_t s) {
    MxGemmParams p = mx_base(c, x, off, limit);
    p.m_tiles_w = m / kBlockM;
    p.n_tiles = n / kBlockN;
    p.sfa0 = cu8(a_sct); p.sfa_k_tiles = d.MB / 128;
    p.sfb0 = cu8(b_sct); p.sfb_k_tiles = d.MB / 128;
    p.out_bf16 = static_cast<__nv_bfloat16*>(dw);
    p.ld_out = n;
    p.out_expert_stride = static_cast<long long>(m) * n;
    p.accumulate = accumulate;
    MxGemmOperands o{};
    o.a0 = a_qt; o.b0 = b_qt;
    o.a_inner = d.MB; o.a_outer = m;
    o.b_inner = d.MB; o.b_outer = n;
    return launch_mx_gemm(kMxEpiStore, true, o, p, d.El * p.m_tiles_w * p.n_tiles, 0, kSlotWgradRouted, s);
}

}  // namespace
}  // namespace mok

extern "C" int mok_fwd_mxfp8(const mok_fwd_mxfp8_args* a, void* stream) {
    if (!a) return MOK_ERR_INVALID;
    Dims d;
    MOK_TRY(check_common(a->c, d));
    const mok_layer_common& c = a->c;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PeerPtrs x_peers{}, combine_peers{};
    MOK_TRY(fill_peers(x_peers, a->x_ptrs, d.W));
    MOK_TRY(fill_peers(combine_peers, a->combine_buffer_ptrs, d.W));
    const void* x_local = x_peers.p[d.rank];
    const int chunks = pipeline_chunks(c, std::min(d.MB, d.cap));
    Pipeline pipe(s, chunks, c.minibatch_size, pipeline_comm_sms(c, chunks));
    const PassCtx whole;       // launches outside the chunked pipeline cover their whole window on all SMs
    MOK_TRY(pipe.error());
    MOK_TRY(pipe.fork());

    MOK_TRY(run_gate_up(c, whole, d, false, 0, d.T, x_local, d.T, a->w_shared_gate, a->w_shared_up, a->gate_shared, a->up_shared,
                        a->hidden_shared, s));
    const bool shared_down_last = chunks > 1;      // as in mok_fwd_bf16
    if (!shared_down_last) MOK_TRY(run_down(c, whole, d, false, 0, d.T, a->hidden_shared, d.T, a->w_shared_down, a->y_shared, s));

    const int n_macro = (d.cap + d.MB - 1) / d.MB;
    for (int m = n_macro - 1; m >= 0; --m) {
        const int off = m * d.MB;
        const int limit = std::min(d.MB, d.cap - off);
        MOK_TRY(pipe.run(m == 0 || chunk_all_windows(true),
            [&](cudaStream_t st, const PassCtx& x) {
                RowMoveParams disp = row_move(c, x, d, off, limit, nullptr);
                disp.peers = x_peers;
                disp.row_divisor = d.K;
                QuantOut xo{u8(a->work_x_q), u8(a->work_x_sc), u8(a->x_qt), u8(a->x_sct), d.MB};
                disp.lean = lean_quant(x) ? 1 : 0;
                return launch_dispatch_quant(disp, xo, false, quant_grid(x), st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                MOK_TRY(mx_gate_up(c, x, d, off, limit, a->work_x_q, a->work_x_sc, a->w_routed_gate_q, a->w_routed_gate_sc,
                                   a->w_routed_up_q, a->w_routed_up_sc, a->gate_q, a->gate_sc, a->up_q, a->up_sc,
                                   a->work_hidden_q, a->work_hidden_sc, a->hidden_qt, a->hidden_sct, st));
                return mx_down(c, x, d, off, limit, a->work_hidden_q, a->work_hidden_sc, a->w_routed_down_q,
                               a->w_routed_down_sc, a->y_routed, st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                if (c.defer_combine) return static_cast<int>(MOK_OK);   // mok_fwd_epilogue_rows reads y_routed in place
                RowMoveParams comb = row_move(c, x, d, off, limit, a->y_routed);
                comb.peers = combine_peers;
                comb.lean = 1;
                return launch_combine_rows(comb, move_grid(x), st);
            }));
        if (m == 0 && shared_down_last)
            MOK_TRY(run_down(c, whole, d, false, 0, d.T, a->hidden_shared, d.T, a->w_shared_down, a->y_shared, s));
        MOK_TRY(pipe.join());
        if (m > 0) MOK_TRY(pipe.fork());
    }
    return MOK_OK;
}

extern "C" int mok_bwd_mxfp8(const mok_bwd_mxfp8_args* a, void* stream) {
    if (!a) return MOK_ERR_INVALID;
    Dims d;
    MOK_TRY(check_common(a->c, d));
    const mok_layer_common& c = a->c;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    PeerPtrs dy_peers{}, dxr_peers{}, rw_peers{}, drw_peers{}, x_peers{};
    MOK_TRY(fill_peers(dy_peers, a->d_y_ptrs, d.W));
    MOK_TRY(fill_peers(dxr_peers, a->d_x_routed_buffer_ptrs, d.W));
    MOK_TRY(fill_peers(rw_peers, a->router_weight_ptrs, d.W));
    MOK_TRY(fill_peers(drw_peers, a->d_router_weight_ptrs, d.W));
    MOK_TRY(fill_peers(x_peers, a->x_ptrs, d.W));
    if (!a->router_weights_routed || !a->d_router_weight_partials) return MOK_ERR_INVALID;
    const void* dy_local = dy_peers.p[d.rank];
    const void* x_local = x_peers.p[d.rank];
    const int partial_cols = d.I / kBlockN;
    const int chunks = pipeline_chunks(c, std::min(d.MB, d.cap));
    Pipeline pipe(s, chunks, c.minibatch_size, pipeline_comm_sms(c, chunks));
    const PassCtx whole;       // launches outside the chunked pipeline cover their whole window on all SMs
    MOK_TRY(pipe.error());
    MOK_TRY(pipe.fork());

    // shared expert, BF16
    MOK_TRY(run_dgrad_down(c, whole, d, false, 0, d.T, dy_local, d.T, a->w_shared_down, a->gate_shared, a->up_shared,
                           a->d_hidden_shared, a->d_gate_shared, a->d_up_shared, nullptr, nullptr, s));
    MOK_TRY(run_dgrad_gate_up(c, whole, d, false, 0, d.T, a->d_gate_shared, a->d_up_shared, d.T, a->w_shared_gate, a->w_shared_up,
                              a->d_x_shared, s));
    MOK_TRY(run_wgrad(c, whole, false, 0, d.T, dy_local, d.H, a->hidden_shared, d.I, d.T, a->d_w_shared_down, 0, s));
    MOK_TRY(run_wgrad(c, whole, false, 0, d.T, a->d_gate_shared, d.I, x_local, d.H, d.T, a->d_w_shared_gate, 0, s));
    MOK_TRY(run_wgrad(c, whole, false, 0, d.T, a->d_up_shared, d.I, x_local, d.H, d.T, a->d_w_shared_up, 0, s));

    const int n_macro = (d.cap + d.MB - 1) / d.MB;
    for (int m = 0; m < n_macro; ++m) {
        const int off = m * d.MB;
        const int limit = std::min(d.MB, d.cap - off);
        if (m > 0) {   // replay dispatch + gate|up of this window into the saved-activation buffers
            RowMoveParams disp = row_move(c, whole, d, off, limit, nullptr);
            disp.peers = x_peers;
            disp.row_divisor = d.K;
            QuantOut xo{u8(a->work_x_q), u8(a->work_x_sc), u8(a->x_qt), u8(a->x_sct), d.MB};
            disp.lean = lean_quant(whole) ? 1 : 0;
            MOK_TRY(launch_dispatch_quant(disp, xo, false, quant_grid(whole), s));
            MOK_TRY(mx_gate_up(c, whole, d, off, limit, a->work_x_q, a->work_x_sc, a->w_routed_gate_q, a->w_routed_gate_sc,
                               a->w_routed_up_q, a->w_routed_up_sc, a->gate_q, a->gate_sc, a->up_q, a->up_sc,
                               a->work_hidden_q, a->work_hidden_sc, a->hidden_qt, a->hidden_sct, s));
            MOK_TRY(pipe.fork());
        }
        MOK_TRY(pipe.run(m == 0 || chunk_all_windows(true),
            [&](cudaStream_t st, const PassCtx& x) {     // reverse-combine: w * d_y, quantised in both layouts
                RowMoveParams rc = row_move(c, x, d, off, limit, nullptr);
                rc.peers = dy_peers;
                rc.scale_peers = rw_peers;
                rc.row_divisor = d.K;
                rc.row_scale_out = a->router_weights_routed;
                QuantOut dyo{u8(a->d_y_q), u8(a->d_y_sc), u8(a->work_d_y_qt), u8(a->work_d_y_sct), d.MB};
                rc.lean = lean_quant(x) ? 1 : 0;
                return launch_dispatch_quant(rc, dyo, true, quant_grid(x), st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                {   // d_hidden = d_y @ Wd (weights pre-transposed to [El, I, H]) + SwiGLU backward
                    MxGemmParams p = mx_base(c, x, off, limit);
                    p.n_tiles = d.I / kBlockN;
                    p.k_tiles_per_seg = d.H / kMxBlockK;
                    p.b_rows_per_expert = d.I;
                    p.sfa0 = cu8(a->d_y_sc); p.sfa_k_tiles = d.H / 128;
                    p.sfb0 = cu8(a->w_routed_down_T_sc); p.sfb_k_tiles = d.H / 128;
                    p.out_bf16 = static_cast<__nv_bfloat16*>(a->d_hidden_routed);
                    p.ld_out = d.I;
                    p.in_q[0] = cu8(a->gate_q); p.in_sc[0] = cu8(a->gate_sc);
                    p.in_q[1] = cu8(a->up_q); p.in_sc[1] = cu8(a->up_sc);
                    p.q[0] = u8(a->d_gate_q); p.sc[0] = u8(a->d_gate_sc);
                    p.q[1] = u8(a->d_up_q); p.sc[1] = u8(a->d_up_sc);
                    p.qt[0] = u8(a->work_d_gate_qt); p.sct[0] = u8(a->work_d_gate_sct);
                    p.qt[1] = u8(a->work_d_up_qt); p.sct[1] = u8(a->work_d_up_sct);
                    p.row_scale = a->router_weights_routed;
                    p.partials = a->d_router_weight_partials;
                    MxGemmOperands o{};
                    o.a0 = a->d_y_q; o.b0 = a->w_routed_down_T_q;
                    o.a_inner = d.H; o.a_outer = d.MB;
                    o.b_inner = d.H; o.b_outer = static_cast<uint64_t>(d.El) * d.I;
                    MOK_TRY(launch_mx_gemm(kMxEpiDgradDown, false, o, p, (limit / kBlockM) * p.n_tiles, x.gemm_ctas,
                                           kSlotDgradDownRouted, st));
                }
                // d_x = d_gate @ Wg + d_up @ Wu (weights pre-transposed to [El, H, I]) in one accumulator
                MxGemmParams p = mx_base(c, x, off, limit);
                p.n_tiles = d.H / kBlockN;
                p.k_tiles_per_seg = d.I / kMxBlockK;
                p.num_segs = 2;
                p.b_rows_per_expert = d.H;
                p.sfa0 = cu8(a->d_gate_sc); p.sfa1 = cu8(a->d_up_sc); p.sfa_k_tiles = d.I / 128;
                p.sfb0 = cu8(a->w_routed_gate_T_sc); p.sfb1 = cu8(a->w_routed_up_T_sc); p.sfb_k_tiles = d.I / 128;
                p.out_bf16 = static_cast<__nv_bfloat16*>(a->d_x_routed);
                p.ld_out = d.H;
                MxGemmOperands o{};
                o.a0 = a->d_gate_q; o.a1 = a->d_up_q; o.b0 = a->w_routed_gate_T_q; o.b1 = a->w_routed_up_T_q;
                o.a_inner = d.I; o.a_outer = d.MB;
                o.b_inner = d.I; o.b_outer = static_cast<uint64_t>(d.El) * d.H;
                return launch_mx_gemm(kMxEpiStore, false, o, p, (limit / kBlockM) * p.n_tiles, x.gemm_ctas, kSlotDgradGateUpRouted, st);
            },
            [&](cudaStream_t st, const PassCtx& x) {
                RowMoveParams rd = row_move(c, x, d, off, limit, a->d_x_routed);
                if (c.defer_combine) return static_cast<int>(MOK_OK);   // mok_bwd_epilogue_rows reads the rows in place
                rd.peers = dxr_peers;
                rd.scale_peers = drw_peers;
                rd.partials = a->d_router_weight_partials;
                rd.partial_cols = 4 * partial_cols   /* the MXFP8 epilogue writes one partial per 64-column slice */;
                rd.lean = 1;
                return launch_combine_rows(rd, move_grid(x), st);
            }));
        const int acc = m > 0 ? 1 : 0;      // weight gradients beside the last reverse-dispatch chunk, as in mok_bwd_bf16
        MOK_TRY(mx_wgrad(c, whole, d, off, limit, a->work_d_y_qt, a->work_d_y_sct, d.H, a->hidden_qt, a->hidden_sct, d.I,
                         a->d_w_routed_down, acc, s));
        MOK_TRY(mx_wgrad(c, whole, d, off, limit, a->work_d_gate_qt, a->work_d_gate_sct, d.I, a->x_qt, a->x_sct, d.H,
                         a->d_w_routed_gate, acc, s));
        MOK_TRY(mx_wgrad(c, whole, d, off, limit, a->work_d_up_qt, a->work_d_up_sct, d.I, a->x_qt, a->x_sct, d.H,
                         a->d_w_routed_up, acc, s));
        MOK_TRY(pipe.join());
    }
    return MOK_OK;
}
