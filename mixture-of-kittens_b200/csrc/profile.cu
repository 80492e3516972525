#include "profile.cuh"

#include <atomic>
#include <cstdio>
#include <mutex>
#include <vector>

#include "../../include/mok_b200.h"

namespace mok {
namespace {
std::atomic<long long> g_launches{0};
std::atomic<int> g_enabled{0};
std::mutex g_mu;
struct Span { int slot; cudaEvent_t a, b; };
std::vector<Span> g_spans;
std::vector<cudaEvent_t> g_pool;

cudaEvent_t take_event() {
    if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}
}  // namespace

void prof_begin(int slot, cudaStream_t stream, int kernels) {
    g_launches.fetch_add(kernels, std::memory_order_relaxed);
    if (!g_enabled.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_mu);
    Span s{slot, take_event(), take_event()};
    if (s.a) cudaEventRecord(s.a, stream);
    g_spans.push_back(s);
}

void prof_end(int slot, cudaStream_t stream) {
    if (!g_enabled.load(std::memory_order_relaxed)) return;
    std::lock_guard<std::mutex> lock(g_mu);
    for (auto it = g_spans.rbegin(); it != g_spans.rend(); ++it) {
        if (it->slot == slot) { if (it->b) cudaEventRecord(it->b, stream); break; }
    }
}
}  // namespace mok

extern "C" long long mok_launch_count(void) { return mok::g_launches.load(); }

extern "C" int mok_profile_enable(int on) {
    mok::g_enabled.store(on ? 1 : 0);
    return MOK_OK;
}

extern "C" int mok_profile_num_slots(void) { return mok::kNumSlots; }

extern "C" const char* mok_profile_slot_name(int slot) {
    static const char* names[mok::kNumSlots] = {
        "scheduler", "mxfp8_quantize", "all_gather_top_experts", "barrier_all", "epilogue",
        "dispatch_rows", "combine_rows",
        "gemm_gate_up_swiglu_shared", "gemm_down_shared", "gemm_gate_up_swiglu_routed", "gemm_down_routed",
        "gemm_dgrad_down_swiglu_bwd_shared", "gemm_dgrad_gate_up_shared", "gemm_wgrad_shared",
        "gemm_dgrad_down_swiglu_bwd_routed", "gemm_dgrad_gate_up_routed", "gemm_wgrad_routed",
        "gemm_plain", "other"};
    return (slot >= 0 && slot < mok::kNumSlots) ? names[slot] : "?";
}

// Waits for the recorded events, adds the elapsed milliseconds and launch counts per slot into the
// caller's arrays (length mok_profile_num_slots()), and forgets the recorded spans.
extern "C" int mok_profile_collect(double* ms_per_slot, long long* launches_per_slot) {
    using namespace mok;
    std::lock_guard<std::mutex> lock(g_mu);
    int rc = MOK_OK;
    for (auto& s : g_spans) {
        if (s.a && s.b) {
            float ms = 0.f;
            if (cudaEventSynchronize(s.b) == cudaSuccess && cudaEventElapsedTime(&ms, s.a, s.b) == cudaSuccess) {
                if (ms_per_slot) ms_per_slot[s.slot] += ms;
                if (launches_per_slot) launches_per_slot[s.slot] += 1;
            } else {
                rc = MOK_ERR_CUDA;
            }
        }
        if (s.a) g_pool.push_back(s.a);
        if (s.b) g_pool.push_back(s.b);
    }
    g_spans.clear();
    return rc;
}

// ---- description of the last failed CUDA call of the calling host thread -------------------------
namespace mok {
namespace {
thread_local char t_cuda_error[256] = "";
}
void note_cuda_error(cudaError_t err, const char* file, int line) {
    const char* base = file;
    for (const char* c = file; *c; ++c) if (*c == '/') base = c + 1;
    snprintf(t_cuda_error, sizeof(t_cuda_error), "%s (%s) at %s:%d", cudaGetErrorName(err), cudaGetErrorString(err), base, line);
}
void note_error_text(const char* text) { snprintf(t_cuda_error, sizeof(t_cuda_error), "%s", text); }
}  // namespace mok

extern "C" const char* mok_last_cuda_error(void) { return mok::t_cuda_error; }
