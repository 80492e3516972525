// Host side of the tcgen05 grouped GEMM: tensor-map construction, instantiation table, and the
// plain-GEMM entry point used by the tests.
#include "gemm.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace mok {

namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}
}  // namespace

int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                 uint32_t box_inner, uint32_t box_outer, int elem_bytes) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) { note_error_text("cuTensorMapEncodeTiled is not available from the driver"); return MOK_ERR_CUDA; }
    // The encoder is a driver call and needs a context current on the calling thread.  A thread that has made no
    // context-binding runtime call yet (PyTorch's autograd worker on device 0, served from the caching allocator)
    // has none, so bind the runtime's primary context once per thread.
    static thread_local bool context_bound = false;
    if (!context_bound) { MOK_CUDA_CHECK(cudaFree(nullptr)); context_bound = true; }
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const CUtensorMapSwizzle sw = elem_bytes == 4 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B;
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) return MOK_OK;
    char text[224];
    snprintf(text, sizeof(text), "cuTensorMapEncodeTiled -> %d (base %p, extents %llu x %llu, row stride %llu B, box %u x %u, %d-byte elements)",
             static_cast<int>(r), base, static_cast<unsigned long long>(inner), static_cast<unsigned long long>(outer),
             static_cast<unsigned long long>(row_stride_bytes), box_inner, box_outer, elem_bytes);
    note_error_text(text);
    return MOK_ERR_CUDA;
}

int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

namespace {
template <int kA, int kB, int kEpi, bool kW, bool k2>
int launch_inst(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1, const CUtensorMap& b1, const GemmParams& p,
                int grid, cudaStream_t stream) {
    auto* kern = grouped_gemm_kernel<kA, kB, kEpi, kW, k2>;
    static bool configured[64] = {false};   // per instantiation and device: the attribute is sticky
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (k2) {      // pairs of CTAs on neighbouring SMs: cluster of 2
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid & ~1);
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = kGemmSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        MOK_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, a0, b0, a1, b1, p));
    } else {
        kern<<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(a0, b0, a1, b1, p);
    }
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

}  // namespace

// two-CTA tiles (256 rows per CTA pair) unless MOK_B200_2CTA=0
bool use_pairs() {
    static const bool on = [] { const char* e = std::getenv("MOK_B200_2CTA"); return !(e && e[0] == '0'); }();
    return on;
}

int launch_grouped_gemm(int a_major, int b_major, int epi, bool wgrad, const GemmOperands& ops, const GemmParams& p,
                        int max_tiles, int max_ctas, int prof_slot, cudaStream_t stream) {
    if (max_tiles <= 0) return MOK_OK;
    // the epilogues use 256-bit global accesses: 32-byte aligned tensors and row pitches
    for (const void* ptr : {static_cast<const void*>(p.out0), static_cast<const void*>(p.out1), static_cast<const void*>(p.out2),
                            static_cast<const void*>(p.in0), static_cast<const void*>(p.in1)})
        if (reinterpret_cast<uintptr_t>(ptr) % 32 != 0) return MOK_ERR_INVALID;
    if (p.ld_out % 16 != 0) return MOK_ERR_INVALID;
    CUtensorMap a0, b0, a1, b1;
    // A: K-major box {64 K, 128 rows}; M-major box {64 M, 64 K-rows}
    const uint32_t a_box_outer = a_major == kMajorK ? kBlockM : kBlockK;
    // B: K-major box {64 K, 256 rows} (128 when the tile is split into gate|up halves); N-major box {64 N, 64 K-rows}
    const bool pairs = use_pairs();
    // (a CTA of a pair stages 128 rows of B, so its box is 128 rows too)
    const uint32_t b_box_outer = b_major == kMajorK ? ((epi == kEpiSwigluFwd || pairs) ? kBlockN / 2 : kBlockN) : kBlockK;
    int rc;
    if ((rc = make_tmap_2d(&a0, ops.a0, ops.a_inner, ops.a_outer, ops.a_inner * 2, 64, a_box_outer, 2))) return rc;
    if ((rc = make_tmap_2d(&b0, ops.b0, ops.b_inner, ops.b_outer, ops.b_inner * 2, 64, b_box_outer, 2))) return rc;
    if ((rc = make_tmap_2d(&a1, ops.a1 ? ops.a1 : ops.a0, ops.a_inner, ops.a_outer, ops.a_inner * 2, 64, a_box_outer, 2))) return rc;
    if ((rc = make_tmap_2d(&b1, ops.b1 ? ops.b1 : ops.b0, ops.b_inner, ops.b_outer, ops.b_inner * 2, 64, b_box_outer, 2))) return rc;
    int ctas = device_sm_count();
    if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
    // max_tiles counts 128-row tiles; a pair covers two of them
    const int want = pairs ? ((max_tiles + 1) / 2) * 2 : max_tiles;
    const int grid = want < ctas ? want : (pairs ? (ctas & ~1) : ctas);
    ProfScope prof(prof_slot, stream);
#define MOK_INST(A, B, EPI, W)                                                              \
    (pairs ? launch_inst<A, B, EPI, W, true>(a0, b0, a1, b1, p, grid, stream)              \
           : launch_inst<A, B, EPI, W, false>(a0, b0, a1, b1, p, grid, stream))

    if (!wgrad && a_major == kMajorK && b_major == kMajorK && epi == kEpiStore)
        return MOK_INST(kMajorK, kMajorK, kEpiStore, false);
    if (!wgrad && a_major == kMajorK && b_major == kMajorK && epi == kEpiSwigluFwd)
        return MOK_INST(kMajorK, kMajorK, kEpiSwigluFwd, false);
    if (!wgrad && a_major == kMajorK && b_major == kMajorMN && epi == kEpiStore)
        return MOK_INST(kMajorK, kMajorMN, kEpiStore, false);
    if (!wgrad && a_major == kMajorK && b_major == kMajorMN && epi == kEpiSwigluBwd)
        return MOK_INST(kMajorK, kMajorMN, kEpiSwigluBwd, false);
    if (wgrad && a_major == kMajorMN && b_major == kMajorMN && epi == kEpiStore)
        return MOK_INST(kMajorMN, kMajorMN, kEpiStore, true);
    return MOK_ERR_UNSUPPORTED;
}

}  // namespace mok

extern "C" int mok_gemm_bf16(const void* a, const void* b, void* c, int m, int n, int k, int a_mn_major, int b_mn_major,
                             int32_t* status, void* stream) {
    using namespace mok;
    if (!a || !b || !c || m <= 0 || n <= 0 || k <= 0) return MOK_ERR_INVALID;
    if (m % (2 * kBlockM) || n % kBlockN || k % kBlockK) return MOK_ERR_INVALID;
    GemmParams p{};
    p.num_tokens = nullptr;
    p.capacity = 0;
    p.row_offset = 0;
    p.tokens_per_expert = nullptr;
    p.num_experts = 1;
    p.n_tiles = n / kBlockN;
    p.num_segs = 1;
    p.out0 = static_cast<__nv_bfloat16*>(c);
    p.ld_out = n;
    p.status = status;
    GemmOperands ops{};
    ops.a0 = a; ops.b0 = b;
    const bool wgrad = a_mn_major != 0;
    if (!wgrad) {
        p.rows_host = m; p.row_limit = m;
        p.k_blocks_per_seg = k / kBlockK;
        ops.a_inner = k; ops.a_outer = m;
        if (b_mn_major) { ops.b_inner = n; ops.b_outer = k; p.b_rows_per_expert = k; }
        else { ops.b_inner = k; ops.b_outer = n; p.b_rows_per_expert = n; }
    } else {
        if (!b_mn_major) return MOK_ERR_UNSUPPORTED;
        p.rows_host = k; p.row_limit = k;       // contraction runs over the rows of both operands
        p.m_tiles_w = m / kBlockM;
        p.out_expert_stride = 0;
        ops.a_inner = m; ops.a_outer = k;
        ops.b_inner = n; ops.b_outer = k;
    }
    const int tiles = (m / kBlockM) * (n / kBlockN);
    return launch_grouped_gemm(a_mn_major ? kMajorMN : kMajorK, b_mn_major ? kMajorMN : kMajorK, kEpiStore, wgrad, ops, p,
                               tiles, 0, kSlotGemmTest, static_cast<cudaStream_t>(stream));
}
