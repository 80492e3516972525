// Host side of the MXFP8 block-scaled grouped GEMM: tensor maps, instantiations, test entry point.
#include "mxgemm.cuh"

namespace mok {
namespace {
template <int kEpi, bool kW>
int launch_mx_inst(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1, const CUtensorMap& b1,
                   const MxGemmParams& p, int grid, cudaStream_t stream) {
    auto* kern = mx_gemm_kernel<kEpi, kW>;
    static bool configured[64] = {false};
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, mx_smem_bytes(kEpi)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kern<<<grid, kMxThreads, mx_smem_bytes(kEpi), stream>>>(a0, b0, a1, b1, p);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
}  // namespace

int launch_mx_gemm(int epi, bool wgrad, const MxGemmOperands& ops, const MxGemmParams& p, int max_tiles, int max_ctas,
                   int prof_slot, cudaStream_t stream) {
    if (max_tiles <= 0) return MOK_OK;
    CUtensorMap a0, b0, a1, b1;
    const uint32_t b_box = epi == kMxEpiGateUp ? kBlockN / 2 : kBlockN;
    int rc;
    if ((rc = make_tmap_2d(&a0, ops.a0, ops.a_inner, ops.a_outer, ops.a_inner, kMxBlockK, kBlockM, 1))) return rc;
    if ((rc = make_tmap_2d(&b0, ops.b0, ops.b_inner, ops.b_outer, ops.b_inner, kMxBlockK, b_box, 1))) return rc;
    if ((rc = make_tmap_2d(&a1, ops.a1 ? ops.a1 : ops.a0, ops.a_inner, ops.a_outer, ops.a_inner, kMxBlockK, kBlockM, 1))) return rc;
    if ((rc = make_tmap_2d(&b1, ops.b1 ? ops.b1 : ops.b0, ops.b_inner, ops.b_outer, ops.b_inner, kMxBlockK, b_box, 1))) return rc;
    int ctas = device_sm_count();
    if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
    const int grid = max_tiles < ctas ? max_tiles : ctas;
    ProfScope prof(prof_slot, stream);
    if (!wgrad && epi == kMxEpiStore) return launch_mx_inst<kMxEpiStore, false>(a0, b0, a1, b1, p, grid, stream);
    if (!wgrad && epi == kMxEpiGateUp) return launch_mx_inst<kMxEpiGateUp, false>(a0, b0, a1, b1, p, grid, stream);
    if (!wgrad && epi == kMxEpiDgradDown) return launch_mx_inst<kMxEpiDgradDown, false>(a0, b0, a1, b1, p, grid, stream);
    if (wgrad && epi == kMxEpiStore) return launch_mx_inst<kMxEpiStore, true>(a0, b0, a1, b1, p, grid, stream);
    return MOK_ERR_UNSUPPORTED;
}
}  // namespace mok

extern "C" int mok_gemm_mxfp8(const void* a_fp8, const void* a_sc, const void* b_fp8, const void* b_sc, void* c, int m, int n,
                              int k, int32_t* status, void* stream) {
    using namespace mok;
    if (!a_fp8 || !a_sc || !b_fp8 || !b_sc || !c || m <= 0 || n <= 0 || k <= 0) return MOK_ERR_INVALID;
    if (m % kBlockM || n % kBlockN || k % kMxBlockK) return MOK_ERR_INVALID;
    MxGemmParams p{};
    p.rows_host = m; p.row_limit = m;
    p.num_experts = 1;
    p.n_tiles = n / kBlockN;
    p.k_tiles_per_seg = k / kMxBlockK;
    p.num_segs = 1;
    p.b_rows_per_expert = n;
    p.sfa0 = static_cast<const uint8_t*>(a_sc); p.sfa_k_tiles = k / kMxBlockK;
    p.sfb0 = static_cast<const uint8_t*>(b_sc); p.sfb_k_tiles = k / kMxBlockK;
    p.out_bf16 = static_cast<__nv_bfloat16*>(c);
    p.ld_out = n;
    p.status = status;
    MxGemmOperands o{};
    o.a0 = a_fp8; o.b0 = b_fp8;
    o.a_inner = k; o.a_outer = m; o.b_inner = k; o.b_outer = n;
    return launch_mx_gemm(kMxEpiStore, false, o, p, (m / kBlockM) * (n / kBlockN), 0, kSlotGemmTest,
                          static_cast<cudaStream_t>(stream));
}
