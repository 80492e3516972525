// Host side of the MXFP8 block-scaled grouped GEMM: tensor maps, instantiations, test entry point.
#include "mxgemm.cuh"

#include <cstdlib>

namespace mok {
namespace {
template <int kEpi, bool kW, bool k2>
int launch_mx_inst(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1, const CUtensorMap& b1,
                   const MxScaleMaps& sf, const MxGemmParams& p, int grid, cudaStream_t stream) {
    auto* kern = mx_gemm_kernel<kEpi, kW, k2>;
    constexpr int smem = mx_smem_bytes(kEpi, k2);
    static bool configured[64] = {false};
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        // setmaxnreg only redistributes the registers the CTA was launched with: refuse to launch a build whose
        // allocation cannot cover the two role budgets (the growing warps would wait for registers that never come)
        cudaFuncAttributes fa{};
        MOK_CUDA_CHECK(cudaFuncGetAttributes(&fa, kern));
        if (kMxThreads * fa.numRegs < 128 * mx_light_regs(kEpi, k2) + (kMxThreads - 128) * mx_epi_regs(kEpi, k2)) {
            note_error_text("mx_gemm_kernel: register allocation of this build is smaller than its setmaxnreg budgets");
            return MOK_ERR_UNSUPPORTED;
        }
        MOK_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (k2) {      // pairs of CTAs on neighbouring SMs: cluster of 2
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid & ~1);
        cfg.blockDim = dim3(kMxThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        MOK_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, a0, b0, a1, b1, sf, p));
    } else {
        kern<<<grid, kMxThreads, smem, stream>>>(a0, b0, a1, b1, sf, p);
    }
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}

// two-CTA tiles unless MOK_B200_MX_2CTA=0 (or MOK_B200_2CTA=0, which switches both GEMM families)
bool use_mx_pairs() {
    static const bool on = [] { const char* e = std::getenv("MOK_B200_MX_2CTA"); return !(e && e[0] == '0'); }();
    return on && use_pairs();
}
}  // namespace

int launch_mx_gemm(int epi, bool wgrad, const MxGemmOperands& ops, const MxGemmParams& p, int max_tiles, int max_ctas,
                   int prof_slot, cudaStream_t stream, bool allow_pairs) {
    if (max_tiles <= 0) return MOK_OK;
    const bool pairs = allow_pairs && use_mx_pairs();
    CUtensorMap a0, b0, a1, b1;
    MxScaleMaps sf;
    // a CTA of a pair stages 128 of the tile's 256 B rows, so its box is 128 rows (as for the gate|up halves)
    const uint32_t b_box = (epi == kMxEpiGateUp || pairs) ? kBlockN / 2 : kBlockN;
    int rc;
    if ((rc = make_tmap_2d(&a0, ops.a0, ops.a_inner, ops.a_outer, ops.a_inner, kMxBlockK, kBlockM, 1))) return rc;
    if ((rc = make_tmap_2d(&b0, ops.b0, ops.b_inner, ops.b_outer, ops.b_inner, kMxBlockK, b_box, 1))) return rc;
    if ((rc = make_tmap_2d(&a1, ops.a1 ? ops.a1 : ops.a0, ops.a_inner, ops.a_outer, ops.a_inner, kMxBlockK, kBlockM, 1))) return rc;
    if ((rc = make_tmap_2d(&b1, ops.b1 ? ops.b1 : ops.b0, ops.b_inner, ops.b_outer, ops.b_inner, kMxBlockK, b_box, 1))) return rc;
    // scale arrays: one 512-byte tile (128 words) per 128 rows x 128 K
    const uint64_t sfa_tiles = (ops.a_outer / 128) * static_cast<uint64_t>(p.sfa_k_tiles);
    const uint64_t sfb_tiles = (ops.b_outer / 128) * static_cast<uint64_t>(p.sfb_k_tiles);
    if (!p.sfa0 || !p.sfb0) return MOK_ERR_INVALID;
    if ((rc = make_tmap_2d(&sf.sfa0, p.sfa0, 128, sfa_tiles, 512, 128, 1, 4))) return rc;
    if ((rc = make_tmap_2d(&sf.sfa1, p.sfa1 ? p.sfa1 : p.sfa0, 128, sfa_tiles, 512, 128, 1, 4))) return rc;
    if ((rc = make_tmap_2d(&sf.sfb0, p.sfb0, 128, sfb_tiles, 512, 128, 1, 4))) return rc;
    if ((rc = make_tmap_2d(&sf.sfb1, p.sfb1 ? p.sfb1 : p.sfb0, 128, sfb_tiles, 512, 128, 1, 4))) return rc;
    int ctas = device_sm_count();
    if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
    // max_tiles counts 128-row tiles; a pair covers two of them
    const int want = pairs ? ((max_tiles + 1) / 2) * 2 : max_tiles;
    const int grid = want < ctas ? want : (pairs ? (ctas & ~1) : ctas);
    ProfScope prof(prof_slot, stream);
#define MOK_MX_INST(EPI, W)                                                                 \
    (pairs ? launch_mx_inst<EPI, W, true>(a0, b0, a1, b1, sf, p, grid, stream)             \
           : launch_mx_inst<EPI, W, false>(a0, b0, a1, b1, sf, p, grid, stream))
    if (!wgrad && epi == kMxEpiStore) return MOK_MX_INST(kMxEpiStore, false);
    if (!wgrad && epi == kMxEpiGateUp) return MOK_MX_INST(kMxEpiGateUp, false);
    if (!wgrad && epi == kMxEpiDgradDown) return MOK_MX_INST(kMxEpiDgradDown, false);
    if (wgrad && epi == kMxEpiStore) return MOK_MX_INST(kMxEpiStore, true);
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
    // a pair of CTAs covers 256 rows; other row counts run the one-CTA form
    return launch_mx_gemm(kMxEpiStore, false, o, p, (m / kBlockM) * (n / kBlockN), 0, kSlotGemmTest,
                          static_cast<cudaStream_t>(stream), m % (2 * kBlockM) == 0);
}
