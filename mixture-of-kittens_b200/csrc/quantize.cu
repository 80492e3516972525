// BF16 -> MXFP8 quantiser (E4M3 data, one E8M0 scale per 1x32 block along the contraction
// axis), normal and transposed outputs, scales in the tcgen05 block-scale layout.
// Arithmetic follows csrc/mxfp8.cuh:45-72 of Mixture-of-Kittens bit for bit:
//   scale = max(amax * 0.002232142857f, 1e-12f); e = cvt.rp.satfinite.ue8m0(scale);
//   q = cvt.rn.satfinite.e4m3(x * 2^(127-e)).
// HBM-bound: reads 2 B/element once, writes 1 B/element per requested layout (+1/32 for scales).
#include "mxfp8.cuh"
#include "profile.cuh"

namespace mok {

namespace {

constexpr int kTile = 128;
constexpr int kStride = kTile + 8;   // bf16 elements per shared-memory row (16-byte aligned rows)

template <bool kNormal, bool kTransposed>
__global__ void __launch_bounds__(256) mxfp8_quantize_kernel(const __nv_bfloat16* __restrict__ x, int M, int N,
                                                             uint8_t* __restrict__ q, uint8_t* __restrict__ sc,
                                                             uint8_t* __restrict__ qt, uint8_t* __restrict__ sct) {
    __shared__ __align__(16) __nv_bfloat16 tile[kTile * kStride];
    __shared__ __align__(16) uint8_t s_sc[512];
    __shared__ __align__(16) uint8_t s_sct[512];
    const int tc = blockIdx.x, tr = blockIdx.y, e = blockIdx.z;
    const int tid = threadIdx.x;
    const __nv_bfloat16* src = x + (static_cast<size_t>(e) * M + static_cast<size_t>(tr) * kTile) * N + static_cast<size_t>(tc) * kTile;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int v = tid + i * 256;           // 2048 16-byte vectors
        const int r = v >> 4, c8 = v & 15;
        const uint4 val = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * N + c8 * 8);
        *reinterpret_cast<uint4*>(&tile[r * kStride + c8 * 8]) = val;
    }
    __syncthreads();

    if constexpr (kNormal) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int b = tid + it * 256;      // block id = row * 4 + kblock
            const int r = b >> 2, kb = b & 3;
            uint32_t in[16], out[8], sb;
            const uint4* p = reinterpret_cast<const uint4*>(&tile[r * kStride + kb * 32]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = p[j];
                in[4 * j] = v.x; in[4 * j + 1] = v.y; in[4 * j + 2] = v.z; in[4 * j + 3] = v.w;
            }
            mx_quantize_block(in, out, sb);
            uint8_t* dst = q + (static_cast<size_t>(e) * M + static_cast<size_t>(tr) * kTile + r) * N + static_cast<size_t>(tc) * kTile + kb * 32;
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(out[0], out[1], out[2], out[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(out[4], out[5], out[6], out[7]);
            s_sc[(r & 31) * 16 + (r >> 5) * 4 + kb] = static_cast<uint8_t>(sb);
        }
    }
    if constexpr (kTransposed) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int b = tid + it * 256;      // block id = rowblock * 128 + column
            const int c = b & 127, rb = b >> 7;
            uint32_t in[16], out[8], sb;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint16_t lo = *reinterpret_cast<const uint16_t*>(&tile[(rb * 32 + 2 * j) * kStride + c]);
                const uint16_t hi = *reinterpret_cast<const uint16_t*>(&tile[(rb * 32 + 2 * j + 1) * kStride + c]);
                in[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
            }
            mx_quantize_block(in, out, sb);
            uint8_t* dst = qt + (static_cast<size_t>(e) * N + static_cast<size_t>(tc) * kTile + c) * M + static_cast<size_t>(tr) * kTile + rb * 32;
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(out[0], out[1], out[2], out[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(out[4], out[5], out[6], out[7]);
            s_sct[(c & 31) * 16 + (c >> 5) * 4 + rb] = static_cast<uint8_t>(sb);
        }
    }
    __syncthreads();
    if (tid < 32) {
        if constexpr (kNormal) {
            uint8_t* d = sc + ((static_cast<size_t>(e) * (M / kTile) + tr) * (N / kTile) + tc) * 512;
            reinterpret_cast<uint4*>(d)[tid] = reinterpret_cast<const uint4*>(s_sc)[tid];
        }
    } else if (tid < 64) {
        if constexpr (kTransposed) {
            uint8_t* d = sct + ((static_cast<size_t>(e) * (N / kTile) + tc) * (M / kTile) + tr) * 512;
            reinterpret_cast<uint4*>(d)[tid - 32] = reinterpret_cast<const uint4*>(s_sct)[tid - 32];
        }
    }
}

}  // namespace
}  // namespace mok

extern "C" int mok_mxfp8_quantize(const void* x_bf16, int num_matrices, int rows, int cols,
                                  void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, void* stream) {
    using namespace mok;
    if (!x_bf16 || num_matrices <= 0 || rows <= 0 || cols <= 0 || rows % 128 || cols % 128) return MOK_ERR_INVALID;
    const bool normal = x_fp8 != nullptr, transposed = x_fp8_t != nullptr;
    if (!normal && !transposed) return MOK_ERR_INVALID;
    if ((normal && !x_sc) || (transposed && !x_sc_t)) return MOK_ERR_INVALID;
    if (rows / 128 > 65535 || num_matrices > 65535) return MOK_ERR_UNSUPPORTED;
    const dim3 grid(cols / 128, rows / 128, num_matrices);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto* x = static_cast<const __nv_bfloat16*>(x_bf16);
    auto* q = static_cast<uint8_t*>(x_fp8); auto* sc = static_cast<uint8_t*>(x_sc);
    auto* qt = static_cast<uint8_t*>(x_fp8_t); auto* sct = static_cast<uint8_t*>(x_sc_t);
    ProfScope prof(kSlotQuantize, s);
    if (normal && transposed) mxfp8_quantize_kernel<true, true><<<grid, 256, 0, s>>>(x, rows, cols, q, sc, qt, sct);
    else if (normal) mxfp8_quantize_kernel<true, false><<<grid, 256, 0, s>>>(x, rows, cols, q, sc, qt, sct);
    else mxfp8_quantize_kernel<false, true><<<grid, 256, 0, s>>>(x, rows, cols, q, sc, qt, sct);
    MOK_CUDA_CHECK(cudaGetLastError());
    return MOK_OK;
}
