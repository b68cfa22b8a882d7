// Host-side construction of TMA tensor maps for [B, H, N, D] tensors with arbitrary
// (16-byte-multiple) batch / head / row strides and unit head-dim stride.
//
// cuTensorMapEncodeTiled is resolved at run time through cudaGetDriverEntryPoint so the
// shared library links against libcudart only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>

namespace bob {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

// Tile box = 64 head-dim elements (one 128-byte swizzle span) x box_rows rows of one head.
// Elements outside the tensor (rows past N, head-dim elements past D) read as zero.
// Returns 0 on success.
inline int make_tile_map(CUtensorMap* map, const void* base, bool is_bf16, int64_t D, int64_t N,
                         int64_t H, int64_t B, int64_t stride_n, int64_t stride_h,
                         int64_t stride_b, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return -100;
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return -101;
    // A dimension of extent 1 never advances; give it a harmless, well-formed stride.
    if (H == 1) stride_h = stride_n * N;
    if (B == 1) stride_b = stride_h * H;
    if (N == 1) stride_n = D < 8 ? 8 : D;
    if ((stride_n * 2) % 16 || (stride_h * 2) % 16 || (stride_b * 2) % 16) return -102;
    if (stride_n <= 0 || stride_h <= 0 || stride_b <= 0) return -102;
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)stride_n * 2, (cuuint64_t)stride_h * 2,
                             (cuuint64_t)stride_b * 2};
    cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -(1000 + (int)r);
}

}  // namespace bob
