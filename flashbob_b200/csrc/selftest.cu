// Known-answer check of the tensor-core plumbing the attention kernels are built from:
// one 128x64x64 product through every operand path they use.
//   out[0] = A * B^T   A, B staged by TMA; B read K-major   (score-shaped products)
//   out[1] = A * B     B read MN-major from the same tile   (output-shaped products)
//   out[2] = A'* B^T   A' written to swizzled shared memory by threads (derived operands)
//   out[3], out[4] = A * [B; B]^T  one N=128 K-major product over two adjacent B tiles
//   out[5], out[6] = A * [B | B]   one N=128 MN-major product whose second 64 columns come from a
//                                  tile `leading byte offset` away (merged output products)
//   out[7] = A''* B^T  A'' written to tensor memory by threads and read from there (derived
//                      operands that never touch shared memory)
// A is [128, 64], B is [64, 64], both fp16 or both bf16 (kind::f16 needs one format for A and B).
#include "internal.h"
#include "ptx.cuh"
#include "tmap.h"

namespace bob {

enum : int { kSelftestTimedOut = 77 };

struct SelftestMaps {
    CUtensorMap a;
    CUtensorMap b;
};

__global__ void __launch_bounds__(128, 1)
selftest_kernel(const __grid_constant__ SelftestMaps maps, const uint16_t* __restrict__ a_raw,
                uint32_t fmt, float* __restrict__ out, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t tile_a = base;                 // 128 rows x 128 B
    const uint32_t tile_b = base + 16384;         // 64 rows x 128 B
    const uint32_t tile_b2 = base + 16384 + 8192; // second copy of B, directly after the first
    const uint32_t tile_a2 = tile_b2 + 8192;      // 128 rows x 128 B
    const uint32_t bar_load = tile_a2 + 16384;
    const uint32_t bar_mma = bar_load + 8;
    const uint32_t bar_mma2 = bar_load + 16;
    const uint32_t tmem_slot = bar_load + 24;
    uint32_t* tmem_slot_ptr =
        reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    if (tid == 0) {
        mbar_init(bar_load, 1);
        mbar_init(bar_mma, 1);
        mbar_init(bar_mma2, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot_ptr;

    if (tid == 0) {
        mbar_arrive_expect_tx(bar_load, 16384 + 2 * 8192);
        tma_load_4d(tile_a, &maps.a, bar_load, 0, 0, 0, 0);
        tma_load_4d(tile_b, &maps.b, bar_load, 0, 0, 0, 0);
        tma_load_4d(tile_b2, &maps.b, bar_load, 0, 0, 0, 0);
    }
    // Threads restate A into the third tile with the swizzle formula.
    {
        const uint4* src = reinterpret_cast<const uint4*>(a_raw + tid * 64);
        #pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint4 v = src[c];
            st_shared_v4(tile_a2 + sw128_offset(tid, c), v.x, v.y, v.z, v.w);
        }
        fence_proxy_async_smem();
    }
    // ... and into tensor memory columns 448..479: row = lane, two elements per 32-bit column.
    {
        const uint4* src = reinterpret_cast<const uint4*>(a_raw + tid * 64);
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16) + 448;
        #pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 v0 = src[2 * c], v1 = src[2 * c + 1];
            const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            tmem_st8(lane_base + 8 * c, w);
        }
        tmem_wait_st();
        tc_fence_before_sync();
    }
    bool ok = mbar_wait(bar_load, 0);
    __syncthreads();
    if (tid == 0 && ok) {
        tc_fence_after_sync();
        const uint32_t id_k = umma_idesc(fmt, fmt, 64, false);
        const uint32_t id_mn = umma_idesc(fmt, fmt, 64, true);
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            umma_ss(tmem + 0, umma_smem_desc(tile_a + ks * 32), umma_smem_desc(tile_b + ks * 32),
                    id_k, ks > 0);
        }
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            umma_ss(tmem + 64, umma_smem_desc(tile_a + ks * 32),
                    umma_smem_desc(tile_b + ks * 2048), id_mn, ks > 0);
        }
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            umma_ss(tmem + 128, umma_smem_desc(tile_a2 + ks * 32),
                    umma_smem_desc(tile_b + ks * 32), id_k, ks > 0);
        }
        const uint32_t id_k128 = umma_idesc(fmt, fmt, 128, false);
        const uint32_t id_mn128 = umma_idesc(fmt, fmt, 128, true);
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            umma_ss(tmem + 192, umma_smem_desc(tile_a + ks * 32), umma_smem_desc(tile_b + ks * 32),
                    id_k128, ks > 0);
        }
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            umma_ss(tmem + 320, umma_smem_desc(tile_a + ks * 32),
                    umma_smem_desc(tile_b + ks * 2048, tile_b2 - tile_b), id_mn128, ks > 0);
        }
        umma_commit(bar_mma);
    }
    ok = ok && mbar_wait(bar_mma, 0);
    tc_fence_after_sync();
    if (ok) {
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        for (int t = 0; t < 7; ++t) {
            for (int c = 0; c < 64; c += 16) {
                float v[16];
                tmem_ld16(lane_base + t * 64 + c, v);
                tmem_wait_ld();
                #pragma unroll
                for (int i = 0; i < 16; ++i) out[(t * 128 + tid) * 64 + c + i] = v[i];
            }
        }
    } else {
        atomicExch(status, 1);
    }
    // second round: the product with the tensor-memory operand reuses accumulator columns 0..63
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0 && ok) {
        tc_fence_after_sync();
        const uint32_t id_k = umma_idesc(fmt, fmt, 64, false);
        #pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            umma_ts_lo(tmem + 0, tmem + 448 + ks * 8, ((tile_b + ks * 32) >> 4) | 0x10000u, id_k, ks > 0);
        }
        umma_commit(bar_mma2);
    }
    ok = ok && mbar_wait(bar_mma2, 0);
    tc_fence_after_sync();
    if (ok) {
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        for (int c = 0; c < 64; c += 16) {
            float v[16];
            tmem_ld16(lane_base + c, v);
            tmem_wait_ld();
            #pragma unroll
            for (int i = 0; i < 16; ++i) out[(7 * 128 + tid) * 64 + c + i] = v[i];
        }
    } else {
        atomicExch(status, 1);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// A wait that nothing completes: the bounded wait must give up and report, not spin forever.
__global__ void timeout_selftest_kernel(int* __restrict__ status, int* sticky) {
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool done = mbar_wait(b, 0);          // nobody arrives on this barrier
    if (threadIdx.x == 0) {
        atomicExch(status, done ? 0 : kSelftestTimedOut);
        // the same second report the attention kernels make when they give up
        if (!done && sticky) { *reinterpret_cast<volatile int*>(sticky) = kSelftestTimedOut; __threadfence_system(); }
    }
}

}  // namespace bob

extern "C" int bob_sm100_timeout_selftest(int* status, void* stream) {
    if (!status) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) return -3;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return -7;
    bob::timeout_selftest_kernel<<<1, 32, 0, s>>>(status, bob::sticky_word(device, true));
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int bob_sm100_selftest(const void* a, const void* b, int is_bf16, float* out,
                                  int* status, void* stream) {
    using namespace bob;
    if (!a || !b || !out || !status) return -1;
    SelftestMaps maps;
    int rc = make_tile_map(&maps.a, a, is_bf16 != 0, 64, 128, 1, 1, 64, 64 * 128, 64 * 128, 128);
    if (rc) return rc;
    rc = make_tile_map(&maps.b, b, is_bf16 != 0, 64, 64, 1, 1, 64, 64 * 64, 64 * 64, 64);
    if (rc) return rc;
    const int smem = 16384 + 2 * 8192 + 16384 + 64 + 1024;
    auto kernel = selftest_kernel;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess)
        return -2;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) return -3;
    kernel<<<1, 128, smem, s>>>(maps, static_cast<const uint16_t*>(a),
                                is_bf16 ? kFmtBF16 : kFmtF16, out, status);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
