// Second backward for callers that cannot provide scratch memory.
//
// bob_sm100_bwd2 needs a small workspace (a status word plus the two fp32 row statistics the
// row-owned kernel hands to the column-owned kernel).  Some hosts have nowhere to get one: code
// running inside a framework's memory-planning phase, a real-time loop that forbids allocator
// calls after start-up, an embedding runtime that owns every byte of device memory and exposes no
// allocator to plug-ins.  For them the workspace lives here, in a fixed array that is part of the
// loaded module: every GPU that loads this library holds kNoAllocScratchBytes (8 MiB + 256 B)
// until the process exits, whether or not this entry point is ever called.
//
// The array is shared by all calls and keeps the previous call's contents.  The status word is
// cleared by each call; the statistics are fully rewritten by the row-owned kernel before the
// column-owned kernel reads them, so nothing else needs clearing.  Two calls whose kernels overlap
// on the GPU (different streams, or different host threads) race on the array: serialise them.
#include "../../include/bob_sm100.h"

#include <cuda_runtime.h>
#include <mutex>

namespace {

constexpr size_t kStatusBlock = 256;
constexpr size_t kMaxRows = size_t(1) << 20;                       // B * Hq * Nq
constexpr size_t kNoAllocScratchBytes = kStatusBlock + 2 * kMaxRows * sizeof(float);

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_addr[kMaxDevices] = {};                            // per device, filled on first use

// Device address of the scratch array on `device`.  The first call for a device resolves the
// symbol with that device current; later calls return the cached address.
int scratch_address(int device, void** out) {
    if (device < 0 || device >= kMaxDevices) return -7;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_addr[device]) {
        int prev = -1;
        if (cudaGetDevice(&prev) != cudaSuccess) return -7;
        if (prev != device && cudaSetDevice(device) != cudaSuccess) return -7;
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_scratch);
        if (prev != device) cudaSetDevice(prev);
        if (err != cudaSuccess || !ptr) return -11;
        g_scratch_addr[device] = ptr;
    }
    *out = g_scratch_addr[device];
    return 0;
}

}  // namespace

extern "C" size_t bob_sm100_noalloc_max_rows(void) { return kMaxRows; }

extern "C" int bob_sm100_bwd2_noalloc(const bob_sm100_geom* g, const void* q, const void* k,
                                      const void* v, const void* out, const float* lse,
                                      const float* delta, const float* pk, const void* dO,
                                      const void* dQ, const void* uQ, const void* uK, const void* uV,
                                      void* Qbar, void* Kbar, void* Vbar, void* dObar, void* stream) {
    if (!g) return -1;
    if (g->B <= 0 || g->Hq <= 0 || g->Nq <= 0) return -2;
    const size_t rows = static_cast<size_t>(g->B) * static_cast<size_t>(g->Hq) * static_cast<size_t>(g->Nq);
    if (rows > kMaxRows) return -12;                               // larger than the built-in scratch
    if (bob_sm100_workspace_bytes(BOB_SM100_STAGE_BWD2, g) > kNoAllocScratchBytes) return -12;
    void* scratch = nullptr;
    const int rc = scratch_address(g->device, &scratch);
    if (rc) return rc;
    return bob_sm100_bwd2(g, q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, Qbar, Kbar, Vbar, dObar,
                          scratch, stream);
}
