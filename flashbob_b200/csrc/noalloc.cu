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
//
// The status word of the last call on a device is read back with bob_sm100_noalloc_read_status
// (the array's address is private to this file, so bob_sm100_read_status cannot be used).
#include "internal.h"

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
    if (bob::bwd2_workspace_bytes_unsplit(g) > kNoAllocScratchBytes) return -12;
    void* scratch = nullptr;
    const int rc = scratch_address(g->device, &scratch);
    if (rc) return rc;
    // no host-visible status word (its set-up page-locks memory) and no division of long work items
    // (that needs a larger workspace): this path touches nothing but the fixed array
    return bob::bwd2_impl(g, q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, Qbar, Kbar, Vbar, dObar,
                          scratch, stream, nullptr, bob::kPartBoth, false);
}

// Waits for `stream`, then returns the status word the last bob_sm100_bwd2_noalloc call on `device`
// left in the built-in scratch (0 = every wait completed; also 0 if no call has run there yet).
// Allocates nothing.
extern "C" int bob_sm100_noalloc_read_status(int device, void* stream) {
    if (device < 0 || device >= kMaxDevices) return -7;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        scratch = g_scratch_addr[device];
    }
    if (!scratch) return 0;
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return -7;
    if (prev != device && cudaSetDevice(device) != cudaSuccess) return -7;
    int v = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = 0;
    if (cudaMemcpyAsync(&v, scratch, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess)
        rc = -8;
    if (prev != device) cudaSetDevice(prev);
    return rc ? rc : v;
}
