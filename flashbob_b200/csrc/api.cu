// Host side of the C ABI: argument checks, tensor-map construction and kernel dispatch.
#include "internal.h"
#include "sweep.cuh"
#include "tmap.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace bob {

enum : int {
    kErrNull = -1, kErrGeom = -2, kErrDtype = -3, kErrHeadDim = -4, kErrStride = -5,
    kErrWorkspace = -6, kErrDevice = -7, kErrLaunch = -8, kErrAttr = -9, kErrAlign = -10, kErrRegs = -13,
    kErrNoDriver = -100,
};

// The first 256 bytes of every workspace: word 0 = status, words 8.. = work counters of the launches
// of one call.  The whole block is cleared by each call.
static constexpr size_t kStatusBlock = 256;
static constexpr int kCounterWord0 = 8;

static size_t round256(size_t x) { return (x + 255) / 256 * 256; }

static int check_geom(const bob_sm100_geom* g) {
    if (!g) return kErrNull;
    if (g->B <= 0 || g->Hq <= 0 || g->Hkv <= 0 || g->Nq <= 0 || g->Nk <= 0 || g->D <= 0) return kErrGeom;
    if (g->Hq % g->Hkv) return kErrGeom;
    if (g->Nq > (1 << 28) || g->Nk > (1 << 28)) return kErrGeom;
    if (g->dtype != BOB_SM100_FP16 && g->dtype != BOB_SM100_BF16) return kErrDtype;
    if (g->D % 16 || g->D > 128) return kErrHeadDim;
    if (g->window < 0 || (g->window > 0 && !g->is_causal)) return kErrGeom;
    if (g->q_offset < 0 || g->k_offset < 0) return kErrGeom;
    if (!(g->scale > 0.f) || !std::isfinite(g->scale)) return kErrGeom;
    return 0;
}

// Results are written with 16-byte stores, pk is read and written as float4.
static int check_aligned16(std::initializer_list<const void*> ptrs) {
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) % 16) return kErrAlign;
    return 0;
}
static int check_aligned4(std::initializer_list<const void*> ptrs) {
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) % 4) return kErrAlign;
    return 0;
}

static int check_strides(const int64_t* s, const void* ptr) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return kErrAlign;
    for (int i = 0; i < 3; ++i)
        if (s[i] < 0 || s[i] % 8) return kErrStride;
    return 0;
}

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
        changed = prev != dev;
    }
    ~DeviceGuard() { if (changed && prev >= 0) cudaSetDevice(prev); }
    bool changed = false;
};

// Number of SMs of a device (cached: the attribute query is slow enough to show at small sizes).
static int sm_count(int device) {
    static int cache[64] = {};
    if (device < 0 || device >= 64) return -1;
    if (cache[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) return -1;
        cache[device] = n;
    }
    return cache[device];
}

// Column-owned kernels: number of TN-wide query tiles that the 128 keys of own tile `own_tile` sweep
// (the host's copy of the kernel's item decoding: same clipping of the causal / window range).
static int col_sweep_tiles(const bob_sm100_geom* g, long long doff, int own_tile, int TN) {
    const long long own0 = 128LL * own_tile, own_last = std::min<long long>(own0 + 127, g->Nk - 1);
    long long lo = 0, hi = g->Nq;
    if (g->is_causal) {
        lo = std::max<long long>(0, own0 - doff);
        if (g->window > 0) hi = std::min<long long>(g->Nq, own_last - doff + g->window);
    }
    if (hi <= lo) return 0;
    return (int)((hi + TN - 1) / TN - lo / TN);
}

// Even split of a persistent column-owned launch over `ctas` CTAs: tile pairs per CTA, or 0 when the
// split does not apply (too little work per CTA to pay for the cut items' extra epilogues, or a list
// too long for 32-bit positions).
static int even_split_span(const bob_sm100_geom* g, long long doff, int TN, int ctas) {
#ifndef BOB_EVEN_SPLIT
    // Off: measured slower than the counter-fed item queue (a span of equally many tile pairs holds very
    // different numbers of items, and every item costs a prologue and an epilogue).
    (void)g; (void)doff; (void)TN; (void)ctas;
    return 0;
#endif
    const int n_own_tiles = (g->Nk + 127) / 128;
    const long long per_rank = (long long)g->Hkv * g->B, G = g->Hq / g->Hkv;
    long long total = 0;
    for (int r = 0; r < n_own_tiles; ++r) total += (long long)col_sweep_tiles(g, doff, r, TN) * G * per_rank;
    if (total <= 0 || total >= (1LL << 30)) return 0;
    const long long span = (total + ctas - 1) / ctas;
    return span >= 32 ? (int)span : 0;
}

static size_t even_split_flag_bytes(const bob_sm100_geom* g) {
    return round256((size_t)((g->Nk + 127) / 128) * g->Hkv * g->B * sizeof(int));
}
static size_t even_split_park_bytes(int ctas) { return (size_t)ctas * 2 * 2 * 128 * 64 * sizeof(float); }

// Whether a column-owned launch of this geometry is persistent (one CTA per SM taking many items).
static bool col_launch_is_persistent(const bob_sm100_geom* g, int sms) {
    return (long long)((g->Nk + 127) / 128) * g->Hkv * g->B > sms;
}

struct TensorArg {
    const void* ptr;
    const int64_t* strides;   // batch, head, row
    bool q_side;              // [B, Hq, Nq, D] (true) or [B, Hkv, Nk, D] (false)
};

template <int MODE, int DPAD, int TN, bool BF16, int NG = 1, int CW = 16>
static int launch_sweep(const bob_sm100_geom* g, SweepParams& prm, const TensorArg* tensors,
                        cudaStream_t stream, int counter_slot) {
    using CFG = SweepConfig<MODE, DPAD, TN, NG, CW>;
    using MT = ModeTraits<MODE>;
    auto build = [&](int t, int box_rows) -> int {
        const TensorArg& a = tensors[t];
        if (!a.ptr) return 0;
        int rc = check_strides(a.strides, a.ptr);
        if (rc) return rc;
        return make_tile_map(&prm.map[t], a.ptr, BF16, g->D, a.q_side ? g->Nq : g->Nk,
                             a.q_side ? g->Hq : g->Hkv, g->B, a.strides[2], a.strides[1],
                             a.strides[0], box_rows);
    };
    for (int i = 0; i < MT::NOWN; ++i) {
        int rc = build(own_tensor<MODE>(i), 128);
        if (rc) return rc;
    }
    for (int i = 0; i < MT::NOTH; ++i) {
        int rc = build(other_tensor<MODE>(i), TN);
        if (rc) return rc;
    }
    // The second backward has a build of its own for the usual case of three defined tangents.
    constexpr bool kSecond = (MODE == kBwd2Row || MODE == kBwd2Col);
    const bool allt = kSecond && prm.has_uq && prm.has_uk && prm.has_uv;
    auto kernel = allt ? sweep_kernel<MODE, DPAD, TN, BF16, NG, CW, kSecond>
                       : sweep_kernel<MODE, DPAD, TN, BF16, NG, CW, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CFG::SMEM_BYTES) !=
        cudaSuccess)
        return kErrAttr;
    if constexpr (CFG::REBALANCE) {
        // The kernel's warpgroups trade registers after launch; the trade only balances (and the
        // pointwise warps' request can only ever be met) if the kernel was built with the register
        // count the trade assumes.  Refuse to launch otherwise.
        cudaFuncAttributes a;
        const int regs_at_launch = cudaFuncGetAttributes(&a, kernel) == cudaSuccess ? a.numRegs : 0;
        if (regs_at_launch * CFG::NTHREADS < 256 * CFG::REGS_POINTWISE + 128 * CFG::REGS_ROLE) return kErrRegs;
    }
    // CTAs take work items in rounds (see the kernel): gridDim.x items per round.
    const int n_own = MT::COL ? g->Nk : g->Nq;
    const long long items = (long long)((n_own + 127) / 128) * (MT::COL ? g->Hkv : g->Hq) * g->B;
    if (items > 0x7fffffffLL) return kErrGeom;
    const int sms = sm_count(g->device);
    if (sms <= 0) return kErrDevice;
    // One persistent CTA per SM whenever there are more items than SMs.  (With the earlier static
    // assignment of items to CTAs, head dim 128 was ~4 % faster with one CTA per item and the hardware's
    // own placement; fed from the counter the persistent launch is 0.3-2 % faster there too.)
    const bool persistent = items > sms;
    dim3 grid((unsigned)(persistent ? sms : items), 1, 1);
    // Persistent CTAs take items, longest first, from a counter in the status block (zeroed with it);
    // column-owned ones with a parking area instead split the item list evenly (see the kernel).
    prm.work_counter = persistent ? prm.status + kCounterWord0 + counter_slot : nullptr;
    prm.sk_span = 0;
    if (MT::COL && persistent && prm.sk_park && prm.sk_flags) {
        prm.sk_span = even_split_span(g, prm.delta_off, TN, (int)grid.x);
        if (prm.sk_span > 0 &&
            cudaMemsetAsync(prm.sk_flags, 0, even_split_flag_bytes(g), stream) != cudaSuccess)
            return kErrLaunch;
    }
    kernel<<<grid, CFG::NTHREADS, CFG::SMEM_BYTES, stream>>>(prm);
    return cudaGetLastError() == cudaSuccess ? 0 : kErrLaunch;
}

// Tile table (template arguments: head dim, swept-tile width, dtype, pointwise groups, score columns
// per pointwise thread).
// Head dim <= 64.  Forward: 128-wide tiles, two groups of 128 threads, each thread a whole row, each
// group its own online softmax and output accumulator.  First backward: 128-wide tiles, one group of
// 512 threads (more warps per scheduler measured better than fewer threads holding more columns).
// Second backward: four score accumulators, four operands and two outputs fill tensor memory at
// 64-wide tiles; one group of 256 threads holds a whole tile's columns at 208 registers.
// Head dim 128.  Forward: 64-wide tiles, two groups, a row per thread.  First backward: 64-wide tiles.
// Second backward: tensor memory (512 columns) leaves room for 32-wide tiles only.
template <int MODE, bool BF16>
static int dispatch(const bob_sm100_geom* g, SweepParams& prm, const TensorArg* tensors,
                    cudaStream_t stream, int counter_slot) {
    constexpr bool kSecond = (MODE == kBwd2Row || MODE == kBwd2Col);
    if (g->D <= 64) {
        if constexpr (kSecond)           return launch_sweep<MODE, 64, 64, BF16, 1, 32>(g, prm, tensors, stream, counter_slot);
        else if constexpr (MODE == kFwd) return launch_sweep<MODE, 64, 128, BF16, 2, 128>(g, prm, tensors, stream, counter_slot);
        else                             return launch_sweep<MODE, 64, 128, BF16, 1, 32>(g, prm, tensors, stream, counter_slot);
    }
    if constexpr (kSecond)           return launch_sweep<MODE, 128, 32, BF16>(g, prm, tensors, stream, counter_slot);
    else if constexpr (MODE == kFwd) return launch_sweep<MODE, 128, 64, BF16, 2, 64>(g, prm, tensors, stream, counter_slot);
    else                             return launch_sweep<MODE, 128, 64, BF16>(g, prm, tensors, stream, counter_slot);
}

template <int MODE>
static int dispatch_dtype(const bob_sm100_geom* g, SweepParams& prm, const TensorArg* tensors,
                          cudaStream_t stream, int counter_slot) {
    return g->dtype == BOB_SM100_BF16 ? dispatch<MODE, true>(g, prm, tensors, stream, counter_slot)
                                      : dispatch<MODE, false>(g, prm, tensors, stream, counter_slot);
}

// Only builds with -DBOB_PHASE_TIMERS or -DBOB_TRACE (never the shipped library) read a device pointer (hex) from
// BOB_SM100_PHASE_PTR: 24 cycle counters (12 of a pointwise thread, then 12 of the MMA warp).
static long long* phase_pointer() {
#if defined(BOB_PHASE_TIMERS) || defined(BOB_TRACE)
    const char* e = std::getenv("BOB_SM100_PHASE_PTR");
    return e ? reinterpret_cast<long long*>(std::strtoull(e, nullptr, 16)) : nullptr;
#else
    return nullptr;
#endif
}

// A per-device word in host memory that kernels can write: a CTA whose bounded wait ran out stores its
// status code there as well as in the workspace, so the host can notice without synchronising
// (bob_sm100_last_status).  Page-locked once per device on first use; null if that failed.
int* sticky_word(int device, bool create) {
    static std::mutex mu;
    static int* host[64] = {};
    static int* dev[64] = {};
    static bool tried[64] = {};
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!tried[device] && create) {
        tried[device] = true;
        void* h = nullptr;
        void* d = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
            std::memset(h, 0, 64);
            if (cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess) {
                host[device] = static_cast<int*>(h);
                dev[device] = static_cast<int*>(d);
            } else {
                cudaFreeHost(h);
            }
        }
        cudaGetLastError();
    }
    return create ? dev[device] : host[device];
}

static void fill_common(const bob_sm100_geom* g, SweepParams& p, void* workspace) {
    std::memset(&p, 0, sizeof(p));
    p.B = g->B; p.Hq = g->Hq; p.Hkv = g->Hkv; p.G = g->Hq / g->Hkv; p.Nq = g->Nq; p.Nk = g->Nk;
    p.D = g->D;
    p.is_causal = g->is_causal ? 1 : 0;
    p.window = g->window;
    // Beyond +-2^30 every pair is masked the same way as at the bound (sequence lengths are far
    // smaller), and 32-bit position arithmetic in the kernels cannot overflow.
    const int64_t d = g->q_offset - g->k_offset;
    p.delta_off = static_cast<int>(d > (1 << 30) ? (1 << 30) : (d < -(1 << 30) ? -(1 << 30) : d));
    p.scale = g->scale;
    p.status = static_cast<int*>(workspace);
    p.phase_cycles = phase_pointer();
}

static void set_strided(const void*& dst, long long& sb, long long& sh, long long& sn,
                        const void* ptr, const int64_t* s) {
    dst = ptr; sb = s[0]; sh = s[1]; sn = s[2];
}

}  // namespace bob

using namespace bob;

extern "C" int bob_sm100_version(void) { return 100; }

extern "C" const char* bob_sm100_error_string(int code) {
    switch (code) {
        case 0: return "ok";
        case kErrNull: return "null pointer argument";
        case kErrGeom: return "invalid geometry (sizes, heads, window, offsets or scale)";
        case kErrDtype: return "dtype must be fp16 (0) or bf16 (1)";
        case kErrHeadDim: return "head dimension must be a multiple of 16, at most 128";
        case kErrStride: return "tensor strides must be non-negative multiples of 8 elements";
        case kErrWorkspace: return "workspace missing or misaligned";
        case kErrDevice: return "cannot select the device";
        case kErrLaunch: return "kernel launch failed";
        case kErrAttr: return "cannot raise the dynamic shared memory limit";
        case kErrAlign: return "tensor base address must be 16-byte aligned";
        case kErrRegs: return "kernel was built with too few registers for its register rebalancing";
        case kErrNoDriver: return "cuTensorMapEncodeTiled is unavailable in this driver";
        case -11: return "cannot resolve the built-in scratch array on this device";
        case -12: return "problem too large for the built-in scratch (B*Hq*Nq > 1048576 rows)";
        case -101: return "tensor base address must be 16-byte aligned";
        case -102: return "tensor strides unusable for TMA";
        case 77: return "device: the self-test's wait ran out (as it is meant to)";
        case kStatusTimeoutLoad: return "device: a wait for a TMA load ran out";
        case kStatusTimeoutMma: return "device: a wait in the MMA issuer ran out";
        case kStatusTimeoutPw: return "device: a wait in the pointwise threads ran out";
        default: return code < -1000 ? "cuTensorMapEncodeTiled failed" : "unknown code";
    }
}

// Bytes of the even-split area (flags, then parked partials) a stage's column-owned kernel may use.
static size_t even_split_bytes(const bob_sm100_geom* g) {
#ifndef BOB_EVEN_SPLIT
    (void)g;
    return 0;
#endif
    const int sms = sm_count(g->device);
    if (sms <= 0 || !col_launch_is_persistent(g, sms)) return 0;
    return even_split_flag_bytes(g) + even_split_park_bytes(sms);
}

extern "C" size_t bob_sm100_workspace_bytes(int stage, const bob_sm100_geom* g) {
    if (!g || g->B <= 0 || g->Hq <= 0 || g->Hkv <= 0 || g->Nq <= 0 || g->Nk <= 0) return 0;
    size_t bytes = kStatusBlock;
    if (stage == BOB_SM100_STAGE_BWD2) bytes = bwd2_workspace_bytes_unsplit(g);
    if (stage == BOB_SM100_STAGE_BWD1 || stage == BOB_SM100_STAGE_BWD2) bytes += even_split_bytes(g);
    return bytes;
}

extern "C" int bob_sm100_kernel_launches(int stage, const bob_sm100_geom* g) {
    (void)g;
    return stage == BOB_SM100_STAGE_FWD ? 1 : 2;    // one sweep, or a row-owned and a column-owned sweep
}

extern "C" int bob_sm100_read_status(const void* workspace, void* stream) {
    if (!workspace) return kErrNull;
    int v = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess)
        return kErrLaunch;
    if (cudaStreamSynchronize(s) != cudaSuccess) return kErrLaunch;
    return v;
}

extern "C" int bob_sm100_last_status(int device) {
    int* w = sticky_word(device, false);
    if (!w) return 0;
    return __atomic_exchange_n(w, 0, __ATOMIC_ACQ_REL);
}

// Clears the status block (status word and work counters) of a call's workspace.
static int begin_call(void* workspace, cudaStream_t s) {
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256) return kErrWorkspace;
    return cudaMemsetAsync(workspace, 0, kStatusBlock, s) == cudaSuccess ? 0 : kErrLaunch;
}

extern "C" int bob_sm100_fwd(const bob_sm100_geom* g, const void* q, const void* k, const void* v,
                             void* out, float* lse, void* workspace, void* stream) {
    int rc = check_geom(g);
    if (rc) return rc;
    if (!q || !k || !v || !out || !lse) return kErrNull;
    if ((rc = check_aligned16({out}))) return rc;
    if ((rc = check_aligned4({lse}))) return rc;
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256) return kErrWorkspace;
    DeviceGuard guard(g->device);
    if (!guard.ok) return kErrDevice;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if ((rc = begin_call(workspace, s))) return rc;

    SweepParams p;
    fill_common(g, p, workspace);
    p.sticky = sticky_word(g->device, true);
    p.lse = lse;
    p.res0 = out;
    TensorArg t[kNumTensors] = {};
    t[kTQ] = {q, g->q_strides, true};
    t[kTK] = {k, g->k_strides, false};
    t[kTV] = {v, g->v_strides, false};
    return dispatch_dtype<kFwd>(g, p, t, s, 0);
}

extern "C" int bob_sm100_bwd1(const bob_sm100_geom* g, const void* q, const void* k, const void* v,
                              const void* out, const float* lse, const void* dO, void* dQ, void* dK,
                              void* dV, float* delta, float* pk, void* workspace, void* stream) {
    int rc = check_geom(g);
    if (rc) return rc;
    if (!q || !k || !v || !out || !lse || !dO || !dQ || !dK || !dV || !delta) return kErrNull;
    if ((rc = check_aligned16({dQ, dK, dV, pk}))) return rc;
    if ((rc = check_aligned4({lse, delta}))) return rc;
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256) return kErrWorkspace;
    if ((rc = check_strides(g->out_strides, out))) return rc;
    if ((rc = check_strides(g->do_strides, dO))) return rc;
    DeviceGuard guard(g->device);
    if (!guard.ok) return kErrDevice;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if ((rc = begin_call(workspace, s))) return rc;

    TensorArg t[kNumTensors] = {};
    t[kTQ] = {q, g->q_strides, true};
    t[kTK] = {k, g->k_strides, false};
    t[kTV] = {v, g->v_strides, false};
    t[kTDO] = {dO, g->do_strides, true};

    SweepParams p;
    fill_common(g, p, workspace);
    p.sticky = sticky_word(g->device, true);
    p.lse = const_cast<float*>(lse);
    p.delta = delta;
    p.pk = pk;
    set_strided(p.out, p.out_sb, p.out_sh, p.out_sn, out, g->out_strides);
    set_strided(p.dO, p.dO_sb, p.dO_sh, p.dO_sn, dO, g->do_strides);
    p.res0 = dQ;
    rc = dispatch_dtype<kBwd1Row>(g, p, t, s, 0);   // dQ and delta
    if (rc) return rc;
    p.res0 = dK;
    p.res1 = dV;
    if (even_split_bytes(g)) {
        p.sk_flags = reinterpret_cast<int*>(static_cast<char*>(workspace) + kStatusBlock);
        p.sk_park = reinterpret_cast<float*>(static_cast<char*>(workspace) + kStatusBlock + even_split_flag_bytes(g));
    }
    return dispatch_dtype<kBwd1Col>(g, p, t, s, 1); // dK and dV (reads delta)
}

int bob::bwd2_impl(const bob_sm100_geom* g, const void* q, const void* k, const void* v, const void* out,
                   const float* lse, const float* delta, const float* pk, const void* dO, const void* dQ,
                   const void* uQ, const void* uK, const void* uV, void* Qbar, void* Kbar, void* Vbar,
                   void* dObar, void* workspace, void* stream, int* sticky, int part, bool allow_split) {
    int rc = check_geom(g);
    if (rc) return rc;
    if (!q || !k || !v || !out || !lse || !delta || !pk || !dO || !dQ || !Qbar || !Kbar || !Vbar || !dObar)
        return kErrNull;
    if (part < kPartRow || part > kPartBoth) return kErrGeom;
    if ((rc = check_aligned16({Qbar, Kbar, Vbar, dObar, pk}))) return rc;
    if ((rc = check_aligned4({lse, delta}))) return rc;
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256) return kErrWorkspace;
    if ((rc = check_strides(g->out_strides, out))) return rc;
    if ((rc = check_strides(g->dq_strides, dQ))) return rc;
    DeviceGuard guard(g->device);
    if (!guard.ok) return kErrDevice;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if ((rc = begin_call(workspace, s))) return rc;

    TensorArg t[kNumTensors] = {};
    t[kTQ] = {q, g->q_strides, true};
    t[kTK] = {k, g->k_strides, false};
    t[kTV] = {v, g->v_strides, false};
    t[kTDO] = {dO, g->do_strides, true};
    t[kTUQ] = {uQ, g->uq_strides, true};
    t[kTUK] = {uK, g->uk_strides, false};
    t[kTUV] = {uV, g->uv_strides, false};

    SweepParams p;
    fill_common(g, p, workspace);
    p.sticky = sticky;
    p.has_uq = uQ != nullptr; p.has_uk = uK != nullptr; p.has_uv = uV != nullptr;
    p.lse = const_cast<float*>(lse);
    p.delta = const_cast<float*>(delta);
    p.pk = const_cast<float*>(pk);
    const size_t stat_bytes = round256(static_cast<size_t>(g->B) * g->Hq * g->Nq * sizeof(float));
    p.alpha = reinterpret_cast<float*>(static_cast<char*>(workspace) + kStatusBlock);
    p.ecirc = reinterpret_cast<float*>(static_cast<char*>(workspace) + kStatusBlock + stat_bytes);
    set_strided(p.out, p.out_sb, p.out_sh, p.out_sn, out, g->out_strides);
    set_strided(p.dQ, p.dQ_sb, p.dQ_sh, p.dQ_sn, dQ, g->dq_strides);
    if (part & kPartRow) {
        p.res0 = Qbar;
        p.res1 = dObar;
        rc = dispatch_dtype<kBwd2Row>(g, p, t, s, 0);   // Qbar, dObar, alpha, ecirc
        if (rc) return rc;
    }
    if (part & kPartCol) {
        p.res0 = Kbar;
        p.res1 = Vbar;
        if (allow_split && even_split_bytes(g)) {
            char* area = static_cast<char*>(workspace) + bwd2_workspace_bytes_unsplit(g);
            p.sk_flags = reinterpret_cast<int*>(area);
            p.sk_park = reinterpret_cast<float*>(area + even_split_flag_bytes(g));
        }
        rc = dispatch_dtype<kBwd2Col>(g, p, t, s, 1);   // Kbar, Vbar (reads alpha, ecirc)
    }
    return rc;
}

size_t bob::bwd2_workspace_bytes_unsplit(const bob_sm100_geom* g) {
    return kStatusBlock + 2 * round256(static_cast<size_t>(g->B) * g->Hq * g->Nq * sizeof(float));
}

extern "C" int bob_sm100_bwd2(const bob_sm100_geom* g, const void* q, const void* k, const void* v,
                              const void* out, const float* lse, const float* delta, const float* pk,
                              const void* dO, const void* dQ, const void* uQ, const void* uK, const void* uV,
                              void* Qbar, void* Kbar, void* Vbar, void* dObar, void* workspace,
                              void* stream) {
    return bwd2_impl(g, q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, Qbar, Kbar, Vbar, dObar, workspace,
                     stream, g ? sticky_word(g->device, true) : nullptr, kPartBoth, true);
}

extern "C" int bob_sm100_bwd2_part(int part, const bob_sm100_geom* g, const void* q, const void* k,
                                   const void* v, const void* out, const float* lse, const float* delta,
                                   const float* pk, const void* dO, const void* dQ, const void* uQ,
                                   const void* uK, const void* uV, void* Qbar, void* Kbar, void* Vbar,
                                   void* dObar, void* workspace, void* stream) {
    return bwd2_impl(g, q, k, v, out, lse, delta, pk, dO, dQ, uQ, uK, uV, Qbar, Kbar, Vbar, dObar, workspace,
                     stream, g ? sticky_word(g->device, true) : nullptr, part, true);
}
