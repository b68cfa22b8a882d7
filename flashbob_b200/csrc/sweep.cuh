// One tiled "sweep" kernel for every stage of second-order attention on sm_100a.
//
// A CTA owns 128 rows of one side of the score matrix (query rows in the row-owned stages, key
// columns in the column-owned stages) and sweeps tiles of TN positions of the other side.  For
// each tile pair it
//   1. forms score-shaped products  own[128, D] x other[TN, D]^T  with tcgen05.mma into tensor
//      memory (fp32),
//   2. reads them back (one thread per own row and per 16-column slice), applies the mask and the
//      softmax recomputation from the saved log-sum-exp, builds the derived 16-bit operands and
//      writes them back into tensor memory (tcgen05.st),
//   3. accumulates output-shaped products  operand[128, TN] x other[TN, D]  (operand read from
//      tensor memory, swept tile MN-major from shared memory) into tensor memory accumulators
//      that live for the whole sweep.
// Column-owned stages compute the transposed scores (own = K-side), so the thread that owns key j
// holds column j of the score matrix and the operands come out already transposed; the per-query
// statistics then vary along the tensor-memory columns and are staged in shared memory.
//
// Warp roles: NG groups of 128*NSPLIT pointwise threads, one MMA warp (warp-uniform control flow, one
// elected lane issues) and one TMA warp.  Tiles of the other side sit in a ring of 2 to 6 stages;
// the scores of tile t+1 are issued before the output products of tile t, so the tensor pipe works
// while the pointwise threads convert tile t.  Work items (own tile x head x batch) are handed out
// longest first, either from a global counter (persistent launches) or one per CTA.
//
// The algebra follows the reference's second backward (reference: src/bob/kernels/common.py:15-30
// for the formulas, :463-654 for the row-owned tile body and epilogue, :661-786 for the
// column-owned tile body) and the usual flash-attention forward / first backward.
#pragma once

#include "ptx.cuh"

namespace bob {

// Optional in-kernel phase timers: with -DBOB_PHASE_TIMERS one pointwise thread and the MMA issuer of
// every CTA add the SM cycles they spend in each phase to SweepParams::phase_cycles[0..15].
#if defined(BOB_TRACE)
// Event trace (development builds only): the CTA with blockIdx.x == BOB_TRACE records (event id, SM
// clock) pairs of one pointwise thread (buffer 0), the two MMA warps (buffers 1, 2) and a spare warp
// that watches barrier completions (buffer 3); SweepParams::phase_cycles points to 4 x 8192 words.
#define BOB_TR_MAX 8190
#ifndef BOB_TRACE_MODE
#define BOB_TRACE_MODE MODE          // -DBOB_TRACE_MODE=<mode>: only that mode's kernel records
#endif
#define BOB_PH_DECL int tr_n = 0;
#define BOB_TR(buf, i) { if ((buf) < 4 && MODE == BOB_TRACE_MODE && (int)blockIdx.x == BOB_TRACE && p.phase_cycles && tr_n < BOB_TR_MAX) { p.phase_cycles[(buf) * 8192 + 1 + tr_n] = ((long long)(i) << 48) | (clock64() & 0xFFFFFFFFFFFFLL); ++tr_n; } }
#define BOB_PH(i) { if ((threadIdx.x & 31) == 0) BOB_TR(tr_role, i) }
#define BOB_PH_FLUSH(base, on) if ((on) && tr_role < 4 && MODE == BOB_TRACE_MODE && (int)blockIdx.x == BOB_TRACE && p.phase_cycles) p.phase_cycles[tr_role * 8192] = tr_n;
#elif defined(BOB_PHASE_TIMERS)
#define BOB_PH_DECL long long ph_t = clock64(); long long ph_acc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#define BOB_PH(i) { const long long ph_n = clock64(); ph_acc[i] += ph_n - ph_t; ph_t = ph_n; }
#define BOB_PH_FLUSH(base, on) if ((on) && p.phase_cycles) { for (int ph_i = 0; ph_i < 12; ++ph_i) atomicAdd(reinterpret_cast<unsigned long long*>(p.phase_cycles) + (base) + ph_i, (unsigned long long)ph_acc[ph_i]); }
#else
#define BOB_PH_DECL
#define BOB_PH(i)
#define BOB_PH_FLUSH(base, on)
#endif

enum Mode : int { kFwd = 0, kBwd1Row = 1, kBwd1Col = 2, kBwd2Row = 3, kBwd2Col = 4 };
enum TensorId : int { kTQ = 0, kTK, kTV, kTDO, kTUQ, kTUK, kTUV, kNumTensors };

// Status codes written to the status word by a CTA that gave up on a wait.
enum : int { kStatusOk = 0, kStatusTimeoutLoad = 11, kStatusTimeoutMma = 12, kStatusTimeoutPw = 13 };

struct SweepParams {
    CUtensorMap map[kNumTensors];
    // geometry
    int B, Hq, Hkv, G, Nq, Nk, D;
    int is_causal, window;
    int delta_off;                // q_offset - k_offset, clamped to +-2^30
    float scale;
    int has_uq, has_uk, has_uv;   // 0 = that tangent is undefined (treated as zero, products skipped)
    // global tensors read with plain loads (element strides: batch, head, row; unit head-dim stride)
    const void* out;  long long out_sb, out_sh, out_sn;
    const void* dO;   long long dO_sb, dO_sh, dO_sn;
    const void* dQ;   long long dQ_sb, dQ_sh, dQ_sn;
    // fp32 row statistics, contiguous [B, Hq, Nq]
    float* lse;       // natural log
    float* delta;
    float* alpha;
    float* ecirc;
    // fp32 [B, Hq, Nq, D]: PK = P K, written by the first backward (may be null there: not needed
    // unless a second backward follows), read by the second backward's row-owned kernel
    float* pk;
    // results, contiguous [B, H, N, D] in the input dtype
    void* res0;
    void* res1;
    void* res2;
    int* status;
    int* sticky;                  // optional second word that a CTA giving up also writes (host-visible memory)
    int* work_counter;            // persistent launches: next work item (zeroed by the host); null: one item per CTA
    // Even split (column-owned modes, persistent launches): every CTA takes `sk_span` consecutive tile
    // pairs of the item list, cutting items where its span ends.  The pieces of a cut item park their
    // fp32 partial results in `sk_park` (two slots per CTA) and count themselves in `sk_flags[item]`
    // (zeroed by the host); the last piece to finish adds the parked partials and stores the result.
    int sk_span;                  // 0: off
    float* sk_park;
    int* sk_flags;
    long long* phase_cycles;      // optional cycle counters per pipeline phase (builds with BOB_PHASE_TIMERS)
};

template <int MODE> struct ModeTraits;
template <> struct ModeTraits<kFwd>     { static constexpr int NOWN = 1, NOTH = 2, NSC = 1, NOUT = 1, NOPER = 1; static constexpr bool COL = false; };
template <> struct ModeTraits<kBwd1Row> { static constexpr int NOWN = 2, NOTH = 2, NSC = 2, NOUT = 2, NOPER = 2; static constexpr bool COL = false; };
template <> struct ModeTraits<kBwd1Col> { static constexpr int NOWN = 2, NOTH = 2, NSC = 2, NOUT = 2, NOPER = 2; static constexpr bool COL = true; };
template <> struct ModeTraits<kBwd2Row> { static constexpr int NOWN = 3, NOTH = 4, NSC = 4, NOUT = 2, NOPER = 4; static constexpr bool COL = false; };
template <> struct ModeTraits<kBwd2Col> { static constexpr int NOWN = 4, NOTH = 3, NSC = 4, NOUT = 2, NOPER = 3; static constexpr bool COL = true; };

// Which global tensor fills own slot / other slot `i` of a mode.
template <int MODE> __host__ __device__ constexpr int own_tensor(int i) {
    if (MODE == kFwd) return kTQ;
    if (MODE == kBwd1Row) return i == 0 ? kTQ : kTDO;
    if (MODE == kBwd1Col) return i == 0 ? kTK : kTV;
    if (MODE == kBwd2Row) return i == 0 ? kTQ : (i == 1 ? kTDO : kTUQ);
    return i == 0 ? kTK : (i == 1 ? kTV : (i == 2 ? kTUK : kTUV));
}
template <int MODE> __host__ __device__ constexpr int other_tensor(int i) {
    if (MODE == kFwd || MODE == kBwd1Row) return i == 0 ? kTK : kTV;
    if (MODE == kBwd1Col) return i == 0 ? kTQ : kTDO;
    if (MODE == kBwd2Row) return i == 0 ? kTK : (i == 1 ? kTUK : (i == 2 ? kTV : kTUV));   // K, uK adjacent; V, uV adjacent
    return i == 0 ? kTQ : (i == 1 ? kTUQ : kTDO);                                          // Q, uQ adjacent
}

template <int MODE, int DPAD, int TN, int NG = 1, int CW = 16>
struct SweepConfig {
    using MT = ModeTraits<MODE>;
    // NG pointwise groups take the swept tiles in turn (group g: tiles g, g + NG, ...), each with its
    // own score accumulators and operand columns, so that one group's tensor-memory latencies hide
    // behind the other group's arithmetic and the MMA warp always has a tile to work on (forward:
    // each group also has its own output accumulator).
    // CW score columns per pointwise thread: 16 or 32 (more threads, at most 112 registers each),
    // or, with registers taken over from the MMA / TMA warpgroup (REBALANCE), 32, 64 or 128 held at
    // once by 256 threads.
    static constexpr int NSPLIT = TN / CW;
    static constexpr int GP = 128 * NSPLIT;                // pointwise threads per group
    static constexpr int NPW = GP * NG;                    // pointwise threads
    // Configurations with 256 pointwise threads that hold a whole tile's score columns: the two
    // pointwise warpgroups take registers over from the warpgroup of the MMA and TMA warps (padded
    // to four warps, two of them idle) once the kernel runs.
    static constexpr bool REBALANCE = NPW == 256 &&
        ((NG == 1 && (MODE == kBwd2Row || MODE == kBwd2Col) && CW == 32) ||
         (NG == 1 && (MODE == kBwd1Row || MODE == kBwd1Col) && CW == 64) ||
         (NG == 2 && MODE == kFwd && CW == 128));
    // Two MMA-issuing warps (one for the score-shaped products, one for the output-shaped ones) in the
    // second backward (measured 6-8 % faster at both head dims) and wherever the warpgroup of the role
    // warps has spare warps anyway; in the first backward one warp issues both kinds (there a third
    // role warp costs the 512 pointwise threads registers: 0.36 ms against 0.33 ms).
    static constexpr bool TWO_MMA = REBALANCE || MODE == kBwd2Row || MODE == kBwd2Col;
    // Row-owned second backward with all of a tile's columns loaded at once: the score products are
    // ordered so that S, dP and C are complete before the last product (the second term of F) is
    // issued, and a barrier of its own tells the pointwise threads, whose loads of those three
    // accumulators then run under that last product (row-owned kernel 1.6-1.8 % faster; in the column-owned
    // kernel neither moving uK Q^T to the end nor a barrier before its last product, uV dO^T, paid:
    // 3-4 % slower).
    static constexpr bool SPLIT_SC = REBALANCE && MODE == kBwd2Row;
    static constexpr int NTHREADS = REBALANCE ? 384 : NPW + (TWO_MMA ? 96 : 64);   // + MMA warp(s) + TMA warp
#ifndef BOB_REGS_POINTWISE
#define BOB_REGS_POINTWISE 208       // measured: 224 / 56 starves the role warps' issue loops (column-owned
#define BOB_REGS_ROLE 88             // second backward 0.309 ms; 216 / 72: 0.301; 208 / 88: 0.297; 200 / 104: 0.303)
#endif
    static constexpr int REGS_POINTWISE = BOB_REGS_POINTWISE, REGS_ROLE = BOB_REGS_ROLE;
    static_assert(2 * 128 * REGS_POINTWISE + 128 * REGS_ROLE <= 384 * 168 && REGS_POINTWISE % 8 == 0 && REGS_ROLE % 8 == 0,
                  "register rebalancing must fit the pool of 384 threads x 168 registers");
    static constexpr int KSUB = DPAD / 64;                 // 64-element sub-tiles along the head dim
    static constexpr int OWN_TILE_BYTES = 128 * 128 * KSUB;
    static constexpr int OTH_SUB_BYTES = TN * 128;         // one 64-element-wide sub-tile of a swept tensor
    static constexpr int OTH_STAGE_BYTES = KSUB * MT::NOTH * OTH_SUB_BYTES;   // laid out [sub][slot]
    // tensor memory map: [score accumulators | derived 16-bit operands | output accumulators]
    static constexpr int SC_COLS = MT::NSC * TN;
    static constexpr int OPER_COLS_EACH = TN / 2;          // 128 x TN 16-bit values, two per 32-bit column
    static constexpr int OPER_COLS = MT::NOPER * OPER_COLS_EACH;
    // The forward keeps one output accumulator per pointwise group (each group runs its own online
    // softmax over the tiles it takes; the epilogue merges them).
    static constexpr int NACC = (MODE == kFwd) ? NG : MT::NOUT;
    static_assert(MODE != kFwd || (NG == 2 && CW == TN && (TN == 64 || TN == 128)), "forward: two groups, one thread per row");
    static constexpr int OUT_COLS = NACC * DPAD;
    static constexpr int TMEM_BASE_NEED = NG * (SC_COLS + OPER_COLS) + OUT_COLS;
    // Second backward: where tensor memory has DPAD / 2 columns to spare, the first own tile (Q, or K
    // in the column-owned kernel) is also kept there, 16-bit packed like the derived operands, and its
    // score product reads it from tensor memory: per instruction that product then fetches only the
    // swept tile from shared memory (measured 47-51 cycles against 69-72 at N = 64, 72 against ~100 at
    // N = 128).  Used at head dim 128, where both kernels have the columns (5 % faster); it would also
    // fit the column-owned kernel at head dim 64, where it measured no gain (0.315 against 0.311 ms:
    // the next item's score products then wait for the pointwise threads' copy).
    static constexpr bool OWN_TM = (MODE == kBwd2Row || MODE == kBwd2Col) && NG == 1 && DPAD == 128 && TMEM_BASE_NEED + DPAD / 2 <= 512;
    static constexpr int OWN_TM_COLS = OWN_TM ? DPAD / 2 : 0;
    static constexpr int TMEM_NEED = TMEM_BASE_NEED + OWN_TM_COLS;
    static constexpr int TMEM_COLS = TMEM_NEED <= 128 ? 128 : (TMEM_NEED <= 256 ? 256 : 512);
    static_assert(TMEM_NEED <= 512, "tensor memory budget exceeded");
    // as many stages of swept tiles as shared memory allows, between 2 and 6: the TMA latency of a
    // tile (~2 us) hides behind the tiles before it
    // Row-owned second backward at head dim <= 64: the epilogue's 16-bit global operands (out, dQ:
    // 16 KB each) are copied into shared memory with coalesced asynchronous copies while the item
    // runs, and the results leave through the same buffers with coalesced stores.  (A thread owns one
    // row of the tile; touching global memory row by row costs one 128-byte line per lane and
    // instruction.)  Both directions are the work of the fourth warp of the role warpgroup (the "IO
    // warp"), not of the pointwise threads: between two items the tensor pipe waits for the pointwise
    // threads, so whatever they do not have to do there is gained.  The fp32 pk rows are read straight
    // from global memory into registers when the sweep ends (staging them too would cost the 32 KB
    // that a fourth stage of swept tiles needs, and with three stages the tensor pipe waited ~400
    // cycles per tile for the next swept tiles).
    static constexpr bool STAGED_IO = (MODE == kBwd2Row) && DPAD == 64 && NG == 1 && REBALANCE;
    static constexpr int IO_BYTES = STAGED_IO ? 32 * 1024 : 0;
    static constexpr int FIXED_BYTES = MT::NOWN * OWN_TILE_BYTES + 16 * 1024 + IO_BYTES;
    static constexpr int STAGE_ROOM = (232448 - FIXED_BYTES) / OTH_STAGE_BYTES;
    static constexpr int STAGE_MAX = 6;
    static constexpr int NSTAGE = STAGE_ROOM >= STAGE_MAX ? STAGE_MAX : (STAGE_ROOM >= 2 ? STAGE_ROOM : 2);
    static_assert(NSTAGE > NG, "score products may run NG tiles ahead: they need NG + 1 stages of swept tiles");
    // shared memory map (offsets from a 1024-byte aligned base)
    static constexpr int OFF_OWN = 0;
    static constexpr int OFF_OTH = OFF_OWN + MT::NOWN * OWN_TILE_BYTES;
    static constexpr int OFF_STAT = OFF_OTH + NSTAGE * OTH_STAGE_BYTES;         // [NSTAGE][4][TN] floats
    static constexpr int OFF_RED = OFF_STAT + NSTAGE * 4 * TN * 4;              // [2][NG * NSPLIT][128] floats
    static constexpr int OFF_BAR = OFF_RED + (MODE == kFwd ? 4 : 2) * NG * NSPLIT * 128 * 4;   // forward: two copies
    static constexpr int RING = 4;                                              // work items announced ahead
    static constexpr int NBARS = 1 + 3 * NSTAGE + 3 + 5 * NG + 2 * RING + 1 + 2 + NG;
    static constexpr int OFF_MISC = OFF_BAR + NBARS * 8;                        // tmem slot, abort flag, item ring
    static constexpr int OFF_IO = (OFF_MISC + 16 + 32 * RING + 127) & ~127;     // staged epilogue operands
    static constexpr int SMEM_BYTES = OFF_IO + IO_BYTES + 1024;                 // + alignment slack
    static_assert(SMEM_BYTES <= 232448, "shared memory budget exceeded");
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool BF16>
__device__ __forceinline__ void load16_as_float(const void* base, long long elem_off, float* v) {
    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem_off);
    uint4 a = p[0], b = p[1];
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
        if constexpr (BF16) {
            __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            float2 f = __bfloat1622float2(t);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        } else {
            __half2 t = *reinterpret_cast<const __half2*>(&w[i]);
            float2 f = __half22float2(t);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
}

template <bool BF16>
__device__ __forceinline__ void unpack8_as_float(const uint4 a, float* v) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (BF16) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        } else {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
}

template <bool BF16>
__device__ __forceinline__ void store16_from_float(void* base, long long elem_off, const float* v) {
    uint4 a, b;
    a.x = pack2<BF16>(v[0], v[1]);   a.y = pack2<BF16>(v[2], v[3]);
    a.z = pack2<BF16>(v[4], v[5]);   a.w = pack2<BF16>(v[6], v[7]);
    b.x = pack2<BF16>(v[8], v[9]);   b.y = pack2<BF16>(v[10], v[11]);
    b.z = pack2<BF16>(v[12], v[13]); b.w = pack2<BF16>(v[14], v[15]);
    uint4* p = reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + elem_off);
    p[0] = a; p[1] = b;
}

template <bool V> struct BoolTag { static constexpr bool value = V; };
template <int V> struct IntTag { static constexpr int value = V; };

template <int MODE, int DPAD, int TN, bool BF16, int NG, int CW, bool ALLT = false>
__global__ void __launch_bounds__(SweepConfig<MODE, DPAD, TN, NG, CW>::NTHREADS, 1)
sweep_kernel(const __grid_constant__ SweepParams p) {
    static_assert(!ALLT || MODE == kBwd2Row || MODE == kBwd2Col, "only the second backward has tangents");
    using CFG = SweepConfig<MODE, DPAD, TN, NG, CW>;
    static_assert(CW == 16 || CW == 32 || (CW == 64 && MODE <= kBwd1Col) || (CW == 128 && MODE == kFwd),
                  "16 or 32 columns per pointwise thread (first backward: also 64; forward: 64 or 128)");
    // columns per round of tensor-memory loads (8 where 512 pointwise threads share the second
    // backward's tile: four loaded accumulators and four packed operands must fit 112 registers)
    constexpr int RW = ((MODE == kBwd2Row || MODE == kBwd2Col) && CW == 16 && TN == 64) ? 8 : 16;
    using MT = ModeTraits<MODE>;
    constexpr int NSPLIT = CFG::NSPLIT, NPW = CFG::NPW, GP = CFG::GP, NSTAGE = CFG::NSTAGE, KSUB = CFG::KSUB;
    constexpr bool COL = MT::COL;
    constexpr bool BWD2 = (MODE == kBwd2Row || MODE == kBwd2Col);
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kLn2 = 0.6931471805599453f;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t sbase = (raw_addr + 1023u) & ~1023u;
    uint8_t* sptr = smem_raw + (sbase - raw_addr);
    float* stat_buf = reinterpret_cast<float*>(sptr + CFG::OFF_STAT);
    float* red_buf = reinterpret_cast<float*>(sptr + CFG::OFF_RED);
    volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sptr + CFG::OFF_MISC);  // [0]=tmem, [1]=abort
    const uint32_t bar0 = sbase + CFG::OFF_BAR;
    const uint32_t bar_own = bar0;
    auto bar_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (1 + NSTAGE + s); };
    auto bar_stat = [&](int s) { return bar0 + 8u * (1 + 2 * NSTAGE + s); };     // per stage: row statistics staged
    const uint32_t bar_done = bar0 + 8u * (1 + 3 * NSTAGE);
    const uint32_t bar_pw_all = bar_done + 8;                                  // all pointwise threads
    const uint32_t bar_out_free = bar_done + 16;                               // output accumulators read out
    const uint32_t bar_grp0 = bar_done + 24;                                   // five barriers per group:
    auto bar_sc_full = [&](int g) { return bar_grp0 + 40u * g; };             //   scores ready
    auto bar_sc_empty = [&](int g) { return bar_grp0 + 40u * g + 8; };        //   scores read
    auto bar_op_full = [&](int g) { return bar_grp0 + 40u * g + 16; };        //   operands written
    auto bar_op_empty = [&](int g) { return bar_grp0 + 40u * g + 24; };       //   operands consumed
    auto bar_pw = [&](int g) { return bar_grp0 + 40u * g + 32; };             //   the group's own threads
    const uint32_t bar_ring0 = bar_grp0 + 40u * NG;
    auto bar_item_full = [&](int s) { return bar_ring0 + 8u * s; };           // ring slot announced
    const uint32_t bar_own_tm = bar_ring0 + 8u * (2 * CFG::RING);                // own tile 0 copied into tensor memory
    const uint32_t bar_io_full = bar_own_tm + 8;                               // IO warp: the item's out / dQ rows are staged
    const uint32_t bar_io_ready = bar_own_tm + 16;                             // pointwise warps: the item's results are staged
    auto bar_sc_part = [&](int g) { return bar_own_tm + 24 + 8u * g; };        // S, dP, C ready (SPLIT_SC)
    auto bar_item_empty = [&](int s) { return bar_ring0 + 8u * (CFG::RING + s); };   // ring slot read by every follower (two MMA warps, the pointwise warps)

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // ---- work items ----------------------------------------------------------------------------
    // One item = one own tile of one head of one batch element, swept over the other side.  Items
    // are numbered longest-sweep-first (all heads' heaviest tile, then all heads' second heaviest,
    // ...).  The kernel is persistent: CTA c takes items c, c + gridDim.x, ..., keeps its tensor
    // memory and barriers, and lets the TMA and MMA warps start an item while the pointwise threads
    // still write out the previous one.
    const int n_own = COL ? p.Nk : p.Nq;
    const int n_oth = COL ? p.Nq : p.Nk;
    const int n_own_tiles = (n_own + 127) / 128;
    const int grid_heads = COL ? p.Hkv : p.Hq;
    const int per_rank = grid_heads * p.B;
    const int n_items = n_own_tiles * per_rank;
    const int n_outer = COL ? p.G : 1;
    const int doff = p.delta_off;                // q_offset - k_offset, clamped to +-2^30 by the host
    // kernel parameters that the per-tile code needs, read once
    const bool causal = p.is_causal != 0;
    const int window = p.window;
    // ALLT (second backward): all three tangents are defined, the usual case.  Their flags are then
    // compile-time constants, so the loads and arithmetic of F and C are unconditional instead of
    // predicated on values only known at run time.
    const bool has_uq = ALLT || p.has_uq != 0, has_uk = ALLT || p.has_uk != 0, has_uv = ALLT || p.has_uv != 0;
    struct Item { int own0, head, batch, kv_head, t_lo, t_hi, T, total; };
    // What the ring announces: an item, or a piece of one (tile pairs [lin0, lin0 + len) of its sweep,
    // counted head by head); part != 0 marks a piece of a cut item, whose list position starts at s_item.
    struct Work { int item, lin0, len, part, s_item; };
    auto decode = [&](int item) {
        Item w;
        const int tile_rank = item / per_rank;
        const int rem = item % per_rank;
        w.head = rem % grid_heads;               // query head (row-owned) or KV head (column-owned)
        w.batch = rem / grid_heads;
        // causal: row-owned sweeps grow with the row index, column-owned ones shrink with the column
        const int own_tile = (!COL && causal) ? (n_own_tiles - 1 - tile_rank) : tile_rank;
        w.own0 = own_tile * 128;
        w.kv_head = COL ? w.head : w.head / p.G;
        int lo = 0, hi = n_oth;                  // other-side positions [lo, hi) that can be unmasked
        const int own_last = min(w.own0 + 127, n_own - 1);
        if (causal) {
            if (!COL) {
                hi = (int)min((long long)n_oth, (long long)own_last + doff + 1);
                if (window > 0) lo = (int)max(0LL, (long long)w.own0 + doff - window + 1);
            } else {
                lo = (int)max(0LL, (long long)w.own0 - doff);
                if (window > 0) hi = (int)min((long long)n_oth, (long long)own_last - doff + window);
            }
        }
        w.t_lo = (hi > lo) ? lo / TN : 0;
        w.t_hi = (hi > lo) ? (hi + TN - 1) / TN : 0;
        w.T = w.t_hi - w.t_lo;
        w.total = w.T * n_outer;
        return w;
    };
    // Which items this CTA works on.  The TMA warp decides: with a work counter (persistent launch)
    // it takes the next item of the longest-first list from the counter, otherwise the CTA has the
    // single item blockIdx.x.  It announces each item (then -1 = no more) in a ring of RING slots in
    // shared memory; the MMA warp and the pointwise warps follow the ring.
    constexpr int RING = CFG::RING;
    volatile int* item_ring = reinterpret_cast<volatile int*>(sptr + CFG::OFF_MISC + 16);
#define BOB_ITEM_LOCALS(w, wk)                                                                     \
    const int own0 = (w).own0, head = (w).head, batch = (w).batch, kv_head = (w).kv_head;         \
    const int t_lo = (w).t_lo, t_hi = (w).t_hi, T = (w).T;                                         \
    const int total = (wk).len < 0 ? (w).total : (wk).len;          /* tile pairs of this piece */ \
    const int lin0 = (wk).len < 0 ? 0 : (wk).lin0;                                                 \
    (void)own0; (void)head; (void)batch; (void)kv_head; (void)t_lo; (void)t_hi; (void)T; (void)total; (void)lin0;

    // ---- set-up ------------------------------------------------------------------------------
    if (tid == 0) {
        mbar_init(bar_own, 1);
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); mbar_init(bar_stat(s), 32); }
        for (int g = 0; g < NG; ++g) {
            mbar_init(bar_sc_full(g), 1);
            mbar_init(bar_sc_part(g), 1);
            mbar_init(bar_sc_empty(g), GP / 32);
            mbar_init(bar_op_full(g), GP / 32);
            mbar_init(bar_op_empty(g), 1);
            mbar_init(bar_pw(g), GP / 32);
        }
        mbar_init(bar_done, 1);
        mbar_init(bar_pw_all, NPW / 32);
        mbar_init(bar_out_free, NPW / 32);
        for (int s = 0; s < CFG::RING; ++s) { mbar_init(bar_item_full(s), 1); mbar_init(bar_item_empty(s), (CFG::TWO_MMA ? 2 : 1) + (CFG::STAGED_IO ? 1 : 0) + NPW / 32); }
        mbar_init(bar_own_tm, NPW / 32);
        mbar_init(bar_io_full, 1);
        mbar_init(bar_io_ready, NPW / 32);
        misc[1] = 0;
        mbar_fence_init();
    }
    if (warp == NPW / 32) {
        tmem_alloc(sbase + CFG::OFF_MISC, CFG::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = __shfl_sync(0xffffffffu, misc[0], 0);      // warp-uniform, and known to be
    // [scores of group 0 .. NG-1 | operands of group 0 .. NG-1 | output accumulators]
    const uint32_t tmem_oper = tmem + NG * CFG::SC_COLS;
    const uint32_t tmem_out = tmem_oper + NG * CFG::OPER_COLS;
    const uint32_t tmem_own = tmem_out + CFG::OUT_COLS;                          // own tile 0, packed (OWN_TM only)
    (void)tmem_own;

    auto give_up = [&](int code) {
        misc[1] = 1;
        atomicCAS(p.status, 0, code);
        if (p.sticky) { *reinterpret_cast<volatile int*>(p.sticky) = code; __threadfence_system(); }
    };
    // Followers of the item ring: the k-th announced piece of work (item -1: none left; -2: the wait ran out).
    auto follow_ring = [&](int k) -> Work {
        const int slot = k % RING;
        Work wk = {-2, 0, -1, 0, 0};
        if (!__all_sync(0xffffffffu, mbar_wait(bar_item_full(slot), (k / RING) & 1))) return wk;
        // every lane reads the same words; the broadcast tells the compiler that the values (and all
        // the loop bounds and addresses derived from them) are uniform across the warp
        volatile int* e = item_ring + 8 * slot;
        wk.item = __shfl_sync(0xffffffffu, e[0], 0);
        wk.lin0 = __shfl_sync(0xffffffffu, e[1], 0);
        wk.len = __shfl_sync(0xffffffffu, e[2], 0);
        wk.part = __shfl_sync(0xffffffffu, e[3], 0);
        wk.s_item = __shfl_sync(0xffffffffu, e[4], 0);
        if (lane == 0) mbar_arrive(bar_item_empty(slot));
        return wk;
    };

    auto has_tensor = [&](int t) {
        return t == kTUQ ? has_uq : (t == kTUK ? has_uk : (t == kTUV ? has_uv : true));
    };
    // shared-memory address of sub-tile `sub` of swept-tensor slot `slot` in pipeline stage `stage`
    auto oth_addr = [&](int stage, int sub, int slot) {
        return sbase + CFG::OFF_OTH + stage * CFG::OTH_STAGE_BYTES + (sub * MT::NOTH + slot) * CFG::OTH_SUB_BYTES;
    };

    if (warp >= NPW / 32) {
    if constexpr (CFG::REBALANCE) setmaxnreg_dec<CFG::REGS_ROLE>();    // the whole warpgroup, idle warps too
    if (warp == NPW / 32 + 1) {
        // =========================== TMA producer =============================================
        // Lane 0 issues the TMA copies.  In column-owned modes all 32 lanes also stage the swept
        // tile's per-query statistics, negated, into the stage's statistics buffer:
        // [-lse*log2e | -delta | -alpha | -ecirc], TN floats each.
        int cnt = 0;                             // swept tiles issued so far, over all items
        int s = 0, round = 0;                    // pipeline stage of tile `cnt`, and cnt / NSTAGE
        int n_live = 0;                          // items with at least one tile started so far
        bool alive = true;
        // Even split: this CTA's span [sk_pos, sk_end) of the item list, counted in tile pairs.  The list
        // is ordered by tile rank; the per_rank items of a rank are equally long (sk_len tile pairs each)
        // and the rank's first item starts at list position sk_rank0.
        const bool even_split = COL && p.sk_span > 0;
        long long sk_pos = 0, sk_end = 0, sk_rank0 = 0;
        int sk_rank = 0, sk_len = 0;
        int z_rank = 0, z_idx = 0, z_count = 0;             // cursor over the items that have no tile pair at all
        auto rank_len = [&](int r) { return decode(r * per_rank).T * n_outer; };
        if (even_split) {
            sk_pos = (long long)blockIdx.x * p.sk_span;
            sk_end = sk_pos + p.sk_span;
            for (sk_rank = 0; sk_rank < n_own_tiles; ++sk_rank) {
                sk_len = rank_len(sk_rank);
                const long long nxt = sk_rank0 + (long long)sk_len * per_rank;
                if (sk_pos < nxt) break;
                sk_rank0 = nxt;
            }
        }
        for (int k_item = 0; alive; ++k_item) {
            const int slot = k_item % RING;
            if (k_item >= RING &&
                !__all_sync(0xffffffffu, mbar_wait(bar_item_empty(slot), (k_item / RING - 1) & 1))) {
                if (lane == 0) give_up(kStatusTimeoutLoad);
                break;
            }
            Work wk = {-1, 0, -1, 0, 0};
            if (even_split) {
                if (sk_rank < n_own_tiles && sk_pos < sk_end) {
                    // the next piece of my span
                    const int in_rank = (int)((sk_pos - sk_rank0) / sk_len);
                    const long long s_item = sk_rank0 + (long long)in_rank * sk_len;
                    wk.item = sk_rank * per_rank + in_rank;
                    wk.lin0 = (int)(sk_pos - s_item);
                    wk.len = (int)min(s_item + sk_len - sk_pos, sk_end - sk_pos);
                    wk.part = (wk.len == sk_len) ? 0 : 1;
                    wk.s_item = (int)s_item;
                    sk_pos += wk.len;
                    if (sk_pos == sk_rank0 + (long long)sk_len * per_rank) {     // the rank is used up
                        sk_rank0 = sk_pos;
                        do { ++sk_rank; sk_len = sk_rank < n_own_tiles ? rank_len(sk_rank) : 0; }
                        while (sk_rank < n_own_tiles && sk_len == 0);
                    }
                } else {
                    // my span is used up: the items without any tile pair (their results are zeros, written
                    // by the pointwise threads) are dealt to the CTAs in turn
                    while (z_rank < n_own_tiles && wk.item < 0) {
                        if (rank_len(z_rank) != 0 || z_idx == per_rank) { ++z_rank; z_idx = 0; continue; }
                        if (z_count % (int)gridDim.x == (int)blockIdx.x) { wk.item = z_rank * per_rank + z_idx; wk.len = 0; }
                        ++z_idx; ++z_count;
                    }
                }
            } else {
                if (p.work_counter) { if (lane == 0) wk.item = atomicAdd(p.work_counter, 1); wk.item = __shfl_sync(0xffffffffu, wk.item, 0); }
                else if (k_item == 0) wk.item = (int)blockIdx.x;
                if (wk.item < 0 || wk.item >= n_items) wk.item = -1;
            }
            if (lane == 0) {
                volatile int* e = item_ring + 8 * slot;
                e[0] = wk.item; e[1] = wk.lin0; e[2] = wk.len; e[3] = wk.part; e[4] = wk.s_item;
                mbar_arrive(bar_item_full(slot));
            }
            const int item = wk.item;
            if (item < 0) break;
            const Item w = decode(item);
            BOB_ITEM_LOCALS(w, wk)
            if constexpr (MODE == kBwd1Row || MODE == kBwd2Row) {
                // The pointwise threads start the item by reading their rows' statistics (and, in the
                // first backward, the rows of `out` for delta) with plain loads whose latency nothing
                // hides: ask for those lines now, a few tiles before they get there.
                const long long rs0 = ((long long)batch * p.Hq + head) * p.Nq + own0;
                const int r4 = (lane & 3) * 32;                      // 32 floats per line
                if (lane < 4 && own0 + r4 < n_own) prefetch_l2(p.lse + rs0 + r4);
                if (MODE == kBwd2Row && lane >= 4 && lane < 8 && own0 + r4 < n_own) prefetch_l2(p.delta + rs0 + r4);
                if constexpr (MODE == kBwd1Row) {
                    const uint16_t* g_out = static_cast<const uint16_t*>(p.out) + (long long)batch * p.out_sb + (long long)head * p.out_sh + (long long)own0 * p.out_sn;
                    #pragma unroll
                    for (int r = lane; r < 128; r += 32) {
                        if (own0 + r < n_own) {
                            prefetch_l2(g_out + (long long)r * p.out_sn);
                            if (DPAD > 64 && p.D > 64) prefetch_l2(g_out + (long long)r * p.out_sn + 64);
                        }
                    }
                }
            }
            if (total == 0) continue;
            if (n_live > 0) {
                // the previous item's last products have finished reading its own tiles
                if (!__all_sync(0xffffffffu, mbar_wait(bar_done, (n_live - 1) & 1))) {
                    if (lane == 0) give_up(kStatusTimeoutLoad);
                    break;
                }
            }
            if (lane == 0) {
                uint32_t own_bytes = 0;
                #pragma unroll
                for (int i = 0; i < MT::NOWN; ++i)
                    if (has_tensor(own_tensor<MODE>(i))) own_bytes += CFG::OWN_TILE_BYTES;
                mbar_arrive_expect_tx(bar_own, own_bytes);
                #pragma unroll
                for (int i = 0; i < MT::NOWN; ++i) {
                    const int t = own_tensor<MODE>(i);
                    if (!has_tensor(t)) continue;
                    #pragma unroll
                    for (int ks = 0; ks < KSUB; ++ks)
                        tma_load_4d(sbase + CFG::OFF_OWN + i * CFG::OWN_TILE_BYTES + ks * (128 * 128),
                                    &p.map[t], bar_own, ks * 64, own0, head, batch);
                }
            }
            ++n_live;
            int tile = t_lo + lin0 % T, outer = lin0 / T;     // swept tile of iteration `it`, and its head in the group (T > 0 here)
            for (int it = 0; it < total; ++it) {
                bool go = true;
                if (cnt >= NSTAGE) go = mbar_wait(bar_empty(s), (round - 1) & 1);
                go = __all_sync(0xffffffffu, go);
                if (!go) { if (lane == 0) give_up(kStatusTimeoutLoad); alive = false; break; }
                const int oth_head = COL ? (head * p.G + outer) : kv_head;
                if (lane == 0) {
                    uint32_t bytes = 0;
                    #pragma unroll
                    for (int i = 0; i < MT::NOTH; ++i) {
                        if (has_tensor(other_tensor<MODE>(i))) bytes += KSUB * CFG::OTH_SUB_BYTES;
                    }
                    mbar_arrive_expect_tx(bar_full(s), bytes);
                    #pragma unroll
                    for (int i = 0; i < MT::NOTH; ++i) {
                        const int t = other_tensor<MODE>(i);
                        if (!has_tensor(t)) continue;
                        #pragma unroll
                        for (int ks = 0; ks < KSUB; ++ks)
                            tma_load_4d(oth_addr(s, ks, i), &p.map[t], bar_full(s), ks * 64, tile * TN, oth_head, batch);
                    }
                }
                if constexpr (COL) {
                    float* sb = stat_buf + s * 4 * TN;
                    #pragma unroll
                    for (int r = lane; r < TN; r += 32) {
                        const int i = tile * TN + r;
                        float l2 = 0.f, d = 0.f, al = 0.f, ec = 0.f;
                        if (i < p.Nq) {
                            const long long off = ((long long)batch * p.Hq + oth_head) * p.Nq + i;
                            l2 = p.lse[off] * kLog2e;
                            d = p.delta[off];
                            if constexpr (MODE == kBwd2Col) { al = p.alpha[off]; ec = p.ecirc[off]; }
                        }
                        sb[r] = -l2; sb[TN + r] = -d; sb[2 * TN + r] = -al; sb[3 * TN + r] = -ec;
                    }
                    mbar_arrive(bar_stat(s));
                }
                ++cnt;
                if (++s == NSTAGE) { s = 0; ++round; }
                if (++tile == t_hi) { tile = t_lo; ++outer; }
            }
        }
        // Do not leave while copies into this CTA's shared memory may still be in flight.
        if (lane == 0) {
            for (int k = max(0, cnt - NSTAGE); k < cnt; ++k)
                mbar_wait(bar_full(k % NSTAGE), (k / NSTAGE) & 1);
            if (n_live > 0) mbar_wait(bar_own, (n_live - 1) & 1);
        }
    } else if (CFG::STAGED_IO && warp == NPW / 32 + 3) {
        // =========================== IO warp ==================================================
        // Per item: copy the tile's `out` and `dQ` rows into the two staging buffers (16-byte chunk c of
        // row r at chunk position c ^ (r & 7) of its 128-byte line), tell the pointwise threads, wait
        // until they have replaced them by the results (Qbar over dQ, dObar over out) and write those
        // out, whole 128-byte lines per quarter warp.
        const uint32_t io_out = sbase + CFG::OFF_IO, io_dq = io_out + 16384;
        for (int k_item = 0;; ++k_item) {
            const Work wk = follow_ring(k_item);
            if (wk.item == -2) give_up(kStatusTimeoutLoad);
            if (wk.item < 0) break;
            const Item w = decode(wk.item);
            BOB_ITEM_LOCALS(w, wk)
            const uint16_t* g_out = static_cast<const uint16_t*>(p.out) + (long long)batch * p.out_sb + (long long)head * p.out_sh + (long long)own0 * p.out_sn;
            const uint16_t* g_dq = static_cast<const uint16_t*>(p.dQ) + (long long)batch * p.dQ_sb + (long long)head * p.dQ_sh + (long long)own0 * p.dQ_sn;
            #pragma unroll 4
            for (int k = 0; k < 1024 / 32; ++k) {
                const int id = lane + 32 * k, r = id >> 3, c = id & 7;
                if (own0 + r < n_own && c * 8 < p.D) {
                    const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
                    cp_async16(io_out + off, g_out + (long long)r * p.out_sn + c * 8);
                    cp_async16(io_dq + off, g_dq + (long long)r * p.dQ_sn + c * 8);
                }
            }
            cp_async_commit();
            cp_async_wait_all();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_io_full);
            if (!__all_sync(0xffffffffu, mbar_wait(bar_io_ready, k_item & 1))) { give_up(kStatusTimeoutLoad); break; }
            const long long tile_row0 = ((long long)batch * p.Hq + head) * p.Nq + own0;     // results are contiguous
            uint16_t* g_q = static_cast<uint16_t*>(p.res0) + tile_row0 * p.D;
            uint16_t* g_do = static_cast<uint16_t*>(p.res1) + tile_row0 * p.D;
            #pragma unroll 4
            for (int k = 0; k < 1024 / 32; ++k) {
                const int id = lane + 32 * k, r = id >> 3, c = id & 7;
                if (own0 + r < n_own && c * 8 < p.D) {
                    const uint32_t off = r * 128 + ((c ^ (r & 7)) << 4);
                    *reinterpret_cast<uint4*>(g_q + (long long)r * p.D + c * 8) = ld_shared_v4(io_dq + off);
                    *reinterpret_cast<uint4*>(g_do + (long long)r * p.D + c * 8) = ld_shared_v4(io_out + off);
                }
            }
            __syncwarp();
        }
#ifdef BOB_TRACE
    } else if (warp == NPW / 32 + 3 && CFG::REBALANCE) {
        // spare warp: watches the completion of the score products, of the output products (operands
        // consumed) and of the swept-tile loads, and records when each phase flips
        if (lane == 0 && MODE == BOB_TRACE_MODE && (int)blockIdx.x == BOB_TRACE && p.phase_cycles) {
            int tr_n = 0;
            uint32_t ph_sc = 0, ph_op = 0, ph_full[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long t_end = clock64() + 4000000LL;
            while (clock64() < t_end && tr_n < BOB_TR_MAX - 4) {
                if (mbar_test_wait(bar_sc_full(0), ph_sc)) { BOB_TR(3, 20) ph_sc ^= 1u; }
                if (mbar_test_wait(bar_op_empty(0), ph_op)) { BOB_TR(3, 21) ph_op ^= 1u; }
                #pragma unroll
                for (int st = 0; st < NSTAGE; ++st)
                    if (mbar_test_wait(bar_full(st), ph_full[st])) { BOB_TR(3, 30 + st) ph_full[st] ^= 1u; }
            }
            p.phase_cycles[3 * 8192] = tr_n;
        }
#endif
    } else if (warp == NPW / 32 || (CFG::TWO_MMA && warp == NPW / 32 + 2)) {
        // =========================== MMA issuers ==============================================
        // Two warps issue the products, each from one elected lane: warp NPW/32 the score-shaped
        // ones (as far ahead as the pointwise threads hand score accumulators back), warp NPW/32 + 2
        // the output-shaped ones (as operands arrive).  The tensor pipe takes whichever is ready;
        // neither warp's waits and loop overhead delay the other's instructions.
        const bool score_role = (warp == NPW / 32);       // (with a single MMA warp: this warp does both)
        {
            constexpr uint32_t fmt = BF16 ? kFmtBF16 : kFmtF16;

            // Descriptor low words: (shared-memory address >> 4) | 0x10000 (leading byte offset 16).
            // Everything but the pipeline stage is a compile-time offset from these three bases.
            const uint32_t own16 = ((sbase + CFG::OFF_OWN) >> 4) | 0x10000u;
            const uint32_t oth16 = ((sbase + CFG::OFF_OTH) >> 4) | 0x10000u;

            // score-shaped product: acc[128, NS*TN] (+)= own[slot_a] * other[slot_b .. slot_b+NS-1]^T.
            // NS = 2 takes two adjacent swept tiles as one 2*TN-row operand and fills two adjacent
            // accumulators with one instruction per K step (the own tile is read once, not twice).
            auto score_mma = [&](auto ns_tag, uint32_t sc_base, int acc, int slot_a, int slot_b, uint32_t stage16, bool accumulate) {
                constexpr int NS = decltype(ns_tag)::value;
                constexpr uint32_t idesc = umma_idesc(fmt, fmt, NS * TN, false);
                const uint32_t a = own16 + ((slot_a * CFG::OWN_TILE_BYTES) >> 4);
                const uint32_t b = stage16 + ((slot_b * CFG::OTH_SUB_BYTES) >> 4);
                const bool from_tm = CFG::OWN_TM && slot_a == 0;          // own tile 0 also sits in tensor memory
                if (elect_one()) {
                    #pragma unroll
                    for (int ks = 0; ks < DPAD / 16; ++ks) {
                        const uint32_t ao = ((ks / 4) * (128 * 128) + (ks % 4) * 32) >> 4;
                        const uint32_t bo = ((ks / 4) * (MT::NOTH * CFG::OTH_SUB_BYTES) + (ks % 4) * 32) >> 4;
                        if (from_tm) umma_ts_lo(sc_base + acc * TN, tmem_own + ks * 8, b + bo, idesc, (accumulate || ks > 0) ? 1u : 0u);
                        else umma_ss_lo(sc_base + acc * TN, a + ao, b + bo, idesc, (accumulate || ks > 0) ? 1u : 0u);
                    }
                }
            };
            // output-shaped product: out[128, DPAD] (+)= operand[oper] * other[slot_b]; the operand is
            // read from tensor memory (8 columns per 16-element K step), the swept tile MN-major
            // from shared memory
            auto out_mma = [&](uint32_t op_base, int out, int oper, int slot_b, uint32_t stage16, bool accumulate) {
                // all DPAD output columns in one instruction: at head dim 128 the second 64 columns come
                // from the swept tensor's second sub-tile, one `leading byte offset` further on
                constexpr uint32_t idesc = umma_idesc(fmt, fmt, DPAD, true);
                constexpr uint32_t lbo16 = (KSUB > 1) ? ((MT::NOTH * CFG::OTH_SUB_BYTES) >> 4) : 1u;
                const uint32_t a = op_base + oper * CFG::OPER_COLS_EACH;
                const uint32_t b = (stage16 - 0x10000u) + (lbo16 << 16) + ((slot_b * CFG::OTH_SUB_BYTES) >> 4);
                if (elect_one()) {
                    #pragma unroll
                    for (int ks = 0; ks < TN / 16; ++ks)
                        umma_ts_lo(tmem_out + out * DPAD, a + ks * 8, b + ((ks * 2048) >> 4), idesc,
                                   (accumulate || ks > 0) ? 1u : 0u);
                }
            };
            using NS1 = IntTag<1>;
            using NS2 = IntTag<2>;

            BOB_PH_DECL
#ifdef BOB_TRACE
            const int tr_role = score_role ? 1 : 2;
#endif
            // scores of an item's tile `it` (pointwise group it % NG: a function of the item alone, so that
            // which group sums which tiles, and with it the rounding of the result, does not depend on
            // the items this CTA happened to take before), whose swept tiles sit in pipeline stage
            // `stage` (use number `round`); j = score rounds issued for that group so far
            int n_sc0 = 0, n_sc1 = 0;
            auto issue_scores = [&](int it, int stage, int round) -> bool {
                const uint32_t s = oth16 + ((stage * CFG::OTH_STAGE_BYTES) >> 4);
                const int g = it % NG;
                int& n_sc_g = (g == 0) ? n_sc0 : n_sc1;
                const int j = n_sc_g++;
                const uint32_t sc = tmem + g * CFG::SC_COLS;
                BOB_PH(7)
                if (!__all_sync(0xffffffffu, mbar_wait(bar_full(stage), round & 1))) { give_up(kStatusTimeoutMma); return false; }
                BOB_PH(0)
                if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(bar_sc_empty(g), (j - 1) & 1))) { give_up(kStatusTimeoutMma); return false; }
                BOB_PH(1)
                tc_fence_after_sync();
                if constexpr (MODE == kFwd) {
                    score_mma(NS1{}, sc, 0, 0, 0, s, false);
                } else if constexpr (MODE == kBwd1Row || MODE == kBwd1Col) {
                    score_mma(NS1{}, sc, 0, 0, 0, s, false);     // S  = Q K^T      | S^T  = K Q^T
                    score_mma(NS1{}, sc, 1, 1, 1, s, false);     // dP = dO V^T     | dP^T = V dO^T
                } else if constexpr (MODE == kBwd2Row) {
                    // own: Q, dO, uQ;  swept: K, uK, V, uV;  accumulators: S, F, dP, C
                    if (has_uk) score_mma(NS2{}, sc, 0, 0, 0, s, false);      // S | F  = Q [K; uK]^T
                    else          score_mma(NS1{}, sc, 0, 0, 0, s, false);      // S      = Q K^T
                    if (!CFG::SPLIT_SC && has_uq) score_mma(NS1{}, sc, 1, 2, 0, s, has_uk);   // F     += uQ K^T
                    if (has_uv) score_mma(NS2{}, sc, 2, 1, 2, s, false);      // dP | C = dO [V; uV]^T
                    else          score_mma(NS1{}, sc, 2, 1, 2, s, false);      // dP     = dO V^T
                    if constexpr (CFG::SPLIT_SC) {
                        if (elect_one()) umma_commit(bar_sc_part(g));           // S, dP, C are complete
                        if (has_uq) score_mma(NS1{}, sc, 1, 2, 0, s, has_uk);   // F     += uQ K^T
                    }
                } else {
                    // own: K, V, uK, uV;  swept: Q, uQ, dO;  accumulators: S^T, F^T, dP^T, C^T
                    if (has_uq) score_mma(NS2{}, sc, 0, 0, 0, s, false);      // S^T | F^T = K [Q; uQ]^T
                    else          score_mma(NS1{}, sc, 0, 0, 0, s, false);      // S^T       = K Q^T
                    if (has_uk) score_mma(NS1{}, sc, 1, 2, 0, s, has_uq);   // F^T      += uK Q^T
                    score_mma(NS1{}, sc, 2, 1, 2, s, false);                    // dP^T      = V dO^T
                    if (has_uv) score_mma(NS1{}, sc, 3, 3, 2, s, false);      // C^T       = uV dO^T
                }
                if (elect_one()) umma_commit(bar_sc_full(g));
                BOB_PH(2)
                return true;
            };

            int cnt = 0;                              // swept tiles handled so far, over all items
            int stage = 0, round = 0;                 // pipeline stage of tile `cnt`, and cnt / NSTAGE
            int n_out0 = 0, n_out1 = 0;               // output rounds issued so far, per pointwise group
            int n_live = 0;                           // items with at least one tile handled so far
            bool ok = true;
            for (int k_item = 0; ok; ++k_item) {
            const Work wk = follow_ring(k_item);
            const int item = wk.item;
            if (item == -2) give_up(kStatusTimeoutMma);
            if (item < 0) break;
            const Item w = decode(item);
            BOB_ITEM_LOCALS(w, wk)
            if (total == 0) continue;
            int n_out = 0;                            // output rounds of this item
            // output products of the item's tile `it`, whose swept tiles sit in pipeline stage `st`
            auto issue_outputs = [&](int it, int st) -> bool {
                const uint32_t s = oth16 + ((st * CFG::OTH_STAGE_BYTES) >> 4);
                const int g = it % NG;
                const uint32_t ob = tmem_oper + g * CFG::OPER_COLS;
                int& n_out_g = (g == 0) ? n_out0 : n_out1;
                BOB_PH(7)
                if (!__all_sync(0xffffffffu, mbar_wait(bar_op_full(g), n_out_g & 1))) { give_up(kStatusTimeoutMma); return false; }
                // the first products of an item overwrite the output accumulators: the pointwise
                // threads must have read out the previous item's
                if (n_out == 0 && n_live > 0 &&
                    !__all_sync(0xffffffffu, mbar_wait(bar_out_free, (n_live - 1) & 1))) { give_up(kStatusTimeoutMma); return false; }
                ++n_out_g;
                BOB_PH(3)
                tc_fence_after_sync();
                const bool acc = n_out > 0;
                if constexpr (MODE == kFwd) {
                    out_mma(ob, g, 0, 1, s, n_out >= NG);               // O_g += P V (group g's own accumulator)
                } else if constexpr (MODE == kBwd1Row) {
                    out_mma(ob, 0, 0, 0, s, acc);                       // dQ += dS K
                    if (p.pk) out_mma(ob, 1, 1, 0, s, acc);             // PK += P K
                } else if constexpr (MODE == kBwd1Col) {
                    out_mma(ob, 0, 1, 0, s, acc);                       // dK += dS^T Q
                    out_mma(ob, 1, 0, 1, s, acc);                       // dV += P^T dO
                } else if constexpr (MODE == kBwd2Row) {
                    // operands: P, P*F, P*T, dS;  swept: K, uK, V, uV;  outputs: dObar, Omega
                    if (has_uv) out_mma(ob, 0, 0, 3, s, acc);         // dObar += P uV
                    out_mma(ob, 0, 1, 2, s, acc || has_uv);           // dObar += (P*F) V
                    out_mma(ob, 1, 2, 0, s, acc);                       // Omega += (P*T) K
                    if (has_uk) out_mma(ob, 1, 3, 1, s, true);        // Omega += dS uK
                } else {
                    // operands: Sbar^T, dS^T, (P*(F-alpha))^T;  outputs: Kbar, Vbar
                    out_mma(ob, 0, 0, 0, s, acc);                       // Kbar += Sbar^T Q
                    if (has_uq) out_mma(ob, 0, 1, 1, s, true);        // Kbar += dS^T uQ
                    out_mma(ob, 1, 2, 2, s, acc);                       // Vbar += (P*(F-alpha))^T dO
                }
                // operands consumed; and the swept tiles of this stage are free again (the score
                // products that read them finished before these operands could be formed)
                if (elect_one()) { umma_commit(bar_op_empty(g)); umma_commit(bar_empty(st)); }
                ++n_out;
                BOB_PH(4)
                return true;
            };
            if constexpr (CFG::TWO_MMA) {
                if (score_role) {
                    // the item's own tiles have landed (the TMA warp loads them once the previous item's
                    // last products have finished)
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_own, n_live & 1));
                    if constexpr (CFG::OWN_TM) ok = ok && __all_sync(0xffffffffu, mbar_wait(bar_own_tm, n_live & 1));
                    if (!ok) give_up(kStatusTimeoutMma);
                    tc_fence_after_sync();
                    for (int it = 0; ok && it < total; ++it) {
                        ok = issue_scores(it, stage, round);
                        if (++stage == NSTAGE) { stage = 0; ++round; }
                    }
                } else {
                    for (int it = 0; ok && it < total; ++it) {
                        ok = issue_outputs(it, stage);
                        if (++stage == NSTAGE) { stage = 0; ++round; }
                    }
                    // all products of the item have finished: its own tiles may be replaced, its output
                    // accumulators read
                    if (elect_one()) umma_commit(bar_done);
                }
            } else {
                // One warp issues both kinds: the score products run LOOK tiles ahead of the output
                // products (with two pointwise groups a group's next scores are issued as soon as it has
                // read the current ones; otherwise one tile ahead).
                ok = __all_sync(0xffffffffu, mbar_wait(bar_own, n_live & 1));
                if (!ok) give_up(kStatusTimeoutMma);
                constexpr int LOOK = (MODE == kFwd) ? NG : 1;
                int sc_it = 0, sc_stage = stage, sc_round = round;     // next tile to issue scores for
                auto scores_upto = [&](int last) {
                    while (ok && sc_it < total && sc_it <= last) {
                        ok = issue_scores(sc_it, sc_stage, sc_round);
                        ++sc_it;
                        if (++sc_stage == NSTAGE) { sc_stage = 0; ++sc_round; }
                    }
                };
                scores_upto(LOOK - 1);
                for (int it = 0; ok && it < total; ++it) {
                    scores_upto(it + LOOK);
                    if (!ok) break;
                    ok = issue_outputs(it, stage);
                    if (++stage == NSTAGE) { stage = 0; ++round; }
                }
                if (elect_one()) umma_commit(bar_done);
            }
            cnt += total;
            ++n_live;
            }   // items
            BOB_PH_FLUSH(12, lane == 0)
        }
    }
    } else {
        // =========================== pointwise threads =======================================
        if constexpr (CFG::REBALANCE) setmaxnreg_inc<CFG::REGS_POINTWISE>();
        const int grp = tid / GP;                // pointwise group: takes iterations grp, grp + NG, ...
        const int gtid = tid % GP;
        const int row = gtid & 127;              // own row inside the tile == tensor-memory lane
        const int sp = gtid >> 7;                // which 16-column slice of every score tile
        const int col0 = sp * CW;                // my first column inside a swept tile
        const uint32_t tlane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);   // my lane, column 0
        const uint32_t tsc = tlane + grp * CFG::SC_COLS;                                  // my group's scores
        const float c_exp = p.scale * kLog2e;

        // where my 16 columns (8 packed words) of operand k go in tensor memory
        const uint32_t op_taddr = tlane + NG * CFG::SC_COLS + grp * CFG::OPER_COLS + (col0 >> 1);

        // Synchronise the pointwise threads through an mbarrier so that the wait is bounded.
        uint32_t pw_phase = 0;
        auto pw_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pw(grp));
            const bool r = __all_sync(0xffffffffu, mbar_wait(bar_pw(grp), pw_phase));
            pw_phase ^= 1u;
            if (!r) give_up(kStatusTimeoutPw);
            return r;
        };
        // Every lane of a warp takes the same decision after a wait, so that the warp-wide
        // tensor-memory loads that follow are never executed by part of a warp.
        auto pw_wait = [&](uint32_t bar, uint32_t parity) -> bool {
            const bool r = __all_sync(0xffffffffu, mbar_wait(bar, parity));
            if (!r) give_up(kStatusTimeoutPw);
            return r;
        };
        bool ok = true;
        uint32_t pw_all_phase = 0;               // phase of the all-groups barrier
        int cnt = 0;                             // swept tiles seen so far, over all items
        int stage = 0, round = 0;                // pipeline stage of tile `cnt`, and cnt / NSTAGE
        int n_op = 0;                            // operand rounds my group has written so far
        int n_live = 0;                          // items with at least one tile finished so far
        int n_items_done = 0;                    // items finished so far, with or without tiles
        BOB_PH_DECL
#ifdef BOB_TRACE
        const int tr_role = (warp == 0) ? 0 : 4;     // only warp 0 records (role 4 is dropped)
#endif

        for (int k_item = 0; ok; ++k_item) {
            const Work wk = follow_ring(k_item);
            const int item = wk.item;
            if (item == -2) give_up(kStatusTimeoutPw);
            if (item < 0) break;
        const Item w = decode(item);
        BOB_ITEM_LOCALS(w, wk)
        const int own_idx = own0 + row;
        const bool own_ok = own_idx < n_own;
        const long long row_stat = ((long long)batch * p.Hq + head) * p.Nq + own_idx;   // row-owned only

        // per-row state (row-owned modes): -lse*log2e and -delta of my row
        float nL2 = 0.f, ndlt = 0.f;
        float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);   // row sums alpha, ecirc
        // forward: my group's online softmax over the tiles it takes.  m_ref is the exponent reference
        // (log2 units): it follows the running maximum only when that has grown by more than 8, so
        // that the output accumulator rarely needs rescaling; probabilities stay below 2^8.
        float m_ref = -1e30f, l_run = 0.f;
        int n_op_item = 0;                       // tiles my group has finished in this item
        (void)m_ref; (void)l_run; (void)n_op_item;

        if constexpr (MODE == kBwd1Row) {
            // delta = rowsum(dO * out).  The tile's rows are read cooperatively, 16 bytes per thread with
            // the lanes of a row next to each other (whole 128-byte lines per request), each thread sums
            // its eight products and the lanes of a row combine by shuffles.
            static_assert(NG == 1, "the cooperative delta uses the single group's barrier");
            constexpr int CH = DPAD / 8;                 // 16-byte chunks per row
            const uint16_t* g_out = static_cast<const uint16_t*>(p.out) + (long long)batch * p.out_sb + (long long)head * p.out_sh + (long long)own0 * p.out_sn;
            const uint16_t* g_do = static_cast<const uint16_t*>(p.dO) + (long long)batch * p.dO_sb + (long long)head * p.dO_sh + (long long)own0 * p.dO_sn;
            #pragma unroll
            for (int k = 0; k < 128 * CH / NPW; ++k) {
                const int id = tid + NPW * k, r = id / CH, c = id % CH;
                float part = 0.f;
                if (own0 + r < n_own && c * 8 < p.D) {
                    float a[8], b[8];
                    unpack8_as_float<BF16>(*reinterpret_cast<const uint4*>(g_out + (long long)r * p.out_sn + c * 8), a);
                    unpack8_as_float<BF16>(*reinterpret_cast<const uint4*>(g_do + (long long)r * p.dO_sn + c * 8), b);
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) part = fmaf(a[i], b[i], part);
                }
                #pragma unroll
                for (int m = CH / 2; m >= 1; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
                if (c == 0) red_buf[r] = part;
            }
            ok = pw_sync();
            const float dlt = red_buf[row];
            ok = ok && pw_sync();
            if (grp == 0 && sp == 0 && own_ok) p.delta[row_stat] = dlt;
            ndlt = -dlt;
            if (own_ok) nL2 = -p.lse[row_stat] * kLog2e;
        }
        if constexpr (MODE == kBwd2Row) {
            if (own_ok) { nL2 = -p.lse[row_stat] * kLog2e; ndlt = -p.delta[row_stat]; }
        }
        // Own tile 0 into tensor memory (see SweepConfig::OWN_TM): once the item's own tiles have landed,
        // every thread copies its share of its own row, 16 elements (two 16-byte chunks of the swizzled
        // shared-memory tile = eight packed columns) at a time.  The previous item's products are all
        // finished by now (its epilogue waited for them), so nothing reads the old copy any more.
        if constexpr (CFG::OWN_TM) {
            if (total > 0) {
                ok = pw_wait(bar_own, n_live & 1);
                if (ok) {
                    constexpr int PER = (DPAD / 8) / NSPLIT;             // 16-byte chunks of my row that I copy
                    static_assert(PER % 2 == 0, "two chunks per tensor-memory store");
                    #pragma unroll
                    for (int c = sp * PER; c < (sp + 1) * PER; c += 2) {
                        const uint32_t src = sbase + CFG::OFF_OWN + (c / 8) * (128 * 128);
                        const uint4 lo = ld_shared_v4(src + sw128_offset(row, c % 8));
                        const uint4 hi = ld_shared_v4(src + sw128_offset(row, c % 8 + 1));
                        const uint32_t wds[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                        tmem_st8(tlane + (tmem_own - tmem) + 4 * c, wds);
                    }
                    tmem_wait_st();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_own_tm);
                }
            }
        }
        if constexpr (MODE == kBwd2Row) {
            // my row's pk columns are read when the sweep ends: have them in L2 by then
            constexpr int DCP = DPAD / (NSPLIT * NG);            // fp32 columns per thread, 128 bytes per 32
            const int c0 = (grp * NSPLIT + sp) * DCP;
            #pragma unroll
            for (int c = 0; c < DCP; c += 32)
                if (own_ok && c0 + c < p.D) prefetch_l2(p.pk + (((long long)batch * p.Hq + head) * p.Nq + own_idx) * p.D + c0 + c);
        }
        // epilogue operands staged by the IO warp: 16-byte chunk c of row r sits at chunk position
        // c ^ (r & 7) of its 128-byte line, so that both the row-wise and the chunk-wise accesses are
        // conflict-free
        const uint32_t io_out = sbase + CFG::OFF_IO, io_dq = io_out + 16384;
        const long long tile_row0 = ((long long)batch * p.Hq + head) * p.Nq + own0;   // first row of the contiguous results


        // One swept tile.  FULL: every (row, column) of the tile pair is unmasked and in range.
        auto tile_body = [&](auto full_tag, int it, int tile, int outer, int stage, int round) -> bool {
            constexpr bool FULL = decltype(full_tag)::value;
            const int oth0 = tile * TN;

            BOB_PH(7)
            if constexpr (COL) {
                // the swept tile's row statistics were staged by the producer warp
                if (!pw_wait(bar_stat(stage), round & 1)) return false;
            }
            if (!pw_wait(CFG::SPLIT_SC ? bar_sc_part(grp) : bar_sc_full(grp), n_op & 1)) return false;     // my group's n_op-th tile
            BOB_PH(0)
            tc_fence_after_sync();

            // ---- which of my 16 columns are unmasked: bits [mlo, mhi] of vmask ----------------
            // dist = query position - key position; unmasked iff in range and, when causal,
            // 0 <= dist (< window)
            // Up to 64 columns per thread: a bit mask; more (forward, 128): the range itself.
            using mask_t = typename std::conditional<(CW > 32), unsigned long long, uint32_t>::type;
            constexpr mask_t kAllCols = (CW >= 64) ? ~mask_t(0) : ((CW == 32) ? mask_t(0xFFFFFFFFu) : mask_t(0xFFFFu));
            mask_t vmask = kAllCols;
            int mlo = 0, mhi = CW - 1;
            if constexpr (!FULL) {
                mhi = min(CW - 1, n_oth - (oth0 + col0) - 1);
                if (causal) {
                    if constexpr (!COL) {
                        const int d0 = own_idx + doff - (oth0 + col0);       // dist falls with the column
                        mhi = min(mhi, d0);
                        if (window > 0) mlo = max(mlo, d0 - window + 1);
                    } else {
                        const int d0 = (oth0 + col0) + doff - own_idx;       // dist grows with the column
                        mlo = max(mlo, -d0);
                        if (window > 0) mhi = min(mhi, window - 1 - d0);
                    }
                }
                if (!own_ok) { mlo = 1; mhi = 0; }
                if constexpr (CW <= 64)
                    vmask = (mhi >= mlo) ? ((kAllCols >> (CW - 1 - mhi)) & (kAllCols << mlo)) : mask_t(0);
            }
            auto valid = [&](int c) -> bool {        // column c of mine is unmasked (c is a constant after unrolling)
                if constexpr (FULL) return true;
                else if constexpr (CW <= 64) return ((vmask >> c) & 1) != 0;
                else return c >= mlo && c <= mhi;
            };
            (void)valid; (void)vmask;

            if constexpr (MODE == kFwd) {
                // One thread owns a whole row of the tile.
                float s_[CW];
                #pragma unroll
                for (int h = 0; h < CW / 16; ++h) tmem_ld16(tsc + 16 * h, s_ + 16 * h);
                tmem_wait_ld();
                BOB_PH(1)
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sc_empty(grp));
                // largest unmasked score of my row in this tile (the scale is positive)
                float mr4[4] = {-3.0e38f, -3.0e38f, -3.0e38f, -3.0e38f};     // four chains, for instruction-level parallelism
                #pragma unroll
                for (int c = 0; c < CW; ++c)
                    mr4[c & 3] = fmaxf(mr4[c & 3], valid(c) ? s_[c] : -3.0e38f);
                const float mr = fmaxf(fmaxf(mr4[0], mr4[1]), fmaxf(mr4[2], mr4[3]));
                const float mt = fmaxf(mr * c_exp, -1e30f);
                // move the reference only when the maximum has outgrown it; the whole warp then
                // rescales its rows of the output accumulator (factor 1 where nothing changed)
                const bool grow = mt > m_ref + 8.f;
                const bool rescale = __any_sync(0xffffffffu, grow) && n_op_item > 0;
                float factor = 1.f;
                if (grow) { factor = fast_exp2(m_ref - mt); m_ref = mt; }
                l_run *= factor;
                BOB_PH(2)
                // My group's previous product must have consumed its operand and finished with the
                // accumulator before I touch either.  With 128 columns the probabilities go to tensor
                // memory 16 at a time (registers), so the wait comes first; with 64 they are all
                // formed before the wait.
                constexpr bool WAIT_FIRST = CW > 64;
                uint32_t wall[WAIT_FIRST ? 1 : CW / 2];
                if constexpr (WAIT_FIRST) {
                    if (n_op > 0 && !pw_wait(bar_op_empty(grp), (n_op - 1) & 1)) return false;
                }
                BOB_PH(3)
                auto rescale_rows = [&]() {
                    tc_fence_after_sync();
                    const uint32_t tacc = tlane + NG * (CFG::SC_COLS + CFG::OPER_COLS) + grp * DPAD;
                    #pragma unroll
                    for (int ch = 0; ch < DPAD / 16; ++ch) {
                        float t[16];
                        uint32_t u[16];
                        tmem_ld16(tacc + 16 * ch, t);
                        tmem_wait_ld();
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) u[i] = __float_as_uint(t[i] * factor);
                        tmem_st8(tacc + 16 * ch, u);
                        tmem_st8(tacc + 16 * ch + 8, u + 8);
                    }
                };
                if (WAIT_FIRST && rescale) rescale_rows();
                // probabilities relative to the reference, 16 columns at a time straight into tensor memory
                const float nm = -m_ref;
                float2 sum4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
                const float2 cexp2 = make_float2(c_exp, c_exp), nm2 = make_float2(nm, nm);
                #pragma unroll
                for (int h = 0; h < CW / 16; ++h) {
                    uint32_t w0[8];
                    #pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int c = 16 * h + 2 * k;
                        const float2 x = __ffma2_rn(make_float2(s_[c], s_[c + 1]), cexp2, nm2);
                        float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                        if constexpr (!FULL) {
                            pr.x = valid(c) ? pr.x : 0.f;
                            pr.y = valid(c + 1) ? pr.y : 0.f;
                        }
                        sum4[k & 3] = __fadd2_rn(sum4[k & 3], pr);
                        w0[k] = pack2<BF16>(pr.x, pr.y);
                        if constexpr (!WAIT_FIRST) wall[8 * h + k] = w0[k];
                    }
                    if constexpr (WAIT_FIRST) tmem_st8(op_taddr + 8 * h, w0);
                }
                {
                    const float2 t = __fadd2_rn(__fadd2_rn(sum4[0], sum4[1]), __fadd2_rn(sum4[2], sum4[3]));
                    l_run += t.x + t.y;
                }
                if constexpr (!WAIT_FIRST) {
                    if (n_op > 0 && !pw_wait(bar_op_empty(grp), (n_op - 1) & 1)) return false;
                    if (rescale) rescale_rows();
                    #pragma unroll
                    for (int h = 0; h < CW / 16; ++h) tmem_st8(op_taddr + 8 * h, wall + 8 * h);
                }
                ++n_op_item;
            } else {
                // accumulator order: S, dP (first backward) or S, F, dP, C (second backward).
                // My CW columns are taken in rounds of RW.  LOAD_ALL (second backward, 32 columns per
                // thread): every round's loads are issued at once and the score accumulators are
                // handed back before any arithmetic, so that the next tile's score products run
                // under this tile's arithmetic.  Otherwise one round is in registers at a time and
                // the accumulators are handed back when the last round has been loaded.  Each round's
                // packed operands go to tensor memory as soon as they are formed.
                constexpr int R = CW / RW;
                constexpr bool LOAD_ALL = CFG::REBALANCE;
                constexpr int NB = LOAD_ALL ? R : 1;
                const float2 cexp2 = make_float2(c_exp, c_exp);
                const float2 scale2 = make_float2(p.scale, p.scale);
                const bool has_f = BWD2 && (ALLT || has_uq || has_uk);
                const bool has_c = BWD2 && (ALLT || has_uv);
                float in_s[NB][RW], in_dp[NB][RW], in_f[NB][RW], in_c[NB][RW];
                // part: 0 = every accumulator, 1 = all but F, 2 = F alone
                auto issue_loads = [&](int r, int b, int part = 0) {
                    const int cb = col0 + RW * r;
                    auto ld = [&](uint32_t addr, float* dst) {
                        if constexpr (RW == 16) tmem_ld16(addr, dst); else tmem_ld8(addr, dst);
                    };
                    if (part != 2) {
                        ld(tsc + 0 * TN + cb, in_s[b]);
                        ld(tsc + (BWD2 ? 2 : 1) * TN + cb, in_dp[b]);
                    }
                    if constexpr (BWD2) {
                        if (part != 1 && has_f) ld(tsc + 1 * TN + cb, in_f[b]);
                        if (part != 2 && has_c) ld(tsc + 3 * TN + cb, in_c[b]);
                    }
                };
                auto release_scores = [&]() {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_sc_empty(grp));
                };
                if constexpr (CFG::SPLIT_SC) {
                    // S, dP and C now; F once its second term has been added (the loads above are on
                    // their way while that product runs)
                    #pragma unroll
                    for (int r = 0; r < R; ++r) issue_loads(r, r, 1);
                    // (forming the probabilities here as well, while that product runs, measured slower:
                    // 0.311 against 0.260 ms)
                    if (!pw_wait(bar_sc_full(grp), n_op & 1)) return false;
                    tc_fence_after_sync();
                    #pragma unroll
                    for (int r = 0; r < R; ++r) issue_loads(r, r, 2);
                } else if constexpr (LOAD_ALL) {
                    #pragma unroll
                    for (int r = 0; r < R; ++r) issue_loads(r, r);
                } else {
                    issue_loads(0, 0);
                }
                constexpr bool STORE_LATE = false;       // (all rounds' arithmetic before the wait and the stores: measured slower)
                uint32_t wbuf[STORE_LATE ? R : 1][4][RW / 2];
                auto store_round = [&](int half) {
                    const uint32_t dst = op_taddr + (RW / 2) * half;     // RW / 2 packed words per round
                    auto st = [&](uint32_t addr, const uint32_t* w) {
                        if constexpr (RW == 16) tmem_st8(addr, w); else tmem_st4(addr, w);
                    };
                    const int wb = STORE_LATE ? half : 0;
                    st(dst + 0 * CFG::OPER_COLS_EACH, wbuf[wb][0]);
                    if constexpr (MT::NOPER > 1) st(dst + 1 * CFG::OPER_COLS_EACH, wbuf[wb][1]);
                    if constexpr (MT::NOPER > 2) st(dst + 2 * CFG::OPER_COLS_EACH, wbuf[wb][2]);
                    if constexpr (MT::NOPER > 3) st(dst + 3 * CFG::OPER_COLS_EACH, wbuf[wb][3]);
                };
                #pragma unroll
                for (int half = 0; half < R; ++half) {            // `half` = round of RW columns
                    const int cb = col0 + RW * half;
                    const int b = LOAD_ALL ? half : 0;
                    if (!LOAD_ALL || half == 0) {
                        tmem_wait_ld();
                        BOB_PH(1)
                        if (LOAD_ALL || half + 1 == R) release_scores();
                    }
                    float* s_ = in_s[b];
                    float* dp_ = in_dp[b];
                    float* f_ = in_f[b];
                    float* cc_ = in_c[b];
                    if constexpr (BWD2) {
                        if (!has_f) {
                            #pragma unroll
                            for (int c = 0; c < RW; ++c) f_[c] = 0.f;
                        }
                        if (!has_c) {
                            #pragma unroll
                            for (int c = 0; c < RW; ++c) cc_[c] = 0.f;
                        }
                    }
                    uint32_t* w0 = wbuf[STORE_LATE ? half : 0][0];
                    uint32_t* w1 = wbuf[STORE_LATE ? half : 0][1];
                    uint32_t* w2 = wbuf[STORE_LATE ? half : 0][2];
                    uint32_t* w3 = wbuf[STORE_LATE ? half : 0][3];
                    (void)w1; (void)w2; (void)w3;
                    // negated statistics of these columns (column-owned modes), four columns per load
                    const float4* sb4 = reinterpret_cast<const float4*>(stat_buf + stage * 4 * TN + cb);
                    // The arithmetic of four columns (two packed pairs) in two steps, so that the
                    // exponentials of the next four columns can be issued before the multiplications of
                    // these four: probabilities first, then everything that needs them.
                    struct Grp { float2 pr[2]; float4 q_dl, q_al, q_ec; };
                    auto exps = [&](int c4) {
                        Grp gq;
                        float4 q_l2;
                        if constexpr (COL) {
                            q_l2 = sb4[c4]; gq.q_dl = sb4[TN / 4 + c4];
                            if constexpr (MODE == kBwd2Col) { gq.q_al = sb4[2 * (TN / 4) + c4]; gq.q_ec = sb4[3 * (TN / 4) + c4]; }
                        }
                        #pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int c = 4 * c4 + 2 * h;
                            const int mc = RW * half + c;          // bit index in vmask
                            float2 nl2;
                            if constexpr (COL) nl2 = h ? make_float2(q_l2.z, q_l2.w) : make_float2(q_l2.x, q_l2.y);
                            else nl2 = make_float2(nL2, nL2);
                            const float2 x = __ffma2_rn(make_float2(s_[c], s_[c + 1]), cexp2, nl2);
                            float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                            if constexpr (!FULL) {
                                pr.x = ((vmask >> mc) & 1u) ? pr.x : 0.f;
                                pr.y = ((vmask >> (mc + 1)) & 1u) ? pr.y : 0.f;
                            }
                            gq.pr[h] = pr;
                        }
                        return gq;
                    };
                    auto math = [&](int c4, const Grp& gq) {
                        #pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int c = 4 * c4 + 2 * h;          // columns c, c + 1 of this round
                            const int wi = c >> 1;                 // packed word index inside this round
                            float2 ndl, nal, nec;
                            (void)nal; (void)nec;
                            if constexpr (COL) {
                                ndl = h ? make_float2(gq.q_dl.z, gq.q_dl.w) : make_float2(gq.q_dl.x, gq.q_dl.y);
                                if constexpr (MODE == kBwd2Col) {
                                    nal = h ? make_float2(gq.q_al.z, gq.q_al.w) : make_float2(gq.q_al.x, gq.q_al.y);
                                    nec = h ? make_float2(gq.q_ec.z, gq.q_ec.w) : make_float2(gq.q_ec.x, gq.q_ec.y);
                                }
                            } else {
                                ndl = make_float2(ndlt, ndlt);
                            }
                            const float2 pr = gq.pr[h];
                            const float2 dps = __fadd2_rn(make_float2(dp_[c], dp_[c + 1]), ndl);
                            if constexpr (MODE == kBwd1Row) {
                                const float2 ds = __fmul2_rn(pr, dps);
                                w0[wi] = pack2<BF16>(ds.x, ds.y);                         // dS
                                w1[wi] = pack2<BF16>(pr.x, pr.y);                         // P
                            } else if constexpr (MODE == kBwd1Col) {
                                const float2 ds = __fmul2_rn(pr, dps);
                                w0[wi] = pack2<BF16>(pr.x, pr.y);                         // P^T
                                w1[wi] = pack2<BF16>(ds.x, ds.y);                         // dS^T
                            } else if constexpr (MODE == kBwd2Row) {
                                const float2 f = __fmul2_rn(make_float2(f_[c], f_[c + 1]), scale2);
                                const float2 t = __ffma2_rn(f, dps, make_float2(cc_[c], cc_[c + 1]));
                                const float2 pf = __fmul2_rn(pr, f);
                                const float2 pt = __fmul2_rn(pr, t);
                                const float2 ds = __fmul2_rn(pr, dps);
                                acc_a = __fadd2_rn(acc_a, pf);
                                acc_b = __fadd2_rn(acc_b, pt);
                                w0[wi] = pack2<BF16>(pr.x, pr.y);                         // P
                                w1[wi] = pack2<BF16>(pf.x, pf.y);                         // P*F
                                w2[wi] = pack2<BF16>(pt.x, pt.y);                         // P*T
                                w3[wi] = pack2<BF16>(ds.x, ds.y);                         // dS
                            } else {
                                // T - alpha (dP - delta) - ecirc = (F - alpha) (dP - delta) + (C - ecirc)
                                const float2 fa = __ffma2_rn(make_float2(f_[c], f_[c + 1]), scale2, nal);   // F - alpha
                                const float2 u = __ffma2_rn(fa, dps, __fadd2_rn(make_float2(cc_[c], cc_[c + 1]), nec));
                                const float2 sbar = __fmul2_rn(pr, u);
                                const float2 ds = __fmul2_rn(pr, dps);
                                const float2 ph = __fmul2_rn(pr, fa);
                                w0[wi] = pack2<BF16>(sbar.x, sbar.y);                     // Sbar^T
                                w1[wi] = pack2<BF16>(ds.x, ds.y);                         // dS^T
                                w2[wi] = pack2<BF16>(ph.x, ph.y);                         // (P*(F-alpha))^T
                            }
                        }
                    };
                    #pragma unroll
                    for (int c4 = 0; c4 < RW / 4; ++c4) math(c4, exps(c4));
                    if constexpr (!LOAD_ALL) {
                        if (half + 1 < R) issue_loads(half + 1, 0);
                    }
                    if (STORE_LATE ? (half + 1 == R) : (half == 0)) {
                        BOB_PH(2)
                        // the previous tile's output products must have consumed its operands
                        if (n_op > 0 && !pw_wait(bar_op_empty(grp), (n_op - 1) & 1)) return false;
                        BOB_PH(3)
                    }
                    if constexpr (STORE_LATE) {
                        if (half + 1 == R) {
                            #pragma unroll
                            for (int r = 0; r < R; ++r) store_round(r);
                        }
                    } else {
                        store_round(half);
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_op_full(grp));
            ++n_op;
            BOB_PH(4)
            return true;
        };

        BOB_PH(6)
        {
            // swept tiles [full_lo, full_hi) pair with my own tile entirely unmasked and in range
            int full_lo = 0, full_hi = 0;
            if (own0 + 127 < n_own) {
                long long lo = 0, hi = n_oth / TN;                  // tiles that lie inside the tensor
                if (causal) {
                    // oldest and newest own position of the tile pair against the swept tile's extremes
                    if constexpr (!COL) {
                        hi = min(hi, ((long long)own0 + doff + 1) / TN);                          // dist >= 0 everywhere
                        if (window > 0) {
                            const long long x = (long long)own0 + 127 + doff - window;            // last swept position with dist >= window
                            lo = max(lo, x < 0 ? 0LL : (x + TN) / TN);
                        }
                    } else {
                        const long long a = (long long)own0 + 127 - doff;                         // first swept position with dist >= 0
                        lo = max(lo, a <= 0 ? 0LL : (a + TN - 1) / TN);
                        if (window > 0) {
                            const long long b = (long long)own0 - doff + window;                  // one past the last with dist < window
                            hi = min(hi, b <= 0 ? 0LL : b / TN);
                        }
                    }
                }
                if (hi > lo) { full_lo = (int)lo; full_hi = (int)hi; }
            }
            int tile = t_lo + (T > 0 ? lin0 % T : 0), outer = T > 0 ? lin0 / T : 0;
            for (int it = 0; ok && it < total; ++it) {
                if (it % NG == grp) {                    // my group's turn
                    // is the whole 128 x TN tile pair unmasked and inside both tensors?  (uniform per CTA)
                    const bool full = tile >= full_lo && tile < full_hi;
                    ok = full ? tile_body(BoolTag<true>{}, it, tile, outer, stage, round)
                              : tile_body(BoolTag<false>{}, it, tile, outer, stage, round);
                }
                if (++tile == t_hi) { tile = t_lo; ++outer; }
                if (++stage == NSTAGE) { stage = 0; ++round; }
            }
            cnt += total;
        }

        // ---- epilogue ------------------------------------------------------------------------
        float fwd_k0 = 0.f, fwd_k1 = 0.f;            // forward: weights of the two groups' accumulators
        if constexpr (MODE == kFwd) {
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                // both groups' (reference, sum) of my row -> the row's normaliser and lse.  The
                // exchange buffer alternates between items: a thread may start the next item while
                // another still reads this one's values.
                float* xb = red_buf + (n_items_done & 1) * (2 * NG * 128);
                xb[grp * 128 + row] = m_ref;
                xb[(NG + grp) * 128 + row] = l_run;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pw_all);
                ok = pw_wait(bar_pw_all, pw_all_phase);
                pw_all_phase ^= 1u;
                const float m0 = xb[row], m1 = xb[128 + row];
                const float m = fmaxf(m0, m1);
                const float a0 = fast_exp2(m0 - m), a1 = fast_exp2(m1 - m);
                const float l = a0 * xb[2 * 128 + row] + a1 * xb[3 * 128 + row];
                const float inv = (l > 0.f) ? 1.f / l : 0.f;
                // a group that took no tile of this item has never written its accumulator
                fwd_k0 = (total >= 1) ? a0 * inv : 0.f;
                fwd_k1 = (total >= 2) ? a1 * inv : 0.f;
                if (grp == 0 && own_ok) p.lse[row_stat] = (l > 0.f) ? (m + log2f(l)) * kLn2 : -INFINITY;
            }
        }
        // my row's pk columns, on their way while the row sums are combined and the last products finish
        constexpr int PKN = CFG::STAGED_IO ? DPAD / (NSPLIT * NG) : 1;
        float pk_pre[PKN];
        if constexpr (CFG::STAGED_IO) {
            const int col_pk = (grp * NSPLIT + sp) * PKN;
            const float4* src = reinterpret_cast<const float4*>(p.pk + (tile_row0 + row) * p.D + col_pk);
            #pragma unroll
            for (int i = 0; i < PKN / 4; ++i) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (own_ok && col_pk + 4 * i < p.D) t = __ldg(src + i);
                pk_pre[4 * i] = t.x; pk_pre[4 * i + 1] = t.y; pk_pre[4 * i + 2] = t.z; pk_pre[4 * i + 3] = t.w;
            }
        }
        (void)pk_pre;
        float alpha = 0.f, ecirc = 0.f;
        ok = __all_sync(0xffffffffu, ok);
        if constexpr (MODE == kBwd2Row) {
            constexpr int NPART = NG * NSPLIT;          // every pointwise thread of my row holds a partial sum
            red_buf[(grp * NSPLIT + sp) * 128 + row] = acc_a.x + acc_a.y;
            red_buf[(NPART + grp * NSPLIT + sp) * 128 + row] = acc_b.x + acc_b.y;
            if constexpr (CFG::STAGED_IO) ok = ok && pw_wait(bar_io_full, n_items_done & 1);   // the IO warp has staged out, dQ
            if (ok) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pw_all);
                ok = pw_wait(bar_pw_all, pw_all_phase);
                pw_all_phase ^= 1u;
            }
            #pragma unroll
            for (int k = 0; k < NPART; ++k) { alpha += red_buf[k * 128 + row]; ecirc += red_buf[(NPART + k) * 128 + row]; }
            if (ok && grp == 0 && sp == 0 && own_ok) { p.alpha[row_stat] = alpha; p.ecirc[row_stat] = ecirc; }
        }
        BOB_PH(8)
        if (ok && total > 0) ok = pw_wait(bar_done, n_live & 1);
        tc_fence_after_sync();
        BOB_PH(9)
        if (ok) {
            constexpr int DC = DPAD / (NSPLIT * NG);    // output columns per pointwise thread
            constexpr int NCH = DC / 16;
            const int res_heads = COL ? p.Hkv : p.Hq;
            const long long res_off = (((long long)batch * res_heads + head) * n_own + own_idx) * p.D;
            // All of my accumulator columns come out of tensor memory first (warp-wide loads), so that
            // the MMA warp may start overwriting them for the next item while I combine and store.
            // (With more than two 16-column chunks per thread that would cost too many registers: then
            // the chunks are taken one at a time and the accumulators are released after the last.)
            constexpr bool EARLY = NCH <= 2;
            float acc0[EARLY ? NCH : 1][16], acc1[EARLY ? NCH : 1][16];
            #pragma unroll
            for (int ch = 0; ch < (EARLY ? NCH : 0); ++ch) {
                const int col = (grp * NSPLIT + sp) * DC + 16 * ch;
                if (total > 0 && col < p.D) {
                    tmem_ld16(tlane + NG * (CFG::SC_COLS + CFG::OPER_COLS) + 0 * DPAD + col, acc0[ch]);
                    if constexpr (CFG::NACC > 1) tmem_ld16(tlane + NG * (CFG::SC_COLS + CFG::OPER_COLS) + 1 * DPAD + col, acc1[ch]);
                } else {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) { acc0[ch][i] = 0.f; acc1[ch][i] = 0.f; }
                }
            }
            auto release_outputs = [&]() {
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_out_free);
            };
            bool released = false;
            if (EARLY && total > 0) { release_outputs(); released = true; }
            BOB_PH(10)
            // A piece of a cut item (even split, column-owned modes): park my fp32 partial results,
            // count this piece in, and only if it is the last of its item to finish, add the other
            // pieces' parked partials and go on to store the result.  Nothing waits for anything: a
            // piece is counted after its partials are globally visible.
            bool store_results = true;
            if constexpr (COL && EARLY) {
                if (wk.part != 0 && ok) {
                    const long long span = p.sk_span, s_item = wk.s_item;
                    const int me = (int)blockIdx.x;
                    const int c_first = (int)(s_item / span), c_last = (int)((s_item + w.total - 1) / span);
                    auto slot_of = [&](int c) {          // a CTA's first piece parks in slot 0, a later one in slot 1
                        return (c > c_first || s_item == (long long)c * span) ? 0 : 1;
                    };
                    auto park_at = [&](int c) {
                        return p.sk_park + ((size_t)(2 * c + slot_of(c)) * 2 * 128 + row) * DPAD + (grp * NSPLIT + sp) * DC;
                    };
                    float* mine = park_at(me);
                    #pragma unroll
                    for (int ch = 0; ch < NCH; ++ch) {
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            reinterpret_cast<float4*>(mine + 16 * ch)[i] =
                                make_float4(acc0[ch][4 * i], acc0[ch][4 * i + 1], acc0[ch][4 * i + 2], acc0[ch][4 * i + 3]);
                            reinterpret_cast<float4*>(mine + 128 * DPAD + 16 * ch)[i] =
                                make_float4(acc1[ch][4 * i], acc1[ch][4 * i + 1], acc1[ch][4 * i + 2], acc1[ch][4 * i + 3]);
                        }
                    }
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_pw_all);
                    ok = pw_wait(bar_pw_all, pw_all_phase);
                    pw_all_phase ^= 1u;
                    int* xch = reinterpret_cast<int*>(red_buf);
                    if (tid == 0) xch[0] = atomicAdd(p.sk_flags + item, 1);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_pw_all);
                    ok = ok && pw_wait(bar_pw_all, pw_all_phase);
                    pw_all_phase ^= 1u;
                    store_results = ok && (xch[0] == c_last - c_first);
                    if (store_results) {
                        // Sum every piece's parked partials, my own included, in the order of the CTAs:
                        // the result does not depend on which piece happened to finish last.
                        __threadfence();
                        #pragma unroll
                        for (int ch = 0; ch < NCH; ++ch) {
                            #pragma unroll
                            for (int i = 0; i < 16; ++i) { acc0[ch][i] = 0.f; acc1[ch][i] = 0.f; }
                        }
                        for (int c = c_first; c <= c_last; ++c) {
                            const float* other = park_at(c);
                            #pragma unroll
                            for (int ch = 0; ch < NCH; ++ch) {
                                #pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float4 a = __ldcg(reinterpret_cast<const float4*>(other + 16 * ch) + i);
                                    const float4 b = __ldcg(reinterpret_cast<const float4*>(other + 128 * DPAD + 16 * ch) + i);
                                    acc0[ch][4 * i] += a.x; acc0[ch][4 * i + 1] += a.y; acc0[ch][4 * i + 2] += a.z; acc0[ch][4 * i + 3] += a.w;
                                    acc1[ch][4 * i] += b.x; acc1[ch][4 * i + 1] += b.y; acc1[ch][4 * i + 2] += b.z; acc1[ch][4 * i + 3] += b.w;
                                }
                            }
                        }
                    }
                }
            }
            if (store_results) {
            #pragma unroll
            for (int c = 0; c < DC; c += 16) {
                const int col = (grp * NSPLIT + sp) * DC + c;
                const bool last = (c + 16 >= DC) || (col + 16 >= p.D);
                if (col >= p.D) break;
                float late0[16], late1[16];
                if constexpr (!EARLY) {
                    if (total > 0) {
                        tmem_ld16(tlane + NG * (CFG::SC_COLS + CFG::OPER_COLS) + 0 * DPAD + col, late0);
                        if constexpr (CFG::NACC > 1) tmem_ld16(tlane + NG * (CFG::SC_COLS + CFG::OPER_COLS) + 1 * DPAD + col, late1);
                        if (last) { release_outputs(); released = true; } else tmem_wait_ld();
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) { late0[i] = 0.f; late1[i] = 0.f; }
                    }
                }
                float* a0 = EARLY ? acc0[EARLY ? c / 16 : 0] : late0;
                float* a1 = EARLY ? acc1[EARLY ? c / 16 : 0] : late1;
                if (!own_ok) continue;          // stores are per row
                if constexpr (MODE == kFwd) {
                    // weighted sum of the two groups' accumulators (weight 0: never written, not read)
                    #pragma unroll
                    for (int i = 0; i < 16; ++i)
                        a0[i] = (fwd_k0 != 0.f ? fwd_k0 * a0[i] : 0.f) + (fwd_k1 != 0.f ? fwd_k1 * a1[i] : 0.f);
                    store16_from_float<BF16>(p.res0, res_off + col, a0);
                } else if constexpr (MODE == kBwd1Row) {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) a0[i] *= p.scale;
                    store16_from_float<BF16>(p.res0, res_off + col, a0);                          // dQ
                    if (p.pk) {
                        float4* dst = reinterpret_cast<float4*>(p.pk + res_off + col);            // PK
                        #pragma unroll
                        for (int i = 0; i < 4; ++i)
                            dst[i] = make_float4(a1[4 * i], a1[4 * i + 1], a1[4 * i + 2], a1[4 * i + 3]);
                    }
                } else if constexpr (MODE == kBwd1Col || MODE == kBwd2Col) {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) a0[i] *= p.scale;
                    store16_from_float<BF16>(p.res0, res_off + col, a0);
                    store16_from_float<BF16>(p.res1, res_off + col, a1);
                } else {
                    // accumulators: a0 = P uV + (P*F) V, a1 = (P*T) K + dS uK;  PK comes from the first backward
                    float o[16], g[16], pkv[16];
                    if constexpr (CFG::STAGED_IO) {
                        const uint32_t sw = row & 7;
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) pkv[i] = pk_pre[c + i];
                        #pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const uint32_t off = row * 128 + (((col / 8 + i) ^ sw) << 4);
                            unpack8_as_float<BF16>(ld_shared_v4(io_out + off), o + 8 * i);
                            unpack8_as_float<BF16>(ld_shared_v4(io_dq + off), g + 8 * i);
                        }
                    } else {
                        const float4* src = reinterpret_cast<const float4*>(p.pk + res_off + col);
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float4 t = src[i];
                            pkv[4 * i] = t.x; pkv[4 * i + 1] = t.y; pkv[4 * i + 2] = t.z; pkv[4 * i + 3] = t.w;
                        }
                        load16_as_float<BF16>(p.out, (long long)batch * p.out_sb + (long long)head * p.out_sh +
                                                         (long long)own_idx * p.out_sn + col, o);
                        load16_as_float<BF16>(p.dQ, (long long)batch * p.dQ_sb + (long long)head * p.dQ_sh +
                                                        (long long)own_idx * p.dQ_sn + col, g);
                    }
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float dob = a0[i] - alpha * o[i];                                   // dObar
                        const float qb = p.scale * (a1[i] - ecirc * pkv[i]) - alpha * g[i];       // Qbar
                        a0[i] = qb; a1[i] = dob;
                    }
                    if constexpr (CFG::STAGED_IO) {
                        // results replace my own chunks of the staged operands: Qbar over dQ, dObar over out
                        #pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const uint32_t off = row * 128 + (((col / 8 + i) ^ (row & 7)) << 4);
                            st_shared_v4(io_dq + off, pack2<BF16>(a0[8 * i], a0[8 * i + 1]), pack2<BF16>(a0[8 * i + 2], a0[8 * i + 3]),
                                         pack2<BF16>(a0[8 * i + 4], a0[8 * i + 5]), pack2<BF16>(a0[8 * i + 6], a0[8 * i + 7]));
                            st_shared_v4(io_out + off, pack2<BF16>(a1[8 * i], a1[8 * i + 1]), pack2<BF16>(a1[8 * i + 2], a1[8 * i + 3]),
                                         pack2<BF16>(a1[8 * i + 4], a1[8 * i + 5]), pack2<BF16>(a1[8 * i + 6], a1[8 * i + 7]));
                        }
                    } else {
                        store16_from_float<BF16>(p.res0, res_off + col, a0);
                        store16_from_float<BF16>(p.res1, res_off + col, a1);
                    }
                }
            }
            }   // store_results
            if (total > 0 && !released) release_outputs();   // a thread with no column inside the head dim
        }
        if constexpr (CFG::STAGED_IO) {
            // my rows' results are in shared memory: the IO warp writes the tile out (the arrival
            // publishes my stores; a thread that gave up does not arrive and the IO warp's wait runs out)
            if (ok) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_io_ready);
            }
        }
        if (total > 0) ++n_live;
        ++n_items_done;
        BOB_PH(5)
        }   // items
        BOB_PH_FLUSH(0, tid == 0)
    }
#undef BOB_ITEM_LOCALS

    // ---- teardown --------------------------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == NPW / 32) {
        __syncwarp();
        tmem_dealloc(tmem, CFG::TMEM_COLS);
    }
}

}  // namespace bob
