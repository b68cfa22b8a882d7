// One tiled "sweep" kernel for every stage of second-order attention on sm_100a.
//
// A CTA owns 128 rows of one side of the score matrix (query rows in the row-owned stages, key
// columns in the column-owned stages) and sweeps tiles of TN positions of the other side.  For
// each tile pair it
//   1. forms score-shaped products  own[128, D] x other[TN, D]^T  with tcgen05.mma into tensor
//      memory (fp32),
//   2. reads them back (one thread per own row and per 16-column slice), applies the mask and the
//      softmax recomputation from the saved log-sum-exp, builds the derived 16-bit operands and
//      writes them into 128-byte-swizzled shared memory,
//   3. accumulates output-shaped products  operand[128, TN] x other[TN, D]  into tensor memory
//      accumulators that live for the whole sweep.
// Column-owned stages compute the transposed scores (own = K-side), so the thread that owns key j
// holds column j of the score matrix and the operands come out already transposed; the per-query
// statistics then vary along the tensor-memory columns and are staged in shared memory.
//
// Warp roles: 128*NSPLIT pointwise threads, one MMA-issuing thread, one TMA-producing thread.
// Tiles of the other side are double buffered; scores of tile t+1 are issued before the output
// products of tile t, so the tensor pipe works while the pointwise threads convert tile t.
//
// The algebra follows the reference's second backward (reference: src/bob/kernels/common.py:15-30
// for the formulas, :463-654 for the row-owned tile body and epilogue, :661-786 for the
// column-owned tile body) and the usual flash-attention forward / first backward.
#pragma once

#include "ptx.cuh"

namespace bob {

enum Mode : int { kFwd = 0, kBwd1Row = 1, kBwd1Col = 2, kBwd2Row = 3, kBwd2Col = 4 };
enum TensorId : int { kTQ = 0, kTK, kTV, kTDO, kTUQ, kTUK, kTUV, kNumTensors };

// Status codes written to the status word by a CTA that gave up on a wait.
enum : int { kStatusOk = 0, kStatusTimeoutLoad = 11, kStatusTimeoutMma = 12, kStatusTimeoutPw = 13 };

struct SweepParams {
    CUtensorMap map[kNumTensors];
    // geometry
    int B, Hq, Hkv, G, Nq, Nk, D;
    int is_causal, window;
    long long delta_off;          // q_offset - k_offset
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
    // results, contiguous [B, H, N, D] in the input dtype
    void* res0;
    void* res1;
    void* res2;
    int* status;
};

template <int MODE> struct ModeTraits;
template <> struct ModeTraits<kFwd>     { static constexpr int NOWN = 1, NOTH = 2, NSC = 1, NOUT = 1, NOPER = 1; static constexpr bool COL = false; };
template <> struct ModeTraits<kBwd1Row> { static constexpr int NOWN = 2, NOTH = 2, NSC = 2, NOUT = 1, NOPER = 1; static constexpr bool COL = false; };
template <> struct ModeTraits<kBwd1Col> { static constexpr int NOWN = 2, NOTH = 2, NSC = 2, NOUT = 2, NOPER = 2; static constexpr bool COL = true; };
template <> struct ModeTraits<kBwd2Row> { static constexpr int NOWN = 3, NOTH = 4, NSC = 4, NOUT = 3, NOPER = 4; static constexpr bool COL = false; };
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
    if (MODE == kBwd2Row) return i == 0 ? kTK : (i == 1 ? kTV : (i == 2 ? kTUK : kTUV));
    return i == 0 ? kTQ : (i == 1 ? kTDO : kTUQ);
}

template <int MODE, int DPAD, int TN>
struct SweepConfig {
    using MT = ModeTraits<MODE>;
    static constexpr int NSPLIT = TN / 16;                 // 16 score columns per pointwise thread
    static constexpr int NPW = 128 * NSPLIT;               // pointwise threads
    static constexpr int NTHREADS = NPW + 64;              // + MMA warp + TMA warp
    static constexpr int NSTAGE = 2;
    static constexpr int KSUB = DPAD / 64;                 // 64-element sub-tiles along the head dim
    static constexpr int OWN_TILE_BYTES = 128 * 128 * KSUB;
    static constexpr int OTH_TILE_BYTES = TN * 128 * KSUB;
    static constexpr int OPER_PER_TILE = 64 / TN;          // operands packed per 128-byte-row tile
    static constexpr int NOPER_TILES = (MT::NOPER + OPER_PER_TILE - 1) / OPER_PER_TILE;
    static constexpr int OPER_TILE_BYTES = 128 * 128;
    static constexpr int SC_COLS = MT::NSC * TN;
    static constexpr int OUT_COLS = MT::NOUT * DPAD;
    static constexpr int TMEM_NEED = SC_COLS + OUT_COLS;
    static constexpr int TMEM_COLS = TMEM_NEED <= 128 ? 128 : (TMEM_NEED <= 256 ? 256 : 512);
    static_assert(TMEM_NEED <= 512, "tensor memory budget exceeded");
    // shared memory map (offsets from a 1024-byte aligned base)
    static constexpr int OFF_OWN = 0;
    static constexpr int OFF_OTH = OFF_OWN + MT::NOWN * OWN_TILE_BYTES;
    static constexpr int OFF_OPER = OFF_OTH + NSTAGE * MT::NOTH * OTH_TILE_BYTES;
    static constexpr int OFF_STAT = OFF_OPER + NOPER_TILES * OPER_TILE_BYTES;   // [2][4][TN] floats
    static constexpr int OFF_RED = OFF_STAT + 2 * 4 * TN * 4;                   // [4][NSPLIT][128] floats
    static constexpr int OFF_BAR = OFF_RED + 4 * NSPLIT * 128 * 4;
    static constexpr int NBARS = 1 + 2 * NSTAGE + 6;
    static constexpr int OFF_MISC = OFF_BAR + NBARS * 8;                        // tmem slot, abort flag
    static constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;                     // + alignment slack
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
__device__ __forceinline__ void store16_from_float(void* base, long long elem_off, const float* v) {
    uint4 a, b;
    a.x = pack2<BF16>(v[0], v[1]);   a.y = pack2<BF16>(v[2], v[3]);
    a.z = pack2<BF16>(v[4], v[5]);   a.w = pack2<BF16>(v[6], v[7]);
    b.x = pack2<BF16>(v[8], v[9]);   b.y = pack2<BF16>(v[10], v[11]);
    b.z = pack2<BF16>(v[12], v[13]); b.w = pack2<BF16>(v[14], v[15]);
    uint4* p = reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + elem_off);
    p[0] = a; p[1] = b;
}

// Write 16 consecutive operand columns (starting at column `col0`, a multiple of 16, of a
// 64-column tile) of row `row` into a swizzled operand tile.
template <bool BF16>
__device__ __forceinline__ void store_operand16(uint32_t tile, int row, int col0, const float* v) {
    const uint32_t c = static_cast<uint32_t>(col0) >> 3;
    st_shared_v4(tile + sw128_offset(row, c), pack2<BF16>(v[0], v[1]), pack2<BF16>(v[2], v[3]),
                 pack2<BF16>(v[4], v[5]), pack2<BF16>(v[6], v[7]));
    st_shared_v4(tile + sw128_offset(row, c + 1), pack2<BF16>(v[8], v[9]), pack2<BF16>(v[10], v[11]),
                 pack2<BF16>(v[12], v[13]), pack2<BF16>(v[14], v[15]));
}

__device__ __forceinline__ void store_operand_words(uint32_t tile, int row, int col0, const uint32_t* w) {
    const uint32_t c = static_cast<uint32_t>(col0) >> 3;
    st_shared_v4(tile + sw128_offset(row, c), w[0], w[1], w[2], w[3]);
    st_shared_v4(tile + sw128_offset(row, c + 1), w[4], w[5], w[6], w[7]);
}

template <int MODE, int DPAD, int TN, bool BF16>
__global__ void __launch_bounds__(SweepConfig<MODE, DPAD, TN>::NTHREADS, 1)
sweep_kernel(const __grid_constant__ SweepParams p) {
    using CFG = SweepConfig<MODE, DPAD, TN>;
    using MT = ModeTraits<MODE>;
    constexpr int NSPLIT = CFG::NSPLIT, NPW = CFG::NPW, NSTAGE = CFG::NSTAGE, KSUB = CFG::KSUB;
    constexpr bool COL = MT::COL;
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
    const uint32_t bar_sc_full = bar0 + 8u * (1 + 2 * NSTAGE);
    const uint32_t bar_sc_empty = bar_sc_full + 8;
    const uint32_t bar_op_full = bar_sc_full + 16;
    const uint32_t bar_op_empty = bar_sc_full + 24;
    const uint32_t bar_done = bar_sc_full + 32;
    const uint32_t bar_pw = bar_sc_full + 40;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    // ---- which tile this CTA owns, and the range of tiles it sweeps --------------------------
    const int n_own = COL ? p.Nk : p.Nq;
    const int n_oth = COL ? p.Nq : p.Nk;
    const int n_own_tiles = (n_own + 127) / 128;
    // Row-owned causal tiles get heavier with the row index: start the heavy ones first.
    const int own_tile = (!COL && p.is_causal) ? (n_own_tiles - 1 - (int)blockIdx.x) : (int)blockIdx.x;
    const int own0 = own_tile * 128;
    const int head = blockIdx.y;                 // query head (row-owned) or KV head (column-owned)
    const int batch = blockIdx.z;
    const int kv_head = COL ? head : head / p.G;
    const int n_outer = (MODE == kFwd) ? 2 : (COL ? p.G : 1);

    long long lo = 0, hi = n_oth;                // other-side positions [lo, hi) that can be unmasked
    {
        const long long own_last = (long long)min(own0 + 127, n_own - 1);
        if (p.is_causal) {
            if (!COL) {
                hi = min((long long)n_oth, own_last + p.delta_off + 1);
                if (p.window > 0) lo = max(0LL, (long long)own0 + p.delta_off - p.window + 1);
            } else {
                lo = max(0LL, (long long)own0 - p.delta_off);
                if (p.window > 0) hi = min((long long)n_oth, own_last - p.delta_off + p.window);
            }
        }
    }
    const int t_lo = (hi > lo) ? (int)(lo / TN) : 0;
    const int t_hi = (hi > lo) ? (int)((hi + TN - 1) / TN) : 0;
    const int T = t_hi - t_lo;
    const int total = T * n_outer;

    // ---- set-up ------------------------------------------------------------------------------
    if (tid == 0) {
        mbar_init(bar_own, 1);
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        mbar_init(bar_sc_full, 1);
        mbar_init(bar_sc_empty, NPW / 32);
        mbar_init(bar_op_full, NPW / 32);
        mbar_init(bar_op_empty, 1);
        mbar_init(bar_done, 1);
        mbar_init(bar_pw, NPW / 32);
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
    const uint32_t tmem = misc[0];
    const uint32_t tmem_out = tmem + CFG::SC_COLS;

    auto give_up = [&](int code) {
        misc[1] = 1;
        atomicCAS(p.status, 0, code);
    };
    auto aborted = [&]() { return misc[1] != 0; };

    auto has_tensor = [&](int t) {
        return t == kTUQ ? p.has_uq : (t == kTUK ? p.has_uk : (t == kTUV ? p.has_uv : 1));
    };

    if (warp == NPW / 32 + 1) {
        // =========================== TMA producer =============================================
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
            int issued = 0;
            for (int it = 0; it < total; ++it) {
                const int s = it % NSTAGE;
                if (it >= NSTAGE) {
                    if (!mbar_wait(bar_empty(s), ((it / NSTAGE) - 1) & 1)) { give_up(kStatusTimeoutLoad); break; }
                }
                if (aborted()) break;
                const int outer = it / T;
                const int tile = t_lo + it % T;
                const int oth_head = COL ? (head * p.G + outer) : kv_head;
                uint32_t bytes = 0;
                #pragma unroll
                for (int i = 0; i < MT::NOTH; ++i) {
                    if (MODE == kFwd && outer == 0 && i == 1) continue;
                    if (has_tensor(other_tensor<MODE>(i))) bytes += CFG::OTH_TILE_BYTES;
                }
                mbar_arrive_expect_tx(bar_full(s), bytes);
                #pragma unroll
                for (int i = 0; i < MT::NOTH; ++i) {
                    const int t = other_tensor<MODE>(i);
                    if (MODE == kFwd && outer == 0 && i == 1) continue;
                    if (!has_tensor(t)) continue;
                    #pragma unroll
                    for (int ks = 0; ks < KSUB; ++ks)
                        tma_load_4d(sbase + CFG::OFF_OTH + (s * MT::NOTH + i) * CFG::OTH_TILE_BYTES +
                                        ks * (TN * 128),
                                    &p.map[t], bar_full(s), ks * 64, tile * TN, oth_head, batch);
                }
                ++issued;
            }
            // Do not leave while copies into this CTA's shared memory may still be in flight.
            for (int k = max(0, issued - NSTAGE); k < issued; ++k)
                mbar_wait(bar_full(k % NSTAGE), (k / NSTAGE) & 1);
            mbar_wait(bar_own, 0);
        }
    } else if (warp == NPW / 32) {
        // =========================== MMA issuer ===============================================
        if (lane == 0 && total > 0) {
            constexpr uint32_t fmt = BF16 ? kFmtBF16 : kFmtF16;
            constexpr uint32_t idesc_sc = umma_idesc(fmt, fmt, TN, false);
            constexpr uint32_t idesc_out = umma_idesc(fmt, fmt, 64, true);
            const uint32_t own_base = sbase + CFG::OFF_OWN;

            // score-shaped product: acc[128, TN] (+)= own[slot_a] * other[slot_b]^T
            auto score_mma = [&](int acc, int slot_a, int slot_b, int stage, bool accumulate) {
                const uint32_t a = own_base + slot_a * CFG::OWN_TILE_BYTES;
                const uint32_t b = sbase + CFG::OFF_OTH + (stage * MT::NOTH + slot_b) * CFG::OTH_TILE_BYTES;
                #pragma unroll
                for (int ks = 0; ks < DPAD / 16; ++ks) {
                    const uint32_t ao = (ks / 4) * (128 * 128) + (ks % 4) * 32;
                    const uint32_t bo = (ks / 4) * (TN * 128) + (ks % 4) * 32;
                    umma_ss(tmem + acc * TN, umma_smem_desc(a + ao), umma_smem_desc(b + bo), idesc_sc,
                            (accumulate || ks > 0) ? 1u : 0u);
                }
            };
            // output-shaped product: out[128, DPAD] (+)= operand[oper] * other[slot_b]
            auto out_mma = [&](int out, int oper, int slot_b, int stage, bool accumulate) {
                const uint32_t a = sbase + CFG::OFF_OPER + (oper / CFG::OPER_PER_TILE) * CFG::OPER_TILE_BYTES +
                                   (oper % CFG::OPER_PER_TILE) * (TN * 2);
                const uint32_t b = sbase + CFG::OFF_OTH + (stage * MT::NOTH + slot_b) * CFG::OTH_TILE_BYTES;
                #pragma unroll
                for (int db = 0; db < KSUB; ++db) {
                    #pragma unroll
                    for (int ks = 0; ks < TN / 16; ++ks) {
                        umma_ss(tmem_out + out * DPAD + db * 64, umma_smem_desc(a + ks * 32),
                                umma_smem_desc(b + db * (TN * 128) + ks * 2048), idesc_out,
                                (accumulate || ks > 0) ? 1u : 0u);
                    }
                }
            };

            auto issue_scores = [&](int it) -> bool {
                const int s = it % NSTAGE;
                if (!mbar_wait(bar_full(s), (it / NSTAGE) & 1)) { give_up(kStatusTimeoutMma); return false; }
                if (it > 0 && !mbar_wait(bar_sc_empty, (it - 1) & 1)) { give_up(kStatusTimeoutMma); return false; }
                tc_fence_after_sync();
                if constexpr (MODE == kFwd) {
                    score_mma(0, 0, 0, s, false);
                } else if constexpr (MODE == kBwd1Row || MODE == kBwd1Col) {
                    score_mma(0, 0, 0, s, false);     // S  = Q K^T      | S^T  = K Q^T
                    score_mma(1, 1, 1, s, false);     // dP = dO V^T     | dP^T = V dO^T
                } else if constexpr (MODE == kBwd2Row) {
                    score_mma(0, 0, 0, s, false);                       // S  = Q K^T
                    score_mma(1, 1, 1, s, false);                       // dP = dO V^T
                    if (p.has_uq) score_mma(2, 2, 0, s, false);         // F  = uQ K^T
                    if (p.has_uk) score_mma(2, 0, 2, s, p.has_uq);      //    + Q uK^T
                    if (p.has_uv) score_mma(3, 1, 3, s, false);         // C  = dO uV^T
                } else {
                    score_mma(0, 0, 0, s, false);                       // S^T  = K Q^T
                    score_mma(1, 1, 1, s, false);                       // dP^T = V dO^T
                    if (p.has_uq) score_mma(2, 0, 2, s, false);         // F^T  = K uQ^T
                    if (p.has_uk) score_mma(2, 2, 0, s, p.has_uq);      //      + uK Q^T
                    if (p.has_uv) score_mma(3, 3, 1, s, false);         // C^T  = uV dO^T
                }
                umma_commit(bar_sc_full);
                return true;
            };

            bool ok = mbar_wait(bar_own, 0);
            if (!ok) give_up(kStatusTimeoutMma);
            ok = ok && issue_scores(0);
            int n_out = 0;      // output rounds issued so far
            for (int it = 0; ok && it < total; ++it) {
                if (aborted()) break;
                if (it + 1 < total && !issue_scores(it + 1)) break;
                const int s = it % NSTAGE;
                const int outer = it / T;
                const bool has_out = (MODE != kFwd) || outer == 1;
                if (has_out) {
                    if (!mbar_wait(bar_op_full, n_out & 1)) { give_up(kStatusTimeoutMma); break; }
                    tc_fence_after_sync();
                    const bool acc = n_out > 0;
                    if constexpr (MODE == kFwd) {
                        out_mma(0, 0, 1, s, acc);                       // O += P V
                    } else if constexpr (MODE == kBwd1Row) {
                        out_mma(0, 0, 0, s, acc);                       // dQ += dS K
                    } else if constexpr (MODE == kBwd1Col) {
                        out_mma(0, 1, 0, s, acc);                       // dK += dS^T Q
                        out_mma(1, 0, 1, s, acc);                       // dV += P^T dO
                    } else if constexpr (MODE == kBwd2Row) {
                        if (p.has_uv) out_mma(0, 0, 3, s, acc);         // dObar += P uV
                        out_mma(0, 1, 1, s, acc || p.has_uv);           //        + (P*F) V
                        out_mma(1, 2, 0, s, acc);                       // Omega += (P*T) K
                        if (p.has_uk) out_mma(1, 3, 2, s, true);        //        + dS uK
                        out_mma(2, 0, 0, s, acc);                       // PK    += P K
                    } else {
                        out_mma(0, 0, 0, s, acc);                       // Kbar += Sbar^T Q
                        if (p.has_uq) out_mma(0, 1, 2, s, true);        //       + dS^T uQ
                        out_mma(1, 2, 1, s, acc);                       // Vbar += (P*(F-alpha))^T dO
                    }
                    umma_commit(bar_op_empty);
                    ++n_out;
                }
                umma_commit(bar_empty(s));
            }
            umma_commit(bar_done);
        }
    } else {
        // =========================== pointwise threads =======================================
        const int row = tid & 127;               // own row inside the tile == tensor-memory lane
        const int sp = tid >> 7;                 // which 16-column slice of every score tile
        const int own_idx = own0 + row;
        const bool own_ok = own_idx < n_own;
        const uint32_t tlane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const float c_exp = p.scale * kLog2e;
        const long long row_stat = ((long long)batch * p.Hq + head) * p.Nq + own_idx;   // row-owned only

        // Synchronise the pointwise threads through an mbarrier so that the wait is bounded.
        uint32_t pw_phase = 0;
        auto pw_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pw);
            const bool r = __all_sync(0xffffffffu, mbar_wait(bar_pw, pw_phase));
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

        // per-row state
        float L2 = 0.f, dlt = 0.f;               // row-owned: own row's lse*log2e and delta
        float acc_a = 0.f, acc_b = 0.f;          // row sums (alpha, ecirc) or (running max, running sum)
        if constexpr (MODE == kFwd) { acc_a = -1e30f; acc_b = 0.f; }

        if constexpr (MODE == kBwd1Row) {
            // delta = rowsum(dO * out), each slice sums its share of the head dim
            float part = 0.f;
            if (own_ok) {
                constexpr int DC = DPAD / NSPLIT;
                const long long o_off = (long long)batch * p.out_sb + (long long)head * p.out_sh + (long long)own_idx * p.out_sn;
                const long long g_off = (long long)batch * p.dO_sb + (long long)head * p.dO_sh + (long long)own_idx * p.dO_sn;
                #pragma unroll
                for (int c = 0; c < DC; c += 16) {
                    const int col = sp * DC + c;
                    if (col < p.D) {
                        float a[16], b[16];
                        load16_as_float<BF16>(p.out, o_off + col, a);
                        load16_as_float<BF16>(p.dO, g_off + col, b);
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) part = fmaf(a[i], b[i], part);
                    }
                }
            }
            red_buf[sp * 128 + row] = part;
            ok = pw_sync();
            #pragma unroll
            for (int k = 0; k < NSPLIT; ++k) dlt += red_buf[k * 128 + row];
            ok = ok && pw_sync();
            if (sp == 0 && own_ok) p.delta[row_stat] = dlt;
            if (own_ok) L2 = p.lse[row_stat] * kLog2e;
        }
        if constexpr (MODE == kBwd2Row) {
            if (own_ok) { L2 = p.lse[row_stat] * kLog2e; dlt = p.delta[row_stat]; }
        }

        int n_op = 0;                            // operand rounds written so far
        for (int it = 0; ok && it < total; ++it) {
            const int outer = it / T;
            const int tile = t_lo + it % T;
            const int oth0 = tile * TN;
            const int col0 = sp * 16;            // my first column inside the tile

            if constexpr (COL) {
                // per-query statistics of this tile -> shared memory (double buffered)
                float* sb = stat_buf + (it & 1) * 4 * TN;
                if (tid < TN) {
                    const int i = oth0 + tid;
                    float l2 = 0.f, d = 0.f, al = 0.f, ec = 0.f;
                    if (i < p.Nq) {
                        const long long off = ((long long)batch * p.Hq + (head * p.G + outer)) * p.Nq + i;
                        l2 = p.lse[off] * kLog2e;
                        d = p.delta[off];
                        if constexpr (MODE == kBwd2Col) { al = p.alpha[off]; ec = p.ecirc[off]; }
                    }
                    sb[tid] = l2; sb[TN + tid] = d; sb[2 * TN + tid] = al; sb[3 * TN + tid] = ec;
                }
                // Buffer (it & 1) was last read in iteration it - 2; every thread has since waited
                // for the output products of iteration it - 2, which start only after all threads
                // finished that iteration, so the overwrite above cannot race with a reader.
                if (!pw_sync()) { ok = false; break; }
            }
            if constexpr (MODE == kFwd) {
                if (outer == 1 && it == T) {
                    // between the two passes: combine the slices' (max, sum) into the row's lse
                    red_buf[sp * 128 + row] = acc_a;
                    red_buf[(NSPLIT + sp) * 128 + row] = acc_b;
                    if (!pw_sync()) { ok = false; break; }
                    float m = -1e30f;
                    #pragma unroll
                    for (int k = 0; k < NSPLIT; ++k) m = fmaxf(m, red_buf[k * 128 + row]);
                    float l = 0.f;
                    #pragma unroll
                    for (int k = 0; k < NSPLIT; ++k)
                        l += red_buf[(NSPLIT + k) * 128 + row] * fast_exp2(red_buf[k * 128 + row] - m);
                    L2 = (l > 0.f) ? m + log2f(l) : INFINITY;
                    if (sp == 0 && own_ok) p.lse[row_stat] = (l > 0.f) ? L2 * kLn2 : -INFINITY;
                }
            }

            if (!pw_wait(bar_sc_full, it & 1)) { ok = false; break; }
            tc_fence_after_sync();

            // ---- mask bookkeeping for my 16 columns -------------------------------------------
            // dist = query position - key position; unmasked iff 0 <= dist (< window) when causal
            long long dist0;                     // dist at my first column
            int dstep;                           // change of dist per column
            if constexpr (!COL) { dist0 = (long long)own_idx + p.delta_off - (oth0 + col0); dstep = -1; }
            else                { dist0 = (long long)(oth0 + col0) + p.delta_off - own_idx; dstep = +1; }
            uint32_t vmask = 0;                  // bit c set = column c unmasked
            {
                const int n_left = n_oth - (oth0 + col0);          // columns of mine inside the tensor
                #pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const long long dd = dist0 + (long long)dstep * c;
                    bool v = own_ok && c < n_left;
                    if (p.is_causal) v = v && dd >= 0 && (p.window == 0 || dd < p.window);
                    vmask |= (v ? 1u : 0u) << c;
                }
            }

            float s_[16];
            tmem_ld16(tlane + 0 * TN + col0, s_);

            if constexpr (MODE == kFwd) {
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sc_empty);
                if (outer == 0) {
                    float mx = acc_a;
                    #pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        s_[c] = ((vmask >> c) & 1u) ? s_[c] * c_exp : -1e30f;
                        mx = fmaxf(mx, s_[c]);
                    }
                    float sum = acc_b * fast_exp2(acc_a - mx);
                    #pragma unroll
                    for (int c = 0; c < 16; ++c)
                        sum += ((vmask >> c) & 1u) ? fast_exp2(s_[c] - mx) : 0.f;
                    acc_a = mx; acc_b = sum;
                    continue;
                }
                float pv[16];
                #pragma unroll
                for (int c = 0; c < 16; ++c)
                    pv[c] = ((vmask >> c) & 1u) ? fast_exp2(s_[c] * c_exp - L2) : 0.f;
                if (n_op > 0 && !pw_wait(bar_op_empty, (n_op - 1) & 1)) { ok = false; break; }
                store_operand16<BF16>(sbase + CFG::OFF_OPER, row, col0, pv);
            } else {
                float dp_[16];
                tmem_ld16(tlane + 1 * TN + col0, dp_);
                float f_[16], cc_[16];
                if constexpr (MODE == kBwd2Row || MODE == kBwd2Col) {
                    if (p.has_uq || p.has_uk) tmem_ld16(tlane + 2 * TN + col0, f_);
                    if (p.has_uv) tmem_ld16(tlane + 3 * TN + col0, cc_);
                }
                tmem_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sc_empty);
                if constexpr (MODE == kBwd2Row || MODE == kBwd2Col) {
                    if (!(p.has_uq || p.has_uk)) {
                        #pragma unroll
                        for (int c = 0; c < 16; ++c) f_[c] = 0.f;
                    }
                    if (!p.has_uv) {
                        #pragma unroll
                        for (int c = 0; c < 16; ++c) cc_[c] = 0.f;
                    }
                }
                const float* sb = stat_buf + (it & 1) * 4 * TN + col0;   // column-owned only

                // derived operands, packed to 16 bits as soon as they are formed
                uint32_t w0[8], w1[8], w2[8], w3[8];
                #pragma unroll
                for (int c2 = 0; c2 < 8; ++c2) {
                    float e0[2], e1[2], e2[2], e3[2];
                    #pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = 2 * c2 + h;
                        const bool v = (vmask >> c) & 1u;
                        const float l2 = COL ? sb[c] : L2;
                        const float dl = COL ? sb[TN + c] : dlt;
                        const float pr = v ? fast_exp2(fmaf(s_[c], c_exp, -l2)) : 0.f;
                        const float dps = dp_[c] - dl;
                        e0[h] = e1[h] = e2[h] = e3[h] = 0.f;
                        if constexpr (MODE == kBwd1Row) {
                            e0[h] = pr * dps;                                 // dS
                        } else if constexpr (MODE == kBwd1Col) {
                            e0[h] = pr;                                       // P^T
                            e1[h] = pr * dps;                                 // dS^T
                        } else if constexpr (MODE == kBwd2Row) {
                            const float f = p.scale * f_[c];
                            const float t = fmaf(f, dps, cc_[c]);
                            const float pf = pr * f, pt = pr * t;
                            acc_a += pf; acc_b += pt;
                            e0[h] = pr; e1[h] = pf; e2[h] = pt; e3[h] = pr * dps;
                        } else {
                            const float al = sb[2 * TN + c], ec = sb[3 * TN + c];
                            const float f = p.scale * f_[c];
                            const float t = fmaf(f, dps, cc_[c]);
                            e0[h] = pr * (t - al * dps - ec);                 // Sbar^T
                            e1[h] = pr * dps;                                 // dS^T
                            e2[h] = pr * (f - al);                            // (P*(F-alpha))^T
                        }
                    }
                    w0[c2] = pack2<BF16>(e0[0], e0[1]);
                    if constexpr (MT::NOPER > 1) w1[c2] = pack2<BF16>(e1[0], e1[1]);
                    if constexpr (MT::NOPER > 2) w2[c2] = pack2<BF16>(e2[0], e2[1]);
                    if constexpr (MT::NOPER > 3) w3[c2] = pack2<BF16>(e3[0], e3[1]);
                }
                if (n_op > 0 && !pw_wait(bar_op_empty, (n_op - 1) & 1)) { ok = false; break; }
                auto oper_addr = [&](int k) {
                    return sbase + CFG::OFF_OPER + (k / CFG::OPER_PER_TILE) * CFG::OPER_TILE_BYTES;
                };
                auto oper_col = [&](int k) { return (k % CFG::OPER_PER_TILE) * TN + col0; };
                store_operand_words(oper_addr(0), row, oper_col(0), w0);
                if constexpr (MT::NOPER > 1) store_operand_words(oper_addr(1), row, oper_col(1), w1);
                if constexpr (MT::NOPER > 2) store_operand_words(oper_addr(2), row, oper_col(2), w2);
                if constexpr (MT::NOPER > 3) store_operand_words(oper_addr(3), row, oper_col(3), w3);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_op_full);
            ++n_op;
            if (__any_sync(0xffffffffu, aborted())) { ok = false; break; }
        }

        // ---- epilogue ------------------------------------------------------------------------
        if constexpr (MODE == kFwd) {
            if (total == 0 && sp == 0 && own_ok) p.lse[row_stat] = -INFINITY;
        }
        float alpha = 0.f, ecirc = 0.f;
        ok = __all_sync(0xffffffffu, ok);
        if constexpr (MODE == kBwd2Row) {
            red_buf[sp * 128 + row] = acc_a;
            red_buf[(NSPLIT + sp) * 128 + row] = acc_b;
            if (ok) ok = pw_sync();
            #pragma unroll
            for (int k = 0; k < NSPLIT; ++k) { alpha += red_buf[k * 128 + row]; ecirc += red_buf[(NSPLIT + k) * 128 + row]; }
            if (ok && sp == 0 && own_ok) { p.alpha[row_stat] = alpha; p.ecirc[row_stat] = ecirc; }
        }
        if (ok && total > 0) ok = pw_wait(bar_done, 0);
        tc_fence_after_sync();
        if (ok) {
            constexpr int DC = DPAD / NSPLIT;
            const int res_heads = COL ? p.Hkv : p.Hq;
            const long long res_off = (((long long)batch * res_heads + head) * n_own + own_idx) * p.D;
            #pragma unroll 1
            for (int c = 0; c < DC; c += 16) {
                const int col = sp * DC + c;
                if (col >= p.D) break;
                float a0[16], a1[16], a2[16];
                if (total > 0) {
                    tmem_ld16(tlane + CFG::SC_COLS + 0 * DPAD + col, a0);
                    if constexpr (MT::NOUT > 1) tmem_ld16(tlane + CFG::SC_COLS + 1 * DPAD + col, a1);
                    if constexpr (MT::NOUT > 2) tmem_ld16(tlane + CFG::SC_COLS + 2 * DPAD + col, a2);
                    tmem_wait_ld();
                } else {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) { a0[i] = 0.f; a1[i] = 0.f; a2[i] = 0.f; }
                }
                if (!own_ok) continue;          // tensor-memory loads above are warp-wide; stores are per row
                if constexpr (MODE == kFwd) {
                    store16_from_float<BF16>(p.res0, res_off + col, a0);
                } else if constexpr (MODE == kBwd1Row) {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) a0[i] *= p.scale;
                    store16_from_float<BF16>(p.res0, res_off + col, a0);
                } else if constexpr (MODE == kBwd1Col || MODE == kBwd2Col) {
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) a0[i] *= p.scale;
                    store16_from_float<BF16>(p.res0, res_off + col, a0);
                    store16_from_float<BF16>(p.res1, res_off + col, a1);
                } else {
                    float o[16], g[16];
                    load16_as_float<BF16>(p.out, (long long)batch * p.out_sb + (long long)head * p.out_sh +
                                                     (long long)own_idx * p.out_sn + col, o);
                    load16_as_float<BF16>(p.dQ, (long long)batch * p.dQ_sb + (long long)head * p.dQ_sh +
                                                    (long long)own_idx * p.dQ_sn + col, g);
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float dob = a0[i] - alpha * o[i];                                   // dObar
                        const float qb = p.scale * (a1[i] - ecirc * a2[i]) - alpha * g[i];        // Qbar
                        a0[i] = qb; a1[i] = dob;
                    }
                    store16_from_float<BF16>(p.res0, res_off + col, a0);
                    store16_from_float<BF16>(p.res1, res_off + col, a1);
                }
            }
        }
    }

    // ---- teardown --------------------------------------------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == NPW / 32) {
        __syncwarp();
        tmem_dealloc(tmem, CFG::TMEM_COLS);
    }
}

}  // namespace bob
