/*
 * C ABI of libbob_sm100.so: second-order scaled-dot-product attention on NVIDIA B200 (sm_100a).
 *
 * The reference implementation has no C interface; its boundary is Python.  Each entry point
 * below replaces one Python-level call of the reference (paths are inside the reference project):
 *
 *   bob_sm100_fwd   <- bob.attention.forward / bob.kernels.rectangular.rect_forward
 *                      (src/bob/attention.py:251-267, src/bob/kernels/rectangular.py:220-230),
 *                      called from SDPAWithBoB.forward (src/bob/sdpa.py:303-333)
 *   bob_sm100_bwd1  <- bob.sdpa._first_backward (src/bob/sdpa.py:140-172), i.e.
 *                      bob.attention.first_backward (src/bob/attention.py:270-289) and
 *                      rectangular.rect_first_backward (src/bob/kernels/rectangular.py:233-253)
 *   bob_sm100_bwd2  <- bob.sdpa._second_backward (src/bob/sdpa.py:175-236), i.e. the three
 *                      launchers square.bob_2pass (src/bob/kernels/square.py:383-525),
 *                      gqa.bob_gqa (src/bob/kernels/gqa.py:540-718) and
 *                      rectangular.bob_2pass_rect (src/bob/kernels/rectangular.py:628-777)
 *
 * Conventions
 *   - All tensor arguments are device pointers on device `geom->device`.  Tensors are
 *     [B, H, N, D] with unit stride along D; batch/head/row strides are given in elements and
 *     must be multiples of 8 (16 bytes); base addresses must be 16-byte aligned.
 *   - Results are written contiguous [B, H, N, D] in the input dtype.  lse and delta are
 *     contiguous fp32 [B, Hq, Nq]; lse is the natural-log log-sum-exp (-inf for a query row
 *     with no attending key; such a row's output and gradients are zero).
 *   - Masking uses absolute positions: query i sits at q_offset + i, key j at k_offset + j;
 *     non-causal attends everywhere; causal requires key position <= query position; a window
 *     w > 0 additionally requires query position - key position < w.
 *   - Hq must be a multiple of Hkv; query head h uses KV head h / (Hq / Hkv); dK, dV, Kbar and
 *     Vbar are summed over the query heads of a group.
 *   - D must be a multiple of 16, at most 128.  Result pointers and pk must be 16-byte aligned,
 *     lse and delta 4-byte aligned (checked on the host: error -10).
 *   - No entry point allocates or frees device memory (except bob_sm100_selftest's caller-owned
 *     buffers, which are arguments too).  Scratch is passed in as `workspace`, at least
 *     bob_sm100_workspace_bytes(stage, geom) bytes, 256-byte aligned.  Its first word is a
 *     status word that the call clears and a kernel sets if a bounded wait ran out.
 *   - Work is enqueued on `stream` (a cudaStream_t; NULL = legacy default stream) and the call
 *     returns without synchronising.  Calls are re-entrant; concurrent calls need distinct
 *     workspaces.
 *   - Return value: 0 = enqueued; negative = argument or launch error detected on the host
 *     (nothing enqueued beyond what had already been launched); see bob_sm100_error_string.
 */
#ifndef BOB_SM100_H_
#define BOB_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { BOB_SM100_FP16 = 0, BOB_SM100_BF16 = 1 };
enum { BOB_SM100_STAGE_FWD = 0, BOB_SM100_STAGE_BWD1 = 1, BOB_SM100_STAGE_BWD2 = 2 };

typedef struct bob_sm100_geom {
    int32_t B, Hq, Hkv, Nq, Nk, D;
    int32_t dtype;       /* BOB_SM100_FP16 or BOB_SM100_BF16 */
    int32_t is_causal;   /* 0 or 1 */
    int32_t window;      /* 0 = no window; requires is_causal */
    int32_t device;      /* CUDA device ordinal that owns every pointer */
    int64_t q_offset;    /* absolute position of query row 0 */
    int64_t k_offset;    /* absolute position of key row 0 */
    float scale;         /* softmax scale, finite and > 0 */
    int32_t reserved;
    /* element strides (batch, head, row) of each input tensor */
    int64_t q_strides[3];
    int64_t k_strides[3];
    int64_t v_strides[3];
    int64_t out_strides[3];
    int64_t do_strides[3];
    int64_t dq_strides[3];
    int64_t uq_strides[3];
    int64_t uk_strides[3];
    int64_t uv_strides[3];
} bob_sm100_geom;

/* Library version (major * 100 + minor). */
int bob_sm100_version(void);

/* Human-readable text for a negative return code or a positive status word. */
const char* bob_sm100_error_string(int code);

/* Scratch bytes a stage needs for this geometry (includes the 256-byte status block). */
size_t bob_sm100_workspace_bytes(int stage, const bob_sm100_geom* geom);

/* Number of kernels a stage launches for this geometry (for launch accounting). */
int bob_sm100_kernel_launches(int stage, const bob_sm100_geom* geom);

/* Waits for `stream`, then returns the status word of `workspace` (0 = every wait completed). */
int bob_sm100_read_status(const void* workspace, void* stream);

/* Non-blocking check (no counterpart in the reference): returns and clears the code of the most
 * recent bounded wait that ran out in any bob_sm100_fwd / bwd1 / bwd2 kernel on `device` since the
 * last check, 0 if none.  Kernels write the code into a page-locked host word as they give up, so
 * the host can poll it between calls without synchronising; a time-out is therefore seen at the
 * latest when the caller checks after its next synchronisation, and typically one call late.  The
 * results of a call whose kernel gave up are undefined. */
int bob_sm100_last_status(int device);

/* Forward: out = softmax(scale * q k^T + mask) v and lse. */
int bob_sm100_fwd(const bob_sm100_geom* geom, const void* q, const void* k, const void* v,
                  void* out, float* lse, void* workspace, void* stream);

/* First backward: dQ, dK, dV for cotangent dO, and delta = rowsum(dO * out).
 * pk (nullable): fp32 [B, Hq, Nq, D], receives softmax(S) K, a by-product the second backward
 * needs; pass NULL when no second backward will follow (plain first-order training). */
int bob_sm100_bwd1(const bob_sm100_geom* geom, const void* q, const void* k, const void* v,
                   const void* out, const float* lse, const void* dO, void* dQ, void* dK,
                   void* dV, float* delta, float* pk, void* workspace, void* stream);

/* Second backward: gradients of <uQ, dQ> + <uK, dK> + <uV, dV> with respect to q, k, v and dO.
 * uQ / uK / uV may be NULL: that tangent is undefined and contributes nothing.
 * dQ, delta and pk are the first-backward results for the same inputs (bob_sm100_bwd1's outputs). */
int bob_sm100_bwd2(const bob_sm100_geom* geom, const void* q, const void* k, const void* v,
                   const void* out, const float* lse, const float* delta, const float* pk,
                   const void* dO, const void* dQ, const void* uQ, const void* uK, const void* uV,
                   void* Qbar, void* Kbar, void* Vbar, void* dObar, void* workspace, void* stream);

/* Profiling aid (no counterpart in the reference): bob_sm100_bwd2 restricted to one of its two
 * kernels.  part = 1: only the row-owned kernel (Qbar, dObar and the row statistics in the
 * workspace); part = 2: only the column-owned kernel (Kbar, Vbar; it reads the row statistics a
 * previous part-1 or full call left in the same workspace); part = 3: both, i.e. bob_sm100_bwd2.
 * Results that the skipped kernel would have produced are left untouched. */
int bob_sm100_bwd2_part(int part, const bob_sm100_geom* geom, const void* q, const void* k,
                        const void* v, const void* out, const float* lse, const float* delta,
                        const float* pk, const void* dO, const void* dQ, const void* uQ,
                        const void* uK, const void* uV, void* Qbar, void* Kbar, void* Vbar,
                        void* dObar, void* workspace, void* stream);

/* Second backward without a caller-provided workspace (no counterpart in the reference).
 * For hosts that cannot allocate or hand over scratch memory at call time - a plug-in inside a
 * runtime that owns all device memory, a loop that forbids allocator calls after start-up.  The
 * scratch is a fixed array inside the library: 8 MiB + 256 B of device memory on every GPU that
 * loads the library, held until process exit.  Limit: B * Hq * Nq <= bob_sm100_noalloc_max_rows()
 * (1,048,576); beyond it the call returns -12 and enqueues nothing.  The first call on a device
 * resolves the array's device address (make that call before any stream capture begins).  All calls
 * share the array, which keeps the last call's contents; calls whose kernels overlap on the GPU
 * race on it, so issue them on one stream or otherwise serialise them.  Arguments and results are
 * those of bob_sm100_bwd2 without `workspace`; no device memory is allocated or freed. */
size_t bob_sm100_noalloc_max_rows(void);
int bob_sm100_bwd2_noalloc(const bob_sm100_geom* geom, const void* q, const void* k, const void* v,
                           const void* out, const float* lse, const float* delta, const float* pk,
                           const void* dO, const void* dQ, const void* uQ, const void* uK,
                           const void* uV, void* Qbar, void* Kbar, void* Vbar, void* dObar,
                           void* stream);
/* Status word of the last bob_sm100_bwd2_noalloc call on `device` (waits for `stream` first; 0 =
 * every wait completed).  The built-in scratch has no address a caller could pass to
 * bob_sm100_read_status, hence this reader.  Allocates nothing. */
int bob_sm100_noalloc_read_status(int device, void* stream);

/* Known-answer check of the tensor-core plumbing: a [128,64] x b [64,64] (same 16-bit format).
 * out is fp32 [8,128,64]: out[0] = a b^T; out[1] = a b; out[2] = a b^T with a staged through
 * thread-written swizzled shared memory; out[3], out[4] = the two halves of one 128-wide product
 * a [b; b]^T; out[5], out[6] = the two halves of one 128-wide product a [b | b]; out[7] = a b^T
 * with a written to and read from tensor memory.  status is one device int. */
int bob_sm100_selftest(const void* a, const void* b, int is_bf16, float* out, int* status,
                       void* stream);

/* Failure-detection check: launches one warp that waits on a barrier nothing completes.  The
 * library's bounded wait gives up after about half a second of SM cycles and the kernel writes 77
 * to *status (a device int) and to the current device's host-visible status word (see
 * bob_sm100_last_status) and returns normally; the context stays usable. */
int bob_sm100_timeout_selftest(int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BOB_SM100_H_ */
