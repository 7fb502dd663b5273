/*
 * gdn2_b200 -- C ABI of the B200 (sm_100a) Gated DeltaNet-2 kernels.
 *
 * This header is the drop-in boundary: these are the calls a host binding
 * makes in place of the reference project's cached TVM-FFI executors
 * (`compiled(*tensors, scalars, stream)`).  Every entry point
 *
 *   - takes raw device pointers, 64-bit sizes, a dtype code, a float scale and
 *     the CUDA stream to launch on (the caller makes the owning device
 *     current first);
 *   - never allocates, frees, synchronises or throws; outputs and scratch are
 *     caller-owned;
 *   - returns GDN2_OK or a negative gdn2_status, after validating its
 *     arguments on the host and checking cudaGetLastError() after launch.
 *
 * Layouts (identical to the reference, README.md:48-54 of the reference):
 *   sequence tensors  [B, T, H, 128] contiguous, q/k/v/beta/w in `dtype`
 *                     (bf16 or fp16), g in `g_dtype` (same as dtype, or fp32);
 *   states            [B, H, 128, 128] fp32, key-major rows, value contiguous;
 *   boundary stacks   [B, n_slots, H, 128, 128] fp32, slot j = state (or state
 *                     cotangent) before token t_begin + j*GDN2_TOKEN_INTERVAL,
 *                     last slot = after token t_end-1,
 *                     n_slots = ceil((t_end - t_begin)/GDN2_TOKEN_INTERVAL) + 1.
 *
 * Token sub-ranges: the token-path calls work on tokens [t_begin, t_end) of a
 * [B, T, H, 128] tensor, so that a ragged tail after the last full chunk runs
 * on the same buffers without copies.
 */
#ifndef GDN2_B200_H_
#define GDN2_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GDN2_DIM 128            /* K == V == 128 */
#define GDN2_TOKEN_INTERVAL 16  /* tokens between two token-path boundary slots */
#define GDN2_CHUNK 64           /* tokens per chunk of the tensor-core chunk path */

typedef enum gdn2_dtype {
  GDN2_BF16 = 0,
  GDN2_FP16 = 1,
  GDN2_FP32 = 2 /* only valid for g_dtype */
} gdn2_dtype;

/* bit flags of the `prologue` argument of the *_fused forward entry points */
#define GDN2_PROLOGUE_NORMALIZE_QK 1   /* q, k are raw projections: q / sqrt(sum q^2 + 1e-6), k likewise */
#define GDN2_PROLOGUE_ACTIVATE_GATES 2 /* beta, w, g are pre-activations: sigmoid, sigmoid, -softplus */

typedef enum gdn2_status {
  GDN2_OK = 0,
  GDN2_ERR_NULL_POINTER = -1,
  GDN2_ERR_BAD_SHAPE = -2,
  GDN2_ERR_BAD_DTYPE = -3,
  GDN2_ERR_BAD_RANGE = -4,
  GDN2_ERR_ALIGNMENT = -5,
  GDN2_ERR_UNSUPPORTED = -6,
  GDN2_ERR_LAUNCH = -7,
  GDN2_ERR_DEVICE = -8,
  GDN2_ERR_TOO_LARGE = -9
} gdn2_status;

/* Library/ABI version (major*10000 + minor*100 + patch). */
int gdn2_version(void);

/* Human-readable text for a gdn2_status (static storage). */
const char* gdn2_status_string(int status);

/* Text of the last CUDA error seen by the calling thread's most recent failed
 * entry point (static thread-local storage; empty when none). */
const char* gdn2_last_cuda_error(void);

/* 1 when the current device is compute capability 10.x, else 0 (negative
 * status on a CUDA error).  Replaces the reference's capability gate
 * (src/gdn2_sm120/recurrent.py:412-418, chunk.py:1210-1213). */
int gdn2_device_supported(void);

/*
 * Recurrent / decode forward over tokens [t_begin, t_end).
 * Replaces _token_forward_kernel and its launcher
 * (src/gdn2_sm120/recurrent.py:108-243, 306-340, 576-648).
 *
 *   initial_state  may be NULL (recurrence starts from zero)
 *   out            [B, T, H, 128] in `dtype`; rows [t_begin, t_end) are written
 *   final_state    fp32 state after token t_end-1; may equal initial_state
 *                  exactly (in-place update); may be NULL if not wanted
 *   boundaries     optional boundary stack (see header comment), or NULL
 * State pointers need only 4-byte alignment; 16-byte aligned ones use 128-bit
 * transfers.
 */
int gdn2_token_forward(const void* q, const void* k, const void* v, const void* g,
                       const void* beta, const void* w, const float* initial_state,
                       void* out, float* final_state, float* boundaries,
                       int64_t batch, int64_t time, int64_t heads,
                       int64_t t_begin, int64_t t_end,
                       int dtype, int g_dtype, float scale, void* stream);

/*
 * T == 1 closed form for a zero initial state: S = k (w*v)^T,
 * o = scale (q.k) (w*v).  Reads neither g nor beta.
 * Replaces _token_forward_t1_zero_kernel (src/gdn2_sm120/recurrent.py:246-303,
 * 343-371, 651-701).
 */
int gdn2_token_forward_t1_zero(const void* q, const void* k, const void* v, const void* w,
                               void* out, float* final_state,
                               int64_t batch, int64_t heads,
                               int dtype, float scale, void* stream);

/*
 * Reverse scan of the state cotangent over tokens [t_begin, t_end):
 *   dS' = dS + (scale q) do^T ; du = dS'^T k ; dS <- exp(g) * (dS' - (beta k) du^T).
 * Writes every boundary slot of `d_boundaries` (required) and, when non-NULL,
 * the cotangent of the state before t_begin into `d_initial_state`.
 * d_final_state may be NULL (zero terminal cotangent).
 * Replaces the scalar boundary scan _wy_boundary_dstate_kernel
 * (src/gdn2_sm120/backward_parallel.py:625-718) and its host wrapper
 * wy_boundary_dstate (:1997-2190) for the token path.
 */
int gdn2_token_dstate_scan(const void* q, const void* k, const void* g, const void* beta,
                           const void* d_out, const float* d_final_state,
                           float* d_boundaries, float* d_initial_state,
                           int64_t batch, int64_t time, int64_t heads,
                           int64_t t_begin, int64_t t_end,
                           int dtype, int g_dtype, float scale, void* stream);

/*
 * Chunk-local token VJP over tokens [t_begin, t_end): from the forward state
 * boundaries (written by gdn2_token_forward) and the cotangent boundaries
 * (written by gdn2_token_dstate_scan) recompute each 16-token span forward in
 * fp32 and sweep it in reverse.  Writes rows [t_begin, t_end) of
 * dq, dk, dv, dbeta, dw (`dtype`) and dg (`g_dtype`).
 * Replaces _parallel_chunk_vjp_kernel / _parallel_chunk_vjp_full_kernel and
 * their reduction (src/gdn2_sm120/backward_parallel.py:1052-1421) and the short
 * final-state-only backward kernels (src/gdn2_sm120/backward.py:378-797); unlike
 * those it never reconstructs earlier states by inverting the recurrence.
 */
int gdn2_token_chunk_vjp(const void* q, const void* k, const void* v, const void* g,
                         const void* beta, const void* w, const void* d_out,
                         const float* boundaries, const float* d_boundaries,
                         void* dq, void* dk, void* dv, void* dg, void* dbeta, void* dw,
                         int64_t batch, int64_t time, int64_t heads,
                         int64_t t_begin, int64_t t_end,
                         int dtype, int g_dtype, float scale, void* stream);


/*
 * ---- tensor-core chunk path (64-token chunks) ---------------------------------------
 *
 * The chunk kernels process the tokens [0, full_tokens) of a [batch, T, heads, 128] problem, where
 * full_tokens is a multiple of GDN2_CHUNK: either 64 * floor(T / 64), the caller sending the ragged
 * tail through the token entry points (forward after the chunks, backward before them), or
 * 64 * ceil(T / 64), in which case the last chunk is partial: the kernels read its missing tokens as
 * zeros, which is the identity step of the recurrence, write no output row and no gradient for them,
 * and the state after the last chunk is the state after token T - 1.  Sizes below are asked with the
 * same full_tokens.  Two caller-owned buffers:
 *
 *   workspace  gdn2_chunk_workspace_bytes(batch, full_tokens, heads, training).  Holds the
 *              chunk-end decays and a device status word; with `training` != 0 also what
 *              gdn2_chunk_backward consumes: the residual R and the WY tiles Q_gamma, K_tail, Y^T,
 *              A_qk^T, ((I+L)^-1)^T, one copy of each (the forward scan and the reverse scan read the
 *              same tiles): 160 KiB per 64-token chunk and head.  It must then stay alive and
 *              unmodified until that call has run.
 *   scratch    gdn2_chunk_scratch_bytes(batch, full_tokens, heads, kind).  Tiles that only live
 *              inside one call.  kind 0: forward of an inference call (U and the WY tiles, 144 KiB
 *              per chunk-head); kind 2: forward of a training call (U alone, 32 KiB per chunk-head:
 *              the other tiles are in its workspace); kind 1: backward (dZ, 36 KiB per chunk-head).
 *              Dead when the call's kernels have run, so one scratch buffer serves every call on a
 *              stream; a large batch can be processed as several calls over batch slices that share it.
 * The kernels address tiles, sequence tensors and state checkpoints through tensor maps, which the
 * entry points encode on the host (no device memory involved; recent maps are cached by address and
 * shape).  Buffers, sequence tensors and states must be 16-byte aligned, and batch * time must be
 * below 2^31.
 * Together they replace the intermediate allocations of chunk_forward
 * (src/gdn2_sm120/chunk.py:1317-1362) and of the backward launchers
 * (src/gdn2_sm120/backward_wy.py:1669-1984).
 */
int64_t gdn2_chunk_workspace_bytes(int64_t batch, int64_t full_tokens, int64_t heads, int training);
int64_t gdn2_chunk_scratch_bytes(int64_t batch, int64_t full_tokens, int64_t heads, int kind);

/*
 * Chunkwise forward over tokens [0, full_tokens).  Replaces _prepare_wy_kernel and
 * _inter_chunk_k_split_mma_kernel and their launcher (src/gdn2_sm120/chunk.py:139-331,
 * 438-856, 859-1053).
 *   initial_state  fp32 [B,H,128,128] or NULL (zero)
 *   out            [B,T,H,128] in `dtype`; rows [0, full_tokens) are written
 *   final_state    fp32 state after token full_tokens-1 (may alias initial_state exactly); or NULL
 *   chunk_boundaries  NULL, or fp32 [B, full_tokens/64 + 1, H,128,128]: state before every
 *                  chunk and after the last one (the activation checkpoints of backward)
 *   workspace, scratch  see above (forward scratch: kind 2 when `training`, else kind 0)
 *   training       non-zero: workspace was sized with training = 1, chunk_boundaries is
 *                  required, and everything backward needs is saved
 * All sequence pointers, states, the workspace and the scratch must be 16-byte aligned.
 * If a bounded wait inside a kernel expires, the workspace status word becomes 1 and `out`
 * and `final_state` are filled with NaN from that point on.
 */
int gdn2_chunk_forward(const void* q, const void* k, const void* v, const void* g,
                       const void* beta, const void* w, const float* initial_state,
                       void* out, float* final_state, float* chunk_boundaries,
                       void* workspace, void* scratch, int64_t batch, int64_t time, int64_t heads,
                       int64_t full_tokens, int training, int dtype, int g_dtype, float scale,
                       void* stream);

/*
 * Chunkwise backward over tokens [0, full_tokens): reverse scan of the state cotangent plus
 * the compact-WY chunk VJP, from what gdn2_chunk_forward(training = 1) saved.  Replaces
 * wy_boundary_dstate and compact_wy_chunk_vjp_cute with their kernels
 * (src/gdn2_sm120/backward_parallel.py:537-1049, 1997-2190; backward_wy.py:226-1168, 1669-1984).
 *   d_out            [B,T,H,128] in `dtype` (rows [0, full_tokens) are read)
 *   d_final_state    cotangent of the state after token full_tokens-1, or NULL (zero)
 *   chunk_boundaries the forward's fp32 [B, full_tokens/64 + 1, H,128,128] checkpoints
 *   d_boundaries     caller-owned scratch of the same shape (cotangent at every chunk start)
 *   workspace        the forward's training workspace (read only, apart from its status word)
 *   scratch          backward scratch (see above)
 *   dq, dk, dv, dbeta, dw (`dtype`), dg (`g_dtype`): rows [0, full_tokens) are written
 *   d_initial_state  fp32 [B,H,128,128] or NULL
 * Every pointer must be 16-byte aligned.  The call encodes two TMA tensor maps over
 * chunk_boundaries and d_boundaries on the host (cuTensorMapEncodeTiled, looked up through
 * cudaGetDriverEntryPoint); GDN2_ERR_LAUNCH if the driver does not provide it.
 * If the workspace status word is non-zero when a kernel starts (a wait expired in the forward
 * or earlier in this call), or a wait expires, the gradients are filled with NaN.
 */
int gdn2_chunk_backward(const void* q, const void* k, const void* v, const void* g,
                        const void* beta, const void* w, const void* d_out,
                        const float* d_final_state, const float* chunk_boundaries,
                        float* d_boundaries, const void* workspace, void* scratch,
                        void* dq, void* dk, void* dv, void* dg, void* dbeta, void* dw,
                        float* d_initial_state, int64_t batch, int64_t time, int64_t heads,
                        int64_t full_tokens, int dtype, int g_dtype, float scale, void* stream);

/*
 * Test aid: gdn2_chunk_backward for bf16 inputs with fp32 g, with dq, dk, dv, dbeta, dw written
 * as fp32 (the values before their final rounding to bf16), so that the arithmetic can be
 * held to the fp32 tolerance.  Other dtypes: GDN2_ERR_UNSUPPORTED.  No counterpart in the
 * reference.
 */
int gdn2_chunk_backward_f32grads(const void* q, const void* k, const void* v, const void* g,
                                 const void* beta, const void* w, const void* d_out,
                                 const float* d_final_state, const float* chunk_boundaries,
                                 float* d_boundaries, const void* workspace, void* scratch,
                                 float* dq, float* dk, float* dv, float* dg, float* dbeta, float* dw,
                                 float* d_initial_state, int64_t batch, int64_t time, int64_t heads,
                                 int64_t full_tokens, float scale, void* stream);

/*
 * Synchronise `stream` and return the device status word of a workspace: 0 = ok,
 * 1 = a bounded wait inside a kernel expired (results are NaN).  Diagnostic call
 * for tests and smoke checks; no counterpart in the reference (its kernels have no
 * asynchronous waits).
 */
int gdn2_chunk_read_status(const void* workspace, int64_t batch, int64_t full_tokens,
                           int64_t heads, void* stream);

/*
 * Test aid for the bounded waits: launches one small CTA that allocates tensor memory, waits
 * with the kernels' own bounded waiter (at most `max_polls` polls, clamped to [1, 2^20]) on an
 * mbarrier that nothing ever arms, records status 1 in the workspace's status word when the
 * wait gives up, releases the tensor memory and returns.  Nothing faults, traps or spins
 * without limit.  `workspace` is a workspace of gdn2_chunk_workspace_bytes(batch, full_tokens,
 * heads, training).  No counterpart in the reference.
 */
int gdn2_debug_wait_expires(void* workspace, int64_t batch, int64_t full_tokens, int64_t heads,
                            int64_t max_polls, void* stream);

/*
 * ---- fused input prologue of a layer (next to the primitive, not inside it) ----------------
 *
 * One pass over the [B, T, H, 128] sequence tensors that does what a Gated DeltaNet-2 layer does to
 * its projections before the primitive:
 *     q = q_raw / sqrt(sum_c q_raw^2 + 1e-6), k likewise      (fp32 arithmetic, result in `dtype`)
 *     beta = sigmoid(beta_raw), w = sigmoid(w_raw), g = -softplus(g_raw)
 * and stores the reciprocal norms (fp32 [B, T, H]) for the VJP.  The reference leaves these steps
 * to the caller (README.md:127-131, docs/design.md:32-34); the official implementation it compares
 * against exposes them as use_qk_l2norm_in_kernel / use_gate_in_kernel
 * (src/gdn2_sm120/benchmark.py:230-231).  Either group may be left out by passing NULL for all of
 * its pointers (normalisation: q_raw, k_raw, q, k, inv_norm_q, inv_norm_k; gates: g_raw, beta_raw,
 * w_raw, g, beta, w).  Outputs may alias their inputs exactly.  Pointers 16-byte aligned.
 */
int gdn2_gate_prologue(const void* q_raw, const void* k_raw, const void* g_raw, const void* beta_raw,
                       const void* w_raw, void* q, void* k, void* g, void* beta, void* w,
                       float* inv_norm_q, float* inv_norm_k,
                       int64_t batch, int64_t time, int64_t heads, int dtype, int g_dtype, void* stream);

/*
 * Forward entry points with the prologue fused in: the kernels activate the raw tensors as they load
 * them (gate flags) and scale by the reciprocal row norms they compute on the way (normalisation
 * flag), so an inference call never materialises the activated tensors (the activations use the
 * hardware's exp2 / log2 / reciprocal approximations, about 1e-6 relative, where gdn2_gate_prologue
 * uses the library routines).  `prologue` is a
 * combination of GDN2_PROLOGUE_NORMALIZE_QK and GDN2_PROLOGUE_ACTIVATE_GATES (0 = exactly the
 * plain entry point).  Forward only -- a training call activates with gdn2_gate_prologue, whose
 * outputs backward needs anyway -- hence no checkpoint arguments.  Otherwise as
 * gdn2_token_forward / gdn2_token_forward_t1_zero / gdn2_chunk_forward.  Same counterpart in the
 * official API as gdn2_gate_prologue (use_qk_l2norm_in_kernel / use_gate_in_kernel).
 */
int gdn2_token_forward_fused(const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const void* w, const float* initial_state,
                             void* out, float* final_state,
                             int64_t batch, int64_t time, int64_t heads,
                             int64_t t_begin, int64_t t_end,
                             int dtype, int g_dtype, float scale, int prologue, void* stream);
int gdn2_token_forward_t1_zero_fused(const void* q, const void* k, const void* v, const void* w,
                                     void* out, float* final_state, int64_t batch, int64_t heads,
                                     int dtype, float scale, int prologue, void* stream);
int gdn2_chunk_forward_fused(const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const void* w, const float* initial_state,
                             void* out, float* final_state, void* workspace, void* scratch,
                             int64_t batch, int64_t time, int64_t heads, int64_t full_tokens,
                             int dtype, int g_dtype, float scale, int prologue, void* stream);

/*
 * VJP of gdn2_gate_prologue: from the raw inputs, the stored reciprocal norms and the cotangents of
 * the activated tensors (what gdn2_chunk_backward / gdn2_token_chunk_vjp produced) to the cotangents
 * of the raw tensors:
 *     dq_raw = inv (dq - q^ (q^ . dq)), q^ = q_raw inv;   dbeta_raw = s (1 - s) dbeta, s = sigmoid(beta_raw);
 *     dg_raw = -sigmoid(g_raw) dg.
 * Each output may alias the corresponding incoming cotangent exactly (in-place conversion).
 * Same NULL-group rule as the forward.
 */
int gdn2_gate_prologue_vjp(const void* q_raw, const void* k_raw, const void* g_raw, const void* beta_raw,
                           const void* w_raw, const float* inv_norm_q, const float* inv_norm_k,
                           const void* dq, const void* dk, const void* dg, const void* dbeta, const void* dw,
                           void* dq_raw, void* dk_raw, void* dg_raw, void* dbeta_raw, void* dw_raw,
                           int64_t batch, int64_t time, int64_t heads, int dtype, int g_dtype, void* stream);

/*
 * Per-kernel timing of the chunk entry points.  While enabled, gdn2_chunk_forward and
 * gdn2_chunk_backward record CUDA events on their stream before, between and after their
 * two kernels; gdn2_profile_chunk_kernels waits for the most recent ones and returns the
 * four durations in milliseconds (prep, forward scan, reverse scan, VJP; a value is -1
 * when that call has not run since profiling was enabled).  Off by default; measuring
 * aid for benchmarks, no counterpart in the reference.
 */
int gdn2_profile_enable(int on);
int gdn2_profile_chunk_kernels(float* prep_ms, float* scan_ms, float* bwd_scan_ms, float* vjp_ms);

/*
 * Chunk forward (inference) for callers that must not allocate.  No counterpart in the
 * reference: it exists for hosts such as a serving runtime that partitions device memory
 * once at start-up, or a plugin hook that runs inside another component's memory plan,
 * where obtaining a workspace per call is not possible.  Same kernels and results as
 * gdn2_chunk_forward with training = 0 and chunk_boundaries = NULL, but workspace and scratch
 * are a fixed ~9 MiB array inside the library image (held by every GPU that loads the
 * library, until the process exits).
 *   limit      batch * (full_tokens / 64) * heads <= GDN2_STATIC_MAX_CHUNK_HEADS, otherwise
 *              GDN2_ERR_TOO_LARGE
 *   first call on each device resolves the array's address (one driver query); issue it
 *              before any stream capture begins
 *   sharing    every call on a device uses the same array, which keeps the previous call's
 *              contents; the status word is cleared per call and every tile is rewritten
 *              before use, but calls whose kernels overlap on the GPU race -- serialise them
 * Calls no cudaMalloc / cudaFree / allocating library routine.  Pointers 16-byte aligned.
 */
#define GDN2_STATIC_MAX_CHUNK_HEADS 64
int gdn2_chunk_forward_static(const void* q, const void* k, const void* v, const void* g,
                              const void* beta, const void* w, const float* initial_state,
                              void* out, float* final_state,
                              int64_t batch, int64_t time, int64_t heads, int64_t full_tokens,
                              int dtype, int g_dtype, float scale, void* stream);

/*
 * Synchronise `stream` and return the status word of the fixed array on the current device
 * (as gdn2_chunk_read_status does for a caller-owned workspace) for the problem size of the
 * most recent gdn2_chunk_forward_static call.  GDN2_ERR_UNSUPPORTED before the first such call
 * on the device.  Allocates nothing.  No counterpart in the reference.
 */
int gdn2_chunk_static_read_status(void* stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* GDN2_B200_H_ */
