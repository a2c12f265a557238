/*
 * C ABI of the B200-native fused LM head (linear + cross-entropy) library, libesep_head.so.
 *
 * The library replaces the GPU work of the reference's chunked LM-head path
 *   solution/head/op.py      (_run, _forward, FusedLinearCE, fused_linear_ce, warmup)
 *   solution/head/kernels.py (head_row_softmax_kernel)
 * with hand-written sm_100a kernels (tcgen05 MMA, TMEM accumulators, TMA loads). The reference has
 * no native layer: its Python op calls torch.mm (cuBLAS) and a Triton kernel directly. These entry
 * points are what a Python binding (ctypes) of that op calls instead; each comment names the
 * reference lines whose work the function takes over.
 *
 * Conventions
 *   - plain pointers and sizes only; all pointers except `caps`, `plan`, `out_status` are DEVICE
 *     pointers owned by the caller; the library allocates nothing the caller must free
 *   - every function returns an int status (0 = ok, negative = error, see below), never throws
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) and returns without syncing
 *   - dtype: 0 = fp16, 1 = bf16 (x and W must have the same 16-bit type)
 *   - x is [n, h] row-major, W is [v, h] row-major, both 16-byte aligned, h a multiple of 8
 *   - target holds GLOBAL vocabulary ids (int64); ids outside [0, v_global) mean "no CE term"
 */
#ifndef ESEP_HEAD_H_
#define ESEP_HEAD_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  ESEP_OK = 0,
  ESEP_ERR_BAD_ARG = -1,          /* null pointer, bad shape / dtype, h not a multiple of 8   */
  ESEP_ERR_UNSUPPORTED_ARCH = -2, /* device is not compute capability 10.x                    */
  ESEP_ERR_WORKSPACE = -3,        /* workspace pointer null / too small / misaligned           */
  ESEP_ERR_CUDA = -4,             /* a CUDA runtime or driver call failed                      */
  ESEP_ERR_DEVICE_TIMEOUT = -5,   /* a kernel gave up on a bounded wait (see device_status)    */
  ESEP_ERR_ALIGNMENT = -6,        /* x or W not 16-byte aligned                                */
  ESEP_ERR_STATIC_SCRATCH = -7    /* problem too large for esep_head_forward_static            */
};

#define ESEP_DTYPE_F16 0
#define ESEP_DTYPE_BF16 1
#define ESEP_DTYPE_F32 2 /* only as the type of x in esep_head_step (cast to W's type inside) */

/* Number of floats per row in a partial record: max, sum-exp, sum-exp*(z-max), target logit,
 * index of the max (an int32 stored bit-for-bit in the float slot). Layout is [5][n]. */
#define ESEP_RECORD_FIELDS 5
/* Scalars written by esep_head_finalize: loss_sum, n_valid, n_correct, entropy_sum(valid rows). */
#define ESEP_METRIC_SCALARS 4
/* Scalars written by esep_head_step: the four above, then n_labelled (target != -100),
 * n_attended rows (attention mask != 0; all rows without a mask), entropy_sum(attended rows),
 * n_live (rows that took part in the gradient). */
#define ESEP_STEP_SCALARS 8

typedef struct esep_head_caps {
  int cc_major;
  int cc_minor;
  int sm_count;
  int max_clusters_bwd; /* co-resident 4-CTA clusters of the backward kernel */
  int supported;        /* 1 if the kernels can run on this device */
} esep_head_caps;

/* Work decomposition chosen for a problem size; pure host arithmetic (no GPU needed). */
typedef struct esep_head_plan {
  int fwd_row_tiles, fwd_vocab_tiles, fwd_tiles_per_unit, fwd_splits, fwd_grid;
  int bwd_cluster, bwd_hslice, bwd_hblocks, bwd_passes, bwd_total_steps, bwd_full_rounds,
      bwd_rem_pairs, bwd_rem_splits, bwd_steps_per_split, bwd_grid;
  size_t ws_status_off, ws_partial_off, ws_record_off, ws_cew_off, ws_dxpart_off, ws_bytes;
} esep_head_plan;

/* Human-readable text for a status code (static storage). */
const char* esep_head_status_string(int code);

/* Device capabilities. Replaces nothing in the reference (it assumes sm_75 and has no query). */
int esep_head_query(int device, esep_head_caps* caps);

/* One-time, launch-free initialisation for `device` (function attributes, occupancy, driver
 * entry points). Safe from a worker thread, idempotent.
 * Replaces: solution/head/op.py:47-65 (warmup: ahead-of-time compile, no launch). */
int esep_head_warmup(int device);

/* Work decomposition and workspace layout for a problem, given the device's SM count and its
 * number of co-resident backward clusters. Host only.
 * Replaces: the fixed chunk loop geometry of solution/head/op.py:83-87 (nc, z buffer). */
int esep_head_plan_problem(int64_t n, int64_t h, int64_t v_local, int need_grad, int sm_count,
                           int max_clusters_bwd, esep_head_plan* plan);

/* Bytes of scratch the forward / backward calls need for this problem on the current device
 * (0 on error). Replaces: the z chunk buffer allocation, solution/head/op.py:83-84. */
size_t esep_head_workspace_bytes(int64_t n, int64_t h, int64_t v_local, int dtype, int need_grad);

/* Forward sweep over this rank's vocabulary rows [vocab_offset, vocab_offset + v_local):
 * per-row partial record (m, s, t, target logit, argmax index as GLOBAL id) -> record[5][n].
 * Replaces: torch.mm(x, W^T) + head_row_softmax_kernel pass 1 up to the lane merge,
 * solution/head/op.py:90-95 and solution/head/kernels.py:46-75. */
int esep_head_forward_partial(const void* x, const void* w, const int64_t* target, int64_t n,
                              int64_t h, int64_t v_local, int64_t vocab_offset, int dtype,
                              float* record, void* workspace, size_t workspace_bytes,
                              void* stream);

/* Merges `n_records` partial records (layout [n_records][5][n]; 1 on a single GPU, the
 * all-gathered shards in vocab-parallel mode) and writes the per-row outputs and the scalars.
 *   lse, entropy, argmax: every row; target_logit, ce: 0 on ignored rows
 *   cew_out[n]: ce_weight with ignored rows forced to 0 (input of the backward call)
 *   loss[1] = sum cew * ce ; metrics[4] = {loss, n_valid, n_correct, sum entropy over valid rows}
 * Replaces: kernels.py:70-82 (merge, lse, entropy, argmax) and op.py:105-108,125-127
 * (valid mask, where(), loss = (cew * ce).sum()). */
int esep_head_finalize(const float* records, int n_records, const int64_t* target,
                       const float* ce_weight, int64_t n, int64_t v_global, float* lse,
                       float* target_logit, float* ce, float* entropy, int64_t* argmax,
                       float* cew_out, float* loss, float* metrics, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Single-GPU forward = esep_head_forward_partial + esep_head_finalize.
 * Replaces: solution/head/op.py:68-101 (_run, forward part) and :104-128 (_forward). */
int esep_head_forward(const void* x, const void* w, const int64_t* target, const float* ce_weight,
                      int64_t n, int64_t h, int64_t v, int dtype, float* lse, float* target_logit,
                      float* ce, float* entropy, int64_t* argmax, float* cew_out, float* loss,
                      float* metrics, void* workspace, size_t workspace_bytes, void* stream);

/* dHidden of this rank's vocabulary rows: dx[n, h] (fp32) =
 *   cew * (softmax - onehot) restricted to [vocab_offset, vocab_offset + v_local) times W_local.
 * `lse` is the log-sum-exp over the FULL vocabulary, `cew` the masked weights from finalize.
 * On one GPU this is the whole gradient; in vocab-parallel mode the caller sums the shards.
 * Replaces: kernels.py:84-93 (g pass) and op.py:96-100 (g @ W in fp32, scale by cew/G_SCALE). */
int esep_head_backward(const void* x, const void* w, const int64_t* target, const float* cew,
                       const float* lse, int64_t n, int64_t h, int64_t v_local,
                       int64_t vocab_offset, int dtype, float* dx, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Synchronises `stream` and reports the device status word of `workspace`
 * (0 = all kernels completed; otherwise the code of the first bounded wait that gave up).
 * Returns ESEP_ERR_DEVICE_TIMEOUT when *out_status != 0. No reference counterpart. */
int esep_head_device_status(const void* workspace, void* stream, int* out_status);

/* Self-test of the failure path: launches one warp that waits on a barrier nothing ever
 * completes, with a limit of `limit_cycles` SM clocks (at most 2e9). The kernel gives up, writes
 * code 901 to the status word of `workspace` and returns normally; esep_head_device_status then
 * reports ESEP_ERR_DEVICE_TIMEOUT and the context stays usable. This is how every wait inside the
 * real kernels behaves when a producer, a peer CTA or the tensor pipe never answers (their limit is
 * about two seconds). No reference counterpart (the reference has no device-side waits). */
int esep_head_selftest_bounded_wait(void* workspace, size_t workspace_bytes, int64_t limit_cycles,
                                    void* stream);

/* Size of the scratch array built into the library for esep_head_forward_static. */
#define ESEP_STATIC_SCRATCH_BYTES (16u << 20)
size_t esep_head_static_scratch_bytes(void);

/* Forward for callers that cannot allocate device memory. This entry point has no counterpart
 * in the reference; it was added for hosts that hand the library only their own input and
 * output buffers: an inference or training runtime that carves all device memory from one
 * arena at start-up and forbids cudaMalloc afterwards, or code running where a device
 * allocation would synchronise the GPU or break an allocation-free section.
 * Same inputs, outputs and semantics as esep_head_forward, minus the workspace arguments: the
 * per-row partial records and the status word go to a 16 MiB array (ESEP_STATIC_SCRATCH_BYTES)
 * that is part of the loaded library image on every GPU that loads it, until the process exits.
 *   - Limit: the problem must plan to at most ESEP_STATIC_SCRATCH_BYTES of scratch (what
 *     esep_head_plan_problem reports as ws_bytes with need_grad = 0; e.g. 4 340 x 1536 x 151 936
 *     needs about 1.2 MiB, 200 000 rows about 16 MiB). Larger problems return ESEP_ERR_STATIC_SCRATCH and launch nothing.
 *   - The first call on each device looks up the array's device address (no allocation, but a
 *     runtime query); make that first call outside any stream capture.
 *   - The call itself performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *   - All calls on one GPU share the one array, which keeps the previous call's contents; the
 *     function clears the only cell that must start at zero (the status word). Two calls whose
 *     kernels can overlap on the same GPU (different streams) race on it: serialise them. */
int esep_head_forward_static(const void* x, const void* w, const int64_t* target,
                             const float* ce_weight, int64_t n, int64_t h, int64_t v, int dtype,
                             float* lse, float* target_logit, float* ce, float* entropy,
                             int64_t* argmax, float* cew_out, float* loss, float* metrics,
                             void* stream);

/* ---- whole head step: one call, no host synchronisation -------------------------------------- */

/* Bytes of scratch esep_head_step needs for m rows on the current device (0 on error). */
size_t esep_head_step_workspace_bytes(int64_t m, int64_t h, int64_t v, int dtype, int need_grad);

/* Loss, per-row statistics and (need_grad != 0) dHidden of m rows of x against the whole
 * vocabulary, with everything the reference does around its chunk loop done on the device:
 *   - masks: a target outside [0, v) means "no CE term", its weight is forced to 0;
 *   - row classes: rows that carry a loss term with a non-zero weight get their gradient from ONE
 *     pass over the vocabulary (logits computed once: 4*H*V flops per such row); the other
 *     selected rows only get statistics from a forward sweep (2*H*V flops per row). The stable
 *     "live rows first" order, the row counts and the work split of both sweeps are computed on
 *     the device; the host never waits for a count (the reference reads it back every call);
 *   - outputs are written at the caller's row index: lse / entropy / argmax for every selected
 *     row, target_logit / ce 0 where there is no CE term, dx (fp32 [m, h], already multiplied by
 *     the masked weight) exactly 0 on rows without a gradient.
 * Two ways to describe the rows:
 *   flat (labels == NULL):  target[m], ce_weight[m] (NULL = weight 1), every row selected.
 *   step (labels != NULL):  labels[m] and attention_mask[m] (or NULL) of a [m / seq_len, seq_len]
 *     batch: target of position t is labels[t + 1] (-100 past the end), weight 1 on targets other
 *     than -100, a row is selected when it is attended or has a target; rows that are not
 *     selected get 0 in every output (ce / entropy are then the [B, T] per-token loss / entropy).
 * x is [m, h] in W's 16-bit type (x_dtype == dtype) or fp32 (x_dtype == ESEP_DTYPE_F32, cast
 * inside). w_bf16: a bf16 copy of W for the dHidden GEMM of the single pass (pass w itself for
 * bf16 models; may be NULL when need_grad == 0 or where esep_head_step_uses_stored_logits says so). metrics[ESEP_STEP_SCALARS], overflow and top_logit[m] (the largest
 * logit of every selected row, exact) may be NULL.
 * overflow: device int, 1 if a row's largest logit lay more than 115 above its maximum over the
 * first 2048 vocabulary rows; the two-kernel path (esep_head_forward + esep_head_backward), which
 * this call always queues behind that flag, then replaced the sweep's results.
 * Replaces: solution/head/op.py:68-128 (_run, _forward) and the row handling of
 * solution/head/patch.py:443-487 (label shift, row gather, scatter to [B, T], counters). */
int esep_head_step(const void* x, int x_dtype, const void* w, const void* w_bf16, int dtype,
                   int64_t m, int64_t h, int64_t v, const int64_t* target, const float* ce_weight,
                   const int64_t* labels, const int64_t* attention_mask, int64_t seq_len,
                   int need_grad, float* lse, float* target_logit, float* ce, float* entropy,
                   int64_t* argmax, float* cew_out, float* loss, float* metrics, float* dx,
                   float* top_logit, int* overflow, void* workspace, size_t workspace_bytes,
                   void* stream);

/* Older spelling of the flat training call: esep_head_step with target / ce_weight, a gradient
 * and the first four scalars. Same results. */
size_t esep_head_train_workspace_bytes(int64_t n, int64_t h, int64_t v, int dtype);
int esep_head_train(const void* x, const void* w, const void* w_bf16, const int64_t* target,
                    const float* ce_weight, int64_t n, int64_t h, int64_t v, int dtype, float* lse,
                    float* target_logit, float* ce, float* entropy, int64_t* argmax,
                    float* cew_out, float* loss, float* metrics, float* dx, int* overflow,
                    void* workspace, size_t workspace_bytes, void* stream);

/* ---- vocabulary shards built on the single pass ------------------------------------------------
 * Each rank runs esep_head_step on its shard of W as if it were the whole vocabulary (local
 * softmax, unit weights, the local id of the target or 0 as a stand-in when another shard owns
 * it), the ranks exchange one [5][n] record per rank, and esep_head_vp_combine turns the local
 * results into this rank's share of the global ones; the shares of dx are then summed by the
 * caller's all-reduce. The formulas are in csrc/head_aux.cuh. Replaces nothing in the reference
 * (it is single-GPU); the merge rule is the one of solution/head/kernels.py:70-81 written for
 * per-shard log-sum-exps. */

/* local_target[n], unit_weight[n] for the shard [vocab_offset, vocab_offset + v_local). */
int esep_head_vp_prepare(const int64_t* target, int64_t n, int64_t vocab_offset, int64_t v_local,
                         int64_t v_global, int64_t* local_target, float* unit_weight,
                         void* stream);

/* record[5][n] of this shard from its local esep_head_step outputs: lse, entropy, largest logit,
 * target logit (0 unless this shard owns the target), global argmax id (int32 bit for bit). */
int esep_head_vp_pack(const float* lse, const float* entropy, const float* top_logit,
                      const float* target_logit, const int64_t* argmax_local,
                      const int64_t* target, int64_t n, int64_t vocab_offset, int64_t v_local,
                      int64_t v_global, float* record, void* stream);

/* records[n_records][5][n] (all shards, my_record = this shard's position) -> global lse /
 * target_logit / ce / entropy / argmax / masked weight / loss / metrics[4], and dx[n, h]
 * rewritten in place from the local sweep's result to this shard's share of dHidden. */
int esep_head_vp_combine(const float* records, int n_records, int my_record,
                         const int64_t* target, const float* ce_weight, const void* w_shard,
                         int64_t n, int64_t h, int64_t v_local, int64_t vocab_offset,
                         int64_t v_global, int dtype, float* dx, float* lse, float* target_logit,
                         float* ce, float* entropy, int64_t* argmax, float* cew_out, float* loss,
                         float* metrics, void* stream);

/* out[count] (fp16 / bf16 / fp32 by out_dtype) = dx[count] * grad_loss[0], grad_loss a DEVICE
 * scalar; count a multiple of 4, both arrays 16-byte aligned. One pass, no synchronisation.
 * Replaces: FusedLinearCE.backward, solution/head/op.py:143-145 ((dx * grad_loss).to(x.dtype)). */
int esep_head_grad_scale(const float* dx, const float* grad_loss, int64_t count, int out_dtype,
                         void* out, void* stream);

/* ---- the head weight's storage format: one fp16 tensor shared with the embedding ---------------
 *
 * The reference replaces the frozen fp32 tied embed / lm_head weight by ONE fp16 tensor and keeps,
 * for the embedding lookup, a table of the elements that do not survive fp32 -> fp16 -> fp32
 * (solution/head/patch.py:105-123 for the why, :133-215 _Fp16Fixup, :217-226 _embedding_forward16).
 * Here the table is three device arrays in compressed-row form, built in two calls with one host
 * read of the entry count between them (set-up time, as the reference's own .numel()):
 *
 *   row_start int32 [v + 1]   entries of row r are [row_start[r], row_start[r + 1])
 *   flat_idx  int64 [count]   r * h + column of each entry, ascending (= patch.py:145-148)
 *   flat_val  fp32  [count]   the exact value
 */

/* Pass 1. cast != 0: writes w16 = fp16(w32) (round to nearest even) and counts; cast == 0: w16 is
 * the caller's fp16 tensor and is only compared. Leaves row_start complete and
 * stats[0 .. 3) = {entries, rows with entries, most entries in one row}; stats is device memory,
 * int64 [3 + (v + 1023) / 1024] (the tail is scratch: entries per block of 1024 rows).
 * Replaces: `w32.to(torch.float16)` + the compare / nonzero loop of patch.py:141-150. */
int esep_weight_fixup_scan(const float* w32, void* w16, int cast, int64_t v, int64_t h,
                           int32_t* row_start, int64_t* stats, void* stream);

/* Pass 2: fills flat_idx / flat_val (each with room for stats[0] entries). */
int esep_weight_fixup_fill(const float* w32, const void* w16, int64_t v, int64_t h,
                           const int32_t* row_start, int64_t* flat_idx, float* flat_val,
                           void* stream);

/* out [n, h] fp32 = the ORIGINAL fp32 rows ids[0 .. n) bit for bit: gather of fp16 rows, upcast
 * and the rows' entries in one kernel. w16 == NULL: out already holds the upcast rows, only the
 * entries are written (= _Fp16Fixup.apply_rows, patch.py:201-210). row_start == NULL: a weight
 * without entries (= _Fp16Fixup.exact, patch.py:177-194). An id outside [0, v) yields a zero row
 * and sets *status (may be NULL) to 301; nothing is read out of bounds.
 * Replaces: _embedding_forward16 (F.embedding + .to(fp32) + gather / where / scatter_). */
int esep_embed_rows(const void* w16, const int64_t* ids, int64_t n, int64_t v, int64_t h,
                    const int32_t* row_start, const int64_t* flat_idx, const float* flat_val,
                    float* out, int* status, void* stream);

/* out [v, h] fp32 = the original fp32 weight bit for bit (= _Fp16Fixup.exact_weight,
 * patch.py:212-215: the lm_head outside fp16 autocast). */
int esep_weight_exact(const void* w16, int64_t v, int64_t h, int64_t count,
                      const int64_t* flat_idx, const float* flat_val, float* out, void* stream);

/* Which kernels a call with gradient runs over the rows that need one.
 *   single pass  - head_train_kernel (8-CTA clusters at hidden 3200 - 3584): the logits never
 *                  leave the SM; smallest workspace;
 *   two sweeps   - a forward sweep that keeps one 16-bit value per logit in the workspace (rows x
 *                  vocabulary x 2 bytes), then dHidden from that buffer (head_dx_kernel). Needs
 *                  hidden % 64 == 0 and at most 48 GiB for the buffer. The value kept is either
 *                  the softmax weight itself, bf16 2^((logit - reference) log2 e), which
 *                  the dHidden kernel takes by TMA as it is ("stored weights"; its GEMM is bf16,
 *                  so an fp16 model passes a bf16 copy of W; the reference is the row maximum
 *                  over the first 2 048 vocabulary entries + 40, and a row whose maximum lies more
 *                  than 75 above it sends the call to the guarded second attempt, as in the
 *                  single pass), or (logit - reference maximum) log2 e as fp16, which sixteen
 *                  warps of the dHidden kernel turn into weights ("stored logits"; no bf16 copy
 *                  of W, no guard).
 * path 0 (default) and 3: stored weights wherever the two sweeps apply, else the single pass;
 * 2: stored logits wherever they apply, else the single pass; 1: always the single pass (no
 * buffer in the workspace). Measured at 4 340 x 1536 x 151 936 on one B200: 2.91 (stored
 * weights) / 3.39 (stored logits) / 3.55 ms (single pass); at 32 768 x 3584 x 19 008: 7.7 - 8.7 /
 * 8.9 - 9.4 / 13.5 ms.
 * Process-wide, read when a call (or a workspace query) is made: set it before sizing the
 * workspace. Returns the previous value, or ESEP_ERR_BAD_ARG. No
 * counterpart in the reference (its chunk loop is one path). */
int esep_head_set_training_path(int path);

/* Which path a step of this shape will take under the current setting (host-side decision, no
 * launch): 0 single pass, 1 two sweeps over stored logits, 2 two sweeps over stored weights. A
 * caller with an fp16 model needs the bf16 copy of W (`w_bf16` of esep_head_step) when this is
 * 0 or 2; when it is 1, and for bf16 models when it is 2, `w_bf16` may be NULL. */
int esep_head_step_uses_stored_logits(int64_t m, int64_t h, int64_t v, int dtype, int need_grad);

/* Which of the two the most recent esep_head_step on this workspace took (*out_stored = 1: two
 * sweeps). Synchronises the stream (a test / monitoring aid). */
int esep_head_step_path_taken(const void* workspace, void* stream, int* out_stored);

/* Counters: out[0] = per-device initialisations performed so far (function attributes,
 * occupancy queries), out[1] = tensor maps encoded so far (maps are cached by address and
 * shape) - a warmed-up process that repeats a call sees neither number move; out[2] (n >= 3) =
 * kernels launched by the library so far, over all entry points and threads; out[3] (n >= 4) =
 * how many of those were the 8-CTA-cluster training sweep (hidden sizes of 3200 - 3584);
 * out[4] (n >= 5) = how many were the dHidden-from-stored-logits kernel. */
int esep_head_debug_counters(long long* out, int n);

/* ---- the step either side of the head: final residual add + RMSNorm ------------------------- */

/* r_out[n, h] (fp32) = r_in + delta ; rstd[n] = rsqrt(mean(r_out^2) + eps) ;
 * y[n, h] (16-bit, `dtype`) = gamma * (r_out * rstd): the head's input x.
 * delta (16-bit, `dtype`) may be null: then nothing is added and r_out is not written (pass null).
 * h must be a multiple of 4 and at most 8192; all math in fp32. HBM bound, one block per row.
 * Replaces: _add_rmsnorm_fwd, solution/body/norm_rope.py:83-109, as launched for the final norm
 * (solution/body/packed.py:833; AddRMSNorm.forward norm_rope.py:210-257 without exact channels). */
int esep_head_norm_forward(const float* r_in, const void* delta, const float* gamma, int64_t n,
                           int64_t h, float eps, int dtype, float* r_out, void* y, float* rstd,
                           void* stream);

/* Backward of the above from the head's fp32 dHidden `dy` (esep_head_backward's dx, no 16-bit
 * round trip): g = dy * gamma ; proj = sum(g * xhat) / h with xhat = r_out * rstd ;
 * dr[n, h] (fp32) = rstd * (g - xhat * proj) + dr_out ; ddelta (16-bit, `dtype`) = dr rounded.
 * dr_out (gradient that reached r_out from elsewhere) and ddelta may be null.
 * Replaces: _add_rmsnorm_bwd, solution/body/norm_rope.py:116-162 (FROM_Y = 0, one gradient), as
 * launched by AddRMSNorm.backward (norm_rope.py:258-287). gamma gets no gradient there either. */
int esep_head_norm_backward(const float* dy, const float* r_out, const float* rstd,
                            const float* gamma, const float* dr_out, int64_t n, int64_t h,
                            int dtype, float* dr, void* ddelta, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ESEP_HEAD_H_ */
