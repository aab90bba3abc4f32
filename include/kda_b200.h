/* C ABI of libkda_b200.so: hand-written sm_100a CUDA kernels for the KDA (Kimi Delta Attention)
 * gated delta-rule path of meta-pytorch/attention-gym (attn_gym.linear).
 *
 * The reference has no native ABI on this path: its kernels are Triton / CuTeDSL callables bound
 * behind torch.library operators (attn_gym/linear/kda/ops.py:18-136).  Each entry point below is
 * what the CUDA implementation of one of those operators binds to; the citation names the
 * operator (or launcher) it replaces.
 *
 * Conventions
 *   - every pointer is a device pointer; sizes are element counts unless named *_bytes;
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it, never synchronise,
 *     never allocate (callers provide outputs and workspaces) and are re-entrant;
 *   - activations are token-major [N, H, D] with D contiguous; states are [nseq, H, K, V] fp32;
 *   - gates are log2 decays (a = 2^g);
 *   - packed sequences: int32 cu_seqlens[nseq + 1] (starts at 0, non-decreasing, may repeat, may end
 *     before N) and chunk_offsets[nseq + 1] from kda_prepare_chunk_offsets; a dense [B, T] batch is
 *     the packed form with cu_seqlens = {0, T, 2T, ...};
 *   - return value: KDA_OK or a negative KDA_ERR_* code.
 */
#ifndef KDA_B200_H_
#define KDA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KDA_F32 0
#define KDA_BF16 1
#define KDA_F16 2

#define KDA_OK 0
#define KDA_ERR_ARG (-1)         /* null pointer, bad size or inconsistent arguments */
#define KDA_ERR_UNSUPPORTED (-2) /* shape outside what the kernels are built for */
#define KDA_ERR_LAUNCH (-3)      /* the CUDA runtime refused the launch */
#define KDA_ERR_SCRATCH (-4)     /* the problem needs more scratch than the built-in array holds */

/* Library identification: returns 100 * major + minor. */
int kda_b200_version(void);

/* Non-zero if a tensor-memory kernel abandoned a bounded barrier wait or met offsets that leave the
 * packed buffer since the last call (clears the flag); synchronises the device.  Byte 0: the state
 * walks, byte 1: the chunk backward kernel, byte 2: the prepare kernel, byte 3: the gate kernels.  Every wait in those kernels
 * polls a bounded number of times; one that runs out makes the CTA record a code here and leave, so
 * a lost arrival shows up as an error word, never as a hang.  Code 9: cu_seqlens / chunk_offsets
 * describe a sequence that does not lie inside the `tokens` rows of the buffers; its chunks were
 * skipped (the sequence is treated as empty) instead of being read or written -- the device-side
 * counterpart of the reference's offset assertion (kda/chunk_scheduler.py:278-293), which the host
 * cannot check without a synchronisation.  kda_selftest_bounded_wait exercises exactly that path on purpose:
 * a one-warp kernel waits `poll_limit` polls on a barrier nothing arrives on, then returns with
 * code 2 in the error word; the context stays usable.  For tests and debugging; no reference
 * counterpart. */
int kda_device_error_word(void);
int kda_selftest_bounded_wait(int poll_limit, void* stream);

/* Optional per-kernel timing with CUDA events recorded on the launching stream (off by default).
 * kda_stage_timing_read synchronises the recorded events and fills launches[] / total_ms[] (arrays of
 * kda_stage_count() entries, indexed like kda_stage_name); reset != 0 clears the records.
 * No reference counterpart: the reference times stages with torch.profiler ranges
 * (attn_gym/linear/kda/utils.py:269-273). */
int kda_stage_count(void);
const char* kda_stage_name(int stage);
int kda_stage_timing_enable(int on);
int kda_stage_timing_read(int64_t* launches, float* total_ms, int reset);

/* chunk_offsets[i + 1] = sum_{s <= i} ceil(len_s / chunk_size), chunk_offsets[0] = 0.
 * Replaces attn_gym::kda_prepare_chunk_offsets (kda/ops.py:73-76,
 * kda/chunk_scheduler.py:279 `_prepare_ragged_chunk_offsets_kernel`). */
int kda_prepare_chunk_offsets(const int32_t* cu_seqlens, int nseq, int chunk_size,
                              int32_t* chunk_offsets, void* stream);

/* Token-sequential scan (decode step and inference prefill):
 *   S <- diag(2^g) S; d = beta (v - S^T k); S <- S + k d^T; o = scale S^T q.
 * q, k, gate: [*, H, K]; v, out: [*, H, V]; beta: [*, H]; dtypes by code.  Dense: nseq rows of
 * tokens_per_row tokens (cu_seqlens NULL); packed: one row, sequence i = [cu[i], cu[i+1]).
 * initial_state may be NULL (zeros); final_state may be NULL.  Paged form: state_indices != NULL,
 * initial_state is the pool [num_slots, H, K, V] with `slot_stride` elements between slots and is
 * advanced in place; entries <= 0 (or >= num_slots) are padding: zero output rows, pool untouched.
 * Replaces attn_gym::kda_recurrent_fwd / _no_state / _paged (kda/ops.py:60-72,
 * fwd/triton/recurrent.py:41 `_kda_recurrent_fwd_kernel`). */
int kda_recurrent_fwd(const void* q, const void* k, const void* v, const void* gate,
                      const void* beta, int dt_q, int dt_k, int dt_v, int dt_gate, int dt_beta,
                      const float* initial_state, float* final_state, void* out, int dt_out,
                      const int32_t* cu_seqlens, const int32_t* state_indices, int64_t slot_stride,
                      int num_slots, int nseq, int tokens_per_row, int heads, int key_dim,
                      int value_dim, float scale, void* stream);

/* out = log2(e) * chunk_local_cumsum(lower_bound * sigmoid(exp(A_log[h]) * (raw + dt_bias[h, :]))).
 * raw: [batch, tokens, H, dim] (dtype code), out fp32 of the same shape; dim % 4 == 0.
 * num_chunks = batch * ceil(tokens / chunk_size) for dense input, the chunk capacity for packed
 * input (cu_seqlens / chunk_offsets built with the same chunk_size; both NULL when dense).
 * Replaces attn_gym::kda_bounded_gate_fwd_dense / _ragged (fwd/triton/gate_fwd.py:379-393, :59, :220). */
int kda_gate_cumsum_fwd(const void* raw_gate, int dt_raw, const float* A_log, const float* dt_bias,
                        float* out, const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                        int nseq, int batch, int tokens, int heads, int dim, int chunk_size,
                        float lower_bound, int64_t num_chunks, void* stream);

/* Backward of the above: d_raw (dtype of raw) and partial sums over groups of chunks
 * dA_partial, dbias_partial: fp32 [kda_gate_bwd_partial_rows(num_chunks), H * dim]; dA_log[h] = sum
 * over rows and dim of dA_partial, d_dt_bias = sum over rows of dbias_partial.
 * Replaces attn_gym::kda_fused_gate_bwd (bwd/cute/gate_bwd_fused.py:498-502) and
 * attn_gym::kda_bounded_gate_bwd_ragged (fwd/triton/gate_fwd.py:389-393, bwd/triton/gate_bwd.py:141). */
int64_t kda_gate_bwd_partial_rows(int64_t num_chunks);
int kda_gate_cumsum_bwd(const void* raw_gate, int dt_raw, const float* A_log, const float* dt_bias,
                        const float* d_cumulative, void* d_raw, float* dA_partial,
                        float* dbias_partial, const int32_t* cu_seqlens,
                        const int32_t* chunk_offsets, int nseq, int batch, int tokens, int heads,
                        int dim, int chunk_size, float lower_bound, int64_t num_chunks,
                        void* stream);
/* dA_log [heads] and d_dt_bias [heads, dim] (fp32) = sums of the partial rows written by
 * kda_gate_cumsum_bwd (the reference reduces them in its autograd glue,
 * fwd/triton/gate_fwd.py:518-616). */
int kda_gate_bwd_reduce(const float* dA_partial, const float* dbias_partial, int64_t rows, int heads,
                        int dim, float* dA_log, float* d_dt_bias, void* stream);

/* y = x * rsqrt(sum(x^2) + eps) per row of `dim` elements; rstd (fp32 [rows]) may be NULL.
 * Replaces attn_gym::kda_l2norm_fwd / _bwd (fwd/triton/l2norm_fwd.py:84,143; bwd/triton/l2norm_bwd.py:37). */
int kda_l2norm_fwd(const void* x, int dtype, void* y, float* rstd, int64_t rows, int dim, float eps,
                   void* stream);
int kda_l2norm_bwd(const void* y, const float* rstd, const void* dy, int dtype, void* dx,
                   int64_t rows, int dim, void* stream);

/* Output epilogue of the layer in one pass: y = o * rsqrt(mean(o^2) + eps) * weight * sigmoid(gate_logits)
 * over rows of `dim` elements (o, gate_logits, y in `dtype`; weight fp32 [dim]), and its backward:
 * d_o, d_logits in `dtype`, and the weight gradient as kda_output_gate_bwd_partial_rows(rows) fp32
 * rows of [dim] that the caller sums.  dim: a multiple of 4, at most 512.
 * Replaces the three launches of the reference module after chunk_kda (examples/kda_training.py:
 * 507-517 F.rms_norm, :519-532 sigmoid of the gate projection, :535-539 their product). */
int kda_output_gate_fwd(const void* o, const void* gate_logits, const float* weight, int dtype,
                        void* y, int64_t rows, int dim, float eps, void* stream);
int64_t kda_output_gate_bwd_partial_rows(int64_t rows);
int kda_output_gate_bwd(const void* o, const void* gate_logits, const void* dy, const float* weight,
                        int dtype, void* d_o, void* d_logits, float* dw_partial, int64_t rows,
                        int dim, float eps, void* stream);

/* Chunked forward, bf16 q/k/v [tokens, H, 128], fp32 cumulative log2 gate and beta, chunk 64.
 * Writes out (bf16 [tokens, H, 128]), the tape aqk / akk (bf16 [tokens, H, 64]) and, when
 * final_state != NULL, the fp32 final states.  workspace: kda_chunk_fwd_workspace_bytes() bytes,
 * 16-byte aligned; num_chunks is the launch bound on active chunks (the capacity).
 * Replaces attn_gym::kda_chunk_fwd / _with_state / _ragged / _ragged_with_state
 * (kda/ops.py:18-42, fwd/cute/chunk_kda_fwd.py:134-200). */
int64_t kda_chunk_fwd_workspace_bytes(int64_t tokens, int heads);
int kda_chunk_fwd(const void* q, const void* k, const void* v, const float* cum_gate,
                  const float* beta, const float* initial_state, float* final_state, void* out,
                  void* aqk, void* akk, const int32_t* cu_seqlens, const int32_t* chunk_offsets,
                  int nseq, int64_t tokens, int heads, int key_dim, int value_dim, int num_chunks,
                  void* workspace, int64_t workspace_bytes, void* stream);

/* kda_chunk_fwd / kda_chunk_fwd_save for a dense batch of `batch` rows with `tokens_per_row` tokens each
 * (q, k, v, out [batch * tokens_per_row, H, 128]; states [batch, H, 128, 128]): the offsets are built
 * on the device.  A batch with fewer (row, head) chains than half the SMs and rows of at least 128
 * chunks is cut into segments of whole chunks that are walked in parallel and stitched by the affine
 * boundary-state map (the scheme of kda_chunk_slice_map inside one GPU): a pass from zero states, the
 * chain h_in(s+1) = M_s h_in(s) + b_s, and a corrective pass over the leading chunks that the true
 * entering state can still reach (measured: the chunks until the running transition is exactly
 * zero in fp32; all of them when the gates never forget).  Results equal the unsegmented walk to
 * fp32 resolution of the state.  workspace: kda_chunk_fwd_dense_workspace_bytes(.., keep) bytes with
 * keep = 1 for the _save form, whose buffer kda_chunk_bwd_saved accepts as `saved`.
 * kda_set_row_segments forces the number of segments per row (0 = choose; for tests and tuning).
 * Replaces attn_gym::kda_chunk_fwd / _with_state (kda/ops.py:18-29); the reference lowers dense
 * batches to the packed form too (kda/impl/fused.py:175-182) and walks every row serially. */
int64_t kda_chunk_fwd_dense_workspace_bytes(int batch, int64_t tokens_per_row, int heads, int keep);
int kda_chunk_fwd_dense(const void* q, const void* k, const void* v, const float* cum_gate,
                        const float* beta, const float* initial_state, float* final_state, void* out,
                        void* aqk, void* akk, int batch, int64_t tokens_per_row, int heads,
                        int key_dim, int value_dim, void* workspace, int64_t workspace_bytes,
                        void* stream);
int kda_chunk_fwd_dense_save(const void* q, const void* k, const void* v, const float* cum_gate,
                             const float* beta, const float* initial_state, float* final_state,
                             void* out, void* aqk, void* akk, int batch, int64_t tokens_per_row,
                             int heads, int key_dim, int value_dim, void* saved, int64_t saved_bytes,
                             void* stream);
int kda_set_row_segments(int segments);

/* kda_chunk_fwd for callers that cannot allocate device memory while they run (an inference
 * server whose memory pool already owns the whole GPU, a plugin that may not call cudaMalloc after
 * start-up).  Same arguments and results as kda_chunk_fwd without the workspace: the scratch is a
 * static device array of KDA_NOALLOC_SCRATCH_BYTES inside the library.
 * Limit: tokens * heads <= KDA_NOALLOC_SCRATCH_BYTES / 1024 (e.g. 1024 tokens x 32 heads), otherwise
 * KDA_ERR_SCRATCH.  The entry point calls no cudaMalloc / cudaFree or other allocating routine.
 * First call on a device: CUDA loads device code lazily, so this call is what makes the device
 * load the module that holds the array (the device keeps those bytes from then until the process
 * exits) and looks the array's device address up (cudaGetSymbolAddress with that device current).
 * Make it once per device during start-up -- before the host's own pool takes the remaining
 * memory (afterwards the load fails and the call returns KDA_ERR_LAUNCH) and before any stream
 * capture.  Later calls on that device touch no memory management at all.
 * All calls share the array and it keeps the previous call's contents (nothing in it needs
 * clearing); two calls whose kernels overlap on the GPU -- different streams, different host
 * threads -- race on it.
 * It has no counterpart in the reference, whose operators allocate their intermediates with
 * torch. */
#define KDA_NOALLOC_SCRATCH_BYTES (32 * 1024 * 1024)
int kda_chunk_fwd_noalloc(const void* q, const void* k, const void* v, const float* cum_gate,
                          const float* beta, const float* initial_state, float* final_state,
                          void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                          const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                          int key_dim, int value_dim, int num_chunks, void* stream);

/* Chunked backward.  d_out bf16 [tokens, H, 128] (required), d_final_state / initial_state /
 * d_initial_state fp32 or NULL.  dq, dk, dv bf16; dg (w.r.t. the cumulative gate) and dbeta fp32.
 * Replaces attn_gym::kda_chunk_bwd / _with_state_grad (kda/ops.py:44-58,
 * bwd/cute/chunk_kda_bwd.py:21). */
int64_t kda_chunk_bwd_workspace_bytes(int64_t tokens, int heads, int64_t num_chunks);
int kda_chunk_bwd(const void* q, const void* k, const void* v, const float* cum_gate,
                  const float* beta, const void* aqk, const void* akk, const float* initial_state,
                  const void* d_out, const float* d_final_state, void* dq, void* dk, void* dv,
                  float* dg, float* dbeta, float* d_initial_state, const int32_t* cu_seqlens,
                  const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads, int key_dim,
                  int value_dim, int num_chunks, void* workspace, int64_t workspace_bytes,
                  void* stream);

/* Training pair that trades memory for time.  kda_chunk_fwd_save is kda_chunk_fwd that also keeps
 * its intermediates (w, u, kg, qg, v_new and the chunk-entry states h[c], all bf16) in `saved`,
 * a caller-owned buffer of kda_chunk_bwd_workspace_bytes() bytes, 16-byte aligned;
 * kda_chunk_bwd_saved is kda_chunk_bwd that reads them from the same, untouched buffer instead of
 * rebuilding them (it also uses the buffer's remaining part as its workspace).  Results are those
 * of kda_chunk_fwd / kda_chunk_bwd bit for bit.  The reference always rebuilds in the backward
 * pass (bwd/cute/chunk_kda_bwd.py:54-85, the recompute_w_u and delta_h legs); with 180 GB of HBM
 * per GPU keeping 1.5 KiB + 8 KiB / 64 per (token, head) is the cheaper choice by default. */
int kda_chunk_fwd_save(const void* q, const void* k, const void* v, const float* cum_gate,
                       const float* beta, const float* initial_state, float* final_state,
                       void* out, void* aqk, void* akk, const int32_t* cu_seqlens,
                       const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                       int key_dim, int value_dim, int num_chunks, void* saved, int64_t saved_bytes,
                       void* stream);
int kda_chunk_bwd_saved(const void* q, const void* k, const void* v, const float* cum_gate,
                        const float* beta, const void* aqk, const void* akk,
                        const float* initial_state, const void* d_out, const float* d_final_state,
                        void* dq, void* dk, void* dv, float* dg, float* dbeta,
                        float* d_initial_state, const int32_t* cu_seqlens,
                        const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                        int key_dim, int value_dim, int num_chunks, void* saved, int64_t saved_bytes,
                        void* stream);

/* The reverse state-gradient walk of kda_chunk_bwd_saved alone: d_initial_state [nseq, H, 128, 128] for
 * the cotangents (d_out, d_final_state), read from the tapes a kda_chunk_fwd_save call left in `saved`
 * (which stay intact; the buffer's workspace part is overwritten, as by kda_chunk_bwd_saved).  It is
 * what a slice of a context-parallel backward chain computes before the state gradient of the next
 * slice has arrived (the chain's affine term, kda_b200/dist.py); no dq, dk, dv, dG, dbeta are formed.
 * No reference counterpart: the reference has no context parallelism; the walk itself replaces
 * BlackwellDeltaHBwdV1 (bwd/cute/chunk_delta_h_bwd_v1.py:694, loop :1147-1276). */
int kda_chunk_bwd_state_saved(const float* cum_gate, const void* aqk, const void* d_out,
                              const float* d_final_state, float* d_initial_state,
                              const int32_t* cu_seqlens, const int32_t* chunk_offsets, int nseq,
                              int64_t tokens, int heads, int key_dim, int value_dim, int num_chunks,
                              void* saved, int64_t saved_bytes, void* stream);

/* The chunked pair with the q / k L2 normalisation of the layer fused in (the reference runs it as
 * separate launches right before and after the core: fwd/triton/l2norm_fwd.py:22,
 * bwd/triton/l2norm_bwd.py:37, examples/kda_training.py:412-421).  q and k are the unnormalised rows.
 * kda_chunk_fwd_qknorm normalises them inside its first kernel -- y = x * rsqrt(sum x^2 + eps), rounded
 * to bf16 exactly as kda_l2norm_fwd would leave them, so the results are those of kda_l2norm_fwd
 * followed by kda_chunk_fwd / kda_chunk_fwd_save (keep != 0) bit for bit -- and writes the reciprocal
 * norms to rstd_q / rstd_k (fp32 [tokens, heads]).  kda_chunk_bwd_qknorm_saved is kda_chunk_bwd_saved
 * for that forward: it returns dq and dk as gradients of the unnormalised rows,
 * dx = rstd (dy - y <dy, y>).  One full read and write of q and k is saved in each direction. */
int kda_chunk_fwd_qknorm(const void* q, const void* k, const void* v, const float* cum_gate,
                         const float* beta, const float* initial_state, float* final_state, void* out,
                         void* aqk, void* akk, float* rstd_q, float* rstd_k, float eps,
                         const int32_t* cu_seqlens, const int32_t* chunk_offsets, int nseq,
                         int64_t tokens, int heads, int key_dim, int value_dim, int num_chunks,
                         void* workspace, int64_t workspace_bytes, int keep, void* stream);
int kda_chunk_bwd_qknorm_saved(const void* q, const void* k, const void* v, const float* cum_gate,
                               const float* beta, const void* aqk, const void* akk,
                               const float* initial_state, const void* d_out,
                               const float* d_final_state, void* dq, void* dk, void* dv, float* dg,
                               float* dbeta, float* d_initial_state, const int32_t* cu_seqlens,
                               const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                               int key_dim, int value_dim, int num_chunks, const float* rstd_q,
                               const float* rstd_k, void* saved, int64_t saved_bytes, void* stream);

/* The two halves of kda_chunk_fwd: `prepare` = the chunk-parallel part (fills aqk, akk and the
 * workspace), `state` = the serial state recurrence over the workspace (writes out and final_state,
 * either may be NULL).  use_u == 0 runs the homogeneous recurrence: with identity matrices as
 * initial_state, final_state is the dense slice transition M [nseq, H, 128, 128] such that the state
 * leaving the slice is M h_in + b (context parallelism).  The reference fuses neither split nor
 * transition (kda/ops.py:78-89 `kda_delta_h` is its closest stage operator; docs/linear.md:220-222
 * leaves context parallelism to the caller).  chunk_limit (int32 [nseq, H] or NULL) cuts every walk
 * short after that many chunks: only their rows of `out` are written, and final_state, if given,
 * is the state after them. */
int kda_chunk_fwd_prepare(const void* q, const void* k, const void* v, const float* cum_gate,
                          const float* beta, void* aqk, void* akk, const int32_t* cu_seqlens,
                          const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                          int num_chunks, void* workspace, int64_t workspace_bytes, void* stream);
int kda_chunk_fwd_state(const float* cum_gate, const float* initial_state, float* final_state,
                        void* out, const void* aqk, const int32_t* cu_seqlens,
                        const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                        void* workspace, int use_u, const int32_t* chunk_limit, void* stream);

/* What a rank of the context-parallel chain computes while it waits for its entering state, in one
 * launch over the workspace that kda_chunk_fwd_prepare filled: b_out = the state leaving the slice
 * for a zero entering state and transition_out = the dense slice transition M, both
 * [nseq, H, 128, 128] fp32 (then h_out = M h_in + b_out, kda_state_affine); optionally `out`, the
 * outputs for a zero entering state, and chunk_limit_out (int32 [nseq, H], zero-initialised by the
 * caller): the number of leading chunks after which the running transition is exactly zero in fp32.
 * Past those chunks no entering state can change a bit of `out`, so the corrective pass
 * (kda_chunk_fwd_state with the true entering state and chunk_limit = chunk_limit_out) only redoes
 * the leading chunks; with gates that never forget completely the limit is the chunk count and the
 * pass is a full one.  No reference counterpart (docs/linear.md:220-222 leaves context parallelism
 * to the caller). */
int kda_chunk_slice_map(const float* cum_gate, float* b_out, float* transition_out, void* out,
                        int32_t* chunk_limit_out, const void* aqk, const int32_t* cu_seqlens,
                        const int32_t* chunk_offsets, int nseq, int64_t tokens, int heads,
                        void* workspace, void* stream);

/* The serial state recurrences (forward and backward) run 1, 2 or 4 CTAs per (sequence, head),
 * each owning 128 / split value columns of the state, so that a few long chains still fill the
 * GPU; split = 0 (the default) chooses from the number of chains and SMs, as the reference picks
 * its value tile (fwd/triton/chunk_delta_h.py:166, bwd/cute/chunk_delta_h_bwd_v1_dispatch.py:53-55).
 * Every split gives the same bits.  Process-wide; for tests and tuning. */
int kda_set_state_value_split(int split);

/* h_out = transition * h_in + b for `count` independent [key_dim x value_dim] fp32 states
 * (transition: [count, key_dim, key_dim]); key_dim and value_dim multiples of 64.  Applies the
 * boundary-state correction of the context-parallel prefix chain; no reference counterpart. */
int kda_state_affine(const float* transition, const float* h_in, const float* b, float* h_out,
                     int count, int key_dim, int value_dim, void* stream);

/* Causal depthwise convolution y[t,c] = act(sum_j w[c,j] x[t-(W-1)+j, c]), x/y [batch, tokens, C],
 * w [C, W] (W <= 8), same dtype code for x, w, y, state; C a multiple of 16 bytes of elements.
 * initial_state [nseq, W-1, C] (oldest first) or NULL; activation: 0 none, 1 SiLU.
 * Packed input: batch == 1 and cu_seqlens[nseq + 1]; rows past cu_seqlens[nseq] are not written.
 * Replaces attn_gym::_cute_short_conv_fwd (kda/ops.py:91-95, short_conv/cute.py:296). */
int kda_conv1d_fwd(const void* x, const void* weight, const void* initial_state, void* y, int dtype,
                   const int32_t* cu_seqlens, int nseq, int batch, int tokens, int channels,
                   int width, int activation, void* stream);

/* Backward of kda_conv1d_fwd.  dx like x; dw_partial fp32 [kda_conv1d_bwd_blocks(), C, W] (sum over
 * the first axis gives dw); dstate fp32 [nseq, W-1, C] zero-initialised by the caller, or NULL;
 * dpre_scratch fp32 [batch * tokens, C]; may be NULL for W == 4 with bf16 / fp16 tensors, whose
 * one-pass kernel keeps the pre-activation gradient in registers.
 * Replaces attn_gym::_cute_short_conv_bwd (kda/ops.py:106-110; short_conv/cute.py:582, :791, :1960). */
int64_t kda_conv1d_bwd_blocks(int batch, int tokens, int packed);
int kda_conv1d_bwd(const void* x, const void* weight, const void* initial_state, const void* dy,
                   void* dx, float* dw_partial, float* dstate, float* dpre_scratch, int dtype,
                   const int32_t* cu_seqlens, int nseq, int batch, int tokens, int channels,
                   int width, int activation, void* stream);
/* dw [C, W] in `dtype` = the sum of the `rows` partial rows of dw_partial, in a fixed order. */
int kda_conv1d_dw_reduce(const float* dw_partial, int64_t rows, int64_t channels_times_width, void* dw,
                         int dtype, void* stream);

/* One token per sequence over a paged history pool state [num_slots, W-1, C], advanced in place;
 * state_indices NULL means sequence i uses slot i; entries <= 0 are padding (zero output).
 * Replaces attn_gym::_cute_short_conv_decode (kda/ops.py:96-100, short_conv/cute.py:470). */
int kda_conv1d_decode(const void* x, const void* weight, void* state, const int32_t* state_indices,
                      void* y, int dtype, int nseq, int num_slots, int channels, int width,
                      int activation, void* stream);

/* Decode-step preprocessing in one launch: the q | k | v projection x [N, 3 * H * 128] goes through the
 * depthwise causal convolution over the paged history conv_state [num_slots, W-1, 3 * H * 128] (advanced
 * in place; conv_state_indices as for kda_conv1d_decode, NULL = slot i for sequence i) and the
 * activation; q and k are L2-normalised per head (rsqrt(sum y^2 + eps)); the per-token log2 gate is
 * log2(e) * lower_bound * sigmoid(exp(A_log[h]) * (raw_gate + dt_bias[h])).  Writes q, k, v
 * [N, H, 128] in the dtype of x and gate fp32 [N, H, 128]: the operands of kda_recurrent_fwd.
 * head_dim must be 128.  The reference runs this as four launches (short_conv/cute.py:3569,
 * fwd/triton/l2norm_fwd.py:231 twice, fwd/triton/gate_fwd.py:716 with chunk size 1). */
int kda_decode_prep(const void* x, const void* conv_weight, void* conv_state,
                    const int32_t* conv_state_indices, const void* raw_gate, int dt_gate,
                    const float* A_log, const float* dt_bias, void* q, void* k, void* v, float* gate,
                    int dtype, int nseq, int heads, int head_dim, int width, int num_slots,
                    int activation, float lower_bound, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KDA_B200_H_ */
