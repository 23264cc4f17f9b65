/*
 * dgpt.h — C ABI of libdgpt_b200.so: the sm_100a kernels behind diff-gpt's
 * attention forward and KV-cache Monte-Carlo decode.
 *
 * Conventions
 *   - Every pointer marked "device" is a CUDA device pointer owned by the caller
 *     (inputs, outputs and workspaces alike); the library never allocates, frees
 *     or keeps them, except where an entry point says otherwise.
 *   - `stream` is the caller's cudaStream_t passed as void*.  All entry points
 *     enqueue work and return without synchronising; they may be captured into
 *     a CUDA graph.
 *   - Return value 0 = enqueued; negative = DGPT_E_* (nothing was enqueued).
 *     `dgpt_last_error` gives the text of the last failure on the calling thread.
 *   - `dtype` selects the storage type of activations, weights and KV pages:
 *     DGPT_F32 or DGPT_BF16.  Accumulation is always fp32.
 *   - The reference has no FFI layer of its own (it is pure PyTorch); each entry
 *     point names the reference Python call sites whose arithmetic it replaces
 *     (paths are relative to the reference project root).
 */
#ifndef DGPT_H_
#define DGPT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { DGPT_F32 = 0, DGPT_BF16 = 1 };

enum {
  DGPT_OK = 0,
  DGPT_E_ARG = -1,      /* bad argument (shape, alignment, null pointer)            */
  DGPT_E_UNSUPPORTED = -2, /* combination of dtype / head_dim not built               */
  DGPT_E_CUDA = -3,     /* a CUDA runtime call failed at launch                      */
  DGPT_E_WORKSPACE = -4 /* caller's workspace is too small                           */
};

/* Where the K and V vectors of one layer live.
 * Token `slot` of sequence `seq`, head `h`, lives in page
 *     pg = page_table ? page_table[seq * max_pages + slot / page_tokens] : seq
 * at element offset  pg * page_stride + h * head_stride + (slot % page_tokens) * head_dim
 * from k_base (keys) or v_base (values).
 * The dense reference cache (L,2,B,H,T,D) of src/diff_gpt/model/kv_cache.py:25 is the
 * special case page_table = NULL, page_tokens = T, page_stride = H*T*D, head_stride = T*D.
 */
typedef struct dgpt_kv_layout {
  void* k_base;              /* device */
  void* v_base;              /* device */
  int64_t page_stride;       /* elements */
  int64_t head_stride;       /* elements */
  const int32_t* page_table; /* device, [n_seq][max_pages], or NULL */
  int32_t page_tokens;
  int32_t max_pages;
  int64_t n_pages;           /* pages addressable from the bases when a page table is used (0 = not stated) */
} dgpt_kv_layout;

/* Text of the last error raised on this host thread; returns its length. */
int dgpt_last_error(char* buf, size_t n);

/* ABI version (bumped when a signature changes). */
int dgpt_version(void);

/* x = rms_norm(Emb[ids]).
 * Replaces src/diff_gpt/model/gpt.py:154-155.
 * ids: device int32 [n_tokens]; emb: device [V, C]; out: device [n_tokens, C]. */
int dgpt_embed_rmsnorm(const int32_t* ids, const void* emb, void* out, int64_t n_tokens, int32_t C,
                       int32_t V, int32_t dtype, void* stream);

/* Block Attention Residual depth mix, fused with the RMSNorm that follows it.
 *   a_n   = softmax_n( rms_norm(cand_n) . w )          n = 0..n_cands-1
 *   h     = sum_n a_n cand_n                            (written to out_h if non-NULL)
 *   out_rn= rms_norm(h)                                 (written if non-NULL)
 * With n_cands == 1 the mix is the identity (the layer-0 short-circuit), so the call
 * degenerates to a plain RMSNorm — also used for the final norm before the logits.
 * Replaces src/diff_gpt/model/block.py:10-44 plus the rms_norm of block.py:97,104
 * and gpt.py:180.
 * cands: HOST array of n_cands device pointers, each [rows, C] contiguous
 * (duplicates allowed — the reference commits the embedding twice); w: device [C]. */
int dgpt_depthmix(const void* const* cands, int32_t n_cands, const void* w, void* out_h, void* out_rn,
                  int64_t rows, int32_t C, int32_t dtype, void* stream);

/* dgpt_depthmix with the candidates' norm factors carried from one mix to the next.  A committed block output
 * does not change any more, yet every later mix (two per layer) needs rsqrt(mean(cand^2) + eps) of each of its
 * rows again.  cand_inv: HOST array of n_cands device fp32 [rows] pointers (or NULL entries / NULL array): where
 * given, the factor is read instead of being recomputed.  inv_out: device fp32 [rows] or NULL: receives the
 * factor this call computes for candidate inv_out_index (which must not have one passed in).  The factor is the
 * number the plain call computes, so results do not depend on what is cached.  Needs 16-byte aligned rows of a
 * multiple of 16 bytes when any factor is passed or requested (DGPT_E_UNSUPPORTED otherwise). */
int dgpt_depthmix_cached(const void* const* cands, const float* const* cand_inv, int32_t n_cands, const void* w,
                         void* out_h, void* out_rn, float* inv_out, int32_t inv_out_index, int64_t rows, int32_t C,
                         int32_t dtype, void* stream);

/* RoPE on q and k, RMSNorm over head_dim on both, then append k and v to the cache.
 *   token (s, t), s < n_seq, t < T:   position = seq_pos0[s] + step + t   (RoPE row)
 *                                     slot     = seq_slot0[s] + step + t  (cache slot)
 *   with step = *step_ptr (0 when step_ptr is NULL).
 * Rounding follows the reference: the rotated vector is rounded to `dtype`, then
 * normalised in fp32 and rounded again.
 * Replaces src/diff_gpt/model/rope.py:20-27, mha.py:44-48 and kv_cache.py:108-109.
 * q,k,v: device, rows of H*D elements, token row n = s*T + t at n*in_row_stride;
 * q_out: device [n_seq*T, H*D] with row stride q_out_row_stride;
 * cs_table: device [table_len, D/2, 2] (cos, sin) in `dtype`;
 * status: device int32, set to 1 if a position or slot is out of range (the write is skipped). */
int dgpt_rope_qknorm_kvappend(const void* q, const void* k, const void* v, int64_t in_row_stride,
                              void* q_out, int64_t q_out_row_stride, const void* cs_table,
                              int32_t table_len, const dgpt_kv_layout* kv, const int32_t* seq_pos0,
                              const int32_t* seq_slot0, const int32_t* step_ptr, int32_t n_seq,
                              int32_t T, int32_t H, int32_t D, int32_t dtype, int32_t* status,
                              void* stream);

/* Prefill / chunk attention:  o[b,i,h,:] = softmax_j( q[b,i,h,:].k[b,j,h,:] / sqrt(D) ) v[b,j,h,:]
 * over cache slots j < kv_len (and j <= q_offset + i when `causal`).  That single rule covers the
 * three SDPA branches of src/diff_gpt/model/mha.py:61-81.  When `lse` is non-NULL the natural-log
 * sum of exponentials of the scaled scores is written too ([B, Tq, H] fp32), so the result can be merged
 * with attention over further keys (the shared-prefix phase of the Monte-Carlo decode);
 * in that mode `o` may be requested in fp32 (o_f32 != 0) regardless of `dtype`.
 * q: device, element (b,i,h,d) at b*q_batch_stride + i*q_row_stride + h*D + d;  o likewise.
 * kv: sequence index = b;  kv_len: device int32 [B] or NULL (then kv_len_all is used).
 * impl: 0 = choose (bf16 with D = 64 or 128 runs on the tcgen05 tensor cores, everything else takes
 * the warp-level online-softmax kernel; of the two tensor-core kernels the warp-specialised one is taken
 * from 1024 keys on, the two-CTAs-per-SM one below), 1 = warp-level kernel, 2 = warp-specialised
 * tensor-core kernel or fail, 3 = tensor-core kernel with two CTAs per SM or fail, 4 = persistent tensor-core kernel
 * with two query tiles per CTA or fail.
 * max_ctas: 0, or a cap on the CTAs of the two-CTAs-per-SM kernel, which then loop over the query tiles - for a
 * caller that runs the kernel on a second stream and wants it to stay on part of the GPU (ignored elsewhere).
 * status: device int32, set non-zero if a bounded wait inside the tensor-core kernel ran out. */
int dgpt_fmha_prefill(const void* q, int64_t q_batch_stride, int64_t q_row_stride,
                      const dgpt_kv_layout* kv, const int32_t* kv_len, int32_t kv_len_all, void* o,
                      int64_t o_batch_stride, int64_t o_row_stride, int32_t o_f32, float* lse,
                      int32_t B, int32_t H, int32_t Tq, int32_t D, int32_t q_offset, int32_t causal,
                      int32_t dtype, int32_t impl, int32_t max_ctas, int32_t* status, void* stream);

/* Bytes of workspace dgpt_decode_attn needs for R rows, H heads, head_dim D and n_splits (a multiple of 16;
 * the workspace pointer itself must be 16-byte aligned). */
size_t dgpt_decode_attn_workspace_bytes(int32_t R, int32_t H, int32_t D, int32_t n_splits);

/* Decode attention for one new token per row (Tq = 1), split along the keys.
 * Row r attends to cache slots  [0, len0[r])  and  [start1[r], start1[r] + len1[r] + step)  of
 * sequence r  (step = *step_ptr or 0).  If prefix_o / prefix_lse are given, range 0 has already been
 * reduced by dgpt_fmha_prefill (shared-prefix phase) and is skipped here; its partial result is merged.
 * The merged output is multiplied by sigmoid(gate) when gate is non-NULL.
 * Replaces src/diff_gpt/model/mha.py:65-68 and :83-84.
 * q, gate, y: device [R, H*D] with their row strides; workspace: device, from the _bytes call
 * (unused when n_splits == 1). */
int dgpt_decode_attn(const void* q, int64_t q_row_stride, const dgpt_kv_layout* kv, const int32_t* len0,
                     const int32_t* start1, const int32_t* len1, const int32_t* step_ptr,
                     const float* prefix_o, const float* prefix_lse, const void* gate,
                     int64_t gate_row_stride, void* y, int64_t y_row_stride, void* workspace,
                     size_t workspace_bytes, int32_t n_splits, int32_t R, int32_t H, int32_t D,
                     int32_t dtype, void* stream);

/* The two halves of dgpt_decode_attn as separate launches, for callers that run the shared-prompt
 * contraction (dgpt_fmha_prefill with lse) and the per-row pass on two streams at once.
 * dgpt_decode_attn_partial reduces cache slots [0, len0[r]) (skipped when len0 is NULL) and
 * [start1[r], start1[r] + len1[r] + step) of sequence r and writes the normalised result
 * part_o [R, H, D] fp32 with its natural-log sum of exponentials part_lse [R, H] fp32
 * (-inf and zeros for a row without keys).
 * dgpt_attn_merge combines two such partials, y = (e^lse_a o_a + e^lse_b o_b) / (e^lse_a + e^lse_b),
 * rounds to `dtype` and multiplies by sigmoid(gate) when gate is non-NULL.
 * Together they replace src/diff_gpt/model/mha.py:65-68 and :83-84 exactly as dgpt_decode_attn does. */
int dgpt_decode_attn_partial(const void* q, int64_t q_row_stride, const dgpt_kv_layout* kv,
                             const int32_t* len0, const int32_t* start1, const int32_t* len1,
                             const int32_t* step_ptr, float* part_o, float* part_lse, int32_t R,
                             int32_t H, int32_t D, int32_t dtype, void* stream);
int dgpt_attn_merge(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                    const void* gate, int64_t gate_row_stride, void* y, int64_t y_row_stride, int32_t R,
                    int32_t H, int32_t D, int32_t dtype, void* stream);

/* dgpt_decode_attn for callers that cannot allocate device memory.  (No counterpart in the reference:
 * its attention never needs scratch memory.)
 * Who needs it: a host that must not call cudaMalloc where it launches — an inference server whose
 * memory is handed out once at start-up, a plugin that receives nothing but its input and output
 * buffers, a real-time loop that may not enter the allocator.  With n_splits > 1 the kernel has to
 * park per-split partial results somewhere; here they go into a fixed 16 MiB array that is part of the
 * library image (every GPU that loads the library keeps that array until the process exits), so the
 * caller passes only inputs and outputs, and the call performs no cudaMalloc/cudaFree and uses no
 * allocating library routine.
 * Limits and rules:
 *   - R * H * n_splits * (D + 2) * 4 bytes must fit in dgpt_decode_attn_static_capacity_bytes()
 *     (16 MiB); larger requests return DGPT_E_WORKSPACE with the numbers in dgpt_last_error.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call before starting any stream capture.  The address is kept per process and per
 *     device; it is not valid across cudaDeviceReset (do not reset a device between calls).
 *   - All calls share the one array and it keeps the previous call's contents.  Nothing in it has to
 *     start at zero: every (split, row, head) slot is rewritten by the first pass before the combine
 *     pass reads it.  Two calls that overlap on the GPU (different streams, or graphs replayed
 *     concurrently) race on it: serialise them.
 * Arguments are those of dgpt_decode_attn without the workspace pair; results are identical. */
size_t dgpt_decode_attn_static_capacity_bytes(void);
int dgpt_decode_attn_static(const void* q, int64_t q_row_stride, const dgpt_kv_layout* kv,
                            const int32_t* len0, const int32_t* start1, const int32_t* len1,
                            const int32_t* step_ptr, const float* prefix_o, const float* prefix_lse,
                            const void* gate, int64_t gate_row_stride, void* y, int64_t y_row_stride,
                            int32_t n_splits, int32_t R, int32_t H, int32_t D, int32_t dtype, void* stream);

/* out[r, j] = g*sigmoid(alpha*g)*(l+1) with g = min(in[r,2j], limit), l = clamp(in[r,2j+1], -limit, limit).
 * Replaces src/diff_gpt/model/swi_glu.py:11-19.  in: [rows, 2*n_out]; out: [rows, n_out]. */
int dgpt_swiglu(const void* in, void* out, int64_t rows, int32_t n_out, float alpha, float limit,
                int32_t dtype, void* stream);

/* In-place y[r, c] *= sigmoid(gate[r, c]) — the output gate after prefill attention (the decode kernel
 * applies it in its epilogue).  Replaces src/diff_gpt/model/mha.py:84.  y, gate: device [rows, n_cols]. */
int dgpt_sigmoid_gate(void* y, int64_t y_row_stride, const void* gate, int64_t gate_row_stride,
                      int64_t rows, int32_t n_cols, int32_t dtype, void* stream);

/* In-place logits = cap * tanh(logits / cap) (no-op when cap == 0).
 * Replaces src/diff_gpt/model/gpt.py:182-186.  logits: device [n] */
int dgpt_softcap(void* logits, int64_t n, float cap, int32_t dtype, void* stream);

/* Linear layer on the tcgen05 tensor cores, optionally with the SwiGLU of the feed-forward block in its epilogue:
 *   acc[m, n] = sum_k a[m, k] * w[n, k]                     (w as nn.Linear stores it: [N, K])
 *   epilogue 0:  out[m, n]     = acc[m, n]                  out: [M, N]
 *   epilogue 1:  out[m, n / 2] = swiglu(acc[m, n], acc[m, n + 1]) for even n, the rule of dgpt_swiglu applied to
 *                the accumulator rounded to bf16 (as the reference's Linear output is)      out: [M, N / 2]
 *   epilogue 2:  out[m, n]     = resid[m, n] + acc[m, n], rounded once (resid may be out itself)   out: [M, N]
 * Replaces nn.Linear of src/diff_gpt/model/feed_forward.py:10-14 followed by swi_glu.py:11-19 (epilogue 1), any
 * bias-free nn.Linear of the path (epilogue 0), or a projection with the residual add that follows it
 * (src/diff_gpt/model/block.py:98-106, epilogue 2).  resid is ignored for epilogues 0 and 1.  bf16 only; pointers 16-byte aligned, K and the row strides
 * multiples of 8 elements, N a multiple of 16.  status: device int32, set non-zero if a bounded wait ran out. */
int dgpt_linear(const void* a, int64_t a_row_stride, const void* w, int64_t w_row_stride, void* out,
                int64_t out_row_stride, const void* resid, int64_t resid_row_stride, int32_t M, int32_t N,
                int32_t K, int32_t epilogue, float alpha, float limit, int32_t dtype, int32_t* status,
                void* stream);

/* The time-bounded mbarrier wait that every tcgen05 kernel of the library uses, run by itself in a one-CTA
 * kernel (no counterpart in the reference).  Two threads wait on a barrier that needs one arrival.  arrive != 0:
 * the arrival is made and both waits succeed.  arrive == 0: nothing arrives; the first thread gives up after
 * limit_cycles SM clock cycles (at most 2e9, about a second) and raises the CTA's abort flag, the second gives
 * up on seeing the flag; the kernel then returns normally.  out: device int32 [4] = {first wait ok, second wait
 * ok, code of the wait that gave up (0 if none), cycles the first thread waited}. */
int dgpt_bounded_wait_probe(int32_t arrive, int64_t limit_cycles, int32_t* out, void* stream);

/* out[r] = log(sum_j exp(logits[r, j])) - logits[r, targets[r]]: the negative log-likelihood of one given
 * token per row, without materialising the log-probabilities.  The log-probability is rounded once to
 * `dtype` as the reference's log_softmax output is.  Replaces the log_softmax + gather of
 * src/diff_gpt/diff_gpt.py:352-356 (DiffGPT.anomaly_scores).
 * logits: device [R, V] with row stride; targets: device int32 [R]; out: device fp32 [R].
 * A target outside [0, V) gives NaN for its row and sets bit 2 of *status (status may be NULL). */
int dgpt_token_nll(const void* logits, int64_t logits_row_stride, const int32_t* targets, float* out,
                   int32_t R, int32_t V, int32_t dtype, int32_t* status, void* stream);

/* Generated tokens -> float64 values for all trajectories of a series at once:
 *   value = (token - vocab_size / 2) / scale[channel], then order[channel] cumulative sums in time order,
 *   continued from the running sums the context leaves behind (state[channel][m] = level m + 1 at the end of
 *   the prompt).  Each addition has the operands and the order of the reference's numpy cumsum over the whole
 *   sequence, so the results are bit-identical to decoding every trajectory on the host.
 * Replaces the per-sample decode loop of src/diff_gpt/diff_gpt.py:236-252 (encoder_decoder.py:373-397, :97-152).
 * tokens: device int32 [n_traj, horizon * n_chan] (time-major, channel fastest) with row stride;
 * scale: device f64 [n_chan]; order: device int32 [n_chan] (each <= max_order <= 8);
 * state: device f64 [n_chan, max_order]; out: device f64 [n_traj, horizon, n_chan]. */
int dgpt_integrate_tokens(const int32_t* tokens, int64_t token_row_stride, int32_t n_traj, int32_t horizon,
                          int32_t n_chan, int32_t vocab_size, const double* scale, const int32_t* order,
                          const double* state, int32_t max_order, double* out, void* stream);

/* Values of many series -> prompt tokens in one launch (one thread per series and channel walks the rows):
 *   order[channel]-th finite differences, times scale[channel], then the quantiser the reference picks for the
 *   column: rounding (order 0 among per-column orders), the first-order sigma-delta, or the cascade of
 *   `order` first-order loops when vocab_size > 2^order + 2.  Every float64 operation is the one numpy
 *   performs, in its order: tokens and start rows are bit-identical to the host codec's.
 * Replaces the per-series call of src/diff_gpt/encoder_decoder.py:278-370 (:36-94, :155-226, :229-275).
 * values: device f64 [n_series, rows, n_chan] with series stride (elements);
 * order: device int32 [n_chan] (each <= max_order <= 8, max_order = the largest); scalar_order: 1 when the
 * model was given ONE order for all columns (start rows are then the first value of each difference level,
 * else the first max_order raw rows); scale: device f64 [n_chan];
 * tokens: device int32 [n_series, rows - max_order, n_chan];
 * start: device f64 [n_series, max_order, n_chan] or NULL;
 * state: device f64 [n_series, n_chan, max(max_order, 1)] or NULL: the running sums the decoder has reached at
 * the end of the prompt, which dgpt_integrate_tokens continues from. */
int dgpt_encode_series(const double* values, int64_t series_stride, int32_t n_series, int32_t rows,
                       int32_t n_chan, int32_t vocab_size, const int32_t* order, int32_t max_order,
                       int32_t scalar_order, const double* scale, int32_t* tokens, double* start,
                       double* state, void* stream);

/* *step_ptr += delta, as a one-thread kernel on `stream`: the last node of a captured decode step,
 * so that replaying the same launch sequence walks through the positions.  (The reference keeps the
 * position on the host: src/diff_gpt/model/kv_cache.py:113-115.) */
int dgpt_step_advance(int32_t* step_ptr, int32_t delta, void* stream);

/* Soft-cap, top-p filter and temperature sampling of one token per row, with teacher forcing.
 *   z        = cap * tanh(logits / cap)                  (cap == 0: z = logits)
 *   nucleus  = tokens whose probability mass BEFORE them, in descending softmax(z) order, is < top_p
 *              (top_p >= 1 disables the filter, top_p <= 0 keeps only the top token; ties broken by lower id first)
 *   token    = argmax z over the nucleus                 if temperature == 0
 *            = a draw from softmax(z / temperature) restricted to the nucleus.  Uniforms come from
 *              Philox4x32-10 with key = seed and counter = (traj id low, traj id high, step + step_base, a).
 *              Rows of up to 12000 tokens draw by rejection: attempt a = 0..7 is an inverse-CDF draw over
 *              ALL tokens, accepted if the token lies in the nucleus (accepted draws follow exactly the
 *              restricted distribution); after 8 rejections, and for wider rows always, the nucleus boundary
 *              is computed and one inverse-CDF draw is made inside it with a = 8 (wider rows: a = 0).
 *              The stream is a function of (seed, traj id, step) only: it does not depend on the batch,
 *              on the launch shape or on which GPU holds the row.
 *   f = force_schedule[(row / force_group_rows) * force_group_stride + step]   (one schedule per group of rows;
 *       stride 0 = one schedule for all);  if force_schedule && f >= 0: token = f, mask = 0, else mask = 1
 * step = *step_ptr (0 when NULL).  traj_ids (device int64 [R]) overrides traj_id0 + row when non-NULL.
 * Replaces src/diff_gpt/model/gpt.py:182-186 (cap), sampler/temperature.py:21-25,
 * sampler/nucleus.py:29-40 and the sample-or-force logic of model/engine.py:106-146.
 * logits: device [R, V] with row stride; out_tokens/out_masks: device int32 [R] (masks may be NULL);
 * history_tokens / history_masks: device int32 [R, history_stride] or NULL — column `step` is written. */
int dgpt_sample(const void* logits, int64_t logits_row_stride, int32_t R, int32_t V, float cap,
                float temperature, float top_p, uint64_t seed, int64_t traj_id0, const int64_t* traj_ids,
                int32_t step_base, const int32_t* step_ptr, const int32_t* force_schedule,
                int32_t force_group_rows, int64_t force_group_stride, int32_t* out_tokens, int32_t* out_masks, int32_t* history_tokens,
                int32_t* history_masks, int64_t history_stride, int32_t dtype, void* stream);

/* The model's head in one call: tied-embedding logits, soft-cap, and the draw of one token per row with teacher forcing.
 *   logits[r, v] = sum_c xn[r, c] * emb[v, c]          (xn = the final RMSNorm's output, dgpt_depthmix with one candidate)
 *   then exactly the rule of dgpt_sample (cap, top-p, temperature, forcing, history).
 * Replaces the tied nn.Linear and the cap of src/diff_gpt/model/gpt.py:181-186 together with
 * sampler/temperature.py:21-25, sampler/nucleus.py:29-40 and the sample-or-force step of model/engine.py:106-146.
 * Two forms, chosen by the arguments:
 *   - top_p < 1 (with temperature > 0), or logits_out non-NULL: the GEMM (tcgen05) writes bf16 logits [R, V] to
 *     logits_out, then the sampling kernel reads them; tokens are those of dgpt_linear + dgpt_sample.
 *   - otherwise the logits are never stored: the GEMM's epilogue soft-caps them, adds Gumbel noise from
 *     Philox4x32-10 with key = seed and counter = (traj id low, traj id high, step + step_base, 2^31 | token / 4)
 *     - the arg-max of z / T + noise is a draw from softmax(z / T); no noise for temperature 0 - and keeps each row's
 *     best (key, token) in `workspace`; ties go to the lower token.  Same distribution as dgpt_sample, another stream.
 * xn: device [R, C]; emb: device [V, C] (nn.Embedding layout); workspace: device, 8-byte aligned, from
 * dgpt_lmhead_workspace_bytes (second form only; cleared by the call).  bf16 only; C a multiple of 8, V of 16.
 * The remaining arguments are those of dgpt_sample.  status: device int32, set non-zero if a bounded wait ran out. */
size_t dgpt_lmhead_workspace_bytes(int32_t R);
int dgpt_lmhead_sample(const void* xn, int64_t xn_row_stride, const void* emb, int64_t emb_row_stride, float cap,
                       float temperature, float top_p, uint64_t seed, int64_t traj_id0, const int64_t* traj_ids,
                       int32_t step_base, const int32_t* step_ptr, const int32_t* force_schedule,
                       int32_t force_group_rows, int64_t force_group_stride, int32_t* out_tokens, int32_t* out_masks,
                       int32_t* history_tokens, int32_t* history_masks, int64_t history_stride, void* logits_out,
                       int64_t logits_row_stride, void* workspace, size_t workspace_bytes, int32_t R, int32_t C,
                       int32_t V, int32_t dtype, int32_t* status, void* stream);

/* filtered = logits where the token is in the top-p set (same rule as dgpt_sample, no soft-cap), -inf elsewhere.
 * Lets a top-p filter sit in front of an arbitrary inner sampler.
 * Replaces src/diff_gpt/sampler/nucleus.py:29-39.  logits, filtered: device [R, V] with row strides. */
int dgpt_nucleus_filter(const void* logits, int64_t logits_row_stride, void* filtered,
                        int64_t filtered_row_stride, int32_t R, int32_t V, float top_p, int32_t dtype,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DGPT_H_ */
