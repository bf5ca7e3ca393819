/*
 * dejavu_b200.h — C ABI of the B200 (sm_100a) contextual-sparse decode kernels.
 *
 * Every entry point
 *   - takes raw device pointers, plain sizes and a CUDA stream (as void*; NULL = legacy default stream),
 *   - only enqueues work on that stream: it never synchronises and never allocates or frees memory
 *     (scratch is caller-provided) unless its comment says otherwise,
 *   - returns DJV_OK (0) or a negative DJV_ERR_* code; djv_last_error() then holds a message
 *     for the calling thread,
 *   - does NOT validate index *values* on the device (like the kernels it replaces:
 *     Dejavu/src/ops/triton/gather_gemv.py:70), only shapes, alignment and limits on the host.
 *
 * All matrices are row-major fp16 ("half") unless stated. "ld" arguments are row strides in elements.
 * Citations name the interface in FMInference/DejaVu that each entry point replaces.
 */
#ifndef DEJAVU_B200_H
#define DEJAVU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DJV_OK 0
#define DJV_ERR_INVALID (-1)     /* bad pointer / shape / alignment / limit            */
#define DJV_ERR_UNSUPPORTED (-2) /* legal request this build has no kernel for         */
#define DJV_ERR_CUDA (-3)        /* CUDA runtime reported an error at launch           */
#define DJV_ERR_SCRATCH (-4)     /* caller-provided scratch too small                  */
#define DJV_ERR_TIMEOUT (-5)     /* a bounded device-side wait ran out (status word)   */

/* activation codes (Dejavu/src/ops/triton/gather_gemv.py:211) */
#define DJV_ACT_ID 0
#define DJV_ACT_RELU 1
#define DJV_ACT_GELU 2
#define DJV_ACT_GELU_APPROX 3
#define DJV_ACT_SQUARED_RELU 4

/* Limits shared with the host-side shims. */
#define DJV_MAX_BATCH 32        /* rows of x for the GEMV kernels                        */
#define DJV_KV_WINDOW 16        /* lazy K/V window (Dejavu/src/models/modules/mha_dejavu.py:1243) */

int djv_version(void);
/* Message of the last failing call on this thread ("" if none). */
const char *djv_last_error(void);
const char *djv_status_string(int status);
/* Number of kernels launched by this library on this process since load (all threads). */
unsigned long long djv_launch_count(void);
/* Per calling thread, default 0. While set, the gather / head-sparse kernels launched by this thread read
 * their index list (idx, head_idx, the attention state) and start fetching weight rows BEFORE they wait for the
 * kernel launched just before them on the stream (they are launched with programmatic dependent launch and
 * would otherwise idle until it has drained). It is a hint that the index arguments are already complete at
 * that point (produced on another stream and joined with an event some kernels earlier); it never changes a
 * result: the prefetching kernels only issue L2 prefetches from what they find, and the one-pass sparse MLP
 * kernel, which starts real copies, re-reads the list after the wait and starts over if it changed (and only
 * takes the hint when it is given the row count to bound the values, see djv_mlp_sparse_fused). Note that an
 * event wait in front of a programmatically launched kernel does not by itself order that kernel's pre-wait
 * reads after the event: inside a captured CUDA graph such an edge can be programmatic as well. Activations are
 * always read after the wait. Kernels without an index list (idx == NULL) always prefetch. No reference
 * counterpart. */
void djv_set_early_weight_prefetch(int enabled);

/* Per calling thread, default 1. Every kernel of the library is launched with programmatic dependent launch and
 * lets its successor start (and wait) as soon as all its own blocks have started: the successor's launch latency
 * and prologue overlap the kernel's tail. That pays when kernels are short and fit the device in one wave (decode
 * with one sequence: OPT-66B 7.18 ms per token with it, 7.4 without). In decode steps of several sequences it was
 * measured to cost far more than it hides (OPT-6.7B, ms per step with / without: 2 sequences 4.58 / 2.37, 16
 * sequences 6.3 / 4.7). The step timeline shows why: successors launched early sit on the multiprocessors waiting,
 * and a kernel of another stream that they depend on through an event (in the batched step: the host framework's
 * own reduction kernels of the look-ahead predictor) finds no free slot for some 200 us per layer. 0 launches the
 * kernels of this thread as plain stream-ordered kernels. Never changes a result. */
void djv_set_programmatic_launch(int enabled);

/* ---------------------------------------------------------------------------------------------
 * L2 warm-up for short index lists (no counterpart in the reference). When the rows a rank reads per layer fit
 * the L2 cache, the kernels of the decode step are bound by memory latency; these calls ask, as soon as an
 * index list exists, for the rows it names to be brought into L2 (bulk prefetches issued by a tiny kernel), so
 * that the consumers find them there. Pure hints: no result depends on them; indices outside [0, Z) are skipped.
 *   djv_prefetch_rows_l2: rows idx[0..M) of up to three matrices sharing the list (NULL = absent), a row being
 *     row_bytes contiguous bytes at base + idx[m] * ld_bytes (fc1 / fc2^T rows; the q, k, v slabs of a head).
 *   djv_prefetch_segments_l2: for every row n < nrows of w the seg_bytes at n * ld_bytes + idx[i] * seg_bytes
 *     (the columns of out_proj.weight that belong to the listed heads). idx int32.
 * ------------------------------------------------------------------------------------------- */
int djv_prefetch_rows_l2(const void *w0, const void *w1, const void *w2, const void *idx, int idx_is_64, int M,
                         int Z, long long ld_bytes, long long row_bytes, void *stream);
int djv_prefetch_segments_l2(const void *w, const int32_t *idx, int M, int Z, int nrows, long long ld_bytes,
                             int seg_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Gather GEMV (fc1):  y[b,m] = act( sum_n w[idx[m],n] * x[b,n] + bias[idx[m]] ),  b<B, m<M.
 * Replaces gather_gemv / gather_gemv_kernel, Dejavu/src/ops/triton/gather_gemv.py:198-254, 23-195.
 *   y (B,M) fp16 | w (Z,N) rows of stride ldw | x (B,N) | idx (M,) int32 or int64 (idx_is_64), or
 *   NULL for the identity (dense GEMV over rows 0..M-1) | bias (Z,) or NULL.
 * Requirements: N % 8 == 0, ldw % 8 == 0, w/x 16-byte aligned, 1 <= B <= DJV_MAX_BATCH.
 * fp32 accumulation, one rounding to fp16 at the store.
 * ------------------------------------------------------------------------------------------- */
int djv_gather_gemv(void *y, const void *w, const void *x, const void *idx, const void *bias,
                    int B, int N, int M, long long ldw, int idx_is_64, int act, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Gather transposed GEMV (fc2):  y[b,n] = sum_m w[idx[m],n] * x[b,m] + bias[n].
 * Replaces gather_transposed_gemv, Dejavu/src/ops/triton/gather_gemv.py:572-644 (both its
 * atomic-add and its deterministic kernel, :432-569 and :263-425). Deterministic: partial sums over
 * fixed row chunks are written to scratch and combined in a fixed order (B <= 2: by the last block to finish;
 * 3 <= B <= 32: tensor-core kernel, one pass over the gathered rows whatever B is, then a small second kernel
 * that adds the row chunks).
 *   y (B,N) fp16 | w (Z,N) stride ldw = W2 transposed | x (B,M) | idx (M,) or NULL | bias (N,) or NULL.
 *   scratch: at least djv_gather_transposed_gemv_scratch_bytes(B,N,M) bytes, 256-byte aligned, and its
 *   first 4096 bytes must be ZERO before the first call (the kernel leaves them zero again).
 *   Calls that share scratch must not overlap on the GPU.
 * ------------------------------------------------------------------------------------------- */
size_t djv_gather_transposed_gemv_scratch_bytes(int B, int N, int M);
int djv_gather_transposed_gemv(void *y, const void *w, const void *x, const void *idx,
                               const void *bias, int B, int N, int M, long long ldw, int idx_is_64,
                               void *scratch, size_t scratch_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * The same product as djv_gather_transposed_gemv, for callers that have no scratch memory to give.
 * This entry point has no counterpart in the reference: it exists for hosts that cannot allocate device
 * memory at the call site (all of it already handed to their own pool, allocation forbidden in the calling
 * context, or a binding with no workspace concept).
 * The scratch is a built-in device array of DJV_STATIC_SCRATCH_BYTES that every GPU loading the library
 * holds until exit; requests that need more (large B*N with many row chunks) are refused with
 * DJV_ERR_SCRATCH and a message. The call allocates and frees nothing. The first call made while a given
 * device is current resolves the array's device address: issue that first call outside of any stream
 * capture. All calls on a device share the array, so calls that could overlap on the GPU must be ordered
 * by the caller; the array's previous contents never influence a result.
 *   1 <= B <= 4, M >= 1; other arguments as djv_gather_transposed_gemv.
 * ------------------------------------------------------------------------------------------- */
#define DJV_STATIC_SCRATCH_BYTES (4096u + (256u << 10))
int djv_gather_transposed_gemv_static(void *y, const void *w, const void *x, const void *idx,
                                      const void *bias, int B, int N, int M, long long ldw, int idx_is_64,
                                      void *stream);

/* ---------------------------------------------------------------------------------------------
 * Sparse MLP in one call: y = gather_transposed_gemv(relu(gather_gemv(x,W1,idx,b1)), W2t, idx, b2).
 * Replaces mlp_sparse, Dejavu/src/ops/triton/gather_gemv.py:647-657. h is rounded to fp16 between
 * the two products exactly as there (:233). h (B,M) fp16 is caller-provided workspace.
 * ------------------------------------------------------------------------------------------- */
int djv_mlp_sparse(void *y, void *h, const void *w1, const void *w2t, const void *x, const void *idx,
                   const void *bias1, const void *bias2, int B, int N, int M, long long ldw1,
                   long long ldw2t, int idx_is_64, void *scratch, size_t scratch_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * The same sparse MLP in ONE kernel and one pass over the gathered rows: the block that streams row idx[m] of
 * W1 and of W2t computes h_m = relu(w1[idx[m],:] . x + bias1[idx[m]]), rounds it to fp16 as the reference
 * does between its two kernels (Dejavu/src/ops/triton/gather_gemv.py:233), and at once adds
 * h_m * w2t[idx[m],:] to the output sums. Replaces mlp_sparse, gather_gemv.py:647-657 (two launches, a
 * zero-fill and a cast there). Deterministic. 1 <= B <= 4, N % 64 == 0, N <= 24576, M >= 1
 * (djv_mlp_sparse_fused_supported says whether a shape qualifies; use djv_mlp_sparse otherwise).
 *   scratch: djv_mlp_sparse_fused_scratch_bytes(B,N,M) bytes, 256-byte aligned, first 4096 bytes ZERO before
 *   the first call (left zero again); calls that share scratch must not overlap on the GPU.
 * Z: number of rows of w1 / w2t, or 0. With Z > 0 the kernel checks every index value it uses: a value outside
 * [0, Z) is counted (djv_mlp_ring_bad_indices) and row 0 is read in its place, instead of an access outside the
 * matrices. With Z = 0 index values are not checked, as in the kernels this replaces. Only with Z > 0 does the
 * kernel honour djv_set_early_weight_prefetch: it then starts its weight copies from the index list as it finds
 * it before its predecessor has finished, reads the list again afterwards and starts the copies anew should
 * any entry have changed, so the hint can never change a result.
 * djv_mlp_ring_timeouts(): how many bounded waits on the kernel's own asynchronous copies ever ran out in
 * this process (0 in a healthy run; synchronises).
 * ------------------------------------------------------------------------------------------- */
int djv_mlp_sparse_fused_supported(int B, int N, int M);
/* 1 when the index list is short enough for every block to keep all of its rows in flight at once (the regime
 * the one-pass kernel is built for: a tensor-parallel shard's few hundred rows); host-side heuristic. */
int djv_mlp_sparse_fused_single_batch(int B, int N, int M);
size_t djv_mlp_sparse_fused_scratch_bytes(int B, int N, int M);
unsigned djv_mlp_ring_timeouts(void);
unsigned djv_mlp_ring_bad_indices(void);
int djv_mlp_sparse_fused(void *y, const void *w1, const void *w2t, const void *x, const void *idx,
                         const void *bias1, const void *bias2, int B, int N, int M, int Z, long long ldw1,
                         long long ldw2t, int idx_is_64, void *scratch, size_t scratch_bytes, void *stream);

/* y[n] = sum_b x[b,n] for x (B,N) fp16, added in fp32 in row order and rounded once: the batch sum in front of
 * (or behind) the linear sparsity predictors when several sequences share one index set. No reference counterpart
 * (its decode path keeps one sequence, mha_dejavu.py:1318, 1469). */
int djv_batch_sum(void *y, const void *x, int B, int N, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Top-K index selection over one score vector.
 * Replaces mlp_sp_logit.topk(K, sorted=False) / att_sp_logit.topk(K) + .to(int32),
 * Dejavu/src/models/modules/mha_dejavu.py:1069, 1369, 1506-1507.
 * Rule: the K largest scores; ties on the K-th score go to the LOWEST indices; NaN ranks above +inf.
 * Output: K indices in ascending index order, written as int32 to idx32 and/or int64 to idx64
 * (either may be NULL). scores: fp16 (score_is_f32 = 0) or fp32. 0 <= K <= n, n*elemsize <= 1600 KiB
 * (DJV_ERR_UNSUPPORTED above). n >= 4096 runs as a cluster of 8 blocks (each holds an eighth of the keys in its
 * shared memory), shorter vectors as one block; both give the same index list.
 * ------------------------------------------------------------------------------------------- */
int djv_topk(int32_t *idx32, int64_t *idx64, const void *scores, int n, int K, int score_is_f32,
             void *stream);

/* ---------------------------------------------------------------------------------------------
 * Head-sparse QKV projection with the reference's operator semantics:
 *   y[t,q,h,:] = x[t,:] . w[q,h,:,:]^T + bias[q,h,:]  for h in head_idx and token rows t with
 *   batch_idx[i,t] >= 0 (i = position of h in head_idx); other entries of y are left untouched.
 * Replaces qkv_proj_sparse, Dejavu/src/ops/triton/attention_proj_sparse.py:110-194.
 *   y (T,3,nheads,hd) | w (3,nheads,hd,d) contiguous | x (T,d), T <= 16 | head_idx (nnz,) int32 |
 *   batch_idx (nnz,T) int32 | bias (3,nheads,hd) or NULL. hd in {32,64,128}, d % 8 == 0.
 * ------------------------------------------------------------------------------------------- */
int djv_qkv_proj_sparse(void *y, const void *w, const void *x, const int32_t *head_idx,
                        const int32_t *batch_idx, const void *bias, int T, int d, int nheads, int hd,
                        int nnz, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Head-sparse output projection: y[b,n] = sum_{h in head_idx} x[b,h,:] . w[n,h,:] + bias[n].
 * Replaces out_proj_sparse, Dejavu/src/ops/triton/attention_proj_sparse.py:274-338.
 *   y (B,d) | w (d,nheads,hd) contiguous (= out_proj.weight viewed per head) | x (B,nheads,hd) |
 *   head_idx (nnz,) int32 | bias (d,) or NULL. B <= 16.
 * n_active_dev: optional device int32; when non-NULL only the first *n_active_dev entries of head_idx
 * are used (nnz is then the capacity of head_idx).
 * ------------------------------------------------------------------------------------------- */
int djv_out_proj_sparse(void *y, const void *w, const void *x, const int32_t *head_idx,
                        const int32_t *n_active_dev, const void *bias, int B, int d, int nheads, int hd,
                        int nnz, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Scatter recomputed K / V rows of selected heads into the decode caches.
 * Replace k_cache_copy_sparse / v_cache_copy_sparse,
 * Dejavu/src/ops/triton/attention_proj_sparse.py:525-590, 396-456.
 *   k, v (T,nheads,hd) (may be strided views: row stride ld_t, head stride ld_h, in elements)
 *   k_cache (1,nheads,hd/8,S,8)   v_cache (1,nheads,S,hd)
 *   head_idx (nnz,) int32 | seqlen_idx (nnz,T) int32, negative = skip |
 *   padding: device int32 added to every destination position, or NULL (= 0).
 * ------------------------------------------------------------------------------------------- */
int djv_k_cache_copy_sparse(const void *k, void *k_cache, const int32_t *head_idx,
                            const int32_t *seqlen_idx, const int32_t *padding, int T, int nheads,
                            int hd, int S, int nnz, long long ld_t, long long ld_h, void *stream);
int djv_v_cache_copy_sparse(const void *v, void *v_cache, const int32_t *head_idx,
                            const int32_t *seqlen_idx, const int32_t *padding, int T, int nheads,
                            int hd, int S, int nnz, long long ld_t, long long ld_h, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Lazy-K/V decode state of one attention layer, kept on the device so that a captured CUDA graph
 * replays correctly. Replaces ParallelTracker + x_cache + counter + cache_offset,
 * Dejavu/src/models/modules/mha_dejavu.py:1124-1149, 1243-1253, 1318-1329, 1355-1359, 1485-1492.
 *
 * struct layout (int32 words) of `state`, DJV_ATTN_STATE_WORDS + nheads words in total:
 *   [0] slot      position of the current token inside the 16-token window (0..15)
 *   [1] base      cache position of window slot 0
 *   [2] n_eff     number of heads in use this step (after the every-16th-step flush rule)
 *   [3] status    0, or DJV_ERR_* written by a kernel that found the state inconsistent
 *   [4..7] reserved
 *   [8 .. 8+nheads)          pending[h]: bit s set = head h has no K,V yet for window slot s
 *   [8+nheads .. 8+2*nheads) eff_heads[i], i < n_eff: heads in use this step
 *   [8+2*nheads .. 8+3*nheads) rowmask[i]: window slots whose K,V this step computes for eff_heads[i]
 * ------------------------------------------------------------------------------------------- */
#define DJV_ATTN_STATE_HDR 8
#define DJV_ATTN_STATE_WORDS(nheads) (DJV_ATTN_STATE_HDR + 3 * (nheads))

/* state := {slot 0, base = prompt_len, nothing pending}. */
int djv_attn_state_reset(int32_t *state, int nheads, int prompt_len, void *stream);

/* One decode step of the head-sparse attention block for batch 1 (mha_dejavu.py:1312-1359, 1422-1446):
 *   1. x_ring[slot] = x; choose the heads in use: head_idx[0..nnz) (device int32), or ALL heads when
 *      slot == 15 (flush rule, :1320-1325) or when head_idx == NULL (dense step);
 *   2. for each head in use: K,V for every window slot it still lacks (plus the current one) are
 *      projected from x_ring and written straight into the caches at base+slot; q of the current
 *      token goes to q_out (nheads,hd); heads not in use get the current slot marked pending;
 *   3. single-query softmax attention over cache positions [0, base+slot] for the heads in use,
 *      scale = softmax_scale, context written to ctx (nheads,hd) (rows of unused heads untouched);
 *   4. advance: slot+1, and after slot 15: slot = 0, base += 16.
 * Step 4 happens in djv_attn_step_finish so that djv_out_proj_sparse can still read eff_heads/n_eff.
 *   wqkv (3,nheads,hd,d) | bqkv (3,nheads,hd) or NULL | x (d,) | x_ring (16,d) |
 *   k_cache (1,nheads,hd/8,S,8) | v_cache (1,nheads,S,hd) | scratch >= djv_attn_step_scratch_bytes().
 * ------------------------------------------------------------------------------------------- */
size_t djv_attn_step_scratch_bytes(int nheads, int hd, int S);
int djv_attn_step(void *ctx, void *q_out, const void *wqkv, const void *bqkv, const void *x,
                  void *x_ring, void *k_cache, void *v_cache, int32_t *state,
                  const int32_t *head_idx, int nnz, int d, int nheads, int hd, int S,
                  float softmax_scale, void *scratch, size_t scratch_bytes, void *stream);
/* The same step as two calls, for a caller that wants to fork other work onto a second stream between the
 * projection and the attention (the look-ahead head predictor, mha_dejavu.py:1364-1370):
 * djv_attn_step_project = steps 1-2, djv_attn_step_attend = step 3 (q = the q_out of the first call). */
int djv_attn_step_project(void *q_out, const void *wqkv, const void *bqkv, const void *x, void *x_ring,
                          void *k_cache, void *v_cache, int32_t *state, const int32_t *head_idx, int nnz,
                          int d, int nheads, int hd, int S, int step_is_open, void *stream);
/* The same two calls for B sequences that decode in lockstep and share ONE state: one head selection per layer
 * and step (the reference's decode path keeps one sequence, mha_dejavu.py:1318, 1469; its kernels take one index
 * list for all rows of a batch) and therefore one window position and one set of pending rows. Per-sequence data is
 * contiguous over the batch: q_out / q / ctx (B,nheads,hd), x (B,d), x_ring (B,16,d), k_cache (B,nheads,hd/8,S,8),
 * v_cache (B,nheads,S,hd); scratch >= djv_decode_attn_scratch_bytes(nheads, B, hd, S). One launch each whatever B
 * is: the blocks of all sequences that work on the same weight rows run side by side and share them through L2. */
int djv_attn_step_project_batch(void *q_out, const void *wqkv, const void *bqkv, const void *x, void *x_ring,
                                void *k_cache, void *v_cache, int32_t *state, const int32_t *head_idx, int nnz,
                                int d, int nheads, int hd, int S, int B, void *stream);
int djv_attn_step_attend_batch(void *ctx, const void *q, const void *k_cache, const void *v_cache, int32_t *state,
                               int B, int nheads, int hd, int S, float softmax_scale, void *scratch,
                               size_t scratch_bytes, void *stream);
/* Top-K of the head predictor's scores (one score per head of this rank) that also opens the decode step
 * of the attention layer the selection is for: djv_topk(idx32, ...) followed by the head-selection half of
 * step 1 above on `state`, in one launch, off the critical path (mha_dejavu.py:1364-1370 computes the
 * selection for the next layer on a side stream). The x_ring[slot] = x half of step 1 is then done by
 * djv_attn_step_project(..., step_is_open = 1, ...), which also skips its own step-1 launch; head_idx and
 * nnz of that call are this call's idx32 and K. */
int djv_topk_attn_prep(int32_t *idx32, const void *scores, int n, int K, int score_is_f32, int32_t *state,
                       int S, void *stream);
int djv_attn_step_attend(void *ctx, const void *q, const void *k_cache, const void *v_cache, int32_t *state,
                         int nheads, int hd, int S, float softmax_scale, void *scratch, size_t scratch_bytes,
                         void *stream);
int djv_attn_step_finish(int32_t *state, int nheads, void *stream);

/* Single-query attention over the caches for an explicit head list (no lazy state):
 *   ctx[b,h,:] = softmax(scale * q[b,h,:] . K[b,h,0..len))) V[b,h,0..len)  for h in head_idx
 * Replaces the call ft_attention.single_query_attention(...), mha_dejavu.py:1439-1446 (third-party
 * kernel, flash-attention v0.2.8 csrc/ft_attention) restricted to the heads that are read afterwards.
 *   q, ctx (B,nheads,hd) | k_cache (B,nheads,hd/8,S,8) | v_cache (B,nheads,S,hd) |
 *   head_idx (nnz,) int32 or NULL = all heads | len = number of cached positions to attend to.
 * ------------------------------------------------------------------------------------------- */
size_t djv_decode_attn_scratch_bytes(int nnz, int B, int hd, int S);
int djv_decode_attn(void *ctx, const void *q, const void *k_cache, const void *v_cache,
                    const int32_t *head_idx, int nnz, int B, int nheads, int hd, int S, int len,
                    float softmax_scale, void *scratch, size_t scratch_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Residual add + LayerNorm:  r = x + residual (+ xbias);  y = LN(r) * gamma + beta.
 * Replaces the un-fused `residual = dropped + residual; hidden = norm(residual)`,
 * Dejavu/src/models/modules/block_dejavu.py:575-584, 625-636. r is rounded to fp16 before the
 * statistics are taken, as the reference's fp16 add does.
 *   x, residual, r_out, y (B,d) | xbias (d,) or NULL | residual may be NULL (r = x) |
 *   r_out may alias residual.
 * ------------------------------------------------------------------------------------------- */
int djv_add_layernorm(void *y, void *r_out, const void *x, const void *residual, const void *xbias,
                      const void *gamma, const void *beta, int B, int d, float eps, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Tensor-parallel one-shot all-reduce fused with the residual add and LayerNorm that follow it:
 *   r = sum_ranks(partial) + residual;  y = LN(r)
 * Replaces all_reduce(out, process_group) at mha_dejavu.py:1498 and
 * Dejavu/src/ops/fused_dense_sparse_dejavu.py:937-940 together with the add + norm of
 * block_dejavu.py:575-584, 625-636. Every rank stores its partial into every rank's receive buffer
 * (plain stores over NVLink, the data is its own arrival flag) and sums the pieces it received in rank
 * order (deterministic, identical on all ranks); waits on peers are bounded and report
 * DJV_ERR_TIMEOUT through comm->status instead of hanging.
 *
 * djv_comm is created per process from peer-mapped buffers the host exchanged (CUDA IPC):
 *   bufs[r] : rank r's receive buffer of djv_comm_buffer_bytes(world, slot_bytes) bytes, mapped into this
 *             process; bufs[rank] is this rank's own and is initialised by djv_comm_create.
 * world = 1 is allowed (one buffer, this process's own): the same kernels then run on a single GPU.
 * Every rank must have returned from djv_comm_create before any rank runs an exchange.
 *
 * Numbering. The exchanges of one decode step are numbered seq = 0, 1, 2, ... by the caller, identically on
 * every rank; a producer (*_push) and every consumer of the same exchange pass the same seq. After the last
 * kernel of the step that touches the exchange (all streams joined) the caller runs
 * djv_comm_end_step(comm, number of exchanges of the step), and numbering restarts at 0. seq is a launch
 * argument, so a captured CUDA graph of one step replays correctly. Consecutive exchanges use consecutive
 * receive slots (4 per rank).
 * Exactly ONE consumer of each exchange, on the stream that also runs the producers, passes
 * DJV_EXCHANGE_REFILL: it recycles the slot used two exchanges earlier. Further consumers of the same exchange
 * (on other streams) must not pass it, and whatever they produce must be waited for by the refilling consumer
 * of exchange seq + 2 (in the decode step: the look-ahead predictor's result is needed two exchanges later).
 * ------------------------------------------------------------------------------------------- */
typedef struct djv_comm djv_comm;
#define DJV_EXCHANGE_REFILL 1
/* Set-up helpers (these DO allocate / free with cudaMalloc / cudaFree and zero the memory): a buffer
 * that is the base of its own allocation, as CUDA IPC handles require. */
int djv_ipc_alloc(size_t bytes, void **dev_ptr_out);
int djv_ipc_free(void *dev_ptr);
int djv_ipc_get_handle(const void *dev_ptr, unsigned char handle_out[64]);
int djv_ipc_open(const unsigned char handle[64], void **dev_ptr_out);
int djv_ipc_close(void *dev_ptr);
size_t djv_comm_buffer_bytes(int world, size_t slot_bytes);
int djv_comm_create(djv_comm **out, int rank, int world, void *const *bufs, size_t slot_bytes);
int djv_comm_destroy(djv_comm *comm);
/* Reads the device status word (synchronises the stream the comm last ran on). */
int djv_comm_status(djv_comm *comm);
/* Closes a step: the next step's exchange 0 follows this step's exchange n_exchanges - 1 (one tiny kernel). */
int djv_comm_end_step(djv_comm *comm, int n_exchanges, void *stream);
/* The two producers of a rank's partial sums can send them into every rank's receive buffer themselves, as
 * they finish each piece, so that the NVLink trip overlaps their tail and the launch of the consumer:
 * same arguments as djv_gather_transposed_gemv / djv_out_proj_sparse with `comm, seq` in place of y (B <= 4,
 * B*N*2 <= slot_bytes). The consumers of that exchange pass partial = NULL.
 * Exactly one producer call per exchange, on the same stream as its refilling consumer, before it. */
int djv_gather_transposed_gemv_push(djv_comm *comm, int seq, const void *w, const void *x, const void *idx,
                                    const void *bias, int B, int N, int M, long long ldw, int idx_is_64,
                                    void *scratch, size_t scratch_bytes, void *stream);
int djv_out_proj_sparse_push(djv_comm *comm, int seq, const void *w, const void *x, const int32_t *head_idx,
                             const int32_t *n_active_dev, const void *bias, int B, int d, int nheads, int hd,
                             int nnz, void *stream);
/* Consumer as a kernel of its own (one cluster of 8 blocks per row).
 * partial: this rank's (B,d) fp16 partial sums, or NULL when a *_push call has sent them. B*d*2 <= slot_bytes.
 * gamma = beta = NULL: no LayerNorm, y = r (either of y, r_out may be NULL). flags: DJV_EXCHANGE_REFILL. */
int djv_allreduce_add_layernorm(djv_comm *comm, int seq, int flags, void *y, void *r_out, const void *partial,
                                const void *residual, const void *gamma, const void *beta, int B, int d,
                                float eps, void *stream);
/* The second half of a decoder block in one launch (typedef above):
 *   r = sum_ranks(pieces of exchange seq_in) + residual;  x = LN(r) * gamma + beta;
 *   out = djv_mlp_sparse_fused(x, ...)  ->  sent as exchange seq_out (seq_out >= 0), or stored to y.
 * Replaces the chain all_reduce -> residual add -> norm2 -> mlp_sparse -> (all_reduce), i.e.
 * Dejavu/src/models/modules/mha_dejavu.py:1498, block_dejavu.py:625-636,
 * Dejavu/src/ops/fused_dense_sparse_dejavu.py:914-940. The weight stream of the MLP starts before the wait on
 * the peers (see djv_set_early_weight_prefetch). r_out (B,N) or NULL receives r. flags: DJV_EXCHANGE_REFILL.
 * Shapes and scratch as djv_mlp_sparse_fused; B*N*2 <= slot_bytes. */
int djv_mlp_sparse_fused_exchange(djv_comm *comm, int seq_in, int flags, int seq_out, void *y, void *r_out,
                                  const void *residual, const void *gamma, const void *beta, float eps,
                                  const void *w1, const void *w2t, const void *idx, const void *bias1,
                                  const void *bias2, int B, int N, int M, int Z, long long ldw1, long long ldw2t,
                                  int idx_is_64, void *scratch, size_t scratch_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DEJAVU_B200_H */
