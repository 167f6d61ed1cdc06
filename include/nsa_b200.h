/* C interface of libnsa_b200: the Native Sparse Attention hot path as sm_100a CUDA kernels.
 *
 * Conventions for every entry point
 *   - all pointers are DEVICE pointers unless stated otherwise; nothing is allocated or freed
 *     by the library (callers own every buffer, including scratch);
 *   - strides are in ELEMENTS; the innermost (head_dim) stride is 1; token and head strides
 *     must be multiples of 8 elements and base addresses 16-byte aligned;
 *   - `dtype` is NSA_DTYPE_BF16 (0) or NSA_DTYPE_FP16 (1); head_dim is 64 or 128;
 *   - `stream` is a cudaStream_t; the call is asynchronous on that stream of the CURRENT device;
 *   - return value: 0 ok, -1 invalid argument, -2 unsupported configuration, -3 scratch too
 *     small, 1000+e CUDA runtime error e.  Device-side anomalies (a bounded wait that gave
 *     up, an index out of range) never hang or trap: they are OR-ed into a per-device status
 *     word that nsa_last_device_status() returns and clears.
 *
 * Each declaration cites the function of the reference project
 * (XunhaoLai/native-sparse-attention-triton, paths relative to its root) whose device work it
 * replaces.
 */
#ifndef NSA_B200_H_
#define NSA_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

#define NSA_DTYPE_BF16 0
#define NSA_DTYPE_FP16 1

/* Library version, (major << 16) | minor. */
int nsa_version(void);

/* OR of the device-side error bits raised since the last call (1 = bounded wait timed out,
 * 2 = index out of range); synchronises `stream`.  No counterpart in the reference. */
int nsa_last_device_status(void* stream);

/* Forward of attention over selected KV blocks.
 * Replaces _topk_sparse_attention_fwd / forward_kernel,
 * native_sparse_attention/ops/triton/topk_sparse_attention.py:26-173,828-909.
 *   q [total_len, num_q_heads, d], k/v [total_len, num_kv_heads, d], o like q,
 *   topk_idx int32 [num_kv_heads, total_len, topk] (valid ids first, -1 padding),
 *   cu_seqlens int32 [batch+1], lse fp32 [total_len, num_q_heads] (base-2, scaled logits).
 *   strides[11] = {q_n, q_h, k_n, k_h, v_n, v_h, o_n, o_h, idx_h, idx_n, idx_k}. */
int nsa_topk_sparse_attn_fwd(const void* q, const void* k, const void* v, const int* topk_idx,
                             const int* cu_seqlens, void* o, float* lse, int total_len, int batch,
                             int num_q_heads, int num_kv_heads, int head_dim, int topk, int block_size,
                             const long long* strides, float sm_scale, int dtype, void* stream);

/* Forward of dense varlen GQA attention with the strided-causal mask
 *     query at in-sequence position t sees key i  iff  t >= i*stride + window - 1   (causal != 0)
 * window = kernel_size, stride = kernel_stride: attention over compressed keys, replaces
 * _compressed_attention_fwd / forward_kernel, native_sparse_attention/ops/triton/compressed_attention.py:27-158,538-615.
 * window = stride = 1 (causal) or causal = 0 (full): replaces _flash_attention_fwd,
 * native_sparse_attention/ops/triton/flash_attention.py:26-165,563-657.
 *   q [total_q, Hq, d], k/v [total_k, Hkv, d], o like q, lse fp32 [total_q, Hq] (base 2);
 *   rows without a visible key get o = 0 and lse = -inf.
 *   strides[8] = {q_n, q_h, k_n, k_h, v_n, v_h, o_n, o_h}. */
int nsa_varlen_attn_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens_q,
                        const int* cu_seqlens_k, void* o, float* lse, int total_q, int total_k, int batch,
                        int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim, int causal,
                        int window, int stride, const long long* strides, float sm_scale, int dtype,
                        void* stream);

/* Block scores and top-k block selection for every query token, from q, the compressed keys and the
 * forward pass's lse.  Replaces _get_attention_score + transform_score + torch.topk/sort/mask,
 * native_sparse_attention/ops/triton/compressed_attention.py:851-1179,1245-1330.
 *   topk_idx int32 [Hkv, total_q, min(topk, ceil(max_seqlen_q/block_size))]: ascending ids, -1 padding.
 *   strides[7] = {q_n, q_h, k_n, k_h, idx_h, idx_n, idx_k}. */
int nsa_compressed_attn_topk(const void* q, const void* k, const float* lse, const int* cu_seqlens_q,
                             const int* cu_seqlens_k, int* topk_idx, int total_q, int total_k, int batch,
                             int max_seqlen_q, int num_q_heads, int num_kv_heads, int head_dim,
                             int kernel_size, int kernel_stride, int block_size, int topk, int init_blocks,
                             int local_blocks, const long long* strides, float sm_scale, int dtype,
                             void* stream);

/* Linear compression forward: y[m,h,:] = concat_k(x[s+m*stride+k,h,:]) @ w[h] (+ concat_k(pe[h,k,:]) @ w[h]).
 * Replaces LinearCompress.forward + the bias einsum,
 * native_sparse_attention/ops/triton/linear_compress.py:26-136,309-417,497-525.
 *   x [N, H, d] (strides x_stride_n, x_stride_h), w [H, kernel_size*d, d] contiguous, pe [H, kernel_size, d]
 *   contiguous or NULL, y [total_y, H, d] contiguous, y_cu_seqlens int32 [batch+1],
 *   bias_scratch [H, d] of the storage type (needed iff pe != NULL); total_len = N, the rows of x (the bound of the
 *   TMA views of x: head_dim 128 with at least 128 windows in some sequence runs as one tcgen05 GEMM per
 *   (sequence, head) whose operands TMA fetches; other shapes on the warp-level tensor-core kernel). */
int nsa_linear_compress_fwd(const void* x, const void* w, const void* pe, const int* cu_seqlens,
                            const int* y_cu_seqlens, void* y, void* bias_scratch, int total_len, int batch,
                            int total_y, int max_y_len, int num_heads, int head_dim, int kernel_size,
                            int kernel_stride, long long x_stride_n, long long x_stride_h, int dtype, void* stream);

/* Weighted (w [H, kernel_size]) or average (w == NULL) pooling compression forward.
 * Replaces SlidingWindowWeightedPool.forward + the bias einsum/mean,
 * native_sparse_attention/ops/triton/weighted_pool.py:23-85,182-239,301-363.
 *   Arguments as nsa_linear_compress_fwd (total_len = rows of x, max_y_len = longest compressed sequence).  Inputs of
 *   8192 windows or more (head_dim 128) stream through shared memory in TMA chunks, every row fetched once; shorter ones
 *   (and the single rows of a decode step) use one thread per window and 16-byte column group. */
int nsa_pool_compress_fwd(const void* x, const void* w, const void* pe, const int* cu_seqlens,
                          const int* y_cu_seqlens, void* y, void* bias_scratch, int total_len, int batch,
                          int total_y, int max_y_len, int num_heads, int head_dim, int kernel_size,
                          int kernel_stride, long long x_stride_n, long long x_stride_h, int dtype, void* stream);

/* The compression of a decode step for both pooling modes, K and V in one launch: every sequence contributes exactly
 * one window, the kernel_size rows of its staging buffer (x_k, x_v: [batch, kernel_size, H, d] views with strides
 * x_stride_b, x_stride_n, x_stride_h), so no cu_seqlens is read.  w_k / w_v [H, kernel_size] or NULL (average); bias_k /
 * bias_v [H, d] (the position embedding folded through the weights by nsa_pool_bias, which does not change between steps)
 * or NULL; y_k, y_v [batch, H, d] contiguous.  Replaces the two compress_func calls on the staging buffers in
 * native_sparse_attention/infer/inference_func.py:56-87 when both are pooling operators. */
int nsa_pool_compress_decode_pair(const void* x_k, const void* x_v, const void* w_k, const void* w_v, const void* bias_k,
                                  const void* bias_v, void* y_k, void* y_v, int batch, int num_heads, int head_dim,
                                  int kernel_size, long long x_stride_b, long long x_stride_n, long long x_stride_h,
                                  int dtype, void* stream);

/* bias[h, :] = sum_k w[h, k] * pe[h, k, :] (w == NULL: the mean over k), in the storage type: the term the pooling
 * operators add to every compressed row (native_sparse_attention/ops/triton/weighted_pool.py:301-363). */
int nsa_pool_bias(const void* pe, const void* w, void* bias, int num_heads, int head_dim, int kernel_size, int dtype,
                  void* stream);

/* Number of split-KV partitions the decode kernels want for this problem (>= 1; max_tiles = 64-key tiles of the longest
 * row a pair can have), and the floats of scratch a call with that many splits needs: control words (a task counter and a
 * per-(sequence, KV head) counter at the FRONT of the scratch: batch*num_kv_heads + 1 ints), the splits' partial results
 * and, for the compressed operator, the logits of every compressed key (cache_len keys per pair).  The control words must
 * be ZERO before the first call that uses a scratch buffer; every completed call leaves them zero again (they count with
 * wrap-around), so a buffer cleared once can be reused by any sequence of calls that do not overlap on the GPU -- except
 * that a call with MORE pairs than the previous call on the same buffer must clear its (longer) control region again,
 * because the previous call's partial results start right behind the shorter one.  One split of the flash / top-k
 * operators needs no scratch.  No counterpart in the reference. */
int nsa_decode_num_splits(int batch, int num_kv_heads, int max_tiles);
long long nsa_decode_scratch_floats(int batch, int num_kv_heads, int head_dim, int num_splits);
long long nsa_compressed_decode_scratch_floats(int batch, int num_kv_heads, int head_dim, int num_splits, int cache_len);

/* Single-token attention over the first seqlens[b] rows of a dense cache.
 * Replaces decode_kernel, native_sparse_attention/ops/triton/flash_attention_decode.py:22-217.
 *   q [B, Hq, d], k/v [B, cache_len, Hkv, d] (strided views allowed), o [B, Hq, d].
 *   strides[13] = {q_b, q_h, k_b, k_n, k_h, v_b, v_n, v_h, o_b, o_h, idx_h, idx_b, idx_k}. */
int nsa_flash_attn_decode(const void* q, const void* k, const void* v, const int* seqlens, void* o,
                          float* scratch, long long scratch_floats, int num_splits, int batch, int cache_len,
                          int num_q_heads, int num_kv_heads, int head_dim, const long long* strides,
                          float sm_scale, int dtype, void* stream);

/* nsa_flash_attn_decode for callers that are not allowed to allocate device memory (a server that gave its
 * whole memory budget to its own pool at start-up, a loop that must avoid the device synchronisation an
 * allocation can imply).  It has no counterpart in the reference.  The split-KV scratch is an 8 MiB array
 * inside the library's device image (held by every GPU that loads the library, until the process exits);
 * the caller passes inputs and the output only.  No cudaMalloc/cudaFree or allocating routine is called.
 *   num_splits: 0 = the library chooses (nsa_decode_num_splits, lowered until the scratch fits the array, so
 *       this never fails for size); > 0 = that many (at most 64, at most one per 64-key tile): the call then needs
 *       nsa_decode_scratch_floats(batch, num_kv_heads, head_dim, splits) floats and returns -3 when that exceeds
 *       nsa_flash_attn_decode_static_capacity() floats -- ask for fewer splits (1 needs none).
 *   The first call on a device may come from any host thread (the address lookup is serialised).
 *   The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device,
 *   with that device current): make that first call before any stream capture.
 *   All calls on a device share the one array and it keeps the previous call's contents; its control words start at
 *   zero and every completed call returns them to zero, every other slot is written before it is read, so the caller
 *   clears nothing, but two calls that overlap on the GPU (different streams, or host threads) race on it: serialise them. */
long long nsa_flash_attn_decode_static_capacity(void);
int nsa_flash_attn_decode_static(const void* q, const void* k, const void* v, const int* seqlens, void* o,
                                 int num_splits, int batch, int cache_len, int num_q_heads, int num_kv_heads,
                                 int head_dim, const long long* strides, float sm_scale, int dtype, void* stream);

/* Single-token attention over the selected blocks of a dense cache.
 * Replaces forward_kernel, native_sparse_attention/ops/triton/topk_sparse_attention_decode.py:22-237.
 *   topk_idx int32 [Hkv, B, topk]. */
int nsa_topk_sparse_attn_decode(const void* q, const void* k, const void* v, const int* topk_idx,
                                const int* seqlens, void* o, float* scratch, long long scratch_floats,
                                int num_splits, int batch, int cache_len, int num_q_heads, int num_kv_heads,
                                int head_dim, int topk, int block_size, const long long* strides,
                                float sm_scale, int dtype, void* stream);

/* Single-token attention over the compressed cache + block scores + top-k selection in one kernel (split-KV; the warp
 * that finishes a (sequence, KV head) pair merges the partial results, scores the blocks and selects).
 * Replaces compressed_attention_decode (about 15 ATen launches),
 * native_sparse_attention/ops/torch/compressed_attention_decode.py:21-153.
 *   topk_idx int32 [Hkv, B, min(topk, ceil(max_seqlen/block_size))] or NULL (output only).
 *   scratch: nsa_compressed_decode_scratch_floats(batch, num_kv_heads, head_dim, num_splits, cache_len) floats, always
 *   needed (-3 otherwise).  -2 when cache_len + ceil(max_seqlen/block_size) floats exceed two key tiles (about 8000 at
 *   head_dim 128: contexts beyond ~100 K tokens at stride 16). */
int nsa_compressed_attn_decode(const void* q, const void* k, const void* v, const int* seqlens,
                               const int* compress_seqlens, void* o, int* topk_idx, float* scratch,
                               long long scratch_floats, int num_splits, int batch, int cache_len, int max_seqlen,
                               int num_q_heads, int num_kv_heads, int head_dim, int kernel_size, int kernel_stride,
                               int block_size, int topk, int init_blocks, int local_blocks, const long long* strides,
                               float sm_scale, int dtype, void* stream);

/* Bytes of scratch nsa_varlen_attn_bwd needs.  No counterpart in the reference (it allocates
 * [G, total_k, Hkv, d] per-head buffers inside _compressed_attention_bwd, compressed_attention.py:664-669). */
long long nsa_varlen_attn_bwd_workspace(int total_q, int total_k, int num_q_heads, int num_kv_heads, int head_dim);

/* Backward of nsa_varlen_attn_fwd: dq, dk, dv from (q, k, v, o, do, lse).
 * Replaces _compressed_attention_bwd (backward_sum_o_do, backward_dkdv, backward_dq and the .sum(0) over heads),
 * native_sparse_attention/ops/triton/compressed_attention.py:161-535,618-780, and _flash_attention_bwd,
 * native_sparse_attention/ops/triton/flash_attention.py:168-560,660-822.
 *   strides[16] = {q_n,q_h, k_n,k_h, v_n,v_h, o_n,o_h, do_n,do_h, dq_n,dq_h, dk_n,dk_h, dv_n,dv_h}.
 *   dk/dv partial sums of CTAs sharing a key tile are combined with fp32 atomic adds (run-to-run
 *   differences at fp32 rounding level, as in the reference's atomic-based kernels). */
int nsa_varlen_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                        const float* lse, const int* cu_seqlens_q, const int* cu_seqlens_k, void* dq, void* dk,
                        void* dv, void* workspace, long long workspace_bytes, int total_q, int total_k, int batch,
                        int max_seqlen_q, int max_seqlen_k, int num_q_heads, int num_kv_heads, int head_dim,
                        int causal, int window, int stride, const long long* strides, float sm_scale, int dtype,
                        void* stream);

/* Sliding-window branch of the NSA layer: causal varlen self-attention where query t sees keys t - window_left .. t
 * (window_left + 1 keys).  The reference has no operator of its own here: its layer calls the third-party
 * flash_attn.flash_attn_varlen_func(causal=True, window_size=(window_size, -1)),
 * native_sparse_attention/module/native_sparse_attention.py:213-223; these two entry points replace that call.
 * Same tensors, strides, lse convention and workspace (nsa_varlen_attn_bwd_workspace with total_k = total_q) as
 * nsa_varlen_attn_fwd / nsa_varlen_attn_bwd with one cu_seqlens for queries and keys.  head_dim 128 only (-2 otherwise). */
int nsa_window_attn_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens, void* o, float* lse,
                        int total_len, int batch, int max_seqlen, int num_q_heads, int num_kv_heads, int head_dim,
                        int window_left, const long long* strides, float sm_scale, int dtype, void* stream);
int nsa_window_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                        const int* cu_seqlens, void* dq, void* dk, void* dv, void* workspace, long long workspace_bytes,
                        int total_len, int batch, int max_seqlen, int num_q_heads, int num_kv_heads, int head_dim,
                        int window_left, const long long* strides, float sm_scale, int dtype, void* stream);

/* Bytes of scratch nsa_topk_sparse_attn_bwd needs (fp32 dk/dv accumulators, (lse, delta) pairs, inverted index). */
long long nsa_topk_sparse_attn_bwd_workspace(int total_len, int batch, int num_q_heads, int num_kv_heads,
                                             int head_dim, int topk, int block_size);

/* Backward of nsa_topk_sparse_attn_fwd.  Builds the block -> tokens inverted index on the device
 * (histogram, scan, scatter; no host synchronisation) and runs the dQ and dK/dV passes.
 * Replaces _topk_sparse_attention_bwd: backward_sum_o_do, count_query, reorder_topk_idx (argsort + 4 host
 * syncs), backward_dkdv with its [G, N, Hkv, d] buffers and .sum(0), backward_dq,
 * native_sparse_attention/ops/triton/topk_sparse_attention.py:176-477,480-825,912-1109.
 *   cu_seqblocks int32 [batch+1]: prefix sum of ceil(seqlen / block_size).
 *   strides[19] = the 16 of nsa_varlen_attn_bwd followed by {idx_h, idx_n, idx_k}. */
int nsa_topk_sparse_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                             const float* lse, const int* topk_idx, const int* cu_seqlens,
                             const int* cu_seqblocks, void* dq, void* dk, void* dv, void* workspace,
                             long long workspace_bytes, int total_len, int batch, int num_q_heads,
                             int num_kv_heads, int head_dim, int topk, int block_size, const long long* strides,
                             float sm_scale, int dtype, void* stream);

/* Backward of nsa_linear_compress_fwd: dx [N,H,d], dw [H, kernel_size*d, d], dpe [H, kernel_size, d] (iff pe).
 * Deterministic (no floating-point atomics).  Replaces linear_compress_bwd_kernel and the autograd of the
 * bias einsum, native_sparse_attention/ops/triton/linear_compress.py:139-306,419-494,520-524.
 *   dbias_scratch fp32 [H, d] is needed iff pe != NULL; max_seqlen is the longest input sequence. */
int nsa_linear_compress_bwd(const void* x, const void* w, const void* pe, const void* dy, const int* cu_seqlens,
                            const int* y_cu_seqlens, void* dx, void* dw, void* dpe, float* dbias_scratch,
                            int total_len, int batch, int total_y, int max_seqlen, int num_heads, int head_dim,
                            int kernel_size, int kernel_stride, long long x_stride_n, long long x_stride_h,
                            int dtype, void* stream);

/* Backward of nsa_pool_compress_fwd: dx, dw [H, kernel_size] (iff w), dpe (iff pe).  Deterministic.
 * Replaces sliding_pool_dxdw_kernel + dw.sum(1) and the autograd of the bias,
 * native_sparse_attention/ops/triton/weighted_pool.py:88-179,241-298,320-324,357-362.
 *   workspace: fp32, nsa_pool_compress_bwd_workspace_floats(...) words: the column sums of dy ([H, d], needed iff pe) followed
 *   by the partial rows of dw that the one-pass kernel for long inputs (131 072 tokens or more, head_dim 128, kernel_size
 *   <= 32) leaves per (CTA, thread group); a workspace of only H * d words (or NULL without pe) is accepted and keeps long
 *   inputs on the per-thread kernels.  max_seqlen is the longest input sequence. */
long long nsa_pool_compress_bwd_workspace_floats(int total_len, int batch, int max_seqlen, int num_heads, int head_dim,
                                                 int kernel_size, int kernel_stride);
int nsa_pool_compress_bwd(const void* x, const void* w, const void* pe, const void* dy, const int* cu_seqlens,
                          const int* y_cu_seqlens, void* dx, void* dw, void* dpe, float* workspace,
                          long long workspace_floats, int total_len, int batch, int total_y, int max_seqlen,
                          int num_heads, int head_dim, int kernel_size, int kernel_stride, long long x_stride_n,
                          long long x_stride_h, int dtype, void* stream);

/* Gated sum of the three branch outputs of an NSA layer,
 *   out[n, h, :] = gate[n, h, 0] * o_cmp[n, h, :] + gate[n, h, 1] * o_sel[n, h, :] + gate[n, h, 2] * o_win[n, h, :],
 * in one pass with fp32 arithmetic and one rounding.  The reference has no operator for it: its layer evaluates the
 * expression in eager PyTorch, native_sparse_attention/module/native_sparse_attention.py:226-232 (training / prefill)
 * and native_sparse_attention/infer/nsa_inference.py:146-150 (prefill and decode; there n is the batch index).
 *   gate [total_len, num_heads, 3] (the three gates of a head contiguous), o_* and out [total_len, num_heads, head_dim];
 *   strides[10] in elements = {gate_n, gate_h, cmp_n, cmp_h, sel_n, sel_h, win_n, win_h, out_n, out_h}; the head_dim axis is
 *   contiguous, row strides of o_* and out multiples of 8, base pointers 16-byte aligned.  head_dim 64 or 128. */
int nsa_gate_combine_fwd(const void* gate, const void* o_cmp, const void* o_sel, const void* o_win, void* out, int total_len,
                         int num_heads, int head_dim, const long long* strides, int dtype, void* stream);

/* Backward of nsa_gate_combine_fwd: d_o_i = gate_i * dout, d_gate[n, h, i] = sum_d dout[n, h, d] * o_i[n, h, d] (fp32 sum in a
 * fixed order, rounded once).  Replaces the autograd graph of the same expression (three multiplies, two adds).
 *   strides[18] = {gate_n, gate_h, cmp_n, cmp_h, sel_n, sel_h, win_n, win_h, dout_n, dout_h, dgate_n, dgate_h,
 *                  dcmp_n, dcmp_h, dsel_n, dsel_h, dwin_n, dwin_h}. */
int nsa_gate_combine_bwd(const void* gate, const void* o_cmp, const void* o_sel, const void* o_win, const void* dout,
                         void* d_gate, void* d_cmp, void* d_sel, void* d_win, int total_len, int num_heads, int head_dim,
                         const long long* strides, int dtype, void* stream);

/* Rotary position embedding of a varlen batch, y = x * cos + rotate_half(x) * sin, positions taken from cu_seqlens on the
 * device.  Replaces RotaryEmbedding.forward with generate_pos_embs / generate_cos_sin (a Python loop over the batch, table
 * slices, three elementwise passes and a concatenation), native_sparse_attention/module/rope.py:36-41,126-155,158-209;
 * call sites module/native_sparse_attention.py:180-183,205 and infer/nsa_inference.py:94-103.
 *   x, y [total_rows, num_heads, head_dim] (strides in elements; y may be x); inv_freq fp32 [head_dim / 2] (from the
 *   caller's frequency initialiser); angle = inv_freq[j] * position in fp32; cos and sin are multiplied by
 *   attention_scaling and rounded to the tensor's dtype as the reference's tables are, the rotation itself runs in fp32.
 *   step == 0 (prefill / training): row n, the t-th token of its sequence, has position t * stride.
 *   step  > 0 (decode): total_rows == batch and row b has position (cu_seqlens[b+1] - cu_seqlens[b] + step - 1) * stride.
 *   inverse != 0 rotates by the opposite angle: the backward pass (dx from dy).  head_dim 64 or 128. */
int nsa_rope(const void* x, void* y, const float* inv_freq, const int* cu_seqlens, int total_rows, int batch, int num_heads,
             int head_dim, int step, int stride, float attention_scaling, int inverse, long long x_stride_n,
             long long x_stride_h, long long y_stride_n, long long y_stride_h, int dtype, void* stream);

/* ---- KV-cache maintenance of NSA inference (device-side counters, no host synchronisation) ----
 * Replace NSACache.prepare_compress / update_kv and _fill_kv_cache, native_sparse_attention/module/kv_cache.py:233-449,
 * 452-555 (a Triton copy kernel sized by .max().item(), and about twenty indexing launches per decode step).
 * Every cache is [2 (key, value)][max_batch][rows][heads][head_dim] of 16-bit elements; cache strides are
 * {kv, batch, row, head} in elements, head_dim contiguous, all strides multiples of 8, bases 16-byte aligned; counters are
 * int32 [max_batch].  A row that does not fit is dropped and bit 2 (bad index) of the device status word is raised. */

/* Prefill: copy rows of a varlen batch into a cache and set its counters (row t of the kept part goes to cache row t).
 *   mode 0: whole sequences (selected-block cache; compressed cache, with the compressed tokens and their cu_seqlens);
 *   mode 1: the last `window` rows of each sequence (sliding-window ring), kv_cache.py:381-391;
 *   mode 2: the rows after the last full compression hop, window = kernel_size, hop = kernel_stride (staging buffer of
 *           tokens the next compressed token needs), kv_cache.py:266-276.
 *   strides[8] = {cache_kv, cache_b, cache_row, cache_h, key_n, key_h, value_n, value_h}. */
int nsa_kv_cache_fill(void* cache, int* cache_len, const void* key, const void* value, const int* cu_seqlens, int mode,
                      int window, int hop, int total_rows, int batch, int cache_rows, int num_heads, int head_dim,
                      const long long* strides, void* stream);

/* Decode, before compression (_prepare_compress_decode, kv_cache.py:278-307): staging buffers that are full drop their
 * first kernel_stride rows, then every sequence appends its new key/value row [batch, heads, head_dim].
 *   strides[8] as above (key_n / value_n = stride between sequences). */
int nsa_kv_cache_stage_decode(void* stage_cache, int* stage_len, const void* key, const void* value, int batch,
                              int kernel_size, int kernel_stride, int num_heads, int head_dim, const long long* strides,
                              void* stream);

/* Decode, after compression and rotary embedding (_update_kv_decode, kv_cache.py:393-449): append the compressed token
 * of every sequence whose staging buffer is full (stage_len[b] == kernel_size), the new token to the selected-block cache,
 * and the new token to the sliding-window ring at slot count % sliding_rows; bump the three counters.
 *   strides[24] = {compress cache kv, b, row, h; sparse cache ...; sliding cache ...; then (n, h) of compress_key,
 *   compress_value, sparse_key, sparse_value, sliding_key, sliding_value}. */
int nsa_kv_cache_append_decode(void* compress_cache, int* compress_len, void* sparse_cache, int* sparse_len,
                               void* sliding_cache, int* sliding_len, const int* stage_len, const void* compress_key,
                               const void* compress_value, const void* sparse_key, const void* sparse_value,
                               const void* sliding_key, const void* sliding_value, int batch, int kernel_size,
                               int compress_rows, int sparse_rows, int sliding_rows, int num_heads, int head_dim,
                               const long long* strides, void* stream);

/* Rotary embedding of one decode row per sequence at a position read from the device: row b sits at lengths[b] * stride
 * (lengths = a cache counter BEFORE the new token is appended), so that a decode step does not depend on a host-side step
 * number and can be replayed from a CUDA graph.  Otherwise as nsa_rope. */
int nsa_rope_decode(const void* x, void* y, const float* inv_freq, const int* lengths, int batch, int num_heads, int head_dim,
                    int stride, float attention_scaling, int inverse, long long x_stride_n, long long x_stride_h,
                    long long y_stride_n, long long y_stride_h, int dtype, void* stream);

/* The three rotations of one decode step in one launch: query [batch, num_q_heads, d] and key [batch, num_kv_heads, d] at
 * position lengths_qk[b], compressed key [batch, num_kv_heads, d] at lengths_ck[b] * stride_ck (infer/nsa_inference.py:94-103
 * with step > 0).  strides[12] = {x_n, x_h, y_n, y_h} for query, key, compressed key.  Otherwise as nsa_rope_decode. */
int nsa_rope_decode3(const void* q, void* yq, const void* k, void* yk, const void* ck, void* yck, const float* inv_freq,
                     const int* lengths_qk, const int* lengths_ck, int batch, int num_q_heads, int num_kv_heads, int head_dim,
                     int stride_ck, float attention_scaling, const long long* strides, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_H_ */
