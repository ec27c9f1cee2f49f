/*
 * hsa_b200 — C ABI of the B200 (sm_100a) hierarchical sparse attention library.
 *
 * Every entry point replaces one host-side interface of the reference project's
 * `hierarchical_attention` package (paths below are inside that project).  The
 * library is stream-ordered and never synchronises; unless a function says
 * otherwise it allocates nothing: outputs and scratch are the caller's.
 *
 * Conventions
 *   - All pointers are DEVICE pointers, except where a parameter says "host".
 *   - A tensor is passed as an hsa_view: base pointer plus batch and row strides
 *     in ELEMENTS.  The innermost [H, D] block of a row is contiguous.
 *   - dtype: 0 = float32, 1 = bfloat16, 2 = float16.  Accumulation is float32.
 *   - Key/value rows are ordered [N leaves | level-1 parents | ... | root]
 *     (2N-1 rows), as in hierarchical_attention/modules/attention.py:178.
 *   - Return value: 0 = ok; < 0 = invalid argument (hsa_last_error() explains);
 *     > 0 = a cudaError_t from the launch.
 *   - `stream` is a cudaStream_t passed as void*.
 */
#ifndef HSA_B200_H
#define HSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HSA_F32 0
#define HSA_BF16 1
#define HSA_F16 2

#define HSA_ERR_ARG (-1)      /* bad shape, size or flag              */
#define HSA_ERR_ALIGN (-2)    /* pointer or stride breaks alignment   */
#define HSA_ERR_DTYPE (-3)    /* unknown dtype code                   */
#define HSA_ERR_WORKSPACE (-4)/* workspace missing or too small       */

typedef struct hsa_view {
    void *ptr;
    int64_t batch_stride; /* elements between consecutive batch entries */
    int64_t row_stride;   /* elements between consecutive node rows     */
} hsa_view;

/* Library version, major*10000 + minor*100 + patch. */
int hsa_version(void);

/* Message of the last error on the calling thread ("" if none).  Host string. */
const char *hsa_last_error(void);

/* Compute capability the kernels were compiled for (100 for sm_100a). */
int hsa_compiled_arch(void);

/*
 * Tree topology tables.  Replaces build_tree_topology
 * (hierarchical_attention/ops/topology.py:6-150).
 *   fwd_idx  [N, L] int32 : key row of the sibling subtree leaf n sees at level l
 *   fwd_mask [N, L] uint8 : 1 = excluded (future) when causal, else 0
 *   gather   [2N-1, 3] int32 : (start, end, level) leaf range feeding each node's
 *                              gradient, or (-1,-1,-1)
 * N must be a power of two, N >= 1; L = log2 N.  Any output pointer may be NULL.
 */
int hsa_topology_build(int N, int causal, int32_t *fwd_idx, uint8_t *fwd_mask,
                       int32_t *gather, void *stream);

/*
 * Initial parents: pairwise-mean pyramid.  Replaces generate_span_input_Y
 * (hierarchical_attention/ops/topology.py:153-169).
 *   x [B, N, d] -> y [B, M, d], M = hsa_span_input_y_rows(N); each level is
 *   rounded to the storage dtype as the reference's per-level torch ops do.
 * Any N >= 2 (odd tails are dropped level by level, as in the reference).
 */
int64_t hsa_span_input_y_rows(int64_t N);
int hsa_span_input_y_fwd(hsa_view x, hsa_view y, int B, int N, int d, int dtype, void *stream);
/* gx [B, N, d] = gradient of the pyramid w.r.t. x given gy [B, M, d]. */
int hsa_span_input_y_bwd(hsa_view gy, hsa_view gx, int B, int N, int d, int dtype, void *stream);

/*
 * Parent-node update, one tree level.  Replaces build_parent_nodes /
 * BuildParentNodesFunc.forward (hierarchical_attention/ops/functional.py:28-62,271)
 * and its kernel (ops/triton/build_parents.py:8-99).
 *   Qp, Kp, Vp, Out : [B, P, H, D];  Kc, Vc : [B, 2P, H, D]  (children of parent i
 *   are rows 2i, 2i+1).  W, if not NULL, receives the three softmax weights
 *   [B, P, H, 3] float32 contiguous.
 */
int hsa_parent_nodes_fwd(hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view Kc, hsa_view Vc,
                         hsa_view Out, float *W, int B, int P, int H, int D, int dtype,
                         void *stream);

/*
 * Backward of the parent-node update.  Replaces BuildParentNodesFunc.backward
 * (ops/functional.py:65-111; ops/triton/build_parents.py:106-204).  The softmax
 * weights are recomputed from Q/K in float32; every gradient row has one writer.
 */
int hsa_parent_nodes_bwd(hsa_view dOut, hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view Kc,
                         hsa_view Vc, hsa_view dQp, hsa_view dKp, hsa_view dVp, hsa_view dKc,
                         hsa_view dVc, int B, int P, int H, int D, int dtype, void *stream);

/*
 * The bottom-up refresh above level `start_level` as one launch per tree, forward and backward.  Replaces the level
 * loop of HierarchicalAttention.cross_update_Y (hierarchical_attention/modules/attention.py:128-157: per level a
 * projection of the previous level's output with Wk_y / Wv_y, dropout of the values, the parent kernel) and of its
 * autograd backward; the reference's author notes the launch problem at ops/triton/build_parents.py:207-216.
 *   Qp, Kp, Vp : [B, N-1, H*D] projections of all parents (level l = rows N - N/2^l ..), bfloat16, any row stride
 *   R          : [B, N-1, H*D] refreshed parents; rows of levels < start_level must be there, the rest is written
 *   KVc        : [B, N-1, 2*H*D] child projections [K | V] of every non-root row of R (row r of KVc = projection of
 *                row r of R); rows of levels < start_level - 1 must be there (their parents run outside), the rest is written
 *   Wkv        : [2*H*D, H*D] bfloat16 contiguous, Wk_y stacked on Wv_y
 *   dropout    : rng_state NULL = none; else the value half of KVc is masked with site / threshold / drop_scale and
 *                element ids of the [B, N-1, 2*H*D] tensor (hsa_dropout_apply / hsa_gemm_ex regenerate the same masks)
 * Backward: dRf [B, N-1, H*D] float32 holds the gradient of R on entry (from the output projection) and dRb its bfloat16
 *   copy; both are updated in place level by level; dQp, dKp, dVp rows of levels >= start_level and dKVc rows of levels
 *   >= start_level - 1 are written (value half already masked).  The weight gradient dKVc^T R is left to the caller
 *   (one product over all levels).
 * The launch is cooperative (one CTA per SM, all resident); CTAs meet at a counter in `state` (hsa_parent_tree_state_bytes
 * bytes of device memory, cleared by the call) and wait there at most the library's wait limit; a CTA that gives up writes
 * a non-zero status that makes all others leave.  hsa_parent_tree_status reads it (0 = every level completed); it
 * synchronises.  H*D a multiple of 256, D 64 or 128, 1 <= start_level < log2 N.
 */
size_t hsa_parent_tree_state_bytes(void);
int hsa_parent_tree_status(const void *state, unsigned int *status);
int hsa_parent_tree_fwd(hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view R, hsa_view KVc, const void *Wkv, int B, int N,
                        int H, int D, int start_level, const unsigned long long *rng_state, unsigned int site,
                        unsigned int threshold, float drop_scale, void *state, void *stream);
int hsa_parent_tree_bwd(hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view KVc, hsa_view dRf, hsa_view dRb, hsa_view dQp,
                        hsa_view dKp, hsa_view dVp, hsa_view dKVc, const void *Wkv, int B, int N, int H, int D,
                        int start_level, const unsigned long long *rng_state, unsigned int site,
                        unsigned int threshold, float drop_scale, void *state, void *stream);

/*
 * Span attention forward.  Replaces hierarchical_attention /
 * HierarchicalAttentionFunc.forward (ops/functional.py:114-168,274;
 * ops/triton/sparse_attn.py:8-179).
 *   Q, Out : [B, N, H, D];  K, V : [B, 2N-1, H, D].
 *   Each leaf n attends to leaves n-R..n+R (causal: n-R..n) and to one sibling
 *   node per level l (causal: only where bit l of n is set), joint softmax,
 *   scale 1/sqrt(D).  `radius` is the reference's window_size.
 *   LSE, if not NULL, receives log-sum-exp of the scaled logits [B, N, H] float32
 *   (what the backward needs; the reference stores all weights instead).
 *   The tree tables are generated in closed form inside the kernel; they equal
 *   hsa_topology_build's output bit for bit.
 *   `algo`: 0 = automatic, 1 = portable CUDA-core kernel, 2 = tensor-core kernel (bf16/f16,
 *   D in {64,128}, N >= 64 only; HSA_ERR_ARG otherwise), 3 / 4 = tensor-core kernel with
 *   64-leaf / 128-leaf tiles (4: causal, radius <= 16, N >= 128 only).  In the backward
 *   2 and 3 select the 4-warp tensor-core kernel; 0 and 4 prefer the 8-warp task-parallel
 *   kernel (causal, radius <= 16) and fall back to the 4-warp one.
 */
int hsa_span_attn_fwd(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N,
                      int H, int D, int radius, int causal, int dtype, int algo, void *stream);

/*
 * Candidate logits (weights = 0) or softmax weights (weights = 1) of span attention, one row of
 * C = 2*radius + 1 + log2(N) float32 entries per (batch, leaf, head): out [B, N, H, C] contiguous.  Entries
 * 0 .. 2*radius are the window slots (key leaf n - radius + c), the rest one slot per tree level; this is the
 * layout of the `Weights` tensor HierarchicalAttentionFunc.forward saves
 * (hierarchical_attention/ops/functional.py:131-132; kernel ops/triton/sparse_attn.py:57-145), which weights = 1
 * reproduces: softmax over the valid slots, 0 elsewhere.  weights = 0 gives the scaled logits q.k / sqrt(D) before
 * the softmax, -inf where a slot is outside the sequence or masked.  Portable kernel, any dtype.
 */
int hsa_span_attn_logits(hsa_view Q, hsa_view K, float *out, int B, int N, int H, int D, int radius,
                         int causal, int weights, int dtype, void *stream);

/*
 * The "logits" op of the reference's first Triton prototype, build_hierarchical_logits
 * (Hierarchical_Attention_Triton.py:456-514; kernels :327-393 and :414-454): for node rows of
 * Q, K [B, total_nodes, H, D]
 *   self_out  [B, seq_len, H]       float32 : scale * Q[b, t] . K[b, t]
 *   cross_out [B, total_nodes-1, H] float32 : entry r = scale * Q[b, r^1] . K[b, r]   (each node's key scored by
 *                                             its sibling's query; the root has no sibling)
 * scale = 1/sqrt(D).  Either output may be NULL.  (The prototype's self-logits kernel does not compile as
 * shipped, :389; this follows what its launcher and its commented-out body state.)
 */
int hsa_sibling_logits(hsa_view Q, hsa_view K, float *self_out, float *cross_out, int B, int total_nodes,
                       int seq_len, int H, int D, int dtype, void *stream);

/*
 * Span attention of one new leaf per sequence against a key/value cache: the step of an incremental decoder.
 * The reference's generate() re-runs the whole forward for every token
 * (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:483-504); causally, leaf n needs only
 * leaves n-radius..n and, for every set bit l of n, the left sibling of its level-l ancestor — rows that are
 * complete once leaf n-1 has been seen.
 *   q, out : [B, 1, H, D] (row stride unused);  K, V : [B, 2N-1, H, D] caches in the usual row order.
 */
int hsa_span_attn_decode(hsa_view q, hsa_view K, hsa_view V, hsa_view out, int B, int N, int H, int D,
                         int radius, int n, int dtype, void *stream);

/*
 * Diagnostic with no reference counterpart.  The TMA-staged kernels (128-leaf and 64-leaf forward, 8-warp
 * backward) wait for their bulk copies on mbarriers with a time limit (about a second).  A CTA whose wait runs
 * out counts itself, writes NaN instead of results (forward: its Out and LSE rows; backward: its dQ rows and its
 * partial rows of the upper levels, which reach dK / dV) and returns; the launch still reports success, because
 * the library never synchronises.  *count receives the number of such CTAs on the current device since the
 * library was loaded: 0 in any healthy run.  A caller that wants certainty checks it after synchronising (the
 * Python binding does so after every span-attention call when HSA_B200_DEBUG=1).  This call synchronises with
 * the device (cudaMemcpyFromSymbol).
 */
int hsa_span_attn_fwd_wait_expired(unsigned int *count);

/*
 * Test hook with no reference counterpart, for the give-up path described above: later launches of the
 * TMA-staged kernels wait at most `limit_cycles` clock cycles, and the first barrier of every CTA expects
 * `extra_tx_bytes` more bytes than its copies deliver.  With extra_tx_bytes > 0 every copy still completes but
 * that barrier never does, so each CTA gives up once the limit has passed, with nothing left in flight.
 * (2000000000, 0) restores normal operation.  Host-side state only; nothing is launched.
 */
int hsa_debug_wait_test(long long limit_cycles, unsigned int extra_tx_bytes);

/*
 * Span attention backward.  Replaces HierarchicalAttentionFunc.backward
 * (ops/functional.py:170-264; ops/triton/sparse_attn.py:185-624).
 *   Inputs Q, K, V, Out, LSE (from the forward) and dOut [B, N, H, D];
 *   outputs dQ [B, N, H, D], dK, dV [B, 2N-1, H, D] — every row written, rows
 *   nobody attends to get zeros.  Deterministic: no floating-point atomics.
 *   `workspace` must hold hsa_span_attn_bwd_workspace_bytes(...) bytes, 256-byte aligned.
 */
size_t hsa_span_attn_bwd_workspace_bytes(int B, int N, int H, int D, int radius, int causal,
                                         int dtype, int algo);
int hsa_span_attn_bwd(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE,
                      hsa_view dOut, hsa_view dQ, hsa_view dK, hsa_view dV, void *workspace,
                      size_t workspace_bytes, int B, int N, int H, int D, int radius, int causal,
                      int dtype, int algo, void *stream);

/*
 * Label-smoothed cross entropy over rows of logits whose last dimension may be padded.
 * Replaces the criterion of the reference's training loop, nn.CrossEntropyLoss(ignore_index=pad,
 * label_smoothing=0.1) applied to the [B*N, vocab] logits
 * (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:514, 562-572).
 *   logits  [M, >= V] with `row_stride` elements between rows; only columns [0, V) are classes
 *   targets [M] int64; rows with targets == ignore_index give zero loss and zero gradient; any other
 *           target outside [0, V) makes that row's loss NaN (the reference's criterion asserts on the
 *           device instead)
 *   loss_rows [M], lse [M] float32 outputs (the caller reduces loss_rows; "mean" divides by the
 *   number of rows that are not ignored)
 * Backward: dlogits [M, Vp] (same dtype) = grad_scale[0] * d loss_row / d logits; the padding
 * columns [V, Vp) are written as zeros.  grad_scale is a DEVICE float (upstream gradient divided by
 * the number of counted rows), so no host synchronisation is needed.
 */
int hsa_cross_entropy_fwd(const void *logits, int64_t row_stride, const int64_t *targets,
                          float *loss_rows, float *lse, int64_t M, int V, float smoothing,
                          int64_t ignore_index, int dtype, void *stream);
int hsa_cross_entropy_bwd(const void *logits, int64_t row_stride, const int64_t *targets,
                          const float *lse, const float *grad_scale, void *dlogits,
                          int64_t drow_stride, int64_t M, int V, int Vp, float smoothing,
                          int64_t ignore_index, int dtype, void *stream);

/*
 * LayerNorm over the last dimension of [rows, d] (contiguous), forward and backward, for the LM that
 * calls the attention layer (the reference uses nn.LayerNorm: Hierarchical_Transformer_Pretrain.py:368-372;
 * three of them per decoder layer).  gamma / beta / statistics are float32; x, y, dy, dx are `dtype`.
 * d must satisfy hsa_layer_norm_supported(d).  The backward needs `partial`: float32 scratch of
 * hsa_layer_norm_bwd_ctas(rows) * 2 * d entries; weight and bias gradients are summed in a fixed order.
 */
int hsa_layer_norm_supported(int d);
int hsa_layer_norm_bwd_ctas(int64_t rows);
int hsa_layer_norm_fwd(const void *x, const float *gamma, const float *beta, void *y, float *mean,
                       float *rstd, int64_t rows, int d, float eps, int dtype, void *stream);
int hsa_layer_norm_bwd(const void *x, const void *dy, const float *gamma, const float *mean,
                       const float *rstd, void *dx, float *dgamma, float *dbeta, float *partial,
                       int64_t rows, int d, int dtype, void *stream);

/*
 * Dense product on the tcgen05 tensor cores, for the contractions of the layer that share a dense operand: the
 * projections Wq/Wk/Wv/out_proj (hierarchical_attention/modules/attention.py:101-103,116-117,141-142,162,182-187,220
 * call nn.Linear for each), the feed-forward pair and the LM head of the model around it
 * (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:331-340,480), and their backward products.
 *
 *   C[b, m, n] (+)= sum_k A[b, m, k] * B[n, k] (+ bias[n])        bfloat16 operands, float32 accumulation
 *
 *   a_layout 0: A is stored [batches, rows, K] (hsa_view strides);  B is one matrix for all batch entries:
 *               b_layout 0: stored [N, K] (an nn.Linear weight: Y = X W^T);  b_layout 1: stored [K, N] (dX = dY W).
 *               C : [batches, rows, N].
 *   a_layout 1: A is stored [batches, K, rows] and B [batches, K, N] (b_layout must be 1): the sum runs over k AND
 *               over the batch entries, C : [rows, N] (one matrix: dW = dY^T X over all tokens).
 *   out_dtype HSA_BF16 or HSA_F32; accumulate != 0 adds to C (float32 only); bias: float32 [N] or NULL.
 *   splits > 1 cuts the K range into that many pieces (for few-tile, long-K products); their float32 partial tiles go
 *   to `workspace` (hsa_gemm_workspace_bytes, 256-byte aligned) and are summed in split order: deterministic.
 *   hsa_gemm_choose_splits suggests a count that fills the GPU.
 * N a multiple of 8 (and rows, with a_layout 1); pointers and strides 16-byte aligned.  hsa_gemm_aborts: number of thread blocks (since the
 * library was loaded, current device) that gave up a bounded wait on an mbarrier; 0 in a healthy run; synchronises.
 */
/*
 * Element-wise tail fused into the product's epilogue (hsa_gemm_ex, splits == 1, a_layout == 0), applied in this
 * order to v = acc + bias:  relu;  dropout on columns [drop_col_begin, drop_col_end) (kept entries times drop_scale);
 * gate (v = gate > 0 ? v * gate_scale : 0, gate a bfloat16 tensor shaped like the output: the backward of
 * relu + dropout given their forward output);  + residual (float32, shaped like the output);  then the store, and
 * for float32 outputs optionally a bfloat16 copy of the stored values.  These are the element-wise steps the
 * reference runs as separate kernels around its nn.Linear calls: dropout of the value projections
 * (hierarchical_attention/modules/attention.py:117,135,142,187), bias + dropout + residual of the decoder layer
 * (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:406,419,424), relu + dropout of the
 * feed-forward (:337-340).
 * Dropout masks are a pure function of (*rng_state, site, element id), element id = position in the logical
 * [batches, drop_rows_total, N] tensor (this product writes rows drop_row_offset .. of it); hsa_dropout_apply
 * regenerates them.  drop_site1 != 0 applies a second, independent mask (values dropped twice).
 * drop_threshold = p * 2^32 (its upper 16 bits are compared: p is honoured to 2^-16), drop_scale = 1/(1-p) (squared with
 * two masks).  drop_col_begin and drop_col_end are multiples of 32 (drop_col_end may also be N); the logical tensor has at
 * most 2^33 elements.  A zeroed struct is "no tail".
 */
typedef struct hsa_gemm_epilogue {
    int relu;
    const unsigned long long *rng_state;      /* device; NULL = no dropout */
    unsigned int drop_site0, drop_site1, drop_threshold;
    float drop_scale;
    int drop_col_begin, drop_col_end;
    long long drop_rows_total, drop_row_offset;
    const void *gate; long long gate_bs, gate_rs; float gate_scale;
    const float *residual; long long res_bs, res_rs;
    void *copy_bf16; long long copy_bs, copy_rs;
    /* Cross-entropy statistics of the (bfloat16) output taken as logits: see hsa_linear_ce_combine. */
    float *ce_partial;            /* [batches * rows, 2 * column tiles, 4] float32; NULL = none */
    const long long *ce_targets;  /* [batches * rows] int64 */
    int ce_classes;               /* columns >= ce_classes are padding, not classes */
    int ce_skip_store;            /* != 0: do not write the logits at all (loss only) */
} hsa_gemm_epilogue;

size_t hsa_gemm_workspace_bytes(int batches, int rows, int N, int K, int a_layout, int b_layout, int splits);
int hsa_gemm_choose_splits(int batches, int rows, int N, int K);
int hsa_gemm(hsa_view A, hsa_view B, hsa_view C, const float *bias, int batches, int rows, int N, int K,
             int a_layout, int b_layout, int out_dtype, int accumulate, int splits, void *workspace,
             size_t workspace_bytes, void *stream);
int hsa_gemm_ex(hsa_view A, hsa_view B, hsa_view C, const float *bias, int batches, int rows, int N, int K,
                int a_layout, int b_layout, int out_dtype, int accumulate, int splits, void *workspace,
                size_t workspace_bytes, const hsa_gemm_epilogue *epilogue, void *stream);
int hsa_gemm_aborts(unsigned int *count);

/*
 * LM head and loss in one pass: the reference computes logits = fc_out(x) and then nn.CrossEntropyLoss(label_smoothing)
 * over the [tokens, vocabulary] matrix (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:480,514,562-572),
 * reading the logits again.  Here the product's epilogue (hsa_gemm_ex with ce_partial set) keeps, per row and per half
 * column tile, the running (max, sum of exponentials, sum, target logit) of the logits it has in registers;
 * hsa_linear_ce_combine merges them into loss_rows[r] and lse[r] (same definitions as hsa_cross_entropy_fwd).  With
 * ce_skip_store the logits are never written (evaluation); for training they are stored once for the backward
 * (hsa_cross_entropy_bwd, which may overwrite them in place).  ce_partial holds hsa_linear_ce_partial_bytes(rows, N) bytes.
 */
size_t hsa_linear_ce_partial_bytes(long long rows, int N);
int hsa_linear_ce_combine(const float *partial, long long rows, int N, const long long *targets, float *loss_rows,
                          float *lse, int classes, float smoothing, long long ignore_index, void *stream);

/*
 * Strided row copy between host and device (cudaMemcpy2DAsync on `stream`): `rows` rows of `row_bytes` bytes,
 * consecutive rows `src_pitch` / `dst_pitch` bytes apart.  kind: 0 = host to device, 1 = device to host,
 * 2 = device to device.  No counterpart in the reference (its tensors are created on the GPU); the host-side
 * entry point uses it to ship only the key/value rows a causal query can attend to: the leaves and the
 * left-child parents, which are exactly the even rows N, N+2, ... of the [N leaves | parents] ordering
 * (hierarchical_attention/ops/topology.py:49-57 masks every right sibling).
 */
int hsa_copy_rows_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t row_bytes,
                        size_t rows, int kind, void *stream);

/* LayerNorm with float32 rows in and bfloat16 rows out (the normalised activations feed bfloat16 products), and its
 * backward: bfloat16 upstream gradient, float32 input gradient dx = add + (gradient through the norm), `add` (NULL: none;
 * may equal dx) being the gradient arriving through the residual connection around the branch
 * (Hierarchical_Transformer_Pretrain.py:386,411,421).  x_bf16 (NULL: none) also receives the input rows themselves as
 * bfloat16, for the products that read the un-normalised rows (the child projections of the leaves). */
int hsa_layer_norm_fwd_mixed(const float *x, const float *gamma, const float *beta, void *y_bf16, void *x_bf16, float *mean,
                             float *rstd, int64_t rows, int d, float eps, void *stream);
int hsa_layer_norm_bwd_mixed(const float *x, const void *dy_bf16, const float *gamma, const float *mean,
                             const float *rstd, const float *add, float *dx, float *dgamma, float *dbeta,
                             float *partial, int64_t rows, int d, void *stream);

/*
 * out[:, :, col_begin : col_begin+ncols] = keep ? in * scale : 0, as bfloat16, with the dropout masks of
 * hsa_gemm_ex (same rng_state value, sites, threshold and element ids): the backward of a dropout that ran inside a
 * product's epilogue.  `in` float32 or bfloat16 (in_dtype), `out` bfloat16; in == out (bfloat16) works in place.
 * Column c of in / out counts as column c + col_shift of the logical tensor (a gradient buffer may hold the
 * columns of several tensors side by side).
 */
int hsa_dropout_apply(hsa_view in, int in_dtype, hsa_view out, int batches, int rows, int col_begin, int ncols,
                      long long N, long long rows_total, long long row_offset, long long col_shift,
                      const unsigned long long *rng_state, unsigned int site0, unsigned int site1,
                      unsigned int threshold, float scale, void *stream);

/*
 * Column sums of a bfloat16 matrix, out[c] = sum_r x[r, c] in float32, in a fixed order: the bias gradients of the
 * projections (the reference leaves them to autograd's reduction kernels).  `partial` holds
 * hsa_column_sums_partial_bytes(rows, cols) bytes.  cols and row_stride multiples of 8.
 */
size_t hsa_column_sums_partial_bytes(long long rows, int cols);
int hsa_column_sums(const void *x, long long row_stride, long long rows, int cols, float *out, float *partial, void *stream);

/*
 * out = bfloat16(mask * in) for a float32 matrix [rows, cols] with contiguous rows, and col_sums[c] = the float32 sum
 * over rows of what was written: the gradient's way through a residual dropout
 * (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:406,419,424) and the bias gradient of the
 * projection under it, which autograd computes in three passes.  The mask is that of hsa_gemm_ex / hsa_dropout_apply
 * for a logical tensor [rows, cols] (element id r * cols + c, same rng_state value, sites, threshold); rng_state null:
 * no mask (a cast).  cols a multiple of 8; `partial`: hsa_column_sums_partial_bytes(rows, cols) bytes.
 */
int hsa_dropout_cast_colsum(const float *in, long long in_row_stride, void *out, long long out_row_stride, long long rows,
                            int cols, const unsigned long long *rng_state, unsigned int site0, unsigned int site1,
                            unsigned int threshold, float scale, float *col_sums, float *partial, void *stream);

/*
 * hsa_cross_entropy_bwd for bfloat16 logits IN PLACE (the logits are overwritten by their gradient) together with the
 * column sums of that gradient, col_sums [Vp] float32: the bias gradient of the LM head, which otherwise costs another
 * pass over the [tokens, vocabulary] matrix.  `partial`: hsa_column_sums_partial_bytes(rows, Vp) bytes.
 */
int hsa_cross_entropy_bwd_inplace(void *logits, long long row_stride, const long long *targets, const float *lse,
                                  const float *grad_scale, long long rows, int V, int Vp, float smoothing,
                                  long long ignore_index, float *col_sums, float *partial, void *stream);

/*
 * Span attention backward without any workspace argument.  No counterpart in the reference
 * project: it exists for hosts that cannot allocate device memory around the call (a plugin
 * execute hook that only receives pre-bound buffers; a server whose GPU memory is fully
 * partitioned at start-up).  Same inputs, outputs and results as hsa_span_attn_bwd with the
 * portable kernels; the scratch is a fixed array inside the library image, so
 *   - B*N*H must not exceed HSA_STATIC_SCRATCH_MAX_ELEMS (else HSA_ERR_WORKSPACE);
 *   - every GPU that loads the library holds that array (4 MiB) until the process exits;
 *   - all calls on one device share it: two calls that may run concurrently on the GPU
 *     (different streams) race on it — serialise them;
 *   - the first call on each device looks up the array's device address; make that first
 *     call outside any stream capture, with the target device current.
 * It calls no cudaMalloc/cudaFree and no allocating library routine.
 */
#define HSA_STATIC_SCRATCH_MAX_ELEMS (1 << 20)
int hsa_span_attn_bwd_static(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE,
                             hsa_view dOut, hsa_view dQ, hsa_view dK, hsa_view dV, int B, int N,
                             int H, int D, int radius, int causal, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* HSA_B200_H */
