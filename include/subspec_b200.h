/*
 * subspec_b200 — C ABI of the sm_100a speculative-decoding hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*), returns an int status (0 = ok, negative = error), never
 * throws, never allocates device memory unless its comment says so and never
 * synchronises the device.  Outputs go to caller-allocated device buffers.
 *
 * The reference project (NYCU-EDgeAi/subspec) has no FFI of its own: its seam
 * is a set of Python call signatures.  Each entry point below cites the
 * reference function(s) whose arithmetic it replaces; the Python package
 * `subspec_b200` keeps those signatures and calls into this library.
 */
#ifndef SUBSPEC_B200_H
#define SUBSPEC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SUBSPEC_API __attribute__((visibility("default")))
#else
#define SUBSPEC_API
#endif

typedef void* subspec_stream_t; /* a cudaStream_t; NULL = legacy default stream */

/* status codes */
#define SUBSPEC_OK 0
#define SUBSPEC_EINVAL (-1)       /* bad argument (null pointer, negative size, bad enum) */
#define SUBSPEC_EUNSUPPORTED (-2) /* shape outside the supported range */
#define SUBSPEC_ECUDA (-3)        /* a CUDA runtime call failed; see subspec_last_cuda_error */
#define SUBSPEC_ESCRATCH (-4)     /* scratch buffer too small / misaligned */
#define SUBSPEC_ETOOLARGE (-5)    /* batch * max_nodes exceeds SUBSPEC_STATIC_SCRATCH_MAX_ROWS */

/* element types of logits / probabilities / KV rows */
#define SUBSPEC_F32 0
#define SUBSPEC_BF16 1
#define SUBSPEC_F16 2

/* what the [rows, vocab] matrix given to the verifier holds */
#define SUBSPEC_IN_LOGITS 0 /* raw target logits: softmax is fused into the pass */
#define SUBSPEC_IN_PROBS 1  /* already-normalised probabilities */

#define SUBSPEC_VERIFY_EXACT 0 /* verify_method="exact" */
#define SUBSPEC_VERIFY_LOSSY 1 /* verify_method="lossy" */
/* Both of the above from ONE pass over the logits (a step that verifies greedily and then lossily reads the
 * same rows twice in the reference): the lossy results go to out_*, the exact ones to out2_*.  The two
 * walks must see the same flattened tree, i.e. every node decoded (n_rows == n_nodes). */
#define SUBSPEC_VERIFY_EXACT_AND_LOSSY 2

#define SUBSPEC_GATE_PROB 0    /* threshold_method="prob"    */
#define SUBSPEC_GATE_ENTROPY 1 /* threshold_method="entropy" */

/* bits of the device status word written by the kernels (0 = clean run) */
#define SUBSPEC_DEV_BAD_TOKEN 1u /* a draft token id was outside [0, vocab) */
#define SUBSPEC_DEV_BAD_CHILD 2u /* a child index was outside [0, n_nodes) */
#define SUBSPEC_DEV_BAD_ROOT 4u  /* a root index was outside [0, n_rows)   */
#define SUBSPEC_DEV_BAD_PAGE 8u  /* a page id was outside [0, num_pages)   */
#define SUBSPEC_DEV_BAD_INDEX 16u /* an accepted-path index was out of range */
#define SUBSPEC_DEV_TIMEOUT 32u  /* a bounded device-side wait ran out       */
#define SUBSPEC_DEV_HIST_OVERFLOW 64u /* sampling: one finite logit value occurs > 65535 times in a row */
#define SUBSPEC_DEV_BAD_PARENT 128u /* tree finaliser: a parent index was not in [0, own index) */
#define SUBSPEC_DEV_BAD_COUNT 256u  /* a device-side node / row count or children offset had to be clamped */

/* element forms of a tree-attention mask written by the expander and the finaliser */
#define SUBSPEC_MASK_BOOL 0     /* one byte per element, 1 = may attend (torch.bool) */
#define SUBSPEC_MASK_ADD_F32 1  /* additive, invert_mask(mask, float32): -0.0 / finfo.min */
#define SUBSPEC_MASK_ADD_BF16 2 /* additive, bfloat16 */
#define SUBSPEC_MASK_ADD_F16 3  /* additive, float16 */

SUBSPEC_API const char* subspec_version(void);
/* cudaGetErrorString of the last CUDA error an entry point saw on this thread */
SUBSPEC_API const char* subspec_last_cuda_error(void);

/* ------------------------------------------------------------------------
 * Tree verify + accept, one launch per batch of independent sequences.
 *
 * Replaces, per sequence (reference file:line):
 *   - GeneratorBase._sample_token(return_probs=True): softmax over every
 *     tree node's target logits   specdecodes/models/generators/base.py:109-139
 *   - verify_tree, exact branch: greedy / sample-and-match walk with bonus
 *     token                       specdecodes/models/utils/tree_verify.py:49-106
 *   - ClassicSDGeneratorBase._verify_step
 *                                 specdecodes/models/generators/classic_sd.py:111-116
 *   - verify_tree, lossy wrapper  specdecodes/models/utils/tree_verify.py:108-163
 *   - lossy_bottom_up_verify: per-node target token, normalised entropy,
 *     reverse-index DP, top-down walk
 *                                 specdecodes/models/utils/lossy_tree_verify.py:9-291
 *
 * Layout.  `logits` is [batch, rows, vocab] with element strides
 * `seq_stride` / `row_stride` (vocab contiguous).  Row u of sequence b is the
 * target distribution produced AT tree node u (local numbering: node 0 is the
 * first decoded node).  Per-node int32 arrays are [batch, max_nodes]; the
 * children of node u are child_idx[b][child_off[b][u] .. child_off[b][u+1])
 * in the reference's list order (child_off is [batch, max_nodes + 1]).
 * `n_nodes[b]` nodes are described; `n_rows[b] <= n_nodes[b]` of them have a
 * logits row.  For the lossy method the caller passes n_nodes == n_rows and
 * only children inside the decoded range (tree_verify.py:137-145).
 *
 * Trees.  The children lists must describe a forest: every index inside
 * [0, n_nodes), no node listed twice, no loop.  The lossy method's tables are
 * filled bottom-up whatever the numbering; the reference additionally assumes
 * that a child's index is larger than its parent's (lossy_tree_verify.py:112).
 * Indices out of range set SUBSPEC_DEV_BAD_CHILD and are skipped.  Every walk
 * on the device stops after n_nodes steps and the table fill after n_nodes
 * rounds, so lists with a loop in them end the launch with
 * SUBSPEC_DEV_BAD_CHILD instead of hanging it.  Counts outside
 * 0 <= n_rows <= n_nodes <= max_nodes and children offsets outside
 * [0, n_nodes] are clamped and reported as SUBSPEC_DEV_BAD_COUNT.  A sequence
 * with n_rows == 0 gets out_meta = {0, 0, 0, 0}.  Results of a launch that set
 * any status bit are not meaningful.
 *
 * Sampling.  do_sample = 0: the target token of a node is the first-index
 * argmax of its row.  do_sample != 0: the row is divided by `temperature`,
 * filtered by `top_k` (TopKLogitsWarper: scores below the k-th largest go) and
 * then by nucleus `top_p` with the semantics of transformers' TopPLogitsWarper
 * (top_p >= 1 disables it), renormalised, and the target token is the
 * inverse-CDF pick for uniforms[b][u] in vocabulary order (this stands in for
 * torch.multinomial's global RNG).  Supported: logits of all three dtypes with
 * either method (for the lossy method the gates then see the filtered
 * distribution, lossy_tree_verify.py:75-77); probabilities in
 * (SUBSPEC_IN_PROBS) are drawn from as they are, so a temperature other than
 * 1, top_k or top_p together with them returns SUBSPEC_EUNSUPPORTED, as does
 * residual acceptance (below) on fp32 logits or on probabilities.
 *
 * Outputs.  out_tokens / out_hidden are [batch, max_out] int64:
 * accepted draft tokens followed by the bonus token, and for each the local
 * index of the context node whose row produced it.  out_meta is [batch, 4]
 * int32: {L = entries written, accept_len, total_len, 0}.
 * The per-node arrays node_* are filled for every decoded node and are what
 * the host needs to rebuild the reference's diagnostics
 * (lossy_tree_verify.py:171-194, 249-337):
 *   node_target[u]     target token of node u
 *   node_entropy[u]    normalised entropy of row u (lossy only, else 0)
 *   node_child_prob[c] P[parent(c), token(c)] (lossy only; root entry unused)
 *   node_exact_after / node_best_len / node_best_next   the DP tables
 *   node_rowmax[u], node_rowsum[u]  softmax shift (log2 domain) and
 *                      denominator, so that P[u, t] =
 *                      exp2(logit[u, t] * log2(e) / T - rowmax[u]) / rowsum[u]
 *
 * Scratch: `scratch` must hold subspec_verify_scratch_bytes() bytes, 256-byte
 * aligned.  It needs no initialisation (unless `flags` says otherwise); calls
 * that share one scratch buffer must not overlap on the GPU.
 * ---------------------------------------------------------------------- */
typedef struct subspec_verify_args {
  uint32_t struct_size; /* sizeof(subspec_verify_args), checked */
  int32_t batch;
  int32_t max_nodes; /* stride of per-node arrays, 1..1024 */
  int32_t vocab;     /* 1..(1<<20) */
  int32_t dtype;     /* SUBSPEC_F32 / BF16 / F16 */
  int32_t input_kind;
  int64_t seq_stride; /* elements between sequences in `logits` */
  int64_t row_stride; /* elements between rows */
  const void* logits;
  const int32_t* n_nodes;   /* [batch] */
  const int32_t* n_rows;    /* [batch] */
  const int32_t* token_ids; /* [batch, max_nodes] */
  const int32_t* child_off; /* [batch, max_nodes + 1] */
  const int32_t* child_idx; /* [batch, max_nodes] */
  const int32_t* root;      /* [batch] local root index */
  /* sampling */
  int32_t do_sample;  /* 0: greedy targets; 1: every decoded row draws its target; 2 (exact method only): only the
                         contexts the walk stands on draw, as the reference's walker does -- same results,
                         a handful of rows read instead of all (node_target is -1 for rows not visited) */
  int32_t top_k;      /* 0 = off; else keep every score >= the k-th largest (TopKLogitsWarper, base.py:58-59) */
  double temperature; /* > 0 */
  double top_p;       /* >= 1 disables the nucleus filter */
  const float* uniforms; /* [batch, max_nodes], required iff do_sample */
  /* method */
  int32_t method; /* SUBSPEC_VERIFY_* */
  int32_t gate;   /* SUBSPEC_GATE_*   */
  double threshold;
  int32_t window; /* clamped at >= 0 like the reference (:55) */
  int64_t eos;    /* -1 = no EOS token */
  /* outputs */
  int32_t max_out; /* >= 2, stride of out_tokens / out_hidden */
  int64_t* out_tokens;
  int64_t* out_hidden;
  int32_t* out_meta; /* [batch, 4] */
  int32_t* node_target;
  float* node_entropy;
  float* node_child_prob;
  float* node_rowmax;
  float* node_rowsum;
  int32_t* node_exact_after;
  int32_t* node_best_len;
  int32_t* node_best_next;
  uint32_t* dev_status; /* one word, OR-ed with SUBSPEC_DEV_* bits; caller zeroes it */
  void* scratch;
  size_t scratch_bytes;
  /* results of the exact walk under SUBSPEC_VERIFY_EXACT_AND_LOSSY (same shapes as out_*); else unused */
  int64_t* out2_tokens;
  int64_t* out2_hidden;
  int32_t* out2_meta;
  /* Residual (p - q) acceptance, an extension with no counterpart in the reference (which samples a target
   * token and looks for it among the children, classic_sd.py:111-116).  acceptance = 1 with do_sample != 0 and
   * the exact method: at a context with filtered target distribution p and draft distribution
   * q = softmax(draft_logits row / draft_temperature), the children are tried in list order; child c with token
   * x is accepted iff accept_uniforms[c] < min(1, p'(x) / q(x)), where p' = p at first and, after every
   * rejection, p' <- normalise(max(p' - q, 0)); when no child is accepted the bonus token is the inverse-CDF
   * draw from p' with uniforms[context]. */
  int32_t acceptance;           /* 0: sample-and-match; 1: residual */
  const void* draft_logits;     /* [batch, rows, vocab], dtype and vocab as `logits` */
  int64_t draft_seq_stride;     /* elements */
  int64_t draft_row_stride;
  double draft_temperature;     /* > 0 */
  const float* accept_uniforms; /* [batch, max_nodes], indexed by the child node */
  uint32_t flags;               /* 0, or SUBSPEC_VERIFY_SCRATCH_CLEAN */
} subspec_verify_args;

/* The caller promises that the first 4 * batch * (max_nodes + 1) bytes of `scratch`
 * (rounded up to 256) were zero before the first call that used the buffer, and
 * that only subspec_verify_batched calls whose dev_status stayed clear have used
 * it since: every such call leaves them zero, and the entry point then puts no
 * clearing operation in front of the kernel (one launch fewer per call; it
 * matters for a single tree, whose whole verification takes ~20 us). */
#define SUBSPEC_VERIFY_SCRATCH_CLEAN 1u

SUBSPEC_API int subspec_verify_scratch_bytes(int32_t batch, int32_t max_nodes, size_t* bytes);
SUBSPEC_API int subspec_verify_batched(const subspec_verify_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * subspec_verify_batched without any allocation on the caller's side.
 * (No counterpart in the reference: it exists for hosts of this library.)
 *
 * Some programs that embed the verifier have no way to produce the scratch
 * buffer subspec_verify_batched asks for: a serving loop that handed all of
 * HBM to its KV pool and weight arena at start-up and may not call cudaMalloc
 * afterwards, or a thin foreign-language binding that owns its input and
 * output buffers but has no device allocator at hand.  For them this entry
 * point runs the same kernel with its scratch (row tickets and split
 * partials) in an array that is part of the library image: a file-scope
 * device array of about 2.7 MB that every GPU loading the library holds until
 * the process ends.  It calls no cudaMalloc / cudaFree and no allocating
 * library routine.  `args->scratch` and `args->scratch_bytes` are ignored;
 * every other field means what it means for subspec_verify_batched, and the
 * results are identical.
 *
 * Limit: batch * max_nodes <= SUBSPEC_STATIC_SCRATCH_MAX_ROWS (for example 64
 * sequences of 64-node trees, or 4 trees of 1024 nodes).  Larger launches
 * return SUBSPEC_ETOOLARGE and do nothing; split the batch or use
 * subspec_verify_batched with a caller-owned buffer.
 *
 * The first call on each device looks up the array's device address (with that
 * device current) and remembers it; make that first call outside any stream
 * capture.  All calls on a device share the one array.  It keeps whatever the
 * previous call left there; the part that must start at zero (the tickets) is
 * cleared on the stream at the start of every call.  Two calls whose kernels
 * can overlap on the same GPU (different streams, or different host threads)
 * race on it and give wrong results: serialise them, or give the concurrent
 * ones their own buffer through subspec_verify_batched.
 * ---------------------------------------------------------------------- */
#define SUBSPEC_STATIC_SCRATCH_MAX_ROWS 4096
SUBSPEC_API int subspec_verify_batched_static_scratch(const subspec_verify_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * Accepted-path KV compaction.
 *
 * For i in [0, n[b]):  row(offset[b] + i) <- row(offset[b] + beam[b][i]) for
 * every layer and for K and V, all sources read before any destination is
 * written.  Replaces
 *   - KvCachePool.reorder_cache_with_offset (clone whole pool, index_copy_,
 *     copy whole pool back)
 *       specdecodes/models/utils/flashinfer/cache_manager.py:119-213
 *   - TreeStaticCache / TreeDynamicCache.reorder_cache_with_offset
 *       specdecodes/models/utils/cache_utils.py:85-103, 166-208
 *
 * Paged layout: pool is [layers, num_pages, 2, page_len, heads, head_dim]
 * (the reference's KvCachePool.cache_data).  Logical position p of sequence b
 * lives in physical page page_table[b][p / page_len] at slot p % page_len
 * (page_table is [batch, pages_per_seq] int32).  page_table == NULL means the
 * identity table the reference assumes (physical page = p / page_len).
 * One row is heads * head_dim elements and must be a multiple of 16 bytes.
 *
 * beam is [batch, max_beam] int32, strictly increasing with beam[i] >= i
 * (the verifier's out_hidden).  offset, n and beam are device arrays, and n
 * may be strided, so that a verify launch can feed this one without a host
 * round trip: n = out_meta with n_stride = 4, beam = out_hidden with
 * max_beam = max_out.
 * ---------------------------------------------------------------------- */
typedef struct subspec_kv_paged_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t layers;
  int32_t num_pages; /* physical pages in the pool */
  int32_t page_len;
  int32_t heads;
  int32_t head_dim;
  int32_t elem_bytes; /* 2 for bf16/fp16, 4 for fp32 */
  void* pool;
  const int32_t* page_table; /* [batch, pages_per_seq] or NULL */
  int32_t pages_per_seq;
  const int32_t* offset; /* [batch] */
  const int32_t* n;      /* rows kept: n[b * n_stride] */
  const int64_t* beam;   /* [batch, max_beam] */
  int32_t max_beam;      /* row stride of beam */
  int32_t n_stride;      /* elements between consecutive entries of n (0 is read as 1) */
  uint32_t* dev_status;
} subspec_kv_paged_args;

SUBSPEC_API int subspec_kv_compact_paged(const subspec_kv_paged_args* args, subspec_stream_t stream);

/* HF layout: `layer_ptrs` is a device array of 2 * layers pointers (K then V
 * of layer 0, K then V of layer 1, ...), each a [batch, heads, tokens,
 * head_dim] tensor with the given element strides (head_dim contiguous). */
typedef struct subspec_kv_hf_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t num_tensors; /* 2 * layers */
  int32_t heads;
  int32_t tokens;
  int32_t head_dim;
  int32_t elem_bytes;
  int64_t batch_stride; /* elements */
  int64_t head_stride;
  int64_t token_stride;
  void* const* layer_ptrs;
  const int32_t* offset; /* [batch] */
  const int32_t* n;      /* rows kept: n[b * n_stride] */
  const int64_t* beam;   /* [batch, max_beam] */
  int32_t max_beam;
  int32_t n_stride;
  uint32_t* dev_status;
} subspec_kv_hf_args;

SUBSPEC_API int subspec_kv_compact_hf(const subspec_kv_hf_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * Draft-tree expansion, one depth step for a batch of sequences.
 *
 * Replaces (reference file:line):
 *   - softmax(logits / temperature) in the draft forward
 *       specdecodes/models/draft_models/classic_sd.py:10-16
 *   - DraftModelBase.topk_sampling / _topk_flatten: probs * parent_probs,
 *     flatten [leaves * vocab], torch.topk(k, sorted), idx // vocab, idx % vocab
 *       specdecodes/models/draft_models/base.py:267-305 (graph variant :307-323)
 *   - TreeData.update + Tree.add_nodes numbering when the tree_* arrays are given
 *       specdecodes/models/draft_models/base.py:31-47,
 *       specdecodes/models/utils/cpu_tree.py:69-117
 *
 * `scores` is [batch, leaves, vocab] (element strides seq_stride / row_stride):
 * draft logits (input_kind = SUBSPEC_IN_LOGITS: probabilities are
 * softmax(logits / temperature) rounded to the dtype, as the reference's
 * forward(with_softmax=True) returns them) or probabilities already
 * (SUBSPEC_IN_PROBS, what topk_sampling takes).  parent_probs is [batch, leaves]
 * in the same dtype (NULL = ones, the first step).  A candidate's score is
 * round(prob * parent_prob) in the dtype.  Outputs, [batch, k], best first, ties
 * by ascending flat index leaf * vocab + token: out_tokens / out_parents int64,
 * out_probs in the dtype (the next step's parent_probs).
 *
 * Optional tree arrays (all NULL, or all given): int32 / fp32 [batch,
 * tree_stride]; node 0 is the root, level `level` fills nodes
 * 1 + level*k .. level*k + k in rank order, with parent node index, cumulative
 * probability (the score) and depth level + 1.
 *
 * Draft-side mask (replaces TreeMaskCache.update_tree_mask and get_tree_mask,
 * specdecodes/models/draft_models/base.py:93-117, and the position ids kept by
 * the speculate loop, draft_models/classic_sd.py:71-72, 113).  With
 * `draft_mask` given, row i of sequence b is written whole:
 *   [ prefix_len[b] x may-attend | column (a - 1) set for every node a that is
 *     the new node 1 + level*k + i or one of its ancestors below the root
 *     | masked up to draft_mask_cols ]
 * which is what the reference's buffer holds after its update for this level:
 * the parent's row followed by a one-hot for the node itself.  The root is the
 * last of the prefix tokens.  prefix_len[b] + (level + 1) * k > draft_mask_cols
 * sets SUBSPEC_DEV_BAD_INDEX and leaves that sequence's rows unwritten.
 * ---------------------------------------------------------------------- */
typedef struct subspec_expand_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t leaves; /* rows per sequence: 1 on the first step, k afterwards */
  int32_t vocab;
  int32_t k; /* 1..32 */
  int32_t dtype;
  int32_t input_kind;
  int64_t seq_stride;
  int64_t row_stride;
  const void* scores;
  const void* parent_probs;
  double temperature; /* used with SUBSPEC_IN_LOGITS */
  int64_t* out_tokens;
  void* out_probs;
  int64_t* out_parents;
  int32_t level;
  int32_t tree_stride;
  int32_t* tree_tokens;
  int32_t* tree_parents;
  float* tree_probs;
  int32_t* tree_depths;
  void* scratch; /* subspec_expand_scratch_bytes(), 256-byte aligned, no initialisation needed (but see flags) */
  size_t scratch_bytes;
  uint32_t* dev_status;
  /* Optional (needs the tree arrays): the draft-side tree mask of the new level and its position ids. */
  void* draft_mask;              /* [batch, k, cols] in the element form draft_mask_kind, or NULL */
  int32_t draft_mask_kind;       /* SUBSPEC_MASK_* */
  int64_t draft_mask_cols;       /* columns written per row, >= prefix_len[b] + (level + 1) * k */
  int64_t draft_mask_row_stride; /* elements; 0 = draft_mask_cols */
  int64_t draft_mask_seq_stride; /* elements; 0 = k * row stride */
  const int32_t* prefix_len;     /* [batch] tokens in front of the tree's first level, or NULL (= 0) */
  int64_t* draft_position_ids;   /* [batch, k] = prefix_len[b] + level, or NULL */
  uint32_t flags;                /* 0, or SUBSPEC_EXPAND_SCRATCH_CLEAN */
  uint32_t reserved;
} subspec_expand_args;

/* The caller promises that the first 4 * batch bytes of `scratch` (rounded up to 256) were zero before the
 * first call that used the buffer, and that only subspec_expand_step calls with this `batch` whose dev_status
 * stayed clear have used it since: every such call leaves them zero, and the entry point then puts no clearing
 * operation in front of the kernel (one launch fewer per level of the draft tree). */
#define SUBSPEC_EXPAND_SCRATCH_CLEAN 1u

SUBSPEC_API int subspec_expand_scratch_bytes(int32_t batch, int32_t leaves, int32_t k, size_t* bytes);
SUBSPEC_API int subspec_expand_step(const subspec_expand_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * Tree finaliser: prune to the `keep` nodes of largest cumulative probability,
 * renumber by rank, and emit everything the tree-decoding forward and the
 * verifier need.
 *
 * Replaces (reference file:line):
 *   - Tree.prune_to_top_n         specdecodes/models/utils/cpu_tree.py:175-215
 *   - Tree.get_tree_data          cpu_tree.py:238-251
 *   - Tree.create_attention_mask  cpu_tree.py:263-286 (ancestor-or-self matrix,
 *                                 prefix_length all-true columns in front, rows
 *                                 from skip_nodes)
 *   - position ids = depths + position_offset, the splice of the mask into the
 *     preallocated [1, 1, max_verify, max_cache_len] buffer and its inversion
 *                                 specdecodes/models/generators/classic_sd.py:33-55, 73-77
 *                                 specdecodes/models/utils/utils.py:4-6
 *
 * Input: the tree arrays subspec_expand_step fills, n_nodes nodes per
 * sequence (node 0 = root, probability 1; every parent index is smaller than
 * the node's own, else SUBSPEC_DEV_BAD_PARENT and the node is treated as a
 * root).  When n_nodes <= keep nothing is pruned and the nodes keep their
 * numbering, as the reference returns early (cpu_tree.py:176-177); otherwise
 * ranking is (probability desc, index asc; the reference leaves ties to
 * torch.topk) and node r of the output is the node of rank r.
 *
 * Outputs are [batch, keep]: keep_idx (old index of new node r), tokens,
 * parents (new numbering, -1 for the root), depths, probs, position_ids
 * (int64); child_off [batch, keep + 1] / child_idx [batch, keep] are the
 * children lists in the layout subspec_verify_batched takes; n_out[b] = nodes
 * kept.  Entries r >= n_out[b] are padding (keep_idx -1).
 *
 * Mask.  Row r - skip_nodes of sequence b (r = skip_nodes .. keep - 1) is
 *   [ prefix_length[b] x may-attend | keep tree columns: column j set iff node
 *     j is r or an ancestor of r | masked up to mask_cols ]
 * in the element form `mask_kind` (SUBSPEC_MASK_*).  mask_cols = 0 means
 * `keep` columns and is valid only without a prefix (prefix_length == NULL);
 * mask_row_stride / mask_seq_stride are in elements, 0 = dense.  With
 * mask_cols = max_cache_len and the strides of the caller's static buffer the
 * kernel writes the rows the reference's _get_tree_mask + invert_mask produce.
 * A padding row attends to itself only.  prefix_length[b] + keep > mask_cols
 * sets SUBSPEC_DEV_BAD_INDEX and leaves that sequence's mask unwritten.
 * ---------------------------------------------------------------------- */
typedef struct subspec_tree_finalize_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t n_nodes; /* <= 4096 */
  int32_t tree_stride;
  int32_t keep; /* <= 1024 */
  const int32_t* tree_tokens;
  const int32_t* tree_parents;
  const float* tree_probs;
  const int32_t* tree_depths;
  const int32_t* position_offset; /* [batch] or NULL (= 0) */
  int32_t* keep_idx;
  int32_t* tokens;
  int32_t* parents;
  int32_t* depths;
  float* probs;
  int64_t* position_ids;
  void* mask;
  int32_t* child_off;
  int32_t* child_idx;
  int32_t* n_out;
  uint32_t* dev_status;          /* one word, OR-ed with SUBSPEC_DEV_* bits; may be NULL */
  const int32_t* prefix_length;  /* [batch] or NULL (= 0) */
  int32_t skip_nodes;            /* 0 .. keep: mask rows start at this node */
  int32_t mask_kind;             /* SUBSPEC_MASK_* */
  int64_t mask_cols;             /* columns written per row; 0 = keep (no prefix) */
  int64_t mask_row_stride;       /* elements; 0 = mask_cols */
  int64_t mask_seq_stride;       /* elements; 0 = (keep - skip_nodes) * row stride */
} subspec_tree_finalize_args;

SUBSPEC_API int subspec_tree_finalize(const subspec_tree_finalize_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * Between one verification and the next (the SubSpec-v2 loop), per sequence:
 *
 *   - re-rooting: next_root = the child of the last context node that carries
 *     the bonus token, in the tree's own numbering, or -1
 *       Tree.find_child_index        specdecodes/models/utils/cpu_tree.py:232-236
 *       its call site                specdecodes/models/generators/subspec_sd_v2.py:231-236
 *   - delayed reorder: the step's hidden indices are appended to beam_cache
 *     (hidden_indices_cache, subspec_sd_v2.py:223-229); when the bonus token
 *     missed every child, or finished[b] is set, the KV rows gathered since the
 *     last reorder are to be kept now: reorder_n[b] = their number,
 *     reorder_offset[b] = kv_len[b] before, kv_len[b] += reorder_n[b], and the
 *     cache restarts empty; otherwise reorder_n[b] = 0 (subspec_sd_v2.py:250-262).
 *     subspec_kv_compact_* then takes n = reorder_n, beam = beam_cache,
 *     offset = reorder_offset, without a host round trip.
 *
 * The tree arrays are the ones the verification ran on (local numbering,
 * node 0 = first decoded node); out_* are its outputs.  skip_nodes[b] is added
 * to every index that leaves this call (NULL = 0).
 * ---------------------------------------------------------------------- */
typedef struct subspec_post_verify_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t max_nodes; /* stride of the per-node arrays, as in subspec_verify_args */
  int32_t max_out;   /* stride of out_tokens / out_hidden */
  const int32_t* n_nodes;
  const int32_t* token_ids;
  const int32_t* child_off;
  const int32_t* child_idx;
  const int64_t* out_tokens;
  const int64_t* out_hidden;
  const int32_t* out_meta;
  const int32_t* skip_nodes; /* [batch] or NULL */
  const uint8_t* finished;   /* [batch] or NULL */
  int32_t* next_root;        /* [batch] out */
  int32_t* accepted;         /* [batch] out, or NULL: next_root >= 0 */
  int64_t* beam_cache;       /* [batch, beam_stride] in/out */
  int32_t beam_stride;
  int32_t* beam_len;       /* [batch] in/out: entries of beam_cache in use */
  int32_t* reorder_n;      /* [batch] out */
  int32_t* reorder_offset; /* [batch] out, or NULL */
  int32_t* kv_len;         /* [batch] in/out, or NULL */
  uint32_t* dev_status;
} subspec_post_verify_args;

SUBSPEC_API int subspec_post_verify(const subspec_post_verify_args* args, subspec_stream_t stream);

/* Tree.prune_to_depth (cpu_tree.py:119-173; _post_verify, subspec_sd_v2.py:44-45): keep the nodes with
 * depth <= max_depth[b] in their original order, in place on the tree arrays [batch, tree_stride]
 * (n_nodes[b] in use; parents re-linked, -1 for a root); keep_idx[r] = old index of new node r,
 * n_out[b] = nodes kept.  child_off [batch, tree_stride + 1] / child_idx [batch, tree_stride], when given
 * (both or neither), are the children lists in subspec_verify_batched's layout and are filtered in place, a
 * node's kept children in the order its list had them.  tree_stride <= 4096. */
typedef struct subspec_tree_prune_depth_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t tree_stride;
  const int32_t* n_nodes;   /* [batch] */
  const int32_t* max_depth; /* [batch] */
  int32_t* tokens;
  int32_t* parents;
  int32_t* depths;
  float* probs; /* or NULL */
  int32_t* keep_idx;
  int32_t* n_out;
  int32_t* child_off; /* or NULL */
  int32_t* child_idx; /* or NULL */
  uint32_t* dev_status;
} subspec_tree_prune_depth_args;

SUBSPEC_API int subspec_tree_prune_depth(const subspec_tree_prune_depth_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * Page bookkeeping of the paged KV cache, for a batch of requests, on the
 * device: one call per step of a generation loop, no host round trip.
 *
 * Replaces (specdecodes/models/utils/flashinfer/cache_manager.py):
 *   - KvCachePool.allocate / deallocate and the free-page mask      :66-80
 *   - RequestKvCache.increment / decrement / crop and the bookkeeping
 *     at the end of reorder_cache_with_offset                       :237-346
 *   - getKvCacheBatchPosition                                       :350-414
 *
 * State (device arrays the caller owns): free_mask, one bit per physical
 * page, set = free; page_table [batch, pages_per_seq], the first n_pages[b]
 * entries of a row being request b's pages in order; kv_len, kv_last_page_len.
 * The call sets kv_len[b] = (set_len ? set_len[b] : kv_len[b]) + add_len[b] +
 * add_all, returns the pages a request no longer needs (cut from the end of
 * its list), gives requests that need more the lowest free pages (requests in
 * batch order), and refreshes kv_last_page_len.  Asking for more pages than
 * are free, or than a row of page_table holds, sets SUBSPEC_DEV_BAD_PAGE.
 *
 * Optional outputs (kv_page_indptr == NULL skips them all): the flattened
 * page table the attention plan takes -- kv_page_indptr [batch + 1],
 * kv_page_indices [sum of n_pages], seq_indptr [batch + 1] (tokens appended per
 * request: kv_len in PREFILL mode, 1 in DECODE, tree_tokens in TREE) -- and, for
 * the append of those tokens, batch_indices / positions [max_append] (token t
 * of request b sits at kv_len[b] - appended + t).
 * ---------------------------------------------------------------------- */
#define SUBSPEC_PAGES_PREFILL 0
#define SUBSPEC_PAGES_DECODE 1
#define SUBSPEC_PAGES_TREE 2
typedef struct subspec_pages_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t num_pages;
  int32_t page_len;
  int32_t pages_per_seq;
  uint32_t* free_mask;       /* [(num_pages + 31) / 32] */
  int32_t* page_table;       /* [batch, pages_per_seq] */
  int32_t* n_pages;          /* [batch] */
  int32_t* kv_len;           /* [batch] */
  int32_t* kv_last_page_len; /* [batch] */
  const int32_t* set_len;    /* [batch] or NULL */
  const int32_t* add_len;    /* [batch] or NULL */
  int32_t add_all;
  int32_t mode;        /* SUBSPEC_PAGES_* */
  int32_t tree_tokens; /* TREE mode */
  int32_t max_append;  /* entries of batch_indices / positions */
  int32_t* seq_indptr;
  int32_t* kv_page_indptr;
  int32_t* kv_page_indices;
  int32_t* batch_indices;
  int32_t* positions;
  uint32_t* dev_status;
} subspec_pages_args;

SUBSPEC_API int subspec_pages_update(const subspec_pages_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * Tree attention over the paged KV cache (one layer), and the append of the
 * tree's own K / V rows that precedes it.
 *
 * Replaces the FlashInfer calls of the reference's paged generators:
 *   - append_paged_kv_cache
 *       specdecodes/models/utils/flashinfer/attention_wrapper.py:234-253
 *   - BatchPrefillWithPagedKVCacheWrapper.plan(custom_mask=...) / run
 *       attention_wrapper.py:104-151, 288-316;
 *       specdecodes/models/utils/flashinfer/attention.py:26-102
 *
 * The pool is KvCachePool.cache_data, [layers, num_pages, 2, page_len,
 * num_kv_heads, head_dim] bf16 or fp16 (FlashInferCache allocates fp16,
 * cache_manager.py:462); request b's rows live in the pages
 * page_table[b][0 .. ], kv_len[b] of them INCLUDING the n_q[b] rows of the tree
 * (append first).  Query token i of request b is cache row kv_len[b] - n_q[b] + i.
 * It sees every row below prefix_len[b] (NULL: kv_len[b] - n_q[b]) and, of the
 * rows from there on, those whose byte in mask[b][i][row] is non-zero: the
 * [rows, prefix + tree columns] matrix subspec_tree_finalize writes (and
 * FlashInfer's custom_mask, or its additive form: mask_kind).  q / out are
 * [batch, q_len, num_q_heads, head_dim] in the pool's type with element strides (any
 * order of the axes in memory, e.g. the [batch, heads, tokens, dim] of an SDPA call); query head h reads KV head h / (num_q_heads /
 * num_kv_heads).  Softmax in fp32, scores scaled by sm_scale; outputs within
 * the rounding of the 16-bit type of an fp32 evaluation.  head_dim 64 or 128.
 * ---------------------------------------------------------------------- */
typedef struct subspec_tree_attn_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t q_len; /* tree tokens per request the buffers are laid out for */
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;
  int32_t layer;
  int32_t layers;
  int32_t num_pages;
  int32_t page_len;
  int32_t pages_per_seq;
  const void* pool;
  const int32_t* page_table; /* [batch, pages_per_seq] */
  const int32_t* kv_len;     /* [batch] */
  const int32_t* n_q;        /* [batch] or NULL (= q_len) */
  const int32_t* prefix_len; /* [batch] or NULL */
  const uint8_t* mask;       /* [batch, q_len, >= kv_len] elements of mask_kind (bytes by default) */
  int64_t mask_batch_stride;
  int64_t mask_row_stride;
  const void* q;
  int64_t q_batch_stride, q_token_stride, q_head_stride; /* elements */
  void* out;
  int64_t o_batch_stride, o_token_stride, o_head_stride;
  double sm_scale;
  uint32_t* dev_status;
  int32_t dtype; /* SUBSPEC_BF16 or SUBSPEC_F16: pool, q and out alike (0 is read as SUBSPEC_BF16) */
  int32_t mask_kind; /* SUBSPEC_MASK_BOOL (bytes, non-zero = visible) or SUBSPEC_MASK_ADD_F32 / _BF16 / _F16
                        (the additive form invert_mask makes: +-0 = visible, anything else hidden); the mask
                        strides count elements of that kind */
  /* Hugging Face static caches (TreeStaticCache: key / value tensors [batch, kv_heads, max_cache_len, head_dim]
   * of one layer) instead of the paged pool: v_cache != NULL, `pool` is the key tensor, page_len the rows a
   * batch entry has room for, num_pages = batch, pages_per_seq = 1, page_table may be NULL (request b is
   * entry b), layer = 0 and layers = 1.  Strides in elements; heads' rows must be head_dim apart or more. */
  const void* v_cache;
  int64_t kv_batch_stride, kv_head_stride, kv_row_stride;
  /* kv_splits > 1: that many CTAs share the cache rows of every (request, KV head, 256 query rows) and a second
   * kernel combines their partial results -- for a few requests with long caches, which would otherwise occupy
   * batch * num_kv_heads CTAs.  split_scratch: batch * num_q_heads * q_len * kv_splits * 130 floats, 16-byte
   * aligned (head_dim + 2 floats per row and range would do), owned by the call until the stream has
   * passed it. */
  int32_t kv_splits;
  int32_t reserved;
  void* split_scratch;
} subspec_tree_attn_args;

SUBSPEC_API int subspec_tree_attention_paged(const subspec_tree_attn_args* args, subspec_stream_t stream);

/* k / v are [batch, q_len, num_kv_heads, head_dim] (16-bit elements; element strides batch_stride /
 * token_stride, heads and dims contiguous); token i < n_q[b] goes to cache row kv_len[b] - n_q[b] + i. */
typedef struct subspec_kv_append_args {
  uint32_t struct_size;
  int32_t batch;
  int32_t q_len;
  int32_t num_kv_heads;
  int32_t head_dim;
  int32_t layer;
  int32_t layers;
  int32_t num_pages;
  int32_t page_len;
  int32_t pages_per_seq;
  void* pool;
  const int32_t* page_table;
  const int32_t* kv_len;
  const int32_t* n_q; /* or NULL */
  const void* k;
  const void* v;
  int64_t batch_stride, token_stride;
  uint32_t* dev_status;
} subspec_kv_append_args;

SUBSPEC_API int subspec_kv_append_paged(const subspec_kv_append_args* args, subspec_stream_t stream);

/* ------------------------------------------------------------------------
 * W4A16 group-wise dequant GEMM (the HQQ 4-bit draft linear).
 *
 *   y[m, n] = sum_k x[m, k] * (q[n, k] - zero[n, k / 64]) * scale[n, k / 64]
 *
 * Replaces the forward of the modules that HqqQuantizer.quantize_model installs
 * (specdecodes/helpers/quantizers/hqq/__init__.py:17-119: hqq's
 * HQQLinear(nbits=4, group_size=64, axis=1) patched by
 * prepare_for_inference(backend="gemlite"); recipe
 * specdecodes/helpers/recipes/subspec/hqq_4bit_postspec.py:21-34).  hqq and
 * gemlite are third-party and not part of the reference tree; the arithmetic
 * above is what their 4-bit, group-64, axis-1 format defines.
 *
 * subspec_w4a16_pack converts the interchange format -- qweight int32
 * [n, k / 8], nibble i of word j holding q[n, 8 j + i]; scale and zero fp16
 * [n, k / 64] -- into the tiled layout the kernel streams (once, at
 * quantisation time).  subspec_w4a16_gemm takes bf16 activations x [m, k]
 * (row stride x_stride elements) and writes bf16 y [m, n].  Arithmetic: weights
 * are dequantised to fp16, activations converted to fp16 (clamped to the fp16
 * range), products accumulated in fp32 on the tensor cores.
 * Limits: 1 <= m <= 256, n % 128 == 0, k % 64 == 0.
 * ---------------------------------------------------------------------- */
typedef struct subspec_w4a16_args {
  uint32_t struct_size;
  int32_t m, n, k;
  const void* x; /* bf16 [m, k] */
  int64_t x_stride;
  const void* packed; /* subspec_w4a16_pack output, 16-byte aligned */
  void* y;            /* bf16 [m, n] */
  int64_t y_stride;
  void* scratch; /* subspec_w4a16_scratch_bytes(m, n, k), 256-byte aligned, no initialisation needed */
  size_t scratch_bytes;
  uint32_t* dev_status;
} subspec_w4a16_args;

SUBSPEC_API int subspec_w4a16_packed_bytes(int32_t n, int32_t k, size_t* bytes);
SUBSPEC_API int subspec_w4a16_pack(const void* qweight, const void* scale, const void* zero, void* packed,
                                   int32_t n, int32_t k, subspec_stream_t stream);
SUBSPEC_API int subspec_w4a16_scratch_bytes(int32_t m, int32_t n, int32_t k, size_t* bytes);
SUBSPEC_API int subspec_w4a16_gemm(const subspec_w4a16_args* args, subspec_stream_t stream);

/* Several projections of the same activations in ONE launch: y[i] = x @ W[i]^T for count weight matrices
 * [n[i], k] packed separately.  The draft's decoder layer calls q/k/v, and gate/up, back to back on one input
 * (the recipe quantises them alike: specdecodes/helpers/recipes/subspec/hqq_4bit_postspec.py:28-34); apart
 * they are launches of 1 to 7 MB of weights each, all fixed cost.  The result of every projection is
 * bit-identical to its own subspec_w4a16_gemm call whenever the two plans split K alike, and within the GEMM's
 * stated tolerance always.  Scratch: subspec_w4a16_scratch_bytes(m, n[0] + ... + n[count-1], k). */
#define SUBSPEC_W4A16_MAX_GROUP 4
typedef struct subspec_w4a16_group_args {
  uint32_t struct_size;
  int32_t m, k;
  int32_t count; /* 1 .. SUBSPEC_W4A16_MAX_GROUP */
  const void* x; /* bf16 [m, k] */
  int64_t x_stride;
  const void* packed[SUBSPEC_W4A16_MAX_GROUP];
  int32_t n[SUBSPEC_W4A16_MAX_GROUP];
  void* y[SUBSPEC_W4A16_MAX_GROUP]; /* bf16 [m, n[i]] */
  int64_t y_stride[SUBSPEC_W4A16_MAX_GROUP];
  void* scratch;
  size_t scratch_bytes;
  uint32_t* dev_status;
} subspec_w4a16_group_args;

SUBSPEC_API int subspec_w4a16_gemm_grouped(const subspec_w4a16_group_args* args, subspec_stream_t stream);

/* -------------------------------------------------------------------------
 * lm_head + tree verification in one call, without the logits in between
 *
 * Replaces, for greedy targets, the tail of the reference's target forward
 * and the verifier behind it: `logits = lm_head(hidden_states)` for the tree
 * rows (generators/classic_sd.py:100-109) followed by verify_tree / the lossy
 * bottom-up verify (verify/exact_tree_verify.py:11-68,
 * verify/lossy_tree_verify.py:27-226).  The GEMM runs on the tensor cores
 * and its epilogue folds every accumulator tile, rounded to the model's
 * 16-bit dtype as the reference's lm_head output is, into per-row statistics (maximum, first
 * arg-max, sum 2^y, sum y 2^y); a second small kernel combines them per row,
 * computes the probabilities of the children's tokens from dot products of the
 * row's hidden state with those tokens' weight rows, and runs the same walk
 * as subspec_verify_batched.  The [rows, vocab] logits are never written.
 *
 * `verify` is a subspec_verify_args as for subspec_verify_batched with:
 * logits / seq_stride / row_stride / input_kind ignored, dtype = SUBSPEC_BF16
 * or SUBSPEC_F16 (the dtype of `hidden`, `weight` and of the logits the call
 * stands for), do_sample = 0, acceptance = 0; every method and gate is accepted.  Its
 * scratch must hold subspec_lm_head_verify_scratch_bytes bytes.  Row u of
 * sequence b is row b * hidden_seq_rows + u of `hidden`.
 *
 * Results against a library GEMM + subspec_verify_batched: the accumulation
 * order of a GEMM is its own, so a logit that sits within fp32 rounding of a
 * 16-bit rounding boundary may come out one step of that dtype apart; targets can
 * differ where the two largest logits of a row are that close, and a child's
 * probability by the factor e^(one such step of its logit).
 * Limits: hidden_dim % 8 == 0, strides % 8 == 0, addresses 16-byte aligned
 * (SUBSPEC_EINVAL otherwise); vocab <= 2^20.
 * ---------------------------------------------------------------------- */
typedef struct subspec_lm_head_verify_args {
  uint32_t struct_size;
  int32_t hidden_dim;        /* K */
  const void* hidden;        /* bf16 / fp16 [batch * hidden_seq_rows, hidden_dim] */
  int64_t hidden_row_stride; /* elements; 0 = hidden_dim */
  const void* weight;        /* same dtype, [vocab, hidden_dim]: the lm_head's weight as nn.Linear holds it */
  int64_t weight_row_stride; /* elements; 0 = hidden_dim */
  int32_t hidden_seq_rows;   /* rows of `hidden` per sequence, >= every n_rows[b] */
  int32_t reserved;
  subspec_verify_args verify;
} subspec_lm_head_verify_args;

SUBSPEC_API int subspec_lm_head_verify_scratch_bytes(int32_t batch, int32_t max_nodes, int32_t hidden_seq_rows,
                                                     int32_t vocab, size_t* bytes);
SUBSPEC_API int subspec_lm_head_verify(const subspec_lm_head_verify_args* args, subspec_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SUBSPEC_B200_H */
