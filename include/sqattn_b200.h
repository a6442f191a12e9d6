/*
 * sqattn_b200 -- C ABI of the B200 (sm_100a) SQAttn attention path.
 *
 * Every entry point takes plain pointers and sizes, enqueues its work on the
 * given CUDA stream and returns a status code; nothing here allocates device
 * memory, synchronises the device or aborts.  All tensor pointers are device
 * pointers unless a comment says "host".  Strides are in ELEMENTS and the
 * last (head_dim) dimension must be contiguous.  Paths in the comments are
 * files of the reference project (yifu-ding/LongContext_SQAttn_paddle) whose
 * interface the entry point replaces.
 */
#ifndef SQATTN_B200_H_
#define SQATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* sqattn_stream_t; /* a cudaStream_t */

/* status codes (0 = ok); sqattn_last_error_string() describes the last failure on this thread */
enum {
  SQATTN_OK = 0,
  SQATTN_ERR_INVALID_ARG = 1, /* null pointer, bad shape/stride/alignment, bad enum (reference: ValueError / assert) */
  SQATTN_ERR_UNSUPPORTED = 2, /* head_dim not 64/128, too many heads, ... */
  SQATTN_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed */
  SQATTN_ERR_WORKSPACE = 4,   /* workspace missing or too small */
  SQATTN_ERR_DEVICE_TIMEOUT = 5 /* reported by sqattn_check_device_status: a bounded device-side wait gave up */
};

enum { SQATTN_F16 = 0, SQATTN_BF16 = 1 };

/* logical [batch, heads, seq, head_dim] view of any layout (HND or NHD) */
typedef struct {
  const void* ptr;
  int64_t stride_b, stride_h, stride_n;
} sqattn_tensor;

typedef struct {
  void* ptr;
  int64_t stride_b, stride_h, stride_n;
} sqattn_tensor_out;

/* ---- prefill ------------------------------------------------------------------------------ */

enum {
  SQATTN_MODE_DENSE_CAUSAL = 0,    /* attn_causal, sqattn/attn_triton.py:216-315 (BLOCK_M=128) */
  SQATTN_MODE_RELATIVE_WINDOW = 1, /* attn_hierarchical_relative_window, sqattn/attn_triton_mix_relative.py:309-483 (BLOCK_M=64) */
  SQATTN_MODE_ABSOLUTE_WINDOW = 2  /* attn_hierarchical_window, sqattn/attn_triton_mix_bad.py:285-426 (BLOCK_M=128) */
};

enum {
  SQATTN_P_FP8_OFF = 0,
  SQATTN_P_FP8_ALL = 1,   /* is_P_fp8_quant=True of the reference kernels (attn_triton.py:81-83) */
  SQATTN_P_FP8_STAGE2 = 2 /* FP8 rounding of P only on int4-window tiles; 16-bit P elsewhere */
};

typedef struct {
  /* q_*: [B, Hq, qo_len, D]; k_*, v: [B, Hkv, kv_len, D]; o: [B, Hq, qo_len, D].
   * q_int4/k_int4 may alias q_int8/k_int8 (what the relative launcher ships, mix_relative.py:440-446).
   * Dense mode reads only q_int8/k_int8/v. */
  sqattn_tensor q_int8, k_int8, q_int4, k_int4, v;
  sqattn_tensor_out o;
  float* lse; /* optional [B, Hq, qo_len] fp32, base-2: log2(l)+m (attn_triton.py:210-213) */
  int32_t batch, num_q_heads, num_kv_heads, qo_len, kv_len, head_dim; /* head_dim 64 or 128 */
  int32_t qk_dtype, v_dtype, o_dtype; /* SQATTN_F16 / SQATTN_BF16 */
  int32_t mode;
  int32_t sink_size;            /* windows modes; relative mode needs a multiple of 64 */
  const float* win8_ratios;     /* host, [Hq]: relative mode (fractions of kv_len) */
  const float* win4_ratios;     /* host, [Hq] */
  const int32_t* win8_sizes;    /* host, [Hq]: absolute mode (tokens) */
  const int32_t* win4_sizes;    /* host, [Hq] */
  int32_t p_fp8_mode;
  int32_t q_is_scaled; /* 0: q is multiplied by 1/sqrt(D)*1.44269504 in its dtype first (what the reference
                          launchers do, mix_relative.py:383-385) into the workspace; 1: caller already did */
  void* workspace;     /* device scratch, sqattn_prefill_workspace_bytes() bytes, 1024-byte aligned */
  size_t workspace_bytes;
  int32_t q_row_offset; /* sequence-parallel shards: q/o hold rows [q_row_offset, q_row_offset + qo_len) of a
                           kv_len-token sequence (multiple of 128); 0 for a whole sequence */
  int32_t q_split_rows; /* 0: one row range.  Otherwise q/o rows [q_split_rows, qo_len) are sequence rows starting at
                           q_row_offset2 (both multiples of 128): a rank that owns two separate row ranges, e.g. chunks
                           r and 2G-1-r of the zig-zag split that balances causal work, runs them in one launch */
  int32_t q_row_offset2;
  int32_t q_fake_quant; /* 0: q_int8 / q_int4 are prepared operands.  t + 1 (t = SQATTN_QTYPE_*): q_int8 is the query as
                           the model produced it and the kernel applies the adapter's per-token fake-quant of type t
                           (sqattn/attn_replacer.py:340-361, fake_quant.py) and the softmax scale to every 128-row tile
                           in shared memory before its first product, bit for bit what sqattn_prep_qkv writes, so the
                           prepared copy of q (940 MB at 131072 tokens x 28 heads) never exists in memory.  Needs one
                           operand set (q_int4 == q_int8 and k_int4 == k_int8: the relative launch as shipped);
                           q_is_scaled is ignored.  It trades memory for time: the tile is quantised by the CTA's four
                           softmax warps, which are the kernel's bottleneck, and measured 7 % (131072 tokens) to 25 %
                           (32768 tokens) slower than the stand-alone pass plus the plain kernel, so the Python
                           operator keeps the stand-alone pass */
  int32_t q_round_half_even; /* rounding of that quantiser, as sqattn_prep_args.round_half_even */
  int32_t head_dim_og;  /* 0 or head_dim: nothing special.  Otherwise the tensors were zero-padded from head_dim_og
                           to head_dim (64 or 128) by the caller and the softmax scale applied when q_is_scaled == 0
                           is 1/sqrt(head_dim_og), as the reference launchers do (sqattn/attn_triton.py:236-253, 314;
                           attn_triton_mix_relative.py:369-385); the caller slices the output back */
} sqattn_prefill_args;

/* Replaces the launch halves of attn_causal / attn_hierarchical_relative_window /
 * attn_hierarchical_window (files above).  Scratch is needed when q has to be scaled
 * (q_is_scaled == 0) and when v is bf16 (the P*V product runs in fp16 like the reference's
 * v.to(fp16), attn_triton.py:84, so a bf16 v is converted once). */
size_t sqattn_prefill_workspace_bytes(const sqattn_prefill_args* args);
int sqattn_prefill(const sqattn_prefill_args* args, sqattn_stream_t stream);

/* ---- adapter input preparation ------------------------------------------------------------ */

enum { SQATTN_QTYPE_INT = 0, SQATTN_QTYPE_E4M3 = 1, SQATTN_QTYPE_E5M2 = 2 };

typedef struct {
  /* inputs as the model hands them over: q [B, N, Hq, D], k/v [B, N, Hkv, D] viewed through strides */
  sqattn_tensor q, k, v;
  /* outputs, contiguous [B, H, N, D] (K/V keep Hkv heads: the reference's repeat_kv copies are
   * bit-identical, so they are not materialised).  q outputs are already multiplied by
   * 1/sqrt(D)*1.44269504 in the input dtype.  v_bit8 is written as fp16. */
  void *q_bit8, *q_bit4, *k_bit8, *k_bit4, *v_bit8;
  int32_t batch, num_q_heads, num_kv_heads, seq_len, head_dim;
  int32_t dtype;             /* input dtype; q/k outputs use it too */
  int32_t qk_qtype, v_qtype; /* SQATTN_QTYPE_* (args.qk_qtype / args.v_qtype of the reference) */
  int32_t round_half_even;   /* 0: ties away from zero (paddle.round); 1: ties to even */
  int32_t skip_bit4;         /* 1: q_bit4/k_bit4 are not needed (not written) */
  void* workspace;           /* device scratch, sqattn_prep_workspace_bytes() bytes (K column sums) */
  size_t workspace_bytes;
  const float* k_mean;       /* optional device [B, Hkv, D] fp32: use this sequence mean of K instead of computing
                                it (sequence-parallel shards pass the mean of the whole sequence) */
  int32_t kv_out_nhd;        /* 1: k_bit8/k_bit4/v_bit8 are written token-major [B, N, Hkv, D] (so that shards
                                all-gather into one contiguous tensor); 0: [B, Hkv, N, D] */
  int32_t parts;             /* bit mask of the tensors to prepare: 1 = Q, 2 = K, 4 = V; 0 means all three.
                                Pipelined callers prepare K and V once and Q chunk by chunk (the unselected
                                pointers may be null) */
} sqattn_prep_args;

/* Replaces attention_fn's input preparation, sqattn/attn_replacer.py:334-365:
 * K minus its sequence mean, INT8/INT4 per-token fake-quant of Q and K, INT8
 * per-(token,channel) fake-quant of V (sqattn/fake_quant.py:23-125, 151-248). */
size_t sqattn_prep_workspace_bytes(const sqattn_prep_args* args);
int sqattn_prep_qkv(const sqattn_prep_args* args, sqattn_stream_t stream);

/* Column sums of K over the sequence, sums[b, h, d] = sum_n k[b, h, n, d] in fp32 (deterministic order): the
 * first half of key.mean(dim=2) (sqattn/attn_replacer.py:338), split out so that sequence-parallel shards can
 * all-reduce their sums.  workspace: batch * num_kv_heads * 64 * head_dim floats. */
int sqattn_k_column_sums(const sqattn_tensor* k, int32_t batch, int32_t num_kv_heads, int32_t seq_len,
                         int32_t head_dim, int32_t dtype, float* sums, void* workspace, size_t workspace_bytes,
                         sqattn_stream_t stream);

/* ---- decode ------------------------------------------------------------------------------- */

struct sqattn_peer_merge_args;

/* Keys and values addressed through an index list instead of a contiguous cache (the attention over the tokens a
 * clustered cache retrieved, without first packing them): key j of (sequence b, KV head h) is row idx[(b * Hkv + h)
 * * cap + j] of the 16-bit matrices k_rows[b * Hkv + h] / v_rows[b * Hkv + h] (device arrays of device pointers),
 * rows row_stride elements apart.  No counterpart in the reference. */
typedef struct sqattn_decode_gather {
  const int32_t* idx;            /* device, [B * Hkv, cap] */
  int32_t cap;
  const void* const* k_rows;     /* device, [B * Hkv] */
  const void* const* v_rows;     /* device, [B * Hkv] */
  int64_t row_stride;            /* elements, a multiple of 8 */
} sqattn_decode_gather;

typedef struct {
  sqattn_tensor q;         /* [B, Hq, 1, D] */
  sqattn_tensor k, v;      /* [B, Hkv, kv_capacity, D] */
  sqattn_tensor_out o;     /* [B, Hq, 1, D] */
  float* lse;              /* optional [B, Hq] fp32 base-2 */
  int32_t batch, num_q_heads, num_kv_heads, head_dim;
  int32_t kv_len;          /* used for every sequence when kv_lens == NULL */
  const int32_t* kv_lens;  /* host, [B] or NULL: ragged batch */
  int32_t dtype, o_dtype;
  int32_t p_fp8;           /* is_P_fp8_quant */
  int32_t q_is_scaled;     /* 0: the kernel applies 1/sqrt(D)*1.44269504 in q's dtype on load */
  int32_t num_splits;      /* 0 = let the length-aware scheduler choose */
  int32_t reference_tail;  /* 1: like the reference kernel (attn_triton_decode.py:215-221), positions between kv_len
                              and the next multiple of 64 count as keys with score 0 and value 0; 0: exact masking */
  void* workspace;         /* device scratch, sqattn_decode_workspace_bytes() bytes */
  size_t workspace_bytes;
  /* multi-GPU split-KV: when partial_o != NULL the merge is skipped and the per-sequence partial
   * (O fp32 [B,Hq,D], LSE fp32 [B,Hq]) of THIS call's keys is written there for sqattn_decode_merge */
  float* partial_o;
  float* partial_lse;
  /* Lengths that live on the device (int32 [B]), for callers that replay a captured CUDA graph while the cache
   * grows: the key ranges are planned on the host for kv_len (the capacity to plan for, kv_lens must be NULL) and
   * the kernel clips every range to the length it reads from this array; ranges past the end contribute nothing. */
  const int32_t* kv_lens_device;
  /* Cross-GPU split-KV in one step: when set, the kernel that merges this call's split-KV partials also exchanges
   * them with the other ranks and merges across ranks (see sqattn_decode_peer_merge; its part_o / part_lse are
   * ignored, its out / lse receive the result; o, lse, partial_o and partial_lse of this struct are not used). */
  const struct sqattn_peer_merge_args* peer;
  int32_t head_dim_og;     /* as in sqattn_prefill_args: the un-padded head_dim the softmax scale is taken from when
                              q_is_scaled == 0 (attn_triton_decode.py:254-271); 0 = head_dim */
  /* When set, k and v are ignored and the keys and values are the listed rows (kv_len = the list capacity to plan
   * for, kv_lens / kv_lens_device = the list lengths); the rows are copied into shared memory by 16-byte
   * asynchronous copies instead of tiled TMA loads.  reference_tail must be 0. */
  const sqattn_decode_gather* gather;
} sqattn_decode_args;

/* Replaces attn_unified's decode branch + _attn_decode_fwd, sqattn/attn_triton_decode.py:175-241,
 * 244-361, as a split-KV kernel.  K is NOT re-centred here (the reference does it per call, 268-269):
 * softmax of one query is invariant to a constant shift of K, so callers centre once or not at all. */
size_t sqattn_decode_workspace_bytes(const sqattn_decode_args* args);
int sqattn_decode(const sqattn_decode_args* args, sqattn_stream_t stream);

/* No counterpart in the reference.  Same computation and results as sqattn_decode, for callers that cannot
 * give it a workspace because they may not allocate device memory where they call from: code running inside
 * a framework's memory-planned region or a serving loop with a frozen memory pool, where a cudaMalloc (or a
 * caching allocator growing its pool) would synchronise the device or is forbidden outright.  The split-KV
 * partials go to a scratch array built into the library (4 MiB + 64 KiB per GPU that loads the library, held
 * until the process exits); args->workspace and workspace_bytes are ignored.  Limits and rules:
 *  - the call is rejected with SQATTN_ERR_WORKSPACE when (key ranges x query heads) partial rows need more than
 *    that (at head_dim 128: 8192 rows, e.g. 292 key ranges of 28 heads); nothing is launched in that case;
 *  - it calls no cudaMalloc/cudaFree and no allocating library routine;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress) with that device
 *    current; make that first call before any stream capture begins;
 *  - all calls on a device share the one array, which keeps the previous call's contents (nothing in it has to
 *    start at zero: every partial row is written before the merge reads it); two calls that overlap on the GPU
 *    (different streams) race on it -- serialise them. */
int sqattn_decode_static_scratch(const sqattn_decode_args* args, sqattn_stream_t stream);

/* Merge num_parts partial results laid out [num_parts, rows, D] / [num_parts, rows] (e.g. the
 * all-gathered per-GPU partials): O = sum 2^(lse_i-max) O_i / sum 2^(lse_i-max).  rows = B*Hq. */
int sqattn_decode_merge(const float* partial_o, const float* partial_lse, int32_t num_parts, int64_t rows,
                        int32_t head_dim, void* o, int32_t o_dtype, float* lse, sqattn_stream_t stream);

/* ---- kmeans (cache_hub/kmeans.py) --------------------------------------------------------- */

/* Scratch of sqattn_kmeans_assign and sqattn_kmeans_index_add (flagged-token list, member lists), 256-byte aligned. */
size_t sqattn_kmeans_workspace_bytes(int32_t groups, int32_t num_tokens, int32_t num_centroids);
/* _triton_assign_kernel, kmeans.py:7-79: idx[g,t] = argmax_c <data[g,t], centroids[g,c]> (lowest c on
 * ties, exact: the fp32 tensor-core scores decide except for near ties, which are re-evaluated in fp64); when sums
 * is given, sums[g,c,:] (fp64, exact) and counts[g,c] hold the members' sum and number (counts must be zeroed by
 * the caller; sums is overwritten).  data [G,T,D], centroids [G,K,D] contiguous, dtype f16/bf16, D in {64,128},
 * K % 32 == 0. */
int sqattn_kmeans_assign(const void* data, const void* centroids, int32_t dtype, int32_t groups,
                         int32_t num_tokens, int32_t num_centroids, int32_t head_dim, int32_t* idx,
                         double* sums, int32_t* counts, void* workspace, size_t workspace_bytes, sqattn_stream_t stream);
/* _triton_update_kernel, kmeans.py:82-124: centroid = sums/counts where counts > 0, optional L2 normalise. */
int sqattn_kmeans_update(void* centroids, int32_t dtype, const double* sums, const int32_t* counts,
                         int32_t groups, int32_t num_centroids, int32_t head_dim, int32_t normalize,
                         sqattn_stream_t stream);
/* triton_reverse_index, kmeans.py:199-262: member lists sorted by token index.
 * cluster_size [G,K] (output), clusters [G,K,max_cluster_size] (zero-filled by the caller); workspace:
 * sqattn_kmeans_workspace_bytes() bytes. */
int sqattn_kmeans_reverse_index(const int32_t* idx, int32_t groups, int32_t num_tokens, int32_t num_centroids,
                                int32_t max_cluster_size, int32_t* clusters, int32_t* cluster_size, void* workspace,
                                size_t workspace_bytes, sqattn_stream_t stream);
/* triton_index_add, kmeans.py:265-329: value sums per cluster; out [G,K,D] in the value dtype.
 * sums_ws: fp64 scratch [G,K,D]; workspace: sqattn_kmeans_workspace_bytes() bytes. */
int sqattn_kmeans_index_add(const void* value, int32_t dtype, const int32_t* idx, int32_t groups,
                            int32_t num_tokens, int32_t num_centroids, int32_t head_dim, double* sums_ws,
                            void* out, void* workspace, size_t workspace_bytes, sqattn_stream_t stream);
/* max over counts[G*K] into *out_max (device int32, zeroed by the caller): data_cnt.max(), kmeans.py:195 */
int sqattn_kmeans_max_count(const int32_t* counts, int64_t n, int32_t* out_max, sqattn_stream_t stream);

/* ---- clustered retrieval (no counterpart in the reference's code; its logs print n_clusters / nprobe / budget
 * arguments of a retrieval step that was not shipped, logs/SQAttn_131072_qwen2.5-7b.log:11,46) ---- */

/* Per KV group g: score_c = <mean over the group's query heads, centroid c> (fp64), clusters taken in descending
 * score (lowest index on ties, empty clusters skipped) until at least `budget` tokens are covered; the tokens of
 * the selected clusters are written to out_idx[g, :out_count[g]] in ascending order (at most `cap`).
 * q [G, heads_per_group, D], centroids [G, K, D], cluster_size [G, K], clusters [G, K, max_cluster_size] as
 * produced by sqattn_kmeans_*; K <= 4096, num_tokens <= 262144.  Tokens [tail_start, num_tokens) are the ones
 * appended since the clusters were last rebuilt: they belong to no cluster yet and are always selected (pass
 * tail_start = num_tokens when there are none). */
int sqattn_retrieve_select(const void* q, const void* centroids, int32_t dtype, const int32_t* cluster_size,
                           const int32_t* clusters, int32_t groups_kv, int32_t heads_per_group, int32_t num_clusters,
                           int32_t head_dim, int32_t max_cluster_size, int32_t num_tokens, int32_t budget,
                           int32_t* out_idx, int32_t* out_count, int32_t cap, int32_t tail_start, sqattn_stream_t stream);
/* dst[g, j, :] = src[g, idx[g, j], :] for j < count[g] (16-bit rows of head_dim elements; strides in elements) */
int sqattn_gather_rows(const void* src, int64_t src_group_stride, int64_t src_row_stride, const int32_t* idx,
                       const int32_t* count, int32_t groups, int32_t cap, int32_t head_dim, void* dst,
                       sqattn_stream_t stream);

/* The two calls above for every sequence of a ragged batch in two launches (select, then gather of keys and
 * values): one item per sequence, the same geometry, budget and cap for all. */
typedef struct sqattn_retrieve_item {
  const void* q;                 /* [G, heads_per_group, D] */
  const void* centroids;         /* [G, K, D] */
  const int32_t* cluster_size;   /* [G, K] */
  const int32_t* clusters;       /* [G, K, max_cluster_size] */
  int32_t num_clusters, max_cluster_size, num_tokens;
  int32_t* out_idx;              /* [G, cap] */
  int32_t* out_count;            /* [G] */
  const void* k_src;             /* [G, tokens, D] through the strides below (elements) */
  const void* v_src;
  int64_t src_group_stride, src_row_stride;
  void* k_dst;                   /* [G, cap, D]; k_dst == v_dst == NULL for every item: select only, no packing */
  void* v_dst;
  int32_t tail_start;            /* as in sqattn_retrieve_select */
  /* block-hybrid caches (cache_hub/cache.py keeps part of the KV on the host): tokens from split_row on are read
   * from k_src2 / v_src2 [G, tokens - split_row, D] (same row stride), which may be pinned host memory mapped
   * into the device's address space; NULL: every token is in k_src / v_src */
  int32_t split_row;
  const void* k_src2;
  const void* v_src2;
  int64_t src2_group_stride;
} sqattn_retrieve_item;
int sqattn_retrieve_batch(const sqattn_retrieve_item* items, int32_t num_items, int32_t dtype, int32_t groups_kv,
                          int32_t heads_per_group, int32_t head_dim, int32_t budget, int32_t cap, sqattn_stream_t stream);

/* ---- window calibration (sqattn/window_search.py) ------------------------------------------------------ */

/* Distance-weighted attention-energy histogram per query head, accumulated into hist [Hq, num_bins] (fp64, not
 * cleared: samples add up like the reference's `histograms[head] += hist`, window_search.py:207-208).
 * relative = 1: compute_relative_attention_histogram_gpu_with_sink (244-283); relative = 0:
 * compute_absolute_attention_histogram_gpu_with_sink (286-321; sink = 0 gives compute_attention_histogram_gpu,
 * 20-48), num_bins = max_len.  The softmax map A = softmax(q k^T / sqrt(D)) with a causal mask
 * (cal_attn_weight, sqattn/attn_replacer.py:253-278) is evaluated blockwise and never stored.
 * q [Hq, N, D], k [Hkv, N, D] contiguous 16-bit. */
int sqattn_window_histogram(const void* q, const void* k, int32_t dtype, int32_t num_q_heads, int32_t num_kv_heads,
                            int32_t seq_len, int32_t head_dim, int32_t relative, int32_t num_bins, int32_t sink,
                            double* hist, sqattn_stream_t stream);

/* ---- cross-GPU merge of decode partials over peer memory (no counterpart in the reference, which has no
 * multi-GPU attention path) ------------------------------------------------------------------------------- */

/* One call per decode step on every rank.  `epoch` points to a device word, zero before the first call, that the
 * kernel itself advances by one (so the same sequence of calls, captured in a CUDA graph, can be replayed); all
 * ranks must have made the same number of calls.  Each rank passes its partial
 * (part_o [rows, head_dim] fp32 already divided by its own sum, part_lse [rows] fp32 base 2, as produced by
 * sqattn_decode with partial_o / partial_lse) and the device pointers of ALL ranks' exchange buffers as mapped
 * in the calling process (symmetric / IPC memory; index = rank).  The kernel stores the partial into every
 * rank's data buffer with plain peer stores (every value as one 8-byte word that also carries the step number, so
 * no flag or fence is needed), waits at most one second for the other ranks' words to arrive in its own buffer
 * (then the output is NaN and SQATTN_ERR_DEVICE_TIMEOUT is reported by sqattn_check_device_status) and writes the
 * merged result.
 * Buffers: data = sqattn_peer_merge_data_bytes(), flags = sqattn_peer_merge_flag_bytes(), zeroed once before the
 * first call.  At most 16 ranks. */
typedef struct sqattn_peer_merge_args {
  void* peer_data[16];
  void* peer_flags[16];
  int32_t rank, world;
  int32_t rows, rows_cap, head_dim;
  uint32_t* epoch;      /* device step counter, see above */
  const float* part_o;
  const float* part_lse;
  void* out;            /* [rows, head_dim] in o_dtype */
  int32_t o_dtype;
  float* lse;           /* optional [rows] */
} sqattn_peer_merge_args;
size_t sqattn_peer_merge_data_bytes(int32_t world, int32_t rows_cap, int32_t head_dim);
size_t sqattn_peer_merge_flag_bytes(int32_t world, int32_t rows_cap);
int sqattn_decode_peer_merge(const sqattn_peer_merge_args* args, sqattn_stream_t stream);

/* ---- decoder-layer row kernels: the caller's side of the operator (model_hub/utils.py) ------------------- */

/* out[r, :] = (x[r, :] * rsqrt(mean(x[r, :]^2) + eps)) * weight, rmsnorm (model_hub/utils.py:14-18); 16-bit rows
 * with element strides, dim a multiple of 8; x and out may alias. */
int sqattn_rmsnorm(const void* x, const void* weight, void* out, int64_t rows, int32_t dim, int64_t x_row_stride,
                   int64_t out_row_stride, float eps, int32_t dtype, sqattn_stream_t stream);
/* apply_rope_with_cos_sin_cache_inplace (model_hub/utils.py:20-106) on the fused QKV projection: the first
 * num_heads heads (query heads then key heads) of every row [rows, row_stride] are rotated in place with
 * cos|sin = cos_sin_cache[pos0 + row % seq_len] (fp32 [cache_rows, head_dim]). */
int sqattn_rope_qk(void* qkv, int64_t row_stride, int64_t rows, int32_t seq_len, int32_t num_heads, int32_t head_dim,
                   const float* cos_sin_cache, int64_t cache_rows, int64_t pos0, int32_t dtype, sqattn_stream_t stream);
/* The same with the first position read from a device word (int64) at run time, added to pos0: for callers that
 * replay a captured graph while the position advances.  Positions past the table are clamped to its last row. */
int sqattn_rope_qk_devpos(void* qkv, int64_t row_stride, int64_t rows, int32_t seq_len, int32_t num_heads,
                          int32_t head_dim, const float* cos_sin_cache, int64_t cache_rows, int64_t pos0,
                          const int64_t* pos_device, int32_t dtype, sqattn_stream_t stream);
/* silu_and_mul (model_hub/utils.py:4-12): x [rows, 2*inter] -> out [rows, inter] = x[:, inter:] * silu(x[:, :inter]) */
int sqattn_silu_mul(const void* x, void* out, int64_t rows, int32_t inter, int32_t dtype, sqattn_stream_t stream);

/* ---- KV cache block mover (cache_hub/flash_attn_cache.py:7-19, 143-151, 200-227) ---------- */

/* Gather rows [row0, row0+rows) of a [*, row_elems] 16-bit matrix that lives in (pinned) host or device
 * memory into dst with one cudaMemcpy2DAsync on the given (side) stream. */
int sqattn_cache_copy_rows(void* dst, int64_t dst_row_stride_bytes, const void* src, int64_t src_row_stride_bytes,
                           int64_t row_bytes, int64_t rows, int32_t to_device, sqattn_stream_t stream);

/* The decode-time append of flash_attn_cache.decode_update_kv_cache (cache_hub/flash_attn_cache.py:239-256):
 * k_cache[b, positions[b], :] = k_new[b, :] and the same for v, for every sequence b, in one launch.  Caches are
 * [batch, capacity, row_elems] 16-bit through the two strides (elements), k_new / v_new [batch, row_elems] with
 * new_seq_stride between sequences, positions a DEVICE int64 [batch] (so a captured graph can be replayed while
 * they advance); positions outside [0, capacity) are skipped.  row_elems = Hkv * head_dim, a multiple of 8. */
int sqattn_cache_append(void* k_cache, void* v_cache, const void* k_new, const void* v_new, const int64_t* positions,
                        int64_t cache_seq_stride, int64_t cache_row_stride, int64_t new_seq_stride, int32_t batch,
                        int32_t row_elems, int64_t capacity, sqattn_stream_t stream);

/* ---- diagnostics -------------------------------------------------------------------------- */

/* Device-side waits (TMA / tensor-core completion barriers, the peer wait of the cross-GPU merge) are bounded; a
 * wait that gives up records a code in a device word that this call reads back and clears (it synchronises the
 * stream).  Returns SQATTN_OK or SQATTN_ERR_DEVICE_TIMEOUT.  While the word is set, every later attention or
 * decode launch on that device fills its output with NaN instead of computing (the failure cannot pass for a
 * result), until this call has cleared it. */
int sqattn_check_device_status(sqattn_stream_t stream);
/* Optional mirror of that word in host memory, so that a caller can notice a failure without synchronising:
 * host_word is a caller-owned int32 in pinned, device-mapped host memory (or NULL to switch the mirror off) that
 * must stay valid while kernels of this library may run on the current device; a wait that gives up also stores
 * its code there.  The caller reads (and clears) the word itself; sqattn_check_device_status does not touch it. */
int sqattn_set_status_mirror(int32_t* host_word);
const char* sqattn_last_error_string(void);
int sqattn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SQATTN_B200_H_ */
