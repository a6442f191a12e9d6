// C ABI of the library (declared in include/sqattn_b200.h).  Host-side argument checking, TMA descriptor
// construction, the length-aware decode scheduler and the kernel launches.  One translation unit.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "decode.cuh"
#include "decoder_ops.cuh"
#include "kmeans.cuh"
#include "kmeans_tc.cuh"
#include "peer_exchange.cuh"
#include "prefill.cuh"
#include "prep.cuh"
#include "retrieval.cuh"
#include "window_search.cuh"

using namespace sq;

namespace {

// softmax scale in the base-2 domain; head_dim_og > 0: the tensors were zero-padded from that head_dim and the
// scale follows the original one (sqattn/attn_triton.py:249-253)
double sm_scale_log2(int head_dim, int head_dim_og = 0) {
  return 1.0 / sqrt(static_cast<double>(head_dim_og > 0 ? head_dim_og : head_dim)) * 1.44269504;
}

// Launch with programmatic stream serialisation: the grid may become resident while the kernel before it in the
// stream drains; the kernel itself waits (griddepcontrol.wait) before it reads anything an earlier kernel produced.
// Which kernels get it is a measured choice (1M-token decode sharded over 2 GPUs, 28 layers per step, graph replay):
// none 4.806 ms, the merge kernels only 4.800 ms, merge and decode kernels 5.245 ms (a decode grid that becomes
// resident behind the running one slows it down), so only the merges do by default.
// SQATTN_B200_OVERLAP (read once) overrides with a bit mask of kernel classes: 1 = merge kernels, 2 = decode kernel.
int overlap_mask() {
  static int mask = -1;
  if (mask < 0) {
    const char* e = getenv("SQATTN_B200_OVERLAP");
    mask = (e && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 1;
  }
  return mask;
}
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(int klass, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = (overlap_mask() & klass) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

int elementwise_grid(long long work_items, int block) {
  long long g = (work_items + block - 1) / block;
  const long long cap = 148ll * 16;  // a few waves of the 148 SMs; kernels use grid-stride loops
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

View4 view_of(const sqattn_tensor& t, int b, int h, int n, int d) {
  View4 v;
  v.ptr = static_cast<const uint8_t*>(t.ptr);
  v.sb = t.stride_b; v.sh = t.stride_h; v.sn = t.stride_n;
  v.b = b; v.h = h; v.n = n; v.d = d;
  return v;
}

bool aligned16(const sqattn_tensor& t) {
  return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && (t.stride_b % 8 == 0) && (t.stride_h % 8 == 0) &&
         (t.stride_n % 8 == 0);
}

// relative window size: ((int64)(ratio_f32 * kv_len) + 127) / 128 * 128 (attn_triton_mix_relative.py:43-46)
int relative_window(float ratio, int kv_len) {
  const float prod = ratio * static_cast<float>(kv_len);
  long long raw = static_cast<long long>(prod);
  long long w = (raw + 127) / 128 * 128;
  if (w > 0x3fffffff) w = 0x3fffffff;
  if (w < -0x3fffffff) w = -0x3fffffff;
  return static_cast<int>(w);
}

struct PrefillPlan {
  size_t q8_off, q4_off, v_off, total;
  bool scale_q, scale_q4, convert_v;
};

int plan_prefill(const sqattn_prefill_args* a, PrefillPlan* pl) {
  if (!a) return fail(SQATTN_ERR_INVALID_ARG, "args is null");
  if (a->head_dim != 64 && a->head_dim != 128)
    return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128 (pad like the reference does)", a->head_dim);
  if (a->batch <= 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || a->qo_len <= 0 || a->kv_len <= 0)
    return fail(SQATTN_ERR_INVALID_ARG, "batch/heads/lengths must be positive");
  if (a->num_q_heads % a->num_kv_heads) return fail(SQATTN_ERR_INVALID_ARG, "num_q_heads must be a multiple of num_kv_heads");
  if (a->num_q_heads > kMaxHeads) return fail(SQATTN_ERR_UNSUPPORTED, "more than %d query heads", kMaxHeads);
  if (a->head_dim_og < 0 || a->head_dim_og > a->head_dim)
    return fail(SQATTN_ERR_INVALID_ARG, "head_dim_og %d must lie in [0, head_dim %d]", a->head_dim_og, a->head_dim);
  if (a->q_row_offset < 0 || a->q_row_offset % 128)
    return fail(SQATTN_ERR_INVALID_ARG, "q_row_offset must be a non-negative multiple of 128, got %d", a->q_row_offset);
  if (a->q_split_rows < 0 || a->q_split_rows % 128 || a->q_split_rows > a->qo_len || a->q_row_offset2 < 0 || a->q_row_offset2 % 128)
    return fail(SQATTN_ERR_INVALID_ARG, "q_split_rows (%d) and q_row_offset2 (%d) must be non-negative multiples of 128, "
                "q_split_rows at most qo_len", a->q_split_rows, a->q_row_offset2);
  {
    // every row range of the shard must end inside the sequence, and on a 128-row boundary unless it ends the sequence
    const int len_a = a->q_split_rows > 0 ? a->q_split_rows : a->qo_len;
    const int end_a = a->q_row_offset + len_a;
    const int end_b = a->q_split_rows > 0 ? a->q_row_offset2 + (a->qo_len - a->q_split_rows) : end_a;
    const bool ok_a = end_a == a->kv_len || (end_a < a->kv_len && len_a % 128 == 0);
    const bool ok_b = end_b == a->kv_len || (end_b < a->kv_len && (a->qo_len - a->q_split_rows) % 128 == 0);
    if (!ok_a || !ok_b)
      return fail(SQATTN_ERR_INVALID_ARG, "qo_len and kv_len must be equal for causal attention "
                  "(a shard of query rows needs every row range to end at or before kv_len, on a multiple of 128 rows "
                  "unless it ends the sequence)");
  }
  const bool windows = a->mode != SQATTN_MODE_DENSE_CAUSAL;
  const bool alias = !windows || (a->q_int4.ptr == a->q_int8.ptr && a->k_int4.ptr == a->k_int8.ptr);
  const size_t qbytes = static_cast<size_t>(a->batch) * a->num_q_heads * a->qo_len * a->head_dim * 2;
  const size_t vbytes = static_cast<size_t>(a->batch) * a->num_kv_heads * a->kv_len * a->head_dim * 2;
  if (a->q_fake_quant < 0 || a->q_fake_quant > 3)
    return fail(SQATTN_ERR_INVALID_ARG, "q_fake_quant %d: 0 (none) or a quantiser type + 1", a->q_fake_quant);
  if (a->q_fake_quant && !alias)
    return fail(SQATTN_ERR_INVALID_ARG, "in-kernel fake-quant of q needs one operand set (q_int4 == q_int8, k_int4 == k_int8)");
  pl->scale_q = !a->q_is_scaled && !a->q_fake_quant;   // the in-kernel quantiser applies the softmax scale itself
  pl->scale_q4 = pl->scale_q && !alias;
  pl->convert_v = a->v_dtype == SQATTN_BF16;
  size_t off = 0;
  pl->q8_off = off; if (pl->scale_q) off += align_up(qbytes, 1024);
  pl->q4_off = off; if (pl->scale_q4) off += align_up(qbytes, 1024);
  pl->v_off = off; if (pl->convert_v) off += align_up(vbytes, 1024);
  pl->total = off;
  return SQATTN_OK;
}

template <int D>
int launch_prefill(const sqattn_prefill_args* a, const PrefillPlan& pl, cudaStream_t stream, float* dump,
                   long long* dump_t = nullptr, float* dump_p = nullptr) {
  const int B = a->batch, Hq = a->num_q_heads, Hkv = a->num_kv_heads, N = a->qo_len;
  const bool windows = a->mode != SQATTN_MODE_DENSE_CAUSAL;
  const bool alias = !windows || (a->q_int4.ptr == a->q_int8.ptr && a->k_int4.ptr == a->k_int8.ptr);
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const float scale = static_cast<float>(sm_scale_log2(D, a->head_dim_og));
  const bool bf16 = a->qk_dtype == SQATTN_BF16;

  sqattn_tensor q8 = a->q_int8, q4 = alias ? a->q_int8 : a->q_int4, v = a->v;
  const int64_t cont_q[3] = {static_cast<int64_t>(Hq) * N * D, static_cast<int64_t>(N) * D, D};
  const int64_t cont_v[3] = {static_cast<int64_t>(Hkv) * a->kv_len * D, static_cast<int64_t>(a->kv_len) * D, D};
  if (pl.scale_q) {
    View4 in = view_of(a->q_int8, B, Hq, N, D);
    const int grid = elementwise_grid(static_cast<long long>(B) * Hq * N * (D / 8), 256);
    if (bf16) strided_map_kernel<true, 0><<<grid, 256, 0, stream>>>(in, ws + pl.q8_off, scale);
    else strided_map_kernel<false, 0><<<grid, 256, 0, stream>>>(in, ws + pl.q8_off, scale);
    q8 = sqattn_tensor{ws + pl.q8_off, cont_q[0], cont_q[1], cont_q[2]};
    if (pl.scale_q4) {
      View4 in4 = view_of(a->q_int4, B, Hq, N, D);
      if (bf16) strided_map_kernel<true, 0><<<grid, 256, 0, stream>>>(in4, ws + pl.q4_off, scale);
      else strided_map_kernel<false, 0><<<grid, 256, 0, stream>>>(in4, ws + pl.q4_off, scale);
      q4 = sqattn_tensor{ws + pl.q4_off, cont_q[0], cont_q[1], cont_q[2]};
    } else {
      q4 = q8;
    }
  }
  if (pl.convert_v) {
    View4 in = view_of(a->v, B, Hkv, a->kv_len, D);
    const int grid = elementwise_grid(static_cast<long long>(B) * Hkv * a->kv_len * (D / 8), 256);
    strided_map_kernel<true, 1><<<grid, 256, 0, stream>>>(in, ws + pl.v_off, 1.0f);
    v = sqattn_tensor{ws + pl.v_off, cont_v[0], cont_v[1], cont_v[2]};
  }
  SQ_CUDA(cudaGetLastError());

  CUtensorMap tq8, tq4, tk8, tk4, tv;
  int rc;
  if ((rc = make_tmap_bhnd(&tq8, q8.ptr, a->qk_dtype, q8.stride_b, q8.stride_h, q8.stride_n, B, Hq, N, D, kBlockM, "q_int8"))) return rc;
  if ((rc = make_tmap_bhnd(&tq4, q4.ptr, a->qk_dtype, q4.stride_b, q4.stride_h, q4.stride_n, B, Hq, N, D, kBlockM, "q_int4"))) return rc;
  if ((rc = make_tmap_bhnd(&tk8, a->k_int8.ptr, a->qk_dtype, a->k_int8.stride_b, a->k_int8.stride_h, a->k_int8.stride_n, B, Hkv, a->kv_len, D, kBlockN, "k_int8"))) return rc;
  const sqattn_tensor& k4 = alias ? a->k_int8 : a->k_int4;
  if ((rc = make_tmap_bhnd(&tk4, k4.ptr, a->qk_dtype, k4.stride_b, k4.stride_h, k4.stride_n, B, Hkv, a->kv_len, D, kBlockN, "k_int4"))) return rc;
  if ((rc = make_tmap_bhnd(&tv, v.ptr, SQATTN_F16, v.stride_b, v.stride_h, v.stride_n, B, Hkv, a->kv_len, D, kBlockN, "v"))) return rc;

  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.o = a->o.ptr; p.o_sb = a->o.stride_b; p.o_sh = a->o.stride_h; p.o_sn = a->o.stride_n;
  p.lse = a->lse; p.dump = dump; p.dump_t = dump_t; p.dump_p = dump_p;
  p.batch = B; p.hq = Hq; p.hkv = Hkv; p.groups = Hq / Hkv; p.n = N; p.kv_len = a->kv_len;
  p.mode = a->mode; p.sink = a->sink_size; p.p_fp8_mode = a->p_fp8_mode; p.o_dtype = a->o_dtype;
  p.qk_bf16 = bf16; p.same_opset = alias; p.nblk = (N + kBlockM - 1) / kBlockM;
  p.blk0 = a->q_row_offset / kBlockM; p.n_total = a->kv_len;
  p.q_fake_quant = a->q_fake_quant; p.q_half_even = a->q_round_half_even; p.q_scale = scale;
  p.blk_split = a->q_split_rows > 0 ? a->q_split_rows / kBlockM : p.nblk;
  p.blk0_b = a->q_row_offset2 / kBlockM;
  for (int h = 0; h < Hq; ++h) {
    if (a->mode == SQATTN_MODE_RELATIVE_WINDOW) {
      p.w8[h] = relative_window(a->win8_ratios[h], a->kv_len);
      p.w4[h] = relative_window(a->win4_ratios[h], a->kv_len);
    } else if (a->mode == SQATTN_MODE_ABSOLUTE_WINDOW) {
      p.w8[h] = a->win8_sizes[h];
      p.w4[h] = a->win4_sizes[h];
    }
  }
  const long long grid = static_cast<long long>(p.nblk) * Hq * B;
  if (grid > 0x7fffffffll) return fail(SQATTN_ERR_UNSUPPORTED, "grid too large");
#define SQ_LAUNCH_PREFILL(KS, VS, MINB)                                                                                 \
  do {                                                                                                                   \
    using L = PrefillSmem<D, KS, VS>;                                                                                    \
    if (dump || dump_t || dump_p) {                                                                                                \
      SQ_CUDA(cudaFuncSetAttribute(prefill_kernel<D, true, KS, VS, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes)); \
      prefill_kernel<D, true, KS, VS, MINB><<<static_cast<unsigned>(grid), 192, L::kDynBytes, stream>>>(tq8, tq4, tk8, tk4, tv, p);    \
    } else {                                                                                                             \
      SQ_CUDA(cudaFuncSetAttribute(prefill_kernel<D, false, KS, VS, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes)); \
      prefill_kernel<D, false, KS, VS, MINB><<<static_cast<unsigned>(grid), 192, L::kDynBytes, stream>>>(tq8, tq4, tk8, tk4, tv, p);   \
    }                                                                                                                    \
  } while (0)
  SQ_LAUNCH_PREFILL(2, 3, 2);  // two K stages (tied to the two S buffers), three V stages, two CTAs per SM
#undef SQ_LAUNCH_PREFILL
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int prefill_impl(const sqattn_prefill_args* a, cudaStream_t stream, float* dump, long long* dump_t = nullptr,
                 float* dump_p = nullptr) {
  PrefillPlan pl;
  int rc = plan_prefill(a, &pl);
  if (rc) return rc;
  if (!a->q_int8.ptr || !a->k_int8.ptr || !a->v.ptr || !a->o.ptr) return fail(SQATTN_ERR_INVALID_ARG, "null tensor pointer");
  if (a->mode < 0 || a->mode > 2) return fail(SQATTN_ERR_INVALID_ARG, "unknown mode %d", a->mode);
  if (a->p_fp8_mode < 0 || a->p_fp8_mode > 2) return fail(SQATTN_ERR_INVALID_ARG, "unknown p_fp8_mode %d", a->p_fp8_mode);
  if (a->mode != SQATTN_MODE_DENSE_CAUSAL) {
    if (a->sink_size < 0) return fail(SQATTN_ERR_INVALID_ARG, "sink_size must be a non-negative integer, got %d", a->sink_size);
    if (!a->q_int4.ptr || !a->k_int4.ptr) return fail(SQATTN_ERR_INVALID_ARG, "null int4 operand pointer");
    if (a->mode == SQATTN_MODE_RELATIVE_WINDOW) {
      if (a->sink_size % 64) return fail(SQATTN_ERR_INVALID_ARG, "relative windows need sink_size %% 64 == 0 (64-key tiles), got %d", a->sink_size);
      if (!a->win8_ratios || !a->win4_ratios) return fail(SQATTN_ERR_INVALID_ARG, "window ratios missing");
    } else if (!a->win8_sizes || !a->win4_sizes) {
      return fail(SQATTN_ERR_INVALID_ARG, "window sizes missing");
    }
  }
  if (!aligned16(a->q_int8) || !aligned16(a->k_int8) || !aligned16(a->v))
    return fail(SQATTN_ERR_INVALID_ARG, "q/k/v need 16-byte aligned pointers and strides that are multiples of 8 elements");
  if ((reinterpret_cast<uintptr_t>(a->o.ptr) % 16) || (a->o.stride_n % 8) || (a->o.stride_h % 8) || (a->o.stride_b % 8))
    return fail(SQATTN_ERR_INVALID_ARG, "o needs a 16-byte aligned pointer and strides that are multiples of 8 elements");
  if (pl.total > 0 && (!a->workspace || a->workspace_bytes < pl.total || (reinterpret_cast<uintptr_t>(a->workspace) % 1024)))
    return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes (1024-byte aligned) required", pl.total);
  return a->head_dim == 128 ? launch_prefill<128>(a, pl, stream, dump, dump_t, dump_p)
                            : launch_prefill<64>(a, pl, stream, dump, dump_t, dump_p);
}

// ---- decode scheduling ---------------------------------------------------------------------------------
struct DecodePlan {
  int chunk;
  int total_items;
  int prefix[kDecMaxBatch + 1];
  int lens[kDecMaxBatch];
};

// Length-aware scheduler: every work item covers `chunk` keys of one sequence; chunk is chosen so that all
// sequences together give about ONE CTA per SM, never less than 256 keys per item.  Measured on B200 (1M keys,
// 28/4 heads): one CTA per SM keeps 96 KB of loads in flight per SM, which already saturates HBM (6.6 TB/s), and
// every further split only adds partial rows for the merge to read: 148 / 296 / 596 CTAs gave 162.7 / 165 / 178
// microseconds per 1 GB layer shard and 4.3 / 7 / 16 microseconds of merge.
int plan_decode(const sqattn_decode_args* a, DecodePlan* pl) {
  if (!a) return fail(SQATTN_ERR_INVALID_ARG, "args is null");
  if (a->head_dim != 64 && a->head_dim != 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128", a->head_dim);
  if (a->batch <= 0 || a->batch > kDecMaxBatch) return fail(SQATTN_ERR_UNSUPPORTED, "batch must be in [1, %d]", kDecMaxBatch);
  if (a->num_kv_heads <= 0 || a->num_q_heads % a->num_kv_heads) return fail(SQATTN_ERR_INVALID_ARG, "bad head counts");
  if (a->num_q_heads / a->num_kv_heads > 16) return fail(SQATTN_ERR_UNSUPPORTED, "more than 16 query heads per KV head");
  if (a->head_dim_og < 0 || a->head_dim_og > a->head_dim)
    return fail(SQATTN_ERR_INVALID_ARG, "head_dim_og %d must lie in [0, head_dim %d]", a->head_dim_og, a->head_dim);
  if (a->kv_lens_device && a->kv_lens) return fail(SQATTN_ERR_INVALID_ARG, "kv_lens and kv_lens_device are exclusive: device lengths are planned for kv_len");
  if (a->gather) {
    const sqattn_decode_gather* g = a->gather;
    if (!g->idx || !g->k_rows || !g->v_rows) return fail(SQATTN_ERR_INVALID_ARG, "gather: null pointer");
    if (g->cap <= 0 || g->row_stride < a->head_dim || g->row_stride % 8)
      return fail(SQATTN_ERR_INVALID_ARG, "gather: cap %d must be positive, row_stride %lld a multiple of 8 not below head_dim", g->cap, static_cast<long long>(g->row_stride));
    if (a->reference_tail) return fail(SQATTN_ERR_INVALID_ARG, "gather: reference_tail is not supported");
    for (int b = 0; b < a->batch; ++b)
      if ((a->kv_lens ? a->kv_lens[b] : a->kv_len) > g->cap)
        return fail(SQATTN_ERR_INVALID_ARG, "gather: sequence %d has more keys than the index list holds (%d)", b, g->cap);
  }
  long long total_tiles = 0;
  for (int b = 0; b < a->batch; ++b) {
    const int len = a->kv_lens ? a->kv_lens[b] : a->kv_len;
    if (len < 0) return fail(SQATTN_ERR_INVALID_ARG, "kv length of sequence %d is %d", b, len);
    if (a->kv_lens && a->kv_len > 0 && len > a->kv_len)
      return fail(SQATTN_ERR_INVALID_ARG, "kv length of sequence %d is %d but the cache holds %d keys", b, len, a->kv_len);
    pl->lens[b] = len;
    total_tiles += (len + kDecTile - 1) / kDecTile;
  }
  int chunk;
  if (a->num_splits > 0) {
    int maxlen = 0;
    for (int b = 0; b < a->batch; ++b) maxlen = pl->lens[b] > maxlen ? pl->lens[b] : maxlen;
    chunk = (maxlen + a->num_splits - 1) / a->num_splits;
  } else {
    const long long target = (148ll + a->num_kv_heads - 1) / a->num_kv_heads;  // items per KV head
    chunk = static_cast<int>((total_tiles + target - 1) / target) * kDecTile;
  }
  chunk = (chunk + kDecTile - 1) / kDecTile * kDecTile;
  if (chunk < 256) chunk = 256;
  pl->chunk = chunk;
  int items = 0;
  for (int b = 0; b < a->batch; ++b) {
    pl->prefix[b] = items;
    items += (pl->lens[b] + chunk - 1) / chunk;
  }
  pl->prefix[a->batch] = items;
  pl->total_items = items;
  return SQATTN_OK;
}

size_t decode_ws_bytes(const sqattn_decode_args* a, const DecodePlan& pl) {
  // a sequence of length 0 has no work item (a rank of a sharded cache may hold none of its keys)
  const size_t rows = static_cast<size_t>(pl.total_items > 0 ? pl.total_items : 1) * a->num_q_heads;
  return align_up(rows * a->head_dim * 4, 256) + align_up(rows * 4, 256);
}

// ---- cross-GPU merge over peer memory --------------------------------------------------------------------
int fill_peer_params(const sqattn_peer_merge_args* a, PeerMergeParams* p) {
  if (a->world < 1 || a->world > kPeerMaxWorld || a->rank < 0 || a->rank >= a->world)
    return fail(SQATTN_ERR_INVALID_ARG, "peer merge: rank %d of %d (at most %d ranks)", a->rank, a->world, kPeerMaxWorld);
  if (a->rows <= 0 || a->rows > a->rows_cap || a->head_dim <= 0 || a->head_dim > 128)
    return fail(SQATTN_ERR_INVALID_ARG, "peer merge: rows %d (capacity %d), head_dim %d", a->rows, a->rows_cap, a->head_dim);
  if (!a->out) return fail(SQATTN_ERR_INVALID_ARG, "peer merge: null output pointer");
  if (!a->epoch) return fail(SQATTN_ERR_INVALID_ARG, "peer merge: the device step counter is null");
  memset(p, 0, sizeof(*p));
  for (int w = 0; w < a->world; ++w) {
    if (!a->peer_data[w] || !a->peer_flags[w]) return fail(SQATTN_ERR_INVALID_ARG, "peer merge: buffer of rank %d is null", w);
    p->data[w] = static_cast<unsigned long long*>(a->peer_data[w]);
    p->flags[w] = static_cast<uint32_t*>(a->peer_flags[w]);
  }
  p->out = a->out; p->lse = a->lse;
  p->rank = a->rank; p->world = a->world; p->rows = a->rows; p->rows_cap = a->rows_cap; p->d = a->head_dim;
  p->o_dtype = a->o_dtype == SQATTN_BF16 ? 1 : 0;
  p->epoch_ptr = a->epoch;
  p->done = p->flags[a->rank] + static_cast<size_t>(a->world) * a->rows_cap;  // the word behind this rank's flags
  return SQATTN_OK;
}

template <int D, bool BF16>
int launch_decode(const sqattn_decode_args* a, const DecodePlan& pl, cudaStream_t stream) {
  CUtensorMap tk, tv;
  int rc;
  // the maps cover the whole cache capacity of each sequence; lengths are enforced in the kernel
  int cap = 1;
  for (int b = 0; b < a->batch; ++b) cap = pl.lens[b] > cap ? pl.lens[b] : cap;
  if (a->gather) {   // the listed rows are copied by the producer warp itself: the maps are never used
    memset(&tk, 0, sizeof(tk));
    memset(&tv, 0, sizeof(tv));
  } else {
    if ((rc = make_tmap_bhnd(&tk, a->k.ptr, a->dtype, a->k.stride_b, a->k.stride_h, a->k.stride_n, a->batch, a->num_kv_heads, cap, D, kDecTile, "k"))) return rc;
    if ((rc = make_tmap_bhnd(&tv, a->v.ptr, a->dtype, a->v.stride_b, a->v.stride_h, a->v.stride_n, a->batch, a->num_kv_heads, cap, D, kDecTile, "v"))) return rc;
  }
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  if (a->gather) {
    p.gather_idx = a->gather->idx; p.gather_cap = a->gather->cap; p.gather_row_stride = a->gather->row_stride;
    p.gather_k = reinterpret_cast<const uint8_t* const*>(a->gather->k_rows);
    p.gather_v = reinterpret_cast<const uint8_t* const*>(a->gather->v_rows);
  }
  p.q = static_cast<const uint8_t*>(a->q.ptr); p.q_sb = a->q.stride_b; p.q_sh = a->q.stride_h;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const size_t rows = static_cast<size_t>(pl.total_items > 0 ? pl.total_items : 1) * a->num_q_heads;
  p.part_o = reinterpret_cast<float*>(ws);
  p.part_lse = reinterpret_cast<float*>(ws + align_up(rows * D * 4, 256));
  p.batch = a->batch; p.hq = a->num_q_heads; p.hkv = a->num_kv_heads; p.groups = a->num_q_heads / a->num_kv_heads; p.d = D;
  p.chunk = pl.chunk; p.p_fp8 = a->p_fp8; p.q_is_scaled = a->q_is_scaled; p.reference_tail = a->reference_tail;
  p.sm_scale = static_cast<float>(sm_scale_log2(D, a->head_dim_og));
  memcpy(p.lens, pl.lens, sizeof(int) * a->batch);
  p.lens_dev = a->kv_lens_device;
  memcpy(p.item_prefix, pl.prefix, sizeof(int) * (a->batch + 1));
  using L = DecodeSmem<D>;
  // a function attribute belongs to the current device: set on every call, like the prefill launch does
  SQ_CUDA(cudaFuncSetAttribute(decode_kernel<D, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynBytes));
  PeerMergeParams pm;
  if (a->peer) {  // checked before anything is launched
    if ((rc = fill_peer_params(a->peer, &pm))) return rc;
    if (a->peer->rows != a->batch * a->num_q_heads || a->peer->head_dim != D)
      return fail(SQATTN_ERR_INVALID_ARG, "peer merge: %d rows x %d expected, exchange describes %d x %d",
                  a->batch * a->num_q_heads, D, a->peer->rows, a->peer->head_dim);
  }
  if (pl.total_items > 0) {
    dim3 grid(pl.total_items, a->num_kv_heads);
    SQ_CUDA(launch_overlapped(2, decode_kernel<D, BF16>, grid, dim3(192), L::kDynBytes, stream, tk, tv, p));
  }

  if (a->peer) {
    // the split-KV merge, the exchange with the other GPUs and the merge across GPUs in one kernel
    pm.part_o = p.part_o; pm.part_lse = p.part_lse; pm.split_mode = 1; pm.hq = a->num_q_heads;
    memcpy(pm.item_prefix, pl.prefix, sizeof(int) * (a->batch + 1));
    SQ_CUDA(launch_overlapped(1, peer_merge_kernel, dim3(pm.rows), dim3(128 * kMergeGroups), 0, stream, pm));
    return SQATTN_OK;
  }
  MergeParams m;
  memset(&m, 0, sizeof(m));
  m.part_o = p.part_o; m.part_lse = p.part_lse;
  m.hq = a->num_q_heads; m.d = D; m.ragged = 1; m.rows = static_cast<long long>(a->batch) * a->num_q_heads;
  memcpy(m.item_prefix, pl.prefix, sizeof(int) * (a->batch + 1));
  if (a->partial_o) {
    m.o = a->partial_o; m.lse = a->partial_lse; m.o_f32 = 1; m.contiguous = 1;
  } else {
    m.o = a->o.ptr; m.lse = a->lse; m.o_dtype = a->o_dtype; m.o_sb = a->o.stride_b; m.o_sh = a->o.stride_h;
  }
  SQ_CUDA(launch_overlapped(1, decode_merge_kernel, dim3(static_cast<unsigned>(m.rows)), dim3(128 * kMergeGroups), 0, stream, m));
  return SQATTN_OK;
}

// ---- kmeans helpers ----------------------------------------------------------------------------------------
// scratch of the clustering entry points: [max centroid norm per group | flagged count | flagged list | arrival
// slot per token | offsets per cluster | member list per group | counts per cluster (index_add only)]
struct KmWorkspace {
  float* max_cnorm2; int* flagged_count; int* flagged; int* slot; int* offsets; int* members; int* counts;
  int flagged_cap;
  size_t total;
};
KmWorkspace km_workspace(void* base, int32_t groups, int32_t num_tokens, int32_t num_centroids) {
  KmWorkspace w;
  const size_t gt = static_cast<size_t>(groups) * num_tokens, gk = static_cast<size_t>(groups) * num_centroids;
  w.flagged_cap = static_cast<int>(gt / 16 > 4096 ? gt / 16 : 4096);
  uint8_t* p = static_cast<uint8_t*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) { uint8_t* r = p ? p + off : nullptr; off += align_up(bytes, 256); return r; };
  w.max_cnorm2 = reinterpret_cast<float*>(take(groups * sizeof(float)));
  w.flagged_count = reinterpret_cast<int*>(take(sizeof(int)));
  w.flagged = reinterpret_cast<int*>(take(static_cast<size_t>(w.flagged_cap) * sizeof(int)));
  w.slot = reinterpret_cast<int*>(take(gt * sizeof(int)));
  w.offsets = reinterpret_cast<int*>(take(gk * sizeof(int)));
  w.members = reinterpret_cast<int*>(take(gt * sizeof(int)));
  w.counts = reinterpret_cast<int*>(take(gk * sizeof(int)));
  w.total = off;
  return w;
}

// members of every cluster (arrival order) from the assignments, then exact fp64 sums of x over them
template <int D, bool BF16>
int km_member_sums(const uint8_t* x, const int32_t* idx, int32_t groups, int32_t num_tokens, int32_t num_centroids,
                          const KmWorkspace& w, int32_t* counts, double* sums, cudaStream_t stream) {
  const long long gt = static_cast<long long>(groups) * num_tokens, gk = static_cast<long long>(groups) * num_centroids;
  kmeans_count_kernel<<<elementwise_grid(gt, 256), 256, 0, stream>>>(idx, counts, w.slot, gt, num_tokens, num_centroids);
  kmeans_offsets_kernel<<<groups, 1024, 0, stream>>>(counts, w.offsets, num_centroids);
  kmeans_scatter_kernel<<<elementwise_grid(gt, 256), 256, 0, stream>>>(idx, w.slot, w.offsets, w.members, gt, num_tokens, num_centroids);
  kmeans_cluster_sum_kernel<D, BF16><<<static_cast<unsigned>((gk * 32 + 255) / 256), 256, 0, stream>>>(
      x, w.members, w.offsets, counts, sums, gk, num_tokens, num_centroids);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

template <int D>
int km_launch_assign(const void* data, const void* centroids, int32_t dtype, int32_t groups, int32_t num_tokens,
                            int32_t num_centroids, int32_t* idx, const KmWorkspace& w, cudaStream_t stream) {
  CUtensorMap td, tc;
  int rc;
  const int64_t sd = static_cast<int64_t>(num_tokens) * D, sc = static_cast<int64_t>(num_centroids) * D;
  if ((rc = make_tmap_bhnd(&td, data, dtype, sd * groups, sd, D, 1, groups, num_tokens, D, 128, "kmeans data"))) return rc;
  if ((rc = make_tmap_bhnd(&tc, centroids, dtype, sc * groups, sc, D, 1, groups, num_centroids, D, kKtCent, "kmeans centroids"))) return rc;
  KmeansTcParams p;
  p.data = static_cast<const uint8_t*>(data); p.idx = idx; p.flagged = w.flagged; p.flagged_count = w.flagged_count;
  p.flagged_cap = w.flagged_cap; p.max_cnorm2 = w.max_cnorm2; p.num_tokens = num_tokens; p.num_centroids = num_centroids;
  p.bf16 = dtype == SQATTN_BF16;
  using L = KmeansTcSmem<D>;
  SQ_CUDA(cudaFuncSetAttribute(kmeans_assign_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  const dim3 grid((num_tokens + kKtTokens - 1) / kKtTokens, groups);
  kmeans_assign_tc_kernel<D><<<grid, 320, L::kTotal, stream>>>(td, tc, p);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

}  // namespace

extern "C" {

size_t sqattn_prefill_workspace_bytes(const sqattn_prefill_args* args) {
  PrefillPlan pl;
  if (plan_prefill(args, &pl)) return 0;
  return pl.total;
}

int sqattn_prefill(const sqattn_prefill_args* args, sqattn_stream_t stream) {
  return prefill_impl(args, reinterpret_cast<cudaStream_t>(stream), nullptr);
}

#ifdef SQATTN_DEBUG_EXPORTS
// Debug builds only: the step list of one CTA, computed on the host (out: up to 12 x {start, ntiles, flags}).
int sqattn_debug_schedule(int mode, int n, int sink, int w8, int w4, int p_fp8_mode, int same_opset, int blk, int* out) {
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.mode = mode; p.n = n; p.kv_len = n; p.sink = sink; p.p_fp8_mode = p_fp8_mode; p.same_opset = same_opset;
  p.w8[0] = w8; p.w4[0] = w4;
  Seg segs[kMaxSegs];
  const int ns = build_schedule(segs, p, blk, 0);
  for (int i = 0; i < ns; ++i) { out[3 * i] = segs[i].start; out[3 * i + 1] = segs[i].ntiles; out[3 * i + 2] = segs[i].flags; }
  return ns;
}
// Debug builds only: where CTA 0 of the cross-GPU merge kernel writes its time stamps ([64][8] int64; null = off)
int sqattn_debug_set_peer_stamps(long long* stamps) {
  SQ_CUDA(cudaMemcpyToSymbol(g_peer_stamps, &stamps, sizeof(stamps)));
  return SQATTN_OK;
}
// Debug builds only: same as sqattn_prefill, and CTA 0 additionally writes every S tile it sees
// ([steps][128 rows][64 keys] fp32) to `dump`.
int sqattn_debug_prefill_dump(const sqattn_prefill_args* args, float* dump, sqattn_stream_t stream) {
  return prefill_impl(args, reinterpret_cast<cudaStream_t>(stream), dump);
}
// ... and the P tiles it hands to the tensor core, same shape
int sqattn_debug_prefill_dump_sp(const sqattn_prefill_args* args, float* dump_s, float* dump_p, sqattn_stream_t stream) {
  return prefill_impl(args, reinterpret_cast<cudaStream_t>(stream), dump_s, nullptr, dump_p);
}
// ... and clock64 stamps of CTA 0's warps, [steps][16] (see SQ_STAMP in prefill.cuh)
int sqattn_debug_prefill_timeline(const sqattn_prefill_args* args, float* dump, long long* stamps, sqattn_stream_t stream) {
  return prefill_impl(args, reinterpret_cast<cudaStream_t>(stream), dump, stamps);
}
#endif

size_t sqattn_prep_workspace_bytes(const sqattn_prep_args* a) {
  if (!a) return 0;
  return static_cast<size_t>(a->batch) * a->num_kv_heads * (kMeanChunks + 1) * a->head_dim * sizeof(float);
}

int sqattn_prep_qkv(const sqattn_prep_args* a, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!a) return fail(SQATTN_ERR_INVALID_ARG, "args is null");
  if (a->head_dim != 64 && a->head_dim != 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128", a->head_dim);
  if (a->qk_qtype < 0 || a->qk_qtype > 2) return fail(SQATTN_ERR_INVALID_ARG, "Invalid quantization type: %d", a->qk_qtype);
  if (a->v_qtype < 0 || a->v_qtype > 2) return fail(SQATTN_ERR_INVALID_ARG, "Invalid quantization type: %d", a->v_qtype);
  const int parts = a->parts ? a->parts : 7;
  const bool do_q = parts & 1, do_k = parts & 2, do_v = parts & 4;
  if ((do_q && (!a->q.ptr || !a->q_bit8)) || (do_k && (!a->k.ptr || !a->k_bit8)) || (do_v && (!a->v.ptr || !a->v_bit8)))
    return fail(SQATTN_ERR_INVALID_ARG, "null tensor pointer");
  if (!a->skip_bit4 && ((do_q && !a->q_bit4) || (do_k && !a->k_bit4))) return fail(SQATTN_ERR_INVALID_ARG, "q_bit4/k_bit4 missing");
  if ((do_q && !aligned16(a->q)) || (do_k && !aligned16(a->k)) || (do_v && !aligned16(a->v)))
    return fail(SQATTN_ERR_INVALID_ARG, "inputs need 16-byte alignment");
  if (a->batch <= 0 || a->seq_len <= 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  const size_t need = sqattn_prep_workspace_bytes(a);
  if (!a->workspace || a->workspace_bytes < need) return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes required", need);
  const int B = a->batch, N = a->seq_len, D = a->head_dim, Hq = a->num_q_heads, Hkv = a->num_kv_heads;
  const bool bf16 = a->dtype == SQATTN_BF16;
  float* partial = static_cast<float*>(a->workspace);
  float* mean_ws = partial + static_cast<size_t>(B) * Hkv * kMeanChunks * D;
  View4 kq = view_of(a->q, B, Hq, N, D), kk = view_of(a->k, B, Hkv, N, D), kv = view_of(a->v, B, Hkv, N, D);
  const float* mean = a->k_mean;
  if (!mean && do_k) {
    const int lanes = 256 / (D / 8);
    dim3 mg(kMeanChunks, B * Hkv);
    if (bf16) kmean_partial_kernel<true><<<mg, 256, lanes * D * sizeof(float), stream>>>(kk, partial);
    else kmean_partial_kernel<false><<<mg, 256, lanes * D * sizeof(float), stream>>>(kk, partial);
    kmean_final_kernel<<<B * Hkv, 128, 0, stream>>>(partial, mean_ws, D, N);
    mean = mean_ws;
  }
  const float qs = static_cast<float>(sm_scale_log2(D));
  uint8_t* q4 = a->skip_bit4 ? nullptr : static_cast<uint8_t*>(a->q_bit4);
  uint8_t* k4 = a->skip_bit4 ? nullptr : static_cast<uint8_t*>(a->k_bit4);
  const OutStrides qo{static_cast<long long>(Hq) * N * D, static_cast<long long>(N) * D, D};
  const OutStrides ko = a->kv_out_nhd ? OutStrides{static_cast<long long>(N) * Hkv * D, D, static_cast<long long>(Hkv) * D}
                                      : OutStrides{static_cast<long long>(Hkv) * N * D, static_cast<long long>(N) * D, D};
  const int rows_per_block = 256 / (D / 8);
  const int gx = elementwise_grid((N + 4 * rows_per_block - 1) / (4 * rows_per_block), 1);
  const dim3 gq(gx, B * Hq), gk(gx, B * Hkv);
  const int gv = elementwise_grid(static_cast<long long>(N) * (D / 8), 256);
  if (bf16) {
    if (do_q) quant_rows_kernel<true, false><<<gq, 256, 0, stream>>>(kq, nullptr, static_cast<uint8_t*>(a->q_bit8), q4, qo, a->qk_qtype, a->round_half_even, qs);
    if (do_k) quant_rows_kernel<true, true><<<gk, 256, 0, stream>>>(kk, mean, static_cast<uint8_t*>(a->k_bit8), k4, ko, a->qk_qtype, a->round_half_even, 1.0f);
    if (do_v) quant_v_kernel<true><<<gv, 256, 0, stream>>>(kv, static_cast<uint8_t*>(a->v_bit8), ko, a->v_qtype, a->round_half_even);
  } else {
    if (do_q) quant_rows_kernel<false, false><<<gq, 256, 0, stream>>>(kq, nullptr, static_cast<uint8_t*>(a->q_bit8), q4, qo, a->qk_qtype, a->round_half_even, qs);
    if (do_k) quant_rows_kernel<false, true><<<gk, 256, 0, stream>>>(kk, mean, static_cast<uint8_t*>(a->k_bit8), k4, ko, a->qk_qtype, a->round_half_even, 1.0f);
    if (do_v) quant_v_kernel<false><<<gv, 256, 0, stream>>>(kv, static_cast<uint8_t*>(a->v_bit8), ko, a->v_qtype, a->round_half_even);
  }
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_k_column_sums(const sqattn_tensor* k, int32_t batch, int32_t num_kv_heads, int32_t seq_len, int32_t head_dim,
                         int32_t dtype, float* sums, void* workspace, size_t workspace_bytes, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!k || !k->ptr || !sums) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (head_dim != 64 && head_dim != 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128", head_dim);
  if (batch <= 0 || num_kv_heads <= 0 || seq_len <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  if (!aligned16(*k)) return fail(SQATTN_ERR_INVALID_ARG, "k needs 16-byte alignment");
  const size_t need = static_cast<size_t>(batch) * num_kv_heads * kMeanChunks * head_dim * sizeof(float);
  if (!workspace || workspace_bytes < need) return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes required", need);
  View4 kk = view_of(*k, batch, num_kv_heads, seq_len, head_dim);
  const int lanes = 256 / (head_dim / 8);
  dim3 mg(kMeanChunks, batch * num_kv_heads);
  float* partial = static_cast<float*>(workspace);
  if (dtype == SQATTN_BF16) kmean_partial_kernel<true><<<mg, 256, lanes * head_dim * sizeof(float), stream>>>(kk, partial);
  else kmean_partial_kernel<false><<<mg, 256, lanes * head_dim * sizeof(float), stream>>>(kk, partial);
  kmean_final_kernel<<<batch * num_kv_heads, 128, 0, stream>>>(partial, sums, head_dim, 0);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

size_t sqattn_decode_workspace_bytes(const sqattn_decode_args* args) {
  DecodePlan pl;
  if (plan_decode(args, &pl)) return 0;
  return decode_ws_bytes(args, pl);
}

int sqattn_decode(const sqattn_decode_args* a, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  DecodePlan pl;
  int rc = plan_decode(a, &pl);
  if (rc) return rc;
  if (!a->q.ptr || (!a->gather && (!a->k.ptr || !a->v.ptr))) return fail(SQATTN_ERR_INVALID_ARG, "null tensor pointer");
  if (!a->partial_o && !a->o.ptr && !a->peer) return fail(SQATTN_ERR_INVALID_ARG, "null output pointer");
  if (a->partial_o && !a->partial_lse) return fail(SQATTN_ERR_INVALID_ARG, "partial_lse missing");
  if (!a->gather && (!aligned16(a->k) || !aligned16(a->v))) return fail(SQATTN_ERR_INVALID_ARG, "k/v need 16-byte alignment");
  if ((reinterpret_cast<uintptr_t>(a->q.ptr) % 4) || (a->q.stride_h % 2) || (a->q.stride_b % 2)) return fail(SQATTN_ERR_INVALID_ARG, "q needs 4-byte alignment");
  const size_t need = decode_ws_bytes(a, pl);
  if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) % 256))
    return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required", need);
  const bool bf16 = a->dtype == SQATTN_BF16;
  if (a->head_dim == 128) return bf16 ? launch_decode<128, true>(a, pl, stream) : launch_decode<128, false>(a, pl, stream);
  return bf16 ? launch_decode<64, true>(a, pl, stream) : launch_decode<64, false>(a, pl, stream);
}

int sqattn_decode_merge(const float* partial_o, const float* partial_lse, int32_t num_parts, int64_t rows,
                        int32_t head_dim, void* o, int32_t o_dtype, float* lse, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!partial_o || !partial_lse || !o) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (num_parts <= 0 || rows <= 0 || head_dim <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  MergeParams m;
  memset(&m, 0, sizeof(m));
  m.part_o = partial_o; m.part_lse = partial_lse; m.o = o; m.lse = lse;
  m.hq = 1; m.d = head_dim; m.o_dtype = o_dtype; m.contiguous = 1; m.num_parts = num_parts; m.rows = rows;
  if (head_dim > 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: at most 128", head_dim);
  decode_merge_kernel<<<static_cast<unsigned>(rows), 128 * kMergeGroups, 0, stream>>>(m);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

// ---- decode for callers that cannot hand over scratch memory ---------------------------------------------
// Scratch for the split-KV partials lives in this file-scope device array instead of a caller workspace.
// Every GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = (4u << 20) + (64u << 10);  // 4 MiB of partial O + 64 KiB of partial LSE
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle; its device address has to be asked for, once per device and
// with that device current.
static int static_scratch_address(void** out) {
  static void* table[64] = {nullptr};
  int dev = 0;
  SQ_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SQATTN_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  if (!table[dev]) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(SQATTN_ERR_CUDA, "cudaGetSymbolAddress(g_decode_static_scratch): %s", cudaGetErrorString(e));
    table[dev] = ptr;
  }
  *out = table[dev];
  return SQATTN_OK;
}

int sqattn_decode_static_scratch(const sqattn_decode_args* args, sqattn_stream_t stream) {
  DecodePlan pl;
  int rc = plan_decode(args, &pl);
  if (rc) return rc;
  const size_t need = decode_ws_bytes(args, pl);
  if (need > kStaticScratchBytes)
    return fail(SQATTN_ERR_WORKSPACE,
                "this call needs %zu bytes of scratch (%d key ranges x %d query heads) but the built-in scratch holds "
                "%zu: fewer sequences or splits, or sqattn_decode with a caller workspace",
                need, pl.total_items, args->num_q_heads, kStaticScratchBytes);
  void* ptr = nullptr;
  if ((rc = static_scratch_address(&ptr))) return rc;
  sqattn_decode_args a = *args;
  a.workspace = ptr;
  a.workspace_bytes = kStaticScratchBytes;
  return sqattn_decode(&a, stream);
}

// ---- kmeans ------------------------------------------------------------------------------------------
#define SQ_KM_DISPATCH(KERNEL, ...)                                         \
  do {                                                                      \
    if (head_dim == 128) {                                                  \
      if (bf16) KERNEL<128, true> __VA_ARGS__; else KERNEL<128, false> __VA_ARGS__; \
    } else {                                                                \
      if (bf16) KERNEL<64, true> __VA_ARGS__; else KERNEL<64, false> __VA_ARGS__;   \
    }                                                                       \
  } while (0)

static int km_check(int32_t groups, int32_t num_tokens, int32_t num_centroids, int32_t head_dim) {
  if (head_dim != 64 && head_dim != 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: only 64 and 128", head_dim);
  if (groups <= 0 || num_tokens <= 0 || num_centroids <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  if (num_centroids % 32) return fail(SQATTN_ERR_INVALID_ARG, "num_centroids must be a multiple of 32");
  if (num_centroids > 49152) return fail(SQATTN_ERR_UNSUPPORTED, "at most 49152 centroids per group (their scores are staged in shared memory)");
  return SQATTN_OK;
}

size_t sqattn_kmeans_workspace_bytes(int32_t groups, int32_t num_tokens, int32_t num_centroids) {
  if (groups <= 0 || num_tokens <= 0 || num_centroids <= 0) return 0;
  return km_workspace(nullptr, groups, num_tokens, num_centroids).total;
}

int sqattn_kmeans_assign(const void* data, const void* centroids, int32_t dtype, int32_t groups, int32_t num_tokens,
                         int32_t num_centroids, int32_t head_dim, int32_t* idx, double* sums, int32_t* counts,
                         void* workspace, size_t workspace_bytes, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc = km_check(groups, num_tokens, num_centroids, head_dim);
  if (rc) return rc;
  if (!data || !centroids || !idx) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (sums && !counts) return fail(SQATTN_ERR_INVALID_ARG, "counts is needed with sums");
  if (static_cast<long long>(groups) * num_tokens > 0x7fffffffll) return fail(SQATTN_ERR_UNSUPPORTED, "more than 2^31 tokens in all groups");
  if ((reinterpret_cast<uintptr_t>(data) | reinterpret_cast<uintptr_t>(centroids)) & 15)
    return fail(SQATTN_ERR_INVALID_ARG, "data and centroids need 16-byte alignment");
  const size_t need = sqattn_kmeans_workspace_bytes(groups, num_tokens, num_centroids);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required", need);
  const KmWorkspace w = km_workspace(workspace, groups, num_tokens, num_centroids);
  const bool bf16 = dtype == SQATTN_BF16;
  const uint8_t* d8 = static_cast<const uint8_t*>(data);
  const uint8_t* c8 = static_cast<const uint8_t*>(centroids);
  SQ_CUDA(cudaMemsetAsync(w.flagged_count, 0, sizeof(int), stream));
  SQ_KM_DISPATCH(kmeans_cnorm_max_kernel, <<<groups, 256, 0, stream>>>(c8, num_centroids, w.max_cnorm2));
  if ((rc = head_dim == 128 ? km_launch_assign<128>(data, centroids, dtype, groups, num_tokens, num_centroids, idx, w, stream)
                            : km_launch_assign<64>(data, centroids, dtype, groups, num_tokens, num_centroids, idx, w, stream)))
    return rc;
  {
    const int smem = num_centroids * static_cast<int>(sizeof(float));   // the fp32 scores of one group
    if (head_dim == 128) {
      if (bf16) SQ_CUDA(cudaFuncSetAttribute(kmeans_recheck_list_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      else SQ_CUDA(cudaFuncSetAttribute(kmeans_recheck_list_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    } else {
      if (bf16) SQ_CUDA(cudaFuncSetAttribute(kmeans_recheck_list_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      else SQ_CUDA(cudaFuncSetAttribute(kmeans_recheck_list_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    SQ_KM_DISPATCH(kmeans_recheck_list_kernel, <<<148 * 4, 256, smem, stream>>>(d8, c8, idx, w.flagged, w.flagged_count, w.flagged_cap,
                                                                             w.max_cnorm2, groups, num_tokens, num_centroids));
  }
  SQ_CUDA(cudaGetLastError());
  if (sums) {
    if (head_dim == 128) rc = bf16 ? km_member_sums<128, true>(d8, idx, groups, num_tokens, num_centroids, w, counts, sums, stream)
                                   : km_member_sums<128, false>(d8, idx, groups, num_tokens, num_centroids, w, counts, sums, stream);
    else rc = bf16 ? km_member_sums<64, true>(d8, idx, groups, num_tokens, num_centroids, w, counts, sums, stream)
                   : km_member_sums<64, false>(d8, idx, groups, num_tokens, num_centroids, w, counts, sums, stream);
    if (rc) return rc;
  }
  return SQATTN_OK;
}

int sqattn_kmeans_update(void* centroids, int32_t dtype, const double* sums, const int32_t* counts, int32_t groups,
                         int32_t num_centroids, int32_t head_dim, int32_t normalize, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc = km_check(groups, 1, num_centroids, head_dim);
  if (rc) return rc;
  if (!centroids || !sums || !counts) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  const bool bf16 = dtype == SQATTN_BF16;
  const long long total = static_cast<long long>(groups) * num_centroids;
  const unsigned grid = static_cast<unsigned>((total * 32 + 255) / 256);
  uint8_t* c8 = static_cast<uint8_t*>(centroids);
  SQ_KM_DISPATCH(kmeans_update_kernel, <<<grid, 256, 0, stream>>>(c8, sums, counts, total, normalize));
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_kmeans_reverse_index(const int32_t* idx, int32_t groups, int32_t num_tokens, int32_t num_centroids,
                                int32_t max_cluster_size, int32_t* clusters, int32_t* cluster_size, void* workspace,
                                size_t workspace_bytes, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!idx || !clusters || !cluster_size) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (groups <= 0 || num_tokens <= 0 || num_centroids <= 0 || max_cluster_size <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  const size_t need = sqattn_kmeans_workspace_bytes(groups, num_tokens, num_centroids);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required", need);
  const KmWorkspace w = km_workspace(workspace, groups, num_tokens, num_centroids);
  const long long gt = static_cast<long long>(groups) * num_tokens, gk = static_cast<long long>(groups) * num_centroids;
  SQ_CUDA(cudaMemsetAsync(w.counts, 0, static_cast<size_t>(gk) * sizeof(int), stream));
  kmeans_count_kernel<<<elementwise_grid(gt, 256), 256, 0, stream>>>(idx, w.counts, w.slot, gt, num_tokens, num_centroids);
  kmeans_offsets_kernel<<<groups, 1024, 0, stream>>>(w.counts, w.offsets, num_centroids);
  kmeans_scatter_kernel<<<elementwise_grid(gt, 256), 256, 0, stream>>>(idx, w.slot, w.offsets, w.members, gt, num_tokens, num_centroids);
  kmeans_sort_members_kernel<<<static_cast<unsigned>((gk * 32 + 255) / 256), 256, 0, stream>>>(
      w.members, w.offsets, w.counts, clusters, cluster_size, gk, num_tokens, num_centroids, max_cluster_size);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_kmeans_index_add(const void* value, int32_t dtype, const int32_t* idx, int32_t groups, int32_t num_tokens,
                            int32_t num_centroids, int32_t head_dim, double* sums_ws, void* out, void* workspace,
                            size_t workspace_bytes, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc = km_check(groups, num_tokens, num_centroids, head_dim);
  if (rc) return rc;
  if (!value || !idx || !sums_ws || !out) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  const size_t need = sqattn_kmeans_workspace_bytes(groups, num_tokens, num_centroids);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(SQATTN_ERR_WORKSPACE, "workspace of %zu bytes (256-byte aligned) required", need);
  const KmWorkspace w = km_workspace(workspace, groups, num_tokens, num_centroids);
  const bool bf16 = dtype == SQATTN_BF16;
  const uint8_t* v8 = static_cast<const uint8_t*>(value);
  SQ_CUDA(cudaMemsetAsync(w.counts, 0, static_cast<size_t>(groups) * num_centroids * sizeof(int), stream));
  if (head_dim == 128) rc = bf16 ? km_member_sums<128, true>(v8, idx, groups, num_tokens, num_centroids, w, w.counts, sums_ws, stream)
                                 : km_member_sums<128, false>(v8, idx, groups, num_tokens, num_centroids, w, w.counts, sums_ws, stream);
  else rc = bf16 ? km_member_sums<64, true>(v8, idx, groups, num_tokens, num_centroids, w, w.counts, sums_ws, stream)
                 : km_member_sums<64, false>(v8, idx, groups, num_tokens, num_centroids, w, w.counts, sums_ws, stream);
  if (rc) return rc;
  const long long n = static_cast<long long>(groups) * num_centroids * head_dim;
  if (bf16) kmeans_store_sums_kernel<true><<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(sums_ws, static_cast<uint8_t*>(out), n);
  else kmeans_store_sums_kernel<false><<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(sums_ws, static_cast<uint8_t*>(out), n);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_kmeans_max_count(const int32_t* counts, int64_t n, int32_t* out_max, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!counts || !out_max || n <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad arguments");
  max_int_kernel<<<elementwise_grid(n, 256), 256, 0, stream>>>(counts, n, out_max);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

// ---- retrieval -----------------------------------------------------------------------------------------
int sqattn_retrieve_select(const void* q, const void* centroids, int32_t dtype, const int32_t* cluster_size,
                           const int32_t* clusters, int32_t groups_kv, int32_t heads_per_group, int32_t num_clusters,
                           int32_t head_dim, int32_t max_cluster_size, int32_t num_tokens, int32_t budget,
                           int32_t* out_idx, int32_t* out_count, int32_t cap, int32_t tail_start, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!q || !centroids || !cluster_size || !clusters || !out_idx || !out_count) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (head_dim != 64 && head_dim != 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: 64 or 128", head_dim);
  if (num_clusters <= 0 || num_clusters > kRetMaxClusters) return fail(SQATTN_ERR_UNSUPPORTED, "1..%d clusters supported", kRetMaxClusters);
  if (num_tokens <= 0 || num_tokens > kRetMaxTokens) return fail(SQATTN_ERR_UNSUPPORTED, "1..%d tokens supported", kRetMaxTokens);
  if (groups_kv <= 0 || heads_per_group <= 0 || budget <= 0 || cap <= 0 || max_cluster_size <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  RetrieveParams p;
  p.q = static_cast<const uint8_t*>(q); p.cent = static_cast<const uint8_t*>(centroids);
  p.cluster_size = cluster_size; p.clusters = clusters; p.out_idx = out_idx; p.out_count = out_count;
  p.groups = heads_per_group; p.num_clusters = num_clusters; p.d = head_dim; p.max_cluster_size = max_cluster_size;
  p.num_tokens = num_tokens; p.budget = budget; p.cap = cap;
  if (tail_start < 0 || tail_start > num_tokens) return fail(SQATTN_ERR_INVALID_ARG, "tail_start %d outside [0, %d]", tail_start, num_tokens);
  p.tail_start = tail_start;
  const size_t smem = sizeof(double) * num_clusters + sizeof(uint32_t) * ((num_tokens + 31) / 32);
  if (dtype == SQATTN_BF16) {
    SQ_CUDA(cudaFuncSetAttribute(retrieve_select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    retrieve_select_kernel<true><<<groups_kv, 1024, smem, stream>>>(p);
  } else {
    SQ_CUDA(cudaFuncSetAttribute(retrieve_select_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    retrieve_select_kernel<false><<<groups_kv, 1024, smem, stream>>>(p);
  }
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_gather_rows(const void* src, int64_t src_group_stride, int64_t src_row_stride, const int32_t* idx,
                       const int32_t* count, int32_t groups, int32_t cap, int32_t head_dim, void* dst,
                       sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!src || !idx || !count || !dst) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (groups <= 0 || cap <= 0 || head_dim <= 0 || head_dim % 8 || src_row_stride % 8 || src_group_stride % 8)
    return fail(SQATTN_ERR_INVALID_ARG, "bad sizes or strides (multiples of 8 elements)");
  dim3 grid(elementwise_grid(static_cast<long long>(cap) * (head_dim / 8), 256) , groups);
  gather_rows_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(src), src_group_stride, src_row_stride, idx, count, cap,
                                               head_dim, static_cast<uint8_t*>(dst));
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_retrieve_batch(const sqattn_retrieve_item* items, int32_t num_items, int32_t dtype, int32_t groups_kv,
                          int32_t heads_per_group, int32_t head_dim, int32_t budget, int32_t cap, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!items || num_items <= 0) return fail(SQATTN_ERR_INVALID_ARG, "no items");
  if (head_dim != 64 && head_dim != 128) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d: 64 or 128", head_dim);
  if (groups_kv <= 0 || heads_per_group <= 0 || budget <= 0 || cap <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  // select only (the caller attends the listed rows in place): no item has a destination
  bool pack = false;
  for (int i = 0; i < num_items; ++i) pack = pack || items[i].k_dst || items[i].v_dst;
  for (int first = 0; first < num_items; first += kRetMaxBatch) {
    const int n = num_items - first < kRetMaxBatch ? num_items - first : kRetMaxBatch;
    RetrieveBatch rb;
    GatherBatch gb;
    memset(&rb, 0, sizeof(rb));
    memset(&gb, 0, sizeof(gb));
    size_t smem = 0;
    for (int i = 0; i < n; ++i) {
      const sqattn_retrieve_item& it = items[first + i];
      if (!it.q || !it.centroids || !it.cluster_size || !it.clusters || !it.out_idx || !it.out_count ||
          (pack && (!it.k_src || !it.v_src || !it.k_dst || !it.v_dst)))
        return fail(SQATTN_ERR_INVALID_ARG, "retrieve item %d: null pointer", first + i);
      if (it.num_clusters <= 0 || it.num_clusters > kRetMaxClusters) return fail(SQATTN_ERR_UNSUPPORTED, "1..%d clusters supported", kRetMaxClusters);
      if (it.num_tokens <= 0 || it.num_tokens > kRetMaxTokens) return fail(SQATTN_ERR_UNSUPPORTED, "1..%d tokens supported", kRetMaxTokens);
      if (it.max_cluster_size <= 0 || it.src_row_stride % 8 || it.src_group_stride % 8) return fail(SQATTN_ERR_INVALID_ARG, "retrieve item %d: bad sizes or strides", first + i);
      RetrieveParams& p = rb.item[i];
      p.q = static_cast<const uint8_t*>(it.q); p.cent = static_cast<const uint8_t*>(it.centroids);
      p.cluster_size = it.cluster_size; p.clusters = it.clusters; p.out_idx = it.out_idx; p.out_count = it.out_count;
      p.groups = heads_per_group; p.num_clusters = it.num_clusters; p.d = head_dim; p.max_cluster_size = it.max_cluster_size;
      p.num_tokens = it.num_tokens; p.budget = budget; p.cap = cap;
      if (it.tail_start < 0 || it.tail_start > it.num_tokens || it.split_row < 0)
        return fail(SQATTN_ERR_INVALID_ARG, "retrieve item %d: tail_start %d / split_row %d out of range", first + i, it.tail_start, it.split_row);
      p.tail_start = it.tail_start;
      const size_t need = sizeof(double) * it.num_clusters + sizeof(uint32_t) * ((it.num_tokens + 31) / 32);
      smem = need > smem ? need : smem;
      gb.item[2 * i] = GatherItem{static_cast<const uint8_t*>(it.k_src), static_cast<uint8_t*>(it.k_dst), it.out_idx, it.out_count,
                                  it.src_group_stride, it.src_row_stride, static_cast<const uint8_t*>(it.k_src2),
                                  it.src2_group_stride, it.split_row};
      gb.item[2 * i + 1] = GatherItem{static_cast<const uint8_t*>(it.v_src), static_cast<uint8_t*>(it.v_dst), it.out_idx, it.out_count,
                                      it.src_group_stride, it.src_row_stride, static_cast<const uint8_t*>(it.v_src2),
                                      it.src2_group_stride, it.split_row};
    }
    const dim3 sgrid(groups_kv, n);
    if (dtype == SQATTN_BF16) {
      SQ_CUDA(cudaFuncSetAttribute(retrieve_select_batch_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      retrieve_select_batch_kernel<true><<<sgrid, 1024, smem, stream>>>(rb);
    } else {
      SQ_CUDA(cudaFuncSetAttribute(retrieve_select_batch_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      retrieve_select_batch_kernel<false><<<sgrid, 1024, smem, stream>>>(rb);
    }
    SQ_CUDA(cudaGetLastError());
    if (!pack) continue;
    const dim3 ggrid(elementwise_grid(static_cast<long long>(cap) * (head_dim / 8), 256), groups_kv, 2 * n);
    gather_rows_batch_kernel<<<ggrid, 256, 0, stream>>>(gb, cap, head_dim);
    SQ_CUDA(cudaGetLastError());
  }
  return SQATTN_OK;
}

// ---- window calibration ----------------------------------------------------------------------------------
int sqattn_window_histogram(const void* q, const void* k, int32_t dtype, int32_t num_q_heads, int32_t num_kv_heads,
                            int32_t seq_len, int32_t head_dim, int32_t relative, int32_t num_bins, int32_t sink,
                            double* hist, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!q || !k || !hist) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (head_dim % 8 || head_dim <= 0 || head_dim > 256) return fail(SQATTN_ERR_UNSUPPORTED, "head_dim %d", head_dim);
  if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || seq_len <= 0 || num_bins <= 0 || sink < 0)
    return fail(SQATTN_ERR_INVALID_ARG, "bad sizes");
  WindowHistParams p;
  p.q = static_cast<const uint8_t*>(q); p.k = static_cast<const uint8_t*>(k); p.hist = hist;
  p.hq = num_q_heads; p.groups = num_q_heads / num_kv_heads; p.n = seq_len; p.d = head_dim; p.nbins = num_bins;
  p.sink = sink; p.relative = relative; p.scale = static_cast<float>(1.0 / sqrt(static_cast<double>(head_dim)));
  const bool bf16 = dtype == SQATTN_BF16;
  if (head_dim == 64 || head_dim == 128) {
    // tensor-core kernel: Q tile + two K tiles (rows padded by 8 elements) + the block histogram
    const size_t smem = static_cast<size_t>(3) * 64 * (head_dim + 8) * 2 + static_cast<size_t>(num_bins) * sizeof(float);
    if (smem > 220 * 1024) return fail(SQATTN_ERR_UNSUPPORTED, "too many bins (%d)", num_bins);
    const dim3 grid((seq_len + kWhRows - 1) / kWhRows, num_q_heads);
#define SQ_WH(BF, DD)                                                                                                      \
    do {                                                                                                                   \
      SQ_CUDA(cudaFuncSetAttribute(window_hist_mma_kernel<BF, DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
      window_hist_mma_kernel<BF, DD><<<grid, 128, smem, stream>>>(p);                                                      \
    } while (0)
    if (head_dim == 128) { if (bf16) SQ_WH(true, 128); else SQ_WH(false, 128); }
    else { if (bf16) SQ_WH(true, 64); else SQ_WH(false, 64); }
#undef SQ_WH
    SQ_CUDA(cudaGetLastError());
    return SQATTN_OK;
  }
  const size_t smem = (8 * static_cast<size_t>(head_dim) + num_bins) * sizeof(float);
  if (smem > 200 * 1024) return fail(SQATTN_ERR_UNSUPPORTED, "too many bins (%d)", num_bins);
  dim3 grid(elementwise_grid((seq_len + 7) / 8, 1), num_q_heads);
  if (bf16) {
    SQ_CUDA(cudaFuncSetAttribute(window_hist_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    window_hist_kernel<true><<<grid, 256, smem, stream>>>(p);
  } else {
    SQ_CUDA(cudaFuncSetAttribute(window_hist_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    window_hist_kernel<false><<<grid, 256, smem, stream>>>(p);
  }
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

// ---- decoder-layer row kernels ---------------------------------------------------------------------------
int sqattn_rmsnorm(const void* x, const void* weight, void* out, int64_t rows, int32_t dim, int64_t x_row_stride,
                   int64_t out_row_stride, float eps, int32_t dtype, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!x || !weight || !out) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (rows <= 0 || rows > 2147483647ll || dim <= 0 || dim % 8 || x_row_stride % 8 || out_row_stride % 8 ||
      x_row_stride < dim || out_row_stride < dim)
    return fail(SQATTN_ERR_INVALID_ARG, "rmsnorm: rows %lld dim %d strides %lld %lld (dim and strides must be multiples of 8)",
                static_cast<long long>(rows), dim, static_cast<long long>(x_row_stride), static_cast<long long>(out_row_stride));
  if (dtype == SQATTN_BF16)
    rmsnorm_kernel<true><<<static_cast<unsigned>(rows), 256, 0, stream>>>(
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), static_cast<uint8_t*>(out), dim, x_row_stride, out_row_stride, eps);
  else
    rmsnorm_kernel<false><<<static_cast<unsigned>(rows), 256, 0, stream>>>(
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(weight), static_cast<uint8_t*>(out), dim, x_row_stride, out_row_stride, eps);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_rope_qk_devpos(void* qkv, int64_t row_stride, int64_t rows, int32_t seq_len, int32_t num_heads,
                          int32_t head_dim, const float* cos_sin_cache, int64_t cache_rows, int64_t pos0,
                          const int64_t* pos_device, int32_t dtype, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!qkv || !cos_sin_cache) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (head_dim <= 0 || head_dim % 16) return fail(SQATTN_ERR_UNSUPPORTED, "rope: head_dim %d must be a multiple of 16", head_dim);
  if (rows <= 0 || seq_len <= 0 || num_heads <= 0 || row_stride % 8 || row_stride < static_cast<int64_t>(num_heads) * head_dim)
    return fail(SQATTN_ERR_INVALID_ARG, "rope: bad sizes");
  if (pos0 < 0 || (!pos_device && pos0 + seq_len > cache_rows))
    return fail(SQATTN_ERR_INVALID_ARG, "rope: positions %lld..%lld exceed the cos/sin cache (%lld rows)",
                static_cast<long long>(pos0), static_cast<long long>(pos0 + seq_len), static_cast<long long>(cache_rows));
  const int grid = elementwise_grid(rows * num_heads * (head_dim / 16), 256);
  const long long* pd = reinterpret_cast<const long long*>(pos_device);
  if (dtype == SQATTN_BF16)
    rope_kernel<true><<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(qkv), row_stride, rows, seq_len, num_heads, head_dim, cos_sin_cache, pos0, pd, cache_rows);
  else
    rope_kernel<false><<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(qkv), row_stride, rows, seq_len, num_heads, head_dim, cos_sin_cache, pos0, pd, cache_rows);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

int sqattn_rope_qk(void* qkv, int64_t row_stride, int64_t rows, int32_t seq_len, int32_t num_heads, int32_t head_dim,
                   const float* cos_sin_cache, int64_t cache_rows, int64_t pos0, int32_t dtype, sqattn_stream_t stream_) {
  return sqattn_rope_qk_devpos(qkv, row_stride, rows, seq_len, num_heads, head_dim, cos_sin_cache, cache_rows, pos0,
                               nullptr, dtype, stream_);
}

int sqattn_silu_mul(const void* x, void* out, int64_t rows, int32_t inter, int32_t dtype, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!x || !out) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (rows <= 0 || inter <= 0 || inter % 8) return fail(SQATTN_ERR_INVALID_ARG, "silu_mul: rows %lld inter %d", static_cast<long long>(rows), inter);
  const int grid = elementwise_grid(rows * (inter / 8), 256);
  if (dtype == SQATTN_BF16) silu_mul_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), rows, inter);
  else silu_mul_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), rows, inter);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

size_t sqattn_peer_merge_data_bytes(int32_t world, int32_t rows_cap, int32_t head_dim) {
  if (world <= 0 || world > kPeerMaxWorld || rows_cap <= 0 || head_dim <= 0) return 0;
  return static_cast<size_t>(2) * world * rows_cap * (head_dim + 1) * sizeof(unsigned long long);
}
size_t sqattn_peer_merge_flag_bytes(int32_t world, int32_t rows_cap) {
  if (world <= 0 || world > kPeerMaxWorld || rows_cap <= 0) return 0;
  return (static_cast<size_t>(world) * rows_cap + 4) * sizeof(uint32_t);
}

int sqattn_decode_peer_merge(const sqattn_peer_merge_args* a, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!a) return fail(SQATTN_ERR_INVALID_ARG, "args is null");
  if (!a->part_o || !a->part_lse) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  PeerMergeParams p;
  int rc = fill_peer_params(a, &p);
  if (rc) return rc;
  p.part_o = a->part_o; p.part_lse = a->part_lse; p.split_mode = 0; p.hq = 1;
  peer_merge_kernel<<<static_cast<unsigned>(p.rows), 128 * kMergeGroups, 0, stream>>>(p);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

// ---- cache ---------------------------------------------------------------------------------------------
int sqattn_cache_copy_rows(void* dst, int64_t dst_row_stride_bytes, const void* src, int64_t src_row_stride_bytes,
                           int64_t row_bytes, int64_t rows, int32_t to_device, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!dst || !src || row_bytes <= 0 || rows <= 0) return fail(SQATTN_ERR_INVALID_ARG, "bad arguments");
  if (dst_row_stride_bytes < row_bytes || src_row_stride_bytes < row_bytes) return fail(SQATTN_ERR_INVALID_ARG, "row stride smaller than row");
  SQ_CUDA(cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_row_stride_bytes), src, static_cast<size_t>(src_row_stride_bytes),
                            static_cast<size_t>(row_bytes), static_cast<size_t>(rows),
                            to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, stream));
  return SQATTN_OK;
}

int sqattn_cache_append(void* k_cache, void* v_cache, const void* k_new, const void* v_new, const int64_t* positions,
                        int64_t cache_seq_stride, int64_t cache_row_stride, int64_t new_seq_stride, int32_t batch,
                        int32_t row_elems, int64_t capacity, sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!k_cache || !v_cache || !k_new || !v_new || !positions) return fail(SQATTN_ERR_INVALID_ARG, "null pointer");
  if (batch <= 0 || row_elems <= 0 || row_elems % 8 || capacity <= 0)
    return fail(SQATTN_ERR_INVALID_ARG, "cache append: batch %d, row of %d elements (multiple of 8), capacity %lld", batch,
                row_elems, static_cast<long long>(capacity));
  if (cache_seq_stride % 8 || cache_row_stride % 8 || new_seq_stride % 8 || cache_row_stride < row_elems ||
      ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(k_new) |
        reinterpret_cast<uintptr_t>(v_new)) & 15))
    return fail(SQATTN_ERR_INVALID_ARG, "cache append: pointers need 16-byte alignment, strides multiples of 8 elements");
  const int grid = elementwise_grid(2ll * batch * (row_elems / 8), 256);
  cache_append_kernel<<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache),
                                                static_cast<const uint8_t*>(k_new), static_cast<const uint8_t*>(v_new),
                                                reinterpret_cast<const long long*>(positions), cache_seq_stride,
                                                cache_row_stride, new_seq_stride, batch, row_elems, capacity);
  SQ_CUDA(cudaGetLastError());
  return SQATTN_OK;
}

// ---- diagnostics -----------------------------------------------------------------------------------------
int sqattn_check_device_status(sqattn_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int code = 0;
  SQ_CUDA(cudaMemcpyFromSymbolAsync(&code, g_device_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream));
  SQ_CUDA(cudaStreamSynchronize(stream));
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbolAsync(g_device_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    return fail(SQATTN_ERR_DEVICE_TIMEOUT, "a device-side wait gave up (code %d: 1xx prefill, 2xx decode)", code);
  }
  return SQATTN_OK;
}

int sqattn_set_status_mirror(int32_t* host_word) {
  int* dev_view = nullptr;
  if (host_word) {
    cudaError_t e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev_view), host_word, 0);
    if (e != cudaSuccess || !dev_view)
      return fail(SQATTN_ERR_INVALID_ARG, "status mirror: the word must be pinned, device-mapped host memory (%s)",
                  cudaGetErrorString(e));
  }
  SQ_CUDA(cudaMemcpyToSymbol(g_status_mirror, &dev_view, sizeof(dev_view)));
  return SQATTN_OK;
}

const char* sqattn_last_error_string(void) { return err_buf(); }
int sqattn_version(void) { return 110; }

}  // extern "C"
