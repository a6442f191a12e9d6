// Centroid-scored retrieval for clustered decode (the step the reference's logs hint at but its code lacks):
// score every cluster by <mean query of the KV group, centroid>, take clusters in descending score until a
// token budget is covered, emit the selected token indices in ascending order, gather their K/V rows.
// Scores are fp64 (exact products of 16-bit centroids and an fp32 mean, index-order sum), the selection is a
// block-level argmax with lowest-index tie-break, so the selected indices are bit-exact and timing-independent.
#pragma once
#include "prep.cuh"

namespace sq {

constexpr int kRetMaxClusters = 4096;
constexpr int kRetMaxTokens = 262144;

struct RetrieveParams {
  const uint8_t* q;         // [G, groups, D] 16-bit
  const uint8_t* cent;      // [G, K, D] 16-bit
  const int* cluster_size;  // [G, K]
  const int* clusters;      // [G, K, max_cluster_size]
  int* out_idx;             // [G, cap]
  int* out_count;           // [G]
  int groups, num_clusters, d, max_cluster_size, num_tokens, budget, cap;
  int tail_start;           // tokens [tail_start, num_tokens) are not clustered yet (appended since the last fold) and
                            // are always selected; tail_start == num_tokens: none
};

template <bool BF16>
__device__ __forceinline__ void retrieve_select_body(const RetrieveParams& p, const int g) {
  extern __shared__ __align__(16) uint8_t rs[];
  double* scores = reinterpret_cast<double*>(rs);                                   // [K]
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(rs + sizeof(double) * p.num_clusters);  // [ceil(T/32)]
  __shared__ float q_mean[128];
  __shared__ double red_v[32];
  __shared__ int red_i[32];
  __shared__ int sel_list[kRetMaxClusters];
  __shared__ int n_sel, total_tok, win_s, warp_sums[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.num_clusters, D = p.d;
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p.q) + static_cast<long long>(g) * p.groups * D;
  const uint16_t* cent = reinterpret_cast<const uint16_t*>(p.cent) + static_cast<long long>(g) * K * D;
  const int* csize = p.cluster_size + static_cast<long long>(g) * K;
  const int* cl = p.clusters + static_cast<long long>(g) * K * p.max_cluster_size;
  const int words = (p.num_tokens + 31) / 32;

  if (tid < D) {  // mean query of the group: fp32, heads added in order
    float s = 0.f;
    for (int h = 0; h < p.groups; ++h) s += to_f32<BF16>(q[h * D + tid]);
    q_mean[tid] = s / static_cast<float>(p.groups);
  }
  for (int w = tid; w < words; w += blockDim.x) bitmap[w] = 0u;
  if (tid == 0) { n_sel = 0; total_tok = 0; }
  __syncthreads();
  // Scores: D/8 lanes per centroid row, 16-byte loads (a warp reads whole rows, coalesced), four rows per lane in
  // flight; each lane adds its eight products in index order, the lanes' sums are combined pairwise in a fixed
  // order, so a score does not depend on timing (and centroids with identical rows get identical scores).
  {
    const int lanes_per_row = D / 8, rows_per_warp = 32 / lanes_per_row;
    const int sub = lane % lanes_per_row, rslot = lane / lanes_per_row;
    constexpr int kInFlight = 4;
    double qd[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) qd[e] = static_cast<double>(q_mean[sub * 8 + e]);
    const int stride = (blockDim.x >> 5) * rows_per_warp;
    for (int c0 = warp * rows_per_warp; c0 < K; c0 += kInFlight * stride) {
      uint4 raw[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int c = c0 + u * stride + rslot;
        raw[u] = (c < K) ? *reinterpret_cast<const uint4*>(cent + static_cast<long long>(c) * D + sub * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int c = c0 + u * stride + rslot;
        float f[8];
        unpack8<BF16>(raw[u], f);
        double sc = 0.0;
#pragma unroll
        for (int e = 0; e < 8; ++e) sc += static_cast<double>(f[e]) * qd[e];
        for (int o = lanes_per_row >> 1; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        if (c < K && sub == 0) scores[c] = (csize[c] > 0) ? sc : -1.0 / 0.0;  // empty clusters are never taken
      }
    }
  }
  __syncthreads();
  // Greedy selection: the best remaining cluster until the budget is covered (ties: lowest index).  The first
  // kSelThreads threads do it (a barrier of 256 threads is cheaper than one of 1024, and there is one pair per
  // selected cluster).  The fp64 scores are first replaced, in place, by 64-bit integers of the same order (0 = taken
  // or empty, below every real score), so that an arg-max over a warp is three warp-wide integer reductions (high
  // word, low word among the lanes that hold the high word, lowest index among the lanes that hold both).  Thread t
  // owns the clusters t, t + kSelThreads, ... and keeps the best of them in registers; a round is that arg-max per
  // warp, the same over the warps' results by warp 0, and a refresh by the one thread that owned the winner.
  constexpr int kSelThreads = 256;
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(scores);
  for (int c = tid; c < K; c += blockDim.x) {
    const double v = scores[c];
    const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(v));
    keys[c] = (v == -1.0 / 0.0) ? 0ull : ((bits >> 63) ? ~bits : (bits | 0x8000000000000000ull));
  }
  __syncthreads();
  if (tid < kSelThreads) {
    unsigned long long* red_k = reinterpret_cast<unsigned long long*>(red_v);
    auto sel_sync = [] { asm volatile("bar.sync 1, 256;" ::: "memory"); };
    auto warp_argmax = [](unsigned long long& k, int& i) {   // every lane gets the warp's (largest key, its lowest index)
      const unsigned hi = static_cast<unsigned>(k >> 32), lo = static_cast<unsigned>(k);
      const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
      const bool c1 = hi == mh;
      const unsigned ml = __reduce_max_sync(0xffffffffu, c1 ? lo : 0u);
      const bool c2 = c1 && lo == ml;
      i = static_cast<int>(__reduce_min_sync(0xffffffffu, c2 ? static_cast<unsigned>(i) : 0x7fffffffu));
      k = (static_cast<unsigned long long>(mh) << 32) | ml;
    };
    unsigned long long my_k = 0ull;
    int my_i = 0x7fffffff;
    auto refresh = [&]() {
      my_k = 0ull; my_i = 0x7fffffff;
      for (int c = tid; c < K; c += kSelThreads) {
        const unsigned long long v = keys[c];
        if (v > my_k) { my_k = v; my_i = c; }   // ascending c: the lowest index of equal keys stays
      }
    };
    refresh();
    constexpr int nwarps = kSelThreads / 32;
    for (int iter = 0; iter < K; ++iter) {
      if (total_tok >= p.budget) break;
      unsigned long long bk = my_k;
      int bi = my_i;
      warp_argmax(bk, bi);
      if (lane == 0) { red_k[warp] = bk; red_i[warp] = bi; }
      sel_sync();
      if (warp == 0) {
        unsigned long long k2 = lane < nwarps ? red_k[lane] : 0ull;
        int i2 = lane < nwarps ? red_i[lane] : 0x7fffffff;
        warp_argmax(k2, i2);
        if (lane == 0) {
          if (k2 == 0ull || i2 == 0x7fffffff) {
            total_tok = 0x7fffffff;  // nothing left
            win_s = -1;
          } else {
            sel_list[n_sel++] = i2;
            total_tok += csize[i2];
            win_s = i2;              // the winner, for its owner
          }
        }
      }
      sel_sync();
      // (win_s is rewritten only behind the next round's first barrier, which no thread passes before it has read it)
      const int won = win_s;
      if (won >= 0 && won % kSelThreads == tid) {
        keys[won] = 0ull;
        refresh();
      }
    }
  }
  __syncthreads();
  // members of the selected clusters -> bitmap over token positions
  const int ns = n_sel;
  for (int s = warp; s < ns; s += (blockDim.x >> 5)) {
    const int c = sel_list[s];
    const int n = min(csize[c], p.max_cluster_size);
    for (int j = lane; j < n; j += 32) {
      const int tok = cl[static_cast<long long>(c) * p.max_cluster_size + j];
      atomicOr(&bitmap[tok >> 5], 1u << (tok & 31));
    }
  }
  __syncthreads();
  // tokens appended since the clusters were last rebuilt: always attended
  for (int tok = p.tail_start + tid; tok < p.num_tokens; tok += blockDim.x) atomicOr(&bitmap[tok >> 5], 1u << (tok & 31));
  __syncthreads();
  // ordered compaction: each thread owns a contiguous run of bitmap words
  const int per = (words + blockDim.x - 1) / blockDim.x;
  const int w0 = min(words, tid * per), w1 = min(words, w0 + per);
  int cnt = 0;
  for (int w = w0; w < w1; ++w) cnt += __popc(bitmap[w]);
  int incl = cnt;
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = warp_sums[lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    warp_sums[lane] = v;
  }
  __syncthreads();
  int pos = incl - cnt + (warp > 0 ? warp_sums[warp - 1] : 0);
  int* out = p.out_idx + static_cast<long long>(g) * p.cap;
  for (int w = w0; w < w1; ++w) {
    uint32_t bits = bitmap[w];
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      if (pos < p.cap) out[pos] = w * 32 + b;
      ++pos;
    }
  }
  if (tid == blockDim.x - 1) p.out_count[g] = min(pos, p.cap);
}

template <bool BF16>
__global__ void __launch_bounds__(1024) retrieve_select_kernel(const __grid_constant__ RetrieveParams p) {
  retrieve_select_body<BF16>(p, blockIdx.x);
}

// All sequences of a ragged batch in one launch: blockIdx.y = sequence, blockIdx.x = KV group.
constexpr int kRetMaxBatch = 32;
struct RetrieveBatch {
  RetrieveParams item[kRetMaxBatch];
};
template <bool BF16>
__global__ void __launch_bounds__(1024) retrieve_select_batch_kernel(const __grid_constant__ RetrieveBatch b) {
  retrieve_select_body<BF16>(b.item[blockIdx.y], blockIdx.x);
}

struct GatherItem {
  const uint8_t* src;   // [G, tokens, D] through strides
  uint8_t* dst;         // [G, cap, D]
  const int* idx;       // [G, cap]
  const int* count;     // [G]
  long long src_group_stride, src_row_stride;
  // block-hybrid caches: rows from split_row on live in a second buffer (pinned host memory, read over PCIe by the
  // same 16-byte loads), row r of it being token split_row + r; src2 == nullptr: everything is in src
  const uint8_t* src2;
  long long src2_group_stride;
  int split_row;
};
struct GatherBatch {
  GatherItem item[2 * kRetMaxBatch];  // keys and values of every sequence
};
__global__ void gather_rows_batch_kernel(const __grid_constant__ GatherBatch b, int cap, int d) {
  const GatherItem& it = b.item[blockIdx.z];
  const int g = blockIdx.y, d8 = d / 8;
  const int n = it.count[g];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < static_cast<long long>(n) * d8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i / d8), c = static_cast<int>(i % d8);
    const int tok = it.idx[static_cast<long long>(g) * cap + j];
    const uint8_t* row = (it.src2 && tok >= it.split_row)
                             ? it.src2 + 2 * (g * it.src2_group_stride + static_cast<long long>(tok - it.split_row) * it.src_row_stride)
                             : it.src + 2 * (g * it.src_group_stride + tok * it.src_row_stride);
    const uint4 v = *reinterpret_cast<const uint4*>(row + c * 16);
    *reinterpret_cast<uint4*>(it.dst + 2 * ((static_cast<long long>(g) * cap + j) * d + c * 8)) = v;
  }
}

// dst[g, j, :] = src[g, idx[g, j], :] for j < count[g]  (16-byte chunks; src rows `src_row_stride` elements apart)
__global__ void gather_rows_kernel(const uint8_t* src, long long src_group_stride, long long src_row_stride, const int* idx,
                                   const int* count, int cap, int d, uint8_t* dst) {
  const int g = blockIdx.y, d8 = d / 8;
  const int n = count[g];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < static_cast<long long>(n) * d8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i / d8), c = static_cast<int>(i % d8);
    const int tok = idx[static_cast<long long>(g) * cap + j];
    const uint4 v = *reinterpret_cast<const uint4*>(src + 2 * (g * src_group_stride + tok * src_row_stride + c * 8));
    *reinterpret_cast<uint4*>(dst + 2 * ((static_cast<long long>(g) * cap + j) * d + c * 8)) = v;
  }
}

}  // namespace sq
