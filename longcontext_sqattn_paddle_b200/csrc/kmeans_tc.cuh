// Key-to-centroid assignment on the 5th-generation tensor cores (cache_hub/kmeans.py:7-79 is the reference
// kernel): scores <k_t, x_c> for 256 tokens x all centroids of a group per CTA as tcgen05 MMAs with the
// accumulators in tensor memory, and a running top-2 per token in the epilogue.
//
//   warp 0        TMA producer: the CTA's two 128-token tiles once, then 256-centroid tiles into a 2-stage ring
//   warp 1        MMA issuer: for every centroid tile, S_a = tokens_a x centroids^T (M128 N256 K16 x D/16) for the
//                 two token tiles a = 0, 1 in turn; owns the 512 TMEM columns (two 256-column accumulators)
//   warps 2..5    epilogue of token tile 0, warps 6..9 of token tile 1: one token per thread (a TMEM lane)
// While the epilogue warps of one token tile scan their 256 scores, the tensor core computes the other tile's, so
// the two never wait for each other as long as a scan (about 3 instructions per score) is shorter than a tile's
// 1024 tensor-pipe clocks.  Every centroid tile staged in shared memory is used by both token tiles, which halves
// the L2 traffic per flop.
//
// Exactness: the fp32 tensor-core score is not the exact inner product, so a token whose best and second-best
// scores are closer than a bound on that error is put on a list and re-scored in fp64 by kmeans_recheck_list_kernel
// (exact products, index-order sum, lowest index on ties): the final assignment is the exact argmax.
#pragma once
#include <cuda.h>

#include "kmeans.cuh"
#include "ptx.cuh"

namespace sq {

constexpr int kKtTokens = 256;    // tokens per CTA (two M = 128 tiles)
constexpr int kKtCent = 256;      // centroids per MMA group (N)
constexpr int kKtStages = 2;
// |tensor-core fp32 sum - exact| is bounded by (terms * 2^-22) * sum|terms| <= 2^-15 |k||x| for 128 terms; the two
// scores that are compared each carry it, and the factor of two on top covers an accumulator that truncates
constexpr float kKtTol = 1.25e-4f;

struct KmeansTcParams {
  const uint8_t* data;      // [G, T, D] for the token norms
  int* idx;                 // [G, T]
  int* flagged;             // [cap] packed g * T + t of tokens to re-score
  int* flagged_count;       // number of entries (may exceed cap: the overflow is re-scored by a full sweep)
  int flagged_cap;
  const float* max_cnorm2;  // [G] largest squared centroid norm of the group
  int num_tokens, num_centroids, bf16;
};

template <int D>
struct KmeansTcSmem {
  static constexpr int kABytes = 128 * D * 2;
  static constexpr int kBBytes = kKtCent * D * 2;
  static constexpr int kAOff = 0;
  static constexpr int kBOff = 2 * kABytes;
  static constexpr int kBarOff = kBOff + kKtStages * kBBytes;
  // a_full, b_full[2], s_full[2], s_empty[2]
  static constexpr int kMiscOff = kBarOff + 8 * 7;
  static constexpr int kTotal = kMiscOff + 16;
};

// max over the centroids of a group of sum_d x_d^2 (fp32): one CTA per group
template <int D, bool BF16>
__global__ void __launch_bounds__(256) kmeans_cnorm_max_kernel(const uint8_t* cent, int num_centroids, float* out) {
  __shared__ float red[8];
  const int g = blockIdx.x;
  const uint8_t* cg = cent + static_cast<long long>(g) * num_centroids * D * 2;
  float m = 0.f;
  for (int c = threadIdx.x; c < num_centroids; c += 256) {
    float s = 0.f;
    for (int ch = 0; ch < D / 8; ++ch) {
      float f[8];
      unpack8<BF16>(*reinterpret_cast<const uint4*>(cg + (static_cast<long long>(c) * D + ch * 8) * 2), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += f[i] * f[i];
    }
    m = fmaxf(m, s);
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    out[g] = m;
  }
}

template <int D>
__global__ void __launch_bounds__(320, 1)
kmeans_assign_tc_kernel(const __grid_constant__ CUtensorMap tm_data, const __grid_constant__ CUtensorMap tm_cent,
                        const __grid_constant__ KmeansTcParams p) {
  using L = KmeansTcSmem<D>;
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  const int g = blockIdx.y, t0 = blockIdx.x * kKtTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto mark_all_for_recheck = [&]() {   // this CTA cannot deliver: every token of it goes through the exact path
    for (int r = threadIdx.x; r < kKtTokens; r += blockDim.x)
      if (t0 + r < p.num_tokens) p.idx[static_cast<long long>(g) * p.num_tokens + t0 + r] = -1;
    if (threadIdx.x == 0) atomicAdd(p.flagged_count, p.flagged_cap + 1);   // forces the full sweep
  };
  if ((sbase & 1023u) || device_failed()) {
    if ((sbase & 1023u) && threadIdx.x == 0) record_failure(400);
    mark_all_for_recheck();
    return;
  }
  const uint32_t a_s = sbase + L::kAOff, b_s = sbase + L::kBOff, bars = sbase + L::kBarOff;
  const uint32_t bar_a_full = bars, bar_b_full = bars + 8, bar_s_full = bars + 24, bar_s_empty = bars + 40;
  volatile uint32_t* tmem_base_s = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOff);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  const int ntiles = (p.num_centroids + kKtCent - 1) / kKtCent;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    mbar_init(bar_a_full, 1);
    for (int i = 0; i < kKtStages; ++i) mbar_init(bar_b_full + 8 * i, 1);
    for (int a = 0; a < 2; ++a) { mbar_init(bar_s_full + 8 * a, 1); mbar_init(bar_s_empty + 8 * a, 128); }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_s)), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_s;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_data); tma_prefetch_desc(&tm_cent);
      mbar_expect_tx(bar_a_full, 2 * L::kABytes);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(a_s + a * L::kABytes + h * (128 * 128), &tm_data, bar_a_full, h * 64, t0 + a * 128, g, 0);
      bool ok = true;
      for (int j = 0; ok && j < ntiles; ++j) {
        const int st = j & 1;
        // stage st was last read by the MMAs of tile j-2, token tile 1: their completion is s_full[1], phase j-2
        if (j >= 2) ok = mbar_wait(bar_s_full + 8, (j - 2) & 1, cta_abort, 401);
        if (!ok) break;
        mbar_expect_tx(bar_b_full + 8 * st, L::kBBytes);
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(b_s + st * L::kBBytes + h * (kKtCent * 128), &tm_cent, bar_b_full + 8 * st, h * 64, j * kKtCent, g, 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tcgen05 issuer
    {  // converged warp, one elected lane issues (operands stay warp-uniform values)
      const uint32_t fmt = p.bf16 ? 1u : 0u;
      const uint32_t idesc = make_idesc(fmt, fmt, 0, 0, 128, kKtCent);
      bool ok = mbar_wait_warp(bar_a_full, 0, cta_abort, 411);
      for (int j = 0; ok && j < ntiles; ++j) {
        const int st = j & 1;
        ok = mbar_wait_warp(bar_b_full + 8 * st, (j >> 1) & 1, cta_abort, 412);
        if (!ok) break;
        const uint64_t b_desc = smem_desc_sw128(b_s + st * L::kBBytes, 16, 1024);
        for (int a = 0; ok && a < 2; ++a) {
          if (j >= 1) ok = mbar_wait_warp(bar_s_empty + 8 * a, (j - 1) & 1, cta_abort, 413);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = smem_desc_sw128(a_s + a * L::kABytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off_a = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
            const uint32_t off_b = (kk >> 2) * (kKtCent * 128) + (kk & 3) * 32;
            mma_ss_elect(tmem + a * kKtCent, a_desc + (off_a >> 4), b_desc + (off_b >> 4), idesc, kk > 0);
          }
          tc_commit_elect(bar_s_full + 8 * a);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: running top-2 per token
    const int a = (warp - 2) >> 2;              // token tile of this warp
    const int quarter = warp & 3;               // TMEM lanes this warp may touch: 32 * (warp % 4) ..
    const int row = quarter * 32 + lane;
    const int tok = t0 + a * 128 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    // |k|^2 of this thread's token, from global memory (the tile has just been loaded: an L2 hit)
    float nrm2 = 0.f;
    if (tok < p.num_tokens) {
      const uint4* kr = reinterpret_cast<const uint4*>(p.data + (static_cast<long long>(g) * p.num_tokens + tok) * D * 2);
      uint4 raw[D / 8];
#pragma unroll
      for (int ch = 0; ch < D / 8; ++ch) raw[ch] = kr[ch];          // all loads in flight before the first use
#pragma unroll
      for (int ch = 0; ch < D / 8; ++ch) {
        float f[8];
        if (p.bf16) unpack8<true>(raw[ch], f); else unpack8<false>(raw[ch], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) nrm2 += f[i] * f[i];
      }
    }
    float best = -INFINITY, second = -INFINITY;
    int best_idx = 0;
    bool ok = true;
    for (int j = 0; ok && j < ntiles; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full + 8 * a, j & 1, cta_abort, 421));
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_tmem = tmem + lane_addr + a * kKtCent;
      // num_centroids is a multiple of 32: a 32-column chunk is whole or absent
      const int nch = min(kKtCent / 32, (p.num_centroids - j * kKtCent) / 32);
      auto scan = [&](const uint32_t (&r)[32], int c0) {
        const float before = best;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float v = __uint_as_float(r[c]);
          second = fmaxf(second, fminf(best, v));
          best = fmaxf(best, v);
        }
        if (best > before) {                     // a new maximum inside this chunk: its first occurrence
          int first = 31;
#pragma unroll
          for (int c = 31; c >= 0; --c)
            if (__uint_as_float(r[c]) == best) first = c;
          best_idx = c0 + first;
        }
      };
      // two register buffers: the load of the next chunk is in flight while this one is scanned
      uint32_t r0[32], r1[32];
      tmem_ld32(s_tmem, r0);
#pragma unroll 1
      for (int ch = 0; ch < nch; ch += 2) {
        tmem_wait_ld();
        if (ch + 1 < nch) tmem_ld32(s_tmem + (ch + 1) * 32, r1);
        scan(r0, j * kKtCent + ch * 32);
        if (ch + 1 < nch) {
          tmem_wait_ld();
          if (ch + 2 < nch) tmem_ld32(s_tmem + (ch + 2) * 32, r0);
          scan(r1, j * kKtCent + (ch + 1) * 32);
        }
      }
      tc_fence_before();
      mbar_arrive(bar_s_empty + 8 * a);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (tok < p.num_tokens) {
      const long long at = static_cast<long long>(g) * p.num_tokens + tok;
      const float tol = kKtTol * sqrtf(nrm2) * sqrtf(p.max_cnorm2[g]);
      const bool sure = ok && (best - second) > tol;
      p.idx[at] = sure ? best_idx : (-1 - best_idx);
      if (!sure) {
        const int slot = atomicAdd(p.flagged_count, 1);
        if (slot < p.flagged_cap) p.flagged[slot] = static_cast<int>(at);
      }
    }
  }

  // ------------------------------------------------------------------ tear-down (also after a wait gave up)
  if (*cta_abort) {
    const uint64_t t_wait = globaltimer_ns();
    while (globaltimer_ns() - t_wait < 200000ull) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// Exact re-scoring of the listed tokens, one CTA per token at a time (the CTAs loop over the list):
//   1. fp32 scores of ALL centroids of the group into shared memory, a half warp (D = 128) per centroid row with
//      16-byte loads, so a token costs one coalesced sweep over its group's centroids;
//   2. the candidates: centroids whose fp32 score lies within the error band of the largest one (the same bound
//      as in the assignment kernel, which also covers this pass's own rounding);
//   3. the candidates' exact scores in fp64 (exact products, index-order sum), the largest wins, the lowest index
//      on ties.  More than kMaxCand candidates (degenerate data, e.g. an all-zero key) take the fp64 path for every
//      centroid.
// When the list overflowed, every token whose idx is still negative is re-scored instead (a sweep over all
// tokens, the list is ignored).
constexpr int kMaxCand = 64;

template <int D, bool BF16>
__device__ __forceinline__ double exact_score(const double* kd, const uint8_t* row) {
  const uint4* x = reinterpret_cast<const uint4*>(row);
  double s = 0.0;
#pragma unroll 4
  for (int ch = 0; ch < D / 8; ++ch) {
    float f[8];
    unpack8<BF16>(x[ch], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += kd[ch * 8 + i] * static_cast<double>(f[i]);
  }
  return s;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(256)
kmeans_recheck_list_kernel(const uint8_t* data, const uint8_t* cent, int* idx, const int* flagged, const int* flagged_count,
                           int flagged_cap, const float* max_cnorm2, int groups, int num_tokens, int num_centroids) {
  extern __shared__ float score_s[];      // [num_centroids]
  __shared__ double kd[D];
  __shared__ float red_s[8];
  __shared__ double best_s[8];
  __shared__ int idx_s[8];
  __shared__ int cand_s[kMaxCand];
  __shared__ int ncand_s;
  constexpr int kLanes = D / 8;           // lanes per centroid row
  constexpr int kRows = 32 / kLanes;      // rows a warp takes at a time
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sub = lane / kLanes, ch = lane % kLanes;
  const int count = *flagged_count;
  const bool sweep = count > flagged_cap;
  const long long total = sweep ? static_cast<long long>(groups) * num_tokens : count;
  for (long long e = blockIdx.x; e < total; e += gridDim.x) {
    const long long at = sweep ? e : flagged[e];
    if (sweep && idx[at] >= 0) continue;
    const int g = static_cast<int>(at / num_tokens);
    const uint8_t* krow = data + at * D * 2;
    const uint8_t* cg = cent + static_cast<long long>(g) * num_centroids * D * 2;
    __syncthreads();
    float kf[8];
    unpack8<BF16>(*reinterpret_cast<const uint4*>(krow + ch * 16), kf);
    if (threadIdx.x < kLanes) {
#pragma unroll
      for (int i = 0; i < 8; ++i) kd[ch * 8 + i] = static_cast<double>(kf[i]);
    }
    if (threadIdx.x == 0) ncand_s = 0;
    float nrm2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) nrm2 += kf[i] * kf[i];
    for (int o = 1; o < kLanes; o <<= 1) nrm2 += __shfl_xor_sync(0xffffffffu, nrm2, o);
    // 1. fp32 scores, four rows per half warp in flight
    float mx = -INFINITY;
    for (int c0 = warp * kRows + sub; c0 < num_centroids; c0 += 8 * kRows * 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 8 * kRows;
        v[u] = c < num_centroids ? *reinterpret_cast<const uint4*>(cg + (static_cast<long long>(c) * D + ch * 8) * 2)
                                 : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 8 * kRows;
        float f[8], sc = 0.f;
        unpack8<BF16>(v[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) sc += kf[i] * f[i];
        for (int o = 1; o < kLanes; o <<= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        if (c < num_centroids) {
          if (ch == 0) score_s[c] = sc;
          mx = fmaxf(mx, sc);
        }
      }
    }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red_s[warp] = mx;
    __syncthreads();
    mx = red_s[0];
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_s[w]);
    // 2. candidates inside the error band
    const float tol = kKtTol * sqrtf(nrm2) * sqrtf(max_cnorm2[g]);
    for (int c = threadIdx.x; c < num_centroids; c += 256) {
      if (score_s[c] >= mx - tol) {
        const int slot = atomicAdd(&ncand_s, 1);
        if (slot < kMaxCand) cand_s[slot] = c;
      }
    }
    __syncthreads();
    const int ncand = ncand_s;
    // 3. exact scores
    double best = -1.0 / 0.0;
    int bi = 0x7fffffff;
    if (ncand <= kMaxCand) {
      if (threadIdx.x < ncand) {
        bi = cand_s[threadIdx.x];
        best = exact_score<D, BF16>(kd, cg + static_cast<long long>(bi) * D * 2);
      }
    } else {
      for (int c = threadIdx.x; c < num_centroids; c += 256) {
        const double sc = exact_score<D, BF16>(kd, cg + static_cast<long long>(c) * D * 2);
        if (sc > best) { best = sc; bi = c; }   // ascending c: the lowest index is kept on ties
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { best_s[warp] = best; idx_s[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < 8; ++w)
        if (best_s[w] > best || (best_s[w] == best && idx_s[w] < bi)) { best = best_s[w]; bi = idx_s[w]; }
      idx[at] = bi;
    }
  }
}

// ---- member sums without floating-point atomics --------------------------------------------------------------
// counts[g, c] = members of cluster c and slot[g, t] = the arrival rank of token t inside its cluster.  The rank
// depends on timing, the sums below do not: adding 16-bit values in fp64 is exact in any order.
__global__ void kmeans_count_kernel(const int* idx, int* counts, int* slot, long long total, int num_tokens, int num_centroids) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i / num_tokens);
    slot[i] = atomicAdd(counts + static_cast<long long>(g) * num_centroids + idx[i], 1);
  }
}
// offsets[g, c] = exclusive prefix sum of counts[g, :]: one CTA per group
__global__ void __launch_bounds__(1024) kmeans_offsets_kernel(const int* counts, int* offsets, int num_centroids) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int g = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* cg = counts + static_cast<long long>(g) * num_centroids;
  int* og = offsets + static_cast<long long>(g) * num_centroids;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < num_centroids; base += 1024) {
    const int c = base + threadIdx.x;
    const int v = c < num_centroids ? cg[c] : 0;
    int incl = v;
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = carry_s;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (c < num_centroids) og[c] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = before + incl;
    __syncthreads();
  }
}
__global__ void kmeans_scatter_kernel(const int* idx, const int* slot, const int* offsets, int* members, long long total,
                                      int num_tokens, int num_centroids) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i / num_tokens);
    const int c = idx[i];
    members[static_cast<long long>(g) * num_tokens + offsets[static_cast<long long>(g) * num_centroids + c] + slot[i]] =
        static_cast<int>(i - static_cast<long long>(g) * num_tokens);
  }
}
// sums[g, c, :] = sum over the members of x[g, t, :] in fp64: one warp per cluster, a half warp per member row
// (16 lanes x 16 bytes), two rows in flight.
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
kmeans_cluster_sum_kernel(const uint8_t* x, const int* members, const int* offsets, const int* counts, double* sums,
                          long long total_clusters, int num_tokens, int num_centroids) {
  static_assert(D == 128 || D == 64, "a half warp covers a row");
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= total_clusters) return;
  const int g = static_cast<int>(w / num_centroids);
  const int cnt = counts[w], off = offsets[w];
  const int* mem = members + static_cast<long long>(g) * num_tokens + off;
  const uint8_t* xg = x + static_cast<long long>(g) * num_tokens * D * 2;
  constexpr int kLanesPerRow = D / 8;          // 16 or 8
  constexpr int kRowsPerIter = 32 / kLanesPerRow;
  const int sub = lane / kLanesPerRow, ch = lane % kLanesPerRow;
  double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  constexpr int kInFlight = 4;                 // member rows a lane has in flight
  for (int m0 = sub; m0 < cnt; m0 += kRowsPerIter * kInFlight) {
    uint4 v[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int m = m0 + u * kRowsPerIter;
      v[u] = m < cnt ? *reinterpret_cast<const uint4*>(xg + (static_cast<long long>(mem[m]) * D + ch * 8) * 2)
                     : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      float f[8];
      unpack8<BF16>(v[u], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += static_cast<double>(f[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    for (int o = kLanesPerRow; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  if (sub == 0) {
    double* dst = sums + w * D + ch * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = acc[i];
  }
}

// Member lists in token order from the arrival-order lists: one warp per cluster ranks its members (a member's
// position is the number of members with a smaller token index) and writes clusters[g, c, :min(n, max_cluster_size)]
// and cluster_size[g, c] (triton_reverse_index, kmeans.py:199-262, whose own order is the atomic arrival order).
__global__ void __launch_bounds__(256)
kmeans_sort_members_kernel(const int* members, const int* offsets, const int* counts, int* clusters, int* cluster_size,
                           long long total_clusters, int num_tokens, int num_centroids, int max_cluster_size) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= total_clusters) return;
  const int g = static_cast<int>(w / num_centroids);
  const int n = counts[w];
  const int* mem = members + static_cast<long long>(g) * num_tokens + offsets[w];
  int* out = clusters + w * max_cluster_size;
  if (lane == 0) cluster_size[w] = n;
  for (int i = lane; i < n; i += 32) {
    const int t = mem[i];
    int rank = 0;
    for (int j = 0; j < n; ++j) rank += mem[j] < t ? 1 : 0;     // token indices are distinct
    if (rank < max_cluster_size) out[rank] = t;
  }
}

}  // namespace sq
