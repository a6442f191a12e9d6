// Key clustering kernels (cache_hub/kmeans.py): assignment by maximum inner product, centroid update,
// sorted member lists, per-cluster value sums.  Results are bit-exact and independent of thread timing:
//  * scores come from a tensor-core contraction in fp32; a token whose best and second-best score are closer
//    than a rigorous bound on the fp32 accumulation error is re-scored against every centroid in fp64 (exact
//    products, index-order sum) and assigned by a warp-level argmax, lowest index winning ties;
//  * member sums are accumulated in fp64, where adding 16-bit inputs is exact (for clusters whose dynamic
//    range stays below 2^45), hence order-independent although atomics are used.
#pragma once
#include "decode.cuh"
#include "prep.cuh"

namespace sq {

constexpr int kKmTokens = 128;  // tokens per CTA (8 warps x 16)
constexpr int kKmChunk = 64;    // centroids per shared-memory chunk

struct Top2 {
  float best, second;
  int idx;
};
__device__ __forceinline__ void top2_push(Top2& t, float v, int i) {
  if (v > t.best || (v == t.best && i < t.idx)) {
    t.second = t.best;
    t.best = v;
    t.idx = i;
  } else {
    t.second = fmaxf(t.second, v);
  }
}
__device__ __forceinline__ void top2_merge(Top2& t, float ob, float os, int oi) {
  if (ob > t.best || (ob == t.best && oi < t.idx)) {
    t.second = fmaxf(t.best, os);
    t.best = ob;
    t.idx = oi;
  } else {
    t.second = fmaxf(t.second, ob);
  }
}

// swizzled byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] 16-bit tile
template <int D>
__device__ __forceinline__ uint32_t km_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (D * 2) + (((chunk & ~7) | ((chunk & 7) ^ (row & 7))) << 4));
}

// idx[g,t] = argmax_c <data[g,t], cent[g,c]>; a negative value -1-c marks a token whose margin was inside
// the error bound and has to go through kmeans_recheck_kernel.
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
kmeans_assign_kernel(const uint8_t* data, const uint8_t* cent, int* idx, int num_tokens, int num_centroids) {
  __shared__ __align__(128) uint8_t tile[2][kKmChunk * D * 2];
  __shared__ float cnorm[kKmChunk];
  const int g = blockIdx.y, t0 = blockIdx.x * kKmTokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const uint8_t* dg = data + static_cast<long long>(g) * num_tokens * D * 2;
  const uint8_t* cg = cent + static_cast<long long>(g) * num_centroids * D * 2;

  auto load_chunk = [&](int buf, int c0) {
    // 64 rows x D/8 16-byte chunks, 256 threads; rows past the last centroid are zero-filled
    for (int i = threadIdx.x; i < kKmChunk * (D / 8); i += 256) {
      const int row = i / (D / 8), ch = i % (D / 8);
      if (c0 + row < num_centroids) {
        const uint32_t dst = smem_u32(&tile[buf][0]) + km_off<D>(row, ch);
        const uint8_t* src = cg + (static_cast<long long>(c0 + row) * D + ch * 8) * 2;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      } else {
        *reinterpret_cast<uint4*>(&tile[buf][km_off<D>(row, ch)]) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // A fragments: this warp's 16 tokens
  uint32_t a[D / 16][4];
  float nrm[2] = {0.f, 0.f};
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int tok = t0 + warp * 16 + gq + (r & 1) * 8;
      const int col = kk * 16 + tq * 2 + (r >> 1) * 8;
      uint32_t v = 0;
      if (tok < num_tokens) v = *reinterpret_cast<const uint32_t*>(dg + (static_cast<long long>(tok) * D + col) * 2);
      a[kk][r] = v;
      const float x0 = to_f32<BF16>(static_cast<uint16_t>(v & 0xffffu)), x1 = to_f32<BF16>(static_cast<uint16_t>(v >> 16));
      nrm[r & 1] += x0 * x0 + x1 * x1;
    }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    nrm[r] += __shfl_xor_sync(0xffffffffu, nrm[r], 1);
    nrm[r] += __shfl_xor_sync(0xffffffffu, nrm[r], 2);
  }
  Top2 top[2] = {{-INFINITY, -INFINITY, 0}, {-INFINITY, -INFINITY, 0}};
  float max_cnorm2 = 0.f;

  const int nchunks = num_centroids / kKmChunk + ((num_centroids % kKmChunk) ? 1 : 0);
  load_chunk(0, 0);
  for (int ci = 0; ci < nchunks; ++ci) {
    const int buf = ci & 1, c0 = ci * kKmChunk;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (ci + 1 < nchunks) load_chunk(buf ^ 1, (ci + 1) * kKmChunk);
    // squared norms of this chunk's centroids (4 threads per centroid)
    {
      const int row = threadIdx.x >> 2, part = threadIdx.x & 3;
      float s = 0.f;
      for (int ch = part; ch < D / 8; ch += 4) {
        float f[8];
        unpack8<BF16>(*reinterpret_cast<const uint4*>(&tile[buf][km_off<D>(row, ch)]), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += f[i] * f[i];
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (part == 0) cnorm[row] = s;
    }
    const uint32_t tb = smem_u32(&tile[buf][0]);
#pragma unroll
    for (int nb = 0; nb < kKmChunk / 8; nb += 2) {
      float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t b0, b1, b2, b3;
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4(tb + km_off<D>((nb + (mi >> 1)) * 8 + r, kk * 2 + (mi & 1)), b0, b1, b2, b3);
        mma_16816<BF16>(s0, a[kk], b0, b1);
        mma_16816<BF16>(s1, a[kk], b2, b3);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c_a = c0 + nb * 8 + tq * 2 + (e & 1), c_b = c_a + 8;
        if (c_a < num_centroids) top2_push(top[e >> 1], s0[e], c_a);
        if (c_b < num_centroids) top2_push(top[e >> 1], s1[e], c_b);
      }
    }
    __syncthreads();
    for (int i = 0; i < kKmChunk; ++i) max_cnorm2 = fmaxf(max_cnorm2, cnorm[i]);
  }
  // combine the 4 lanes of each row; every lane ends with the row's result
#pragma unroll
  for (int r = 0; r < 2; ++r) {
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, top[r].best, o);
      const float os = __shfl_xor_sync(0xffffffffu, top[r].second, o);
      const int oi = __shfl_xor_sync(0xffffffffu, top[r].idx, o);
      top2_merge(top[r], ob, os, oi);
    }
    const int tok = t0 + warp * 16 + gq + r * 8;
    if (tq == 0 && tok < num_tokens) {
      // |fp32 tensor-core sum - exact| <= 128 * 2^-22 * sum|terms| <= 2^-15 |k||x| per score; two scores are compared
      const float tol = 6.2e-5f * sqrtf(nrm[r]) * sqrtf(max_cnorm2);
      const bool sure = (top[r].best - top[r].second) > tol;
      idx[static_cast<long long>(g) * num_tokens + tok] = sure ? top[r].idx : (-1 - top[r].idx);
    }
  }
}

// Exact re-scoring of the flagged tokens: one warp per token, fp64, warp-level argmax (lowest index on ties).
template <int D, bool BF16>
__global__ void kmeans_recheck_kernel(const uint8_t* data, const uint8_t* cent, int* idx, int groups, int num_tokens,
                                      int num_centroids) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(groups) * num_tokens) return;
  if (idx[w] >= 0) return;
  const int g = static_cast<int>(w / num_tokens);
  const uint16_t* k = reinterpret_cast<const uint16_t*>(data) + w * D;
  const uint16_t* cg = reinterpret_cast<const uint16_t*>(cent) + static_cast<long long>(g) * num_centroids * D;
  double best = -1.0 / 0.0;
  int bi = 0x7fffffff;
  for (int c = lane; c < num_centroids; c += 32) {
    const uint16_t* x = cg + static_cast<long long>(c) * D;
    double s = 0.0;
    for (int d = 0; d < D; ++d) s += static_cast<double>(to_f32<BF16>(k[d])) * static_cast<double>(to_f32<BF16>(x[d]));
    if (s > best) { best = s; bi = c; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const double ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  if (lane == 0) idx[w] = bi;
}

// sums[g, idx[g,t], :] += x[g,t,:] (fp64), counts[g, idx] += 1.  One 16-lane group per token.
template <int D, bool BF16>
__global__ void kmeans_accumulate_kernel(const uint8_t* x, const int* idx, double* sums, int* counts, int groups,
                                         int num_tokens, int num_centroids) {
  constexpr int d8 = D / 8;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long tok = tid / d8;
  const int c = static_cast<int>(tid % d8);
  if (tok >= static_cast<long long>(groups) * num_tokens) return;
  const int g = static_cast<int>(tok / num_tokens);
  const int ci = idx[tok];
  float f[8];
  unpack8<BF16>(*reinterpret_cast<const uint4*>(x + (tok * D + c * 8) * 2), f);
  double* dst = sums + (static_cast<long long>(g) * num_centroids + ci) * D + c * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) atomicAdd(dst + i, static_cast<double>(f[i]));
  if (c == 0 && counts) atomicAdd(counts + static_cast<long long>(g) * num_centroids + ci, 1);
}

// centroid = S/C (fp32) where C > 0, optionally / sqrt(sum_d x_d^2) with the sum in fp64 in index order
// (kmeans.py:116-124); one thread per centroid.
template <int D, bool BF16>
__global__ void kmeans_update_kernel(uint8_t* cent, const double* sums, const int* counts, long long total,
                                     int normalize) {
  const long long c = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (c >= total) return;
  const int cnt = counts[c];
  if (cnt <= 0) return;
  const double* s = sums + c * D;
  uint16_t* out = reinterpret_cast<uint16_t*>(cent) + c * D;
  const float fc = static_cast<float>(cnt);
  double nrm = 0.0;
  if (normalize) {
    for (int d = 0; d < D; ++d) {
      const double x = static_cast<double>(__fdiv_rn(static_cast<float>(s[d]), fc));
      nrm += x * x;
    }
    nrm = sqrt(nrm);
  }
  for (int d = 0; d < D; ++d) {
    float x = __fdiv_rn(static_cast<float>(s[d]), fc);
    if (normalize) x = static_cast<float>(static_cast<double>(x) / nrm);
    out[d] = from_f32<BF16>(x);
  }
}

// out[g,c,:] = dtype(fp32(sums))  (the .to(value.dtype) of triton_index_add, kmeans.py:329)
template <bool BF16>
__global__ void kmeans_store_sums_kernel(const double* sums, uint8_t* out, long long n) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) reinterpret_cast<uint16_t*>(out)[i] = from_f32<BF16>(static_cast<float>(sums[i]));
}

// Member lists in token order.  One CTA per group walks the tokens in order, 1024 at a time; inside a chunk
// warps take their turn one after the other, and inside a warp tokens of the same cluster are ranked with
// __match_any_sync, so slot = (members seen so far) + (rank inside the warp).
__global__ void __launch_bounds__(1024)
kmeans_reverse_index_kernel(const int* idx, int num_tokens, int num_centroids, int max_cluster_size, int* clusters,
                            int* cluster_size) {
  const int g = blockIdx.x;
  const int* ig = idx + static_cast<long long>(g) * num_tokens;
  int* cs = cluster_size + static_cast<long long>(g) * num_centroids;
  int* cl = clusters + static_cast<long long>(g) * num_centroids * max_cluster_size;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = threadIdx.x; c < num_centroids; c += blockDim.x) cs[c] = 0;
  __syncthreads();
  for (int base = 0; base < num_tokens; base += 1024) {
    const int tok = base + threadIdx.x;
    const bool live = tok < num_tokens;
    const int c = live ? ig[tok] : -1 - lane;  // dead lanes get distinct keys
    const unsigned peers = __match_any_sync(0xffffffffu, c);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int leader = __ffs(peers) - 1;
    for (int w = 0; w < 32; ++w) {
      if (w == warp && live) {
        int start = 0;
        if (lane == leader) {
          start = cs[c];
          cs[c] = start + __popc(peers);
        }
        start = __shfl_sync(peers, start, leader);
        const int slot = start + rank;
        if (slot < max_cluster_size) cl[static_cast<long long>(c) * max_cluster_size + slot] = tok;
      }
      __syncthreads();
    }
  }
}

__global__ void max_int_kernel(const int* x, long long n, int* out) {
  int m = 0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    m = max(m, x[i]);
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}

}  // namespace sq
