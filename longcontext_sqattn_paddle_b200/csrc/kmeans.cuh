// Key clustering kernels (cache_hub/kmeans.py) around the tensor-core assignment of kmeans_tc.cuh: centroid update,
// sorted member lists, stored value sums.  Results are bit-exact and independent of thread timing:
//  * assignments are the exact argmax (kmeans_tc.cuh: fp32 tensor-core scores, fp64 re-scoring of near ties);
//  * member sums are accumulated in fp64, where adding 16-bit inputs is exact (for clusters whose dynamic
//    range stays below 2^45), hence independent of the order in which the members are visited.
#pragma once
#include "decode.cuh"
#include "prep.cuh"

namespace sq {

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
