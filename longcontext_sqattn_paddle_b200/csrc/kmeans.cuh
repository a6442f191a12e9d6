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
// (kmeans.py:116-124).  One warp per centroid: a lane takes D/32 consecutive dimensions, and the fp64 sum of squares
// is passed from lane to lane so that it is added in index order whatever the warp does in parallel.
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
kmeans_update_kernel(uint8_t* cent, const double* sums, const int* counts, long long total, int normalize) {
  constexpr int kPer = D / 32;
  const long long c = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (c >= total) return;
  const int cnt = counts[c];
  if (cnt <= 0) return;
  const double* s = sums + c * D + lane * kPer;
  uint16_t* out = reinterpret_cast<uint16_t*>(cent) + c * D + lane * kPer;
  const float fc = static_cast<float>(cnt);
  float x[kPer];
#pragma unroll
  for (int i = 0; i < kPer; ++i) x[i] = __fdiv_rn(static_cast<float>(s[i]), fc);
  double nrm = 0.0;
  if (normalize) {
    double run = 0.0;
    for (int l = 0; l < 32; ++l) {
      if (lane == l) {
#pragma unroll
        for (int i = 0; i < kPer; ++i) run += static_cast<double>(x[i]) * static_cast<double>(x[i]);
      }
      run = __shfl_sync(0xffffffffu, run, l);
    }
    nrm = sqrt(run);
  }
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    float v = x[i];
    if (normalize) v = static_cast<float>(static_cast<double>(v) / nrm);
    out[i] = from_f32<BF16>(v);
  }
}

// out[g,c,:] = dtype(fp32(sums))  (the .to(value.dtype) of triton_index_add, kmeans.py:329)
template <bool BF16>
__global__ void kmeans_store_sums_kernel(const double* sums, uint8_t* out, long long n) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) reinterpret_cast<uint16_t*>(out)[i] = from_f32<BF16>(static_cast<float>(sums[i]));
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
