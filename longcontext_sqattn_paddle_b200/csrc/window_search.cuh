// Distance-weighted attention-energy histograms for window calibration (sqattn/window_search.py), computed
// blockwise from q and k: the N x N softmax map the reference materialises first is never stored.
//   relative mode (window_search.py:244-283): sink columns dropped; rel = (i-j)/max(i-sink,1) (0 for rows
//     i <= sink); bin = clamp(floor(rel*bins), 0, bins-1); weight = A[i,j] * (rel*bins + 1)
//   absolute mode (20-48, 286-321): bin = i-j, weight = A[i,j] * (i-j), optional sink columns dropped
// A = softmax_j(q_i.k_j / sqrt(D)) over j <= i (cal_attn_weight, sqattn/attn_replacer.py:253-278).
#pragma once
#include "prep.cuh"

namespace sq {

struct WindowHistParams {
  const uint8_t* q;   // [Hq, N, D]
  const uint8_t* k;   // [Hkv, N, D]
  double* hist;       // [Hq, nbins]
  int hq, groups, n, d, nbins, sink, relative;
  float scale;        // 1/sqrt(D)
};

// One warp per query row; lanes stride over the keys.  Two passes: softmax statistics, then weights.
template <bool BF16>
__global__ void __launch_bounds__(256) window_hist_kernel(const __grid_constant__ WindowHistParams p) {
  extern __shared__ float wh[];  // [8 warps][D] query rows, then [nbins] block histogram
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qrow = wh + warp * p.d;
  float* bhist = wh + 8 * p.d;
  const int h = blockIdx.y, kvh = h / p.groups;
  for (int b = threadIdx.x; b < p.nbins; b += blockDim.x) bhist[b] = 0.f;
  __syncthreads();
  const uint16_t* qh = reinterpret_cast<const uint16_t*>(p.q) + static_cast<long long>(h) * p.n * p.d;
  const uint16_t* kh = reinterpret_cast<const uint16_t*>(p.k) + static_cast<long long>(kvh) * p.n * p.d;
  for (int i = blockIdx.x * 8 + warp; i < p.n; i += gridDim.x * 8) {
    for (int d = lane; d < p.d; d += 32) qrow[d] = to_f32<BF16>(qh[static_cast<long long>(i) * p.d + d]) * p.scale;
    __syncwarp();
    auto score = [&](int j) {
      const uint4* kr = reinterpret_cast<const uint4*>(kh + static_cast<long long>(j) * p.d);
      float s = 0.f;
      for (int c = 0; c < p.d / 8; ++c) {
        float f[8];
        unpack8<BF16>(kr[c], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) s += qrow[c * 8 + e] * f[e];
      }
      return s;
    };
    float m = -INFINITY, l = 0.f;
    for (int j = lane; j <= i; j += 32) {
      const float s = score(j);
      const float mn = fmaxf(m, s);
      l = l * __expf(m - mn) + __expf(s - mn);
      m = mn;
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), ol = __shfl_xor_sync(0xffffffffu, l, o);
      const float mn = fmaxf(m, om);
      l = ((m == -INFINITY) ? 0.f : l * __expf(m - mn)) + ((om == -INFINITY) ? 0.f : ol * __expf(om - mn));
      m = mn;
    }
    const float inv_l = 1.0f / l;
    const float ctx = fmaxf(static_cast<float>(i - p.sink), 1.0f);
    for (int j = lane + p.sink; j <= i; j += 32) {  // sink columns carry no weight
      const float a = __expf(score(j) - m) * inv_l;
      int bin;
      float w;
      if (p.relative) {
        const float rel = (i <= p.sink) ? 0.f : static_cast<float>(i - j) / ctx;
        bin = min(max(static_cast<int>(floorf(rel * p.nbins)), 0), p.nbins - 1);
        w = a * (rel * p.nbins + 1.0f);
      } else {
        bin = i - j;
        w = a * static_cast<float>(i - j);
      }
      if (bin < p.nbins) atomicAdd(&bhist[bin], w);
    }
    __syncwarp();
  }
  __syncthreads();
  for (int b = threadIdx.x; b < p.nbins; b += blockDim.x)
    if (bhist[b] != 0.f) atomicAdd(&p.hist[static_cast<long long>(h) * p.nbins + b], static_cast<double>(bhist[b]));
}

}  // namespace sq
