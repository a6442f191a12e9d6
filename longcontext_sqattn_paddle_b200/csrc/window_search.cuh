// Distance-weighted attention-energy histograms for window calibration (sqattn/window_search.py), computed
// blockwise from q and k: the N x N softmax map the reference materialises first is never stored.
//   relative mode (window_search.py:244-283): sink columns dropped; rel = (i-j)/max(i-sink,1) (0 for rows
//     i <= sink); bin = clamp(floor(rel*bins), 0, bins-1); weight = A[i,j] * (rel*bins + 1)
//   absolute mode (20-48, 286-321): bin = i-j, weight = A[i,j] * (i-j), optional sink columns dropped
// A = softmax_j(q_i.k_j / sqrt(D)) over j <= i (cal_attn_weight, sqattn/attn_replacer.py:253-278).
#pragma once
#include "decode.cuh"
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

// Tensor-core version: one CTA = 64 query rows of one head (16 per warp), keys in 64-key tiles staged with
// cp.async (double buffered), S = q k^T by mma.sync.m16n8k16 on the 16-bit inputs.  Two sweeps over the key tiles
// up to the diagonal: row maximum and sum (online), then the normalised weights into a shared-memory histogram.
// A thread owns, per row, 16 keys of increasing index, i.e. non-increasing bins: it adds runs of equal bins in
// registers and issues one shared-memory atomic per run.
constexpr int kWhRows = 64, kWhKeys = 64;

template <bool BF16, int D>
__global__ void __launch_bounds__(128) window_hist_mma_kernel(const __grid_constant__ WindowHistParams p) {
  constexpr int kStride = D + 8;                       // elements per staged row: 16-byte chunks land in distinct banks
  extern __shared__ __align__(16) uint8_t wsm[];
  uint16_t* qs = reinterpret_cast<uint16_t*>(wsm);                 // [64][kStride]
  uint16_t* ks = qs + kWhRows * kStride;                             // [2][64][kStride]
  float* bhist = reinterpret_cast<float*>(ks + 2 * kWhKeys * kStride);  // [nbins]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  // the longest row blocks (most key tiles) are launched first
  const int h = blockIdx.y, kvh = h / p.groups, i0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * kWhRows;
  const uint16_t* qh = reinterpret_cast<const uint16_t*>(p.q) + static_cast<long long>(h) * p.n * D;
  const uint16_t* kh = reinterpret_cast<const uint16_t*>(p.k) + static_cast<long long>(kvh) * p.n * D;
  for (int b = tid; b < p.nbins; b += 128) bhist[b] = 0.f;
  // Q tile (rows past the end read as zero)
  for (int c = tid; c < kWhRows * (D / 8); c += 128) {
    const int r = c / (D / 8), ch = c % (D / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (i0 + r < p.n) v = *reinterpret_cast<const uint4*>(qh + static_cast<long long>(i0 + r) * D + ch * 8);
    *reinterpret_cast<uint4*>(qs + r * kStride + ch * 8) = v;
  }
  auto load_k = [&](int tile, int buf) {
    const int j0 = tile * kWhKeys;
    for (int c = tid; c < kWhKeys * (D / 8); c += 128) {
      const int r = c / (D / 8), ch = c % (D / 8);
      uint16_t* dst = ks + (buf * kWhKeys + r) * kStride + ch * 8;
      if (j0 + r < p.n) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(kh + static_cast<long long>(j0 + r) * D + ch * 8) : "memory");
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  __syncthreads();
  // A fragments of this warp's 16 rows, all k-steps
  uint32_t qa[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
    for (int r = 0; r < 4; ++r)
      qa[kk][r] = *reinterpret_cast<const uint32_t*>(qs + (warp * 16 + g + (r & 1) * 8) * kStride + kk * 16 + tq * 2 + (r >> 1) * 8);
  const int row_a = i0 + warp * 16 + g, row_b = row_a + 8;      // the two rows this thread holds
  const float c2 = p.scale * 1.44269504f;                       // scores are kept as raw dot products; exp(x*scale) = 2^(x*c2)
  const int last_tile = min((i0 + kWhRows - 1) / kWhKeys, (p.n - 1) / kWhKeys);
  auto scores = [&](int buf, float (&s)[8][4]) {
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
#pragma unroll
      for (int np = 0; np < 4; ++np) {   // 16 keys per ldmatrix.x4
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(smem_u32(ks + (buf * kWhKeys + np * 16 + r + (mi >> 1) * 8) * kStride + kk * 16 + (mi & 1) * 8), b0, b1, b2, b3);
        mma_16816<BF16>(s[2 * np], qa[kk], b0, b1);
        mma_16816<BF16>(s[2 * np + 1], qa[kk], b2, b3);
      }
  };
  // ---- sweep 1: row maxima and sums
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  load_k(0, 0);
  for (int t = 0; t <= last_tile; ++t) {
    if (t + 1 <= last_tile) load_k(t + 1, (t + 1) & 1);
    if (t + 1 <= last_tile) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float s[8][4];
    scores(t & 1, s);
    const int j0 = t * kWhKeys;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + nb * 8 + tq * 2 + (e & 1), i = (e >> 1) ? row_b : row_a;
        if (j > i || j >= p.n) s[nb][e] = -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_r[r], mx[r]);
      if (m_new > -INFINITY) {
        float sum = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) sum += ex2_approx((s[nb][2 * r] - m_new) * c2) + ex2_approx((s[nb][2 * r + 1] - m_new) * c2);
        l_r[r] = l_r[r] * ex2_approx((m_r[r] - m_new) * c2) + sum;   // m_r = -inf: l_r is 0 and the factor is 0
        m_r[r] = m_new;
      }
    }
    __syncthreads();   // the buffer that tile t+2 goes into is the one just read
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
    l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
  }
  // ---- sweep 2: weights into the histogram (sink columns carry no weight: tiles below the sink are skipped)
  const int first_tile = p.sink / kWhKeys;
  // a row's keys come in increasing order over the whole sweep, i.e. its bins never increase: a run of equal bins
  // is summed in registers across tiles and costs one shared-memory atomic when it ends
  int cur[2] = {-1, -1};
  float acc[2] = {0.f, 0.f};
  if (first_tile <= last_tile) {
    load_k(first_tile, first_tile & 1);
    for (int t = first_tile; t <= last_tile; ++t) {
      if (t + 1 <= last_tile) load_k(t + 1, (t + 1) & 1);
      if (t + 1 <= last_tile) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      float s[8][4];
      scores(t & 1, s);
      const int j0 = t * kWhKeys;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int i = r ? row_b : row_a;
        if (i >= p.n) continue;
        const float inv_l = 1.0f / l_r[r];
        const float ctx = fmaxf(static_cast<float>(i - p.sink), 1.0f);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = j0 + nb * 8 + tq * 2 + e;
            if (j < p.sink || j > i) continue;
            const float a = ex2_approx((s[nb][2 * r + e] - m_r[r]) * c2) * inv_l;
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
            if (bin >= p.nbins) continue;
            if (bin != cur[r]) {
              if (cur[r] >= 0) atomicAdd(&bhist[cur[r]], acc[r]);
              cur[r] = bin;
              acc[r] = 0.f;
            }
            acc[r] += w;
          }
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r)
    if (cur[r] >= 0) atomicAdd(&bhist[cur[r]], acc[r]);
  __syncthreads();
  for (int b = tid; b < p.nbins; b += 128)
    if (bhist[b] != 0.f) atomicAdd(&p.hist[static_cast<long long>(h) * p.nbins + b], static_cast<double>(bhist[b]));
}

}  // namespace sq
