// Row-wise kernels of the decoder layer around the attention operator (model_hub/utils.py): RMS norm, rotary
// position embedding applied in place to the fused QKV projection, and SiLU(gate) * up.  HBM-bound streaming
// passes with 16-byte accesses.  Each follows the reference's chain of tensor ops, rounding to the 16-bit
// activation type wherever the reference materialises a tensor of that type.
#pragma once
#include "prep.cuh"

namespace sq {

template <bool BF16>
__device__ __forceinline__ float round16(float f) { return to_f32<BF16>(from_f32<BF16>(f)); }

// out[r, :] = ((x * rsqrt(mean(x^2) + eps)) * w), model_hub/utils.py:14-18.  One CTA per row; the row is read
// once from HBM (the second pass hits L1/L2).  square, mean, the sum with eps, rsqrt and both products each
// produce a 16-bit tensor in the reference, so each is rounded here; the mean accumulates in fp32.
template <bool BF16>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ w,
                                                      uint8_t* __restrict__ out, int dim, long long x_stride,
                                                      long long out_stride, float eps) {
  const long long r = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + 2 * r * x_stride);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + 2 * r * out_stride);
  const int nv = dim / 8;
  float acc = 0.0f;
  for (int v = threadIdx.x; v < nv; v += 256) {
    float f[8];
    unpack8<BF16>(xr[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += round16<BF16>(f[i] * f[i]);
  }
  __shared__ float red[8];
  __shared__ float s_r;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    const float var = round16<BF16>(t / static_cast<float>(dim));
    s_r = round16<BF16>(rsqrtf(round16<BF16>(var + eps)));
  }
  __syncthreads();
  const float rs = s_r;
  for (int v = threadIdx.x; v < nv; v += 256) {
    float f[8], g[8];
    unpack8<BF16>(xr[v], f);
    unpack8<BF16>(wr[v], g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = round16<BF16>(f[i] * rs) * g[i];
    orow[v] = pack8<BF16>(f);
  }
}

// Rotate the first `heads` heads (query heads followed by key heads) of every row of the fused projection
// [rows, row_stride] in place: out[:half] = x1*cos - x2*sin, out[half:] = x1*sin + x2*cos with cos|sin taken from
// cache[pos0 + (row % seq_len)] (fp32, [cache_rows, head_dim]); products and sums in fp32 without contraction,
// one rounding to the activation type (model_hub/utils.py:20-106).
template <bool BF16>
__global__ void __launch_bounds__(256) rope_kernel(uint8_t* __restrict__ qkv, long long row_stride, long long rows,
                                                   int seq_len, int heads, int head_dim,
                                                   const float* __restrict__ cache, long long pos0,
                                                   const long long* __restrict__ pos_dev, long long cache_rows) {
  if (pos_dev) pos0 += *pos_dev;
  const int half = head_dim / 2, vec_per_head = half / 8;
  const long long total = rows * heads * vec_per_head;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += 256ll * gridDim.x) {
    const int v = static_cast<int>(idx % vec_per_head);
    const long long rh = idx / vec_per_head;
    const int h = static_cast<int>(rh % heads);
    const long long row = rh / heads;
    long long pos = pos0 + row % seq_len;
    if (pos >= cache_rows) pos = cache_rows - 1;
    uint8_t* base = qkv + 2 * (row * row_stride + static_cast<long long>(h) * head_dim + v * 8);
    const float4* cs = reinterpret_cast<const float4*>(cache + pos * head_dim + v * 8);
    const float4* sn = reinterpret_cast<const float4*>(cache + pos * head_dim + half + v * 8);
    const float4 c0 = cs[0], c1 = cs[1], s0 = sn[0], s1 = sn[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float a[8], b[8], o1[8], o2[8];
    unpack8<BF16>(*reinterpret_cast<const uint4*>(base), a);
    unpack8<BF16>(*reinterpret_cast<const uint4*>(base + 2 * half), b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o1[i] = __fsub_rn(__fmul_rn(a[i], c[i]), __fmul_rn(b[i], s[i]));
      o2[i] = __fadd_rn(__fmul_rn(a[i], s[i]), __fmul_rn(b[i], c[i]));
    }
    *reinterpret_cast<uint4*>(base) = pack8<BF16>(o1);
    *reinterpret_cast<uint4*>(base + 2 * half) = pack8<BF16>(o2);
  }
}

// out[r, :] = x[r, inter:] * (x[r, :inter] * sigmoid(x[r, :inter])), model_hub/utils.py:4-12; the sigmoid and
// both products are 16-bit tensors in the reference and are rounded as such.  The sigmoid uses the fast exponential
// and reciprocal (relative error ~2^-21, far below the 16-bit rounding that follows): with the exact ones the kernel
// was bound by instructions at half the memory rate.
template <bool BF16>
__global__ void __launch_bounds__(256) silu_mul_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ out,
                                                       long long rows, int inter) {
  const int nv = inter / 8;
  const long long total = rows * nv;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += 256ll * gridDim.x) {
    const long long r = idx / nv;
    const int v = static_cast<int>(idx % nv);
    const uint4* xr = reinterpret_cast<const uint4*>(x + 2 * (r * 2 * inter));
    float g[8], u[8];
    unpack8<BF16>(xr[v], g);
    unpack8<BF16>(xr[nv + v], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = round16<BF16>(__fdividef(1.0f, 1.0f + __expf(-g[i])));
      g[i] = u[i] * round16<BF16>(g[i] * sg);
    }
    reinterpret_cast<uint4*>(out + 2 * (r * inter))[v] = pack8<BF16>(g);
  }
}

// Append one new token per sequence to a layer's K and V caches: cache[b, pos[b], :] = fresh[b, :] for both tensors in
// one launch (cache_hub/flash_attn_cache.py:239-256 does it with two indexed assignments).  pos lives on the
// device (int64), so the call can sit in a captured graph while the positions advance; a position outside
// [0, capacity) is skipped.  Rows are row_elems 16-bit values, moved as 16-byte pieces.
__global__ void __launch_bounds__(256) cache_append_kernel(uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache,
                                                           const uint8_t* __restrict__ k_new, const uint8_t* __restrict__ v_new,
                                                           const long long* __restrict__ pos, long long cache_seq_stride,
                                                           long long cache_row_stride, long long new_seq_stride, int batch,
                                                           int row_elems, long long capacity) {
  const int vec = row_elems / 8;
  for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < 2 * batch * vec; idx += gridDim.x * blockDim.x) {
    const int which = idx / (batch * vec), rem = idx % (batch * vec);
    const int b = rem / vec, c = rem % vec;
    const long long at = pos[b];
    if (at < 0 || at >= capacity) continue;
    const uint8_t* src = (which ? v_new : k_new) + 2 * (b * new_seq_stride) + 16 * c;
    uint8_t* dst = (which ? v_cache : k_cache) + 2 * (b * cache_seq_stride + at * cache_row_stride) + 16 * c;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
}

}  // namespace sq
