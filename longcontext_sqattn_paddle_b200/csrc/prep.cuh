// Elementwise / row-reduction kernels around the attention kernels: q pre-scaling, bf16->f16 copy of V,
// K-mean centring and the fake quantisers of the adapter (sqattn/attn_replacer.py:334-365,
// sqattn/fake_quant.py).  All of them are HBM-bound streaming passes with 16-byte accesses.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace sq {

constexpr float kLog2e = 1.44269504f;  // the literal the reference launchers use

template <bool BF16>
__device__ __forceinline__ float to_f32(uint16_t v) {
  if (BF16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
  return __half2float(__ushort_as_half(v));
}
template <bool BF16>
__device__ __forceinline__ uint16_t from_f32(float f) {
  if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  return __half_as_ushort(__float2half_rn(f));
}
template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = to_f32<BF16>(static_cast<uint16_t>(w[i] & 0xffffu));
    f[2 * i + 1] = to_f32<BF16>(static_cast<uint16_t>(w[i] >> 16));
  }
}
template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = static_cast<uint32_t>(from_f32<BF16>(f[2 * i])) | (static_cast<uint32_t>(from_f32<BF16>(f[2 * i + 1])) << 16);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

struct View4 {  // [B,H,N,D] through element strides
  const uint8_t* ptr;
  long long sb, sh, sn;
  int b, h, n, d;
};
struct OutStrides {  // element strides of an output [B,H,N,D] (contiguous HND or token-major NHD)
  long long sb, sh, sn;
};

// out (contiguous [B,H,N,D]) = f(in): kOp 0: x * scale rounded to the input dtype (q pre-scaling,
// attn_triton_mix_relative.py:383-385); kOp 1: bf16 -> f16 (the kernel-side v.to(fp16), attn_triton.py:84).
template <bool BF16, int kOp>
__global__ void strided_map_kernel(View4 in, uint8_t* out, float scale) {
  const int d8 = in.d / 8;
  const long long total = static_cast<long long>(in.b) * in.h * in.n * d8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % d8);
    long long r = idx / d8;
    const int n = static_cast<int>(r % in.n);
    r /= in.n;
    const int h = static_cast<int>(r % in.h);
    const int b = static_cast<int>(r / in.h);
    const uint4 v = *reinterpret_cast<const uint4*>(in.ptr + 2 * (b * in.sb + h * in.sh + n * in.sn + c * 8));
    float f[8];
    unpack8<BF16>(v, f);
    uint4 o;
    if (kOp == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] *= scale;
      o = pack8<BF16>(f);
    } else {
      o = pack8<false>(f);
    }
    *reinterpret_cast<uint4*>(out + idx * 16) = o;
  }
}

// ---- K mean over the sequence, deterministic two-phase reduction -------------------------------------
constexpr int kMeanChunks = 64;

// partial[bh][chunk][d] = sum over the chunk's rows of k[b, n, h, d]
template <bool BF16>
__global__ void kmean_partial_kernel(View4 k, float* partial) {
  const int bh = blockIdx.y, chunk = blockIdx.x;
  const int b = bh / k.h, h = bh % k.h;
  const int d8 = k.d / 8, lanes = blockDim.x / d8;
  const int c = threadIdx.x % d8, rl = threadIdx.x / d8;
  const int rows_per = (k.n + kMeanChunks - 1) / kMeanChunks;
  const int r0 = chunk * rows_per, r1 = min(k.n, r0 + rows_per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (rl < lanes) {
    for (int n = r0 + rl; n < r1; n += lanes) {
      const uint4 v = *reinterpret_cast<const uint4*>(k.ptr + 2 * (b * k.sb + h * k.sh + n * k.sn + c * 8));
      float f[8];
      unpack8<BF16>(v, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
  extern __shared__ float red[];  // [lanes][d]
  if (rl < lanes) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * k.d + c * 8 + i] = acc[i];
  }
  __syncthreads();
  if (threadIdx.x < k.d) {
    float s = 0.f;
    for (int j = 0; j < lanes; ++j) s += red[j * k.d + threadIdx.x];
    partial[(static_cast<long long>(bh) * kMeanChunks + chunk) * k.d + threadIdx.x] = s;
  }
}
// mean[bh][d] = (sum of the partials in chunk order) / n; n == 0 stores the plain column sums (the
// sequence-parallel path all-reduces the sums of the shards before dividing)
__global__ void kmean_final_kernel(const float* partial, float* mean, int d, int n) {
  const int bh = blockIdx.x;
  if (threadIdx.x < d) {
    float s = 0.f;
    for (int c = 0; c < kMeanChunks; ++c) s += partial[(static_cast<long long>(bh) * kMeanChunks + c) * d + threadIdx.x];
    mean[bh * d + threadIdx.x] = n > 0 ? s / static_cast<float>(n) : s;
  }
}

// ---- fake quantisers ---------------------------------------------------------------------------------
__device__ __forceinline__ float round_mode(float x, int half_even) { return half_even ? rintf(x) : roundf(x); }

// float_quantize of the reference (fake_quant.py:151-204) with its quirks: no subnormals, the mantissa
// never carries into the next binade, exponent clipped to 2^(e-1)-1.
__device__ __forceinline__ float float_quantize_dev(float x, int e_bits, int m_bits, int half_even) {
  const int bias = (1 << (e_bits - 1)) - 1;
  const float eps = exp2f(-static_cast<float>(m_bits));
  const float max_exp = static_cast<float>((1 << (e_bits - 1)) - 1);
  const float min_exp = static_cast<float>(1 - bias);
  const float sign = (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : 0.f);
  const float a = fabsf(x);
  if (a == 0.f) return 0.f;
  const float ex = floorf(log2f(a + 1e-30f));
  const float frac = __fdiv_rn(a, exp2f(ex)) - 1.0f;
  const float exc = fminf(fmaxf(ex, min_exp), max_exp);
  float fq = round_mode(__fdiv_rn(frac, eps), half_even) * eps;
  fq = fminf(fmaxf(fq, 0.0f), 1.0f - eps);
  float xq = (1.0f + fq) * exp2f(exc) * sign;
  const float max_val = (2.0f - eps) * exp2f(max_exp);
  return fminf(fmaxf(xq, -max_val), max_val);
}

// quant -> dequant of one value given the row's absmax (clipped at 1e-5).
//   qtype 0: integer grid with `qmax` (127 / 7), clamp to [-qmax-1, qmax]  (fake_quant.py:114-125)
//   qtype 1/2: emulated e4m3 / e5m2                                         (fake_quant.py:231-248)
__device__ __forceinline__ float fake_quant_value(float x, float absmax, int qtype, float qmax, int half_even) {
  if (qtype == SQATTN_QTYPE_INT) {
    const float scale = __fdiv_rn(absmax, qmax);
    float q = round_mode(__fdiv_rn(x, scale), half_even);
    q = fminf(fmaxf(q, -qmax - 1.0f), qmax);
    return q * scale;
  }
  const float fmax = (qtype == SQATTN_QTYPE_E4M3) ? 448.0f : 57344.0f;
  const float scale = __fdiv_rn(absmax, fmax);
  float s = fminf(fmaxf(__fdiv_rn(x, scale), -fmax), fmax);
  s = float_quantize_dev(s, qtype == SQATTN_QTYPE_E4M3 ? 4 : 5, qtype == SQATTN_QTYPE_E4M3 ? 3 : 2, half_even);
  return s * scale;
}

// Integer grid, fast path for 8 values of one row: q = x * (1/scale) is within 2e-5 of the exact quotient
// x / scale (|q| <= qmax * (1 + 2^-22), so the clamp of the reference never acts), hence unless q lies within
// 1e-4 of a half-integer its nearest integer IS round(x / scale) in either rounding mode; a group with such a
// value (rare) is redone with exact divisions.  Results are identical to fake_quant_value(..., INT, ...).
__device__ __forceinline__ void fake_quant_int8x(const float (&x)[8], float absmax, float qmax, int half_even, float (&out)[8]) {
  const float scale = __fdiv_rn(absmax, qmax), inv = __fdiv_rn(1.0f, scale);
  float worst = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float q = x[i] * inv, r = rintf(q);
    worst = fmaxf(worst, fabsf(q - r));
    out[i] = r * scale;
  }
  if (worst > 0.4999f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = fake_quant_value(x[i], absmax, SQATTN_QTYPE_INT, qmax, half_even);
  }
}

// The integer grid for the 8 values a thread holds of one row, on packed fp32 pairs, returning the 8 results
// rounded to the 16-bit type (and, for queries, multiplied by q_scale and rounded again) as four packed words.
// Every operation is the IEEE round-to-nearest one of the scalar path above, so the bits are the same.
template <bool BF16, bool kScale>
__device__ __forceinline__ uint4 fake_quant_int_row8(const float (&x)[8], float absmax, float qmax, int half_even, float q_scale) {
  const float scale = __fdiv_rn(absmax, qmax), inv = __fdiv_rn(1.0f, scale);
  const uint64_t inv2 = f32x2_pack(inv, inv), sc2 = f32x2_pack(scale, scale), qs2 = f32x2_pack(q_scale, q_scale);
  float g[8];
  float worst = 0.f;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint64_t q2 = f32x2_mul(f32x2_pack(x[2 * p], x[2 * p + 1]), inv2);
    float q0, q1, d0, d1;
    f32x2_unpack(q2, q0, q1);
    const float r0 = rintf(q0), r1 = rintf(q1);
    const uint64_t r2 = f32x2_pack(r0, r1);
    f32x2_unpack(f32x2_sub(q2, r2), d0, d1);
    worst = fmaxf(worst, fmaxf(fabsf(d0), fabsf(d1)));
    f32x2_unpack(f32x2_mul(r2, sc2), g[2 * p], g[2 * p + 1]);
  }
  if (worst > 0.4999f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = fake_quant_value(x[i], absmax, SQATTN_QTYPE_INT, qmax, half_even);
  }
  uint32_t w[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint32_t v = BF16 ? pack_bf16x2(g[2 * p], g[2 * p + 1]) : pack_f16x2(g[2 * p], g[2 * p + 1]);
    if (kScale) {
      float a, b;
      if (BF16) {
        a = __uint_as_float(v << 16);
        b = __uint_as_float(v & 0xffff0000u);
      } else {
        const __half2 h2 = *reinterpret_cast<const __half2*>(&v);
        a = __low2float(h2);
        b = __high2float(h2);
      }
      f32x2_unpack(f32x2_mul(f32x2_pack(a, b), qs2), a, b);
      v = BF16 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
    }
    w[p] = v;
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Per-token fake-quant of Q or K.  Input [B,N,H,D] via strides, outputs contiguous [B,H,N,D].
// kIsK: subtract the (dtype-rounded) sequence mean first, no scaling of the result.
// Q: results are multiplied by 1/sqrt(D)*log2e in the input dtype.
// One 16-lane group per row (D = 128) or one 8-lane group (D = 64); 16-byte loads and stores.
template <bool BF16, bool kIsK>
__global__ void __launch_bounds__(256)
quant_rows_kernel(View4 x, const float* mean, uint8_t* out8, uint8_t* out4, OutStrides os, int qtype, int half_even,
                  float q_scale) {
  constexpr int kUnroll = 4;  // rows in flight per lane group: four independent 16-byte loads per thread
  const int d8 = x.d / 8;
  const int rows_per_block = blockDim.x / d8;
  const int c = threadIdx.x % d8;
  const unsigned grp_mask = (d8 == 16) ? (0xffffu << ((threadIdx.x & 16) ? 16 : 0)) : (0xffu << ((threadIdx.x & 31) / 8 * 8));
  // grid: x walks the tokens of one (batch, head) pair, y = b * H + h
  const int b = static_cast<int>(blockIdx.y) / x.h, h = static_cast<int>(blockIdx.y) % x.h;
  const uint8_t* in_base = x.ptr + 2 * (b * x.sb + h * x.sh + c * 8);
  const long long out_base = (b * os.sb + h * os.sh + c * 8) * 2;
  float mvals[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (kIsK) {
    const float* m = mean + (static_cast<long long>(b) * x.h + h) * x.d + c * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) mvals[i] = to_f32<BF16>(from_f32<BF16>(m[i]));
  }
  const int step = static_cast<int>(gridDim.x) * rows_per_block * kUnroll;
  for (int n0 = static_cast<int>(blockIdx.x) * rows_per_block * kUnroll + threadIdx.x / d8; n0 < x.n; n0 += step) {
    uint4 raw[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int n = n0 + u * rows_per_block;
      live[u] = n < x.n;
      raw[u] = *reinterpret_cast<const uint4*>(in_base + 2 * (static_cast<long long>(live[u] ? n : 0) * x.sn));
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float f[8];
      unpack8<BF16>(raw[u], f);
      if (kIsK) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = to_f32<BF16>(from_f32<BF16>(f[i] - mvals[i]));
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      for (int o = d8 / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(grp_mask, amax, o));
      amax = fmaxf(amax, 1e-5f);
      if (live[u]) {
        const long long ooff = out_base + static_cast<long long>(n0 + u * rows_per_block) * os.sn * 2;
        if (qtype == SQATTN_QTYPE_INT) {
          *reinterpret_cast<uint4*>(out8 + ooff) = fake_quant_int_row8<BF16, !kIsK>(f, amax, 127.0f, half_even, q_scale);
        } else {
          float g[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            g[i] = to_f32<BF16>(from_f32<BF16>(fake_quant_value(f[i], amax, qtype, 127.0f, half_even)));
            if (!kIsK) g[i] *= q_scale;
          }
          *reinterpret_cast<uint4*>(out8 + ooff) = pack8<BF16>(g);
        }
        if (out4) *reinterpret_cast<uint4*>(out4 + ooff) = fake_quant_int_row8<BF16, !kIsK>(f, amax, 7.0f, half_even, q_scale);
      }
    }
  }
}

// "per_channel" fake-quant of V: one range per (token, channel), taken over batch and heads
// (fake_quant.py:30-32 with a [B,H,N,D] tensor).  Output contiguous [B,H,N,D] in f16.
template <bool BF16>
__global__ void quant_v_kernel(View4 v, uint8_t* out, OutStrides os, int qtype, int half_even) {
  const int d8 = v.d / 8;
  const long long total = static_cast<long long>(v.n) * d8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % d8);
    const int n = static_cast<int>(idx / d8);
    float amax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < v.b; ++b)
      for (int h = 0; h < v.h; ++h) {
        float f[8];
        unpack8<BF16>(*reinterpret_cast<const uint4*>(v.ptr + 2 * (b * v.sb + h * v.sh + n * v.sn + c * 8)), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax[i] = fmaxf(amax[i], fabsf(f[i]));
      }
#pragma unroll
    for (int i = 0; i < 8; ++i) amax[i] = fmaxf(amax[i], 1e-5f);
    for (int b = 0; b < v.b; ++b)
      for (int h = 0; h < v.h; ++h) {
        float f[8];
        unpack8<BF16>(*reinterpret_cast<const uint4*>(v.ptr + 2 * (b * v.sb + h * v.sh + n * v.sn + c * 8)), f);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          f[i] = to_f32<BF16>(from_f32<BF16>(fake_quant_value(f[i], amax[i], qtype, 127.0f, half_even)));
        *reinterpret_cast<uint4*>(out + (b * os.sb + h * os.sh + n * os.sn + c * 8) * 2) = pack8<false>(f);
      }
  }
}

}  // namespace sq
