// Cross-GPU merge of split-KV decode partials over peer memory (NVLink), one kernel per decode call:
// every rank holds (O_r, LSE_r) of its key shard for all rows (b, h) - given, or merged here from the split-KV
// partials its decode kernel has just written; a CTA takes one row, stores it straight into the slot `rank` of
// EVERY rank's gather buffer (plain peer stores), publishes a per-row flag on every rank, waits (bounded) until
// the same row of every other rank has been published, and merges the W partials
//   O = sum_r 2^(LSE_r - max) O_r / sum_r 2^(LSE_r - max),  LSE = log2(sum) + max
// in rank order.  There is no dependency between different CTAs, so the kernel cannot deadlock on scheduling;
// the only wait is for the peer GPUs, which run the same kernel for the same decode step.
//
// Buffers (allocated by the host as symmetric memory, one pair per rank, every rank maps all of them):
//   data  float [2][W][rows_cap][D+1]   parity = epoch & 1, so a fast rank's next call never overwrites what a
//                                        slow rank is still reading (a rank finishes call e only after it has
//                                        seen everybody's flag e, i.e. after everybody finished call e-1)
//   flags uint32 [W][rows_cap] + 1      flag[src][row] = last step published for that row by rank src; the extra
//                                        word counts the CTAs of the running launch that have finished
#pragma once
#include "decode.cuh"
#include "prep.cuh"

namespace sq {

constexpr int kPeerMaxWorld = 16;

struct PeerMergeParams {
  float* data[kPeerMaxWorld];        // every rank's data buffer, as mapped in this process
  uint32_t* flags[kPeerMaxWorld];    // every rank's flag buffer
  const float* part_o;               // split_mode 0: [rows, D] this rank's partial; 1: [items, Hq, D] split-KV partials
  const float* part_lse;             // [rows] / [items, Hq]
  void* out;                         // [rows, D] in o_dtype
  float* lse;                        // optional [rows]
  int rank, world, rows, rows_cap, d, o_dtype;
  int split_mode, hq;                // split_mode 1: row (b, h) owns items item_prefix[b] .. item_prefix[b+1]-1
  uint32_t* epoch_ptr;               // device step counter: this launch is step *epoch_ptr + 1 and stores it at its end
  uint32_t* done;                    // CTAs of this launch that have finished (the last one advances the counter)
  int item_prefix[kDecMaxBatch + 1];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One CTA per output row (b, h), 128 * kMergeGroups threads.
__global__ void __launch_bounds__(128 * kMergeGroups) peer_merge_kernel(const __grid_constant__ PeerMergeParams p) {
  __shared__ float w_s[kMergeMaxParts];
  __shared__ float red_s[kMergeGroups][128];
  __shared__ float max_s[32];
  __shared__ int abort_s;
  const uint32_t epoch = *p.epoch_ptr + 1u;   // stored back by the last CTA of this launch
  const int tid = threadIdx.x, nthr = blockDim.x, row = blockIdx.x;
  const int dp = p.d + 1;
  const size_t parity_off = static_cast<size_t>(epoch & 1u) * p.world * p.rows_cap * dp;
  if (tid == 0) abort_s = device_failed() ? 1 : 0;   // an earlier failure on this device: no exchange, NaN out
  __syncthreads();
  const bool skip = abort_s != 0;

  // 0. this rank's partial of the row: given, or merged here from the split-KV partials of the decode kernel
  //    (same arithmetic and summation order as decode_merge_kernel)
  float my_val = 0.f, my_lse = -INFINITY;
  if (!p.split_mode) {
    if (tid < p.d) my_val = p.part_o[static_cast<size_t>(row) * p.d + tid];
    my_lse = p.part_lse[row];
  } else {
    const int b = row / p.hq, h = row % p.hq;
    const int first = p.item_prefix[b], count = p.item_prefix[b + 1] - first;
    const long long base_row = static_cast<long long>(first) * p.hq + h, part_stride = p.hq;
    float mloc = -INFINITY;
    for (int i = tid; i < count; i += nthr) mloc = fmaxf(mloc, p.part_lse[base_row + i * part_stride]);
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    if ((tid & 31) == 0) max_s[tid >> 5] = mloc;
    __syncthreads();
    float mmax = -INFINITY;
    for (int i = 0; i < (nthr + 31) / 32; ++i) mmax = fmaxf(mmax, max_s[i]);
    float den = 0.f;
    for (int base = 0; base < count; base += kMergeMaxParts) {
      const int cnt = min(kMergeMaxParts, count - base);
      __syncthreads();
      for (int i = tid; i < cnt; i += nthr) {
        const float lse_i = p.part_lse[base_row + (base + i) * part_stride];
        w_s[i] = (lse_i == -INFINITY) ? 0.f : exp2f(lse_i - mmax);
      }
      __syncthreads();
      for (int i = 0; i < cnt; ++i) den += w_s[i];
      const int col = tid % 128, grp = tid / 128;
      if (col < p.d) {
        float acc = (base == 0) ? 0.f : red_s[grp][col];
        for (int i = grp; i < cnt; i += kMergeGroups) acc += w_s[i] * p.part_o[(base_row + (base + i) * part_stride) * p.d + col];
        red_s[grp][col] = acc;
      }
    }
    __syncthreads();
    if (tid < p.d) {
      float acc = 0.f;
#pragma unroll
      for (int g = 0; g < kMergeGroups; ++g) acc += (count > 0 && g < nthr / 128) ? red_s[g][tid] : 0.f;
      my_val = (den > 0.f) ? acc / den : (den == den ? 0.f : den);
    }
    my_lse = (den > 0.f) ? log2f(den) + mmax : (den == den ? -INFINITY : den);
  }

  // 1. the row into slot `rank` of every rank's buffer
  for (int w = 0; w < p.world && !skip; ++w) {
    float* dst = p.data[w] + parity_off + (static_cast<size_t>(p.rank) * p.rows_cap + row) * dp;
    if (tid < p.d) dst[tid] = my_val;
    if (tid == 0) dst[p.d] = my_lse;
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish, 3. wait for the same row of every rank (bounded: one second, then the status word is set)
  if (tid < p.world && !skip) {
    st_release_sys(p.flags[tid] + static_cast<size_t>(p.rank) * p.rows_cap + row, epoch);
    const uint32_t* mine = p.flags[p.rank] + static_cast<size_t>(tid) * p.rows_cap + row;
    const uint64_t t0 = globaltimer_ns();
    bool ok = true;
    // epochs only grow; a difference interpreted as signed tolerates wrap-around
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (globaltimer_ns() - t0 > kWaitLimitNs) { ok = false; break; }
      __nanosleep(64);
    }
    if (!ok) {
      abort_s = 1;
      record_failure(301);
    }
  }
  __syncthreads();
  // 4. merge in rank order; the buffer was written by other GPUs: read it around L1
  if (!abort_s) {
    const float* src = p.data[p.rank] + parity_off;
    float mmax = -INFINITY;
    for (int w = 0; w < p.world; ++w) mmax = fmaxf(mmax, __ldcv(src + (static_cast<size_t>(w) * p.rows_cap + row) * dp + p.d));
    float den = 0.f, acc = 0.f;
    for (int w = 0; w < p.world; ++w) {
      const float* rw = src + (static_cast<size_t>(w) * p.rows_cap + row) * dp;
      const float l = __ldcv(rw + p.d);
      const float wt = (l == -INFINITY) ? 0.f : exp2f(l - mmax);
      den += wt;
      if (tid < p.d) acc += wt * __ldcv(rw + tid);
    }
    if (tid < p.d) {
      const float val = (den > 0.f) ? acc / den : (den == den ? 0.f : den);
      const size_t off = static_cast<size_t>(row) * p.d + tid;
      if (p.o_dtype) reinterpret_cast<uint16_t*>(p.out)[off] = from_f32<true>(val);
      else reinterpret_cast<uint16_t*>(p.out)[off] = from_f32<false>(val);
    }
    if (tid == 0 && p.lse) p.lse[row] = (den > 0.f) ? log2f(den) + mmax : -INFINITY;
  } else {
    // the wait gave up (or an earlier one on this device did): the row is marked invalid
    if (tid < p.d) reinterpret_cast<uint16_t*>(p.out)[static_cast<size_t>(row) * p.d + tid] = p.o_dtype ? 0x7fc0 : 0x7e00;
    if (tid == 0 && p.lse) p.lse[row] = __int_as_float(0x7fc00000);
  }
  // 5. the last CTA of the launch advances the step counter (every CTA has read it by now)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
      *p.done = 0u;
      *p.epoch_ptr = epoch;
      __threadfence();
    }
  }
}

}  // namespace sq
