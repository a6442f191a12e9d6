// Cross-GPU merge of split-KV decode partials over peer memory (NVLink), one kernel per decode call:
// every rank holds (O_r, LSE_r) of its key shard for all rows (b, h); a CTA takes four rows, stores them
// straight into the slot `rank` of EVERY rank's gather buffer (plain peer stores), publishes a per-CTA flag on
// every rank, waits (bounded) until the same CTA of every other rank has published, and merges the W partials
//   O = sum_r 2^(LSE_r - max) O_r / sum_r 2^(LSE_r - max),  LSE = log2(sum) + max
// in rank order.  There is no dependency between different CTAs, so the kernel cannot deadlock on scheduling;
// the only wait is for the peer GPUs, which run the same kernel for the same decode step.
//
// Buffers (allocated by the host as symmetric memory, one pair per rank, every rank maps all of them):
//   data  float [2][W][rows_cap][D+1]   parity = epoch & 1, so a fast rank's next call never overwrites what a
//                                        slow rank is still reading (a rank finishes call e only after it has
//                                        seen everybody's flag e, i.e. after everybody finished call e-1)
//   flags uint32 [W][ctas_cap]          flag[src][cta] = last epoch published by that CTA of rank src
#pragma once
#include "prep.cuh"

namespace sq {

constexpr int kPeerMaxWorld = 16;
constexpr int kPeerRowsPerCta = 4;

struct PeerMergeParams {
  float* data[kPeerMaxWorld];        // every rank's data buffer, as mapped in this process
  uint32_t* flags[kPeerMaxWorld];    // every rank's flag buffer
  const float* part_o;               // [rows, D] this rank's partial
  const float* part_lse;             // [rows]
  void* out;                         // [rows, D] in o_dtype
  float* lse;                        // optional [rows]
  int rank, world, rows, rows_cap, ctas_cap, d, o_dtype;
  const uint32_t* epoch_ptr;          // the step counter lives on the device so that a captured graph can be replayed
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void peer_epoch_advance_kernel(uint32_t* epoch) { *epoch += 1u; }

__global__ void __launch_bounds__(128) peer_merge_kernel(const __grid_constant__ PeerMergeParams p) {
  __shared__ int abort_s;
  const uint32_t epoch = *p.epoch_ptr;  // written by the advance kernel launched just before, on the same stream
  const int tid = threadIdx.x, cta = blockIdx.x;
  const int row0 = cta * kPeerRowsPerCta;
  const int nrows = min(kPeerRowsPerCta, p.rows - row0);
  const int dp = p.d + 1;
  const size_t parity_off = static_cast<size_t>(epoch & 1u) * p.world * p.rows_cap * dp;
  if (tid == 0) abort_s = 0;
  // 1. this rank's rows into slot `rank` of every rank's buffer
  for (int w = 0; w < p.world; ++w) {
    float* dst = p.data[w] + parity_off + (static_cast<size_t>(p.rank) * p.rows_cap + row0) * dp;
    for (int r = 0; r < nrows; ++r) {
      for (int c = tid; c < p.d; c += blockDim.x) dst[r * dp + c] = p.part_o[static_cast<size_t>(row0 + r) * p.d + c];
      if (tid == 0) dst[r * dp + p.d] = p.part_lse[row0 + r];
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. publish, 3. wait for the same CTA of every rank (bounded: one second, then the status word is set)
  if (tid < p.world) {
    st_release_sys(p.flags[tid] + static_cast<size_t>(p.rank) * p.ctas_cap + cta, epoch);
    const uint32_t* mine = p.flags[p.rank] + static_cast<size_t>(tid) * p.ctas_cap + cta;
    const uint64_t t0 = globaltimer_ns();
    bool ok = true;
    // epochs only grow; a difference interpreted as signed tolerates wrap-around
    while (static_cast<int32_t>(ld_acquire_sys(mine) - epoch) < 0) {
      if (globaltimer_ns() - t0 > kWaitLimitNs) { ok = false; break; }
      __nanosleep(64);
    }
    if (!ok) {
      abort_s = 1;
      atomicCAS(&g_device_status, 0, 301);
    }
  }
  __syncthreads();
  if (abort_s) return;
  // 4. merge in rank order; the buffer was written by other GPUs: read it around L1
  const float* src = p.data[p.rank] + parity_off;
  for (int r = 0; r < nrows; ++r) {
    const int row = row0 + r;
    float mmax = -INFINITY;
    for (int w = 0; w < p.world; ++w) mmax = fmaxf(mmax, __ldcv(src + (static_cast<size_t>(w) * p.rows_cap + row) * dp + p.d));
    float den = 0.f;
    for (int w = 0; w < p.world; ++w) {
      const float l = __ldcv(src + (static_cast<size_t>(w) * p.rows_cap + row) * dp + p.d);
      den += (l == -INFINITY) ? 0.f : exp2f(l - mmax);
    }
    for (int c = tid; c < p.d; c += blockDim.x) {
      float acc = 0.f;
      for (int w = 0; w < p.world; ++w) {
        const float* rw = src + (static_cast<size_t>(w) * p.rows_cap + row) * dp;
        const float l = __ldcv(rw + p.d);
        const float wt = (l == -INFINITY) ? 0.f : exp2f(l - mmax);
        acc += wt * __ldcv(rw + c);
      }
      const float val = (den > 0.f) ? acc / den : 0.f;
      const size_t off = static_cast<size_t>(row) * p.d + c;
      if (p.o_dtype) reinterpret_cast<uint16_t*>(p.out)[off] = from_f32<true>(val);
      else reinterpret_cast<uint16_t*>(p.out)[off] = from_f32<false>(val);
    }
    if (tid == 0 && p.lse) p.lse[row] = (den > 0.f) ? log2f(den) + mmax : -INFINITY;
  }
}

}  // namespace sq
