// Cross-GPU merge of split-KV decode partials over peer memory (NVLink), one kernel per decode call:
// every rank holds (O_r, LSE_r) of its key shard for all rows (b, h) - given, or merged here from the split-KV
// partials its decode kernel has just written; a CTA takes one row, stores it straight into the slot `rank` of
// EVERY rank's gather buffer (plain peer stores), waits (bounded) until the same row of every other rank has
// arrived in its own buffer, and merges the W partials
//   O = sum_r 2^(LSE_r - max) O_r / sum_r 2^(LSE_r - max),  LSE = log2(sum) + max
// in rank order.  There is no dependency between different CTAs, so the kernel cannot deadlock on scheduling;
// the only wait is for the peer GPUs, which run the same kernel for the same decode step.
//
// The exchange is latency bound (14 KB per rank), so every value travels as ONE 8-byte word {fp32 bits, step
// number}: an aligned 8-byte store is indivisible, so a receiver that reads the current step number in a word
// also has that word's value.  No fence, no separate flag and no second trip over the link are needed; the cost
// of the exchange is one one-way store latency after the slowest rank has produced its row.
//
// Buffers (allocated by the host as symmetric memory, one pair per rank, every rank maps all of them):
//   data  uint64 [2][W][rows_cap][D+1]  parity = step & 1, so a fast rank's next call never overwrites what a
//                                        slow rank is still reading (a rank finishes call e only after it has
//                                        seen everybody's words of step e, i.e. after everybody finished call e-1)
//   flags uint32 [W][rows_cap] + 1      only the last word is used: it counts the CTAs of the running launch that
//                                        have finished (the rest is kept for callers that sized it that way)
#pragma once
#include "decode.cuh"
#include "prep.cuh"

namespace sq {

constexpr int kPeerMaxWorld = 16;

struct PeerMergeParams {
  unsigned long long* data[kPeerMaxWorld];  // every rank's data buffer, as mapped in this process
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

#ifdef SQATTN_DEBUG_EXPORTS
// debug builds only: globaltimer stamps of CTA 0, [call % 64][8]
__device__ long long* g_peer_stamps = nullptr;
#define SQ_PEER_STAMP(slot)                                                                                   \
  do {                                                                                                        \
    if (g_peer_stamps && blockIdx.x == 0 && threadIdx.x == 0) g_peer_stamps[(epoch & 63u) * 8 + (slot)] = globaltimer_ns(); \
  } while (0)
#else
#define SQ_PEER_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One CTA per output row (b, h), 128 * kMergeGroups threads.
__global__ void __launch_bounds__(128 * kMergeGroups) peer_merge_kernel(const __grid_constant__ PeerMergeParams p) {
  __shared__ MergeScratch sm;
  __shared__ float got_s[kPeerMaxWorld][132];
  __shared__ volatile int abort_s;
  griddep_launch();
  griddep_wait();  // the split-KV partials, the step counter and the status word come from earlier kernels
  const uint32_t epoch = *p.epoch_ptr + 1u;   // stored back by the last CTA of this launch
  const int tid = threadIdx.x, nthr = blockDim.x, row = blockIdx.x;
  const int dp = p.d + 1;
  const size_t parity_off = static_cast<size_t>(epoch & 1u) * p.world * p.rows_cap * dp;
  SQ_PEER_STAMP(0);
#ifdef SQATTN_DEBUG_EXPORTS
  if (g_peer_stamps && blockIdx.x == 0 && tid == 0) {   // span of the decode launch that fed this merge
    g_peer_stamps[(epoch & 63u) * 8 + 5] = static_cast<long long>(g_dec_first);
    g_peer_stamps[(epoch & 63u) * 8 + 6] = static_cast<long long>(g_dec_last);
    g_dec_first = ~0ull;
    g_dec_last = 0ull;
  }
#endif
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
    merge_row_partials(p.part_o, p.part_lse, static_cast<long long>(first) * p.hq + h, p.hq, count, p.d, sm, my_val, my_lse);
  }
  SQ_PEER_STAMP(1);
  // 1. the row into slot `rank` of every rank's buffer, each value tagged with the step number
  if (tid < dp && !skip) {
    const unsigned long long word = (static_cast<unsigned long long>(epoch) << 32) |
                                    __float_as_uint(tid < p.d ? my_val : my_lse);
    for (int w = 0; w < p.world; ++w)
      st_relaxed_sys_u64(p.data[w] + parity_off + (static_cast<size_t>(p.rank) * p.rows_cap + row) * dp + tid, word);
  }
  SQ_PEER_STAMP(2);
  // 2. collect the same row of every rank from this rank's buffer (bounded: one second, then the status word is set)
  if (!skip) {
    const unsigned long long* mine = p.data[p.rank] + parity_off;
    const uint64_t t0 = globaltimer_ns();
    for (int idx = tid; idx < p.world * dp; idx += nthr) {
      const int w = idx / dp, c = idx - w * dp;
      const unsigned long long* src = mine + (static_cast<size_t>(w) * p.rows_cap + row) * dp + c;
      unsigned long long word = ld_relaxed_sys_u64(src);
      uint32_t spins = 0;
      while (static_cast<uint32_t>(word >> 32) != epoch) {
        if ((++spins & 63u) == 0u && (abort_s || globaltimer_ns() - t0 > kWaitLimitNs)) {
          abort_s = 1;
          record_failure(301);
          break;
        }
        word = ld_relaxed_sys_u64(src);
      }
      got_s[w][c] = __uint_as_float(static_cast<uint32_t>(word));
    }
  }
  __syncthreads();
  SQ_PEER_STAMP(3);
  // 3. merge in rank order
  if (!abort_s) {
    float mmax = -INFINITY;
    for (int w = 0; w < p.world; ++w) mmax = fmaxf(mmax, got_s[w][p.d]);
    float den = 0.f, acc = 0.f;
    for (int w = 0; w < p.world; ++w) {
      const float l = got_s[w][p.d];
      const float wt = (l == -INFINITY) ? 0.f : exp2f(l - mmax);
      den += wt;
      if (tid < p.d) acc += wt * got_s[w][tid];
    }
    if (tid < p.d) {
      const float val = (den > 0.f) ? acc / den : (den == den ? 0.f : den);
      const size_t off = static_cast<size_t>(row) * p.d + tid;
      if (p.o_dtype) reinterpret_cast<uint16_t*>(p.out)[off] = from_f32<true>(val);
      else reinterpret_cast<uint16_t*>(p.out)[off] = from_f32<false>(val);
    }
    if (tid == 0 && p.lse) p.lse[row] = (den > 0.f) ? log2f(den) + mmax : (den == den ? -INFINITY : den);
  } else {
    // the wait gave up (or an earlier one on this device did): the row is marked invalid
    if (tid < p.d) reinterpret_cast<uint16_t*>(p.out)[static_cast<size_t>(row) * p.d + tid] = p.o_dtype ? 0x7fc0 : 0x7e00;
    if (tid == 0 && p.lse) p.lse[row] = __int_as_float(0x7fc00000);
  }
  // 4. the last CTA of the launch advances the step counter (every CTA has read it by now)
  __syncthreads();
  SQ_PEER_STAMP(4);
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
