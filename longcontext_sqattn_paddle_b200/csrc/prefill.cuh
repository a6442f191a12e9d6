// Causal GQA prefill attention for sm_100a: dense causal and the sink + hierarchical-window variants.
//
// One CTA owns 128 query rows of one head.  Warp roles:
//   warp 0      TMA producer: Q tile once (again when the operand set changes), K / V tiles per 64-key step
//   warp 1      tcgen05 issuer: S = Q K^T (smem x smem -> TMEM), O += P V (TMEM x smem -> TMEM); owns TMEM
//   warps 2..5  online softmax, one query row per thread (TMEM lane), P written back over S in TMEM as f16
// The step order, the 64-key max/sum update and the f16 (optionally e4m3-rounded) P are those of the
// reference tile loop (sqattn/attn_triton_mix_relative.py:76-98 == sqattn/attn_triton.py:64-86).
#pragma once
#include <cuda.h>

#include "prep.cuh"
#include "ptx.cuh"

namespace sq {

constexpr int kMaxHeads = 128;
constexpr int kBlockM = 128;  // query rows per CTA (tcgen05 M)
constexpr int kBlockN = 64;   // keys per step (the reference BLOCK_N)
constexpr int kMaxSegs = 12;
constexpr float kLazyLog2 = 8.0f;  // O is rescaled only when a row's maximum has moved by more than 2^8

// segment flags
constexpr int kSegAct0 = 1;   // rows 0..63 of the CTA take part
constexpr int kSegAct1 = 2;   // rows 64..127 take part
constexpr int kSegDiag = 4;   // additive causal mask (stage 4)
constexpr int kSegInt4 = 8;   // reads the int4 operand set (stage 2)
constexpr int kSegFp8 = 16;   // P rounded through e4m3

struct Seg {
  int start;   // first key of the first tile
  int ntiles;  // number of 64-key tiles
  int flags;
};

struct PrefillParams {
  void* o;
  long long o_sb, o_sh, o_sn;
  float* lse;
  float* dump;  // debug builds only: S tiles of CTA 0
  float* dump_p;  // debug builds only: the P tiles CTA 0 hands to the tensor core (f16 values widened to fp32)
  long long* dump_t;  // debug builds only: clock64 stamps of CTA 0, [step][16]
  int batch, hq, hkv, groups, n, kv_len;
  int mode, sink, p_fp8_mode, o_dtype, qk_bf16, same_opset, nblk;
  // Sequence-parallel shards: the launch's local 128-row blocks [0, blk_split) are blocks blk0.. of the whole
  // sequence and the blocks from blk_split on are blocks blk0_b.. (a rank may own two separate row ranges, e.g. the
  // zig-zag split that balances causal work); blk_split == nblk for a single range.
  int blk0, blk_split, blk0_b;
  // Q fake-quantisation inside the kernel: the Q tile arrives as the model produced it and every softmax thread
  // quantises its own row in shared memory before the first MMA (0 = Q is already prepared; else quantiser type + 1)
  int q_fake_quant, q_half_even;
  float q_scale;
  int n_total;  // rows of the whole sequence (a 64-row half that starts at or after it does not exist)
  int w8[kMaxHeads];
  int w4[kMaxHeads];
};

// Key ranges of the four stages for the query block [qs, qe)
// (attn_triton_mix_relative.py:36-75, attn_triton_mix_bad.py:41-74).
__host__ __device__ __forceinline__ void stage_range(int stage, int qs, int qe, int w8, int w4, int sink, int& lo, int& hi) {
  const int l4 = sink > qe - w4 ? sink : qe - w4;
  const int l8 = sink > qe - w8 ? sink : qe - w8;
  lo = hi = 0;
  if (stage == 1) {
    hi = sink < qs ? sink : qs;
  } else if (stage == 2) {
    if (l4 < l8) { lo = l4; hi = l8; }
  } else if (stage == 3) {
    if (l8 < qs) { lo = l8; hi = qs; }
  } else {
    lo = qs; hi = qe;
  }
}

// Builds the CTA's step list.  BLOCK_M = 128 modes (dense, absolute windows) have one schedule for all
// 128 rows.  The relative-window mode has BLOCK_M = 64: the CTA covers two reference blocks whose stage
// ranges are offset by 0 or 64 keys; their tiles are merged stage by stage and each step records which
// half takes part, so every half sees exactly its own tiles in the reference order.
__host__ __device__ inline int build_schedule(Seg* segs, const PrefillParams& p, int blk, int head) {
  int n = 0;
  const int stage_flags_fp8_all = (p.p_fp8_mode == 1) ? kSegFp8 : 0;
  auto flags_of = [&](int stage) {
    int f = stage_flags_fp8_all;
    if (stage == 4) f |= kSegDiag;
    if (stage == 2) {
      if (!p.same_opset) f |= kSegInt4;
      if (p.p_fp8_mode == 2) f |= kSegFp8;
    }
    return f;
  };
  if (p.mode == 0) {
    const int qs = blk * kBlockM;
    if (qs > 0) segs[n++] = Seg{0, qs / kBlockN, kSegAct0 | kSegAct1 | stage_flags_fp8_all};
    segs[n++] = Seg{qs, kBlockM / kBlockN, kSegAct0 | kSegAct1 | kSegDiag | stage_flags_fp8_all};
    return n;
  }
  const int w8 = p.w8[head], w4 = p.w4[head];
  if (p.mode == 2) {
    const int qs = blk * kBlockM, qe = qs + kBlockM;
    for (int stage = 1; stage <= 4; ++stage) {
      int lo, hi;
      stage_range(stage, qs, qe, w8, w4, p.sink, lo, hi);
      if (hi > lo) segs[n++] = Seg{lo, (hi - lo + kBlockN - 1) / kBlockN, kSegAct0 | kSegAct1 | flags_of(stage)};
    }
    return n;
  }
  // relative windows: two 64-row blocks
  const int qs0 = blk * kBlockM, qs1 = qs0 + 64;
  const bool has1 = qs1 < p.n_total;
  for (int stage = 1; stage <= 4; ++stage) {
    int lo0, hi0, lo1 = 0, hi1 = 0;
    stage_range(stage, qs0, qs0 + 64, w8, w4, p.sink, lo0, hi0);
    if (has1) stage_range(stage, qs1, qs1 + 64, w8, w4, p.sink, lo1, hi1);
    const bool e0 = hi0 <= lo0, e1 = hi1 <= lo1;
    if (e0 && e1) continue;
    const int lo = e0 ? lo1 : (e1 ? lo0 : (lo0 < lo1 ? lo0 : lo1));
    const int hi = e0 ? hi1 : (e1 ? hi0 : (hi0 > hi1 ? hi0 : hi1));
    int run_start = 0, run_act = -1, run_len = 0;
    for (int t = lo; t < hi; t += kBlockN) {
      const int act = ((!e0 && t >= lo0 && t < hi0) ? kSegAct0 : 0) | ((!e1 && t >= lo1 && t < hi1) ? kSegAct1 : 0);
      if (act != run_act) {
        if (run_len > 0 && run_act != 0 && n < kMaxSegs) segs[n++] = Seg{run_start, run_len, run_act | flags_of(stage)};
        run_start = t; run_act = act; run_len = 0;
      }
      ++run_len;
    }
    if (run_len > 0 && run_act != 0 && n < kMaxSegs) segs[n++] = Seg{run_start, run_len, run_act | flags_of(stage)};
  }
  return n;
}

template <int D, int KS_, int VS_>
struct PrefillSmem {
  static constexpr int kKStages = KS_;
  static constexpr int kVStages = VS_;
  static constexpr int kQBytes = kBlockM * D * 2;
  static constexpr int kKBytes = kBlockN * D * 2;
  static constexpr int kVBytes = kBlockN * D * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kVOff = kKOff + kKStages * kKBytes;
  static constexpr int kBarOff = kVOff + kVStages * kVBytes;
  // barriers: q_full, q_empty, k_full[KS], v_full[VS], s_full[2], p_full[2], o_tail[2], q_ready
  static constexpr int kNumBars = 2 + kKStages + kVStages + 2 + 2 + 2 + 1;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;
  static constexpr int kSegOff = kMiscOff + 16;  // tmem base, abort flag, nseg
  static constexpr int kTotal = kSegOff + kMaxSegs * 12;
  static constexpr int kDynBytes = kTotal;  // the dynamic shared memory window itself is 1024-byte aligned
};

// Walks the flattened step list.
struct StepIter {
  const Seg* segs;
  int nseg, seg, t;
  __device__ StepIter(const Seg* s, int n) : segs(s), nseg(n), seg(0), t(0) {}
  __device__ bool done() const { return seg >= nseg; }
  __device__ int flags() const { return segs[seg].flags; }
  __device__ int key0() const { return segs[seg].start + t * kBlockN; }
  __device__ bool first_of_seg() const { return t == 0; }
  __device__ bool last_of_seg() const { return t == segs[seg].ntiles - 1; }
  // operand set of the next segment differs from this one's
  __device__ bool opset_changes_after() const {
    return seg + 1 < nseg && ((segs[seg + 1].flags ^ segs[seg].flags) & kSegInt4);
  }
  __device__ bool opset_changed_before() const {
    return seg > 0 && ((segs[seg - 1].flags ^ segs[seg].flags) & kSegInt4);
  }
  __device__ void next() {
    if (++t >= segs[seg].ntiles) { t = 0; ++seg; }
  }
};

// A CTA that cannot deliver its rows (a wait gave up here or earlier on this device) fills them with NaN so
// that the failure cannot pass for a result.
template <int D>
__device__ __forceinline__ void poison_output(const PrefillParams& p, int bi, int head, int blk) {
  const uint32_t nan2 = p.o_dtype ? 0x7fc07fc0u : 0x7e007e00u;
  const uint4 v = make_uint4(nan2, nan2, nan2, nan2);
  for (int idx = threadIdx.x; idx < kBlockM * (D / 8); idx += blockDim.x) {
    const int row_local = blk * kBlockM + idx / (D / 8);
    if (row_local >= p.n) break;
    uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                    2 * (static_cast<long long>(bi) * p.o_sb + static_cast<long long>(head) * p.o_sh +
                         static_cast<long long>(row_local) * p.o_sn);
    reinterpret_cast<uint4*>(orow)[idx % (D / 8)] = v;
    if (p.lse && idx % (D / 8) == 0)
      p.lse[(static_cast<long long>(bi) * p.hq + head) * p.n + row_local] = __int_as_float(0x7fc00000);
  }
}

template <int D, bool kDump, int KS_, int VS_, int kMinCtas>
__global__ void __launch_bounds__(192, kMinCtas)
prefill_kernel(const __grid_constant__ CUtensorMap tm_q8, const __grid_constant__ CUtensorMap tm_q4,
               const __grid_constant__ CUtensorMap tm_k8, const __grid_constant__ CUtensorMap tm_k4,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ PrefillParams p) {
  using L = PrefillSmem<D, KS_, VS_>;
  constexpr int KS = L::kKStages, VS = L::kVStages;
  constexpr uint32_t kTmemCols = 256;  // S0 [0,64) S1 [64,128) O [128,128+D)
  constexpr uint32_t kOCol = 128;
#define SQ_STAMP(step, slot)                                                            \
  do {                                                                                 \
    if (kDump && blockIdx.x == 0 && p.dump_t && (threadIdx.x & 31) == 0) p.dump_t[(step) * 16 + (slot)] = clock64(); \
  } while (0)

  // Heads vary fastest so that the heads of one KV group run together and share K/V tiles in L2;
  // later (for dense causal: longer) query blocks are launched first.
  const int per_blk = p.hq * p.batch;
  const int blk = p.nblk - 1 - static_cast<int>(blockIdx.x) / per_blk;
  const int rem = static_cast<int>(blockIdx.x) % per_blk;
  const int bi = rem / p.hq, head = rem % p.hq, kvh = head / p.groups;
  const int gblk = blk < p.blk_split ? p.blk0 + blk : p.blk0_b + (blk - p.blk_split);  // block of the whole sequence
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  // the 128-byte swizzle needs 1024-byte aligned tiles: refuse to run rather than compute garbage
  if ((sbase & 1023u) && threadIdx.x == 0) record_failure(100);
  // once a wait has given up anywhere on this device, the remaining CTAs (and every later launch, until the host
  // has read and cleared the status word) only mark their rows as invalid
  if ((sbase & 1023u) || device_failed()) {
    poison_output<D>(p, bi, head, blk);
    return;
  }
  const uint32_t q_s = sbase + L::kQOff, k_s = sbase + L::kKOff, v_s = sbase + L::kVOff;
  const uint32_t bars = sbase + L::kBarOff;
  const uint32_t bar_q_full = bars, bar_q_empty = bars + 8;
  static_assert(KS == 2 && VS == 3, "K stages follow the two S buffers; V has one stage more");
  const uint32_t bar_k_full = bars + 16, bar_v_full = bar_k_full + 8 * KS;
  const uint32_t bar_s_full = bar_v_full + 8 * VS, bar_p_full = bar_s_full + 16, bar_o_tail = bar_p_full + 16;
  const uint32_t bar_q_ready = bar_o_tail + 16;
  volatile uint32_t* tmem_base_s = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOff);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  volatile int* nseg_s = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 8);
  Seg* segs = reinterpret_cast<Seg*>(smem + L::kSegOff);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    *nseg_s = build_schedule(segs, p, gblk, head);
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    for (int i = 0; i < KS; ++i) mbar_init(bar_k_full + 8 * i, 1);
    for (int i = 0; i < VS; ++i) mbar_init(bar_v_full + 8 * i, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(bar_s_full + 8 * i, 1); mbar_init(bar_p_full + 8 * i, 128); }
    mbar_init(bar_o_tail, 1);
    mbar_init(bar_o_tail + 8, 1);
    mbar_init(bar_q_ready, 128);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_s)), kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_s;
  const int nseg = *nseg_s;
  int nsteps = 0;
  for (int i = 0; i < nseg; ++i) nsteps += segs[i].ntiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The issuer commits once per step, after Q K^T of step i (barrier s_full(i)); at that point P V of step i-2
    // and everything before it has completed as well (one thread's MMAs complete in issue order).  So s_full
    // doubles as the "stage is free" signal: K stage i & 1 is free at s_full(i-2), V stage i % 3 (last read by
    // P V of step i-3) at s_full(i-1).
    if (lane == 0) {
      tma_prefetch_desc(&tm_q8); tma_prefetch_desc(&tm_k8); tma_prefetch_desc(&tm_v);
      int q_loads = 0;
      int i = 0;
      bool ok = true;
      for (StepIter it(segs, nseg); ok && !it.done(); it.next(), ++i) {
        const bool int4 = it.flags() & kSegInt4;
        if (i == 0 || (it.first_of_seg() && it.opset_changed_before())) {
          if (q_loads > 0) ok = mbar_wait(bar_q_empty, (q_loads - 1) & 1, cta_abort, 101);
          if (!ok) break;
          mbar_expect_tx(bar_q_full, L::kQBytes);
          const CUtensorMap* tq = int4 ? &tm_q4 : &tm_q8;
#pragma unroll
          for (int h = 0; h < D / 64; ++h) tma_load_4d(q_s + h * (kBlockM * 128), tq, bar_q_full, h * 64, blk * kBlockM, head, bi);
          ++q_loads;
        }
        const int st = i & 1, vst = i % 3;
        if (i >= 2) ok = mbar_wait(bar_s_full + 8 * st, ((i - 2) >> 1) & 1, cta_abort, 102);
        if (!ok) break;
        SQ_STAMP(i, 12);
        mbar_expect_tx(bar_k_full + 8 * st, L::kKBytes);
        const CUtensorMap* tk = int4 ? &tm_k4 : &tm_k8;
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(k_s + st * L::kKBytes + h * (kBlockN * 128), tk, bar_k_full + 8 * st, h * 64, it.key0(), kvh, bi);
        if (i >= 3) ok = mbar_wait(bar_s_full + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, cta_abort, 103);
        if (!ok) break;
        SQ_STAMP(i, 13);
        mbar_expect_tx(bar_v_full + 8 * vst, L::kVBytes);
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(v_s + vst * L::kVBytes + h * (kBlockN * 128), &tm_v, bar_v_full + 8 * vst, h * 64, it.key0(), kvh, bi);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ tcgen05 issuer
    // The whole warp runs this loop converged and one elected lane issues each instruction: written as
    // `if (lane == 0) { ... }` the descriptors and addresses are per-thread values for the compiler and one
    // tcgen05.mma cost the issuing thread ~107 cycles (a commit ~350), 1200 cycles for the 8 MMAs and the commit
    // of a Q K^T against ~540 now (clock stamps of a debug build).  An N = 64 instruction occupies the tensor pipe
    // as long as an N = 128 one.  There is ONE commit per step, behind Q K^T; since one thread's MMAs complete in
    // issue order that commit also reports P V of two steps earlier, which is all the other warps need to know.
    // Issue order QK(i+1), PV(i): S buffer (i+1)&1 still holds P(i-1), which PV(i-1), issued earlier by this
    // same thread, consumes first (the tensor pipe executes one thread's MMAs in issue order).
    {
      const uint32_t fmt = p.qk_bf16 ? 1u : 0u;
      const uint32_t idesc_qk = make_idesc(fmt, fmt, 0, 0, kBlockM, kBlockN);
      const uint32_t idesc_pv = make_idesc(0, 0, 0, 1, kBlockM, D);
      const uint64_t q_desc = smem_desc_sw128(q_s, 16, 1024);
      const uint64_t k_desc0 = smem_desc_sw128(k_s, 16, 1024);
      const uint64_t v_desc0 = smem_desc_sw128(v_s, kBlockN * 128, 1024);
      bool ok = true;
      int q_uses = 0;
      StepIter qk_it(segs, nseg);
      auto issue_qk = [&](int j) {
        if (j == 0 || (qk_it.first_of_seg() && qk_it.opset_changed_before())) {
          // with in-kernel quantisation the tile is ready when the 128 softmax threads have rewritten their rows
          SQ_STAMP(j, 3);
          ok = mbar_wait_warp(p.q_fake_quant ? bar_q_ready : bar_q_full, q_uses & 1, cta_abort, 111);
          SQ_STAMP(j, 15);
          ++q_uses;
          if (!ok) return;
        }
        const int st = j & 1;
        SQ_STAMP(j, 0);
        ok = mbar_wait_warp(bar_k_full + 8 * st, (j >> 1) & 1, cta_abort, 112);
        if (!ok) return;
        tc_fence_after();
        const uint32_t d_tmem = tmem + st * kBlockN;
        const uint64_t k_desc = k_desc0 + static_cast<uint32_t>(st) * (L::kKBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          constexpr uint32_t kHalfQ = kBlockM * 128, kHalfK = kBlockN * 128;
          const uint32_t off_q = (kk >> 2) * kHalfQ + (kk & 3) * 32;
          const uint32_t off_k = (kk >> 2) * kHalfK + (kk & 3) * 32;
          // descriptors differ from the precomputed bases only in the start-address field (units of 16 bytes)
          mma_ss_elect(d_tmem, q_desc + (off_q >> 4), k_desc + (off_k >> 4), idesc_qk, kk > 0);
        }
        tc_commit_elect(bar_s_full + 8 * st);
        SQ_STAMP(j, 1);
        if (qk_it.last_of_seg() && qk_it.opset_changes_after()) tc_commit_elect(bar_q_empty);
        qk_it.next();
      };
      if (nsteps > 0) issue_qk(0);
      for (int i = 0; ok && i < nsteps; ++i) {
        if (i + 1 < nsteps) { issue_qk(i + 1); if (!ok) break; }
        const int st = i & 1;
        const int vst = i % 3;
        // V has usually landed long ago: look at it first, so that nothing stands between P's arrival and the MMAs
        ok = mbar_wait_warp(bar_v_full + 8 * vst, (i / 3) & 1, cta_abort, 114);
        if (!ok) break;
        ok = mbar_wait_warp(bar_p_full + 8 * st, (i >> 1) & 1, cta_abort, 113);
        if (!ok) break;
        SQ_STAMP(i, 2);
        tc_fence_after();
        const uint32_t p_tmem = tmem + st * kBlockN;
        const uint64_t v_desc = v_desc0 + static_cast<uint32_t>(vst) * (L::kVBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < kBlockN / 16; ++kk) {
          // V tile: [64 keys][64 d] 128-byte rows per d-half; MN-major B operand: 64-d chunks 8 KB apart
          // (leading offset), 8-key groups 1 KB apart (stride offset); 16 keys per MMA = 2 KB.
          mma_ts_elect(tmem + kOCol, p_tmem + kk * 8, v_desc + kk * (2048 >> 4), idesc_pv, (i > 0 || kk > 0));
        }
        // Completion of P V(i) is reported by the commit behind Q K^T(i+2); only the last two steps, which no
        // later Q K^T follows, get a commit of their own (slot 0: last step, slot 1: the one before).
        if (i + 2 >= nsteps) tc_commit_elect(bar_o_tail + 8 * (nsteps - 1 - i));
        SQ_STAMP(i, 4);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;  // TMEM lanes a warp may touch: 32*(warp%4) .. +31
    const int row_in_tile = quarter * 32 + lane;
    const int half_bit = (row_in_tile >= 64) ? kSegAct1 : kSegAct0;
    const int row_local = blk * kBlockM + row_in_tile;
    const int row = gblk * kBlockM + row_in_tile;  // position in the whole sequence (causal mask)
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_i = -INFINITY, base = -INFINITY, l_i = 1.0f;  // running maximum; reference of P, l_i and O
    bool ok = true;
    int i = 0;
    if (p.q_fake_quant && nsteps > 0) {
      // The adapter's per-token fake-quant of Q (sqattn/attn_replacer.py:361, fake_quant.py:23-125) and the
      // launcher's q * sm_scale (attn_triton_mix_relative.py:383-385) on this thread's row of the raw tile, in
      // place, with the device functions of the stand-alone preparation kernel (identical bits).  The row's 16-byte
      // chunks sit at chunk ^ (row & 7) inside each 128-byte line of the swizzled tile.
      if (warp == 2 && lane == 0) SQ_STAMP(1, 3);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_q_full, 0, cta_abort, 124));
      if (warp == 2 && lane == 0) SQ_STAMP(1, 15);
      if (ok) {
        uint8_t* qrow = smem + L::kQOff + row_in_tile * 128;
        uint4 raw[D / 8];
        float amax = 0.f;
#pragma unroll
        for (int ch = 0; ch < D / 8; ++ch) {
          raw[ch] = *reinterpret_cast<const uint4*>(qrow + (ch >> 3) * (kBlockM * 128) + (((ch & 7) ^ (row_in_tile & 7)) << 4));
          float f[8];
          if (p.qk_bf16) unpack8<true>(raw[ch], f); else unpack8<false>(raw[ch], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
        }
        amax = fmaxf(amax, 1e-5f);
        const int qtype = p.q_fake_quant - 1;
#pragma unroll
        for (int ch = 0; ch < D / 8; ++ch) {
          float f[8];
          uint4 outv;
          if (p.qk_bf16) unpack8<true>(raw[ch], f); else unpack8<false>(raw[ch], f);
          if (qtype == SQATTN_QTYPE_INT) {
            outv = p.qk_bf16 ? fake_quant_int_row8<true, true>(f, amax, 127.0f, p.q_half_even, p.q_scale)
                             : fake_quant_int_row8<false, true>(f, amax, 127.0f, p.q_half_even, p.q_scale);
          } else {
            float g[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float v = fake_quant_value(f[e], amax, qtype, 127.0f, p.q_half_even);
              g[e] = (p.qk_bf16 ? to_f32<true>(from_f32<true>(v)) : to_f32<false>(from_f32<false>(v))) * p.q_scale;
            }
            outv = p.qk_bf16 ? pack8<true>(g) : pack8<false>(g);
          }
          *reinterpret_cast<uint4*>(qrow + (ch >> 3) * (kBlockM * 128) + (((ch & 7) ^ (row_in_tile & 7)) << 4)) = outv;
        }
        fence_proxy_async();   // the rewritten tile is read by the tensor core through the async proxy
        mbar_arrive(bar_q_ready);
        if (warp == 2 && lane == 0) SQ_STAMP(2, 3);
      }
    }
    for (StepIter it(segs, nseg); ok && !it.done(); it.next(), ++i) {
      const int flags = it.flags();
      const uint32_t s_tmem = tmem + lane_addr + (i & 1) * kBlockN;
      if (warp == 2 && lane == 0) SQ_STAMP(i, 5);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full + 8 * (i & 1), (i >> 1) & 1, cta_abort, 121));
      if (!ok) break;
      tc_fence_after();
      if (warp == 2 && lane == 0) SQ_STAMP(i, 6);
      uint32_t pk[32];
      float alpha = 1.0f;
      if (flags & half_bit) {
        uint32_t r0[32], r1[32];
        tmem_ld32(s_tmem, r0);
        tmem_ld32(s_tmem + 32, r1);
        tmem_wait_ld();
        if (warp == 2 && lane == 0) SQ_STAMP(i, 7);
        float x[64];
#pragma unroll
        for (int c = 0; c < 32; ++c) { x[c] = __uint_as_float(r0[c]); x[32 + c] = __uint_as_float(r1[c]); }
        if (kDump && blockIdx.x == 0 && p.dump) {
#pragma unroll
          for (int c = 0; c < 64; ++c) p.dump[(static_cast<size_t>(i) * kBlockM + row_in_tile) * 64 + c] = x[c];
        }
        if (flags & kSegDiag) {
          const int key0 = it.key0();
#pragma unroll
          for (int c = 0; c < 64; ++c) x[c] = x[c] + ((row >= key0 + c) ? 0.0f : -1000000.0f);
        }
        // four independent chains for the row maximum (three-input max) and the row sum (packed fp32 pairs)
        float mx0 = x[0], mx1 = x[1], mx2 = x[2], mx3 = x[3];
#pragma unroll
        for (int c = 4; c < 60; c += 8) {
          mx0 = max3(mx0, x[c], x[c + 1]); mx1 = max3(mx1, x[c + 2], x[c + 3]);
          mx2 = max3(mx2, x[c + 4], x[c + 5]); mx3 = max3(mx3, x[c + 6], x[c + 7]);
        }
        mx0 = max3(mx0, x[60], x[61]); mx1 = max3(mx1, x[62], x[63]);
        const float m_new = fmaxf(max3(m_i, mx0, mx1), fmaxf(mx2, mx3));
        // P, l and O are kept relative to `base`, which follows the running maximum only when it has moved by
        // more than kLazyLog2 (so P <= 2^kLazyLog2): O then needs its rescale (a wait for the previous P V plus a
        // TMEM round trip) a few times per row instead of whenever the maximum moves.  Steps whose P is rounded
        // through e4m3 keep base == running maximum, i.e. p <= 1 as the rounding rule expects.
        const float thr = (flags & kSegFp8) ? 0.0f : kLazyLog2;
        if (m_new > base + thr) {
          alpha = ex2_approx(base - m_new);
          base = m_new;
        }
        const uint64_t m2 = f32x2_pack(base, base);
        uint64_t sa = f32x2_pack(0.0f, 0.0f), sb = sa;
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          float a0, a1, b0, b1;
          f32x2_unpack(f32x2_sub(f32x2_pack(x[c], x[c + 1]), m2), a0, a1);
          f32x2_unpack(f32x2_sub(f32x2_pack(x[c + 2], x[c + 3]), m2), b0, b1);
          x[c] = ex2_approx(a0); x[c + 1] = ex2_approx(a1); x[c + 2] = ex2_approx(b0); x[c + 3] = ex2_approx(b1);
          sa = f32x2_add(sa, f32x2_pack(x[c], x[c + 1]));
          sb = f32x2_add(sb, f32x2_pack(x[c + 2], x[c + 3]));
        }
        float s0, s1, s2, s3;
        f32x2_unpack(sa, s0, s1);
        f32x2_unpack(sb, s2, s3);
        const float sum = (s0 + s1) + (s2 + s3);
        l_i = l_i * alpha + sum;
        if (warp == 2 && lane == 0) SQ_STAMP(i, 9);
        m_i = m_new;
        if (flags & kSegFp8) {
#pragma unroll
          for (int c = 0; c < 32; ++c) pk[c] = p_fp8_round_f16x2(x[2 * c], x[2 * c + 1]);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) pk[c] = pack_f16x2(x[2 * c], x[2 * c + 1]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = 0u;
      }
      if (kDump && blockIdx.x == 0 && p.dump_p) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const __half2 h = *reinterpret_cast<const __half2*>(&pk[c]);
          float* dst = p.dump_p + (static_cast<size_t>(i) * kBlockM + row_in_tile) * 64 + 2 * c;
          dst[0] = __low2float(h); dst[1] = __high2float(h);
        }
      }
      tmem_st32(s_tmem, pk);
      // acc *= alpha: O lives in TMEM and is rescaled only when some row of this warp moved its maximum
      // (alpha == 1 exactly otherwise, so skipping is bit-identical).
      if (__any_sync(0xffffffffu, alpha != 1.0f) && i > 0) {
        // P V(i-1) has completed when Q K^T(i+1) has (same issuing thread, in order); the last step waits for the
        // commit that follows P V of the step before it
        if (i + 1 < nsteps) ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full + 8 * ((i + 1) & 1), ((i + 1) >> 1) & 1, cta_abort, 122));
        else ok = __all_sync(0xffffffffu, mbar_wait(bar_o_tail + 8, 0, cta_abort, 122));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tmem + lane_addr + kOCol + c0, o);
          tmem_wait_ld();
          const uint64_t al2 = f32x2_pack(alpha, alpha);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float a, b;
            f32x2_unpack(f32x2_mul(f32x2_pack(__uint_as_float(o[c]), __uint_as_float(o[c + 1])), al2), a, b);
            o[c] = __float_as_uint(a); o[c + 1] = __float_as_uint(b);
          }
          tmem_st32(tmem + lane_addr + kOCol + c0, o);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p_full + 8 * (i & 1));
      if (warp == 2 && lane == 0) SQ_STAMP(i, 11);
      if (warp == 3 && lane == 0) SQ_STAMP(i, 8);
      if (warp == 4 && lane == 0) SQ_STAMP(i, 10);
      if (warp == 5 && lane == 0) SQ_STAMP(i, 14);
    }
    if (ok && nsteps > 0) ok = mbar_wait(bar_o_tail, 0, cta_abort, 123);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && nsteps > 0) {
      tc_fence_after();
      const bool in_range = row_local < p.n;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      2 * (static_cast<long long>(bi) * p.o_sb + static_cast<long long>(head) * p.o_sh +
                           static_cast<long long>(row_local) * p.o_sn);
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_addr + kOCol + c0, o);
        tmem_wait_ld();
        if (in_range) {
          uint32_t w[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float a = __uint_as_float(o[2 * c]) / l_i, b = __uint_as_float(o[2 * c + 1]) / l_i;
            w[c] = p.o_dtype ? pack_bf16x2(a, b) : pack_f16x2(a, b);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
          for (int c = 0; c < 4; ++c) dst[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
        }
      }
      if (p.lse && in_range)
        p.lse[(static_cast<long long>(bi) * p.hq + head) * p.n + row_local] = log2f(l_i) + base;
    }
    tc_fence_before();
  }

  // ------------------------------------------------------------------ tear-down (also reached after a wait gave up)
  if (*cta_abort) {
    // copies may still be in flight towards this CTA's shared memory: give them time to land
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  __syncthreads();
  if (*cta_abort) poison_output<D>(p, bi, head, blk);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace sq
