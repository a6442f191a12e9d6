// Prefill kernel with 128-key Q K^T tiles and two softmax warp sets.
//
// An M128 x N64 tcgen05.mma occupies the tensor pipe as long as an N128 one, so the 64-key steps of the
// reference tile loop are issued in PAIRS: one Q K^T MMA group with N = 128 produces the scores of two
// consecutive steps.  Everything the reference defines per 64 keys stays per 64 keys: the first step of a pair is
// processed by warp set A, the second by warp set B (same rows, one thread per row in each set), and
//   m_a = max(m_prev, max S_a)   P_a = f16(2^(S_a - m_a))   O = O * 2^(m_prev - m_a) + P_a V_a
//   m_b = max(m_a,    max S_b)   P_b = f16(2^(S_b - m_b))   O = O * 2^(m_a - m_b)    + P_b V_b
// exactly as the 64-key loop does (sqattn/attn_triton_mix_relative.py:76-98); the two sets only exchange the
// running maximum of their rows through shared memory, so their exponentials run concurrently.  The row sum is
// kept as two partial sums (one per set, each relative to the set's latest maximum) and combined at the end.
//
// One CTA per SM, 11 warps:
//   warps 0..3   softmax set A          warps 4..7   softmax set B
//   warp  8      TMA producer (Q; K and V in two 128-key stages each)
//   warp  9      Q K^T issuer, owns TMEM        warp 10   P V issuer
// TMEM (512 columns): two S pair buffers [0,128) [128,256), O [256,256+D), two P pair buffers [384,448) [448,512)
// (f16, 32 columns per 64-key step).  P has its own columns so that an S buffer is free again as soon as the
// softmax threads have loaded it into registers: Q K^T always runs one pair ahead of the softmax.
#pragma once
#include "prefill.cuh"

namespace sq {

template <int D>
struct WideSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kQBytes = kBlockM * D * 2;
  static constexpr int kKStageBytes = 2 * kBlockN * D * 2;  // 128 keys
  static constexpr int kVTileBytes = kBlockN * D * 2;       // 64 keys
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQBytes;
  static constexpr int kVOff = kKOff + 2 * kKStageBytes;
  static constexpr int kBarOff = kVOff + 4 * kVTileBytes;
  static constexpr int kNumBars = 28;
  static constexpr int kMiscOff = kBarOff + 8 * kNumBars;
  static constexpr int kMaxOff = kMiscOff + 16;               // float mA[128], mB[128], LA[128], LB[128]
  static constexpr int kSegOff = kMaxOff + 4 * kBlockM * 4;
  static constexpr int kDynBytes = kSegOff + kMaxSegs * 12;
};

// 2 when the step after `it` exists and reads the same operand set (it then shares the Q K^T MMA group), else 1
__device__ __forceinline__ int pair_count(const StepIter& it) {
  StepIter nx = it;
  nx.next();
  return (!nx.done() && !((nx.flags() ^ it.flags()) & kSegInt4)) ? 2 : 1;
}

// One 64-key softmax step of one row: x = S (fp32) in, packed f16 P out; returns the row sum of the exponentials.
__device__ __forceinline__ float softmax_row64(float (&x)[64], float m_new, bool fp8, uint32_t (&pk)[32]) {
  const uint64_t m2 = f32x2_pack(m_new, m_new);
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
  if (fp8) {
#pragma unroll
    for (int c = 0; c < 32; ++c) pk[c] = p_fp8_round_f16x2(x[2 * c], x[2 * c + 1]);
  } else {
#pragma unroll
    for (int c = 0; c < 32; ++c) pk[c] = pack_f16x2(x[2 * c], x[2 * c + 1]);
  }
  return (s0 + s1) + (s2 + s3);
}

__device__ __forceinline__ float row_max64(const float (&x)[64]) {
  float mx0 = x[0], mx1 = x[1], mx2 = x[2], mx3 = x[3];
#pragma unroll
  for (int c = 4; c < 60; c += 8) {
    mx0 = max3(mx0, x[c], x[c + 1]); mx1 = max3(mx1, x[c + 2], x[c + 3]);
    mx2 = max3(mx2, x[c + 4], x[c + 5]); mx3 = max3(mx3, x[c + 6], x[c + 7]);
  }
  mx0 = max3(mx0, x[60], x[61]); mx1 = max3(mx1, x[62], x[63]);
  return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

template <int D, bool kDump>
__global__ void __launch_bounds__(352, 1)
prefill_wide_kernel(const __grid_constant__ CUtensorMap tm_q8, const __grid_constant__ CUtensorMap tm_q4,
                    const __grid_constant__ CUtensorMap tm_k8, const __grid_constant__ CUtensorMap tm_k4,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ PrefillParams p) {
  using L = WideSmem<D>;
  constexpr int NC = L::kChunks;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kOCol = 256, kPCol = 384;
#define SQW_STAMP(pair, slot)                                                              \
  do {                                                                                    \
    if (kDump && blockIdx.x == 0 && p.dump_t) p.dump_t[(pair) * 16 + (slot)] = clock64();  \
  } while (0)

  if (*reinterpret_cast<volatile int*>(&g_device_status) != 0) return;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t sbase = smem_u32(smem);
  if (sbase & 1023u) {
    if (threadIdx.x == 0) atomicCAS(&g_device_status, 0, 100);
    return;
  }
  const uint32_t q_s = sbase + L::kQOff, k_s = sbase + L::kKOff, v_s = sbase + L::kVOff;
  const uint32_t bars = sbase + L::kBarOff;
  // every barrier family below has two members, indexed by the pair's parity (its S / K / V buffer)
  const uint32_t bar_q_full = bars, bar_q_empty = bars + 8;
  const uint32_t bar_k_full = bars + 16, bar_va_full = bars + 32, bar_vb_full = bars + 48, bar_s_full = bars + 64;
  const uint32_t bar_pa_full = bars + 80, bar_pb_full = bars + 96, bar_pva_done = bars + 112, bar_pair_done = bars + 128;
  const uint32_t bar_ma = bars + 144, bar_mb = bars + 176;  // four each: one per 32-row quarter
  const uint32_t bar_s_read = bars + 208;                   // S buffer loaded into registers by all eight softmax warps
  volatile uint32_t* tmem_base_s = reinterpret_cast<volatile uint32_t*>(smem + L::kMiscOff);
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  volatile int* nseg_s = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 8);
  volatile float* mA = reinterpret_cast<volatile float*>(smem + L::kMaxOff);
  volatile float* mB = mA + kBlockM;
  volatile float* LA = mB + kBlockM;
  volatile float* LB = LA + kBlockM;
  Seg* segs = reinterpret_cast<Seg*>(smem + L::kSegOff);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_blk = p.hq * p.batch;
  const int blk = p.nblk - 1 - static_cast<int>(blockIdx.x) / per_blk;
  const int rem = static_cast<int>(blockIdx.x) % per_blk;
  const int bi = rem / p.hq, head = rem % p.hq, kvh = head / p.groups;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    *nseg_s = build_schedule(segs, p, blk + p.blk0, head);
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_k_full + 8 * i, 1);
      mbar_init(bar_va_full + 8 * i, 1);
      mbar_init(bar_vb_full + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_pa_full + 8 * i, 128);
      mbar_init(bar_pb_full + 8 * i, 128);
      mbar_init(bar_pva_done + 8 * i, 1);
      mbar_init(bar_pair_done + 8 * i, 1);
      mbar_init(bar_s_read + 8 * i, 8);
    }
    for (int i = 0; i < 4; ++i) { mbar_init(bar_ma + 8 * i, 32); mbar_init(bar_mb + 8 * i, 32); }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 9) {
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

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    // K stage pr & 1 is free when Q K^T of pair pr-2 has completed (s_full), V stage pr & 1 when the P V
    // products of pair pr-2 have (pair_done): completion barriers double as "empty" barriers.
    if (lane == 0) {
      tma_prefetch_desc(&tm_q8); tma_prefetch_desc(&tm_k8); tma_prefetch_desc(&tm_v);
      int q_loads = 0, pr = 0;
      bool ok = true;
      StepIter it(segs, nseg);
      while (ok && !it.done()) {
        const int cnt = pair_count(it);
        const int buf = pr & 1;
        const bool int4 = it.flags() & kSegInt4;
        if (pr == 0 || (it.first_of_seg() && it.opset_changed_before())) {
          if (q_loads > 0) ok = mbar_wait(bar_q_empty, (q_loads - 1) & 1, cta_abort, 101);
          if (!ok) break;
          mbar_expect_tx(bar_q_full, L::kQBytes);
          const CUtensorMap* tq = int4 ? &tm_q4 : &tm_q8;
#pragma unroll
          for (int c = 0; c < NC; ++c) tma_load_4d(q_s + c * (kBlockM * 128), tq, bar_q_full, c * 64, blk * kBlockM, head, bi);
          ++q_loads;
        }
        StepIter second = it;
        second.next();
        const int key_a = it.key0(), key_b = (cnt == 2) ? second.key0() : 0;
        if (pr >= 2) ok = mbar_wait(bar_s_full + 8 * buf, ((pr - 2) >> 1) & 1, cta_abort, 102);
        if (!ok) break;
        const CUtensorMap* tk = int4 ? &tm_k4 : &tm_k8;
        SQW_STAMP(pr, 15);
        mbar_expect_tx(bar_k_full + 8 * buf, cnt * NC * (kBlockN * 128));
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const uint32_t dst = k_s + buf * L::kKStageBytes + c * (2 * kBlockN * 128);
          tma_load_4d(dst, tk, bar_k_full + 8 * buf, c * 64, key_a, kvh, bi);
          if (cnt == 2) tma_load_4d(dst + kBlockN * 128, tk, bar_k_full + 8 * buf, c * 64, key_b, kvh, bi);
        }
        if (pr >= 2) ok = mbar_wait(bar_pair_done + 8 * buf, ((pr - 2) >> 1) & 1, cta_abort, 103);
        if (!ok) break;
        SQW_STAMP(pr, 4);
        mbar_expect_tx(bar_va_full + 8 * buf, L::kVTileBytes);
#pragma unroll
        for (int c = 0; c < NC; ++c)
          tma_load_4d(v_s + (2 * buf) * L::kVTileBytes + c * (kBlockN * 128), &tm_v, bar_va_full + 8 * buf, c * 64, key_a, kvh, bi);
        if (cnt == 2) {
          mbar_expect_tx(bar_vb_full + 8 * buf, L::kVTileBytes);
#pragma unroll
          for (int c = 0; c < NC; ++c)
            tma_load_4d(v_s + (2 * buf + 1) * L::kVTileBytes + c * (kBlockN * 128), &tm_v, bar_vb_full + 8 * buf, c * 64, key_b, kvh, bi);
        }
        it = second;
        if (cnt == 2) it.next();
        ++pr;
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ Q K^T issuer
    if (lane == 0) {
      const uint32_t fmt = p.qk_bf16 ? 1u : 0u;
      const uint32_t idesc1 = make_idesc(fmt, fmt, 0, 0, kBlockM, kBlockN), idesc2 = make_idesc(fmt, fmt, 0, 0, kBlockM, 2 * kBlockN);
      const uint64_t q_desc = smem_desc_sw128(q_s, 16, 1024);
      const uint64_t k_desc0 = smem_desc_sw128(k_s, 16, 1024);
      bool ok = true;
      int q_uses = 0, pr = 0;
      StepIter it(segs, nseg);
      while (ok && !it.done()) {
        const int cnt = pair_count(it);
        const int buf = pr & 1;
        if (pr == 0 || (it.first_of_seg() && it.opset_changed_before())) {
          ok = mbar_wait(bar_q_full, q_uses & 1, cta_abort, 111);
          ++q_uses;
          if (!ok) break;
        }
        ok = mbar_wait(bar_k_full + 8 * buf, (pr >> 1) & 1, cta_abort, 112);
        if (!ok) break;
        SQW_STAMP(pr, 0);
        // the S buffer is free once the softmax warps have loaded the scores of pair pr-2 into registers
        if (pr >= 2) ok = mbar_wait(bar_s_read + 8 * buf, ((pr - 2) >> 1) & 1, cta_abort, 115);
        if (!ok) break;
        SQW_STAMP(pr, 1);
        tc_fence_after();
        const uint64_t k_desc = k_desc0 + static_cast<uint32_t>(buf) * (L::kKStageBytes >> 4);
        const uint32_t idesc = cnt == 2 ? idesc2 : idesc1;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off_q = (kk >> 2) * (kBlockM * 128) + (kk & 3) * 32;
          const uint32_t off_k = (kk >> 2) * (2 * kBlockN * 128) + (kk & 3) * 32;
          mma_ss(tmem + buf * 128, q_desc + (off_q >> 4), k_desc + (off_k >> 4), idesc, kk > 0);
        }
        tc_commit(bar_s_full + 8 * buf);
        SQW_STAMP(pr, 2);
        if (cnt == 2) it.next();
        if (it.last_of_seg() && it.opset_changes_after()) tc_commit(bar_q_empty);
        it.next();
        ++pr;
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ P V issuer
    if (lane == 0) {
      const uint32_t idesc_pv = make_idesc(0, 0, 0, 1, kBlockM, D);
      const uint64_t v_desc0 = smem_desc_sw128(v_s, kBlockN * 128, 1024);
      bool ok = true;
      int pr = 0, b_uses[2] = {0, 0};
      StepIter it(segs, nseg);
      while (ok && !it.done()) {
        const int cnt = pair_count(it);
        const int buf = pr & 1;
        ok = mbar_wait(bar_pa_full + 8 * buf, (pr >> 1) & 1, cta_abort, 113);
        if (!ok) break;
        SQW_STAMP(pr, 3);
        ok = mbar_wait(bar_va_full + 8 * buf, (pr >> 1) & 1, cta_abort, 114);
        if (!ok) break;
        tc_fence_after();
        {
          const uint64_t v_desc = v_desc0 + static_cast<uint32_t>(2 * buf) * (L::kVTileBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < kBlockN / 16; ++kk)
            mma_ts(tmem + kOCol, tmem + kPCol + buf * 64 + kk * 8, v_desc + kk * (2048 >> 4), idesc_pv, (pr > 0 || kk > 0));
        }
        tc_commit(bar_pva_done + 8 * buf);
        SQW_STAMP(pr, 5);
        if (cnt == 2) {
          const int ph = (buf ? b_uses[1] : b_uses[0]) & 1;
          if (buf) ++b_uses[1]; else ++b_uses[0];
          ok = mbar_wait(bar_pb_full + 8 * buf, ph, cta_abort, 116);
          if (!ok) break;
          SQW_STAMP(pr, 6);
          ok = mbar_wait(bar_vb_full + 8 * buf, ph, cta_abort, 117);
          if (!ok) break;
          tc_fence_after();
          const uint64_t v_desc = v_desc0 + static_cast<uint32_t>(2 * buf + 1) * (L::kVTileBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < kBlockN / 16; ++kk)
            mma_ts(tmem + kOCol, tmem + kPCol + buf * 64 + 32 + kk * 8, v_desc + kk * (2048 >> 4), idesc_pv, true);
          it.next();
        }
        tc_commit(bar_pair_done + 8 * buf);
        SQW_STAMP(pr, 7);
        it.next();
        ++pr;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax sets A (warps 0-3) and B (4-7)
    const bool set_b = warp >= 4;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int half_bit = (row_in_tile >= 64) ? kSegAct1 : kSegAct0;
    const int row_local = blk * kBlockM + row_in_tile;
    const int row = row_local + p.blk0 * kBlockM;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t bar_pub = (set_b ? bar_mb : bar_ma) + 8 * quarter;   // this set publishes its maximum here
    const uint32_t bar_sub = (set_b ? bar_ma : bar_mb) + 8 * quarter;   // and reads the other set's from here
    float m_run = -INFINITY;          // running maximum of the row after this thread's latest step
    float m_ref = -INFINITY;          // the maximum l_part is relative to
    float l_part = set_b ? 0.0f : 1.0f;
    bool ok = true;
    int pr = 0, step = 0;
    StepIter it(segs, nseg);
    while (ok && !it.done()) {
      const int cnt = pair_count(it);
      const int buf = pr & 1;
      StepIter mine = it;
      if (set_b && cnt == 2) mine.next();
      const bool work = !set_b || cnt == 2;          // set B idles on an unpaired step
      const int flags = work ? mine.flags() : 0;
      const bool active = work && (flags & half_bit);
      const int my_step = step + (set_b ? 1 : 0);
      const uint32_t s_tmem = tmem + lane_addr + buf * 128 + (set_b ? kBlockN : 0);
      float x[64];
      uint32_t pk[32];
      float lmax = -INFINITY;
      if (work) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full + 8 * buf, (pr >> 1) & 1, cta_abort, 121));
        if (!ok) break;
        tc_fence_after();
        if (lane == 0 && quarter == 0) SQW_STAMP(pr, set_b ? 12 : 8);
      }
      if (active) {
        uint32_t r0[32], r1[32];
        tmem_ld32(s_tmem, r0);
        tmem_ld32(s_tmem + 32, r1);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) { x[c] = __uint_as_float(r0[c]); x[32 + c] = __uint_as_float(r1[c]); }
        if (kDump && blockIdx.x == 0 && p.dump) {
#pragma unroll
          for (int c = 0; c < 64; ++c) p.dump[(static_cast<size_t>(my_step) * kBlockM + row_in_tile) * 64 + c] = x[c];
        }
        if (flags & kSegDiag) {
          const int key0 = mine.key0();
#pragma unroll
          for (int c = 0; c < 64; ++c) x[c] = x[c] + ((row >= key0 + c) ? 0.0f : -1000000.0f);
        }
        lmax = row_max64(x);
      }
      // this warp no longer needs the S buffer (idle warps report too: the barrier counts all eight warps)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_s_read + 8 * buf);
      // the row's maximum before this step: set A takes set B's from the previous pair, set B takes set A's
      float m_prev = -INFINITY;
      if (set_b || pr > 0) {
        const int ph = set_b ? (pr & 1) : ((pr - 1) & 1);
        ok = __all_sync(0xffffffffu, mbar_wait(bar_sub, ph, cta_abort, 124));
        if (!ok) break;
        m_prev = (set_b ? mA : mB)[row_in_tile];
      }
      if (lane == 0 && quarter == 0) SQW_STAMP(pr, set_b ? 13 : 9);
      const float m_new = active ? fmaxf(m_prev, lmax) : m_prev;
      (set_b ? mB : mA)[row_in_tile] = m_new;
      mbar_arrive(bar_pub);
      m_run = m_new;
      float alpha = 1.0f;
      if (active) {
        alpha = ex2_approx(m_prev - m_new);
        const float sum = softmax_row64(x, m_new, flags & kSegFp8, pk);
        l_part = l_part * ex2_approx(m_ref - m_new) + sum;
        m_ref = m_new;
        if (lane == 0 && quarter == 0 && !set_b) SQW_STAMP(pr, 10);
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = 0u;
      }
      if (work) {
        // the P columns of this buffer were last read by the P V products of pair pr-2
        if (pr >= 2) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar_pair_done + 8 * buf, ((pr - 2) >> 1) & 1, cta_abort, 129));
          if (!ok) break;
          tc_fence_after();
        }
        tmem_st32(tmem + lane_addr + kPCol + buf * 64 + (set_b ? 32 : 0), pk);
        // O *= alpha before this step's P V, only when some row of the warp moved its maximum; O is stable once
        // the previous step's P V has completed
        if (__any_sync(0xffffffffu, alpha != 1.0f) && my_step > 0) {
          if (set_b) ok = __all_sync(0xffffffffu, mbar_wait(bar_pva_done + 8 * buf, (pr >> 1) & 1, cta_abort, 122));
          else ok = __all_sync(0xffffffffu, mbar_wait(bar_pair_done + 8 * ((pr - 1) & 1), ((pr - 1) >> 1) & 1, cta_abort, 123));
          if (!ok) break;
          tc_fence_after();
          const uint64_t al2 = f32x2_pack(alpha, alpha);
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_addr + kOCol + c0, o);
            tmem_wait_ld();
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
        mbar_arrive((set_b ? bar_pb_full : bar_pa_full) + 8 * buf);
        if (lane == 0 && quarter == 0) SQW_STAMP(pr, set_b ? 14 : 11);
      }
      it.next();
      if (cnt == 2) it.next();
      step += cnt;
      ++pr;
    }
    // ---- epilogue: l = l_A * 2^(ref_A - m) + l_B * 2^(ref_B - m); set A writes columns [0, D/2), set B the rest
    // Set A reads the final maximum (set B's last publication) and publishes its partial sum; set B adds its own
    // and publishes the total.  Each set arrives on its barrier only after it has consumed the other's previous
    // publication, so a waiter is never more than one phase behind.
    const int npairs = pr;
    float m_fin = m_run, l_fin = 1.0f;
    if (ok && npairs > 0) {
      if (!set_b) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_sub, (npairs - 1) & 1, cta_abort, 125));
        if (ok) {
          m_fin = mB[row_in_tile];
          LA[row_in_tile] = l_part * ex2_approx(m_ref - m_fin);
          mbar_arrive(bar_pub);
          ok = __all_sync(0xffffffffu, mbar_wait(bar_sub, npairs & 1, cta_abort, 126));
          if (ok) l_fin = LB[row_in_tile];
        }
      } else {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_sub, npairs & 1, cta_abort, 128));
        if (ok) {
          l_fin = LA[row_in_tile] + l_part * ex2_approx(m_ref - m_fin);
          LB[row_in_tile] = l_fin;
          mbar_arrive(bar_pub);
        }
      }
    }
    if (ok && npairs > 0)
      ok = mbar_wait(bar_pair_done + 8 * ((npairs - 1) & 1), ((npairs - 1) >> 1) & 1, cta_abort, 127);
    ok = __all_sync(0xffffffffu, ok);
    if (ok && npairs > 0) {
      tc_fence_after();
      const bool in_range = row_local < p.n;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.o) +
                      2 * (static_cast<long long>(bi) * p.o_sb + static_cast<long long>(head) * p.o_sh +
                           static_cast<long long>(row_local) * p.o_sn);
      const int c_begin = set_b ? D / 2 : 0;
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_begin + D / 2; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_addr + kOCol + c0, o);
        tmem_wait_ld();
        if (in_range) {
          uint32_t w[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float a = __uint_as_float(o[2 * c]) / l_fin, b = __uint_as_float(o[2 * c + 1]) / l_fin;
            w[c] = p.o_dtype ? pack_bf16x2(a, b) : pack_f16x2(a, b);
          }
          uint4* dst = reinterpret_cast<uint4*>(orow + c0 * 2);
#pragma unroll
          for (int c = 0; c < 4; ++c) dst[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
        }
      }
      if (p.lse && in_range && !set_b)
        p.lse[(static_cast<long long>(bi) * p.hq + head) * p.n + row_local] = log2f(l_fin) + m_fin;
    }
    tc_fence_before();
  }

  // ------------------------------------------------------------------ tear-down (also reached after a wait gave up)
  if (*cta_abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace sq
