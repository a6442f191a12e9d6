// Split-KV single-query (decode) attention.  HBM-bound: the job is to stream K and V exactly once at
// full bandwidth.  One CTA handles one (sequence, KV head, key range) work item for ALL query heads of
// the KV group, so the group's K/V are read once (the reference reads them once per query head,
// sqattn/attn_triton_decode.py:204-241).
//   warp 4      TMA producer: 64-key K and V tiles into a 3-stage shared-memory ring (128-byte swizzle); when the
//               keys are an index list into a cache, warps 4 and 5 copy the listed rows into the same layout with
//               16-byte asynchronous copies (D/8 lanes per row, so that a request covers whole 128-byte lines;
//               each warp takes every other row group).  Warp 5 idles otherwise.
//   warps 0..3  16 keys of every tile each: S = q K^T and O += P V on mma.sync m16n8k16 (query heads padded
//               to the 16-row M dimension), warp-shuffle row max / sum, private online-softmax state;
//               the four states are merged through shared memory at the end of the item.
// A second kernel merges the per-range partials (base-2 LSE).
#pragma once
#include <cuda.h>

#include "prep.cuh"
#include "ptx.cuh"

namespace sq {

constexpr int kDecMaxBatch = 128;
constexpr int kDecTile = 64;
constexpr int kDecStages = 3;

struct DecodeParams {
  const uint8_t* q;
  long long q_sb, q_sh;
  float* part_o;    // [items, Hq, D] fp32, each normalised by its own l
  float* part_lse;  // [items, Hq]
  int batch, hq, hkv, groups, d;
  int chunk;  // keys per work item (multiple of 64)
  int p_fp8, q_is_scaled;
  int reference_tail;  // keys between a sequence's length and the next multiple of 64 count with score 0
  float sm_scale;  // 1/sqrt(D) * 1.44269504 evaluated in double on the host, like the Python launcher
  int lens[kDecMaxBatch];
  const int* lens_dev;  // when set, the lengths are read from the device at run time (lens[] holds the planned capacity)
  int item_prefix[kDecMaxBatch + 1];  // first work item of each sequence
  // Keys and values through an index list (the tokens a clustered cache retrieved): key j of (sequence, KV head) is
  // row gather_idx[(bi * hkv + kvh) * gather_cap + j] of gather_k / gather_v [bi * hkv + kvh]; nullptr: the tiled caches
  const int* gather_idx;
  const uint8_t* const* gather_k;
  const uint8_t* const* gather_v;
  long long gather_row_stride;  // elements
  int gather_cap;
};

// 16-byte asynchronous copy global -> shared, and an arrival on `bar` once all of this thread's copies have landed
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <int D>
struct DecodeSmem {
  static constexpr int kTileBytes = kDecTile * D * 2;            // one K or V tile
  static constexpr int kStageBytes = 2 * kTileBytes;             // K then V
  static constexpr int kBarOff = kDecStages * kStageBytes;       // full[3], empty[3]
  static constexpr int kMiscOff = kBarOff + 8 * 2 * kDecStages;  // abort flag
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynBytes = kTotal + 1024;
  // the merge scratch (4 warps x (16 x D fp32 + 32 floats)) reuses the tile ring
  static_assert(4 * (16 * D + 32) * 4 <= kDecStages * kStageBytes, "merge scratch must fit in the ring");
};

// byte offset of 16-byte chunk `chunk` of key row `key` inside a [64 keys][D] tile stored as D/64 halves of
// 128-byte rows with the TMA 128-byte swizzle
__device__ __forceinline__ uint32_t tile_off(int key, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (kDecTile * 128) + key * 128 + (((chunk & 7) ^ (key & 7)) << 4));
}

#ifdef SQATTN_DEBUG_EXPORTS
// debug builds only: when the first CTA of a decode launch started and the last one ended (globaltimer)
__device__ unsigned long long g_dec_first = ~0ull, g_dec_last = 0ull;
#endif

template <int D, bool BF16>
__global__ void __launch_bounds__(192, 2)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ DecodeParams p) {
  using L = DecodeSmem<D>;
  // Launched with programmatic stream serialisation: this grid may become resident while its predecessor in the
  // stream drains; nothing the predecessor produced (lengths, q, the status word) is read before this wait, and
  // the kernel that follows (the merge) may be made resident right away, it waits for this grid in turn.
  griddep_launch();
  griddep_wait();
#ifdef SQATTN_DEBUG_EXPORTS
  if (threadIdx.x == 0) atomicMin(&g_dec_first, globaltimer_ns());
#endif
  // after a wait has given up on this device (here or in an earlier launch) the partials of this work item are
  // marked invalid, so that the merge hands NaN to the caller instead of stale scratch
  auto poison_partials = [&](int nthr) {
    const float nan = __int_as_float(0x7fc00000);
    for (int idx = threadIdx.x; idx < p.groups * D; idx += nthr) {
      const long long orow = static_cast<long long>(blockIdx.x) * p.hq + blockIdx.y * p.groups + idx / D;
      p.part_o[orow * D + idx % D] = nan;
      if (idx % D == 0) p.part_lse[orow] = nan;
    }
  };
  if (device_failed()) {
    poison_partials(blockDim.x);
    return;
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar_full = sbase + L::kBarOff, bar_empty = bar_full + 8 * kDecStages;
  volatile int* cta_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // work item -> (sequence, key range): binary search in the per-sequence item prefix
  const int item = blockIdx.x, kvh = blockIdx.y;
  int lo = 0, hi = p.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.item_prefix[mid] <= item) lo = mid; else hi = mid;
  }
  const int bi = lo;
  const int len = p.lens_dev ? min(p.lens_dev[bi], p.lens[bi]) : p.lens[bi];
  const int key_begin = (item - p.item_prefix[bi]) * p.chunk;
  const int key_end = min(len, key_begin + p.chunk);  // real keys
  // The reference kernel loads keys past kv_len as zeros without masking their scores (masked tl.load,
  // attn_triton_decode.py:215-221), so its last 64-key tile is padded with keys of score 0 and value 0.
  const int proc_end = p.reference_tail ? min((len + kDecTile - 1) / kDecTile * kDecTile, key_begin + p.chunk) : key_end;
  const int ntiles = (proc_end - key_begin + kDecTile - 1) / kDecTile;

  if (threadIdx.x == 0) {
    *cta_abort = 0;
    // a stage is full after the producer's one arrival + its bytes (TMA), or after the copies of all 64 lanes of the
    // two copying warps (index list)
    for (int i = 0; i < kDecStages; ++i) { mbar_init(bar_full + 8 * i, p.gather_idx ? 64 : 1); mbar_init(bar_empty + 8 * i, 4); }
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp >= 4 && p.gather_idx) {
    const int half = warp - 4;   // warps 4 and 5 copy the even and the odd row groups of every tile
    const long long grp = static_cast<long long>(bi) * p.hkv + kvh;
    const int* idx = p.gather_idx + grp * p.gather_cap;
    const uint8_t* kb = p.gather_k[grp];
    const uint8_t* vb = p.gather_v[grp];
    bool ok = true;
    // the list entries of a tile are fetched one tile ahead, so that their latency hides behind the wait for a stage
    auto fetch = [&](int t, int (&tok)[2]) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int key = key_begin + t * kDecTile + lane + 32 * rr;
        tok[rr] = (t < ntiles && key < key_end) ? idx[key] : -1;   // rows past the end are never read as data
      }
    };
    int tok[2], nxt[2];
    fetch(0, tok);
    for (int t = 0; ok && t < ntiles; ++t) {
      const int st = t % kDecStages;
      fetch(t + 1, nxt);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * st, ((t / kDecStages) & 1) ^ 1, cta_abort, 201));
      if (!ok) break;
      const uint32_t k_tile = sbase + st * L::kStageBytes, v_tile = k_tile + L::kTileBytes;
      // D / 8 consecutive lanes copy one row (whole 128-byte lines per request); lane l holds the list entries of
      // rows l and l + 32 of the tile and hands them out by shuffle
      constexpr int kLanesPerRow = D / 8, kRowsPerInstr = 32 / kLanesPerRow;
      const int c = lane % kLanesPerRow, rsel = lane / kLanesPerRow;
#pragma unroll 4
      for (int r0 = half * kRowsPerInstr; r0 < kDecTile; r0 += 2 * kRowsPerInstr) {
        const int r = r0 + rsel;
        const int t_lo = __shfl_sync(0xffffffffu, tok[0], r & 31), t_hi = __shfl_sync(0xffffffffu, tok[1], r & 31);
        const int tk = r < 32 ? t_lo : t_hi;
        if (tk >= 0) {
          const long long off = static_cast<long long>(tk) * p.gather_row_stride * 2 + c * 16;
          cp_async_16(k_tile + tile_off(r, c), kb + off);
          cp_async_16(v_tile + tile_off(r, c), vb + off);
        }
      }
      cp_async_arrive(bar_full + 8 * st);
      tok[0] = nxt[0]; tok[1] = nxt[1];
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // nothing of this warp is in flight when the CTA winds down
  } else if (warp >= 4) {
    if (warp == 4 && lane == 0) {
      tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
      bool ok = true;
      for (int t = 0; ok && t < ntiles; ++t) {
        const int st = t % kDecStages;
        ok = mbar_wait(bar_empty + 8 * st, ((t / kDecStages) & 1) ^ 1, cta_abort, 201);
        if (!ok) break;
        mbar_expect_tx(bar_full + 8 * st, L::kStageBytes);
        const int key0 = key_begin + t * kDecTile;
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          tma_load_4d(sbase + st * L::kStageBytes + h * (kDecTile * 128), &tm_k, bar_full + 8 * st, h * 64, key0, kvh, bi);
          tma_load_4d(sbase + st * L::kStageBytes + L::kTileBytes + h * (kDecTile * 128), &tm_v, bar_full + 8 * st, h * 64,
                      key0, kvh, bi);
        }
      }
    }
  } else {
    // ---- q fragments: rows = query heads of this KV group (padded to 16), 16 head_dim values per k-step
    const int g = lane >> 2, tq = lane & 3;
    const float sm_scale = p.sm_scale;
    uint32_t qa[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = g + (r & 1) * 8;
        const int col = kk * 16 + tq * 2 + (r >> 1) * 8;
        uint32_t v = 0;
        if (row < p.groups) {
          const uint8_t* src = p.q + 2 * (bi * p.q_sb + static_cast<long long>(kvh * p.groups + row) * p.q_sh + col);
          v = *reinterpret_cast<const uint32_t*>(src);
          if (!p.q_is_scaled) {
            const float a = to_f32<BF16>(static_cast<uint16_t>(v & 0xffffu)) * sm_scale;
            const float b = to_f32<BF16>(static_cast<uint16_t>(v >> 16)) * sm_scale;
            v = static_cast<uint32_t>(from_f32<BF16>(a)) | (static_cast<uint32_t>(from_f32<BF16>(b)) << 16);
          }
        }
        qa[kk][r] = v;
      }
    }
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_r[2] = {-INFINITY, -INFINITY};
    float l_r[2] = {0.f, 0.f};  // per-lane partial row sums; reduced across the 4 lanes of a row at the end
    const int wk = warp * 16;   // this warp's keys inside a tile
    bool ok = true;
    for (int t = 0; ok && t < ntiles; ++t) {
      const int st = t % kDecStages;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * st, (t / kDecStages) & 1, cta_abort, 202));
      if (!ok) break;
      const uint32_t k_tile = sbase + st * L::kStageBytes, v_tile = k_tile + L::kTileBytes;
      const int key0 = key_begin + t * kDecTile + wk;  // first key of this warp
      if (key0 < proc_end) {
        // rows past the end of the sequence may hold anything (the cache is larger than the sequence):
        // their scores are overwritten below, and their V rows are zeroed so that 0 * garbage cannot make a NaN
        if (key0 + 16 > key_end) {
          for (int r = max(0, key_end - key0); r < 16; ++r)
            for (int c = lane; c < D / 8; c += 32)
              *reinterpret_cast<uint4*>(smem + st * L::kStageBytes + L::kTileBytes + tile_off(wk + r, c)) =
                  make_uint4(0, 0, 0, 0);
          __syncwarp();
        }
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          uint32_t b0, b1, b2, b3;
          // matrices: (keys 0-7, d lo) (keys 0-7, d hi) (keys 8-15, d lo) (keys 8-15, d hi)
          const int mi = lane >> 3, r = lane & 7;
          ldmatrix_x4(k_tile + tile_off(wk + r + (mi >> 1) * 8, kk * 2 + (mi & 1)), b0, b1, b2, b3);
          mma_16816<BF16>(s[0], qa[kk], b0, b1);
          mma_16816<BF16>(s[1], qa[kk], b2, b3);
        }
        // mask keys past the end; row maxima over this warp's 16 keys
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + nb * 8 + tq * 2 + (e & 1);
            if (key >= key_end) s[nb][e] = (key < proc_end) ? 0.f : -INFINITY;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
          }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
          mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
          const float m_new = fmaxf(m_r[r], mx[r]);
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[r] = ex2_approx(m_r[r] - m_use);
          m_r[r] = m_new;
          mx[r] = m_use;
        }
        uint32_t pa[4], pa_lo[4] = {0u, 0u, 0u, 0u};
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          float pv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) { pv[e] = ex2_approx(s[nb][e] - mx[e >> 1]); sum[e >> 1] += pv[e]; }
          uint32_t lo16, hi16;
          if (p.p_fp8) {
            lo16 = p_fp8_round_f16x2(pv[0], pv[1]);
            hi16 = p_fp8_round_f16x2(pv[2], pv[3]);
            if (BF16) {
              // V is bf16, so the tensor-core product takes bf16 operands.  The e4m3-rounded P is an f16 value with
              // up to 11 significant bits: it is split into a bf16 head and a bf16 remainder (exact: at most 3
              // bits are left), and P V is the sum of two products, so the rounded P reaches the product unchanged
              // as in the reference's p (f16) * v (fp32), attn_triton_decode.py:229-234.
              const __half2 a = *reinterpret_cast<__half2*>(&lo16), b = *reinterpret_cast<__half2*>(&hi16);
              const float f0 = __low2float(a), f1 = __high2float(a), f2 = __low2float(b), f3 = __high2float(b);
              lo16 = pack_bf16x2(f0, f1);
              hi16 = pack_bf16x2(f2, f3);
              const float h0 = __uint_as_float(lo16 << 16), h1 = __uint_as_float(lo16 & 0xffff0000u);
              const float h2 = __uint_as_float(hi16 << 16), h3 = __uint_as_float(hi16 & 0xffff0000u);
              pa_lo[nb * 2] = pack_bf16x2(f0 - h0, f1 - h1);
              pa_lo[nb * 2 + 1] = pack_bf16x2(f2 - h2, f3 - h3);
            }
          } else {
            lo16 = BF16 ? pack_bf16x2(pv[0], pv[1]) : pack_f16x2(pv[0], pv[1]);
            hi16 = BF16 ? pack_bf16x2(pv[2], pv[3]) : pack_f16x2(pv[2], pv[3]);
          }
          pa[nb * 2] = lo16;      // rows g,   keys nb*8 + ...
          pa[nb * 2 + 1] = hi16;  // rows g+8
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_r[r] = l_r[r] * alpha[r] + sum[r];
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
          o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
        }
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          uint32_t b0, b1, b2, b3;
          // transposed 8x8 loads: (keys 0-7, d chunk 2j) (keys 8-15, 2j) (keys 0-7, 2j+1) (keys 8-15, 2j+1)
          const int mi = lane >> 3, r = lane & 7;
          ldmatrix_x4_trans(v_tile + tile_off(wk + r + (mi & 1) * 8, j * 2 + (mi >> 1)), b0, b1, b2, b3);
          mma_16816<BF16>(o[2 * j], pa, b0, b1);
          mma_16816<BF16>(o[2 * j + 1], pa, b2, b3);
          if (BF16 && p.p_fp8) {
            mma_16816<BF16>(o[2 * j], pa_lo, b0, b1);
            mma_16816<BF16>(o[2 * j + 1], pa_lo, b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * st);
    }
    // ---- merge the four warps' states through shared memory (the ring is idle now)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 1);
      l_r[r] += __shfl_xor_sync(0xffffffffu, l_r[r], 2);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // all consumer warps are done with the ring
    float* scratch = reinterpret_cast<float*>(smem);
    float* my = scratch + warp * (16 * D + 32);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int col = j * 8 + tq * 2;
      my[g * D + col] = o[j][0]; my[g * D + col + 1] = o[j][1];
      my[(g + 8) * D + col] = o[j][2]; my[(g + 8) * D + col + 1] = o[j][3];
    }
    if (tq == 0) {
      my[16 * D + g] = m_r[0]; my[16 * D + g + 8] = m_r[1];
      my[16 * D + 16 + g] = l_r[0]; my[16 * D + 16 + g + 8] = l_r[1];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // the abort flag is stable here: the producer has issued its last copy before the consumers pass the last
    // full barrier, and a consumer that gave up did so before the barrier above
    if (*cta_abort) {
      poison_partials(128);
    } else if (ok) {
      for (int idx = threadIdx.x; idx < p.groups * D; idx += 128) {
        const int row = idx / D, col = idx % D;
        float mw[4], mmax = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) { mw[w] = scratch[w * (16 * D + 32) + 16 * D + row]; mmax = fmaxf(mmax, mw[w]); }
        float acc = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float sc = (mw[w] == -INFINITY) ? 0.f : ex2_approx(mw[w] - mmax);
          acc += sc * scratch[w * (16 * D + 32) + row * D + col];
          l += sc * scratch[w * (16 * D + 32) + 16 * D + 16 + row];
        }
        const long long orow = static_cast<long long>(item) * p.hq + kvh * p.groups + row;
        p.part_o[orow * D + col] = (l > 0.f) ? acc / l : 0.f;
        if (col == 0) p.part_lse[orow] = (l > 0.f) ? log2f(l) + mmax : -INFINITY;
      }
    }
  }
  if (*cta_abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
#ifdef SQATTN_DEBUG_EXPORTS
  __syncthreads();
  if (threadIdx.x == 0) atomicMax(&g_dec_last, globaltimer_ns());
#endif
}

struct MergeParams {
  const float* part_o;    // [parts..., rows, D]
  const float* part_lse;  // [parts..., rows]
  void* o;                // rows x D in o_dtype, or fp32 when o_f32
  float* lse;             // optional [rows]
  long long o_sb, o_sh;   // output strides (elements) for row = b*hq + h; ignored when contiguous
  int hq, d, o_dtype, o_f32, contiguous;
  int num_parts;          // uniform mode: parts are [num_parts, rows, D]
  long long rows;
  int ragged;             // ragged mode: parts of sequence b are items item_prefix[b] .. item_prefix[b+1]-1
  int item_prefix[kDecMaxBatch + 1];
};

// O = sum_i 2^(lse_i - max) O_i / sum_i 2^(lse_i - max);  lse = log2(sum) + max
// One CTA (128 * kMergeGroups threads) per output row (b, h).  Thread (group g, column c) takes every
// kMergeGroups-th partial of column c.  The partial values of a round are loaded into registers BEFORE the
// weights are known (the loads do not depend on them), so a row costs about one trip to L2 however many
// partials it has up to kMergeRound; larger counts go in rounds.  The groups are combined in a fixed order, so
// the result does not depend on timing.
constexpr int kMergeGroups = 4;
constexpr int kMergeDepth = 16;                          // partial values in flight per thread
constexpr int kMergeRound = kMergeGroups * kMergeDepth;  // partials per round
constexpr int kMergeMaxParts = 2048;

struct MergeScratch {
  float w[kMergeMaxParts];
  float red[kMergeGroups][128];
  float mx[32];
};

// Merges `count` partials of one row: partial i sits at row (base_row + i * part_stride) of part_o [.., d] /
// part_lse [..].  Returns this thread's column (tid < d) of the merged, normalised row and the row's LSE (a NaN
// partial, left by a launch that failed, makes both NaN).  All threads of the CTA must call it.
__device__ __forceinline__ void merge_row_partials(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                                   long long base_row, long long part_stride, int count, int d,
                                                   MergeScratch& sm, float& out_val, float& out_lse) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int col = tid % 128, grp = tid / 128;
  float v[kMergeDepth];
  auto load_round = [&](int base) {
#pragma unroll
    for (int u = 0; u < kMergeDepth; ++u) {
      const int i = base + grp + u * kMergeGroups;
      v[u] = (i < count && col < d) ? part_o[(base_row + i * part_stride) * d + col] : 0.f;
    }
  };
  load_round(0);
  float mloc = -INFINITY;
  for (int i = tid; i < count; i += nthr) mloc = fmaxf(mloc, part_lse[base_row + i * part_stride]);
  for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
  if ((tid & 31) == 0) sm.mx[tid >> 5] = mloc;
  __syncthreads();
  float mmax = -INFINITY;
  for (int i = 0; i < (nthr + 31) / 32; ++i) mmax = fmaxf(mmax, sm.mx[i]);
  float den = 0.f, acc = 0.f;
  for (int base = 0; base < count; base += kMergeMaxParts) {  // more than kMergeMaxParts partials: in batches
    const int cnt = min(kMergeMaxParts, count - base);
    __syncthreads();
    for (int i = tid; i < cnt; i += nthr) {
      const float lse_i = part_lse[base_row + (base + i) * part_stride];
      sm.w[i] = (lse_i == -INFINITY) ? 0.f : exp2f(lse_i - mmax);
    }
    __syncthreads();
    for (int i = 0; i < cnt; ++i) den += sm.w[i];  // same order in every thread
    for (int r0 = 0; r0 < cnt; r0 += kMergeRound) {
      if (base + r0 > 0) load_round(base + r0);
#pragma unroll
      for (int u = 0; u < kMergeDepth; ++u) {
        const int i = r0 + grp + u * kMergeGroups;
        if (i < cnt) acc += sm.w[i] * v[u];
      }
    }
  }
  sm.red[grp][col] = acc;
  __syncthreads();
  float tot = 0.f;
  if (tid < d) {
#pragma unroll
    for (int g = 0; g < kMergeGroups; ++g) tot += (g < nthr / 128) ? sm.red[g][tid] : 0.f;
  }
  out_val = (den > 0.f) ? tot / den : (den == den ? 0.f : den);
  out_lse = (den > 0.f) ? log2f(den) + mmax : (den == den ? -INFINITY : den);
}

__global__ void __launch_bounds__(128 * kMergeGroups) decode_merge_kernel(const __grid_constant__ MergeParams p) {
  __shared__ MergeScratch sm;
  griddep_launch();
  griddep_wait();  // the partials come from the kernel launched just before
  const long long row = blockIdx.x;  // b*hq + h
  const int b = static_cast<int>(row / p.hq), h = static_cast<int>(row % p.hq);
  int first = 0, count = p.num_parts;
  long long part_stride = p.rows;  // in rows
  long long base_row = row;
  if (p.ragged) {
    first = p.item_prefix[b];
    count = p.item_prefix[b + 1] - first;
    part_stride = p.hq;
    base_row = static_cast<long long>(first) * p.hq + h;
  }
  float val, lse;
  merge_row_partials(p.part_o, p.part_lse, base_row, part_stride, count, p.d, sm, val, lse);
  const int tid = threadIdx.x;
  if (tid < p.d) {
    const int col = tid;
    const long long off = p.contiguous ? row * p.d + col : b * p.o_sb + h * p.o_sh + col;
    if (p.o_f32) reinterpret_cast<float*>(p.o)[off] = val;
    else if (p.o_dtype) reinterpret_cast<uint16_t*>(p.o)[off] = from_f32<true>(val);
    else reinterpret_cast<uint16_t*>(p.o)[off] = from_f32<false>(val);
    if (col == 0 && p.lse) p.lse[row] = lse;
  }
}

}  // namespace sq
