// Paged GQA attention on the Blackwell tensor cores (tcgen05), head_dim 256, fp8 (e4m3) KV pages.
//
// One kernel family for prefill and decode.  A CTA owns (sequence, KV head, query tile[, KV split]):
// its MMA rows are (query head of the GQA group) x (token of the tile), so the whole group shares
// every K / V page it streams -- the role of the reference's paged kernels
// (crates/saber-kernels/hip/sattn_prefill.h:1-8: 64 queries x GQA 6 per workgroup with fp8 operand
// legs; sattn_decode.h:1-8: key segments with partial (m, l, O) outputs; sattn_combine.h:1-6).
//
//   S = Q K^T   tcgen05.mma kind::f8f6f4, M = 128 rows, N = 128 keys, K = 256 dims (8 steps);
//               Q is quantised to e4m3 with one scale per row when the tile is loaded, K pages
//               are multiplied as they lie in the pool -- no widening pass;
//   softmax     four warps, one thread per row (= TMEM lane): two passes over the row of S in
//               tensor memory (maximum, then exp2), probabilities to e4m3 in shared memory;
//               the running reference maximum only moves when a tile exceeds it by 2^8 (the
//               probabilities then still fit e4m3), so the accumulator is rarely rescaled;
//   O += P V    tcgen05.mma, M = 128, N = 256 dims, K = 128 keys (4 steps), accumulator in TMEM
//               for the whole key range; S is double-buffered so the tensor core works on the
//               next tile's scores while the softmax warps work on this one.
//
// Page order in the pool (written by rope_kv with page_layout = 1).  Both operands are read with
// NO-swizzle K-major descriptors, whose unit is a core matrix of 8 rows x 16 bytes:
//   K page  [2 key groups][16 dim chunks][8 keys][16 dims]   -> in shared memory the pages of a
//           tile simply follow one another: next 16 dims = +128 B, next 8 keys = +2048 B;
//   V page  [32 dim groups][8 dims][16 keys]                 -> next 16 keys = next page
//           (+4096 B), next 8 dims = +128 B.
// So a page lands with ONE bulk copy (4 KiB) and is an MMA operand as it lands.
//
// Every wait is bounded; a wait that runs out sets the status word and the CTA unwinds.
#include "attn.h"
#include "launch.cuh"
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace saber {

constexpr int kTcThreads = 192;
constexpr int kTcKeys = 128;             // keys per tile
constexpr int kTcPages = kTcKeys / kPageTokens;
constexpr uint32_t kTcQBytes = 32768;    // 128 rows x 256 B
constexpr uint32_t kTcPBytes = 16384;    // 128 rows x 128 B
constexpr uint32_t kTcKVBytes = 32768;   // 8 pages x 4 KiB
constexpr uint32_t kTcSmem = kTcQBytes + 2 * kTcPBytes + 4 * kTcKVBytes + 1024;

// No-swizzle K-major shared-memory descriptor: lbo = byte distance of core matrices adjacent along
// K, sbo = along M / N (8-row groups).
__device__ __forceinline__ uint64_t tc_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

#ifdef SABER_STAMPS
__device__ unsigned long long g_attn_stamps[128];
#define ATTN_STAMP(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) g_attn_stamps[(i)] = globaltimer_ns(); } while (0)
#else
#define ATTN_STAMP(i) do { } while (0)
#endif

__global__ void __launch_bounds__(kTcThreads) attn_tc_kernel(const AttnParams p, const int qt_tokens) {
  pdl_wait();      // (the index tables and the queries are the predecessors' output)
  extern __shared__ uint8_t tc_smem_raw[];
  __shared__ uint64_t bars[16];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem = (smem_u32(tc_smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = smem;
  const uint32_t p_s = q_s + kTcQBytes;              // two probability buffers
  const uint32_t k_s = p_s + 2 * kTcPBytes;          // two stages
  const uint32_t v_s = k_s + 2 * kTcKVBytes;
  const uint32_t bar0 = smem_u32(&bars[0]);
  // K and V run on rings of their own: a K stage is free as soon as its scores are computed, long
  // before the tile's P V, so the keys of tile j + 2 are already in flight while tile j is in the softmax
  const uint32_t k_full = bar0, k_empty = bar0 + 16, v_full = bar0 + 32, v_empty = bar0 + 48;
  const uint32_t s_full = bar0 + 64, p_full = bar0 + 80, o_done = bar0 + 96, q_full = bar0 + 104;

  const int group = p.nq / p.nkv;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z / p.splits, sp = blockIdx.z % p.splits;
  const int head0 = kvh * group;
  const int row0 = p.cu_q[b];
  const int n = p.cu_q[b + 1] - row0;
  const int t0 = blockIdx.x * qt_tokens;
  if (t0 >= n) return;                                 // (uniform for the CTA, before any barrier)
  const int ntok = min(qt_tokens, n - t0);
  const int live = ntok * group;                       // MMA rows in use (<= 128)
  const int rpq = (live + 3) >> 2;                     // live rows per TMEM lane quarter
  const int kvlen = p.kv_len[b];
  const int kbase = kvlen - (n - 1) + t0;              // keys visible to token 0 of the tile (exclusive bound)
  const int kmax = kbase + ntok - 1;
  const int pages = (kmax + kPageTokens - 1) / kPageTokens;
  // sliding window: pages wholly below the first row's window are never touched
  const int pg_first = p.window > 0 ? min(max(0, kbase - p.window) / kPageTokens, pages) : 0;
  const int per = (pages - pg_first + p.splits - 1) / p.splits;
  const int pg0 = pg_first + sp * per, pg1 = min(pages, pg0 + per);
  const int npages = max(0, pg1 - pg0);
  const int ntiles = (npages + kTcPages - 1) / kTcPages;
  const int key_end = pg1 * kPageTokens;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(k_empty + 8 * i, 1);
      mbar_init(v_full + 8 * i, 1);
      mbar_init(v_empty + 8 * i, 1);
      mbar_init(s_full + 8 * i, 1);
      mbar_init(p_full + 8 * i, 128);
    }
    mbar_init(o_done, 1);
    mbar_init(q_full, 128);
    abort_s = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_o = tmem + 256;
  if (threadIdx.x == 0) { ATTN_STAMP(0); }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: pages -> stages
    // lane 0 feeds the K ring, lane 1 the V ring
    if (lane < 2) {
      const bool is_v = lane == 1;
      const uint32_t full = is_v ? v_full : k_full, empty = is_v ? v_empty : k_empty;
      const uint32_t ring = is_v ? v_s : k_s;
      int issued = 0;
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(empty + 8 * s, ((j >> 1) - 1) & 1, p.err, kErrWaitEmpty)) { ok = false; break; }
        mbar_arrive_expect_tx(full + 8 * s, kTcKVBytes);
        for (int pg = 0; pg < kTcPages; ++pg) {
          const int page = pg0 + j * kTcPages + pg;
          int blk = 0;                                   // beyond the range: the null block (zeros)
          if (page < pg1) {
            blk = page < p.max_blocks ? p.block_table[static_cast<size_t>(b) * p.max_blocks + page] : -1;
            if (blk < 0 || (p.n_blocks > 0 && blk >= p.n_blocks)) {   // never follow a bad table entry
              if (p.err) atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrBadIndex));
              blk = 0;
            }
          }
          const uint8_t* src = p.kv_cache + (static_cast<size_t>(blk) * p.nkv + kvh) * (2 * kPageTokens * kHeadDim) + (is_v ? 4096 : 0);
          bulk_g2s(ring + s * kTcKVBytes + pg * 4096, src, 4096, full + 8 * s);
        }
        issued = j + 1;
      }
      if (!ok) {
        abort_s = 1u;
        for (int j = max(0, issued - 2); j < issued; ++j)       // own copies in flight must land first
          mbar_wait(full + 8 * (j & 1), (j >> 1) & 1, p.err, kErrWaitDrain);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && ntiles > 0) {
      const uint32_t idesc_s = make_idesc(kCFmtF32, kFmtE4M3, kFmtE4M3, 128, kTcKeys);
      const uint32_t idesc_o = make_idesc(kCFmtF32, kFmtE4M3, kFmtE4M3, 128, 256);
      bool ok = mbar_wait(q_full, 0, p.err, kErrWaitFull);
      auto qk = [&](int j) {                    // S[j & 1] = Q K_j^T
        const uint64_t a = tc_desc(q_s, 128, 2048);
        const uint64_t bd = tc_desc(k_s + (j & 1) * kTcKVBytes, 128, 2048);
        const uint32_t d = tmem + static_cast<uint32_t>(j & 1) * kTcKeys;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)          // 32 dims = two 16-byte chunks = +256 B
          mma_f8_ss(d, a + static_cast<uint64_t>(ks * 16), bd + static_cast<uint64_t>(ks * 16), idesc_s, ks != 0 ? 1u : 0u);
        mma_commit(s_full + 8 * (j & 1));
        mma_commit(k_empty + 8 * (j & 1));
      };
      if (ok) ok = mbar_wait(k_full, 0, p.err, kErrWaitFull);
      if (ok) { tc_fence_after_sync(); qk(0); }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          if (!mbar_wait(k_full + 8 * ((j + 1) & 1), ((j + 1) >> 1) & 1, p.err, kErrWaitFull)) { ok = false; break; }
          tc_fence_after_sync();
          qk(j + 1);
        }
        if (!mbar_wait(v_full + 8 * (j & 1), (j >> 1) & 1, p.err, kErrWaitFull)) { ok = false; break; }
        if (!mbar_wait(p_full + 8 * (j & 1), (j >> 1) & 1, p.err, kErrWaitReady)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t a = tc_desc(p_s + (j & 1) * kTcPBytes, 128, 1024);
        const uint64_t bd = tc_desc(v_s + (j & 1) * kTcKVBytes, 4096, 128);
#pragma unroll
        for (int ks = 0; ks < kTcKeys / 32; ++ks)     // 32 keys: two probability chunks (+256 B), two pages (+8192 B)
          mma_f8_ss(tmem_o, a + static_cast<uint64_t>(ks * 16), bd + static_cast<uint64_t>(ks * 512), idesc_o,
                    (j != 0 || ks != 0) ? 1u : 0u);
        mma_commit(v_empty + 8 * (j & 1));
        mma_commit(o_done);
      }
      if (!ok) abort_s = 1u;
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = MMA row
    const int qd = warp & 3;                            // TMEM lane quarter of this warp
    const int idx = qd * rpq + lane;                    // live-row index: rows are dealt evenly to the quarters
    const bool row_live = lane < rpq && idx < live;
    const bool warp_live = qd * rpq < live;
    const int h = row_live ? idx / ntok : 0, tok = row_live ? idx - h * ntok : 0;
    const int r = qd * 32 + lane;                       // MMA row = TMEM lane
    const uint32_t t_lane = static_cast<uint32_t>(qd * 32) << 16;
    // ---- Q rows: bf16 -> e4m3 with one scale per row, stored as core matrices (8 rows x 16 dims).
    // A warp walks the live rows of its lane quarter; the 32 lanes fetch one row (512 B) together.
    float q_scale = 0.f;
    for (int i0 = 0; i0 < 32; i0 += 8) {
      // eight rows per round: their loads go out together (one memory round trip per round)
      uint4 raw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u, li = qd * rpq + i;
        raw[u] = make_uint4(0, 0, 0, 0);
        if (i < rpq && li < live) {
          const int hh = li / ntok, tt = li - hh * ntok;
          raw[u] = *(reinterpret_cast<const uint4*>(
              p.q + (static_cast<size_t>(row0 + t0 + tt) * p.nq + head0 + hh) * kHeadDim) + lane);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u;
        const int rr = qd * 32 + i;                               // MMA row
        const uint32_t dst = q_s + (rr >> 3) * 2048 + (rr & 7) * 16 + (lane >> 1) * 128 + (lane & 1) * 8;
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
        float f[8];
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t2 = __bfloat1622float2(h2[e]);
          f[2 * e] = t2.x; f[2 * e + 1] = t2.y;
          amax = fmaxf(amax, fmaxf(fabsf(t2.x), fabsf(t2.y)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float inv = amax > 0.f ? 448.f / amax : 0.f;      // (a dead row is all zeros: stays zeros)
        if (lane == i) q_scale = amax / 448.f;
        const uint32_t lo = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f[0] * inv, f[1] * inv), __NV_SATFINITE, __NV_E4M3)) |
                            (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f[2] * inv, f[3] * inv), __NV_SATFINITE, __NV_E4M3)) << 16);
        const uint32_t hi = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f[4] * inv, f[5] * inv), __NV_SATFINITE, __NV_E4M3)) |
                            (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f[6] * inv, f[7] * inv), __NV_SATFINITE, __NV_E4M3)) << 16);
        asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(dst), "r"(lo), "r"(hi) : "memory");
      }
    }
    fence_proxy_async_smem();
    mbar_arrive(q_full);
    if (warp == 4 && lane == 0) { ATTN_STAMP(1); }

    const float scale_log2 = p.sm_scale * p.k_scale * q_scale * 1.4426950408889634f;
    const int klim = kbase + tok;                        // keys below this bound are visible to the row
    float m_ref = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles; ++j) {
      const uint32_t ts = tmem + t_lane + static_cast<uint32_t>(j & 1) * kTcKeys;
      if (ok) ok = mbar_wait(s_full + 8 * (j & 1), (j >> 1) & 1, p.err, kErrWaitAcc);
      if (!ok || abort_s) { ok = false; break; }
      tc_fence_after_sync();
      if (warp == 4 && lane == 0 && j < 20) { ATTN_STAMP(8 + 4 * j); }
      const int key0 = (pg0 + j * kTcPages) * kPageTokens;
      const int kcap = min(klim, key_end) - key0;        // columns below this bound are live for the row
      const int kfloor = p.window > 0 ? klim - p.window - key0 : 0;     // ... and, with a window, columns from this one on
      float alpha = 1.f;
      if (warp_live) {
        const uint32_t prow = p_s + (j & 1) * kTcPBytes + (r >> 3) * 1024 + (r & 7) * 16;
        const bool full_tile = kcap >= kTcKeys && kfloor <= 0;   // no masking needed for this row
        // (every decision that steers a TMEM load below is made for the WHOLE warp: the loads are
        // warp-collective)
        // Rows without a reference maximum yet (first tile with live keys) take a maximum pass first.
        if (__any_sync(0xffffffffu, row_live && m_ref == -INFINITY)) {
          float tmax = -INFINITY;
#pragma unroll
          for (int c0 = 0; c0 < kTcKeys; c0 += 32) {
            uint32_t sv[32];
            tmem_ld32(ts + c0, sv);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (full_tile || (c0 + i < kcap && c0 + i >= kfloor)) tmax = fmaxf(tmax, __uint_as_float(sv[i]));
          }
          if (row_live && m_ref == -INFINITY) m_ref = tmax * scale_log2;     // (nothing accumulated yet: no rescale)
        }
        // Probability pass against the standing reference, the tile's own maximum on the side.  Only
        // when a row's tile exceeds its reference by more than 2^8 (the probabilities would leave
        // e4m3) the reference moves and the warp does the pass once more.
        float l_tile = 0.f;
        for (int attempt = 0; attempt < 2; ++attempt) {
          const float msafe = m_ref == -INFINITY ? 0.f : m_ref;
          float tmax = -INFINITY;
          l_tile = 0.f;
#pragma unroll
          for (int c0 = 0; c0 < kTcKeys; c0 += 32) {
            uint32_t sv[32];
            tmem_ld32(ts + c0, sv);
            tmem_ld_wait();
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float pv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int c = c0 + 4 * i + e;
                const float sc = __uint_as_float(sv[4 * i + e]);
                const bool on = row_live && (full_tile || (c < kcap && c >= kfloor));
                tmax = on ? fmaxf(tmax, sc) : tmax;
                pv[e] = on ? exp2f(sc * scale_log2 - msafe) : 0.f;
                l_tile += pv[e];
              }
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(pv[0], pv[1]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(pv[2], pv[3]), __NV_SATFINITE, __NV_E4M3);
              w[i] = lo | (hi << 16);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(prow + (c0 >> 4) * 128), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(prow + ((c0 >> 4) + 1) * 128), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
          }
          const float tm = tmax * scale_log2;            // (-inf when the row has no live key in the tile)
          const bool over = row_live && tm > m_ref + 8.f;
          if (over) {
            alpha = exp2f(m_ref - tm);                   // m_ref is finite here: the maximum pass set it
            m_ref = tm;
          }
          if (!__any_sync(0xffffffffu, over)) break;
        }
        l_run = l_run * alpha + l_tile;
      }
      fence_proxy_async_smem();
      if (warp == 4 && lane == 0 && j < 20) { ATTN_STAMP(9 + 4 * j); }
      if (j > 0) {
        // the previous tile's P V must have retired before its accumulator may be rescaled, and
        // before this thread's probability buffer (tile j - 2's) may be considered free next time
        if (ok) ok = mbar_wait(o_done, (j - 1) & 1, p.err, kErrWaitAcc);
        if (!ok) break;
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          tc_fence_after_sync();
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(tmem_o + t_lane + c0, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(tmem_o + t_lane + c0, ov);
          }
          tmem_st_wait();
        }
      }
      tc_fence_before_sync();
      mbar_arrive(p_full + 8 * (j & 1));
      if (warp == 4 && lane == 0 && j < 20) { ATTN_STAMP(10 + 4 * j); }
    }
    if (!ok) abort_s = 1u;
    // ---- epilogue: O / l (one query tile, no split) or the partial (m, l, O) of this key segment
    if (ok && ntiles > 0) ok = mbar_wait(o_done, (ntiles - 1) & 1, p.err, kErrWaitAcc);
    if (warp == 4 && lane == 0) { ATTN_STAMP(2); }
    if (ok && warp_live) {
      tc_fence_after_sync();
      if (p.splits == 1) {
        const float inv = l_run > 0.f ? p.v_scale / l_run : 0.f;
        __nv_bfloat16* dst = row_live ? p.out + (static_cast<size_t>(row0 + t0 + tok) * p.nq + head0 + h) * kHeadDim : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
          uint32_t ov[32];
          if (ntiles > 0) { tmem_ld32(tmem_o + t_lane + c0, ov); tmem_ld_wait(); }
          if (row_live) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float a0 = ntiles > 0 ? __uint_as_float(ov[2 * i]) * inv : 0.f;
              const float a1 = ntiles > 0 ? __uint_as_float(ov[2 * i + 1]) * inv : 0.f;
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(a0, a1);
              pk[i] = *reinterpret_cast<const uint32_t*>(&b2);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(dst + c0 + 8 * i) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
        }
      } else {
        const size_t pbase = row_live ? ((static_cast<size_t>(b) * p.nq + head0 + h) * p.splits + sp) * 16 + tok : 0;
        float* dst = p.part_o + pbase * kHeadDim;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
          uint32_t ov[32];
          if (ntiles > 0) { tmem_ld32(tmem_o + t_lane + c0, ov); tmem_ld_wait(); }
          if (row_live) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              *reinterpret_cast<uint4*>(dst + c0 + 4 * i) =
                  ntiles > 0 ? make_uint4(ov[4 * i], ov[4 * i + 1], ov[4 * i + 2], ov[4 * i + 3]) : make_uint4(0, 0, 0, 0);
          }
        }
        if (row_live) {
          p.part_ml[pbase * 2] = m_ref;
          p.part_ml[pbase * 2 + 1] = l_run;
        }
      }
    }
  }
  if (warp == 4 && lane == 0) { ATTN_STAMP(3); }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace saber

#ifdef SABER_STAMPS
extern "C" int saber_attn_stamps(unsigned long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, saber::g_attn_stamps, sizeof(unsigned long long) * 128));
}
#endif

extern "C" int saber_attn_tc_launch(const saber::AttnParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->nq % p->nkv || p->splits < 1) return static_cast<int>(cudaErrorInvalidValue);
  const int group = p->nq / p->nkv;
  if (group > 16) return static_cast<int>(cudaErrorInvalidValue);
  const int max_rows = p->q_tiles * 16;                 // the caller's bound on the rows of one sequence
  int qt = 128 / group;                                 // tokens of one query tile
  if (p->splits > 1) {
    if (max_rows > 16 || max_rows * group > 128) return static_cast<int>(cudaErrorInvalidValue);   // partials hold 16 rows
    qt = 16;
  }
  const int tiles = (max_rows + qt - 1) / qt;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTcSmem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  dim3 grid(tiles, p->nkv, p->nseq * p->splits);
  saber::launch(attn_tc_kernel, grid, dim3(kTcThreads), kTcSmem, stream, 0, *p, qt);
  return static_cast<int>(cudaGetLastError());
}
