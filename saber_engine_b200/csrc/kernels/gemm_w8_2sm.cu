// int8 x int8 GEMM for long row runs (prefill) on CTA pairs: `tcgen05.mma.cta_group::2`.
//
// A cluster of two CTAs (two neighbouring SMs) computes a 512-row x 256-feature output tile as two 256-row
// halves.  Per k-block each CTA loads ITS two 128-row token tiles (one of each half) and ITS half of the
// weight tile (128 of the 256 feature rows); the leader CTA issues M = 256 MMAs that read both CTAs' shared
// memory, one group per half, and each CTA ends up with two 128-row x 256-column accumulators in its own
// tensor memory.  Per CTA and k-block that is 48 KiB from L2 for 1024 tensor-pipe clocks of work -- the
// one-CTA form (two token tiles per CTA) fetches 64 KiB for the same work, and at 2048 rows both forms are
// bound by that L2 -> SM traffic, not by the tensor pipe (measured: one accumulator per CTA, 32 KiB per 512
// clocks, ran at a third of the pipe).
//
// Hand-over inside the pair (all mbarriers, every wait bounded):
//   full[s]       local: this CTA's two bulk copies of stage s have landed
//   peer_full[s]  in the leader: the peer's relay thread saw ITS full[s] and arrived remotely
//   empty[s]      both CTAs: the leader's commit (multicast to the pair) after the MMAs of stage s
//   acc           both CTAs: the leader's commit after the last MMA; each CTA reads its own lanes
// No load is multicast: every CTA fetches its own operands with plain bulk copies.
// The CTAs of a pair leave together (cluster barrier): a CTA's shared memory and barriers stay valid while
// its partner can still reach them.
//
// Weights: the int8 tile image [N_pad/256][K/128][32768] (rows 0..127 of a tile are its first 16 KiB).
// Tokens: the tiled int8 rows [K/128][M_pad][128].  Output: bf16(acc * a_scale[m] * w_scale[n]), the same
// arithmetic as the one-CTA kernel's plain epilogue, so the bytes are the same.
//
// Parity: the reference's prefill GEMM bodies (`crates/saber-kernels/hip/macaq_iu8f.hip`, WMMA int8 tiles);
// the pairing of SMs has no counterpart there.
#include "gemm_i8.h"
#include "launch.cuh"
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>

namespace saber {

namespace {

constexpr int k2Threads = 192;            // warp 0: copies, warp 1: MMA issue (leader) / relay (peer), warps 2-5: epilogue
constexpr int k2MaxStages = 4;
constexpr uint32_t k2StageBytes = 49152;  // 2 x 16 KiB of token rows (one tile of each 256-row half) + 16 KiB of weight rows

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, uint32_t* err, uint32_t code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((spin & 1023u) == 0u && clock64() - t0 > kWaitLimitCycles) {
      if (err) atomicCAS(err, 0u, code);
      return false;
    }
  }
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_i8_ss2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the leader's commit: one arrival on the barrier at this offset in every CTA of `mask`
__device__ __forceinline__ void mma_commit2(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}

}  // namespace

// grid (2 * M_pad / 512, N_pad / 256), cluster (2, 1, 1), block 192: row tiles run fastest, so the pairs that are
// scheduled together share a weight tile (from memory once, from L2 for the other row tiles)
__global__ void __launch_bounds__(k2Threads, 1) gemm_w8_2sm_kernel(const GemmI8Params p, const int stages) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[3 * k2MaxStages + 1];   // full | peer_full | empty | acc
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;                      // an epilogue thread's wait ran out: all four warps skip together
  __shared__ float w_scale_s[256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
  const int tile_m = blockIdx.x >> 1, tile_n = blockIdx.y;
  const int n0 = tile_n * 256;
  const int m0 = tile_m * 512 + static_cast<int>(rank) * 128;      // this CTA's token rows: m0 .. + 127 and m0 + 256 .. + 383
  const int KB = p.K >> 7;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_peer = smem_u32(&bars[k2MaxStages]);
  const uint32_t bar_empty = smem_u32(&bars[2 * k2MaxStages]);
  const uint32_t bar_acc = smem_u32(&bars[3 * k2MaxStages]);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_peer + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc, 1);
    abort_s = 0;
    mbar_init_fence();
  }
  for (int i = threadIdx.x; i < 256; i += k2Threads) w_scale_s[i] = p.w_scale[n0 + i];
  if (warp == 1) {
    tmem_alloc2(smem_u32(&tmem_base_s), 512);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before anyone signals across
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_base_s;

  if (warp == 0) {
    // ---------------------------------------------------------------- copies of this CTA's operands
    if (lane == 0) {
      const uint8_t* wp = p.w + static_cast<size_t>(tile_n) * KB * 32768 + static_cast<size_t>(rank) * 16384;
      const int8_t* ap = p.a + static_cast<size_t>(m0) * 128;
      const size_t a_kb_stride = static_cast<size_t>(p.M_pad) * 128;
      const uint64_t pol = l2_policy_evict_normal();
      int issued = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const int pre = min(stages, KB);
      // the weight halves go out at once, the token rows after the kernel that produced them has completed
      for (int it = 0; it < pre; ++it) {
        mbar_arrive_expect_tx(bar_full + 8 * it, k2StageBytes);
        bulk_g2s_hint(smem_base + it * k2StageBytes + 32768, wp + static_cast<size_t>(it) * 32768, 16384, bar_full + 8 * it, pol);
      }
      pdl_wait();
      for (int it = 0; it < pre; ++it) {
        bulk_g2s(smem_base + it * k2StageBytes, ap + static_cast<size_t>(it) * a_kb_stride, 16384, bar_full + 8 * it);
        bulk_g2s(smem_base + it * k2StageBytes + 16384, ap + static_cast<size_t>(it) * a_kb_stride + 256 * 128, 16384, bar_full + 8 * it);
      }
      issued = pre;
      if (pre == stages) { s = 0; ph = 1u; } else { s = pre; }
      for (int it = pre; it < KB; ++it) {
        if (!mbar_wait_cluster(bar_empty + 8 * s, ph ^ 1u, p.err, kErrWaitEmpty)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_full + 8 * s, k2StageBytes);
        bulk_g2s_hint(smem_base + s * k2StageBytes + 32768, wp + static_cast<size_t>(it) * 32768, 16384, bar_full + 8 * s, pol);
        bulk_g2s(smem_base + s * k2StageBytes, ap + static_cast<size_t>(it) * a_kb_stride, 16384, bar_full + 8 * s);
        bulk_g2s(smem_base + s * k2StageBytes + 16384, ap + static_cast<size_t>(it) * a_kb_stride + 256 * 128, 16384, bar_full + 8 * s);
        issued = it + 1;
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (!ok) {   // unwinding: no copy of this CTA may still be in flight when it leaves
        for (int it = max(0, issued - stages); it < issued; ++it)
          mbar_wait(bar_full + 8 * (it % stages), (it / stages) & 1, p.err, kErrWaitDrain);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      if (rank == 0) {
        // -------------------------------------------------------------- leader: the pair's MMAs
        const uint32_t idesc = make_idesc(kCFmtS32, kFmtS8, kFmtS8, 256, 256);
        const uint64_t desc_hi = make_desc_k128(0);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int it = 0; it < KB; ++it) {
          if (!mbar_wait(bar_full + 8 * s, ph, p.err, kErrWaitFull)) { ok = false; break; }
          if (!mbar_wait_cluster(bar_peer + 8 * s, ph, p.err, kErrWaitPeer)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * k2StageBytes, b_addr = a_addr + 32768;
          const uint64_t b_desc = desc_hi | static_cast<uint64_t>((b_addr & 0x3FFFFu) >> 4);
#pragma unroll
          for (int j2 = 0; j2 < 2; ++j2) {        // the two 256-row halves: their own token tiles and accumulator columns
            const uint64_t a_desc = desc_hi | static_cast<uint64_t>(((a_addr + j2 * 16384) & 0x3FFFFu) >> 4);
#pragma unroll
            for (int q = 0; q < 4; ++q) mma_i8_ss2(tmem_d + j2 * 256, a_desc + 2 * q, b_desc + 2 * q, idesc, (it | q) != 0 ? 1u : 0u);
          }
          mma_commit2(bar_empty + 8 * s, 3);
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        mma_commit2(bar_acc, 3);
        if (!ok) mbar_wait_cluster(bar_acc, 0, nullptr, 0);      // what was issued retires before the tensor memory goes back
      } else {
        // -------------------------------------------------------------- peer: tell the leader when a stage has landed here
        int s = 0;
        uint32_t ph = 0;
        for (int it = 0; it < KB; ++it) {
          if (!mbar_wait(bar_full + 8 * s, ph, p.err, kErrWaitFull)) break;
          mbar_arrive_remote(mapa_shared(bar_peer + 8 * s, 0));
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: this CTA's 128 rows x 256 columns
    const int tid_t = threadIdx.x - 64;                 // 0..127 = row = tensor-memory lane
    const int q4 = warp & 3;                            // the lanes this warp may read: 32 (warp % 4) ..
    const int row = q4 * 32 + lane;
    const uint32_t t_lane = tmem_d + (static_cast<uint32_t>(q4 * 32) << 16);
    if (!mbar_wait_cluster(bar_acc, 0, p.err, kErrWaitAcc)) abort_s = 1;
    named_bar_sync(1, 128);
    if (abort_s == 0) {
      tc_fence_after_sync();
      // the bf16 tile is staged in the (now idle) stages, 16-byte chunks XOR-swizzled by the row, then whole rows leave
      uint8_t* stage_g = gen_base;
      for (int j2 = 0; j2 < 2; ++j2) {
        const int mb = m0 + j2 * 256;
        const int rows_live = min(128, p.M - mb);
        if (rows_live <= 0) break;                        // (uniform) the second half of a ragged pair is empty
        if (j2 > 0) named_bar_sync(1, 128);               // the staging buffer is free again
        const bool live = row < rows_live;
        const float asc = live ? p.a_scale[mb + row] : 0.f;
        for (int c = 0; c < 256; c += 32) {
          uint32_t r[32];
          tmem_ld32(t_lane + j2 * 256 + c, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float lo = static_cast<float>(static_cast<int32_t>(r[2 * j])) * (asc * w_scale_s[c + 2 * j]);
            const float hi = static_cast<float>(static_cast<int32_t>(r[2 * j + 1])) * (asc * w_scale_s[c + 2 * j + 1]);
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
            pk[j] = *reinterpret_cast<const uint32_t*>(&b2);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t chunk = static_cast<uint32_t>((c >> 3) + j) ^ (static_cast<uint32_t>(row) & 31u);
            *reinterpret_cast<uint4*>(stage_g + row * 512 + (chunk << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
          }
        }
        named_bar_sync(1, 128);
        const int wq = tid_t >> 5;
        const int col = lane * 8;
        if (n0 + col < p.N) {
          for (int rw = wq; rw < rows_live; rw += 4) {
            const uint32_t chunk = static_cast<uint32_t>(lane) ^ (static_cast<uint32_t>(rw) & 31u);
            const uint4 v = *reinterpret_cast<const uint4*>(stage_g + rw * 512 + (chunk << 4));
            *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(mb + rw) * p.ldo + n0 + col) = v;
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // the partner is done with this CTA's shared memory and barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_d, 512);
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Persistent form: one cluster per SM pair walks a list of 512 x 256 output tiles (row groups running fastest).
// The copy ring never drains between tiles -- the next tile's operands arrive while the current tile's
// accumulators are read out -- and the MMAs of the next tile start on an accumulator as soon as BOTH CTAs have
// read it (tfree[half], an mbarrier in the leader that the peer reaches with a remote arrive).  The bf16 rows are
// staged in 32 KiB of their own (a quarter tile at a time), since the ring is busy.
// grid (2 * pairs), cluster (2, 1, 1), block 192; pairs <= SMs / 2.
constexpr uint32_t k2StagingBytes = 32768;
__global__ void __launch_bounds__(k2Threads, 1) gemm_w8_2sm_persistent_kernel(const GemmI8Params p, const int stages) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[3 * k2MaxStages + 3];   // full | peer_full | empty | acc | tfree[2]
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t abort_s;
  __shared__ float w_scale_s[256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pairs = gridDim.x >> 1, pair = blockIdx.x >> 1;
  const int m_groups = (p.M + 511) / 512, n_tiles = p.N_pad / 256;
  const int total = m_groups * n_tiles;
  const int my_tiles = pair < total ? (total - pair + pairs - 1) / pairs : 0;
  const int KB = p.K >> 7;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t ring = smem_base;
  uint8_t* const stage_g = gen_base + static_cast<size_t>(stages) * k2StageBytes;      // bf16 staging behind the ring
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_peer = smem_u32(&bars[k2MaxStages]);
  const uint32_t bar_empty = smem_u32(&bars[2 * k2MaxStages]);
  const uint32_t bar_acc = smem_u32(&bars[3 * k2MaxStages]);
  const uint32_t bar_tfree = smem_u32(&bars[3 * k2MaxStages + 1]);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_peer + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_acc, 1);
    mbar_init(bar_tfree, 2);          // one arrival per CTA of the pair
    mbar_init(bar_tfree + 8, 2);
    abort_s = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(&tmem_base_s), 512);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_base_s;

  if (warp == 0) {
    // ---------------------------------------------------------------- copies: one stream of k-blocks over all tiles
    if (lane == 0) {
      const size_t a_kb_stride = static_cast<size_t>(p.M_pad) * 128;
      const uint64_t pol = l2_policy_evict_normal();
      int s = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true, waited = false;
      for (int ti = 0; ti < my_tiles && ok; ++ti) {
        const int t = pair + ti * pairs;
        const int tile_m = t % m_groups, tile_n = t / m_groups;
        const int m0 = tile_m * 512 + static_cast<int>(rank) * 128;
        const uint8_t* wp = p.w + static_cast<size_t>(tile_n) * KB * 32768 + static_cast<size_t>(rank) * 16384;
        const int8_t* ap = p.a + static_cast<size_t>(m0) * 128;
        for (int kb = 0; kb < KB; ++kb) {
          if (issued >= stages && !mbar_wait_cluster(bar_empty + 8 * s, ph ^ 1u, p.err, kErrWaitEmpty)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_full + 8 * s, k2StageBytes);
          bulk_g2s_hint(ring + s * k2StageBytes + 32768, wp + static_cast<size_t>(kb) * 32768, 16384, bar_full + 8 * s, pol);
          if (!waited) { pdl_wait(); waited = true; }      // token rows: only after the kernel that produced them
          bulk_g2s(ring + s * k2StageBytes, ap + static_cast<size_t>(kb) * a_kb_stride, 16384, bar_full + 8 * s);
          bulk_g2s(ring + s * k2StageBytes + 16384, ap + static_cast<size_t>(kb) * a_kb_stride + 256 * 128, 16384, bar_full + 8 * s);
          ++issued;
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {   // unwinding: no copy of this CTA may still be in flight when it leaves
        for (int it = max(0, issued - stages); it < issued; ++it)
          mbar_wait(bar_full + 8 * (it % stages), (it / stages) & 1, p.err, kErrWaitDrain);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      if (rank == 0) {
        // -------------------------------------------------------------- leader: the pair's MMAs, tile after tile
        const uint32_t idesc = make_idesc(kCFmtS32, kFmtS8, kFmtS8, 256, 256);
        const uint64_t desc_hi = make_desc_k128(0);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        int committed_tiles = 0;
        for (int ti = 0; ti < my_tiles && ok; ++ti) {
          for (int kb = 0; kb < KB; ++kb) {
            if (!mbar_wait(bar_full + 8 * s, ph, p.err, kErrWaitFull)) { ok = false; break; }
            if (!mbar_wait_cluster(bar_peer + 8 * s, ph, p.err, kErrWaitPeer)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_addr = ring + s * k2StageBytes, b_addr = a_addr + 32768;
            const uint64_t b_desc = desc_hi | static_cast<uint64_t>((b_addr & 0x3FFFFu) >> 4);
#pragma unroll
            for (int j2 = 0; j2 < 2; ++j2) {
              if (kb == 0 && ti > 0) {      // the accumulator of the previous tile has been read by both CTAs
                if (!mbar_wait_cluster(bar_tfree + 8 * j2, (ti - 1) & 1, p.err, kErrWaitAcc)) { ok = false; break; }
                tc_fence_after_sync();
              }
              const uint64_t a_desc = desc_hi | static_cast<uint64_t>(((a_addr + j2 * 16384) & 0x3FFFFu) >> 4);
#pragma unroll
              for (int q = 0; q < 4; ++q) mma_i8_ss2(tmem_d + j2 * 256, a_desc + 2 * q, b_desc + 2 * q, idesc, (kb | q) != 0 ? 1u : 0u);
            }
            if (!ok) break;
            mma_commit2(bar_empty + 8 * s, 3);
            if (++s == stages) { s = 0; ph ^= 1u; }
          }
          if (!ok) break;
          mma_commit2(bar_acc, 3);
          committed_tiles = ti + 1;
        }
        // what was issued retires before the tensor memory goes back
        if (!ok && committed_tiles > 0) mbar_wait_cluster(bar_acc, (committed_tiles - 1) & 1, nullptr, 0);
      } else {
        // -------------------------------------------------------------- peer: tell the leader when a stage has landed here
        int s = 0;
        uint32_t ph = 0;
        const long long all = static_cast<long long>(my_tiles) * KB;
        for (long long it = 0; it < all; ++it) {
          if (!mbar_wait(bar_full + 8 * s, ph, p.err, kErrWaitFull)) break;
          mbar_arrive_remote(mapa_shared(bar_peer + 8 * s, 0));
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: per tile, this CTA's 2 x 128 rows x 256 columns
    const int tid_t = threadIdx.x - 64;
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t t_lane = tmem_d + (static_cast<uint32_t>(q4 * 32) << 16);
    const uint32_t tfree_leader = mapa_shared(bar_tfree, 0);
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int t = pair + ti * pairs;
      const int tile_m = t % m_groups, tile_n = t / m_groups;
      const int n0 = tile_n * 256;
      const int m0 = tile_m * 512 + static_cast<int>(rank) * 128;
      w_scale_s[tid_t] = p.w_scale[n0 + tid_t];               // (the previous tile's readers are past their last barrier)
      w_scale_s[tid_t + 128] = p.w_scale[n0 + tid_t + 128];
      if (!mbar_wait_cluster(bar_acc, ti & 1, p.err, kErrWaitAcc)) abort_s = 1;
      named_bar_sync(1, 128);
      if (abort_s != 0) break;                                // (uniform: read after the barrier)
      tc_fence_after_sync();
      for (int j2 = 0; j2 < 2; ++j2) {
        const int mb = m0 + j2 * 256;
        const int rows_live = min(128, p.M - mb);             // may be <= 0: the accumulator is still handed back
        const bool live = row < rows_live;
        const float asc = live ? p.a_scale[mb + row] : 0.f;
        for (int hc = 0; hc < 2; ++hc) {                      // 128 columns at a time through the 32 KiB staging buffer
          for (int c = 0; c < 128; c += 32) {
            uint32_t r[32];
            tmem_ld32(t_lane + j2 * 256 + hc * 128 + c, r);
            tmem_ld_wait();
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float lo = static_cast<float>(static_cast<int32_t>(r[2 * j])) * (asc * w_scale_s[hc * 128 + c + 2 * j]);
              const float hi = static_cast<float>(static_cast<int32_t>(r[2 * j + 1])) * (asc * w_scale_s[hc * 128 + c + 2 * j + 1]);
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
              pk[j] = *reinterpret_cast<const uint32_t*>(&b2);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t chunk = static_cast<uint32_t>((c >> 3) + j) ^ (static_cast<uint32_t>(row) & 15u);
              *reinterpret_cast<uint4*>(stage_g + row * 256 + (chunk << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            }
          }
          if (hc == 1) tc_fence_before_sync();                // this thread's reads of accumulator j2 are complete
          named_bar_sync(1, 128);
          if (hc == 1 && tid_t == 0) {                        // hand accumulator j2 back: one arrival per CTA at the leader
            if (rank == 0) mbar_arrive(bar_tfree + 8 * j2);
            else mbar_arrive_remote(tfree_leader + 8 * j2);
          }
          // whole 256-byte row pieces leave: lanes 0-15 one row, lanes 16-31 the next
          const int col = hc * 128 + (lane & 15) * 8;
          if (n0 + col < p.N) {
            for (int rw = (tid_t >> 5) * 2 + (lane >> 4); rw < rows_live; rw += 8) {
              const uint32_t chunk = static_cast<uint32_t>(lane & 15) ^ (static_cast<uint32_t>(rw) & 15u);
              const uint4 v = *reinterpret_cast<const uint4*>(stage_g + rw * 256 + (chunk << 4));
              *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(mb + rw) * p.ldo + n0 + col) = v;
            }
          }
          named_bar_sync(1, 128);                             // the staging buffer is free again
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_d, 512);
  }
}

}  // namespace saber

// 1 when the shape can run on CTA pairs: int8 weights, whole 512-row groups of token tiles, no tail, no collective.
extern "C" int saber_gemm_w8_2sm_ok(const saber::GemmI8Params* p) {
  return p->w4 == 0 && p->splits == 1 && p->M >= 512 && (p->M_pad % 512) == 0 && (p->K % 128) == 0 && (p->N_pad % 256) == 0 &&
                 (p->N % 8) == 0 && (p->ldo % 8) == 0 && p->tail_mode == 0 && p->tp_nranks <= 1 && p->ag_flags == nullptr &&
                 p->group_tiles == nullptr && p->bias == nullptr && p->epi == 0 && p->halves != 2
             ? 1
             : 0;
}

static int g_2sm_persistent = 1;
extern "C" void saber_set_gemm_2sm_persistent(int on) { g_2sm_persistent = on; }

extern "C" int saber_gemm_w8_2sm_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream) {
  using namespace saber;
  if (!saber_gemm_w8_2sm_ok(p)) return static_cast<int>(cudaErrorInvalidValue);
  if (g_2sm_persistent) {
    if (stages <= 0 || stages > k2MaxStages) stages = k2MaxStages;
    if (stages < 2) stages = 2;
    const int smem = stages * static_cast<int>(k2StageBytes) + static_cast<int>(k2StagingBytes) + 1024;
    static bool configured_p[64];
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) return static_cast<int>(cudaErrorInvalidValue);
    if (dev >= 0 && dev < 64 && !configured_p[dev]) {
      cudaError_t e = cudaFuncSetAttribute(gemm_w8_2sm_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           k2MaxStages * static_cast<int>(k2StageBytes) + static_cast<int>(k2StagingBytes) + 1024);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured_p[dev] = true;
    }
    const int total = ((p->M + 511) / 512) * (p->N_pad / 256);
    const int pairs = total < sms / 2 ? total : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(k2Threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    unsigned n = 1;
    if (pdl_enabled() != 0) {
      attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_w8_2sm_persistent_kernel, *p, stages));
  }
  if (stages <= 0 || stages > k2MaxStages) stages = k2MaxStages;
  if (stages < 2) stages = 2;
  const int smem = stages * static_cast<int>(k2StageBytes) + 1024;
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_w8_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         k2MaxStages * static_cast<int>(k2StageBytes) + 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ((p->M + 511) / 512), p->N_pad / 256, 1);
  cfg.blockDim = dim3(k2Threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  unsigned n = 1;
  if (pdl_enabled() != 0) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_w8_2sm_kernel, *p, stages));
}
