// W4A8 / W8A8 integer GEMM for sm_100a:  out[m, n] = bf16( acc_i32[m, n] * a_scale[m] * w_scale[n] )
// with acc = exact int32 sum over K of a_i8[m, k] * w_i8[n, k].
//
// Parity: this is the role of the reference's default linear path, an exact-int32 W4A8 GEMM with
// per-token activation scales and per-row weight scales where int4 weights are widened to
// 16*w int8 (crates/saber-kernels/hip/macaq_iu8.hip:1-25), including its split-K "last arriver
// reduces" decode form (macaq_iu8.hip:52-150).  The design is not the reference's: it is built
// for the Blackwell tensor core.
//
// Shape of the kernel ("swap-AB"): the WEIGHT tile (128 output features x 128 k) is the M=128
// operand of tcgen05.mma.kind::i8 and the TOKEN tile (nt tokens x 128 k, nt a multiple of 16 up
// to 256) is the N operand, so a decode step with 1..64 rows wastes no tensor-core rows and a
// prefill chunk uses nt=256.  Accumulators live in TMEM (128 lanes x nt int32 columns).
//
// Warp roles (320 threads):
//   warp 0    one elected lane streams weight tiles and activation tiles with bulk async copies
//             (TMA, untiled form: both operands are stored pre-tiled, see below) into a ring of
//             shared-memory stages, completion counted on an mbarrier per stage.
//   warp 1    allocates TMEM; one lane issues 4 x tcgen05.mma (K=32 each) per stage and commits
//             the stage's "empty" barrier, then the accumulator barrier.
//   warps 2-9 W4 only, two groups of four warps taking alternate k-blocks: widen the packed
//             int4 stage in place to int8 (see pack law), then fence.proxy.async + arrive on the
//             stage's "ready" barrier.  Afterwards warps 2-5 are the epilogue: tcgen05.ld their 32 TMEM lanes, scale, store bf16 (direct),
//             or add int32 partials to the split-K workspace where the last-arriving CTA of a
//             tile finishes it (exact: integer addition is order-free) and re-zeroes the scratch.
//
// Operand storage (no tensor maps needed, every copy is one contiguous 16-byte-aligned span):
//   weights      [n_tile][k_block][tile]; an int8 tile is the 16 KiB image of 128 rows x 128 bytes
//                under the 128-byte swizzle (16-byte chunk index XOR (row & 7)).  A W4 tile is
//                8 KiB: byte j = (image[j] >> 4) | (image[j + 8192] & 0xF0) where image holds
//                16*w, so widening is two mask operations per word and lands conflict-free.
//   activations  [k_block][M_pad][128 bytes], the same swizzle keyed on (m & 7); written in that
//                order by the quantising producers.
#include "gemm_i8.h"
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>

namespace saber {

constexpr int kMaxStages = 16;
constexpr int kABufs = 4;           // W4: int8 A-operand buffers in TMEM (32 columns each)
constexpr int kGemmThreads = 320;   // TMA warp, MMA warp, two groups of four transform warps

__global__ void __launch_bounds__(kGemmThreads)
gemm_i8_kernel(const GemmI8Params p, const int stages, const int n_acc) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[2 * kMaxStages + 2 * kABufs + 1];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t is_last_s;
  __shared__ float a_scale_s[256];
  __shared__ uint32_t abort_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool dbg_on = p.dbg != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
#define SABER_STAMP(i) do { if (dbg_on) p.dbg[i] = globaltimer_ns(); } while (0)
  if (threadIdx.x == 0) SABER_STAMP(0);
  const int tile_n = blockIdx.x;
  const int tile_m = blockIdx.y;
  const int split = blockIdx.z;

  const int KB = p.K >> 7;
  const int kb_per = (KB + p.splits - 1) / p.splits;
  const int kb0 = split * kb_per;
  const int kb1 = min(KB, kb0 + kb_per);
  const int nkb = kb1 - kb0;  // host guarantees >= 1
  const int m0 = tile_m * p.nt;
  const uint32_t wbytes = p.w4 ? 8192u : 16384u;
  const uint32_t abytes = static_cast<uint32_t>(p.nt) * 128u;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_smem = smem_base;                                           // stages x abytes
  const uint32_t w_smem = smem_base + static_cast<uint32_t>(stages) * abytes;  // stages x wbytes
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_empty = smem_u32(&bars[kMaxStages]);
  const uint32_t bar_ready = smem_u32(&bars[2 * kMaxStages]);           // kABufs
  const uint32_t bar_afree = smem_u32(&bars[2 * kMaxStages + kABufs]);  // kABufs
  const uint32_t bar_acc = smem_u32(&bars[2 * kMaxStages + 2 * kABufs]);

  uint32_t acc_cols = 32;
  while (acc_cols < static_cast<uint32_t>(p.nt)) acc_cols <<= 1;
  // n_acc independent accumulators: consecutive MMAs then do not wait on one another's result
  // (a chain of dependent tcgen05.mma into one accumulator pays the full MMA latency per link,
  // which for narrow token tiles is far longer than the MMA's own work); the epilogue adds them.
  const uint32_t acc_total = acc_cols * static_cast<uint32_t>(n_acc);
  uint32_t tmem_cols = 32;
  while (tmem_cols < acc_total + (p.w4 ? kABufs * 32u : 0u)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int u = 0; u < kABufs; ++u) {
      mbar_init(bar_ready + 8 * u, 4);  // one arrival per transform warp of the owning group
      mbar_init(bar_afree + 8 * u, 1);
    }
    mbar_init(bar_acc, 1);
    abort_s = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (threadIdx.x == 0) SABER_STAMP(1);
  const uint32_t tmem_d = tmem_base_s;          // accumulator: columns [0, nt)
  const uint32_t tmem_a = tmem_base_s + acc_total;  // W4: A buffers, 32 columns each

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = l2_policy_evict_first();
      const uint8_t* wsrc = p.w + (static_cast<size_t>(tile_n) * KB + kb0) * wbytes;
      const int8_t* asrc = p.a + (static_cast<size_t>(kb0) * p.M_pad + m0) * 128;
      int issued = 0;
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, p.err, kErrWaitEmpty)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_full + 8 * s, wbytes + abytes);
        bulk_g2s_hint(w_smem + s * wbytes, wsrc + static_cast<size_t>(it) * wbytes, wbytes,
                      bar_full + 8 * s, pol);
        bulk_g2s(a_smem + s * abytes, asrc + static_cast<size_t>(it) * p.M_pad * 128, abytes,
                 bar_full + 8 * s);
        issued = it + 1;
        if (it == 0) SABER_STAMP(2);
      }
      if (!ok) {
        // Unwinding: do not leave the CTA while one of its own copies is still in flight.
        for (int it = max(0, issued - stages); it < issued; ++it)
          mbar_wait(bar_full + 8 * (it % stages), (it / stages) & 1, p.err, kErrWaitDrain);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(kCFmtS32, kFmtS8, kFmtS8, 128, p.nt);
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        const int s = it % stages;
        const uint64_t b_desc = make_desc_k128(a_smem + s * abytes);
        if (p.w4) {
          const int u = it % kABufs;
          if (!mbar_wait(bar_ready + 8 * u, (it / kABufs) & 1, p.err, kErrWaitReady)) { ok = false; break; }
          tc_fence_after_sync();
          if (it == 0) SABER_STAMP(5);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {  // K = 32 per MMA: 8 TMEM columns of A, 32 bytes of B
            if (p.dbg_mma && k4 >= p.dbg_mma) break;
            const int g = it * 4 + k4;
            mma_i8_ts(tmem_d + (g % n_acc) * acc_cols, tmem_a + u * 32 + k4 * 8, b_desc + 2 * k4, idesc,
                      g >= n_acc ? 1u : 0u);
          }
          mma_commit(bar_afree + 8 * u);
        } else {
          if (!mbar_wait(bar_full + 8 * s, (it / stages) & 1, p.err, kErrWaitReady)) { ok = false; break; }
          tc_fence_after_sync();
          const uint64_t a_desc = make_desc_k128(w_smem + s * wbytes);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            if (p.dbg_mma && k4 >= p.dbg_mma) break;
            const int g = it * 4 + k4;
            mma_i8_ss(tmem_d + (g % n_acc) * acc_cols, a_desc + 2 * k4, b_desc + 2 * k4, idesc,
                      g >= n_acc ? 1u : 0u);
          }
        }
        mma_commit(bar_empty + 8 * s);
      }
      if (ok) mma_commit(bar_acc);
      SABER_STAMP(6);
    }
  } else {
    // ---------------------------------------------------------------- transform, then epilogue
    const int tid_t = (threadIdx.x - 64) & 127;  // 0..127 inside the group
    const int tgroup = (threadIdx.x - 64) >> 7;  // the two groups take alternate k-blocks
    const int q4 = warp & 3;                     // TMEM lane quarter this warp may access
    bool ok = true;
    if (tgroup == 0) {  // epilogue warps stage the per-token scales while the pipeline fills
      for (int j = tid_t; j < p.nt; j += 128) a_scale_s[j] = (m0 + j < p.M) ? p.a_scale[m0 + j] : 0.f;
    }
    if (p.w4) {
      // Thread = one weight row: 64 packed bytes in, 32 int8 column words out, straight into the
      // TMEM A buffer (lane = row).  Packed tile order is [16-byte chunk j][row][16 bytes], so a
      // warp's loads are contiguous; packed word i carries column word i in its low nibbles and
      // column word 16 + i in its high nibbles.
      const int row = q4 * 32 + lane;
      for (int it = tgroup; it < nkb; it += 2) {
        const int s = it % stages;
        const int u = it % kABufs;
        if (!mbar_wait(bar_full + 8 * s, (it / stages) & 1, p.err, kErrWaitFull)) { ok = false; break; }
        if (it == 0 && tid_t == 0) SABER_STAMP(3);
        const uint32_t base = w_smem + s * wbytes + static_cast<uint32_t>(row) * 16u;
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(pk[4 * j]), "=r"(pk[4 * j + 1]), "=r"(pk[4 * j + 2]), "=r"(pk[4 * j + 3])
                       : "r"(base + j * 2048u));
        uint32_t cols[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          cols[i] = (pk[i] << 4) & 0xF0F0F0F0u;
          cols[16 + i] = pk[i] & 0xF0F0F0F0u;
        }
        if (!mbar_wait(bar_afree + 8 * u, ((it / kABufs) & 1) ^ 1u, p.err, kErrWaitEmpty)) { ok = false; break; }
        tc_fence_after_sync();
        tmem_st32(tmem_a + (static_cast<uint32_t>(q4 * 32) << 16) + u * 32, cols);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ready + 8 * u);
        if (it == 0 && tid_t == 0) SABER_STAMP(4);
      }
    }
    if (tgroup == 0) {
      // the four epilogue warps decide TOGETHER whether to run the epilogue: the named barriers
      // below have no time limit, so no warp may skip one that the others enter
      if (ok) ok = mbar_wait(bar_acc, 0, p.err, kErrWaitAcc);
      if (!ok) abort_s = 1u;
      named_bar_sync(1, 128);  // also publishes a_scale_s
      ok = abort_s == 0u;
    } else {
      ok = false;  // only the first group (TMEM lane quarters 2,3,0,1) is the epilogue
    }
    if (ok) {
      tc_fence_after_sync();
      if (tid_t == 0) SABER_STAMP(7);
      const int q = q4;
      const int n_live_acc = min(n_acc, nkb * 4);  // accumulators that received at least one MMA
      const int row = q * 32 + lane;
      const int n = tile_n * 128 + row;
      const bool n_ok = n < p.N;
      const float wsn = n_ok ? p.w_scale[n] : 0.f;
      const int mt = min(p.nt, p.M - m0);  // live token rows of this tile
      const int nchunks = (mt + 15) >> 4;
      if (p.splits == 1) {
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[16];
          tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c * 16, r);
          tmem_ld_wait();
          for (int a = 1; a < n_live_acc; ++a) {
            uint32_t r2[16];
            tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + a * acc_cols + c * 16, r2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] += r2[j];
          }
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c * 16 + j;
              if (m < p.M) {
                const float v = static_cast<float>(static_cast<int32_t>(r[j])) * (a_scale_s[c * 16 + j] * wsn);
                p.out[static_cast<size_t>(m) * p.ldo + n] = __float2bfloat16(v);
              }
            }
          }
        }
      } else {
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[16];
          tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + c * 16, r);
          tmem_ld_wait();
          for (int a = 1; a < n_live_acc; ++a) {
            uint32_t r2[16];
            tmem_ld16(tmem_d + (static_cast<uint32_t>(q * 32) << 16) + a * acc_cols + c * 16, r2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] += r2[j];
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c * 16 + j;
            if (m < p.M) atomicAdd(p.ws + static_cast<size_t>(m) * p.N_pad + tile_n * 128 + row,
                                   static_cast<int32_t>(r[j]));
          }
        }
        __threadfence();
        named_bar_sync(1, 128);
        const int tile_id = tile_m * gridDim.x + tile_n;
        if (tid_t == 0) {
          const uint32_t old = atomicAdd(p.counters + tile_id, 1u);
          is_last_s = (old == static_cast<uint32_t>(p.splits - 1)) ? 1u : 0u;
        }
        named_bar_sync(1, 128);
        if (is_last_s) {
          __threadfence();
          int32_t* wbase = p.ws + static_cast<size_t>(m0) * p.N_pad + tile_n * 128 + row;
          for (int j0 = 0; j0 < mt; j0 += 16) {
            int32_t acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)   // independent loads first, then the dependent work
              acc[j] = (j0 + j < mt) ? __ldcg(wbase + static_cast<size_t>(j0 + j) * p.N_pad) : 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j0 + j < mt) {
                wbase[static_cast<size_t>(j0 + j) * p.N_pad] = 0;  // scratch is left zeroed
                if (n_ok)
                  p.out[static_cast<size_t>(m0 + j0 + j) * p.ldo + n] =
                      __float2bfloat16(static_cast<float>(acc[j]) * (a_scale_s[j0 + j] * wsn));
              }
            }
          }
          if (tid_t == 0) p.counters[tile_id] = 0u;
        }
      }
    }
  }

  if (threadIdx.x == 64) SABER_STAMP(8);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, tmem_cols);
  if (threadIdx.x == 32) SABER_STAMP(9);
#undef SABER_STAMP
}

}  // namespace saber

extern "C" int saber_gemm_i8_smem_bytes_w(int nt, int stages, int w4) {
  return stages * ((w4 ? 8192 : 16384) + nt * 128) + 1024;
}
extern "C" int saber_gemm_i8_smem_bytes(int nt, int stages) {
  return saber_gemm_i8_smem_bytes_w(nt, stages, 0);
}

extern "C" int saber_gemm_i8_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream) {
  using namespace saber;
  if (p->nt < 16 || p->nt > 256 || (p->nt & 15) || (p->K & 127) || p->K <= 0 || p->M <= 0 ||
      (p->N_pad & 127) || p->splits < 1 || (p->M_pad % p->nt) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const int KB = p->K >> 7;
  const int kb_per = (KB + p->splits - 1) / p->splits;
  if ((p->splits - 1) * kb_per >= KB) return static_cast<int>(cudaErrorInvalidValue);
  const int kSmemLimit = 224 * 1024;  // opt-in maximum minus the kernel's static shared memory
  if (stages <= 0) {
    // default: small token tiles leave room for two CTAs per SM (one's epilogue overlaps the
    // other's main loop); wide tiles take the whole SM
    const int budget = p->nt <= 128 ? 112 * 1024 : kSmemLimit;
    stages = (budget - 1024) / ((p->w4 ? 8192 : 16384) + p->nt * 128);
  }
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  while (stages > 2 && saber_gemm_i8_smem_bytes_w(p->nt, stages, p->w4) > kSmemLimit) --stages;
  // The two transform groups take alternate k-blocks; with an even ring depth every stage always
  // belongs to the same group, so each waiter sees every phase of the barriers it waits on (a
  // parity wait may lag its barrier by at most one phase).
  if (p->w4 && (stages & 1)) --stages;
  if (stages < 2) stages = 2;
  const int smem = saber_gemm_i8_smem_bytes_w(p->nt, stages, p->w4);
  if (smem > kSmemLimit) return static_cast<int>(cudaErrorInvalidValue);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemLimit);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(p->N_pad / 128, (p->M + p->nt - 1) / p->nt, p->splits);
  // accumulator count: as many as fit beside the A buffers without exceeding 256 TMEM columns
  // (two CTAs per SM) for narrow tiles, 512 for wide ones
  int acc_cols = 32;
  while (acc_cols < p->nt) acc_cols <<= 1;
  const int a_cols = p->w4 ? kABufs * 32 : 0;
  int n_acc = 1;
  const int budget_cols = (acc_cols <= 64) ? 256 : 512;
  while (n_acc < 4 && acc_cols * (n_acc + 1) + a_cols <= budget_cols) ++n_acc;
  gemm_i8_kernel<<<grid, kGemmThreads, smem, stream>>>(*p, stages, n_acc);
  return static_cast<int>(cudaGetLastError());
}
