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
// Warp roles (192 threads):
//   warp 0    one elected lane streams weight tiles and activation tiles with bulk async copies
//             (TMA, untiled form: both operands are stored pre-tiled, see below) into a ring of
//             shared-memory stages, completion counted on an mbarrier per stage.
//   warp 1    allocates TMEM; one lane issues 4 x tcgen05.mma (K=32 each) per stage and commits
//             the stage's "empty" barrier, then the accumulator barrier.
//   warps 2-5 W4 only: widen the packed int4 stage in place to int8 (see pack law), then
//             fence.proxy.async + arrive on the stage's "ready" barrier.  Afterwards the same four
//             warps are the epilogue: tcgen05.ld their 32 TMEM lanes, scale, store bf16 (direct),
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

constexpr int kMaxStages = 12;
constexpr int kGemmThreads = 192;

__global__ void __launch_bounds__(kGemmThreads)
gemm_i8_kernel(const GemmI8Params p, const int stages) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[3 * kMaxStages + 1];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t is_last_s;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
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
  const uint32_t w_smem = smem_base;                                   // stages x 16 KiB
  const uint32_t a_smem = smem_base + static_cast<uint32_t>(stages) * 16384u;  // stages x abytes
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_empty = smem_u32(&bars[kMaxStages]);
  const uint32_t bar_ready = smem_u32(&bars[2 * kMaxStages]);
  const uint32_t bar_acc = smem_u32(&bars[3 * kMaxStages]);

  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.nt)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_ready + 8 * s, 128);
    }
    mbar_init(bar_acc, 1);
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_base_s;

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
        bulk_g2s_hint(w_smem + s * 16384u + (p.w4 ? 8192u : 0u), wsrc + static_cast<size_t>(it) * wbytes,
                      wbytes, bar_full + 8 * s, pol);
        bulk_g2s(a_smem + s * abytes, asrc + static_cast<size_t>(it) * p.M_pad * 128, abytes,
                 bar_full + 8 * s);
        issued = it + 1;
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
        const uint32_t ph = (it / stages) & 1;
        const uint32_t wait_bar = (p.w4 ? bar_ready : bar_full) + 8 * s;
        if (!mbar_wait(wait_bar, ph, p.err, kErrWaitReady)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t a_desc = make_desc_k128(w_smem + s * 16384u);
        const uint64_t b_desc = make_desc_k128(a_smem + s * abytes);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          // 32 int8 = 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units.
          mma_i8_ss(tmem_d, a_desc + 2 * k4, b_desc + 2 * k4, idesc, (it | k4) != 0 ? 1u : 0u);
        }
        mma_commit(bar_empty + 8 * s);
      }
      if (ok) mma_commit(bar_acc);
    }
  } else {
    // ---------------------------------------------------------------- transform, then epilogue
    const int tid_t = threadIdx.x - 64;  // 0..127
    bool ok = true;
    if (p.w4) {
      for (int it = 0; it < nkb; ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(bar_full + 8 * s, ph, p.err, kErrWaitFull)) { ok = false; break; }
        const uint32_t base = w_smem + s * 16384u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t off = static_cast<uint32_t>(i * 128 + tid_t) * 16u;
          uint32_t v0, v1, v2, v3;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                       : "r"(base + 8192u + off));
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + off),
                       "r"((v0 << 4) & 0xF0F0F0F0u), "r"((v1 << 4) & 0xF0F0F0F0u),
                       "r"((v2 << 4) & 0xF0F0F0F0u), "r"((v3 << 4) & 0xF0F0F0F0u)
                       : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + 8192u + off),
                       "r"(v0 & 0xF0F0F0F0u), "r"(v1 & 0xF0F0F0F0u), "r"(v2 & 0xF0F0F0F0u),
                       "r"(v3 & 0xF0F0F0F0u)
                       : "memory");
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_ready + 8 * s);
      }
    }
    if (ok) ok = mbar_wait(bar_acc, 0, p.err, kErrWaitAcc);
    if (ok) {
      tc_fence_after_sync();
      const int q = warp & 3;  // TMEM lane quarter this warp may read
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
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int m = m0 + c * 16 + j;
              if (m < p.M) {
                const float v = static_cast<float>(static_cast<int32_t>(r[j])) * (p.a_scale[m] * wsn);
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
          for (int j = 0; j < mt; ++j) {
            const int m = m0 + j;
            int32_t* wp = p.ws + static_cast<size_t>(m) * p.N_pad + tile_n * 128 + row;
            const int32_t acc = __ldcg(wp);
            *wp = 0;  // the scratch is left zeroed for the next launch
            if (n_ok) {
              const float v = static_cast<float>(acc) * (p.a_scale[m] * wsn);
              p.out[static_cast<size_t>(m) * p.ldo + n] = __float2bfloat16(v);
            }
          }
          if (tid_t == 0) p.counters[tile_id] = 0u;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, tmem_cols);
}

}  // namespace saber

extern "C" int saber_gemm_i8_smem_bytes(int nt, int stages) {
  return stages * (16384 + nt * 128) + 1024;
}

extern "C" int saber_gemm_i8_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream) {
  using namespace saber;
  if (p->nt < 16 || p->nt > 256 || (p->nt & 15) || (p->K & 127) || p->K <= 0 || p->M <= 0 ||
      (p->N_pad & 127) || p->splits < 1 || (p->M_pad % p->nt) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const int KB = p->K >> 7;
  const int kb_per = (KB + p->splits - 1) / p->splits;
  if ((p->splits - 1) * kb_per >= KB) return static_cast<int>(cudaErrorInvalidValue);
  const int kSmemLimit = 226 * 1024;  // opt-in maximum minus the kernel's static shared memory
  if (stages <= 0) {
    // default: small token tiles leave room for two CTAs per SM (one's epilogue overlaps the
    // other's main loop); wide tiles take the whole SM
    const int budget = p->nt <= 64 ? 112 * 1024 : kSmemLimit;
    stages = (budget - 1024) / (16384 + p->nt * 128);
  }
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  while (stages > 2 && saber_gemm_i8_smem_bytes(p->nt, stages) > kSmemLimit) --stages;
  const int smem = saber_gemm_i8_smem_bytes(p->nt, stages);
  if (smem > kSmemLimit) return static_cast<int>(cudaErrorInvalidValue);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemLimit);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid(p->N_pad / 128, (p->M + p->nt - 1) / p->nt, p->splits);
  gemm_i8_kernel<<<grid, kGemmThreads, smem, stream>>>(*p, stages);
  return static_cast<int>(cudaGetLastError());
}
