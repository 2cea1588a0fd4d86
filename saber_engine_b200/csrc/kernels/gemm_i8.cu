// W4A8 / W8A8 integer GEMM for sm_100a:  out[m, n] = bf16( acc_i32[m, n] * a_scale[m] * w_scale[n] )
// with acc = exact int32 sum over K of a_i8[m, k] * w_i8[n, k].
//
// Parity: this is the role of the reference's default linear path, an exact-int32 W4A8 GEMM with
// per-token activation scales and per-row weight scales where int4 weights are widened to
// 16*w int8 (crates/saber-kernels/hip/macaq_iu8.hip:1-25), including its split-K "last arriver
// reduces" decode form (macaq_iu8.hip:52-150).  The design is not the reference's: it is built
// around how the Blackwell tensor core spends its time.
//
// Orientation.  A tcgen05.mma of shape M x N x 32 bytes takes about M clocks whatever N is (the
// array is N <= 256 wide and streams the M rows), so a weight-streaming GEMM wants the WEIGHTS on
// the N side, 256 output features per instruction, and the few token rows on the M side.  Measured
// on B200: with weights as the M = 128 operand a single CTA retired one 128 x 128-byte k-block
// per ~0.4 us, capping W4 decode near 4.5 TB/s of packed weights; this orientation halves the
// tensor time per weight byte.  Token rows beyond the live ones are never loaded: D rows are
// independent, so whatever shared memory holds there only lands in accumulator rows nobody reads.
//
// Warp roles (320 threads):
//   warp 0    one lane streams weight and activation tiles with bulk async copies (TMA, untiled
//             form: both operands are stored pre-tiled) into a deep ring of stages (packed int4
//             stages are 16 KiB, so six of them keep ~100 KB of weights in flight per SM),
//             completion counted on one mbarrier per stage.
//   warp 1    allocates TMEM (256 int32 columns x 128 lanes); one lane issues 4 x
//             tcgen05.mma.kind::i8 (K = 32 each) per stage and commits the stage's "empty" barrier.
//   warps 2-9 W4 only: all eight warps widen a packed int4 stage into one of three int8 operand
//             buffers (two mask operations per word, conflict-free), then
//             fence.proxy.async and one elected arrive per warp on the stage's "ready" barrier.
//             Afterwards warps 2-5 are the epilogue: tcgen05.ld their 32 TMEM lanes (lane = token),
//             scale, 16-byte bf16 stores (direct), or int32 red.add into the split-K scratch where
//             the last-arriving CTA of a tile finishes it (exact: integer addition is order-free)
//             and re-zeroes the scratch.
//   Loop indices in the single-thread roles advance incrementally: a division by a run-time value
//   costs that lone thread more than the copy or MMA it is about to issue.
//
// Operand storage (no tensor maps needed, every copy is one contiguous 16-byte-aligned span):
//   weights      [n_tile (256 rows)][k_block (128)][tile]; an int8 tile is the 32 KiB image of 256
//                rows x 128 bytes under the 128-byte swizzle (16-byte chunk index XOR (row & 7)).
//                A W4 tile is 16 KiB: byte j = (image[j] >> 4) | (image[j + 16384] & 0xF0) where
//                image holds 16*w.
//   activations  [k_block][M_pad][128 bytes], the same swizzle keyed on (m & 7); written in that
//                order by the quantising producers.
#include "gemm_i8.h"
#include "launch.cuh"
#include "gemm_i8_noalloc.h"
#include "ptx_sm100.cuh"
#include "rowops_body.cuh"
#include <cuda_bf16.h>
#include <type_traits>

namespace saber {

constexpr int kMaxStages = 12;
constexpr int kGemmThreads = 320;
constexpr uint32_t kTileBytes = 32768;   // int8 image of one weight tile (256 x 128)
constexpr int kTailFlagsAt = 64 + 256 * 32;   // word offset of the per-tile "accumulator block is clean" flags in tail_sync
constexpr int kUBufs = 3;                // W4: widened int8 operand buffers (transform, MMA and
                                         // the buffer-free round trip overlap with three)

// GELU of a rounded linear output: tanh form (x * 0.5 * (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))) or erf form.
__device__ __forceinline__ float gelu_f(float x, bool erf_form) {
  if (erf_form) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}

// Grid-wide barrier for grids that are resident as a whole (one CTA per SM, grid <= SM count).  ONE
// thread per CTA calls, after a CTA-level barrier that ordered the other threads' writes before it.
// `ctr` is zero when the kernel starts.  The wait is bounded like every other wait here: when it
// runs out the status word is set and the caller goes on (its results are then garbage, the error
// is what the host reads).  grid_depart is the second round of arrivals.
__device__ __forceinline__ bool grid_arrive_wait(uint32_t* ctr, uint32_t n_ctas, uint32_t* err) {
  __threadfence();
  // (inc wraps to zero on the 2 n-th increment: n arrivals, then n departures, re-arm the word)
  asm volatile("red.global.inc.u32 [%0], %1;" ::"l"(ctr), "r"(2u * n_ctas - 1u) : "memory");
  const long long t0 = clock64();
  for (uint32_t polls = 0;; ++polls) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(ctr) : "memory");
    if (seen >= n_ctas) return true;
    if ((polls & 1023u) == 1023u && clock64() - t0 > kWaitLimitCycles) {
      if (err) atomicCAS(err, 0u, static_cast<uint32_t>(kErrWaitSplit));
      return false;
    }
  }
}
// Second round of arrivals: fire and forget, the last one wraps the counter back to zero.
__device__ __forceinline__ void grid_depart(uint32_t* ctr, uint32_t n_ctas) {
  asm volatile("red.global.inc.u32 [%0], %1;" ::"l"(ctr), "r"(2u * n_ctas - 1u) : "memory");
}

// kLean: the grouped (mixture-of-experts) instantiation -- no split-K and no tensor-parallel code,
// two operand buffers instead of three, at most 102 registers -- so that TWO CTAs share an SM: an
// expert tile is only 16 k-blocks long, and the second CTA's main loop hides the first one's
// start-up latency (cold weights: 3-4 us to the first MMA) and epilogue.
// kBf: the bf16 x bf16 instantiation (optional scales, bias, activation / residual epilogue); the
// integer and MXFP4 instantiations compile none of it.
// kFp4: native block-scaled FP4 x FP4 (tcgen05.mma kind::mxf4nvf4 / kind::mxf4): both operands stay
// packed e2m1 in shared memory (a 32 KiB stage is 256 features x 256 k), their block scales ride
// behind the tiles, are copied into tensor memory by tcgen05.cp and applied by the tensor core; no
// transform warps, fp32 accumulators, the per-token and per-tensor scales in the epilogue.
template <bool kLean, bool kBf = false, bool kFp4 = false>
__device__ __forceinline__ void gemm_i8_body(const GemmI8Params& p, const int stages, const RowOpParams* tail) {
  const int nub = (kLean || p.mtiles == 2) ? 2 : kUBufs;     // operand buffers in use
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bars[2 * kMaxStages + 2 * kUBufs + 1];
  __shared__ uint32_t tmem_base_s;
  __shared__ uint32_t is_last_s;
  __shared__ uint32_t abort_s;
  __shared__ float w_scale_s[256];
  __shared__ float bias_s[kBf ? 256 : 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef SABER_STAMPS
  // timing stamps (instrumented build only): CTA (0,0,0), or (dbg_mma == 2) 16 slots for every CTA
  const bool dbg_all = p.dbg != nullptr && p.dbg_mma == 2;
  const bool dbg_on = p.dbg != nullptr && (dbg_all || (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0));
  const size_t dbg_base = dbg_all ? 16u * ((static_cast<size_t>(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) : 0u;
#define SABER_STAMP(i) do { if (dbg_on) p.dbg[dbg_base + (i)] = globaltimer_ns(); } while (0)
#else
#define SABER_STAMP(i) do { } while (0)
#endif
  if (threadIdx.x == 0) SABER_STAMP(0);
  // Programmatic dependent launch: this kernel may be running ahead of its predecessor, so only
  // WEIGHTS (which no kernel writes) are touched before pdl_wait().  It never triggers its own
  // dependents early: CTAs of a successor placed while this grid holds the SMs would pile up on
  // the few SMs it leaves free.
  // half tiles (p.halves == 2): two CTAs share a packed weight tile, each widens and multiplies only
  // its 128 rows of it (the low or the high nibbles) -- twice the CTAs without split-K
  const int halves = (!kLean && !kBf && p.halves == 2) ? 2 : 1;
  // Two token tiles per CTA (long row runs): the grid is (token tile pairs, feature tiles), so CTAs that are
  // scheduled together share a weight tile -- it comes from memory once and from L2 for the other row tiles
  // (with the feature tile running fastest every row-tile wave would stream the whole weight again).
  const bool raster_m = !kLean && p.mtiles == 2;
  const int grid_n = raster_m ? static_cast<int>(gridDim.y) : static_cast<int>(gridDim.x);
  const int tile_n = raster_m ? static_cast<int>(blockIdx.y)
                              : (halves == 2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x));
  const int half = halves == 2 ? static_cast<int>(blockIdx.x & 1u) : 0;
  const int tile_m = raster_m ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.y);
  const int split = blockIdx.z;

  const int KB = p.K >> 7;
  const int kb_per = (KB + p.splits - 1) / p.splits;
  const int kb0 = split * kb_per;
  const int kb1 = min(KB, kb0 + kb_per);
  const int nkb = kb1 - kb0;  // host guarantees >= 1
  // grouped mode: this CTA's token rows and expert come from the tile table
  // token tiles per CTA: 2 (prefill) = every widened weight block feeds two MMAs into two accumulators
  const int mt2 = (!kLean && p.mtiles == 2) ? 2 : 1;
  int m0 = tile_m * p.nt * mt2;
  int rows_here = -1;
  const uint8_t* w_base = p.w;
  const float* w_scale_base = p.w_scale;
  if (p.group_tiles != nullptr) {
    pdl_wait();                                 // the tile table is the routing kernels' output
    if (tile_m >= *p.group_ntiles) return;      // uniform for the whole CTA, before any barrier
    const int4 t = p.group_tiles[tile_m];
    m0 = t.y;
    rows_here = t.z;
    w_base += static_cast<size_t>(t.x) * p.group_w_stride;
    w_scale_base += static_cast<size_t>(t.x) * p.N_pad;
  }
  const int n0 = tile_n * 256 + half * 128;
  // weight formats: 0 = int8 tiles, 1 = packed int4, 2 = MXFP4 (packed e2m1 + 1 KiB of block shifts)
  // 3 = bf16 x bf16: both operands pass through like int8 tiles (K counted in bytes), fp32 accumulators
  const bool mx = !kBf && !kFp4 && p.w4 == 2;
  constexpr bool bf = kBf;
  const bool widen = !kBf && !kFp4 && p.w4 != 0;
  // FP4: w4 = 4 is NVFP4 (e4m3 scale per 16 values: 16 scales per row and k-block), 5 is MXFP4 (e8m0 per 32: 8).
  // Scales are stored as 512-byte atoms (128 rows x 4 scales, byte (r % 32) * 16 + (r / 32) * 4 + s):
  // the shape tcgen05.cp moves into four tensor-memory columns.
  const bool nv = kFp4 && p.w4 == 4;
  const uint32_t sf_atoms = nv ? 4u : 2u;                   // atoms along K per k-block and 128 rows
  const uint32_t sfa_bytes = kFp4 ? sf_atoms * 512u : 0u;   // tokens: one 128-row chunk
  const uint32_t wbytes = kFp4 ? 32768u + 2u * sf_atoms * 512u : (mx ? 17408u : (widen ? 16384u : 32768u));
  const uint32_t abytes = static_cast<uint32_t>(p.nt) * 128u * static_cast<uint32_t>(mt2);

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // token ring | W4: three int8 operand buffers | weight ring (W4: packed 16 KiB stages, W8: 32 KiB)
  const uint32_t a_smem = smem_base;
  const uint32_t u_smem = smem_base + static_cast<uint32_t>(stages) * abytes;
  const uint32_t w_smem = u_smem + (widen ? nub * kTileBytes : 0u);
  const uint32_t sfa_smem = w_smem + static_cast<uint32_t>(stages) * wbytes;     // FP4: token scales, one 128-row chunk per stage
  const uint32_t bar_full = smem_u32(&bars[0]);
  const uint32_t bar_empty = smem_u32(&bars[kMaxStages]);
  const uint32_t bar_ready = smem_u32(&bars[2 * kMaxStages]);           // kUBufs
  const uint32_t bar_ufree = smem_u32(&bars[2 * kMaxStages + kUBufs]);  // kUBufs
  const uint32_t bar_acc = smem_u32(&bars[2 * kMaxStages + 2 * kUBufs]);
  const uint32_t kTmemCols = (kFp4 || (!kLean && p.mtiles == 2)) ? 512u : 256u;     // FP4: 256 accumulator + 2 x 48 scale columns
  constexpr int kMaxSplits = 8;   // split-K factor the reduction is unrolled for

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int u = 0; u < nub; ++u) {
      mbar_init(bar_ready + 8 * u, 4);  // one arrival per warp of the transform group that owns the block
      mbar_init(bar_ufree + 8 * u, 1);
    }
    mbar_init(bar_acc, 1);
    abort_s = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (threadIdx.x == 0) SABER_STAMP(1);
  const uint32_t tmem_d = tmem_base_s;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      const uint64_t pol = raster_m ? l2_policy_evict_normal() : l2_policy_evict_first();   // pairs: the tile is re-read by the other row tiles
      const uint8_t* wp = w_base + (static_cast<size_t>(tile_n) * KB + kb0) * wbytes;
      const int8_t* ap = p.a + (static_cast<size_t>(kb0) * p.M_pad + m0) * 128;
      const size_t a_kb_stride = static_cast<size_t>(p.M_pad) * 128;
      // FP4: the token scales of this CTA's 128-row chunk, one run of atoms per k-block
      const size_t sf_kb_stride = static_cast<size_t>((p.M_pad + 127) >> 7) * sfa_bytes;
      const uint8_t* sfp = kFp4 ? p.a_sf + static_cast<size_t>(kb0) * sf_kb_stride + static_cast<size_t>(m0 >> 7) * sfa_bytes : nullptr;
      int issued = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      // first pass over the ring: the weight tiles go out at once, the token tiles only after the
      // predecessor kernel (which produced them) has completed
      const int pre = min(stages, nkb);
      for (int it = 0; it < pre; ++it) {
        mbar_arrive_expect_tx(bar_full + 8 * it, wbytes + abytes + sfa_bytes);
        bulk_g2s_hint(w_smem + it * wbytes, wp, wbytes, bar_full + 8 * it, pol);
        wp += wbytes;
        if (it == 0) SABER_STAMP(2);
      }
      pdl_wait();
      if (!kLean && p.ag_flags != nullptr) {
        // all-gather fused into the operand load: the owners of these token rows push them into
        // local memory and raise one flag per 128-row tile; wait for it (bounded) before the
        // first token-tile copy of this CTA
        const uint32_t seq = *p.ag_seq_base + static_cast<uint32_t>(p.ag_site) + 1u;
        const uint32_t* flag = p.ag_flags + (seq & 1u) * 64u + static_cast<uint32_t>(m0 >> 7);
        const int last_tile = min((p.M - 1) >> 7, (m0 + p.nt * mt2 - 1) >> 7) - (m0 >> 7);   // 0, or 1 with two token tiles
        const long long t0 = clock64();
        for (uint32_t polls = 0;; ++polls) {
          uint32_t v, v2;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v2) : "l"(flag + last_tile) : "memory");
          if (static_cast<int32_t>(v - seq) >= 0 && static_cast<int32_t>(v2 - seq) >= 0) break;
          // (half the limit of the pipeline's own waits, so that this cause is the one recorded)
          if ((polls & 1023u) == 1023u && clock64() - t0 > kWaitLimitCycles / 2) {
            atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrWaitPeer));
            break;     // the status word is set; the copies below read whatever is there
          }
        }
      }
      for (int it = 0; it < pre; ++it) {
        bulk_g2s(a_smem + it * abytes, ap, abytes, bar_full + 8 * it);
        ap += a_kb_stride;
        if constexpr (kFp4) {
          bulk_g2s(sfa_smem + it * sfa_bytes, sfp, sfa_bytes, bar_full + 8 * it);
          sfp += sf_kb_stride;
        }
      }
      issued = pre;
      if (pre == stages) { s = 0; ph = 1u; } else { s = pre; }
      for (int it = pre; it < nkb; ++it) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, p.err, kErrWaitEmpty)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_full + 8 * s, wbytes + abytes + sfa_bytes);
        bulk_g2s_hint(w_smem + s * wbytes, wp, wbytes, bar_full + 8 * s, pol);
        bulk_g2s(a_smem + s * abytes, ap, abytes, bar_full + 8 * s);
        if constexpr (kFp4) {
          bulk_g2s(sfa_smem + s * sfa_bytes, sfp, sfa_bytes, bar_full + 8 * s);
          sfp += sf_kb_stride;
        }
        wp += wbytes;
        ap += a_kb_stride;
        issued = it + 1;
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (!kLean && ok && p.next_w != nullptr) {
        // every copy of this CTA is issued: ask L2 for the leading weight tiles of the next GEMM's
        // CTAs (weights are never written, so this is safe whatever runs in between)
        const int g_ctas = gridDim.x * gridDim.y * gridDim.z;
        const int me = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
        const int n_next = p.next_tiles * p.next_splits;
        for (int j = me; j < n_next; j += g_ctas) {
          const int tn = j / p.next_splits, sp = j - tn * p.next_splits;
          const int kbeg = sp * p.next_kb_per;
          const int cnt = min(p.next_pref, p.next_KB - kbeg);
          const uint8_t* src = p.next_w + (static_cast<size_t>(tn) * p.next_KB + kbeg) * static_cast<size_t>(p.next_wbytes);
          for (int t = 0; t < cnt; ++t)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src + static_cast<size_t>(t) * p.next_wbytes),
                         "r"(static_cast<uint32_t>(p.next_wbytes)) : "memory");
        }
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
      // M = 128 token rows (only the first nt are real), N = 256 output features
      const uint32_t idesc = mx ? make_idesc(kCFmtF32, kFmtE4M3, kFmtE4M3, 128, 256)
                           : bf ? make_idesc(kCFmtF32, kFmtBF16, kFmtBF16, 128, 256)
                                : make_idesc(kCFmtS32, kFmtS8, kFmtS8, 128, halves == 2 ? 128 : 256);
      const uint64_t desc_hi = make_desc_k128(0);  // everything but the start address
      uint32_t a_addr = a_smem;
      int s = 0, u = 0;
      uint32_t ph = 0, uph = 0;
      bool ok = true;
      for (int it = 0; it < nkb; ++it) {
        uint32_t w_addr;
        if (widen) {
          if (!mbar_wait(bar_ready + 8 * u, uph, p.err, kErrWaitReady)) { ok = false; break; }
          w_addr = u_smem + u * kTileBytes;
        } else {
          if (!mbar_wait(bar_full + 8 * s, ph, p.err, kErrWaitReady)) { ok = false; break; }
          w_addr = w_smem + s * wbytes;
        }
        tc_fence_after_sync();
        if (it == 0) SABER_STAMP(5);
        const uint64_t a_desc = desc_hi | static_cast<uint64_t>((a_addr & 0x3FFFFu) >> 4);
        const uint64_t b_desc = desc_hi | static_cast<uint64_t>((w_addr & 0x3FFFFu) >> 4);
        // 32 int8 = 32 bytes along K inside the 128-byte swizzle row: +2 in 16-byte units
        for (int j2 = 0; j2 < mt2; ++j2) {
          const uint32_t dj = tmem_d + static_cast<uint32_t>(j2) * 256u;             // accumulator of token tile j2
          const uint64_t aj = a_desc + static_cast<uint64_t>(j2) * (static_cast<uint64_t>(p.nt) * 128u >> 4);
          if constexpr (kFp4) {
            // the block's scales go to tensor memory first (copies and MMAs of one thread run in
            // order), into the column set of the block's parity: per 64-value MMA step four columns
            // of token scales and eight of feature scales (two 128-row chunks)
            const uint32_t sf_t = tmem_d + 256u + static_cast<uint32_t>(it & 1) * 48u;
            const uint32_t sfa_s = sfa_smem + static_cast<uint32_t>(s) * sfa_bytes;
            const uint32_t sfb_s = w_addr + 32768u;
            for (uint32_t g = 0; g < sf_atoms; ++g) {
              tmem_cp_sf(sf_t + g * 12u, sf_desc(sfa_s + g * 512u));
              tmem_cp_sf(sf_t + g * 12u + 4u, sf_desc(sfb_s + (g * 2u) * 512u));
              tmem_cp_sf(sf_t + g * 12u + 8u, sf_desc(sfb_s + (g * 2u + 1u) * 512u));
            }
            for (uint32_t j = 0; j < 4; ++j) {
              // NVFP4: step j has its own atom (four scales per row); MXFP4: an atom serves two steps, bytes 0-1 then 2-3
              const uint32_t g = nv ? j : (j >> 1);
              const uint32_t sid = nv ? 0u : ((j & 1u) << 1);
              const uint32_t id = make_idesc_bs(kFmtE2M1Packed, kFmtE2M1Packed, 128, 256, nv ? 0u : 1u, sid, sid);
              mma_fp4_bs(nv, dj, aj + 2 * j, b_desc + 2 * j, id, sf_t + g * 12u, sf_t + g * 12u + 4u, (it != 0 || j != 0) ? 1u : 0u);
            }
          } else if (mx) {   // fp8 x fp8 -> fp32 (the weights were folded to e4m3 by the transform warps)
            mma_f8_ss(dj, aj, b_desc, idesc, it != 0 ? 1u : 0u);
            mma_f8_ss(dj, aj + 2, b_desc + 2, idesc, 1u);
            mma_f8_ss(dj, aj + 4, b_desc + 4, idesc, 1u);
            mma_f8_ss(dj, aj + 6, b_desc + 6, idesc, 1u);
          } else if (bf) {   // 16 bf16 = 32 bytes along K per instruction: the same +2 steps
            mma_f16_ss(dj, aj, b_desc, idesc, it != 0 ? 1u : 0u);
            mma_f16_ss(dj, aj + 2, b_desc + 2, idesc, 1u);
            mma_f16_ss(dj, aj + 4, b_desc + 4, idesc, 1u);
            mma_f16_ss(dj, aj + 6, b_desc + 6, idesc, 1u);
          } else {
            mma_i8_ss(dj, aj, b_desc, idesc, it != 0 ? 1u : 0u);
            mma_i8_ss(dj, aj + 2, b_desc + 2, idesc, 1u);
            mma_i8_ss(dj, aj + 4, b_desc + 4, idesc, 1u);
            mma_i8_ss(dj, aj + 6, b_desc + 6, idesc, 1u);
          }
        }
        mma_commit(bar_empty + 8 * s);
        if (widen) {
          mma_commit(bar_ufree + 8 * u);
          if (++u == nub) { u = 0; uph ^= 1u; }
        }
        a_addr += abytes;
        if (++s == stages) { s = 0; ph ^= 1u; a_addr = a_smem; }
      }
      mma_commit(bar_acc);
      // Unwinding after a wait that ran out: the MMAs issued so far must have retired before the
      // CTA gives its tensor memory back (the status word already tells the host the result is void).
      if (!ok) mbar_wait(bar_acc, 0, nullptr, 0);
      SABER_STAMP(6);
    } else if (!kLean && !kBf && p.tail_mode == 1 && blockIdx.x == 0 && blockIdx.y == 0) {
      // in-tile silu * mul + quant: the row maxima start from zero; this launch's first CTA cleans
      // them here (the previous user finished with its whole grid) and raises the "clean" flag
      pdl_wait();
      for (int i = lane - 1; i < p.tail_M_pad; i += 31) p.tail_sync[64 + static_cast<size_t>(i) * 32] = 0u;
      __threadfence();
      __syncwarp(0xFFFFFFFEu);
      if (lane == 1)
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.tail_sync + kTailFlagsAt + 255), "r"(1u) : "memory");
    } else if (!kLean && !kBf && p.tail_mode == 3 && split == 0) {
      // Row tail on the accumulator blocks: nobody re-zeroes a block after reading it (16-byte
      // zero stores from one CTA per row share sectors across CTAs and are ruinously slow), so the
      // first split of every tile cleans its block HERE, in whole lines, while the pipeline
      // runs; the splits check the tile's "clean" flag before they add.  These 31 lanes are
      // otherwise idle.
      pdl_wait();                              // the previous launch may still be reading the blocks
      const int tile_lin = tile_m * grid_n + tile_n;
      int4* blk = reinterpret_cast<int4*>(p.acc + static_cast<size_t>(tile_lin) * p.nt * 256);
      const int n16 = p.nt * 64;               // 16-byte pieces of the block
      for (int i = lane - 1; i < n16; i += 31) __stcg(blk + i, make_int4(0, 0, 0, 0));
      __threadfence();
      __syncwarp(0xFFFFFFFEu);
      if (lane == 1)
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.tail_sync + kTailFlagsAt + tile_lin), "r"(1u) : "memory");
    }
  } else {
    // ---------------------------------------------------------------- transform, then epilogue
    const int tid_t = (threadIdx.x - 64) & 127;  // 0..127: index inside the epilogue group
    const int tgroup = (threadIdx.x - 64) >> 7;  // 0: warps 2-5 (also the epilogue), 1: warps 6-9
    const int tid8 = threadIdx.x - 64;           // 0..255 over all eight transform warps
    const int q4 = warp & 3;                     // TMEM lane quarter this warp may access
    bool ok = true;
    if (tgroup == 0) {  // epilogue warps stage the per-feature scales while the pipeline fills
      if constexpr (kBf) {
        for (int j = tid_t; j < 256; j += 128) {
          w_scale_s[j] = (n0 + j < p.N) ? (p.w_scale ? w_scale_base[n0 + j] : 1.f) : 0.f;
          bias_s[j] = (p.bias && n0 + j < p.N) ? p.bias[n0 + j] : 0.f;
        }
      } else {
        for (int j = tid_t; j < 256; j += 128) w_scale_s[j] = (n0 + j < p.N) ? w_scale_base[n0 + j] : 0.f;
      }
    }
    if (widen) {
      // The two groups of four warps take the k-blocks in turn (group g: blocks g, g + 2, ...).  A
      // warp's chain for one block -- read the packed stage, wait for a free operand buffer, write,
      // proxy fence, arrive -- is long and mostly latency; with the groups alternating, one
      // group's fence and arrival overlap the other group's reads and writes.
      // Phase bookkeeping: a parity wait is only unambiguous for a waiter that has seen the phase
      // before it, so BOTH groups pass through every stage's "full" barrier in block order (the
      // wait for the other group's block returns at once in steady state); the operand-buffer
      // barriers are only waited on by the block's owner, which is safe because the MMAs retire in
      // order (the owner's previous wait already implies the phase in between).
      int s = 0, u = 0;
      uint32_t ph = 0, ufree_ph = 1;
      for (int it = 0; it < nkb; ++it) {
        const int s_now = s, u_now = u;
        const uint32_t ph_now = ph, ufree_now = ufree_ph;
        if (++s == stages) { s = 0; ph ^= 1u; }
        if (++u == nub) { u = 0; ufree_ph ^= 1u; }
        if (!mbar_wait(bar_full + 8 * s_now, ph_now, p.err, kErrWaitFull)) { ok = false; break; }
        if ((it & 1) != tgroup) continue;
        if (it == 0 && tid8 == 0) SABER_STAMP(3);
        const uint32_t src = w_smem + s_now * wbytes;
        const uint32_t dst = u_smem + u_now * kTileBytes;
        uint32_t v[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t off = static_cast<uint32_t>(i * 128 + tid_t) * 16u;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(v[i][0]), "=r"(v[i][1]), "=r"(v[i][2]), "=r"(v[i][3])
                       : "r"(src + off));
        }
        if (!mbar_wait(bar_ufree + 8 * u_now, ufree_now, p.err, kErrWaitEmpty)) { ok = false; break; }
        if (mx) {
          // MXFP4: a 16-bit half of a packed word = four e2m1 codes of one row = the selector of a
          // byte permute over the eight e4m3 magnitudes, shifted down by the block's exponent
          // distance k to the row's largest block (entries whose exponent field would reach 0
          // are flushed); the sign bits come from a second permute over {0x00, 0x80}.
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t ci = static_cast<uint32_t>(i * 128 + tid_t);
            const uint32_t r = ci >> 3, lc = (ci & 7u) ^ (r & 7u);
            uint32_t klo, khi;
            asm volatile("ld.shared.u8 %0, [%1];" : "=r"(klo) : "r"(src + 16384u + r * 4u + (lc >> 1)));
            asm volatile("ld.shared.u8 %0, [%1];" : "=r"(khi) : "r"(src + 16384u + (r + 128u) * 4u + (lc >> 1)));
            uint32_t ta[2], tb[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t k = h ? khi : klo;
              const uint32_t ma = (k < 11u ? 0x0000FF00u : 0u) | (k < 12u ? 0xFFFF0000u : 0u);
              const uint32_t mb = (k < 13u ? 0x0000FFFFu : 0u) | (k < 14u ? 0xFFFF0000u : 0u);
              const uint32_t sub = (k << 3) * 0x01010101u;
              ta[h] = (0x64605800u & ma) - (sub & ma);
              tb[h] = (0x74706C68u & mb) - (sub & mb);
            }
            uint32_t olo[4], ohi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w = v[i][j];
              const uint32_t wl = w & 0xFFFFu, wh = w >> 16;
              olo[j] = __byte_perm(ta[0], tb[0], wl & 0x7777u) | __byte_perm(0x00008000u, 0u, (wl >> 3) & 0x1111u);
              ohi[j] = __byte_perm(ta[1], tb[1], wh & 0x7777u) | __byte_perm(0x00008000u, 0u, (wh >> 3) & 0x1111u);
            }
            const uint32_t off = ci * 16u;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + off), "r"(olo[0]), "r"(olo[1]),
                         "r"(olo[2]), "r"(olo[3]) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 16384u + off), "r"(ohi[0]), "r"(ohi[1]),
                         "r"(ohi[2]), "r"(ohi[3]) : "memory");
          }
        } else if (halves == 2) {
          const uint32_t sh = half ? 0u : 4u;      // this CTA's 128 rows: the high or the low nibbles
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t off = static_cast<uint32_t>(i * 128 + tid_t) * 16u;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + off),
                         "r"((v[i][0] << sh) & 0xF0F0F0F0u), "r"((v[i][1] << sh) & 0xF0F0F0F0u),
                         "r"((v[i][2] << sh) & 0xF0F0F0F0u), "r"((v[i][3] << sh) & 0xF0F0F0F0u)
                         : "memory");
          }
        } else
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t off = static_cast<uint32_t>(i * 128 + tid_t) * 16u;
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + off),
                       "r"((v[i][0] << 4) & 0xF0F0F0F0u), "r"((v[i][1] << 4) & 0xF0F0F0F0u),
                       "r"((v[i][2] << 4) & 0xF0F0F0F0u), "r"((v[i][3] << 4) & 0xF0F0F0F0u)
                       : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + 16384u + off),
                       "r"(v[i][0] & 0xF0F0F0F0u), "r"(v[i][1] & 0xF0F0F0F0u),
                       "r"(v[i][2] & 0xF0F0F0F0u), "r"(v[i][3] & 0xF0F0F0F0u)
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ready + 8 * u_now);
        if (it == 0 && tid8 == 0) SABER_STAMP(4);
      }
    }
    // Two token tiles per CTA: BOTH transform groups run the epilogue, one accumulator each (either
    // group's four warps cover the four TMEM lane quarters), with their own staging buffer and their
    // own named barrier.  Otherwise only the first group does.
    const bool pair = !kLean && mt2 == 2;
    const int ebar = 1 + (pair ? tgroup : 0);
    // wide forms: both groups read the accumulator out (half of the columns each: either group's
    // four warps cover the four TMEM lane quarters) -- the in-tile silu * mul + quant and the
    // staging of split-K partial sums for the bulk reduction
    const bool bulk = !kLean && !kBf && !kFp4 && !mx && p.splits > 1 && p.acc != nullptr;
    const bool smq = !kLean && !kBf && p.tail_mode == 1;
    const bool wide = bulk || smq;
    if (tgroup == 0 || pair || wide) {
      // the epilogue warps decide TOGETHER whether to run the epilogue: the named barriers
      // below have no time limit, so no warp may skip one that the others enter
      if (ok) ok = mbar_wait(bar_acc, 0, p.err, kErrWaitAcc);
      if (!ok) abort_s = 1u;
      if (pair || wide) named_bar_sync(3, 256); else named_bar_sync(1, 128);  // also publishes w_scale_s
      ok = abort_s == 0u;
    } else {
      ok = false;  // only the first group (TMEM lane quarters 2,3,0,1) is the epilogue
    }
    if constexpr (!kLean && !kBf) {
      if (bulk) {
        // split-K partial sums: the live rows go to shared memory as [c4][nt rows][4 ints] (a warp's
        // 32 rows store 512 contiguous bytes), rows between the live count and nt as zeros
        if (ok) {
          tc_fence_after_sync();
          const int mt = min(p.nt, p.M - m0);
          const int row = q4 * 32 + lane;
          const uint32_t stage_s = widen ? u_smem : w_smem;     // idle by now, at least 128 KiB in a row
          const uint32_t t_lane = tmem_d + (static_cast<uint32_t>(q4 * 32) << 16);
          if (q4 * 32 < p.nt) {
            const bool live = row < mt;
            for (int c = tgroup * 128; c < tgroup * 128 + 128; c += 32) {
              uint32_t r[32];
              tmem_ld32(t_lane + c, r);
              tmem_ld_wait();
              if (row < p.nt) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const uint32_t a = stage_s + (static_cast<uint32_t>((c >> 2) + j) * p.nt + row) * 16u;
                  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(live ? r[4 * j] : 0u),
                               "r"(live ? r[4 * j + 1] : 0u), "r"(live ? r[4 * j + 2] : 0u), "r"(live ? r[4 * j + 3] : 0u)
                               : "memory");
                }
              }
            }
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(3, 256);
        if (tgroup == 1) ok = false;       // the first group goes on alone
      }
      if (p.tail_mode == 1) {
        // silu(gate) * up and the per-token int8 quantisation inside the tile (paired weight tiles:
        // columns c and 128 + c of the accumulator are the gate and up feature of the same index).
        // The first group stages the bf16-rounded linear outputs in shared memory (one token row
        // per thread, as the accumulator arrives); then ALL eight transform warps walk the rows, a
        // warp per row and four products per lane, so the transcendental work is spread over 256
        // threads whatever the number of live rows.  Row maxima meet in global memory (one cache
        // line per row), ONE grid-wide barrier, and every CTA writes its 128 bytes of each row
        // straight into the next GEMM's operand.  Rounding points are those of the separate
        // kernels: linear output to bf16, product to bf16, absmax / 127, round-half-even.
        const uint32_t stage_s = widen ? u_smem : w_smem;
        const int mt = min(p.nt, p.M - m0);
        pdl_wait();
        if (ok) {
          tc_fence_after_sync();
          const int row = q4 * 32 + lane;
          if (q4 * 32 < mt) {
            const bool live = row < mt;
            const float asc = live ? p.a_scale[m0 + row] : 0.f;
            const uint32_t t_lane = tmem_d + (static_cast<uint32_t>(q4 * 32) << 16);
            for (int c = tgroup * 128; c < tgroup * 128 + 128; c += 32) {
              uint32_t r[32];
              tmem_ld32(t_lane + c, r);
              tmem_ld_wait();
              if (live) {
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
                  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage_s + row * 512 + (chunk << 4)),
                               "r"(pk[4 * j]), "r"(pk[4 * j + 1]), "r"(pk[4 * j + 2]), "r"(pk[4 * j + 3]) : "memory");
                }
              }
            }
          }
        }
        uint32_t* rowmax = p.tail_sync + 64;           // one 128-byte line per row
        if (tid8 == 0) {       // the row maxima were put back to zero by this launch's first CTA (see the MMA warp)
          const uint32_t* flag = p.tail_sync + kTailFlagsAt + 255;
          const long long t0 = clock64();
          for (uint32_t polls = 0;; ++polls) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v != 0u) break;
            if ((polls & 1023u) == 1023u && clock64() - t0 > kWaitLimitCycles) {
              atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrWaitSplit));
              break;
            }
          }
        }
        named_bar_sync(2, 256);
        const bool go = abort_s == 0u;
        const int w8 = warp - 2;                       // 0..7
        constexpr int kRowsPerWarp = 16;               // nt <= 128
        uint32_t act[kRowsPerWarp][2];                 // four products per row as bf16 pairs
        if (go) {
#pragma unroll
          for (int i = 0; i < kRowsPerWarp; ++i) {
            const int rw = w8 + 8 * i;
            if (rw >= mt) break;
            // lane l: products 4l .. 4l+3 = gate columns 4l.. and up columns 128 + 4l..
            const uint32_t cg = (static_cast<uint32_t>(lane) >> 1) ^ (static_cast<uint32_t>(rw) & 31u);
            const uint32_t cu = (16u + (static_cast<uint32_t>(lane) >> 1)) ^ (static_cast<uint32_t>(rw) & 31u);
            const uint32_t sub = (static_cast<uint32_t>(lane) & 1u) << 3;
            uint32_t g0, g1, u0, u1;
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(g0), "=r"(g1) : "r"(stage_s + rw * 512 + (cg << 4) + sub));
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(u0), "=r"(u1) : "r"(stage_s + rw * 512 + (cu << 4) + sub));
            const float2 ga = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g0));
            const float2 gb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g1));
            const float2 ua = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u0));
            const float2 ub = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u1));
            const __nv_bfloat162 x0 = __floats2bfloat162_rn(silu_f(ga.x) * ua.x, silu_f(ga.y) * ua.y);
            const __nv_bfloat162 x1 = __floats2bfloat162_rn(silu_f(gb.x) * ub.x, silu_f(gb.y) * ub.y);
            const float2 y0 = __bfloat1622float2(x0), y1 = __bfloat1622float2(x1);
            float amax = fmaxf(fmaxf(fabsf(y0.x), fabsf(y0.y)), fmaxf(fabsf(y1.x), fabsf(y1.y)));
            amax = warp_max(amax);
            if (lane == 0) atomicMax(rowmax + static_cast<size_t>(m0 + rw) * 32, __float_as_uint(amax));   // non-negative floats order like their bits
            act[i][0] = *reinterpret_cast<const uint32_t*>(&x0);
            act[i][1] = *reinterpret_cast<const uint32_t*>(&x1);
          }
        }
        named_bar_sync(2, 256);
        if (tid8 == 0) SABER_STAMP(10);
        const uint32_t n_ctas = gridDim.x * gridDim.y * gridDim.z;
        if (tid8 == 0) grid_arrive_wait(p.tail_sync, n_ctas, p.err);
        named_bar_sync(2, 256);
        if (tid8 == 0) SABER_STAMP(13);
        const int rows_pad = min(p.nt, p.tail_M_pad - m0);     // live rows, then padding rows (zeros)
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
          const int rw = w8 + 8 * i;
          if (rw >= rows_pad) break;
          const int mm = m0 + rw;
          const bool lv = go && rw < mt;
          const float am = lv ? __uint_as_float(__ldcg(rowmax + static_cast<size_t>(mm) * 32)) : 0.f;
          const float inv = am > 0.f ? 127.f / am : 0.f;
          uint32_t word = 0u;
          if (lv) {
            const float2 y0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&act[i][0]));
            const float2 y1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&act[i][1]));
            word = quant4(y0.x, y0.y, y1.x, y1.y, inv, 0);
          }
          int8_t* dst = p.tail_q + (static_cast<size_t>(tile_n) * p.tail_M_pad + mm) * 128;
          *reinterpret_cast<uint32_t*>(dst + ((((lane >> 2) ^ (mm & 7)) & 7) << 4) + ((lane & 3) << 2)) = word;
          if (tile_n == 0 && lane == 0) p.tail_scale[mm] = am / 127.f;
        }
        // second round of arrivals (fire and forget); the last CTA of the grid lowers the flag
        if (tid8 == 0) {
          if (blockIdx.x == gridDim.x - 1 && blockIdx.y == gridDim.y - 1) p.tail_sync[kTailFlagsAt + 255] = 0u;
          grid_depart(p.tail_sync, n_ctas);
        }
        ok = false;        // the generic epilogue below is not for this launch
      }
    }
    if (ok) {
      tc_fence_after_sync();
      pdl_wait();   // already satisfied (the token tiles have landed); orders this thread's reads and writes
      if (tid_t == 0) SABER_STAMP(7);
      const int mt = rows_here >= 0 ? rows_here : min(p.nt, p.M - m0);   // live token rows of this tile
      const int row = q4 * 32 + lane;       // token row inside the tile = TMEM lane
      const int m = m0 + row;
      const bool live = row < mt;
      const bool warp_live = q4 * 32 < mt;  // warp-uniform: this lane quarter holds live rows
      const uint32_t t_lane = tmem_d + (static_cast<uint32_t>(q4 * 32) << 16);
      const int ncols = halves == 2 ? 128 : min(256, p.N_pad - n0);
      // accumulator words are int32 (integer formats) or fp32 bits (MXFP4)
      auto acc_f = [&](uint32_t raw) -> float {
        return (mx || bf || kFp4) ? __uint_as_float(raw) : static_cast<float>(static_cast<int32_t>(raw));
      };
      // tensor-parallel mode: a finished 16-byte group of outputs goes to every rank's receive
      // region (slot = parity of the call's sequence number, source = this rank)
      const bool tp = !kLean && p.tp_nranks > 1;
      uint32_t tp_seq = 0, tp_par = 0;
      if (tp) {
        tp_seq = *p.tp_seq_base + static_cast<uint32_t>(p.tp_site) + 1u;
        tp_par = tp_seq & 1u;
      }
      int tp_owner = (!kLean && p.tp_rpr > 0) ? m0 / p.tp_rpr : -1;   // reduce-scatter: the one destination
      auto tp_push16 = [&](int mm, int nn, const uint4& v) {
        const size_t off = ((static_cast<size_t>(tp_par) * p.tp_nranks + p.tp_rank) * p.tp_rows + mm) * p.tp_ld + nn;
        if (tp_owner >= 0) {
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.tp_recv[tp_owner]) + off) = v;
          return;
        }
        for (int peer = 0; peer < p.tp_nranks; ++peer)
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.tp_recv[peer]) + off) = v;
      };
      auto tp_signal = [&](int tile_id) {   // called by all 128 epilogue threads after their stores
        named_bar_sync(ebar, 128);          // every thread's pushes precede the barrier ...
        if (tp_owner >= 0 ? tid_t == tp_owner : tid_t < p.tp_nranks) {
          __threadfence_system();           // ... and this fence is cumulative over what the barrier ordered
          uint32_t* f = p.tp_flags[tid_t] + (static_cast<size_t>(tp_par) * p.tp_nranks + p.tp_rank) * kTpMaxTiles + tile_id;
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(tp_seq) : "memory");
        }
      };
      if (kLean || p.splits == 1) {
        // The accumulator arrives one token row per thread; stored like that, the 32 lanes of a
        // warp would write 32 different rows (16-byte pieces, and over NVLink 16-byte packets).
        // So the bf16 tile is first staged in shared memory -- the operand buffers are idle by
        // now -- with its 16-byte chunks XOR-swizzled by the row, then every warp writes whole
        // rows: 512 contiguous bytes per store instruction, to local memory or to every rank.
        // (pair mode: the first group stages in the token ring -- at least two 32 KiB stages --, the second
        // in the operand buffers / weight ring)
        const uint32_t stage_s = (pair && tgroup == 0) ? a_smem : (widen ? u_smem : w_smem);     // >= 64 KiB in every mode
        const int j2_lo = pair ? tgroup : 0, j2_hi = pair ? tgroup + 1 : mt2;
        for (int j2 = j2_lo; j2 < j2_hi; ++j2) {
        const int mb = m0 + j2 * p.nt;             // first row of this accumulator's token tile
        const int mtj = rows_here >= 0 ? rows_here : min(p.nt, p.M - mb);
        if (mtj <= 0) break;                       // (uniform) the second tile of a ragged pair is empty
        const bool livej = row < mtj, warp_livej = q4 * 32 < mtj;
        const uint32_t tl = t_lane + static_cast<uint32_t>(j2) * 256u;
        if (!kLean && p.tp_rpr > 0) tp_owner = mb / p.tp_rpr;
        if (j2 > j2_lo) named_bar_sync(ebar, 128);   // the staging buffer is free again
        if (warp_livej) {
          const float asc = livej ? ((!kBf || p.a_scale) ? p.a_scale[mb + row] : 1.f) : 0.f;
          for (int c = 0; c < ncols; c += 32) {
            uint32_t r[32];
            tmem_ld32(tl + c, r);
            tmem_ld_wait();
            if (livej) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float lo = acc_f(r[2 * j]) * (asc * w_scale_s[c + 2 * j]);
                float hi = acc_f(r[2 * j + 1]) * (asc * w_scale_s[c + 2 * j + 1]);
                if constexpr (kBf) { lo += bias_s[c + 2 * j]; hi += bias_s[c + 2 * j + 1]; }
                __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                if constexpr (kBf) {
                  if (p.epi == 1 || p.epi == 2) {   // the activation works on the rounded linear output
                    const float2 y = __bfloat1622float2(b2);
                    b2 = __floats2bfloat162_rn(gelu_f(y.x, p.epi == 2), gelu_f(y.y, p.epi == 2));
                  }
                }
                pk[j] = *reinterpret_cast<const uint32_t*>(&b2);
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t chunk = static_cast<uint32_t>((c >> 3) + j) ^ (static_cast<uint32_t>(row) & 31u);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(stage_s + row * 512 + (chunk << 4)),
                             "r"(pk[4 * j]), "r"(pk[4 * j + 1]), "r"(pk[4 * j + 2]), "r"(pk[4 * j + 3])
                             : "memory");
              }
            }
          }
        }
        named_bar_sync(ebar, 128);
        {
          const int wq = tid_t >> 5;                  // 0..3: rows wq, wq + 4, ...
          const int col = lane * 8;                   // this lane's 8 output features of the row
          const bool col_ok = n0 + col < p.N;         // (N is a multiple of 8 whenever ldo is)
          const bool full = n0 + col + 8 <= p.N;
          for (int rw = wq; rw < mtj; rw += 4) {
            uint4 v;
            const uint32_t chunk = static_cast<uint32_t>(lane) ^ (static_cast<uint32_t>(rw) & 31u);
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(stage_s + rw * 512 + (chunk << 4)));
            if (!col_ok || col >= ncols) continue;
            if (kBf && p.epi == 3 && p.res != nullptr) {     // residual add on the rounded linear output
              const __nv_bfloat16* rp = p.res + static_cast<size_t>(mb + rw) * p.ldo + n0 + col;
              __nv_bfloat16* pv = reinterpret_cast<__nv_bfloat16*>(&v);
              if (full) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rp);
                const __nv_bfloat16* pr = reinterpret_cast<const __nv_bfloat16*>(&rv);
#pragma unroll
                for (int j = 0; j < 8; ++j) pv[j] = __float2bfloat16(__bfloat162float(pv[j]) + __bfloat162float(pr[j]));
              } else {
                for (int j = 0; j < 8; ++j)
                  if (n0 + col + j < p.N) pv[j] = __float2bfloat16(__bfloat162float(pv[j]) + __bfloat162float(rp[j]));
              }
            }
            if (tp) {
              tp_push16(mb + rw, n0 + col, v);
            } else if (full) {
              *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(mb + rw) * p.ldo + n0 + col) = v;
            } else {
              const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&v);
              __nv_bfloat16* o = p.out + static_cast<size_t>(mb + rw) * p.ldo + n0 + col;
              for (int j = 0; j < 8; ++j)
                if (n0 + col + j < p.N) o[j] = pb[j];
            }
          }
        }
        if (tp) tp_signal((tile_m * mt2 + j2) * grid_n + tile_n);
        }
      } else if constexpr (!kLean) {
        // each split writes its own partial tile; inside a (split, tile) block the 16-byte group of
        // four columns c4 of row r sits at (c4 * 128 + r) * 16 bytes, so the 32 lanes of a warp
        // (32 consecutive rows) store -- and later load -- 512 contiguous bytes
        const int tile_lin = tile_m * grid_n + tile_n;
        const size_t blk_stride = 128u * 256u;   // ints per (split, tile) block
        // Integer partial sums can be added in any order, so the splits of a tile do not keep private
        // copies: each stages its live rows in shared memory and hands them to ONE asynchronous bulk
        // reduction (TMA add.s32) into the tile's accumulator block in L2 -- zero when the kernel
        // starts, re-zeroed by whoever reads it out.  The block is [c4][nt rows][4 ints].  MXFP4
        // partials are fp32 and keep the private copies (their sum must not depend on the arrival order).
        const int rstride = bulk ? p.nt : 128;   // rows per four-column group of a block
        int32_t* wblk = p.ws + (static_cast<size_t>(split) * (gridDim.x * gridDim.y) + tile_lin) * blk_stride;
        int32_t* ablk = bulk ? p.acc + static_cast<size_t>(tile_lin) * p.nt * 256u : nullptr;
        if (bulk) {
          const uint32_t stage_s = widen ? u_smem : w_smem;     // staged by both groups above
          if (tid_t == 0) {
            if (p.tail_mode == 3) {            // the block must have been cleaned by this launch's first split
              const uint32_t* flag = p.tail_sync + kTailFlagsAt + tile_lin;
              const long long t0 = clock64();
              for (uint32_t polls = 0;; ++polls) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                if (v != 0u) break;
                if ((polls & 1023u) == 1023u && clock64() - t0 > kWaitLimitCycles) {
                  atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrWaitSplit));
                  break;
                }
              }
            }
            const uint32_t total = static_cast<uint32_t>(p.nt) * 1024u;
            for (uint32_t off = 0; off < total; off += 16384u)
              asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.s32 [%0], [%1], %2;" ::"l"(
                               reinterpret_cast<uint8_t*>(ablk) + off), "r"(stage_s + off), "r"(min(16384u, total - off))
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
        } else if (warp_live) {
          for (int c = 0; c < ncols; c += 32) {
            uint32_t r[32];
            tmem_ld32(t_lane + c, r);
            tmem_ld_wait();
            if (live) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(wblk + (static_cast<size_t>((c >> 2) + j) * 128 + row) * 4) =
                    make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
          }
        }
        __threadfence();
        named_bar_sync(1, 128);
        if (tid_t == 0) SABER_STAMP(10);
        if (!(bulk && p.tail_mode == 3)) {     // (tail mode 3: the row tail reads the accumulator blocks itself)
        const int tile_id = tile_lin;
        // Two ways to add the splits.  Cooperative (every CTA of the grid is resident, the launcher
        // guarantees it): all splits of a tile wait for one another and each reduces the rows
        // c4 = split (mod splits) -- four-column groups -- so the pass is spread over `splits` SMs.  Otherwise the last
        // arriver reduces the whole tile alone.
        int part = 0, nparts = 1;
        if (p.coop) {
          if (tid_t == 0) {
            atomicAdd(p.counters + tile_id, 1u);
            uint32_t seen = 0;
            const long long t0 = clock64();
            uint32_t okw = 1u;
            for (uint32_t polls = 0;; ++polls) {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.counters + tile_id) : "memory");
              if (seen >= static_cast<uint32_t>(p.splits)) break;
              if ((polls & 1023u) == 1023u && clock64() - t0 > kWaitLimitCycles) {
                atomicCAS(p.err, 0, kErrWaitSplit);
                okw = 0u;
                break;
              }
            }
            is_last_s = okw;
          }
          part = split;
          nparts = p.splits;
        } else if (tid_t == 0) {
          const uint32_t old = atomicAdd(p.counters + tile_id, 1u);
          is_last_s = (old == static_cast<uint32_t>(p.splits - 1)) ? 1u : 0u;
        }
        named_bar_sync(1, 128);
        if (tid_t == 0) SABER_STAMP(11);
        if (is_last_s) {
          __threadfence();
          // items = (four-column group of this part, live row), rows fastest: consecutive threads
          // read consecutive 16-byte groups.  All splits of an item are loaded before any is
          // used, two items per round: one memory round trip per round.
          const int n_c4 = ncols >> 2;
          // one GPU: a part owns a CONTIGUOUS span of four-column groups, so that its share of every row is one
          // run of bytes: the rounded outputs are staged in shared memory (8-byte pieces, 16-byte chunks
          // XOR-swizzled by the row) and leave as whole spans, a warp per row (stored one piece per row and
          // lane they were 32 partial sectors per instruction: 7.8 us of a 27 us launch)
          const int c4_lo = (n_c4 * part) / nparts, c4_hi = (n_c4 * (part + 1)) / nparts;
          const int c4_part = c4_hi - c4_lo;
          const uint32_t stage_o = widen ? u_smem : w_smem;     // idle by now (the bulk reduction has read it)
          // tensor-parallel: the parts split the ROWS and lanes run over the column groups, so
          // that a warp's pushes to a peer are contiguous bytes of one row
          const int rows_part = mt > part ? (mt - part + nparts - 1) / nparts : 0;
          const int n_items = tp ? rows_part * n_c4 : c4_part * mt;
          const size_t tiles_all = static_cast<size_t>(gridDim.x) * gridDim.y;
          int32_t* rblk = bulk ? ablk : p.ws + static_cast<size_t>(tile_lin) * blk_stride;
          const int nsp = bulk ? 1 : p.splits;     // blocks to add per item
          auto reduce_items = [&](auto ilp_c, auto maxs_c) {
          constexpr int kIlp = decltype(ilp_c)::value;
          constexpr int kMaxS = decltype(maxs_c)::value;
          for (int base = tid_t; base < n_items; base += 128 * kIlp) {
            int4 y[kIlp][kMaxS];
            int rr[kIlp], c4[kIlp];
#pragma unroll
            for (int u = 0; u < kIlp; ++u) {
              const int idx = min(base + u * 128, n_items - 1);
              if (tp) {
                const int ri = idx / n_c4;
                c4[u] = idx - ri * n_c4;
                rr[u] = part + ri * nparts;
              } else {
                const int ci = idx / mt;
                rr[u] = idx - ci * mt;
                c4[u] = c4_lo + ci;
              }
#pragma unroll
              for (int sp = 0; sp < kMaxS; ++sp)
                if (sp < nsp)
                  y[u][sp] = __ldcg(reinterpret_cast<const int4*>(
                      rblk + static_cast<size_t>(sp) * tiles_all * blk_stride + (static_cast<size_t>(c4[u]) * rstride + rr[u]) * 4));
            }
#pragma unroll
            for (int u = 0; u < kIlp; ++u) {
              if (base + u * 128 >= n_items) continue;
              if (bulk)   // the accumulator block goes back to zero for the next launch
                __stcg(reinterpret_cast<int4*>(rblk + (static_cast<size_t>(c4[u]) * rstride + rr[u]) * 4), make_int4(0, 0, 0, 0));
              float f[4];
              if (mx || kFp4) {   // fp32 partials: added in split order, the same on every launch
                f[0] = f[1] = f[2] = f[3] = 0.f;
#pragma unroll
                for (int sp = 0; sp < kMaxS; ++sp)
                  if (sp < nsp) {
                    f[0] += __int_as_float(y[u][sp].x); f[1] += __int_as_float(y[u][sp].y);
                    f[2] += __int_as_float(y[u][sp].z); f[3] += __int_as_float(y[u][sp].w);
                  }
              } else {
                int4 x = make_int4(0, 0, 0, 0);
#pragma unroll
                for (int sp = 0; sp < kMaxS; ++sp)
                  if (sp < nsp) { x.x += y[u][sp].x; x.y += y[u][sp].y; x.z += y[u][sp].z; x.w += y[u][sp].w; }
                f[0] = static_cast<float>(x.x); f[1] = static_cast<float>(x.y);
                f[2] = static_cast<float>(x.z); f[3] = static_cast<float>(x.w);
              }
              const int c = c4[u] << 2;
              const float asc = p.a_scale[m0 + rr[u]];
              const __nv_bfloat162 b0 = __floats2bfloat162_rn(f[0] * (asc * w_scale_s[c]), f[1] * (asc * w_scale_s[c + 1]));
              const __nv_bfloat162 b1 = __floats2bfloat162_rn(f[2] * (asc * w_scale_s[c + 2]), f[3] * (asc * w_scale_s[c + 3]));
              const uint2 pk = make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
              if (tp) {
                if (n0 + c < p.N) {
                  const size_t off = ((static_cast<size_t>(tp_par) * p.tp_nranks + p.tp_rank) * p.tp_rows + m0 + rr[u]) * p.tp_ld + n0 + c;
                  if (tp_owner >= 0)
                    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.tp_recv[tp_owner]) + off) = pk;
                  else
                    for (int peer = 0; peer < p.tp_nranks; ++peer)
                      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.tp_recv[peer]) + off) = pk;
                }
              } else {
                const uint32_t sa = stage_o + static_cast<uint32_t>(rr[u]) * 512u +
                                    (((static_cast<uint32_t>(c4[u]) >> 1) ^ (static_cast<uint32_t>(rr[u]) & 31u)) << 4) + ((static_cast<uint32_t>(c4[u]) & 1u) << 3);
                asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(sa), "r"(pk.x), "r"(pk.y) : "memory");
              }
            }
          }
          };
          // the budget is ~16 loads in flight per thread: more items per round when there are few splits
          if (bulk) reduce_items(std::integral_constant<int, 8>{}, std::integral_constant<int, 1>{});
          else if (p.splits <= 2) reduce_items(std::integral_constant<int, 8>{}, std::integral_constant<int, 2>{});
          else if (p.splits <= 4) reduce_items(std::integral_constant<int, 4>{}, std::integral_constant<int, 4>{});
          else reduce_items(std::integral_constant<int, 2>{}, std::integral_constant<int, 8>{});
          if (!tp) {
            named_bar_sync(1, 128);             // every piece of this part is staged
            for (int rw = tid_t >> 5; rw < mt; rw += 4) {
              for (int g = c4_lo + lane; g < c4_hi; g += 32) {
                const uint32_t sa = stage_o + static_cast<uint32_t>(rw) * 512u +
                                    (((static_cast<uint32_t>(g) >> 1) ^ (static_cast<uint32_t>(rw) & 31u)) << 4) + ((static_cast<uint32_t>(g) & 1u) << 3);
                uint2 pk;
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pk.x), "=r"(pk.y) : "r"(sa));
                const int c = g << 2;
                __nv_bfloat16* o = p.out + static_cast<size_t>(m0 + rw) * p.ldo + n0 + c;
                if (n0 + c + 4 <= p.N) {
                  *reinterpret_cast<uint2*>(o) = pk;
                } else {
                  const __nv_bfloat16* pb = reinterpret_cast<const __nv_bfloat16*>(&pk);
                  for (int j = 0; j < 4; ++j)
                    if (n0 + c + j < p.N) o[j] = pb[j];
                }
              }
            }
          }
          if (!p.coop) {
            if (tid_t == 0) p.counters[tile_id] = 0u;
            if (tp) tp_signal(tile_id);
          }
        }
        if (tid_t == 0) SABER_STAMP(12);
        if (p.coop) {
          // tensor-parallel: every part raises its OWN flag (index tile * splits + split) as soon as
          // its rows are pushed; the consumer waits for all parts of the tiles it reads
          if (tp) tp_signal(tile_id * p.splits + split);
          // second round of arrivals, off the critical path: the CTA that finishes last re-arms the counter
          if (tid_t == 0) {
            const uint32_t old = atomicAdd(p.counters + tile_id, 1u);
            if (old == static_cast<uint32_t>(2 * p.splits - 1)) p.counters[tile_id] = 0u;
          }
        }
        }
      }
    }
  }

  if (threadIdx.x == 64) SABER_STAMP(8);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, kTmemCols);
  if (threadIdx.x == 32) SABER_STAMP(9);
  if constexpr (!kLean && !kBf) {
    if ((p.tail_mode == 2 || p.tail_mode == 3) && tail != nullptr) {
      // Row tail.  Every CTA arrives here whatever happened above (an aborted pipeline has set the
      // status word; the barrier still completes), then the rows are dealt round-robin to the CTAs.
      const uint32_t n_ctas = gridDim.x * gridDim.y * gridDim.z;
      const uint32_t me = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      {
        // while the barrier forms: pull what the first row of this CTA reads besides the GEMM's
        // output (its residual row, the norm weights) into L1 -- neither is written by this launch
        const int rows0 = tail->q ? tail->M_pad : tail->M;
        if (static_cast<int>(me) < rows0 && static_cast<int>(me) < tail->M) {
          for (int ch = threadIdx.x; ch < (tail->K >> 4); ch += kGemmThreads) {
            if (tail->res) {
              const __nv_bfloat16* r = tail->res + static_cast<size_t>(me) * tail->ldres + (ch << 4);
              asm volatile("prefetch.global.L1 [%0];" ::"l"(r));
            }
            asm volatile("prefetch.global.L1 [%0];" ::"l"(tail->w + (ch << 4)));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(tail->w + (ch << 4) + 8));
            if (p.tail_mode == 3) {
              asm volatile("prefetch.global.L1 [%0];" ::"l"(tail->acc_w_scale + (ch << 4)));
              asm volatile("prefetch.global.L1 [%0];" ::"l"(tail->acc_w_scale + (ch << 4) + 8));
            }
          }
        }
      }
      if (threadIdx.x == 0) grid_arrive_wait(p.tail_sync, n_ctas, p.err);
      __syncthreads();
      if (threadIdx.x == 0) SABER_STAMP(13);
      if (p.tail_mode == 3 && me == n_ctas - 1)      // every split has added: the "clean" flags go down for the next launch
        for (int i = threadIdx.x; i < static_cast<int>(gridDim.x * gridDim.y); i += kGemmThreads) p.tail_sync[kTailFlagsAt + i] = 0u;
      float* red = w_scale_s;     // the per-feature scales are no longer needed
      const int rows = tail->q ? tail->M_pad : tail->M;
      for (int r = static_cast<int>(me); r < rows; r += static_cast<int>(n_ctas)) {
        if (p.tail_mode == 3) {
          if (tail->K <= 16 * kGemmThreads) row_reg_body<kRowAddRms, 1, true, true>(*tail, r, red);
          else row_reg_body<kRowAddRms, 2, true, true>(*tail, r, red);
        } else {
          if (tail->K <= 16 * kGemmThreads) row_reg_body<kRowAddRms, 1, true>(*tail, r, red);
          else row_reg_body<kRowAddRms, 2, true>(*tail, r, red);
        }
      }
      if (threadIdx.x == 0) SABER_STAMP(14);
      if (threadIdx.x == 0) grid_depart(p.tail_sync, n_ctas);
    }
  }
#undef SABER_STAMP
}

__global__ void __launch_bounds__(kGemmThreads) gemm_i8_kernel(const GemmI8Params p, const int stages) {
  gemm_i8_body<false>(p, stages, nullptr);
}
// the same body with a row tail: the row producer's parameter block rides as a second argument
__global__ void __launch_bounds__(kGemmThreads) gemm_i8_tail_kernel(const GemmI8Params p, const int stages,
                                                                    const __grid_constant__ RowOpParams tail) {
  gemm_i8_body<false>(p, stages, &tail);
}
__global__ void __launch_bounds__(kGemmThreads) gemm_bf16_kernel(const GemmI8Params p, const int stages) {
  gemm_i8_body<false, true>(p, stages, nullptr);
}
__global__ void __launch_bounds__(kGemmThreads) gemm_fp4_kernel(const GemmI8Params p, const int stages) {
  gemm_i8_body<false, false, true>(p, stages, nullptr);
}
__global__ void __launch_bounds__(kGemmThreads, 2) gemm_i8_lean_kernel(const GemmI8Params p, const int stages) {
  gemm_i8_body<true>(p, stages, nullptr);
}

}  // namespace saber

namespace saber {
static int g_coop_launch = 0;
static int g_gemm_2sm = 0;     // int8 weights, long row runs: CTA pairs (gemm_w8_2sm.cu) instead of two token tiles per CTA
constexpr int kMaxDevices = 64;
// Per-device set-up (function attributes are per device): returns 0 and the SM count of the current device.
static int device_setup(int* sm_count) {
  static int sms[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  if (sms[dev] == 0) {
    const int kSmemLimit = 224 * 1024;
    cudaFuncSetAttribute(gemm_i8_lean_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    cudaFuncSetAttribute(gemm_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    cudaFuncSetAttribute(gemm_i8_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    e = cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return static_cast<int>(e);
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    sms[dev] = n;
  }
  *sm_count = sms[dev];
  return 0;
}
}  // namespace saber

// Number of flags per output tile a tensor-parallel launch of `p` raises (the consumer must wait
// for all of them): the split-K factor when the cooperative reduction runs, else one.
extern "C" int saber_gemm_i8_parts(const saber::GemmI8Params* p) {
  int sm_count = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  const int grid_y = p->group_tiles ? p->M_pad / 16 : (p->M + p->nt - 1) / p->nt;
  const bool coop = p->splits > 1 && p->coop >= 0 && (p->N_pad / 256) * grid_y * p->splits <= sm_count;
  return coop ? p->splits : 1;
}

extern "C" int saber_gemm_i8_smem_bytes(int nt, int stages) {
  return saber_gemm_i8_smem_bytes_w(nt, stages, 0);
}
// The token-side descriptor spans 128 rows although only nt are loaded: its reads run on into the
// operand buffers / weight ring, which lie behind the token ring inside the same allocation.
extern "C" int saber_gemm_i8_smem_bytes_w(int nt, int stages, int w4) {
  if (w4 == 4) return stages * (32768 + 4096 + nt * 128 + 2048) + 1024;
  if (w4 == 5) return stages * (32768 + 2048 + nt * 128 + 1024) + 1024;
  if (w4 == 2) return stages * (17408 + nt * 128) + 3 * 32768 + 1024;
  return w4 == 1 ? stages * (16384 + nt * 128) + 3 * 32768 + 1024 : stages * (32768 + nt * 128) + 1024;
}

extern "C" int saber_gemm_i8_launch(const saber::GemmI8Params* p, int stages, cudaStream_t stream) {
  using namespace saber;
  if (p->ag_flags != nullptr && (p->M + 127) / 128 > 64) return static_cast<int>(cudaErrorInvalidValue);
  if (p->nt < 16 || p->nt > 128 || (p->nt & 15) || (p->K & 127) || p->K <= 0 || p->M <= 0 ||
      (p->N_pad & 255) || p->splits < 1 || p->splits > 8 || (p->M_pad % p->nt) != 0 || (p->ldo & 7))
    return static_cast<int>(cudaErrorInvalidValue);
  if (p->w4 == 4 || p->w4 == 5) {
    // native FP4: K counts values (256 per k-block); inside the kernel K counts the 128-byte rows of a block
    if ((p->K & 255) || p->a_sf == nullptr || p->group_tiles || p->tail_mode != 0 || p->tp_nranks > 1 || p->ag_flags != nullptr ||
        p->halves == 2 || p->bias || p->epi || (p->M > 128 && p->nt != 128))
      return static_cast<int>(cudaErrorInvalidValue);
    GemmI8Params q = *p;
    q.K = p->K >> 1;
    q.mtiles = 1;
    const int KBf = q.K >> 7;
    const int kb_per_f = (KBf + p->splits - 1) / p->splits;
    if ((p->splits - 1) * kb_per_f >= KBf) return static_cast<int>(cudaErrorInvalidValue);
    if (stages <= 0) stages = 5;
    if (stages > kMaxStages) stages = kMaxStages;
    while (stages > 2 && saber_gemm_i8_smem_bytes_w(p->nt, stages, p->w4) > 224 * 1024) --stages;
    const int smem_f = saber_gemm_i8_smem_bytes_w(p->nt, stages, p->w4);
    int sms = 0;
    const int e = device_setup(&sms);
    if (e != 0) return e;
    dim3 grid_f(p->N_pad / 256, (p->M + p->nt - 1) / p->nt, p->splits);
    q.coop = (p->splits > 1 && p->coop >= 0 && static_cast<int>(grid_f.x * grid_f.y * grid_f.z) <= sms) ? 1 : 0;
    return static_cast<int>(saber::launch(gemm_fp4_kernel, grid_f, dim3(kGemmThreads), smem_f, stream,
                                          ((q.coop != 0 && g_coop_launch) ? 1 : 0) | 2, q, stages));
  }
  const int KB = p->K >> 7;
  const int kb_per = (KB + p->splits - 1) / p->splits;
  if ((p->splits - 1) * kb_per >= KB) return static_cast<int>(cudaErrorInvalidValue);
  if (p->tp_nranks > 1) {
    const int tiles = (p->N_pad / 256) * ((p->M + p->nt - 1) / p->nt);
    if ((p->tp_rpr > 0 && (p->tp_rpr % p->nt) != 0) || p->tp_nranks > 8 || (p->N & 7) || (p->tp_ld & 7) || tiles * saber_gemm_i8_parts(p) > kTpMaxTiles || p->M > p->tp_rows)
      return static_cast<int>(cudaErrorInvalidValue);
  }
  const int kSmemLimit = 224 * 1024;  // opt-in maximum minus the kernel's static shared memory
  const bool widen_l = p->w4 == 1 || p->w4 == 2;
  if (p->w4 < 0 || p->w4 > 3 || (p->w4 == 3 && (p->splits != 1 || p->group_tiles))) return static_cast<int>(cudaErrorInvalidValue);
  if ((p->bias || p->epi) && p->w4 != 3) return static_cast<int>(cudaErrorInvalidValue);   // bias / activation / residual: bf16 mode only
  if (stages <= 0) stages = widen_l ? 8 : 5;   // one CTA per SM, as deep a ring as fits
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  while (stages > 2 && saber_gemm_i8_smem_bytes_w(p->nt, stages, p->w4) > kSmemLimit) --stages;
  const int smem = saber_gemm_i8_smem_bytes_w(p->nt, stages, p->w4);
  if (smem > kSmemLimit) return static_cast<int>(cudaErrorInvalidValue);
  int sm_count = 0;
  const int cfg_err = device_setup(&sm_count);
  if (cfg_err != 0) return cfg_err;
  // grouped mode: every tile holds at least 16 rows of the padded expert-major row space
  const int grid_y = p->group_tiles ? p->M_pad / 16 : (p->M + p->nt - 1) / p->nt;
  const int halves = p->halves == 2 ? 2 : 1;
  if (halves == 2 && (p->w4 != 1 || p->splits != 1 || p->group_tiles || p->tail_mode != 0 || p->tp_nranks > 1 ||
                      p->ag_flags != nullptr || p->mtiles == 2))
    return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(p->N_pad / 256 * halves, grid_y, p->splits);
  const bool resident = static_cast<int>(grid.x * grid.y * grid.z) <= sm_count;
  GemmI8Params q = *p;
  // one CTA per SM (shared memory): the whole grid is resident iff it has no more CTAs than SMs
  q.coop = (p->splits > 1 && p->coop >= 0 && resident) ? 1 : 0;
  if (p->tail_mode != 0) {
    // the tails wait for the whole grid: every CTA must be resident, one token-tile form only
    if (!resident || p->group_tiles || p->w4 == 3 || p->tail_sync == nullptr || p->mtiles == 2 ||
        false)
      return static_cast<int>(cudaErrorInvalidValue);
    if (p->tail_mode == 1 &&
        (p->splits != 1 || p->w4 == 2 || p->tp_nranks > 1 || p->N != p->N_pad || p->tail_q == nullptr ||
         p->tail_scale == nullptr || p->tail_M_pad < p->M || p->tail_M_pad > 256 || (p->tail_M_pad % p->nt) != 0))
      return static_cast<int>(cudaErrorInvalidValue);
    if (p->tail_mode == 2 &&
        (p->tail_row == nullptr || p->tail_row_mode != kRowAddRms || (p->tail_row->K & 127) ||
         p->tail_row->K > 2 * 16 * kGemmThreads))
      return static_cast<int>(cudaErrorInvalidValue);
    if (p->tail_mode != 1 && p->tail_mode != 2) return static_cast<int>(cudaErrorInvalidValue);
  }
  // grouped tiles: the lean instantiation, two CTAs per SM, when two ring stages fit its budget
  if (p->group_tiles && widen_l && p->splits == 1) {
    const int lean_smem = 2 * ((p->w4 == 2 ? 17408 : 16384) + p->nt * 128) + 2 * 32768 + 1024;
    if (lean_smem <= 112 * 1024)
      return static_cast<int>(saber::launch(gemm_i8_lean_kernel, grid, dim3(kGemmThreads), lean_smem, stream, 2, q, 2));
  }
  if (g_gemm_2sm && p->mtiles >= 0 && p->nt == 128 && saber_gemm_w8_2sm_ok(p) &&
      static_cast<int>(grid.x * grid.y) > sm_count)
    return saber_gemm_w8_2sm_launch(p, 0, stream);
  // long row runs: two token tiles per CTA (pairs must be whole inside M_pad).  4-bit weights are widened once
  // for both tiles; int8 and bf16 weights pass through unwidened and are read from shared memory once for both.
  q.mtiles = 1;
  if (p->mtiles >= 0 && !p->group_tiles && p->splits == 1 && p->nt == 128 && p->M > 128 &&
      (p->M_pad / 128) % 2 == 0 && p->tail_mode == 0 && halves == 1 &&
      (p->mtiles == 2 || static_cast<int>(grid.x * grid.y) > sm_count)) {
    // (only when one tile per CTA needs more than one wave of CTAs: a grid that is resident as a whole
    // gains nothing from pairing tiles, its CTAs would just run twice as long)
    // (bf16 weights pass through unwidened: no operand buffers, the 32 KiB stage feeds the MMA directly)
    const int wb = p->w4 == 2 ? 17408 : (p->w4 == 1 ? 16384 : 32768);
    const int ubytes = widen_l ? 2 * 32768 : 0;
    int st2 = 3;
    while (st2 > 2 && st2 * (wb + 2 * 16384) + ubytes + 1024 > kSmemLimit) --st2;
    const int smem2 = st2 * (wb + 2 * 16384) + ubytes + 1024;
    if (smem2 <= kSmemLimit) {
      q.mtiles = 2;
      dim3 grid2((p->M + 255) / 256, p->N_pad / 256, 1);      // token tile pairs run fastest (see raster_m in the kernel)
      return static_cast<int>(saber::launch(p->w4 == 3 ? gemm_bf16_kernel : gemm_i8_kernel, grid2, dim3(kGemmThreads), smem2, stream, 2, q, st2));
    }
  }
  // CTAs that wait for one another (split-K parts, tails) need the grid resident as a whole: it has
  // at most one CTA per SM and no kernel of this library waits on a LATER launch, so a plain
  // (programmatic) launch gets there; the cooperative attribute, which serialises the launch, is a switch.
  const int lflags = ((q.coop != 0 && g_coop_launch) ? 1 : 0) | 2;
  if (p->tail_mode == 2) {
    q.tail_row = nullptr;
    RowOpParams tail = *p->tail_row;
    // One GPU, integer partial sums meeting in the accumulator blocks: the row tail reads the blocks
    // itself (scales, rounds to bf16 exactly as the GEMM's own read-out would), so the splits neither
    // wait for one another nor write and re-read the bf16 tile.  These launches use blocks of their
    // own (acc_tail) which they clean themselves: the shared blocks stay zero between launches.
    if (p->splits > 1 && p->acc_tail != nullptr && p->w4 != 2 && p->tp_nranks <= 1 && tail.tp_nranks <= 1 &&
        tail.a == p->out && tail.K == p->N && tail.lda == p->ldo && p->N == p->N_pad) {
      q.tail_mode = 3;
      q.acc = p->acc_tail;
      tail.acc = p->acc_tail;
      tail.acc_a_scale = p->a_scale;
      tail.acc_w_scale = p->w_scale;
      tail.acc_nt = p->nt;
      tail.acc_tiles_n = p->N_pad / 256;
    }
    return static_cast<int>(saber::launch(gemm_i8_tail_kernel, grid, dim3(kGemmThreads), smem, stream, lflags, q, stages, tail));
  }
  return static_cast<int>(saber::launch(p->w4 == 3 ? gemm_bf16_kernel : gemm_i8_kernel, grid, dim3(kGemmThreads), smem, stream, lflags, q, stages));
}

extern "C" int saber_gemm_i8_tail_ok(const saber::GemmI8Params* p) {
  int sm_count = 0;
  if (saber::device_setup(&sm_count) != 0) return 0;
  if (p->group_tiles || p->w4 >= 3 || p->nt <= 0) return 0;
  const int grid_y = (p->M + p->nt - 1) / p->nt;
  return (p->N_pad / 256) * (p->halves == 2 ? 2 : 1) * grid_y * p->splits <= sm_count ? 1 : 0;
}

extern "C" void saber_set_coop_launch(int on) { saber::g_coop_launch = on; }
extern "C" void saber_set_gemm_2sm(int on) { saber::g_gemm_2sm = on; }
extern "C" int saber_get_gemm_2sm() { return saber::g_gemm_2sm; }

// ------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in gemm_i8_noalloc.h).
//
// Some callers of this library may not allocate device memory at all: code that runs inside a
// region where cudaMalloc is forbidden or would deadlock (a stream that is being captured, a
// latency-critical loop that must never touch the allocator's locks, a host that gave the whole
// device to a framework-owned pool and exposes no allocator to plug-ins).  For them the split-K
// scratch of the GEMM (partial tiles, arrival counters, status word) lives in the array below,
// inside the library image: every GPU that loads the library holds these bytes until the process
// exits, whether or not the entry point is ever called.
namespace saber {
constexpr size_t kNoAllocPartialInts = 4u * 1024u * 1024u;           // 16 MiB of int32 partial sums
constexpr size_t kNoAllocCounterWords = 1024;                         // one per (m tile, n tile)
constexpr size_t kNoAllocHeaderBytes = 256 + kNoAllocCounterWords * 4;  // status word (padded) + counters
constexpr size_t kNoAllocBytes = kNoAllocHeaderBytes + kNoAllocPartialInts * 4;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
constexpr int kNoAllocMaxDevices = 64;
static void* g_noalloc_ptr[kNoAllocMaxDevices];        // device address of the array, per device
}  // namespace saber

extern "C" int saber_gemm_i8_noalloc(const uint8_t* w, const float* w_scale, const int8_t* a,
                                     const float* a_scale, __nv_bfloat16* out, uint32_t* status,
                                     int M, int M_pad, int N, int N_pad, int K, int nt, int splits,
                                     int w4, int ldo, cudaStream_t stream) {
  using namespace saber;
  if (splits < 1 || M_pad <= 0 || N_pad <= 0) return kNoAllocBadArgs;
  const size_t tiles = static_cast<size_t>(N_pad / 256) * static_cast<size_t>((M + nt - 1) / (nt > 0 ? nt : 1));
  const size_t need = static_cast<size_t>(splits) * tiles * 128u * 256u;   // one 128 x 256 block per (split, tile)
  if ((splits > 1 && need > kNoAllocPartialInts) || tiles > kNoAllocCounterWords) return kNoAllocTooLarge;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) return kNoAllocBadArgs;
  if (g_noalloc_ptr[dev] == nullptr) {
    // Set-up, once per device and with that device current.  In host code the array's NAME is only
    // a host-side stand-in: handing it to a kernel would fault (or, where the GPU can reach host
    // memory, quietly use the wrong bytes); the device address has to be asked for.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    int sms = 0;
    const int se = device_setup(&sms);      // shared-memory opt-in of every GEMM kernel, on THIS device
    if (se != 0) return se;
    g_noalloc_ptr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
  // The array keeps whatever the last call left: the status word and the counters must start at
  // zero (a call that gave up half-way leaves counters behind); partial tiles are overwritten.
  e = cudaMemsetAsync(base, 0, kNoAllocHeaderBytes, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  GemmI8Params p{};
  p.w = w; p.w_scale = w_scale; p.a = a; p.a_scale = a_scale; p.out = out;
  p.err = status ? status : reinterpret_cast<uint32_t*>(base);
  p.counters = reinterpret_cast<uint32_t*>(base + 256);
  p.ws = reinterpret_cast<int32_t*>(base + kNoAllocHeaderBytes);
  p.M = M; p.M_pad = M_pad; p.N = N; p.N_pad = N_pad; p.K = K;
  p.nt = nt; p.splits = splits; p.w4 = w4; p.ldo = ldo;
  return saber_gemm_i8_launch(&p, 0, stream);
}

// Reads back the library's own status word of the current device (what a call with status == null
// used): 0, or the code of the first bounded wait that ran out since the last call cleared it.
// Synchronises with `stream` first.  Returns a negative value when the entry point has not been
// used on this device yet.
extern "C" int saber_gemm_i8_noalloc_status(cudaStream_t stream) {
  using namespace saber;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices || g_noalloc_ptr[dev] == nullptr)
    return kNoAllocBadArgs;
  uint32_t word = 0;
  if (cudaMemcpyAsync(&word, g_noalloc_ptr[dev], sizeof(word), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return kNoAllocBadArgs;
  return static_cast<int>(word);
}
