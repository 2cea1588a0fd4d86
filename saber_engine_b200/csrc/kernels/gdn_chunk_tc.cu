// Chunked Gated DeltaNet prefill on the tensor cores (the algebra of gdn_chunk.cu, 64-row chunks):
//
//   prep  (parallel over value head x chunk): the pair products K K^T and Q K^T as tf32 `mma.sync`
//         tiles, the two triangular solves in fp32 (one right-hand-side column per thread, the
//         strictly lower matrix read as broadcast float4), and the chunk's operands written as bf16
//         tiles in the 128-byte-swizzled K-major layout the scan's MMAs read straight from shared
//         memory:  -W [i][k],  gamma_i q_i [i][k],  P [i][j],  (exp(G_C - G_j) k_j)^T [k][j],  and
//         U' [i][v] in fp32.
//   scan  (one CTA per value head and sequence, chunks in order): the state S [v][k] lives in
//         TENSOR MEMORY as the fp32 accumulator of its own update.  Per chunk, with S0 the state at
//         the chunk's start (a bf16 copy in shared memory is the A operand):
//             D_U | D_O [v][i] = S0 [(-W) ; gamma Q]^T        tcgen05.mma  128 x 128 x 128 (one B tile of 128 rows)
//             U^T [v][j]       = U'^T + D_U                   (threads: tensor memory -> bf16 tile)
//             D_O | S         += U^T [P ; K~^T]^T             tcgen05.mma  128 x 192 x 64 onto D_O and the scaled S0
//         (D_U, D_O and S are neighbouring column ranges of tensor memory, so each pair of products is one MMA shape)
//         Operands of the next chunk arrive by bulk copies (two stages) while the current one runs;
//         one thread issues the MMAs, four warps own the 128 tensor-memory lanes (one state row
//         each), completion travels through mbarriers.  Every wait is bounded: a wait that runs out
//         records its cause in the status word, the roles leave their loops, copies in flight are
//         waited for and the tensor memory is given back.
//
// bf16 operands with fp32 accumulation: the state copy that feeds the products is rounded to bf16
// once per chunk (the accumulator itself stays fp32), so outputs differ from the row-by-row kernel
// by about 2^-9 relative -- below the int8 rounding that follows the layer.
//
// Parity: crates/saber-kernels/hip/sgdn_scan.h:1-14 (chunk scan on WMMA tiles) and
// crates/saber-kernels/hip/saber_gdn_kkt_solve.hip:1-10 (the per-chunk triangular solve).
#include "gdn.h"
#include "launch.cuh"
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>

namespace saber {

namespace {

constexpr int kC = 64;                      // rows per chunk
constexpr int kPad = 132;                   // padded row stride (floats) of the fp32 K / Q tiles in the prep kernel
// the chunk's operand image (bytes): one bulk-copy stage of the scan
constexpr uint32_t kImgWQ = 0;              // -W ; gamma q   2 k-blocks x [128 rows: i of W, then i of q] x 128 B
constexpr uint32_t kImgP = 32768;           // P         [64 rows i] x 128 B   (K = j)   } one B tile of 192 rows
constexpr uint32_t kImgK = 40960;           // K~^T      [128 rows k] x 128 B  (K = j)   }
constexpr uint32_t kImgU = 57344;           // U'        fp32 [64 i][128 v]
constexpr uint32_t kImgBytes = 90112;       // 88 KiB: what a stage of the scan holds
constexpr uint32_t kImgStride = 90240;      // in memory the chunk's decay exp(G_C) (one float) follows the operands
constexpr int kScanThreads = 192;           // warps 0-3: one state row per thread; warp 4: copies; warp 5: MMAs
constexpr uint32_t kScanSmem = 2 * kImgBytes + 32768 + 16384 + 1024;   // stages | S0 tile | U^T tile | alignment

__device__ __forceinline__ float tc_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ size_t tc_chunk_slot(const int32_t* cu_rows, int b, int c) {
  return static_cast<size_t>(cu_rows[b] / kC + b + c);
}

__device__ __forceinline__ uint32_t f2tf32(float f) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
  return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

}  // namespace

// grid (HV, max_chunks, nseq), block 256.  dynamic smem: K | Q (fp32, padded) | A [64][64] | P [64][64]
__global__ void __launch_bounds__(256, 2) gdn_chunk_prep_tc_kernel(const GdnRecParams p, uint8_t* __restrict__ images) {
  // (no early trigger: the scan's CTAs take a whole SM's shared memory each and would sit on SMs this grid still needs)
  pdl_wait();
  extern __shared__ __align__(16) float cs[];
  float* Ks = cs;                          // [64][kPad]
  float* Qs = Ks + kC * kPad;              // [64][kPad]
  float* As = Qs + kC * kPad;              // [64][64] strictly lower: beta_i exp(G_i - G_j) k_i . k_j
  float* Ps = As + kC * kC;                // [64][64] lower incl. diagonal: exp(G_i - G_j) q_i . k_j
  __shared__ float Gs[kC], Bs[kC];
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  if (p.slots[b] < 0) return;
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  const int r0 = c * kC;
  if (r0 >= n) return;
  const int m = min(kC, n - r0);           // live rows of this chunk
  const int hk = h / (p.HV / p.HK);
  const int t = threadIdx.x;
  const int warp = t >> 5, lane = t & 31;
  const float neg_a = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[h];
  // right-hand sides of the solves, one column per thread (W columns for t < 128, U' columns else): the
  // value column comes from memory, so its 64 loads go out first and land behind the pair products
  float x[kC];
  const bool is_w = t < 128;
  const int col = is_w ? t : t - 128;
  if (!is_w) {
    const float* vcol = p.qkv + static_cast<size_t>(row0 + r0) * p.C + p.n_q + p.n_k + h * 128 + col;
#pragma unroll
    for (int i = 0; i < kC; ++i) x[i] = (i < m) ? vcol[static_cast<size_t>(i) * p.C] : 0.f;
  }
  for (int idx = t; idx < kC * 32; idx += 256) {        // float4 loads of the q and k rows
    const int r = idx >> 5, i4 = idx & 31;
    float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), qv = kv;
    if (r < m) {
      const float* xr = p.qkv + static_cast<size_t>(row0 + r0 + r) * p.C;
      qv = *reinterpret_cast<const float4*>(xr + hk * 128 + i4 * 4);
      kv = *reinterpret_cast<const float4*>(xr + p.n_q + hk * 128 + i4 * 4);
    }
    *reinterpret_cast<float4*>(Ks + r * kPad + i4 * 4) = kv;
    *reinterpret_cast<float4*>(Qs + r * kPad + i4 * 4) = qv;
  }
  if (t < kC) {
    float g = 0.f, be = 0.f;
    if (t < m) {
      const size_t mm = static_cast<size_t>(row0 + r0 + t);
      const float bb = __bfloat162float(p.ba[mm * p.ldba + h]);
      const float aa = __bfloat162float(p.ba[mm * p.ldba + p.HV + h]);
      g = neg_a * tc_softplus(aa + dtb);
      be = 1.f / (1.f + __expf(-bb));
    }
    // cumulative log decay: inclusive scan over the 64 rows (two warps, then the carry)
    float acc = g;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, acc, o);
      if (lane >= o) acc += up;
    }
    Gs[t] = acc;
    Bs[t] = be;
  }
  __syncthreads();
  if (t >= 32 && t < kC) Gs[t] += Gs[31];
  __syncthreads();
  const float gC = Gs[kC - 1];

  // ---- pair products on tf32 tiles: warp -> rows 16 mt .., columns 32 nh .. (four 8-wide tiles)
  {
    const int mt = warp >> 1, nh = warp & 1;
    const int g = lane >> 2, tq = lane & 3;
    float kk[4][4], qk[4][4];
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) kk[x][y] = qk[x][y] = 0.f;
    const bool any = nh * 32 <= mt * 16 + 15;        // the warp's columns reach the diagonal or below it
    if (any) {
      const float* ka = Ks + (mt * 16 + g) * kPad + tq;
      const float* qa = Qs + (mt * 16 + g) * kPad + tq;
      for (int ks = 0; ks < 16; ++ks) {
        uint32_t ak[4], aq[4];
        ak[0] = f2tf32(ka[ks * 8]);           ak[1] = f2tf32(ka[8 * kPad + ks * 8]);
        ak[2] = f2tf32(ka[ks * 8 + 4]);       ak[3] = f2tf32(ka[8 * kPad + ks * 8 + 4]);
        aq[0] = f2tf32(qa[ks * 8]);           aq[1] = f2tf32(qa[8 * kPad + ks * 8]);
        aq[2] = f2tf32(qa[ks * 8 + 4]);       aq[3] = f2tf32(qa[8 * kPad + ks * 8 + 4]);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          if (nh * 32 + nt * 8 > mt * 16 + 15) continue;      // tile wholly above the diagonal (warp-uniform)
          const float* kb = Ks + (nh * 32 + nt * 8 + g) * kPad + ks * 8 + tq;
          uint32_t bk[2];
          bk[0] = f2tf32(kb[0]);
          bk[1] = f2tf32(kb[4]);
          mma_tf32(kk[nt], ak, bk);
          mma_tf32(qk[nt], aq, bk);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = mt * 16 + g + (e >> 1) * 8;
        const int j = nh * 32 + nt * 8 + tq * 2 + (e & 1);
        const float d = j <= i ? __expf(Gs[i] - Gs[j]) : 0.f;
        As[i * kC + j] = j < i ? Bs[i] * d * kk[nt][e] : 0.f;
        Ps[i * kC + j] = d * qk[nt][e];
      }
    }
  }
  __syncthreads();

  uint8_t* img = images + (tc_chunk_slot(p.cu_rows, b, c) * p.HV + h) * static_cast<size_t>(kImgStride);
  // ---- forward substitution in place.  A is strictly lower, so whole float4 groups are used: the entries
  // at and right of the diagonal are zero and cancel the (finite) right-hand sides still sitting in x[j >= i].
  {
    if (is_w) {
#pragma unroll
      for (int i = 0; i < kC; ++i) x[i] = Bs[i] * __expf(Gs[i]) * Ks[i * kPad + col];
    } else {
#pragma unroll
      for (int i = 0; i < kC; ++i) x[i] *= Bs[i];
    }
#pragma unroll
    for (int i = 0; i < kC; ++i) {
      float acc = x[i];
      const float4* a4 = reinterpret_cast<const float4*>(As + i * kC);
#pragma unroll
      for (int j4 = 0; j4 < (i + 3) / 4; ++j4) {
        const float4 a = a4[j4];
        acc -= a.x * x[4 * j4] + a.y * x[4 * j4 + 1] + a.z * x[4 * j4 + 2] + a.w * x[4 * j4 + 3];
      }
      x[i] = acc;
    }
    if (is_w) {
      // -W as the B operand [i][k]: k-block col / 64, row i, byte (col % 64) * 2 inside the swizzled row
      uint8_t* wt = img + kImgWQ + (col >> 6) * 16384;
#pragma unroll
      for (int i = 0; i < kC; ++i)
        *reinterpret_cast<__nv_bfloat16*>(wt + sw128_offset(i, (col & 63) * 2)) = __float2bfloat16(-x[i]);
    } else {
      float* ut = reinterpret_cast<float*>(img + kImgU);
#pragma unroll
      for (int i = 0; i < kC; ++i) ut[i * 128 + col] = x[i];
    }
  }
  // ---- gamma_i q_i as the B operand [i][k]: 16-byte pieces (8 values along k)
  for (int idx = t; idx < kC * 16; idx += 256) {
    const int i = idx >> 4, k0 = (idx & 15) * 8;
    const float gi = __expf(Gs[i]);
    const float* q = Qs + i * kPad + k0;
    uint4 v;
    v.x = pack_bf16x2(q[0] * gi, q[1] * gi);
    v.y = pack_bf16x2(q[2] * gi, q[3] * gi);
    v.z = pack_bf16x2(q[4] * gi, q[5] * gi);
    v.w = pack_bf16x2(q[6] * gi, q[7] * gi);
    *reinterpret_cast<uint4*>(img + kImgWQ + (k0 >> 6) * 16384 + sw128_offset(64 + i, (k0 & 63) * 2)) = v;
  }
  // ---- (exp(G_C - G_j) k_j)^T as the B operand [k][j]: 16-byte pieces (8 values along j)
  for (int idx = t; idx < 128 * 8; idx += 256) {
    const int k = idx & 127, j0 = (idx >> 7) * 8;
    float e[8];
#pragma unroll
    for (int x2 = 0; x2 < 8; ++x2) e[x2] = Ks[(j0 + x2) * kPad + k] * __expf(gC - Gs[j0 + x2]);
    uint4 v;
    v.x = pack_bf16x2(e[0], e[1]);
    v.y = pack_bf16x2(e[2], e[3]);
    v.z = pack_bf16x2(e[4], e[5]);
    v.w = pack_bf16x2(e[6], e[7]);
    *reinterpret_cast<uint4*>(img + kImgK + sw128_offset(k, j0 * 2)) = v;
  }
  // ---- P as the B operand [i][j]
  for (int idx = t; idx < kC * 8; idx += 256) {
    const int i = idx >> 3, j0 = (idx & 7) * 8;
    const float* pr = Ps + i * kC + j0;
    uint4 v;
    v.x = pack_bf16x2(pr[0], pr[1]);
    v.y = pack_bf16x2(pr[2], pr[3]);
    v.z = pack_bf16x2(pr[4], pr[5]);
    v.w = pack_bf16x2(pr[6], pr[7]);
    *reinterpret_cast<uint4*>(img + kImgP + sw128_offset(i, j0 * 2)) = v;
  }
  if (t == 0) *reinterpret_cast<float*>(img + kImgBytes) = __expf(gC);
}

// grid (HV, nseq), block 192
__global__ void __launch_bounds__(kScanThreads, 1) gdn_chunk_scan_tc_kernel(const GdnRecParams p,
                                                                           const uint8_t* __restrict__ images) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[8];     // full[2] | empty[2] | s_ready | u_ready | mma1 | mma2
  __shared__ uint32_t tmem_base_s;
  const int h = blockIdx.x, b = blockIdx.y;
  const int slot = p.slots[b];
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  if (slot < 0 || n <= 0) return;               // uniform for the CTA, before any barrier
  const int nchunks = (n + kC - 1) / kC;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage0 = smem_base;
  const uint32_t s_tile = smem_base + 2 * kImgBytes;          // S0 as bf16 [128 v][128 k]: two k-blocks of 16 KiB
  const uint32_t u_tile = s_tile + 32768;                     // U^T as bf16 [128 v][64 j]
  uint8_t* const gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = smem_u32(&bars[2]);
  const uint32_t bar_s = smem_u32(&bars[4]), bar_u = smem_u32(&bars[5]);
  const uint32_t bar_m1 = smem_u32(&bars[6]), bar_m2 = smem_u32(&bars[7]);
  constexpr uint32_t kCols = 256;               // D_U: 64 columns, D_O: 64, S: 128
  if (threadIdx.x == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_full + 8, 1);
    mbar_init(bar_empty, 1);
    mbar_init(bar_empty + 8, 1);
    mbar_init(bar_s, 128);
    mbar_init(bar_u, 128);
    mbar_init(bar_m1, 1);
    mbar_init(bar_m2, 1);
    mbar_init_fence();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&tmem_base_s), kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_base_s;
  const uint32_t d_u = tmem, d_o = tmem + 64u, d_s = tmem + 128u;
  const size_t slot0 = tc_chunk_slot(p.cu_rows, b, 0);
  const uint8_t* img0 = images + (slot0 * p.HV + h) * static_cast<size_t>(kImgStride);
  const size_t img_step = static_cast<size_t>(p.HV) * kImgStride;     // consecutive chunks of a sequence
  pdl_wait();                                   // the images are the prep kernel's output

  if (warp == 4) {
    // ------------------------------------------------------------------ copies
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int c = 0; c < nchunks; ++c) {
        const int s = c & 1;
        if (c >= 2 && !mbar_wait(bar_empty + 8 * s, ((c >> 1) - 1) & 1, p.err, kErrWaitEmpty)) { ok = false; break; }
        mbar_arrive_expect_tx(bar_full + 8 * s, kImgBytes);
        const uint8_t* src = img0 + static_cast<size_t>(c) * img_step;
        const uint32_t dst = stage0 + s * kImgBytes;
        bulk_g2s(dst + kImgWQ, src + kImgWQ, 32768, bar_full + 8 * s);
        bulk_g2s(dst + kImgP, src + kImgP, 24576, bar_full + 8 * s);
        bulk_g2s(dst + kImgU, src + kImgU, 32768, bar_full + 8 * s);
        issued = c + 1;
      }
      if (!ok) {
        // unwinding: do not leave while a copy of this CTA is still in flight
        for (int c = max(0, issued - 2); c < issued; ++c) mbar_wait(bar_full + 8 * (c & 1), (c >> 1) & 1, p.err, kErrWaitDrain);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t id128 = make_idesc(kCFmtF32, kFmtBF16, kFmtBF16, 128, 128);
      const uint32_t id192 = make_idesc(kCFmtF32, kFmtBF16, kFmtBF16, 128, 192);
      const uint64_t desc_hi = make_desc_k128(0);
      const uint64_t a_s = desc_hi | static_cast<uint64_t>((s_tile & 0x3FFFFu) >> 4);
      const uint64_t a_u = desc_hi | static_cast<uint64_t>((u_tile & 0x3FFFFu) >> 4);
      bool ok = true;
      int committed = 0;
      for (int c = 0; c < nchunks && ok; ++c) {
        const int s = c & 1;
        const uint32_t st = stage0 + s * kImgBytes;
        const uint64_t b_wq = desc_hi | static_cast<uint64_t>(((st + kImgWQ) & 0x3FFFFu) >> 4);
        const uint64_t b_pk = desc_hi | static_cast<uint64_t>(((st + kImgP) & 0x3FFFFu) >> 4);
        if (!mbar_wait(bar_full + 8 * s, (c >> 1) & 1, p.err, kErrWaitFull)) { ok = false; break; }
        if (!mbar_wait(bar_s, c & 1, p.err, kErrWaitReady)) { ok = false; break; }
        tc_fence_after_sync();
        // D_U | D_O = S0 [(-W) ; gamma Q]^T: K = 128 as two k-blocks x four 16-value steps
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int q = 0; q < 4; ++q)
            mma_f16_ss(d_u, a_s + kb * (16384 >> 4) + 2 * q, b_wq + kb * (16384 >> 4) + 2 * q, id128, (kb | q) != 0 ? 1u : 0u);
        mma_commit(bar_m1);
        if (!mbar_wait(bar_u, c & 1, p.err, kErrWaitReady)) { ok = false; committed = 2 * c + 1; break; }
        tc_fence_after_sync();
        // D_O | S += U^T [P ; K~^T]^T : K = 64 (j), 192 accumulator columns from D_O on
#pragma unroll
        for (int q = 0; q < 4; ++q) mma_f16_ss(d_o, a_u + 2 * q, b_pk + 2 * q, id192, 1u);
        mma_commit(bar_empty + 8 * s);
        mma_commit(bar_m2);
        committed = 2 * c + 2;
      }
      // unwinding: the MMAs issued so far have to retire before the tensor memory goes back
      if (!ok && committed > 0) {
        const int c = (committed - 1) >> 1;
        mbar_wait((committed & 1) ? bar_m1 : bar_m2, c & 1, nullptr, 0);
      }
    }
  } else {
    // ------------------------------------------------------------------ state rows: thread = value row v
    const int v = threadIdx.x;                                  // 0..127 = tensor-memory lane
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    float* srow = p.state + ((static_cast<size_t>(slot) * p.HV + h) * 128 + v) * 128;
    uint8_t* s_row_gen = gen_base + 2 * kImgBytes;              // generic pointer of the S0 tile
    uint8_t* u_row_gen = s_row_gen + 32768;
    bool ok = true;
    int m_prev = 0;
    for (int c = 0; c <= nchunks && ok; ++c) {
      const bool last = c == nchunks;
      if (c > 0) {
        if (!mbar_wait(bar_m2, (c - 1) & 1, p.err, kErrWaitAcc)) { ok = false; break; }
        tc_fence_after_sync();
        // outputs of chunk c - 1 first: the next products overwrite D_O
        uint32_t r0[32], r1[32];
        tmem_ld32(d_o + lane_off, r0);
        tmem_ld32(d_o + lane_off + 32, r1);
        tmem_ld_wait();
        float* orow = p.out + static_cast<size_t>(row0 + (c - 1) * kC) * (static_cast<size_t>(p.HV) * 128) + h * 128 + v;
        const size_t ldo = static_cast<size_t>(p.HV) * 128;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < m_prev) orow[i * ldo] = __uint_as_float(r0[i]);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (32 + i < m_prev) orow[(32 + i) * ldo] = __uint_as_float(r1[i]);
      }
      // ---- (a) state at the start of chunk c (row v, 128 values along k)
      uint32_t sr[128];
      if (c > 0) {
#pragma unroll
        for (int g = 0; g < 4; ++g) tmem_ld32(d_s + lane_off + g * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[g * 32]));
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const float4 f = *reinterpret_cast<const float4*>(srow + x * 4);
          sr[4 * x] = __float_as_uint(f.x); sr[4 * x + 1] = __float_as_uint(f.y);
          sr[4 * x + 2] = __float_as_uint(f.z); sr[4 * x + 3] = __float_as_uint(f.w);
        }
      }
      if (last) {                         // the final state goes back to memory as fp32
#pragma unroll
        for (int x = 0; x < 32; ++x)
          *reinterpret_cast<float4*>(srow + x * 4) = make_float4(__uint_as_float(sr[4 * x]), __uint_as_float(sr[4 * x + 1]),
                                                                 __uint_as_float(sr[4 * x + 2]), __uint_as_float(sr[4 * x + 3]));
        break;
      }
      // the bf16 copy the first product multiplies with: k = 8 q .. 8 q + 7 is 16 bytes of k-block q / 8
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        uint4 w;
        w.x = pack_bf16x2(__uint_as_float(sr[8 * q]), __uint_as_float(sr[8 * q + 1]));
        w.y = pack_bf16x2(__uint_as_float(sr[8 * q + 2]), __uint_as_float(sr[8 * q + 3]));
        w.z = pack_bf16x2(__uint_as_float(sr[8 * q + 4]), __uint_as_float(sr[8 * q + 5]));
        w.w = pack_bf16x2(__uint_as_float(sr[8 * q + 6]), __uint_as_float(sr[8 * q + 7]));
        *reinterpret_cast<uint4*>(s_row_gen + (q >> 3) * 16384 + sw128_offset(v, (q & 7) * 16)) = w;
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(bar_s);
      // gamma_C S0 back into tensor memory while the first product runs (the second product adds onto it:
      // ordered by the store wait before this thread's arrival on bar_u)
      const float gc = *reinterpret_cast<const float*>(img0 + static_cast<size_t>(c) * img_step + kImgBytes);
#pragma unroll
      for (int x = 0; x < 128; ++x) sr[x] = __float_as_uint(__uint_as_float(sr[x]) * gc);
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_st32(d_s + lane_off + g * 32, *reinterpret_cast<const uint32_t(*)[32]>(&sr[g * 32]));
      m_prev = min(kC, n - c * kC);
      // ---- (c) U^T = U'^T + D_U as the bf16 A operand of the last two products
      const int s = c & 1;
      if (!mbar_wait(bar_full + 8 * s, (c >> 1) & 1, p.err, kErrWaitFull)) { ok = false; break; }   // U' of this stage
      if (!mbar_wait(bar_m1, c & 1, p.err, kErrWaitAcc)) { ok = false; break; }
      tc_fence_after_sync();
      const float* up = reinterpret_cast<const float*>(gen_base + s * kImgBytes + kImgU) + v;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld32(d_u + lane_off + half * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float u8[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) u8[x] = __uint_as_float(r[8 * q + x]) + up[(half * 32 + q * 8 + x) * 128];
          uint4 w;
          w.x = pack_bf16x2(u8[0], u8[1]);
          w.y = pack_bf16x2(u8[2], u8[3]);
          w.z = pack_bf16x2(u8[4], u8[5]);
          w.w = pack_bf16x2(u8[6], u8[7]);
          *reinterpret_cast<uint4*>(u_row_gen + sw128_offset(v, half * 64 + q * 16)) = w;
        }
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(bar_u);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kCols);
  }
}

}  // namespace saber

extern "C" size_t saber_gdn_chunk_tc_scratch_bytes(int max_rows, int nseq, int HV) {
  const size_t slots = static_cast<size_t>(max_rows / saber::kC + nseq + 1);
  return slots * HV * saber::kImgStride;
}

extern "C" int saber_gdn_chunk_tc_launch(const saber::GdnRecParams* p, int nseq, int max_rows, float* scratch,
                                         cudaStream_t stream) {
  using namespace saber;
  if (p->HV % p->HK || !p->commit || scratch == nullptr || max_rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  // (q | k | v channel offsets are read as float4; the bulk copies want 16-byte aligned images)
  if ((p->C & 3) || (p->n_q & 3) || (p->n_k & 3) || (reinterpret_cast<uintptr_t>(scratch) & 15u) || (reinterpret_cast<uintptr_t>(p->qkv) & 15u))
    return static_cast<int>(cudaErrorInvalidValue);
  const int prep_smem = (2 * kC * kPad + 2 * kC * kC) * sizeof(float);
  static bool configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gdn_chunk_prep_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(gdn_chunk_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kScanSmem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  uint8_t* images = reinterpret_cast<uint8_t*>(scratch);
  const int max_chunks = (max_rows + kC - 1) / kC;
  saber::launch(gdn_chunk_prep_tc_kernel, dim3(p->HV, max_chunks, nseq), dim3(256), prep_smem, stream, 0, *p, images);
  saber::launch(gdn_chunk_scan_tc_kernel, dim3(p->HV, nseq), dim3(kScanThreads), kScanSmem, stream, 0, *p,
                static_cast<const uint8_t*>(images));
  return static_cast<int>(cudaGetLastError());
}
