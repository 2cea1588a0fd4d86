// Paged GQA attention for head_dim 256 with an fp8 (e4m3) KV cache, page = 16 tokens.
//
//   rope_kv   per (row, head): Gemma RMSNorm (1 + w) over the head, interleaved M-RoPE over the
//             first rot_dim dims (rotate-half pairing), queries written bf16, keys and values
//             written to the paged cache as fp8 with per-layer scales.  One launch replaces the
//             reference's qk_norm_rope + kv_append pair (crates/saber-kernels/hip/attn_glue.hip:97-130).
//   attn      one CTA = (tile of 16 query tokens, KV head [x head group], sequence x KV split);
//             warp w owns query head w of the GQA group, so a K/V page converted once to bf16 in
//             shared memory is reused by every head of the group.  Online softmax in the exp2
//             domain, ragged rows per sequence from cu_q, right-aligned causal mask
//             klimit(row) = kv_len - (n - 1) + row (the law of the reference's paged kernels,
//             crates/saber-kernels/hip/sattn_prims.h:26-55, sattn_decode.h:1-8).  Decode splits the
//             keys over CTAs and a combine kernel merges (m, l, O) partials (sattn_combine.h:1-6).
//
// The contraction here runs on warp-level mma (m16n8k16 bf16): decode attention is bound by the
// KV bytes it streams, not by tensor throughput.
#include "launch.cuh"
#include "ptx_sm100.cuh"
#include "attn.h"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace saber {

// ------------------------------------------------------------------------------- rope + kv append
__global__ void __launch_bounds__(128) rope_kv_kernel(const RopeKvParams p) {
  pdl_wait();
  __shared__ float y[kHeadDim];
  __shared__ float red[4];
  const int m = blockIdx.x;
  const int hh = blockIdx.y;
  const bool is_q = hh < p.nq;
  const int kh = hh - p.nq;
  const int t = threadIdx.x;
  const __nv_bfloat16* src =
      p.qkv + static_cast<size_t>(m) * p.ld + (is_q ? p.q_off + hh * kHeadDim : p.k_off + kh * kHeadDim);
  const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 2 * t));
  float ss = x.x * x.x + x.y * x.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((t & 31) == 0) red[t >> 5] = ss;
  __syncthreads();
  ss = red[0] + red[1] + red[2] + red[3];
  const float rstd = rsqrtf(ss * (1.f / kHeadDim) + p.eps);
  const float* w = is_q ? p.q_norm_w : p.k_norm_w;
  y[2 * t] = __bfloat162float(__float2bfloat16(x.x * rstd * (w[2 * t] + p.w_offset)));
  y[2 * t + 1] = __bfloat162float(__float2bfloat16(x.y * rstd * (w[2 * t + 1] + p.w_offset)));
  __syncthreads();
  float o2[2];
  const int half = p.rot_dim >> 1;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int d = 2 * t + e;
    float v = y[d];
    if (d < p.rot_dim) {
      const int j = d % half;
      int axis = 0;
      if ((j % 3) == 1 && j < 3 * p.sec_h) axis = 1;
      else if ((j % 3) == 2 && j < 3 * p.sec_w) axis = 2;
      const float posv = static_cast<float>(p.pos[static_cast<size_t>(axis) * p.M + m]);
      const float inv_freq = exp2f(-(2.f * j / p.rot_dim) * log2f(p.theta));
      float sn, cs;
      sincosf(posv * inv_freq, &sn, &cs);
      v = d < half ? y[d] * cs - y[d + half] * sn : y[d] * cs + y[d - half] * sn;
    }
    o2[e] = v;
  }
  if (is_q) {
    *reinterpret_cast<__nv_bfloat162*>(p.q_out + (static_cast<size_t>(m) * p.nq + hh) * kHeadDim + 2 * t) =
        __floats2bfloat162_rn(o2[0], o2[1]);
  } else {
    const int slot = p.slot_map[m];
    if (slot >= 0) {
      const int blk = slot / kPageTokens, off = slot % kPageTokens;
      const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
          p.qkv + static_cast<size_t>(m) * p.ld + p.v_off + kh * kHeadDim + 2 * t));
      const __nv_fp8x2_storage_t k2 = __nv_cvt_float2_to_fp8x2(
          make_float2(o2[0] * p.k_inv_scale, o2[1] * p.k_inv_scale), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t v2 = __nv_cvt_float2_to_fp8x2(
          make_float2(vv.x * p.v_inv_scale, vv.y * p.v_inv_scale), __NV_SATFINITE, __NV_E4M3);
      uint8_t* page = p.kv_cache + (static_cast<size_t>(blk) * p.nkv + kh) * (2 * kPageTokens * kHeadDim);
      if (p.page_layout == 1) {
        // core-matrix order: K [key group][dim chunk][8 keys][16 dims], V [dim group][8 dims][16 keys]
        const int d = 2 * t;
        uint8_t* kdst = page + (off >> 3) * 2048 + (d >> 4) * 128 + (off & 7) * 16 + (d & 15);
        *reinterpret_cast<__nv_fp8x2_storage_t*>(kdst) = k2;
        uint8_t* vdst = page + kPageTokens * kHeadDim + (d >> 3) * 128 + (d & 7) * 16 + off;
        vdst[0] = static_cast<uint8_t>(v2 & 0xFFu);
        vdst[16] = static_cast<uint8_t>(v2 >> 8);
      } else {
        uint8_t* kdst = page + off * kHeadDim;
        uint8_t* vdst = kdst + kPageTokens * kHeadDim;
        *reinterpret_cast<__nv_fp8x2_storage_t*>(kdst + 2 * t) = k2;
        *reinterpret_cast<__nv_fp8x2_storage_t*>(vdst + 2 * t) = v2;
      }
    }
  }
}

// ------------------------------------------------------------------------------- attention
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// 16 fp8 e4m3 (one uint4) -> 16 fp16 (two uint4): one conversion instruction per pair, exact
__device__ __forceinline__ void fp8x16_to_f16(const uint4 in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(
          static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
      o[2 * i + h] = static_cast<uint32_t>(hr.x) | (static_cast<uint32_t>(hr.y) << 16);
    }
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

constexpr int kAttnMaxWarps = 8;      // two warps (head-dim halves) per 16-row tile, up to four tiles per CTA
constexpr int kAttnMaxRing = 8;       // raw fp8 pages in flight per CTA (8 KiB each), fewer when shared memory is short
constexpr int kAttnOpBytes = 32768;   // the operand buffer: K [32 keys][256] fp16 | V [32 keys][256] fp16
constexpr int kAttnSmemBudget = 112 * 1024;   // two CTAs per SM

// One CTA = one (sequence, KV head, 16-token query tile, KV split).  A 16-row tile holds `hpt` query
// heads of the GQA group, `pack` rows each (tile row = head * pack + row): the heads of a group
// share K and V, so with few rows per sequence (decode) several heads ride in one MMA tile -- 2
// heads at 8 rows, 3 at 5, all 6 at one row -- instead of padding each to 16 rows.  Two warps work
// on a tile: both compute S = Q K^T (16 x 32) and the softmax, each accumulates one half of the
// head dim of O (64 accumulator registers instead of 128), which lets two CTAs share an SM.
// The raw fp8 pages of the split stream through a ring in shared memory, filled by bulk copies
// that complete on mbarriers; each iteration takes two pages, all threads widen them to fp16 into
// the operand buffer.
template <int MAXW, int MINB>
__global__ void __launch_bounds__(32 * MAXW, MINB) attn_paged_kernel(const AttnParams p,
                                                                           const int tpb,
                                                                           const int hgroups,
                                                                           const int hpt,
                                                                           const int pack,
                                                                           const int ring) {
  pdl_wait();
  extern __shared__ __align__(128) uint8_t attn_smem[];
  __shared__ uint64_t full_bar[kAttnMaxRing];
  // layout: Q [tpb][16][256] fp16 | operand buffer | raw ring; 512-byte rows, 16-byte chunk index
  // XOR (row & 7)
  const uint32_t q_s = static_cast<uint32_t>(__cvta_generic_to_shared(attn_smem));
  const uint32_t k_s = q_s + tpb * 8192;
  const uint32_t v_s = k_s + 16384;
  const uint32_t ring_s = k_s + kAttnOpBytes;
  const uint32_t bar_s = static_cast<uint32_t>(__cvta_generic_to_shared(full_bar));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = warp >> 1, dh = warp & 1;       // tile of this warp, half of the head dim it accumulates
  const int g = lane >> 2, t = lane & 3;
  const int group = p.nq / p.nkv;
  const int kvh = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
  const int b = blockIdx.z / p.splits, sp = blockIdx.z % p.splits;
  const int hin = (hg * tpb + tile) * hpt;         // first head (inside the group) of this warp's tile
  const bool active = hin < group;
  const int head0 = kvh * group + hin;
  auto row_head = [&](int rr) { return rr / pack; };
  auto row_tok = [&](int rr) { return rr - (rr / pack) * pack; };
  const int row0 = p.cu_q[b];
  const int n = p.cu_q[b + 1] - row0;
  const int t0 = blockIdx.x * 16;
  if (t0 >= n) return;
  const int ntok = min(16, n - t0);
  const int kvlen = p.kv_len[b];
  const int kbase = kvlen - (n - 1) + t0;  // klimit of tile row 0
  const int kmax = kbase + ntok - 1;       // klimit of the last live row
  const int pages = (kmax + kPageTokens - 1) / kPageTokens;
  const int per = (pages + p.splits - 1) / p.splits;
  const int pg0 = sp * per, pg1 = min(pages, pg0 + per);
  const int npages = max(0, pg1 - pg0);
  const int key_end = pg1 * kPageTokens;   // keys at or beyond belong to the next split

  if (threadIdx.x == 0) {
    for (int i = 0; i < ring; ++i) mbar_init(bar_s + 8 * i, 1);
    mbar_init_fence();
  }
  __syncthreads();
  auto issue = [&](int i) {   // page i of this split -> ring stage i % ring (thread 0 only)
    const int st = i % ring;
    int blk = pg0 + i < p.max_blocks ? p.block_table[static_cast<size_t>(b) * p.max_blocks + pg0 + i] : -1;
    if (blk < 0 || (p.n_blocks > 0 && blk >= p.n_blocks)) {   // never follow a bad table entry
      if (p.err) atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrBadIndex));
      blk = 0;
    }
    const uint8_t* src = p.kv_cache + (static_cast<size_t>(blk) * p.nkv + kvh) * (2 * kPageTokens * kHeadDim);
    mbar_arrive_expect_tx(bar_s + 8 * st, 2 * kPageTokens * kHeadDim);
    bulk_g2s(ring_s + st * 8192, src, 2 * kPageTokens * kHeadDim, bar_s + 8 * st);
  };
  int issued = 0;
  if (threadIdx.x == 0) {
    for (; issued < min(ring, npages); ++issued) issue(issued);
  }

  // ---- Q tile (bf16 -> fp16: exact for every value the normed, rotated q can take); both warps of a tile load it
  if (active) {
    for (int i = lane + 32 * dh; i < 16 * 32; i += 64) {
      const int r = i >> 5, c = i & 31;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int qh = row_head(r), qr = row_tok(r);
      if (qh < hpt && hin + qh < group && qr < ntok) {
        const uint4 raw = *reinterpret_cast<const uint4*>(
            p.q + (static_cast<size_t>(row0 + t0 + qr) * p.nq + head0 + qh) * kHeadDim + c * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          o[j] = pack_f16(f.x, f.y);
        }
        v = make_uint4(o[0], o[1], o[2], o[3]);
      }
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                       q_s + tile * 8192 + r * 512 + ((c ^ (r & 7)) << 4)),
                   "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                   : "memory");
    }
  }

  float O[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const float scale_log2 = p.sm_scale * p.k_scale * 1.4426950408889634f;
  const int nthreads = blockDim.x;
  const int niter = (npages + 1) >> 1;
  bool ok = true;

  for (int it = 0; it < niter; ++it) {
    // ---- widen the two pages of this iteration into the operand buffer
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = 2 * it + half;
      if (i < npages) {
        const int st = i % ring;
        if (ok) ok = mbar_wait(bar_s + 8 * st, (i / ring) & 1, p.err, kErrWaitFull);
        for (int idx = threadIdx.x; idx < 512; idx += nthreads) {
          const int isv = idx >> 8, key = half * 16 + ((idx & 255) >> 4), c = (idx & 15) * 2;
          uint4 raw, lo, hi;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                       : "r"(ring_s + st * 8192 + idx * 16));
          fp8x16_to_f16(raw, lo, hi);
          const uint32_t base = (isv ? v_s : k_s) + key * 512;
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + ((c ^ (key & 7)) << 4)),
                       "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w)
                       : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + (((c + 1) ^ (key & 7)) << 4)),
                       "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                       : "memory");
        }
      } else {
        // no second page: its keys are masked, but V must hold finite numbers (0 * inf = nan)
        for (int idx = threadIdx.x; idx < 512; idx += nthreads) {
          const int key = 16 + (idx >> 5), c = idx & 31;
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(v_s + key * 512 + (c << 4)), "r"(0u) : "memory");
        }
      }
    }
    // the operand buffer is complete and the two ring stages are free
    if (__syncthreads_or(ok ? 0 : 1)) { ok = false; break; }
    if (threadIdx.x == 0) {
      fence_proxy_async_smem();   // order the generic reads of the stages before the async refill
      for (int half = 0; half < 2; ++half)
        if (issued < npages && issued - ring <= 2 * it + half) { issue(issued); ++issued; }
    }
    if (active) {
      // ---- S = Q K^T  (16 x 32, computed by both warps of the tile)
      float S[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        uint32_t a[4], kb0[4], kb1[4];
        {
          const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * ks + (lane >> 4);
          ldsm_x4(q_s + tile * 8192 + r * 512 + ((c ^ (r & 7)) << 4), a);
        }
        {
          const int r = (lane & 7) + (lane >> 4) * 8, c = 2 * ks + ((lane >> 3) & 1);
          ldsm_x4(k_s + r * 512 + ((c ^ (r & 7)) << 4), kb0);
          ldsm_x4(k_s + (16 + r) * 512 + ((c ^ (r & 7)) << 4), kb1);
        }
        mma_f16(S[0], a, kb0[0], kb0[1]);
        mma_f16(S[1], a, kb0[2], kb0[3]);
        mma_f16(S[2], a, kb1[0], kb1[1]);
        mma_f16(S[3], a, kb1[2], kb1[3]);
      }
      // ---- scale, mask, online softmax (rows g and g + 8)
      float rmax[2] = {-INFINITY, -INFINITY};
      const int key0 = (pg0 + 2 * it) * kPageTokens;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int rr = g + (e >> 1) * 8;
          const int key = key0 + nt * 8 + 2 * t + (e & 1);
          const int mh = row_head(rr), mr = row_tok(rr);
          const bool live = mh < hpt && hin + mh < group && mr < ntok && key < kbase + mr && key < key_end;
          const float sv = live ? S[nt][e] * scale_log2 : -INFINITY;
          S[nt][e] = sv;
          rmax[e >> 1] = fmaxf(rmax[e >> 1], sv);
        }
      }
      float alpha[2], msafe[2];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        rmax[h2] = fmaxf(rmax[h2], __shfl_xor_sync(0xffffffffu, rmax[h2], 1));
        rmax[h2] = fmaxf(rmax[h2], __shfl_xor_sync(0xffffffffu, rmax[h2], 2));
        const float mnew = fmaxf(m_run[h2], rmax[h2]);
        msafe[h2] = mnew == -INFINITY ? 0.f : mnew;
        alpha[h2] = exp2f(m_run[h2] - msafe[h2]);
        m_run[h2] = mnew;
      }
      uint32_t pa[2][4];
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {   // 16 keys each
        float pv[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) pv[nt][e] = exp2f(S[2 * kk + nt][e] - msafe[e >> 1]);
        if (kk == 0) {
          l_run[0] *= alpha[0];
          l_run[1] *= alpha[1];
        }
        l_run[0] += pv[0][0] + pv[0][1] + pv[1][0] + pv[1][1];
        l_run[1] += pv[0][2] + pv[0][3] + pv[1][2] + pv[1][3];
        pa[kk][0] = pack_f16(pv[0][0], pv[0][1]);
        pa[kk][1] = pack_f16(pv[0][2], pv[0][3]);
        pa[kk][2] = pack_f16(pv[1][0], pv[1][1]);
        pa[kk][3] = pack_f16(pv[1][2], pv[1][3]);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        O[i][0] *= alpha[0]; O[i][1] *= alpha[0];
        O[i][2] *= alpha[1]; O[i][3] *= alpha[1];
      }
      // ---- O += P V on this warp's half of the head dim
#pragma unroll
      for (int dt = 0; dt < 8; ++dt) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          uint32_t vb[4];
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * (dh * 8 + dt) + (lane >> 4);
          ldsm_x4_t(v_s + r * 512 + ((c ^ (r & 7)) << 4), vb);
          mma_f16(O[2 * dt], pa[kk], vb[0], vb[1]);
          mma_f16(O[2 * dt + 1], pa[kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();    // every warp is done with the operand buffer before the next pages are widened into it
  }
  if (!ok) {
    // a page never arrived: the status word is set; do not leave while own copies may still land
    if (threadIdx.x == 0)
      for (int i = max(0, issued - ring); i < issued; ++i)
        mbar_wait(bar_s + 8 * (i % ring), (i / ring) & 1, p.err, kErrWaitDrain);
    return;
  }
  if (!active) return;

#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
    l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
  }
  if (p.splits == 1) {
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int rr = g + h2 * 8;
      const int oh = row_head(rr), orow = row_tok(rr);
      if (oh >= hpt || hin + oh >= group || orow >= ntok) continue;
      const float inv = l_run[h2] > 0.f ? p.v_scale / l_run[h2] : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<size_t>(row0 + t0 + orow) * p.nq + head0 + oh) * kHeadDim + dh * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + 2 * t) =
            __floats2bfloat162_rn(O[i][2 * h2] * inv, O[i][2 * h2 + 1] * inv);
    }
  } else {
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int rr0 = g + h2 * 8;
      const int oh = row_head(rr0), rr = row_tok(rr0);
      if (oh >= hpt || hin + oh >= group) continue;
      const size_t pbase = ((static_cast<size_t>(b) * p.nq + head0 + oh) * p.splits + sp) * 16;
      float* dst = p.part_o + (pbase + rr) * kHeadDim + dh * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) = make_float2(O[i][2 * h2], O[i][2 * h2 + 1]);
      if (t == 0 && dh == 0) {
        p.part_ml[(pbase + rr) * 2] = m_run[h2];
        p.part_ml[(pbase + rr) * 2 + 1] = l_run[h2];
      }
    }
  }
}

// grid (nseq * nq, 16), block 256: merge the split partials of one (sequence, head, row).
__global__ void __launch_bounds__(256) attn_combine_kernel(const AttnParams p) {
  pdl_wait();
  const int b = blockIdx.x / p.nq, head = blockIdx.x % p.nq;
  const int rr = blockIdx.y;
  const int row0 = p.cu_q[b];
  const int n = p.cu_q[b + 1] - row0;
  if (rr >= n) return;
  const size_t pbase = (static_cast<size_t>(b) * p.nq + head) * p.splits * 16;
  float mx = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, p.part_ml[(pbase + s * 16 + rr) * 2]);
  const float msafe = mx == -INFINITY ? 0.f : mx;
  float L = 0.f, acc = 0.f;
  const int d = threadIdx.x;
  for (int s = 0; s < p.splits; ++s) {
    const float w = exp2f(p.part_ml[(pbase + s * 16 + rr) * 2] - msafe);
    L += w * p.part_ml[(pbase + s * 16 + rr) * 2 + 1];
    acc += w * p.part_o[(pbase + s * 16 + rr) * kHeadDim + d];
  }
  const float inv = L > 0.f ? p.v_scale / L : 0.f;
  p.out[(static_cast<size_t>(row0 + rr) * p.nq + head) * kHeadDim + d] = __float2bfloat16(acc * inv);
}

}  // namespace saber

extern "C" int saber_rope_kv_launch(const saber::RopeKvParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->M <= 0) return 0;
  if (p->rot_dim > kHeadDim || (p->rot_dim & 3)) return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(rope_kv_kernel, dim3(dim3(p->M, p->nq + p->nkv)), dim3(128), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_attn_launch(const saber::AttnParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->nq % p->nkv || p->splits < 1) return static_cast<int>(cudaErrorInvalidValue);
  if (p->impl == 1) {      // tcgen05 kernel (core-matrix pages); the split partials share the combine kernel
    const int e = saber_attn_tc_launch(p, stream);
    if (e != 0) return e;
    if (p->splits > 1)
      saber::launch(attn_combine_kernel, dim3(dim3(p->nseq * p->nq, 16)), dim3(256), 0, stream, 0, *p);
    return static_cast<int>(cudaGetLastError());
  }
  if (p->splits > 1 && p->q_tiles != 1) return static_cast<int>(cudaErrorInvalidValue);
  if (p->window > 0) return static_cast<int>(cudaErrorInvalidValue);      // sliding windows: the tcgen05 kernel only
  const int group = p->nq / p->nkv;
  // decode (one query tile): pack several heads of the group into one 16-row tile
  int hpt = 1, pack = 16;
  if (p->q_tiles == 1 && p->pack_rows >= 1 && p->pack_rows <= 8) {
    pack = p->pack_rows;
    hpt = 16 / pack < group ? 16 / pack : group;
  }
  const int tiles = (group + hpt - 1) / hpt;              // 16-row tiles per KV head, two warps each
  // decode: up to four tiles per CTA, two CTAs per SM.  Prefill (many query tiles, no packing): one
  // CTA with all six tiles of the group, so that every page is widened once per KV head.
  const bool wide = p->q_tiles > 1 && tiles > kAttnMaxWarps / 2 && tiles <= 6;
  const int max_tpb = wide ? 6 : kAttnMaxWarps / 2;
  const int hgroups = (tiles + max_tpb - 1) / max_tpb;
  const int tpb = (tiles + hgroups - 1) / hgroups;
  const int budget = wide ? 200 * 1024 : kAttnSmemBudget;
  int ring = (budget - tpb * 8192 - kAttnOpBytes) / 8192;
  ring = ring > kAttnMaxRing ? kAttnMaxRing : ring;
  const int smem = tpb * 8192 + kAttnOpBytes + ring * 8192;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attn_paged_kernel<kAttnMaxWarps, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBudget);
    cudaFuncSetAttribute(attn_paged_kernel<12, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  dim3 grid(p->q_tiles, p->nkv * hgroups, p->nseq * p->splits);
  if (wide)
    saber::launch(attn_paged_kernel<12, 1>, dim3(grid), dim3(64 * tpb), smem, stream, 0, *p, tpb, hgroups, hpt, pack, ring);
  else
    saber::launch(attn_paged_kernel<kAttnMaxWarps, 2>, dim3(grid), dim3(64 * tpb), smem, stream, 0, *p, tpb, hgroups, hpt, pack, ring);
  if (p->splits > 1)
    saber::launch(attn_combine_kernel, dim3(dim3(p->nseq * p->nq, 16)), dim3(256), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}
