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
      uint8_t* kdst = p.kv_cache +
                      ((static_cast<size_t>(blk) * p.nkv + kh) * 2 * kPageTokens + off) * kHeadDim;
      uint8_t* vdst = kdst + kPageTokens * kHeadDim;
      const float2 vv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(
          p.qkv + static_cast<size_t>(m) * p.ld + p.v_off + kh * kHeadDim + 2 * t));
      *reinterpret_cast<__nv_fp8x2_storage_t*>(kdst + 2 * t) = __nv_cvt_float2_to_fp8x2(
          make_float2(o2[0] * p.k_inv_scale, o2[1] * p.k_inv_scale), __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<__nv_fp8x2_storage_t*>(vdst + 2 * t) = __nv_cvt_float2_to_fp8x2(
          make_float2(vv.x * p.v_inv_scale, vv.y * p.v_inv_scale), __NV_SATFINITE, __NV_E4M3);
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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// 16 fp8 e4m3 (one uint4) -> 16 bf16 (two uint4)
__device__ __forceinline__ void fp8x16_to_bf16(const uint4 in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x, in.y, in.z, in.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(
          static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xFFFFu), __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      o[2 * i + h] = pack_bf16(f.x, f.y);
    }
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

constexpr int kAttnMaxWarps = 6;

__global__ void __launch_bounds__(32 * kAttnMaxWarps) attn_paged_kernel(const AttnParams p,
                                                                        const int hpb,
                                                                        const int hgroups) {
  pdl_wait();
  extern __shared__ __align__(16) uint8_t attn_smem[];
  // layout: Q [hpb][16][256] bf16 | K [16][256] bf16 | V [16][256] bf16, 512-byte rows, 16-byte
  // chunk index XOR (row & 7)
  const uint32_t q_s = static_cast<uint32_t>(__cvta_generic_to_shared(attn_smem));
  const uint32_t k_s = q_s + hpb * 8192;
  const uint32_t v_s = k_s + 8192;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.nq / p.nkv;
  const int kvh = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
  const int b = blockIdx.z / p.splits, sp = blockIdx.z % p.splits;
  const int hin = hg * hpb + warp;
  const bool active = hin < group;
  const int head = kvh * group + hin;
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

  // ---- Q tile
  if (active) {
    for (int i = lane; i < 16 * 32; i += 32) {
      const int r = i >> 5, c = i & 31;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < ntok)
        v = *reinterpret_cast<const uint4*>(
            p.q + (static_cast<size_t>(row0 + t0 + r) * p.nq + head) * kHeadDim + c * 8);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                       q_s + warp * 8192 + r * 512 + ((c ^ (r & 7)) << 4)),
                   "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                   : "memory");
    }
  }

  float O[32][4];
#pragma unroll
  for (int i = 0; i < 32; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const float scale_log2 = p.sm_scale * p.k_scale * 1.4426950408889634f;

  // ---- page prefetch into registers
  const int nthreads = blockDim.x;
  uint4 pre[3];
  auto prefetch = [&](int pg) {
    const int blk = p.block_table[static_cast<size_t>(b) * p.max_blocks + pg];
    const uint8_t* src =
        p.kv_cache + (static_cast<size_t>(blk) * p.nkv + kvh) * (2 * kPageTokens * kHeadDim);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int idx = threadIdx.x + i * nthreads;
      if (idx < 512) pre[i] = __ldg(reinterpret_cast<const uint4*>(src) + idx);
    }
  };
  // with fewer than 171 threads three chunks per thread do not cover 512: loop variant below
  const int rounds = (512 + nthreads * 3 - 1) / (nthreads * 3);  // 1 for >= 171 threads
  if (pg0 < pg1 && rounds == 1) prefetch(pg0);

  for (int pg = pg0; pg < pg1; ++pg) {
    __syncthreads();  // everyone is done with the previous page (and Q is written)
    if (rounds == 1) {
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int idx = threadIdx.x + i * nthreads;
        if (idx < 512) {
          const int isv = idx >> 8, key = (idx & 255) >> 4, c = (idx & 15) * 2;
          uint4 lo, hi;
          fp8x16_to_bf16(pre[i], lo, hi);
          const uint32_t base = (isv ? v_s : k_s) + key * 512;
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + ((c ^ (key & 7)) << 4)),
                       "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w)
                       : "memory");
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                           base + (((c + 1) ^ (key & 7)) << 4)),
                       "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                       : "memory");
        }
      }
    } else {
      const int blk = p.block_table[static_cast<size_t>(b) * p.max_blocks + pg];
      const uint8_t* src =
          p.kv_cache + (static_cast<size_t>(blk) * p.nkv + kvh) * (2 * kPageTokens * kHeadDim);
      for (int idx = threadIdx.x; idx < 512; idx += nthreads) {
        const int isv = idx >> 8, key = (idx & 255) >> 4, c = (idx & 15) * 2;
        uint4 lo, hi;
        fp8x16_to_bf16(__ldg(reinterpret_cast<const uint4*>(src) + idx), lo, hi);
        const uint32_t base = (isv ? v_s : k_s) + key * 512;
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + ((c ^ (key & 7)) << 4)),
                     "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w)
                     : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                         base + (((c + 1) ^ (key & 7)) << 4)),
                     "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                     : "memory");
      }
    }
    __syncthreads();
    if (rounds == 1 && pg + 1 < pg1) prefetch(pg + 1);
    if (!active) continue;

    // S = Q K^T  (16 x 16 per warp)
    float S[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      uint32_t a[4], kb[4];
      {
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * ks + (lane >> 4);
        ldsm_x4(q_s + warp * 8192 + r * 512 + ((c ^ (r & 7)) << 4), a);
      }
      {
        const int r = (lane & 7) + (lane >> 4) * 8, c = 2 * ks + ((lane >> 3) & 1);
        ldsm_x4(k_s + r * 512 + ((c ^ (r & 7)) << 4), kb);
      }
      mma_bf16(S[0], a, kb[0], kb[1]);
      mma_bf16(S[1], a, kb[2], kb[3]);
    }
    // scale, mask, online softmax (rows g and g + 8)
    float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rr = g + (e >> 1) * 8;
        const int key = pg * kPageTokens + nt * 8 + 2 * t + (e & 1);
        const bool ok = rr < ntok && key < kbase + rr;
        const float s = ok ? S[nt][e] * scale_log2 : -INFINITY;
        S[nt][e] = s;
        rmax[e >> 1] = fmaxf(rmax[e >> 1], s);
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
    uint32_t pa[4];
    {
      float pv[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[nt][e] = exp2f(S[nt][e] - msafe[e >> 1]);
      l_run[0] = l_run[0] * alpha[0] + pv[0][0] + pv[0][1] + pv[1][0] + pv[1][1];
      l_run[1] = l_run[1] * alpha[1] + pv[0][2] + pv[0][3] + pv[1][2] + pv[1][3];
      pa[0] = pack_bf16(pv[0][0], pv[0][1]);
      pa[1] = pack_bf16(pv[0][2], pv[0][3]);
      pa[2] = pack_bf16(pv[1][0], pv[1][1]);
      pa[3] = pack_bf16(pv[1][2], pv[1][3]);
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      O[i][0] *= alpha[0]; O[i][1] *= alpha[0];
      O[i][2] *= alpha[1]; O[i][3] *= alpha[1];
    }
    // O += P V
#pragma unroll
    for (int dt = 0; dt < 16; ++dt) {
      uint32_t vb[4];
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * dt + (lane >> 4);
      ldsm_x4_t(v_s + r * 512 + ((c ^ (r & 7)) << 4), vb);
      mma_bf16(O[2 * dt], pa, vb[0], vb[1]);
      mma_bf16(O[2 * dt + 1], pa, vb[2], vb[3]);
    }
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
      if (rr >= ntok) continue;
      const float inv = l_run[h2] > 0.f ? p.v_scale / l_run[h2] : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<size_t>(row0 + t0 + rr) * p.nq + head) * kHeadDim;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + 2 * t) =
            __floats2bfloat162_rn(O[i][2 * h2] * inv, O[i][2 * h2 + 1] * inv);
    }
  } else {
    const size_t pbase = ((static_cast<size_t>(b) * p.nq + head) * p.splits + sp) * 16;
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int rr = g + h2 * 8;
      float* dst = p.part_o + (pbase + rr) * kHeadDim;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) = make_float2(O[i][2 * h2], O[i][2 * h2 + 1]);
      if (t == 0) {
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
  if (p->splits > 1 && p->q_tiles != 1) return static_cast<int>(cudaErrorInvalidValue);
  const int group = p->nq / p->nkv;
  const int hgroups = (group + kAttnMaxWarps - 1) / kAttnMaxWarps;
  const int hpb = (group + hgroups - 1) / hgroups;
  const int smem = hpb * 8192 + 16384;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attn_paged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * 8192 + 16384);
    configured = true;
  }
  dim3 grid(p->q_tiles, p->nkv * hgroups, p->nseq * p->splits);
  saber::launch(attn_paged_kernel, dim3(grid), dim3(32 * hpb), smem, stream, 0, *p, hpb, hgroups);
  if (p->splits > 1)
    saber::launch(attn_combine_kernel, dim3(dim3(p->nseq * p->nq, 16)), dim3(256), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}
