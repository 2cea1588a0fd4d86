// Device-side body of the register-resident row producers, shared by the stand-alone row kernels
// (rowops.cu, one CTA per row) and by the GEMM's fused row tail (gemm_i8.cu: after a grid-wide
// barrier the GEMM's own CTAs walk the rows of the tile they have just produced together, so the
// add + RMSNorm + quantise step that follows a row-parallel linear costs no launch of its own).
//
// The law is the one stated at the top of rowops.cu; both callers produce the same bytes.
#pragma once
#include "rowops.h"
#include "gemm_i8.h"
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>

namespace saber {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Every thread of the CTA calls (the barriers are __syncthreads).
template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* red) {
  v = kMax ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // protect `red` against the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  float r = (lane < nw) ? red[lane] : 0.f;
  r = kMax ? warp_max(r) : warp_sum(r);
  return r;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// four values -> four quantised bytes (int8 round-to-nearest with clamp, or fp8 e4m3 saturating)
__device__ __forceinline__ uint32_t quant4(float a, float b, float c, float d, float inv, int qfmt) {
  if (qfmt == 1) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a * inv, b * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c * inv, d * inv), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
  }
  const float x[4] = {a, b, c, d};
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int qi = __float2int_rn(x[j] * inv);
    qi = max(-127, min(127, qi));
    word |= (static_cast<uint32_t>(qi) & 0xFFu) << (8 * j);
  }
  return word;
}

// One NVFP4 block: 16 values of row m, chunk `ch` (values [16 ch, 16 ch + 16)), token scale g = amax / (6 * 448).
// Block scale = e4m3(block amax / (6 g)) (round to nearest, saturating), codes = e2m1(v / (scale * g)) to
// nearest even; eight packed bytes go to the row's 128-byte line of k-block ch / 16 (16-byte chunks
// XOR-swizzled by the row like every activation tile), the scale byte to its atom.
__device__ __forceinline__ void fp4_store_chunk(const float (&v)[16], float g, int ch, int m, int M_pad,
                                                int8_t* q, uint8_t* q_sf, int sf_m_tiles) {
  float bmax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
  const float want = g > 0.f ? fminf(bmax / 6.f / g, 448.f) : 0.f;
  const __nv_fp8_storage_t sfb = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
  const float sf = __half2float(__half(__nv_cvt_fp8_to_halfraw(sfb, __NV_E4M3)));
  const float denom = fmaxf(sf * g, 1e-30f);
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_fp4x2_storage_t b = __nv_cvt_float2_to_fp4x2(make_float2(v[2 * i] / denom, v[2 * i + 1] / denom), __NV_E2M1, cudaRoundNearest);
    w[i >> 2] |= static_cast<uint32_t>(b) << (8 * (i & 3));
  }
  const int kb = ch >> 4, c8 = ch & 15;
  const size_t off = (static_cast<size_t>(kb) * M_pad + m) * 128 + ((((c8 >> 1) ^ (m & 7)) & 7) << 4) + ((c8 & 1) << 3);
  *reinterpret_cast<uint2*>(q + off) = make_uint2(w[0], w[1]);
  const size_t so = ((static_cast<size_t>(kb) * sf_m_tiles + (m >> 7)) * 4 + (c8 >> 2)) * 512 + ((m & 31) << 4) + (((m >> 5) & 3) << 2) + (c8 & 3);
  q_sf[so] = sfb;
}

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

template <bool kCg = false>
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  Bf16x8 raw;
  if (kCg) {   // produced by other CTAs of the same kernel: read through L2
    const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p));
    raw = *reinterpret_cast<const Bf16x8*>(&u);
  } else {
    raw = *reinterpret_cast<const Bf16x8*>(p);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(raw.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  Bf16x8 raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) raw.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<Bf16x8*>(p) = raw;
}

// One token row `m`, handled by ALL threads of the CTA (blockDim.x threads, any multiple of 32 up
// to 1024): a thread owns the 16-value chunks tid, tid + blockDim.x, ... (at most MAXC of them) and
// keeps them in registers between the passes.  kCg: the primary input was written by other CTAs of
// the running kernel (fused tail) and is read through L2.  `red` is 32 floats of shared memory.
// Rows m >= p.M are padding rows: zeros.  Returns without side effects for rows a sequence-parallel
// rank does not own.
template <int MODE, int MAXC, bool kCg, bool kAcc = false>
__device__ __forceinline__ void row_reg_body(const RowOpParams& p, const int m, float* red) {
  const int K = p.K;
  const int nthr = blockDim.x;
  const int nchunk = K >> 4;
  const bool sp = MODE == kRowAddRms && p.sp_rpr > 0 && p.tp_nranks > 1;
  if (sp && (m >= p.M || m / p.sp_rpr != p.sp_rank)) return;   // sequence parallel: not this rank's row
  if (m >= p.M) {  // padding row: zeros
    if (p.q) {
      const int npiece = p.qfmt == 2 ? (K >> 5) : nchunk;      // 16-byte pieces of the row (packed FP4: half as many)
      for (int ch = threadIdx.x; ch < npiece; ch += nthr) {
        const int kb = ch >> 3, c = ch & 7;
        int8_t* dst = p.q + (static_cast<size_t>(kb) * p.M_pad + m) * 128 + (((c ^ (m & 7)) & 7) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
      if (threadIdx.x == 0) p.scale[m] = 0.f;
    }
    return;
  }
  uint32_t tp_par = 0;
  if (MODE == kRowAddRms && p.tp_nranks > 1) {
    const uint32_t seq = *p.tp_seq_base + static_cast<uint32_t>(p.tp_site) + 1u;
    tp_par = seq & 1u;
    const int nflags = p.tp_nranks * p.tp_tiles_n;
    for (int f = threadIdx.x; f < nflags; f += nthr) {
      const int src = f / p.tp_tiles_n, tn = f - src * p.tp_tiles_n;
      const int tile_id = (m / p.tp_nt) * p.tp_tiles_n + tn;
      const uint32_t* flag = p.tp_flags + (static_cast<size_t>(tp_par) * p.tp_nranks + src) * kTpMaxTiles + tile_id;
      const long long t0 = clock64();
      uint32_t spins = 0;
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (static_cast<int32_t>(v - seq) >= 0) break;
        if ((++spins & 1023u) == 0u && clock64() - t0 > kWaitLimitCycles) {
          if (p.err) atomicCAS(p.err, 0u, static_cast<uint32_t>(kErrWaitPeer));
          break;
        }
      }
    }
    __syncthreads();
  }
  float hv[MAXC][16];   // the row's values of this thread (ADD_RMS: first the sums, then the normed row)
  float amax = 0.f;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int ch = threadIdx.x + c * nthr;
    if (ch >= nchunk) continue;
    const int k0 = ch << 4;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int k = k0 + half * 8;
      float x[8];
      if (MODE == kRowAddRms) {
        if (p.tp_nranks > 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = 0.f;
          for (int src = 0; src < p.tp_nranks; ++src) {   // fixed order: identical sums on every rank
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(
                p.tp_recv + ((static_cast<size_t>(tp_par) * p.tp_nranks + src) * p.tp_rows + m) * p.tp_ld + k));
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(h2[i]);
              x[2 * i] += f.x;
              x[2 * i + 1] += f.y;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(__float2bfloat16(x[i]));
        } else if (kAcc) {
          // eight columns of this row = two four-column groups of the accumulator block of their tile
          const int tm = m / p.acc_nt, r = m - tm * p.acc_nt;
          const int tn = k >> 8, c4 = (k & 255) >> 2;
          int32_t* blk = p.acc + (static_cast<size_t>(tm) * p.acc_tiles_n + tn) * p.acc_nt * 256;
          const float asc = p.acc_a_scale[m];
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const int4* src = reinterpret_cast<const int4*>(blk + (static_cast<size_t>(c4 + g) * p.acc_nt + r) * 4);
            const int4 v = __ldcg(src);      // (the GEMM's first split cleans the block at the start of the next launch)
            const float4 ws = *reinterpret_cast<const float4*>(p.acc_w_scale + k + 4 * g);
            const __nv_bfloat162 b0 = __floats2bfloat162_rn(static_cast<float>(v.x) * (asc * ws.x), static_cast<float>(v.y) * (asc * ws.y));
            const __nv_bfloat162 b1 = __floats2bfloat162_rn(static_cast<float>(v.z) * (asc * ws.z), static_cast<float>(v.w) * (asc * ws.w));
            const float2 f0 = __bfloat1622float2(b0), f1 = __bfloat1622float2(b1);
            x[4 * g] = f0.x; x[4 * g + 1] = f0.y; x[4 * g + 2] = f1.x; x[4 * g + 3] = f1.y;
          }
        } else if (p.a) {
          load8<kCg>(p.a + static_cast<size_t>(m) * p.lda + k, x);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = 0.f;
        }
        if (p.res) {
          float r[8];
          load8(p.res + static_cast<size_t>(m) * p.ldres + k, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] += r[i];
          store8(p.res + static_cast<size_t>(m) * p.ldres + k, x);
          if (p.res_copy) store8(p.res_copy + static_cast<size_t>(m) * p.ldres + k, x);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
      } else {
        if (MODE == kRowSiluMul) {
          float g[8], u[8];
          const int kg = p.silu_pair ? ((k >> 7) << 8) + (k & 127) : k;      // paired tiles: gate | up per 128 features
          const int ku = p.silu_pair ? kg + 128 : K + k;
          load8<kCg>(p.a + static_cast<size_t>(m) * p.lda + kg, g);
          load8<kCg>(p.a + static_cast<size_t>(m) * p.lda + ku, u);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = silu_f(g[i]) * u[i];
        } else if (MODE == kRowGateSig) {
          float a[8], b[8];
          load8<kCg>(p.a + static_cast<size_t>(m) * p.lda + k, a);
          load8(p.b + static_cast<size_t>(m) * p.ldb + k, b);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = a[i] * sigmoid_f(b[i]);
        } else {
          load8<kCg>(p.a + static_cast<size_t>(m) * p.lda + k, x);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[i] = __bfloat162float(__float2bfloat16(x[i]));
          amax = fmaxf(amax, fabsf(x[i]));
        }
        if (p.out) store8(p.out + static_cast<size_t>(m) * p.ldout + k, x);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) hv[c][half * 8 + i] = x[i];
    }
  }
  if (MODE == kRowAddRms) {
    ss = block_reduce<false>(ss, red);
    const float rstd = rsqrtf(ss / static_cast<float>(K) + p.eps);
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * nthr;
      if (ch >= nchunk) continue;
      const int k0 = ch << 4;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float x[8];
        const float4 w0 = *reinterpret_cast<const float4*>(p.w + k0 + half * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(p.w + k0 + half * 8 + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[i] = __bfloat162float(__float2bfloat16(hv[c][half * 8 + i] * rstd * (wv[i] + p.w_offset)));
          amax = fmaxf(amax, fabsf(x[i]));
          hv[c][half * 8 + i] = x[i];
        }
        if (p.out) store8(p.out + static_cast<size_t>(m) * p.ldout + k0 + half * 8, x);
      }
    }
  }
  if (p.had_sign != nullptr && p.q) {
    // 32-point Hadamard per block = this thread's 16 values (one chunk) and its lane neighbour's
    // (chunks 2j and 2j + 1 belong to lanes 2i and 2i + 1): four butterfly stages in registers,
    // the fifth across the lane pair.  The quantisation scale is taken AFTER the rotation.
    amax = 0.f;
    const bool odd = threadIdx.x & 1;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * nthr;
      const bool on = ch < nchunk;               // (nchunk is even: K is a multiple of 128)
      if (on) {
#pragma unroll
        for (int i = 0; i < 16; ++i) hv[c][i] *= p.had_sign[(ch << 4) + i];
#pragma unroll
        for (int st = 1; st < 16; st <<= 1)
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if ((i & st) == 0) {
              const float a = hv[c][i], b2 = hv[c][i | st];
              hv[c][i] = a + b2;
              hv[c][i | st] = a - b2;
            }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, hv[c][i], 1);
        const float r = (odd ? other - hv[c][i] : hv[c][i] + other) * 0.17677669529663687f;   // 1 / sqrt(32)
        hv[c][i] = __bfloat162float(__float2bfloat16(r));
        if (on) amax = fmaxf(amax, fabsf(hv[c][i]));
      }
    }
  }
  amax = block_reduce<true>(amax, red);
  if (p.q && p.qfmt == 2) {
    const float g = amax / (6.f * 448.f);
    if (threadIdx.x == 0) p.scale[m] = g;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * nthr;
      if (ch >= nchunk) continue;
      fp4_store_chunk(hv[c], g, ch, m, p.M_pad, p.q, p.q_sf, p.sf_m_tiles);
    }
  } else if (p.q) {
    const float qmax = p.qfmt == 1 ? 448.f : 127.f;
    const float inv = amax > 0.f ? qmax / amax : 0.f;
    if (threadIdx.x == 0 && !sp) p.scale[m] = amax / qmax;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      const int ch = threadIdx.x + c * nthr;
      if (ch >= nchunk) continue;
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = quant4(hv[c][i * 4], hv[c][i * 4 + 1], hv[c][i * 4 + 2], hv[c][i * 4 + 3], inv, p.qfmt);
      const int kb = ch >> 3, cc = ch & 7;
      const size_t off = (static_cast<size_t>(kb) * p.M_pad + m) * 128 + (((cc ^ (m & 7)) & 7) << 4);
      if (sp) {
        for (int peer = 0; peer < p.tp_nranks; ++peer)
          *reinterpret_cast<uint4*>(p.sp_q[peer] + off) = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
        *reinterpret_cast<uint4*>(p.q + off) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    if (sp) {
      if (threadIdx.x == 0)
        for (int peer = 0; peer < p.tp_nranks; ++peer) p.sp_scale[peer][m] = amax / qmax;
      // the row is on every rank once these stores are visible; the CTA that completes the 128-row
      // tile raises its arrival flag everywhere
      __syncthreads();
      if (threadIdx.x == 0) {
        __threadfence_system();
        const int tile = m >> 7;
        const int rows_in_tile = min(128, p.M - (tile << 7));
        const uint32_t old = atomicAdd(p.sp_counter + tile, 1u);
        if (old == static_cast<uint32_t>(rows_in_tile - 1)) {
          p.sp_counter[tile] = 0u;
          __threadfence_system();
          const uint32_t seq = *p.tp_seq_base + static_cast<uint32_t>(p.tp_site) + 1u;
          for (int peer = 0; peer < p.tp_nranks; ++peer)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.sp_flags[peer] + (seq & 1u) * 64u + tile), "r"(seq) : "memory");
        }
      }
    }
  }
}

}  // namespace saber
