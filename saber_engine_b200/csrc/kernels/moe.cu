// Mixture-of-experts routing for sm_100a: softmax over the router logits, top-k (lower id wins
// ties), optional renormalisation, then an expert-major placement of the routes into 16-row-padded
// segments plus the tile table the grouped GEMM walks, and the weighted combine.
//
// Parity: crates/saber-kernels/hip/moe_route.hip:1-30 (softmax fp32 -> top-10, lower id wins ties ->
// renorm -> expert-major sort into 16-row blocks + tile tables; only this rank's experts are placed)
// and moe_combine_bf16 (sum of w * Y in top-k order + shared expert).  Three launches here:
// topk (warp per token), plan (one block: scan, tile table), place (thread per route).
#include "launch.cuh"
#include "moe.h"
#include "gemm_i8.h"
#include <math.h>
#include <cuda_fp8.h>

namespace saber {

constexpr int kMoeTpMaxTiles = kTpMaxTiles;   // same flag regions as the row-parallel GEMM

__device__ __forceinline__ float e_safe(float x, float mx) { return x == -INFINITY ? 0.f : __expf(x - mx); }

// grid = ceil(M / 8), block 256: one warp per token.
__global__ void __launch_bounds__(256) moe_topk_kernel(const MoeRouteParams p) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * 8 + warp;
  if (m >= p.M) return;
  constexpr int kPerLane = 32;                 // up to 1024 experts
  float v[kPerLane];
  const int per = (p.E + 31) / 32;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < p.E ? __bfloat162float(p.logits[static_cast<size_t>(m) * p.ld + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int i = 0; i < per; ++i) {
    v[i] = e_safe(v[i], mx);
    sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float picked_w[kMoeMaxTopK];
  int picked_e[kMoeMaxTopK];
  float wsum = 0.f;
  for (int k = 0; k < p.top_k; ++k) {
    float bv = -1.f;
    int be = p.E;
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > bv) { bv = v[i]; be = e; }     // ascending e per lane: the lower id wins ties
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    picked_w[k] = bv * inv;
    picked_e[k] = be;
    wsum += picked_w[k];
    if ((be & 31) == lane) v[be >> 5] = -1.f;   // taken
  }
  if (lane == 0) {
    const float rn = p.norm_topk ? 1.f / wsum : 1.f;
    for (int k = 0; k < p.top_k; ++k) {
      p.topk_id[m * p.top_k + k] = picked_e[k];
      p.topk_w[m * p.top_k + k] = picked_w[k] * rn;
      const int le = picked_e[k] - p.e_lo;
      if (le >= 0 && le < p.e_n) atomicAdd(p.counts + le, 1);
    }
  }
}

// One block of 1024 threads (one per local expert): exclusive scans of the padded row counts and of
// the tile counts (warp shuffles, then the 32 warp totals), every thread writes its expert's tiles;
// cursors and counts are cleared for the placement pass and for the next step's routing.
__device__ __forceinline__ int block_excl_scan_1024(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();                       // warp_tot may still be read by the previous scan
  if (lane == 31) warp_tot[w] = inc;
  __syncthreads();
  int base = 0, tot = 0;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    const int x = warp_tot[k];
    if (k < w) base += x;
    tot += x;
  }
  total = tot;
  return base + inc - v;
}

__global__ void __launch_bounds__(1024) moe_plan_kernel(const MoeRouteParams p) {
  pdl_wait();
  __shared__ int warp_tot[32];
  const int t = threadIdx.x;
  int c = 0;
  if (t < p.e_n) {
    c = p.counts[t];
    p.counts[t] = 0;                     // the next routing pass accumulates from zero
    p.cursors[t] = 0;
  }
  int rows_total, tiles_total;
  const int off = block_excl_scan_1024((c + 15) & ~15, warp_tot, rows_total);
  const int toff = block_excl_scan_1024((c + p.nt - 1) / p.nt, warp_tot, tiles_total);
  if (t < p.e_n) {
    p.offsets[t] = off;
    int i = toff;
    for (int r = 0; r < c; r += p.nt) p.tiles[i++] = make_int4(t, off + r, min(p.nt, c - r), 0);
  }
  if (t == 0) {
    p.offsets[p.e_n] = rows_total;
    p.ntiles[0] = tiles_total;
    p.ntiles[1] = rows_total;
  }
  for (int i = t; i < p.rows_cap; i += blockDim.x) p.src_row[i] = -1;
}

// thread per route: claim a row in the expert's segment.
__global__ void moe_place_kernel(const MoeRouteParams p) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.M * p.top_k) return;
  const int le = p.topk_id[i] - p.e_lo;
  if (le < 0 || le >= p.e_n) { p.slot_of[i] = -1; return; }
  const int pos = p.offsets[le] + atomicAdd(p.cursors + le, 1);
  p.slot_of[i] = pos;
  p.src_row[pos] = i / p.top_k;
}

// block = K / 16 threads (one 16-byte chunk each); the CTAs stride over the LIVE rows (a device-side
// count): the grid is static (graph capture) but small, instead of one CTA per row of the worst case.
// to_fp8: the sorted rows feed MXFP4 experts, whose GEMM multiplies fp8 x fp8: an int8 value q (row scale s)
// leaves as e4m3(q * 448 / 127) with row scale s * 127 / 448 (round to nearest even, saturating).
__global__ void moe_gather_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, int M_pad,
                                  const int32_t* __restrict__ src_row, const int32_t* __restrict__ ntiles,
                                  int8_t* __restrict__ q_out, float* __restrict__ scale_out, int M_pad_out, int to_fp8) {
  pdl_trigger();
  pdl_wait();
  const int live = ntiles[1];
  const int kb = threadIdx.x >> 3, c = threadIdx.x & 7;       // k-block, logical 16-byte chunk
  for (int r = blockIdx.x; r < live; r += gridDim.x) {
    const int m = src_row[r];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m >= 0)
      v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(kb) * M_pad + m) * 128 + ((c ^ (m & 7)) << 4));
    if (to_fp8) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float f0 = static_cast<float>(static_cast<int8_t>(w[i] & 0xFFu)) * (448.f / 127.f);
        const float f1 = static_cast<float>(static_cast<int8_t>((w[i] >> 8) & 0xFFu)) * (448.f / 127.f);
        const float f2 = static_cast<float>(static_cast<int8_t>((w[i] >> 16) & 0xFFu)) * (448.f / 127.f);
        const float f3 = static_cast<float>(static_cast<int8_t>(w[i] >> 24)) * (448.f / 127.f);
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f2, f3), __NV_SATFINITE, __NV_E4M3);
        w[i] = lo | (hi << 16);
      }
    }
    *reinterpret_cast<uint4*>(q_out + (static_cast<size_t>(kb) * M_pad_out + r) * 128 + ((c ^ (r & 7)) << 4)) = v;
    if (threadIdx.x == 0) scale_out[r] = m >= 0 ? scale[m] * (to_fp8 ? 127.f / 448.f : 1.f) : 0.f;
  }
}

// grid = (ceil(H / 256), ceil(M / nt)), block 256: lane -> 8 columns, warp -> rows w, w + 8, ...
// out[m] = sum_k w[m,k] * y[slot_of[m,k]] (+ sigmoid(g[m]) * shared[m]), routes in top-k order.
__global__ void __launch_bounds__(256) moe_combine_kernel(const MoeCombineParams p) {
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 256 + lane * 8;
  const int m0 = blockIdx.y * p.nt;
  const bool tp = p.tp_nranks > 1;
  uint32_t seq = 0, par = 0;
  if (tp) {
    seq = *p.tp_seq_base + static_cast<uint32_t>(p.tp_site) + 1u;
    par = seq & 1u;
  }
  if (n < p.H) {
    for (int r = warp; r < p.nt; r += 8) {
      const int m = m0 + r;
      if (m >= p.M) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < p.top_k; ++k) {
        const int slot = p.slot_of[m * p.top_k + k];
        if (slot < 0) continue;
        const float w = p.topk_w[m * p.top_k + k];
        const uint4 raw = *reinterpret_cast<const uint4*>(p.y + static_cast<size_t>(slot) * p.H + n);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += w * f.x;
          acc[2 * i + 1] += w * f.y;
        }
      }
      if (p.shared) {
        float gs = 1.f;
        if (p.shared_gate) gs = 1.f / (1.f + __expf(-__bfloat162float(p.shared_gate[static_cast<size_t>(m) * p.ldg])));
        const uint4 raw = *reinterpret_cast<const uint4*>(p.shared + static_cast<size_t>(m) * p.H + n);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += gs * f.x;
          acc[2 * i + 1] += gs * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      if (tp) {
        const size_t off = ((static_cast<size_t>(par) * p.tp_nranks + p.tp_rank) * p.tp_rows + m) * p.tp_ld + n;
        for (int peer = 0; peer < p.tp_nranks; ++peer)
          *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.tp_recv[peer]) + off) = o;
      } else {
        *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(m) * p.H + n) = o;
      }
    }
  }
  if (tp) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.tp_nranks) {
      const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
      uint32_t* f = p.tp_flags[threadIdx.x] + (static_cast<size_t>(par) * p.tp_nranks + p.tp_rank) * kMoeTpMaxTiles + tile_id;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
    }
  }
}

}  // namespace saber

extern "C" int saber_moe_route_launch(const saber::MoeRouteParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->E > 1024 || p->e_n > 1024 || p->top_k > kMoeMaxTopK || p->top_k < 1 || p->nt < 16 || (p->nt & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(moe_topk_kernel, dim3((p->M + 7) / 8), dim3(256), 0, stream, 0, *p);
  saber::launch(moe_plan_kernel, dim3(1), dim3(1024), 0, stream, 0, *p);
  saber::launch(moe_place_kernel, dim3((p->M * p->top_k + 255) / 256), dim3(256), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_moe_gather_launch(const int8_t* q, const float* scale, int M_pad, const int32_t* src_row,
                                       const int32_t* ntiles, int8_t* q_out, float* scale_out, int rows_cap,
                                       int M_pad_out, int K, int to_fp8, cudaStream_t stream) {
  if ((K & 127) || K / 16 > 1024 || rows_cap > M_pad_out) return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(saber::moe_gather_kernel, dim3(rows_cap < 1184 ? rows_cap : 1184), dim3(K / 16), 0, stream, 0, q, scale, M_pad, src_row, ntiles, q_out, scale_out, M_pad_out, to_fp8);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_moe_combine_launch(const saber::MoeCombineParams* p, cudaStream_t stream) {
  if ((p->H & 7) || p->nt < 1) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid((p->H + 255) / 256, (p->M + p->nt - 1) / p->nt);
  if (p->tp_nranks > 1 &&
      (p->tp_nranks > 8 || static_cast<int>(grid.x * grid.y) > saber::kMoeTpMaxTiles || p->M > p->tp_rows || (p->tp_ld & 7)))
    return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(saber::moe_combine_kernel, dim3(grid), dim3(256), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}
