// The vision tower's own kernels: rows -> bf16 GEMM operand (cast or LayerNorm, optional 4-row
// grouping for the merger), the position-table gather, and non-causal attention with 2-D rotary
// embedding.  The tower's linears (patch embed, qkv, proj, fc1 + GELU, fc2 + residual, merger) run on
// the tcgen05 GEMM in its bf16 mode with bias / activation / residual in the epilogue.
//
// Parity: the reference tower's op list and rounding points (crates/saber-kernels/hip/vision.hip:1-30):
// every linear rounds to bf16 once and the activation / residual work on the rounded value;
// LayerNorm, softmax and rotary arithmetic run in fp32; rotated q and k are rounded to bf16; the
// attention products run on mma.sync (bf16 operands, fp32 accumulators).
#include "vision.h"
#include "launch.cuh"

namespace saber {

constexpr int kVisThreads = 128;
constexpr int kVisMaxChunks = 5;     // 8-value chunks per thread: rows of up to 5120 values

__device__ __forceinline__ float block_sum128(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5;
  __syncthreads();                       // red may still be read from the previous call
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

__global__ void __launch_bounds__(kVisThreads) vis_rows_kernel(const VisRowsParams p) {
  __shared__ float red[4];
  pdl_wait();
  const int m = blockIdx.x;
  const int nch = p.K_pad >> 3;
  float v[kVisMaxChunks][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kVisMaxChunks; ++i) {
    const int c = threadIdx.x + i * kVisThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    if (c < nch && c * 8 < p.K) {
      if (p.x_f32) {
        const float4* s = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + static_cast<size_t>(m) * p.ldx + c * 8);
        const float4 a = s[0], b = s[1];
        v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
        v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
      } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.x) + static_cast<size_t>(m) * p.ldx + c * 8);
        const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(b[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j];
    }
  }
  float mean = 0.f, rstd = 1.f;
  if (p.ln_w != nullptr) {
    mean = block_sum128(sum, red) / static_cast<float>(p.K);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < kVisMaxChunks; ++i) {
      const int c = threadIdx.x + i * kVisThreads;
      if (c < nch && c * 8 < p.K) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; sq += d * d; }
      }
    }
    rstd = rsqrtf(block_sum128(sq, red) / static_cast<float>(p.K) + p.eps);
  }
  const int row_o = m / p.group;
  const int col_base = (m % p.group) * p.K;
#pragma unroll
  for (int i = 0; i < kVisMaxChunks; ++i) {
    const int c = threadIdx.x + i * kVisThreads;
    if (c >= nch) continue;
    uint4 o;
    __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
    const bool in = c * 8 < p.K;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float y = v[i][j];
      if (in && p.ln_w != nullptr) y = (y - mean) * rstd * p.ln_w[c * 8 + j] + p.ln_b[c * 8 + j];
      ob[j] = __float2bfloat16(in ? y : 0.f);
    }
    const int col0 = col_base + c * 8;
    const int kb = col0 >> 6, chunk = (col0 & 63) >> 3;
    *reinterpret_cast<uint4*>(p.tiled + (static_cast<size_t>(kb) * p.M_pad + row_o) * 128 +
                              ((chunk ^ (row_o & 7)) << 4)) = o;
  }
}

__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16(x)); }

__global__ void __launch_bounds__(kVisThreads) vis_pos_add_kernel(const VisPosAddParams p) {
  pdl_wait();
  const int m = blockIdx.x;
  int id[4];
  float w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { id[i] = p.idx[m * 4 + i]; w[i] = rbf(p.wt[m * 4 + i]); }
  for (int k = threadIdx.x; k < p.K; k += kVisThreads) {
    float s = rbf(__bfloat162float(p.table[static_cast<size_t>(id[0]) * p.ldt + k]) * w[0]);
#pragma unroll
    for (int i = 1; i < 4; ++i) s = rbf(s + rbf(__bfloat162float(p.table[static_cast<size_t>(id[i]) * p.ldt + k]) * w[i]));
    __nv_bfloat16* x = p.x + static_cast<size_t>(m) * p.ldx + k;
    *x = __float2bfloat16(__bfloat162float(*x) + s);
  }
}

// ------------------------------------------------------------------------------------ rotary
// In place on the q and k parts of qkv: out[d] = x[d] cos - x[d+36] sin, out[d+36] = x[d+36] cos + x[d] sin
// (fp32 arithmetic, one rounding to bf16).  One CTA per row.
constexpr int kHd = 72, kHalf = 36;

__global__ void __launch_bounds__(kVisThreads) vis_rope_kernel(const VisAttnParams p, int rows) {
  pdl_wait();
  const int m = blockIdx.x;
  if (m >= rows) return;
  __nv_bfloat16* base = const_cast<__nv_bfloat16*>(p.qkv) + static_cast<size_t>(m) * p.ldq;
  const float* cs = p.cos_t + static_cast<size_t>(m) * kHalf;
  const float* sn = p.sin_t + static_cast<size_t>(m) * kHalf;
  const int pairs = 2 * p.heads * kHalf;              // q heads, then k heads
  for (int i = threadIdx.x; i < pairs; i += kVisThreads) {
    const int hd = i / kHalf, d = i - hd * kHalf;     // hd < heads: q head, else k head (k starts at width = heads * 72)
    __nv_bfloat16* x = base + hd * kHd;
    const float x1 = __bfloat162float(x[d]), x2 = __bfloat162float(x[d + kHalf]);
    x[d] = __float2bfloat16(x1 * cs[d] - x2 * sn[d]);
    x[d + kHalf] = __float2bfloat16(x2 * cs[d] + x1 * sn[d]);
  }
}

// ------------------------------------------------------------------------------------ attention
// Non-causal attention inside one image on rotated q / k.  A CTA of four warps owns 64 query rows of
// one head (16 per warp, the m16n8k16 tile); keys and values stream through shared memory 64 rows at
// a time (keys row-major with the head dim padded to 80, values transposed so that two consecutive
// keys of one dim are one 32-bit word); S = Q K^T and O += P V run on mma.sync with fp32
// accumulators, the softmax is the running-maximum form in the base-2 domain.
constexpr int kQRows = 64, kKT = 64, kKStride = 88, kVStride = 72;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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

__global__ void __launch_bounds__(kVisThreads) vis_attn_kernel(const VisAttnParams p) {
  __shared__ __align__(16) __nv_bfloat16 k_s[kKT][kKStride];
  __shared__ __align__(16) __nv_bfloat16 vt_s[kHd][kVStride];
  pdl_wait();
  const int4 blk = p.blocks[blockIdx.x];
  const int seq0 = blk.x, len = blk.y, q0 = blk.z;
  const int h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // the padding columns of the key tile are never written again
  for (int i = threadIdx.x; i < kKT * 8; i += kVisThreads) k_s[i >> 3][kHd + (i & 7)] = __float2bfloat16(0.f);
  // this warp's query fragments, straight from global memory (rows past the image read row 0, never stored)
  uint32_t qf[5][4];
  {
    const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
    const __nv_bfloat16* qa = p.qkv + static_cast<size_t>(seq0 + (r0 < len ? r0 : 0)) * p.ldq + h * kHd;
    const __nv_bfloat16* qb = p.qkv + static_cast<size_t>(seq0 + (r1 < len ? r1 : 0)) * p.ldq + h * kHd;
#pragma unroll
    for (int ks = 0; ks < 5; ++ks) {
      const int c0 = ks * 16 + 2 * t, c1 = c0 + 8;
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(qa + c0);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(qb + c0);
      qf[ks][2] = c1 < kHd ? *reinterpret_cast<const uint32_t*>(qa + c1) : 0u;
      qf[ks][3] = c1 < kHd ? *reinterpret_cast<const uint32_t*>(qb + c1) : 0u;
    }
  }
  const float qs = p.scale * 1.4426950408889634f;
  float o[9][4];
#pragma unroll
  for (int j = 0; j < 9; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  for (int k0 = 0; k0 < len; k0 += kKT) {
    __syncthreads();                                    // the previous tile has been consumed
    for (int i = threadIdx.x; i < kKT * 9; i += kVisThreads) {
      const int j = i / 9, c = i - j * 9;               // key row of the tile, 8-value chunk of the head
      uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
      if (k0 + j < len) {
        const __nv_bfloat16* kp = p.qkv + static_cast<size_t>(seq0 + k0 + j) * p.ldq + p.width + h * kHd + c * 8;
        kv = *reinterpret_cast<const uint4*>(kp);
        vv = *reinterpret_cast<const uint4*>(kp + p.width);
      }
      *reinterpret_cast<uint4*>(&k_s[j][c * 8]) = kv;
      const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(&vv);
#pragma unroll
      for (int e = 0; e < 8; ++e) vt_s[c * 8 + e][j] = vb[e];
    }
    __syncthreads();
    const int valid = min(kKT, len - k0);
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const __nv_bfloat16* kr = &k_s[nt * 8 + g][2 * t];
#pragma unroll
      for (int ks = 0; ks < 5; ++ks)
        mma_bf16(s[nt], qf[ks], *reinterpret_cast<const uint32_t*>(kr + ks * 16),
                 *reinterpret_cast<const uint32_t*>(kr + ks * 16 + 8));
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = nt * 8 + 2 * t + (c & 1);
        s[nt][c] = key < valid ? s[nt][c] * qs : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);      // finite: key 0 of the tile is valid
    const float c0 = exp2f(m0 - n0), c1 = exp2f(m1 - n1);      // 0 on the first tile
    m0 = n0; m1 = n1;
    l0 *= c0; l1 *= c1;
#pragma unroll
    for (int j = 0; j < 9; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - n0); s[nt][1] = exp2f(s[nt][1] - n0);
      s[nt][2] = exp2f(s[nt][2] - n1); s[nt][3] = exp2f(s[nt][3] - n1);
      l0 += s[nt][0] + s[nt][1];
      l1 += s[nt][2] + s[nt][3];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {                    // 16 keys per step: score tiles 2kk and 2kk + 1
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < 9; ++j) {
        const __nv_bfloat16* vr = &vt_s[j * 8 + g][kk * 16 + 2 * t];
        mma_bf16(o[j], a, *reinterpret_cast<const uint32_t*>(vr), *reinterpret_cast<const uint32_t*>(vr + 8));
      }
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < 9; ++j) {
    const int ch = h * 9 + j;                           // 16-byte chunk of the output row (72 = 9 chunks per head)
    const int kb = ch >> 3, chunk = ch & 7;
    if (r0 < len) {
      const int mrow = seq0 + r0;
      *reinterpret_cast<uint32_t*>(p.out_tiled + (static_cast<size_t>(kb) * p.M_pad + mrow) * 128 +
                                   ((chunk ^ (mrow & 7)) << 4) + 4 * t) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
    }
    if (r1 < len) {
      const int mrow = seq0 + r1;
      *reinterpret_cast<uint32_t*>(p.out_tiled + (static_cast<size_t>(kb) * p.M_pad + mrow) * 128 +
                                   ((chunk ^ (mrow & 7)) << 4) + 4 * t) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
    }
  }
}

}  // namespace saber

extern "C" int saber_vis_rows_launch(const saber::VisRowsParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->M <= 0) return 0;
  if ((p->K & 7) || (p->K_pad & 7) || p->K_pad < p->K || p->K_pad > kVisMaxChunks * kVisThreads * 8 ||
      (p->group != 1 && p->group != 4) || (p->group == 1 && (p->K_pad & 63)) ||
      (p->group > 1 && ((p->K & 63) || p->K_pad != p->K)) || (p->ldx & 7) || (p->M + p->group - 1) / p->group > p->M_pad)
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(saber::launch(vis_rows_kernel, dim3(p->M), dim3(kVisThreads), 0, stream, 0, *p));
}

extern "C" int saber_vis_pos_add_launch(const saber::VisPosAddParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->M <= 0) return 0;
  return static_cast<int>(saber::launch(vis_pos_add_kernel, dim3(p->M), dim3(kVisThreads), 0, stream, 0, *p));
}

extern "C" int saber_vis_attn_launch(const saber::VisAttnParams* p, int n_blocks, cudaStream_t stream) {
  using namespace saber;
  if (n_blocks <= 0) return 0;
  if ((p->width & 7) || p->heads * kHd != p->width || (p->ldq & 7)) return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(saber::launch(vis_attn_kernel, dim3(n_blocks, p->heads), dim3(kVisThreads), 0, stream, 0, *p));
}

extern "C" int saber_vis_rope_launch(const saber::VisAttnParams* p, int rows, cudaStream_t stream) {
  using namespace saber;
  if (rows <= 0) return 0;
  if (p->heads * kHd != p->width) return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(saber::launch(vis_rope_kernel, dim3(rows), dim3(kVisThreads), 0, stream, 0, *p, rows));
}
