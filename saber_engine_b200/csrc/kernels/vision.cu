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
// one head (16 per warp, the m16n8k16 tile).  Keys and values stream through a double-buffered
// shared-memory ring, 64 rows at a time, by 16-byte asynchronous copies (rows past the image are
// zero filled); both stay row-major -- row strides of 176 and 144 bytes put the eight rows of an
// 8 x 8 matrix load on eight different 16-byte bank groups -- and reach the MMA as ldmatrix
// fragments (values through the transposing form).  S = Q K^T and O += P V run on mma.sync with
// fp32 accumulators; the softmax is the running-maximum form in the base-2 domain.
constexpr int kKT = 64, kKStride = 88, kVStride = 72;

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
__device__ __forceinline__ void vis_ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void vis_ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void vis_ldsm_x2_t(uint32_t addr, uint32_t (&r)[2]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
               : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
// 16-byte asynchronous copy; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__global__ void __launch_bounds__(kVisThreads, 4) vis_attn_kernel(const VisAttnParams p) {
  __shared__ __align__(16) __nv_bfloat16 k_s[2][kKT][kKStride];
  __shared__ __align__(16) __nv_bfloat16 v_s[2][kKT][kVStride];
  pdl_wait();
  const int4 blk = p.blocks[blockIdx.x];
  const int seq0 = blk.x, len = blk.y, q0 = blk.z;
  const int h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // the padding columns (head dim 72 -> 80) of the key tiles are never written again
  for (int i = threadIdx.x; i < 2 * kKT * 8; i += kVisThreads)
    k_s[i >> 9][(i >> 3) & (kKT - 1)][kHd + (i & 7)] = __float2bfloat16(0.f);
  const __nv_bfloat16* kbase = p.qkv + static_cast<size_t>(seq0) * p.ldq + p.width + h * kHd;
  auto issue = [&](int tile, int buf) {
    const int k0 = tile * kKT;
    for (int i = threadIdx.x; i < kKT * 9; i += kVisThreads) {
      const int j = i / 9, c = i - j * 9;               // key row of the tile, 8-value chunk of the head
      const bool in = k0 + j < len;
      const __nv_bfloat16* kp = kbase + static_cast<size_t>(in ? k0 + j : 0) * p.ldq + c * 8;
      cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(&k_s[buf][j][c * 8])), kp, in ? 16 : 0);
      cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(&v_s[buf][j][c * 8])), kp + p.width, in ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(0, 0);
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
  const int ntiles = (len + kKT - 1) / kKT;
  // ldmatrix lane addressing: keys (lane & 7) + 8 * (lane >> 4) and column half (lane >> 3) & 1 for
  // the key operand; keys (lane & 7) + 8 * ((lane >> 3) & 1) and dim block (lane >> 4) for values
  const int kr = (lane & 7) + (lane >> 4) * 8, kc = ((lane >> 3) & 1) * 8;
  const int vr = (lane & 7) + ((lane >> 3) & 1) * 8, vc = (lane >> 4) * 8;
  for (int it = 0; it < ntiles; ++it) {
    const int buf = it & 1;
    if (it + 1 < ntiles) {
      issue(it + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int valid = min(kKT, len - it * kKT);
    const uint32_t kb = static_cast<uint32_t>(__cvta_generic_to_shared(&k_s[buf][0][0]));
    const uint32_t vb = static_cast<uint32_t>(__cvta_generic_to_shared(&v_s[buf][0][0]));
    float s[8][4];
#pragma unroll
    for (int np = 0; np < 4; ++np) {                    // pairs of 8-key score tiles
      s[2 * np][0] = s[2 * np][1] = s[2 * np][2] = s[2 * np][3] = 0.f;
      s[2 * np + 1][0] = s[2 * np + 1][1] = s[2 * np + 1][2] = s[2 * np + 1][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 5; ++ks) {
        uint32_t b[4];
        vis_ldsm_x4(kb + static_cast<uint32_t>(((np * 16 + kr) * kKStride + ks * 16 + kc) * 2), b);
        mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
      }
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
      const uint32_t vrow = vb + static_cast<uint32_t>(((kk * 16 + vr) * kVStride + vc) * 2);
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {                  // dim blocks 2jp and 2jp + 1
        uint32_t b[4];
        vis_ldsm_x4_t(vrow + jp * 32, b);
        mma_bf16(o[2 * jp], a, b[0], b[1]);
        mma_bf16(o[2 * jp + 1], a, b[2], b[3]);
      }
      uint32_t b2[2];                                   // dim block 8 (lanes 16-31 repeat the addresses of 0-15)
      vis_ldsm_x2_t(vb + static_cast<uint32_t>(((kk * 16 + vr) * kVStride + 64) * 2), b2);
      mma_bf16(o[8], a, b2[0], b2[1]);
    }
    __syncthreads();                                    // this buffer is refilled by the next iteration's copies
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
    const int kbk = ch >> 3, chunk = ch & 7;
    if (r0 < len) {
      const int mrow = seq0 + r0;
      *reinterpret_cast<uint32_t*>(p.out_tiled + (static_cast<size_t>(kbk) * p.M_pad + mrow) * 128 +
                                   ((chunk ^ (mrow & 7)) << 4) + 4 * t) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
    }
    if (r1 < len) {
      const int mrow = seq0 + r1;
      *reinterpret_cast<uint32_t*>(p.out_tiled + (static_cast<size_t>(kbk) * p.M_pad + mrow) * 128 +
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
