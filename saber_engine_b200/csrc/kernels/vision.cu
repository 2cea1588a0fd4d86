// The vision tower's own kernels: rows -> bf16 GEMM operand (cast or LayerNorm, optional 4-row
// grouping for the merger), the position-table gather, and non-causal attention with 2-D rotary
// embedding.  The tower's linears (patch embed, qkv, proj, fc1 + GELU, fc2 + residual, merger) run on
// the tcgen05 GEMM in its bf16 mode with bias / activation / residual in the epilogue.
//
// Parity: the reference tower's op list and rounding points (crates/saber-kernels/hip/vision.hip:1-30):
// every linear rounds to bf16 once and the activation / residual work on the rounded value;
// LayerNorm, softmax and rotary arithmetic run in fp32; rotated q and k are rounded to bf16.
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

// ------------------------------------------------------------------------------------ attention
// One thread per query row (128 rows per CTA), one head per blockIdx.y.  Keys and values of the
// image stream through shared memory 32 rows at a time as fp32 (keys rotated on the way in); a
// thread scores eight keys, folds their maximum into its running softmax and accumulates.
constexpr int kHd = 72, kHalf = 36, kKeys = 32;

__global__ void __launch_bounds__(kVisThreads) vis_attn_kernel(const VisAttnParams p) {
  __shared__ __align__(16) float k_s[kKeys][kHd];
  __shared__ __align__(16) float v_s[kKeys][kHd];
  pdl_wait();
  const int4 blk = p.blocks[blockIdx.x];
  const int seq0 = blk.x, len = blk.y, qrel = blk.z + threadIdx.x;
  const int h = blockIdx.y;
  const bool live = qrel < len;
  const int qrow = seq0 + (live ? qrel : 0);
  const float qs = p.scale * 1.4426950408889634f;       // scores in the base-2 domain
  float q[kHd], acc[kHd];
  {
    const __nv_bfloat16* qp = p.qkv + static_cast<size_t>(qrow) * p.ldq + h * kHd;
    const float* cs = p.cos_t + static_cast<size_t>(qrow) * kHalf;
    const float* sn = p.sin_t + static_cast<size_t>(qrow) * kHalf;
#pragma unroll
    for (int d = 0; d < kHalf; ++d) {
      const float x1 = __bfloat162float(qp[d]), x2 = __bfloat162float(qp[d + kHalf]);
      q[d] = rbf(x1 * cs[d] - x2 * sn[d]) * qs;
      q[d + kHalf] = rbf(x2 * cs[d] + x1 * sn[d]) * qs;
    }
#pragma unroll
    for (int d = 0; d < kHd; ++d) acc[d] = 0.f;
  }
  float mrun = -INFINITY, lrun = 0.f;
  for (int k0 = 0; k0 < len; k0 += kKeys) {
    __syncthreads();
    {   // stage 32 keys (rotated) and values: thread = (key, quarter of the 36 rotary pairs)
      const int j = threadIdx.x >> 2, part = threadIdx.x & 3;
      const bool kin = k0 + j < len;
      const int krow = seq0 + (kin ? k0 + j : 0);
      const __nv_bfloat16* kp = p.qkv + static_cast<size_t>(krow) * p.ldq + p.width + h * kHd;
      const __nv_bfloat16* vp = kp + p.width;
      const float* cs = p.cos_t + static_cast<size_t>(krow) * kHalf;
      const float* sn = p.sin_t + static_cast<size_t>(krow) * kHalf;
#pragma unroll
      for (int i = 0; i < 9; ++i) {
        const int d = part * 9 + i;
        const float x1 = __bfloat162float(kp[d]), x2 = __bfloat162float(kp[d + kHalf]);
        k_s[j][d] = kin ? rbf(x1 * cs[d] - x2 * sn[d]) : 0.f;
        k_s[j][d + kHalf] = kin ? rbf(x2 * cs[d] + x1 * sn[d]) : 0.f;
        v_s[j][d] = kin ? __bfloat162float(vp[d]) : 0.f;
        v_s[j][d + kHalf] = kin ? __bfloat162float(vp[d + kHalf]) : 0.f;
      }
    }
    __syncthreads();
    const int valid = min(kKeys, len - k0);
#pragma unroll 1
    for (int jb = 0; jb < kKeys; jb += 8) {
      if (jb >= valid) break;
      float s[8];
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4* kr = reinterpret_cast<const float4*>(k_s[jb + j]);
        float a = 0.f;
#pragma unroll
        for (int d4 = 0; d4 < kHd / 4; ++d4) {
          const float4 kv = kr[d4];
          a = fmaf(q[4 * d4], kv.x, a);
          a = fmaf(q[4 * d4 + 1], kv.y, a);
          a = fmaf(q[4 * d4 + 2], kv.z, a);
          a = fmaf(q[4 * d4 + 3], kv.w, a);
        }
        s[j] = (jb + j < valid) ? a : -INFINITY;
        tmax = fmaxf(tmax, s[j]);
      }
      const float mnew = fmaxf(mrun, tmax);          // finite: key jb is valid
      const float corr = exp2f(mrun - mnew);         // 0 on the first group (mrun = -inf)
      mrun = mnew;
      lrun *= corr;
#pragma unroll
      for (int d = 0; d < kHd; ++d) acc[d] *= corr;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float pj = exp2f(s[j] - mnew);
        lrun += pj;
        const float4* vr = reinterpret_cast<const float4*>(v_s[jb + j]);
#pragma unroll
        for (int d4 = 0; d4 < kHd / 4; ++d4) {
          const float4 vv = vr[d4];
          acc[4 * d4] = fmaf(pj, vv.x, acc[4 * d4]);
          acc[4 * d4 + 1] = fmaf(pj, vv.y, acc[4 * d4 + 1]);
          acc[4 * d4 + 2] = fmaf(pj, vv.z, acc[4 * d4 + 2]);
          acc[4 * d4 + 3] = fmaf(pj, vv.w, acc[4 * d4 + 3]);
        }
      }
    }
  }
  if (live) {
    const float inv = 1.f / lrun;
    const int mrow = seq0 + qrel;
#pragma unroll
    for (int c = 0; c < kHd / 8; ++c) {
      uint4 o;
      __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) ob[j] = __float2bfloat16(acc[c * 8 + j] * inv);
      const int col0 = h * kHd + c * 8;
      const int kb = col0 >> 6, chunk = (col0 & 63) >> 3;
      *reinterpret_cast<uint4*>(p.out_tiled + (static_cast<size_t>(kb) * p.M_pad + mrow) * 128 +
                                ((chunk ^ (mrow & 7)) << 4)) = o;
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
