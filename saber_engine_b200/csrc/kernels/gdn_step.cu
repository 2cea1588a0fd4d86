// One launch per Gated DeltaNet layer in a decode step: causal conv + SiLU + L2 norm, the gated
// delta-rule recurrence (base + stash + replay), the per-head gated RMSNorm and the per-token int8
// quantisation of the out_proj operand.
//
// Parity: the reference folds the same chain -- conv and recurrence in one launch
// (crates/saber-kernels/hip/sgdn_rec.h:1-30, saber_gdn_fused_update), the gated norm + quantisation
// ticketed onto it (saber_gdn_fnq.hip:1-30).  The arithmetic is that of the separate kernels of
// gdn.cu and rowops.cu, operation for operation, so both paths produce the same bytes.
//
// CTA = (value head, sequence), 256 threads: thread = (state row v, half of the key dim), 64 state
// values each as packed fp32 pairs.  Phases:
//   0  conv: the CTA computes the q and k channels of its key head and the v channels of its value
//      head for this step's rows (a key head's q / k are recomputed by each of its value heads:
//      a few hundred FMAs), straight into the staging buffers of the recurrence.  The conv window
//      lives in two buffers per slot that alternate every step (readers of a step never meet its
//      writer); a per-slot word says which one is current and is flipped by the sequence's last CTA.
//   1  recurrence: replay of the rows accepted last step, committed state stored, then this step's
//      rows on the register copy; rows leave a stash (k, v, g, beta).
//   2  gated RMSNorm of the head's outputs -> bf16 rows in a scratch buffer and the head's row
//      maxima; the LAST head CTA of a sequence (a ticket) quantises the sequence's rows.
#include "gdn.h"
#include "launch.cuh"
#include "rowops_body.cuh"
#include <cuda_bf16.h>

namespace saber {

__device__ __forceinline__ float gs_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gs_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

typedef unsigned long long gs_f32x2;
__device__ __forceinline__ gs_f32x2 gs_pack2(float lo, float hi) {
  gs_f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float gs_sum2(gs_f32x2 v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo + hi;
}
__device__ __forceinline__ gs_f32x2 gs_fma2(gs_f32x2 a, gs_f32x2 b, gs_f32x2 c) {
  gs_f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ gs_f32x2 gs_mul2(gs_f32x2 a, gs_f32x2 b) {
  gs_f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

constexpr int kStepRows = 16;            // rows of one sequence in a decode step (and replayed rows)
constexpr int kStepThreads = 256;

__global__ void __launch_bounds__(kStepThreads, 2) gdn_step_kernel(const GdnStepParams p) {
  pdl_trigger();   // the GEMM that follows streams its first weight tiles on the SMs this grid's last round leaves idle
  pdl_wait();
  constexpr int KP = 64 + 4;             // padded half stride in shared memory (bank spread)
  __shared__ __align__(16) float ks[kStepRows][2 * KP];
  __shared__ __align__(16) float qs[kStepRows][2 * KP];
  __shared__ __align__(16) float vsm[kStepRows][128];
  __shared__ __align__(16) float ksr[kStepRows][2 * KP];
  __shared__ __align__(16) float vsr[kStepRows][128];      // replayed v rows, later the head's outputs
  __shared__ float gsm[kStepRows], bsm[kStepRows], gsr[kStepRows], bsr[kStepRows];
  __shared__ float red[2][kStepRows][4];
  __shared__ uint32_t last_s;
  const int b = blockIdx.y;
  const int slot = p.slots[b];
  if (slot < 0) return;
  const int h = blockIdx.x;
  const int hk = h / (p.HV / p.HK);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = p.cu_rows[b];
  const int n = min(p.cu_rows[b + 1] - row0, kStepRows);
  const int shift = min(p.shift[b], min(p.stash_rows, kStepRows));
  __nv_bfloat16* hist_slot = p.hist + static_cast<size_t>(slot) * (2 * p.hist_rows + 1) * p.C;
  int* hist_word = reinterpret_cast<int*>(hist_slot + static_cast<size_t>(2 * p.hist_rows) * p.C);
  const int par = *hist_word & 1;                         // which conv window is current
  const __nv_bfloat16* hist_rd = hist_slot + static_cast<size_t>(par) * p.hist_rows * p.C;
  __nv_bfloat16* hist_wr = hist_slot + static_cast<size_t>(par ^ 1) * p.hist_rows * p.C;

  // ---- the recurrence's global reads go out first: replayed rows and the state
  const int vloc = tid >> 1, kh = tid & 1;
  float* sp = p.state + ((static_cast<size_t>(slot) * p.HV + h) * 128 + vloc) * 128 + kh * 64;
  constexpr int kStashStride = 128 + 128 + 4;             // k | v | g, beta (one v slice: the whole head)
  float* stash = p.stash + ((static_cast<size_t>(slot) * p.stash_rows) * p.HV + h) * kStashStride;
  const size_t stash_row = static_cast<size_t>(p.HV) * kStashStride;
  for (int idx = tid; idx < shift * 32; idx += kStepThreads) {
    const int r = idx >> 5, i = (idx & 31) * 4;
    const float4 t4 = *reinterpret_cast<const float4*>(stash + static_cast<size_t>(r) * stash_row + i);
    *reinterpret_cast<float4*>(&ksr[r][(i >> 6) * KP + (i & 63)]) = t4;
  }
  for (int idx = tid; idx < shift * 32; idx += kStepThreads) {
    const int r = idx >> 5, i = (idx & 31) * 4;
    *reinterpret_cast<float4*>(&vsr[r][i]) = *reinterpret_cast<const float4*>(stash + static_cast<size_t>(r) * stash_row + 128 + i);
  }
  if (tid < shift) {
    gsr[tid] = stash[static_cast<size_t>(tid) * stash_row + 256];
    bsr[tid] = stash[static_cast<size_t>(tid) * stash_row + 257];
  }
  // the state (this thread's 256 bytes) starts its way from memory now and is read after the conv
  asm volatile("prefetch.global.L2 [%0];" ::"l"(sp));
  asm volatile("prefetch.global.L2 [%0];" ::"l"(sp + 32));

  // ---- phase 0: conv + SiLU (+ L2 norm for q, k); threads 0-127 own q channel t and v channel t,
  // threads 128-255 own k channel t - 128
  {
    const int c = tid & 127;
    const bool is_k = tid >= 128;
    const int gch_qk = (is_k ? p.n_q : 0) + hk * 128 + c;
    const int gch_v = p.n_q + p.n_k + h * 128 + c;
    // the key head's q / k window is rewritten by ONE of its value heads, v by its own head
    const bool qk_writer = (h % (p.HV / p.HK)) == 0;
    float y[kStepRows];
    auto conv_channel = [&](int gch, bool writer) {
      const __nv_bfloat16* hp = hist_rd + gch;
      float b0 = __bfloat162float(hp[static_cast<size_t>(shift) * p.C]);
      float b1 = __bfloat162float(hp[static_cast<size_t>(shift + 1) * p.C]);
      float b2 = __bfloat162float(hp[static_cast<size_t>(shift + 2) * p.C]);
      __nv_bfloat16* hw = hist_wr + gch;
      if (writer) {
        hw[0] = __float2bfloat16(b0);
        hw[p.C] = __float2bfloat16(b1);
        hw[2 * static_cast<size_t>(p.C)] = __float2bfloat16(b2);
      }
      const float w0 = p.conv_w[gch * 4 + 0], w1 = p.conv_w[gch * 4 + 1], w2 = p.conv_w[gch * 4 + 2], w3 = p.conv_w[gch * 4 + 3];
#pragma unroll
      for (int r = 0; r < kStepRows; ++r) {
        if (r < n) {
          const __nv_bfloat16 xb = p.x[static_cast<size_t>(row0 + r) * p.ldx + gch];
          const float x = __bfloat162float(xb);
          y[r] = gs_silu(w0 * b0 + w1 * b1 + w2 * b2 + w3 * x);
          b0 = b1; b1 = b2; b2 = x;
          if (writer && r < p.hist_rows - 3) hw[static_cast<size_t>(3 + r) * p.C] = xb;
        }
      }
    };
    conv_channel(gch_qk, qk_writer);
    // L2 norm over the 128 channels of the head, row by row (the reduction order of the conv kernel)
#pragma unroll
    for (int r = 0; r < kStepRows; ++r) {
      if (r < n) {
        float ss = y[r] * y[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[is_k][r][warp & 3] = ss;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kStepRows; ++r) {
      if (r < n) {
        const float ss = red[is_k][r][0] + red[is_k][r][1] + red[is_k][r][2] + red[is_k][r][3];
        float v = y[r] * rsqrtf(ss + 1e-6f);
        if (!is_k) v *= p.q_scale;
        (is_k ? ks : qs)[r][(c >> 6) * KP + (c & 63)] = v;
      }
    }
    if (!is_k) {
      conv_channel(gch_v, true);
#pragma unroll
      for (int r = 0; r < kStepRows; ++r)
        if (r < n) vsm[r][c] = y[r];
    }
  }
  gs_f32x2 S[32];   // this thread's 64 state values as packed pairs
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const ulonglong2 t = reinterpret_cast<const ulonglong2*>(sp)[i];
    S[2 * i] = t.x;
    S[2 * i + 1] = t.y;
  }
  const float neg_a = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[h];
  if (tid < n) {
    const size_t m = static_cast<size_t>(row0 + tid);
    const float bb = __bfloat162float(p.ba[m * p.ldba + h]);
    const float aa = __bfloat162float(p.ba[m * p.ldba + p.HV + h]);
    gsm[tid] = neg_a * gs_softplus(aa + dtb);
    bsm[tid] = 1.f / (1.f + __expf(-bb));
  }
  __syncthreads();

  // ---- phase 1: the recurrence (the arithmetic of gdn_recurrent_kernel, one v slice)
  auto replay = [&](const float* kv, float u, float g) {     // a row whose u is known (the stash keeps u, not v)
    const ulonglong2* kv2 = reinterpret_cast<const ulonglong2*>(kv);
    const float decay = __expf(g);
    const gs_f32x2 dec2 = gs_pack2(decay, decay), u2 = gs_pack2(u, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const ulonglong2 kk = kv2[i];
      S[2 * i] = gs_fma2(u2, kk.x, gs_mul2(S[2 * i], dec2));
      S[2 * i + 1] = gs_fma2(u2, kk.y, gs_mul2(S[2 * i + 1], dec2));
    }
  };
  auto apply = [&](const float* kv, const float* qv, float vval, float g, float beta, bool want_o, float& u_out) -> float {
    const ulonglong2* kv2 = reinterpret_cast<const ulonglong2*>(kv);
    const ulonglong2* qv2 = reinterpret_cast<const ulonglong2*>(qv);
    const float decay = __expf(g);
    const gs_f32x2 dec2 = gs_pack2(decay, decay);
    gs_f32x2 acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const ulonglong2 kk = kv2[i];
      S[2 * i] = gs_mul2(S[2 * i], dec2);
      S[2 * i + 1] = gs_mul2(S[2 * i + 1], dec2);
      acc[(2 * i) & 3] = gs_fma2(S[2 * i], kk.x, acc[(2 * i) & 3]);
      acc[(2 * i + 1) & 3] = gs_fma2(S[2 * i + 1], kk.y, acc[(2 * i + 1) & 3]);
    }
    float dot = (gs_sum2(acc[0]) + gs_sum2(acc[1])) + (gs_sum2(acc[2]) + gs_sum2(acc[3]));
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float u = (vval - dot) * beta;
    u_out = u;
    const gs_f32x2 u2 = gs_pack2(u, u);
    gs_f32x2 oac[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const ulonglong2 kk = kv2[i];
      S[2 * i] = gs_fma2(u2, kk.x, S[2 * i]);
      S[2 * i + 1] = gs_fma2(u2, kk.y, S[2 * i + 1]);
      if (want_o) {
        const ulonglong2 qq = qv2[i];
        oac[(2 * i) & 3] = gs_fma2(S[2 * i], qq.x, oac[(2 * i) & 3]);
        oac[(2 * i + 1) & 3] = gs_fma2(S[2 * i + 1], qq.y, oac[(2 * i + 1) & 3]);
      }
    }
    float o = 0.f;
    if (want_o) {
      o = (gs_sum2(oac[0]) + gs_sum2(oac[1])) + (gs_sum2(oac[2]) + gs_sum2(oac[3]));
      o += __shfl_xor_sync(0xffffffffu, o, 1);
    }
    return o;
  };
  if (shift > 0) {
    for (int r = 0; r < shift; ++r) replay(&ksr[r][kh * KP], vsr[r][vloc], gsr[r]);
#pragma unroll
    for (int i = 0; i < 16; ++i)
      reinterpret_cast<ulonglong2*>(sp)[i] = make_ulonglong2(S[2 * i], S[2 * i + 1]);
  }
  __syncthreads();                         // every thread is done with the replayed v rows: the buffer becomes the output rows
  for (int r = 0; r < n; ++r) {
    float u;
    const float o = apply(&ks[r][kh * KP], &qs[r][kh * KP], vsm[r][vloc], gsm[r], bsm[r], true, u);
    if (kh == 0) {
      vsr[r][vloc] = o;
      vsm[r][vloc] = u;          // (this thread pair is the only reader of vsm[r][vloc]: the stash takes u)
    }
  }
  __syncthreads();
  // stash of this step's rows: k [128] | v [128] | g, beta
  for (int idx = tid; idx < n * 128; idx += kStepThreads) {
    const int r = idx >> 7, i = idx & 127;
    if (r < p.stash_rows) {
      stash[static_cast<size_t>(r) * stash_row + i] = ks[r][(i >> 6) * KP + (i & 63)];
      stash[static_cast<size_t>(r) * stash_row + 128 + i] = vsm[r][i];
    }
  }
  if (tid < n && tid < p.stash_rows) {
    stash[static_cast<size_t>(tid) * stash_row + 256] = gsm[tid];
    stash[static_cast<size_t>(tid) * stash_row + 257] = bsm[tid];
  }
  __syncthreads();

  // ---- phase 2: gated RMSNorm of the head (one warp per row, four values per lane), bf16 rows out
  for (int r = warp; r < n; r += kStepThreads / 32) {
    const size_t m = static_cast<size_t>(row0 + r);
    float a[4], z[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a[i] = vsr[r][lane * 4 + i];
      z[i] = __bfloat162float(p.z[m * p.ldz + h * 128 + lane * 4 + i]);
    }
    float ss = a[0] * a[0] + a[1] * a[1] + a[2] * a[2] + a[3] * a[3];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss * (1.f / 128.f) + p.eps);
    float amax = 0.f;
    __nv_bfloat16 o4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float wv = p.norm_w[lane * 4 + i] + p.w_offset;
      o4[i] = __float2bfloat16(a[i] * rstd * wv * silu_f(z[i]));
      amax = fmaxf(amax, fabsf(__bfloat162float(o4[i])));
    }
    amax = warp_max(amax);
    *reinterpret_cast<uint2*>(p.hout + m * (static_cast<size_t>(p.HV) * 128) + h * 128 + lane * 4) =
        *reinterpret_cast<const uint2*>(o4);
    if (lane == 0) p.amax_part[m * p.HV + h] = amax;
  }
  // ---- ticket: the last head CTA of the sequence quantises its rows and flips the conv-window word
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t old = atomicAdd(p.tickets + b, 1u);
    last_s = old == static_cast<uint32_t>(p.HV - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  if (tid == 0) {
    p.tickets[b] = 0u;
    *hist_word = par ^ 1;
  }
  const int K = p.HV * 128;
  // row maxima first (warp w takes rows w, w + 8), then every (row, 16-value chunk) item is independent:
  // four items in flight per thread
  float* row_inv = &red[0][0][0];            // (the conv's reduction buffer is free by now)
  const float qmax = p.qfmt == 1 ? 448.f : 127.f;
  for (int r = warp; r < n; r += kStepThreads / 32) {
    const size_t m = static_cast<size_t>(row0 + r);
    float am = 0.f;
    for (int i = lane; i < p.HV; i += 32) am = fmaxf(am, __ldcg(p.amax_part + m * p.HV + i));
    am = warp_max(am);
    if (lane == 0) {
      row_inv[r] = am > 0.f ? qmax / am : 0.f;
      p.scale[m] = am / qmax;
    }
  }
  __syncthreads();
  const int cpr = K >> 4;                     // chunks per row
  const int items = n * cpr;
  constexpr int kFly = 4;
  for (int it0 = tid; it0 < items; it0 += kStepThreads * kFly) {
    uint4 lo[kFly], hi[kFly];
#pragma unroll
    for (int f = 0; f < kFly; ++f) {
      const int it = it0 + f * kStepThreads;
      if (it < items) {
        const int r = it / cpr, ch = it - r * cpr;
        const __nv_bfloat16* src = p.hout + static_cast<size_t>(row0 + r) * K + (ch << 4);
        lo[f] = __ldcg(reinterpret_cast<const uint4*>(src));
        hi[f] = __ldcg(reinterpret_cast<const uint4*>(src + 8));
      }
    }
#pragma unroll
    for (int f = 0; f < kFly; ++f) {
      const int it = it0 + f * kStepThreads;
      if (it < items) {
        const int r = it / cpr, ch = it - r * cpr;
        const int m = row0 + r;
        const float inv = row_inv[r];
        const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo[f]);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi[f]);
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float2 f0 = __bfloat1622float2(l2[2 * i]), f1 = __bfloat1622float2(l2[2 * i + 1]);
          w[i] = quant4(f0.x, f0.y, f1.x, f1.y, inv, p.qfmt);
          const float2 g0 = __bfloat1622float2(h2[2 * i]), g1 = __bfloat1622float2(h2[2 * i + 1]);
          w[2 + i] = quant4(g0.x, g0.y, g1.x, g1.y, inv, p.qfmt);
        }
        const int kb = ch >> 3, cc = ch & 7;
        const size_t off = (static_cast<size_t>(kb) * p.M_pad + m) * 128 + (((cc ^ (m & 7)) & 7) << 4);
        *reinterpret_cast<uint4*>(p.q + off) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

}  // namespace saber

extern "C" int saber_gdn_step_launch(const saber::GdnStepParams* p, int nseq, cudaStream_t stream) {
  using namespace saber;
  if (p->HV % p->HK || p->C % 128 || p->n_q % 128 || p->n_k % 128 || p->max_rows > kStepRows || p->hist_rows < 3)
    return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(gdn_step_kernel, dim3(p->HV, nseq), dim3(kStepThreads), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}
