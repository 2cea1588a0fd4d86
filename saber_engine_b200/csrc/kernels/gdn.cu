// Gated DeltaNet (linear attention) step kernels for sm_100a.
//
// Math (per value head, state S[V=128][K=128], one token):
//   g = -exp(A_log) * softplus(a + dt_bias);  beta = sigmoid(b)
//   S <- S * exp(g);  u = (v - S k) * beta;  S <- S + u (x) k;  o = S q
// with q, k the causal depthwise conv (4 taps) + SiLU outputs, L2-normalised per head, q scaled by
// 1/sqrt(128).  Parity: crates/saber-kernels/hip/sgdn_rec.h:1-30 (recurrence), sgdn_conv.h:1-10
// (conv), and the base + stash + replay form of sgdn_replay.h:1-12: the state in memory is always
// the COMMITTED state; a speculative step's rows run on a register copy and leave only a small
// stash (k, u, g per row: u = beta (v - S k) as the row computed it); the next step first replays the `shift` rows that were accepted,
// stores the new committed state, and then answers its own rows.  No per-row state snapshots.
//
// Two launches per layer: conv_update (thread = channel, block = one 128-wide head so the q/k L2
// norm is a block reduction) and recurrent (CTA = (value head, v-slice, sequence), two threads per
// state row holding 64 fp32 each).  Prefill chunks use the same kernels with commit=1: rows are
// consumed for good, the final state is stored and conv_commit rewrites the conv window.
#include "launch.cuh"
#include "gdn.h"
#include <cuda_bf16.h>

namespace saber {

__device__ __forceinline__ float gdn_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gdn_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// First row of the slot's current conv window (a slot with two windows names the current one in the
// first word of its last row).
__device__ __forceinline__ __nv_bfloat16* gdn_hist_current(const GdnConvParams& p, int slot) {
  if (!p.dual) return p.hist + static_cast<size_t>(slot) * p.hist_rows * p.C;
  __nv_bfloat16* base = p.hist + static_cast<size_t>(slot) * (2 * p.hist_rows + 1) * p.C;
  const int cur = *reinterpret_cast<const int*>(base + static_cast<size_t>(2 * p.hist_rows) * p.C) & 1;
  return base + static_cast<size_t>(cur) * p.hist_rows * p.C;
}

// ---------------------------------------------------------------------------------- conv update
// grid (C / 128, nseq, row chunks), block 128.  The conv is causal with a 4-tap window, so chunks of
// kConvChunk rows are independent: a chunk reads the three inputs before its first row from x (or,
// for the first rows of the step, from the committed window in `hist`).
constexpr int kConvChunk = 32;
__global__ void __launch_bounds__(128) gdn_conv_update_kernel(const GdnConvParams p) {
  pdl_trigger();   // the recurrence that follows loads its state (which no kernel of this step writes before it) meanwhile
  pdl_wait();
  __shared__ float red[4];
  const int b = blockIdx.y;
  const int slot = p.slots[b];
  if (slot < 0) return;
  const int ch = blockIdx.x * 128 + threadIdx.x;
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  const int r_first = blockIdx.z * kConvChunk;
  if (r_first >= n) return;
  const int r_last = min(n, r_first + kConvChunk);
  const int shift = p.shift[b];
  __nv_bfloat16* hp = gdn_hist_current(p, slot) + ch;
  // window = the three inputs that precede this chunk's first row: input j < 0 of the step is row
  // shift + 3 + j of the history (the committed window shifted by the accepted rows)
  auto input_at = [&](int j) -> float {
    return j >= 0 ? __bfloat162float(p.x[static_cast<size_t>(row0 + j) * p.ldx + ch])
                  : __bfloat162float(hp[static_cast<size_t>(shift + 3 + j) * p.C]);
  };
  float b0 = input_at(r_first - 3), b1 = input_at(r_first - 2), b2 = input_at(r_first - 1);
  if (!p.commit && r_first == 0) {
    hp[0] = __float2bfloat16(b0);
    hp[p.C] = __float2bfloat16(b1);
    hp[2 * static_cast<size_t>(p.C)] = __float2bfloat16(b2);
  }
  const float w0 = p.conv_w[ch * 4 + 0], w1 = p.conv_w[ch * 4 + 1], w2 = p.conv_w[ch * 4 + 2],
              w3 = p.conv_w[ch * 4 + 3];
  const bool is_q = ch < p.n_q, is_k = !is_q && ch < p.n_q + p.n_k;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = r_first; r < r_last; ++r) {
    const __nv_bfloat16 xb = p.x[static_cast<size_t>(row0 + r) * p.ldx + ch];
    const float x = __bfloat162float(xb);
    float y = gdn_silu(w0 * b0 + w1 * b1 + w2 * b2 + w3 * x);
    b0 = b1; b1 = b2; b2 = x;
    if (!p.commit && r < p.hist_rows - 3) hp[static_cast<size_t>(3 + r) * p.C] = xb;
    if (is_q || is_k) {  // uniform per block: a block is one head
      float ss = y * y;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      __syncthreads();
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = red[0] + red[1] + red[2] + red[3];
      y *= rsqrtf(ss + 1e-6f);
      if (is_q) y *= p.q_scale;
    }
    p.out[static_cast<size_t>(row0 + r) * p.C + ch] = y;
  }
}

// After a committing (prefill) step: window = last three inputs of (old window ++ this step's rows).
__global__ void __launch_bounds__(128) gdn_conv_commit_kernel(const GdnConvParams p) {
  pdl_wait();
  const int b = blockIdx.y;
  const int slot = p.slots[b];
  if (slot < 0) return;
  const int ch = blockIdx.x * 128 + threadIdx.x;
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  if (n <= 0) return;
  const int shift = p.shift[b];
  __nv_bfloat16* hp = gdn_hist_current(p, slot) + ch;
  __nv_bfloat16 win[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int j = n + i;  // index into (old window(3) ++ rows(n)), last three are j = n..n+2
    win[i] = j < 3 ? hp[static_cast<size_t>(shift + j) * p.C]
                   : p.x[static_cast<size_t>(row0 + j - 3) * p.ldx + ch];
  }
  if (p.dual) {   // both windows get the committed inputs: whichever the slot's word names is right
    __nv_bfloat16* h0 = p.hist + static_cast<size_t>(slot) * (2 * p.hist_rows + 1) * p.C + ch;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      h0[static_cast<size_t>(i) * p.C] = win[i];
      h0[static_cast<size_t>(p.hist_rows + i) * p.C] = win[i];
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 3; ++i) hp[static_cast<size_t>(i) * p.C] = win[i];
}

// ---------------------------------------------------------------------------------- recurrence
// Packed fp32 pairs: sm_100 issues two fp32 FMAs per instruction (fma.rn.f32x2), which halves the
// instruction count of the state update -- the kernel is bound by issue slots, not by memory.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float sum2(f32x2 v) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo + hi;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// grid (HV * VS, nseq); block = 2 * (128 / VS) threads; thread = (v row, k half).
// Rows are staged in shared memory in batches of kRecBatch (all loads of a batch are issued
// together, so the per-row loop touches no global memory except its one output element).
constexpr int kRecBatch = 16;

__device__ __forceinline__ void gdn_cp16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst_smem))),
               "l"(src) : "memory");
}

template <int VS>
__global__ void __launch_bounds__(256 / VS) gdn_recurrent_kernel(const GdnRecParams p) {
  pdl_trigger();   // successors (the norm rows, then a GEMM) get resident on the SMs the last round leaves idle
  constexpr int VR = 128 / VS;         // v rows per CTA
  constexpr int NT = 2 * VR;           // threads
  constexpr int KP = 64 + 4;           // padded half stride in shared memory (bank spread)
  __shared__ __align__(16) float ks[kRecBatch][2 * KP];
  __shared__ __align__(16) float qs[kRecBatch][2 * KP];
  __shared__ __align__(16) float vsm[kRecBatch][VR];
  __shared__ float gsm[kRecBatch], bsm[kRecBatch];
  // the replayed rows of the previous step have buffers of their own: they are fetched together
  // with this step's first batch and the state, so the kernel waits for global memory once
  __shared__ __align__(16) float ksr[kRecBatch][2 * KP];
  __shared__ __align__(16) float vsr[kRecBatch][VR];
  __shared__ float gsr[kRecBatch], bsr[kRecBatch];
  const int b = blockIdx.y;
  const int slot = p.slots[b];
  if (slot < 0) return;
  const int h = blockIdx.x / VS, vs = blockIdx.x % VS;
  const int hk = h / (p.HV / p.HK);
  const int tid = threadIdx.x;
  const int vloc = tid >> 1, kh = tid & 1;
  const int v = vs * VR + vloc;
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  const int shift = min(p.shift[b], min(p.stash_rows, kRecBatch));
  const int stash_stride = 128 + VR + 4;
  float* sp = p.state + ((static_cast<size_t>(slot) * p.HV + h) * 128 + v) * 128 + kh * 64;
  float* stash = p.stash + ((static_cast<size_t>(slot) * p.stash_rows) * p.HV * VS +
                            static_cast<size_t>(h) * VS + vs) * stash_stride;
  const size_t stash_row = static_cast<size_t>(p.HV) * VS * stash_stride;
  // The state goes out FIRST, before the wait for the predecessor (the conv kernel): the index tables were
  // uploaded before the program started and the state was last written by the previous step.
  f32x2 S[32];   // this thread's 64 state values as packed pairs
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const ulonglong2 t = reinterpret_cast<const ulonglong2*>(sp)[i];
    S[2 * i] = t.x;
    S[2 * i + 1] = t.y;
  }
  pdl_wait();

  // ---- everything else this CTA reads from global memory goes out now: replay rows, first batch
  const int nb0 = min(kRecBatch, n);
  for (int idx = tid; idx < shift * 32; idx += NT) {
    const int r = idx >> 5, i = (idx & 31) * 4;
    gdn_cp16(&ksr[r][(i >> 6) * KP + (i & 63)], stash + static_cast<size_t>(r) * stash_row + i);
  }
  for (int idx = tid; idx < shift * (VR / 4); idx += NT) {
    const int r = idx / (VR / 4), i = (idx % (VR / 4)) * 4;
    gdn_cp16(&vsr[r][i], stash + static_cast<size_t>(r) * stash_row + 128 + i);
  }
  for (int idx = tid; idx < nb0 * 64; idx += NT) {
    const int r = idx >> 6, c = idx & 63, i = (c & 31) * 4;
    const float* xr = p.qkv + static_cast<size_t>(row0 + r) * p.C;
    if (c < 32) gdn_cp16(&qs[r][(i >> 6) * KP + (i & 63)], xr + hk * 128 + i);
    else gdn_cp16(&ks[r][(i >> 6) * KP + (i & 63)], xr + p.n_q + hk * 128 + i);
  }
  for (int idx = tid; idx < nb0 * (VR / 4); idx += NT) {
    const int r = idx / (VR / 4), i = (idx % (VR / 4)) * 4;
    gdn_cp16(&vsm[r][i], p.qkv + static_cast<size_t>(row0 + r) * p.C + p.n_q + p.n_k + h * 128 + vs * VR + i);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  float g_rep = 0.f, b_rep = 0.f, bb0 = 0.f, aa0 = 0.f;
  if (tid < shift) {
    g_rep = stash[static_cast<size_t>(tid) * stash_row + 128 + VR];
    b_rep = stash[static_cast<size_t>(tid) * stash_row + 128 + VR + 1];
  }
  if (tid < nb0) {
    const size_t m = static_cast<size_t>(row0 + tid);
    bb0 = __bfloat162float(p.ba[m * p.ldba + h]);
    aa0 = __bfloat162float(p.ba[m * p.ldba + p.HV + h]);
  }
  const float neg_a = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[h];
  if (tid < shift) { gsr[tid] = g_rep; bsr[tid] = b_rep; }
  if (tid < nb0) {
    gsm[tid] = neg_a * gdn_softplus(aa0 + dtb);
    bsm[tid] = 1.f / (1.f + __expf(-bb0));
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();

  // replay of a row whose u is known: S <- S e^g + u (x) k (the same two operations, in the same
  // order, that the row itself applied: the state comes out bit-identical, without its dot product)
  auto replay = [&](const float* kv, float u, float g) {
    const ulonglong2* kv2 = reinterpret_cast<const ulonglong2*>(kv);
    const float decay = __expf(g);
    const f32x2 dec2 = pack2(decay, decay), u2 = pack2(u, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const ulonglong2 kk = kv2[i];
      S[2 * i] = fma2(u2, kk.x, mul2(S[2 * i], dec2));
      S[2 * i + 1] = fma2(u2, kk.y, mul2(S[2 * i + 1], dec2));
    }
  };
  auto apply = [&](const float* kv, const float* qv, float vval, float g, float beta,
                   bool want_o, float& u_out) -> float {
    const ulonglong2* kv2 = reinterpret_cast<const ulonglong2*>(kv);   // 16-byte aligned rows
    const ulonglong2* qv2 = reinterpret_cast<const ulonglong2*>(qv);
    const float decay = __expf(g);
    const f32x2 dec2 = pack2(decay, decay);
    f32x2 acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const ulonglong2 kk = kv2[i];
      S[2 * i] = mul2(S[2 * i], dec2);
      S[2 * i + 1] = mul2(S[2 * i + 1], dec2);
      acc[(2 * i) & 3] = fma2(S[2 * i], kk.x, acc[(2 * i) & 3]);
      acc[(2 * i + 1) & 3] = fma2(S[2 * i + 1], kk.y, acc[(2 * i + 1) & 3]);
    }
    float dot = (sum2(acc[0]) + sum2(acc[1])) + (sum2(acc[2]) + sum2(acc[3]));
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float u = (vval - dot) * beta;
    u_out = u;
    const f32x2 u2 = pack2(u, u);
    f32x2 oac[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const ulonglong2 kk = kv2[i];
      S[2 * i] = fma2(u2, kk.x, S[2 * i]);
      S[2 * i + 1] = fma2(u2, kk.y, S[2 * i + 1]);
      if (want_o) {
        const ulonglong2 qq = qv2[i];
        oac[(2 * i) & 3] = fma2(S[2 * i], qq.x, oac[(2 * i) & 3]);
        oac[(2 * i + 1) & 3] = fma2(S[2 * i + 1], qq.y, oac[(2 * i + 1) & 3]);
      }
    }
    float o = 0.f;
    if (want_o) {
      o = (sum2(oac[0]) + sum2(oac[1])) + (sum2(oac[2]) + sum2(oac[3]));
      o += __shfl_xor_sync(0xffffffffu, o, 1);
    }
    return o;
  };

  // ---- replay the accepted rows of the previous step, then store the committed state
  if (shift > 0) {
    for (int r = 0; r < shift; ++r) replay(&ksr[r][kh * KP], vsr[r][vloc], gsr[r]);      // (vsr holds the stashed u)
#pragma unroll
    for (int i = 0; i < 16; ++i)
      reinterpret_cast<ulonglong2*>(sp)[i] = make_ulonglong2(S[2 * i], S[2 * i + 1]);
  }

  // ---- this step's rows, a batch at a time
  for (int r0 = 0; r0 < n; r0 += kRecBatch) {
    const int nb = min(kRecBatch, n - r0);
    if (r0 > 0) {      // (the first batch arrived with the state)
      for (int idx = tid; idx < nb * 128; idx += NT) {
        const int r = idx >> 7, i = idx & 127;
        const float* xr = p.qkv + static_cast<size_t>(row0 + r0 + r) * p.C;
        qs[r][(i >> 6) * KP + (i & 63)] = xr[hk * 128 + i];
        ks[r][(i >> 6) * KP + (i & 63)] = xr[p.n_q + hk * 128 + i];
      }
      for (int idx = tid; idx < nb * VR; idx += NT) {
        const int r = idx / VR, i = idx % VR;
        vsm[r][i] = p.qkv[static_cast<size_t>(row0 + r0 + r) * p.C + p.n_q + p.n_k + h * 128 + vs * VR + i];
      }
      if (tid < nb) {
        const size_t m = static_cast<size_t>(row0 + r0 + tid);
        const float bb = __bfloat162float(p.ba[m * p.ldba + h]);
        const float aa = __bfloat162float(p.ba[m * p.ldba + p.HV + h]);
        gsm[tid] = neg_a * gdn_softplus(aa + dtb);
        bsm[tid] = 1.f / (1.f + __expf(-bb));
      }
      __syncthreads();
    }
    for (int r = 0; r < nb; ++r) {
      float u;
      const float o = apply(&ks[r][kh * KP], &qs[r][kh * KP], vsm[r][vloc], gsm[r], bsm[r], true, u);
      if (kh == 0) {
        p.out[static_cast<size_t>(row0 + r0 + r) * (static_cast<size_t>(p.HV) * 128) + h * 128 + v] = o;
        vsm[r][vloc] = u;        // (the thread pair of this state row is the only reader of vsm[r][vloc], and both of
                                 //  its lanes took the value before the shuffles inside apply: the stash takes u from here)
      }
    }
    if (!p.commit) {
      __syncthreads();      // u of every row is in shared memory
      for (int idx = tid; idx < nb * 128; idx += NT) {
        const int r = idx >> 7, i = idx & 127;
        if (r0 + r < p.stash_rows)
          stash[static_cast<size_t>(r0 + r) * stash_row + i] = ks[r][(i >> 6) * KP + (i & 63)];
      }
      for (int idx = tid; idx < nb * VR; idx += NT) {
        const int r = idx / VR, i = idx % VR;
        if (r0 + r < p.stash_rows) stash[static_cast<size_t>(r0 + r) * stash_row + 128 + i] = vsm[r][i];
      }
      if (tid < nb && r0 + tid < p.stash_rows) {
        stash[static_cast<size_t>(r0 + tid) * stash_row + 128 + VR] = gsm[tid];
        stash[static_cast<size_t>(r0 + tid) * stash_row + 128 + VR + 1] = bsm[tid];
      }
    }
    __syncthreads();
  }
  if (p.commit && n > 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      reinterpret_cast<ulonglong2*>(sp)[i] = make_ulonglong2(S[2 * i], S[2 * i + 1]);
  }
}

// ---------------------------------------------------------------------------------- prefill rows
// Committing (prefill) form of the recurrence for long row runs.  A prefill rung is one sequence
// walking thousands of rows in order, so what counts is the latency of one row step.  A thread holds
// VR state rows (16 values of each): one read of its k and q parts from shared memory serves VR
// rows, and the rows give every dependent chain (decay, dot, reduction, update) VR independent
// instances.  Batches of 16 rows arrive by 16-byte asynchronous copies into a double buffer while
// the previous batch is computed; the reduction of a row's output rides with the next row's
// dot-product reduction.  No stash and no replay (a prefill chunk starts from the committed state).
// grid (HV * 4, nseq), block 256 / VR: thread = (group of VR v rows of a 32-row slice, k part); the
// thread's values of a row are k = 32 x + 4 kq + c (x, c < 4): the eight parts read 128 contiguous
// bytes per x.
constexpr int kPfBatch = 16;

__device__ __forceinline__ void gdn_cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst_smem))),
               "l"(src) : "memory");
}

template <int VR>   // state rows per thread: 4 (block 64) or 2 (block 128)
__global__ void __launch_bounds__(256 / VR) gdn_prefill_rows_kernel(const GdnRecParams p) {
  constexpr int kThreads = 256 / VR;
  pdl_wait();
  __shared__ __align__(16) float ks[2][kPfBatch][128];
  __shared__ __align__(16) float qs[2][kPfBatch][128];
  __shared__ __align__(16) float vsm[2][kPfBatch][32];
  __shared__ float dsm[2][kPfBatch], bsm[2][kPfBatch];     // decay = exp(g), beta
  const int b = blockIdx.y;
  const int slot = p.slots[b];
  if (slot < 0) return;
  const int h = blockIdx.x >> 2, vs = blockIdx.x & 3;
  const int hk = h / (p.HV / p.HK);
  const int tid = threadIdx.x;
  const int vg = tid >> 3, kq = tid & 7;
  const int v0 = vs * 32 + vg * VR;
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  if (n <= 0) return;
  float* sp = p.state + ((static_cast<size_t>(slot) * p.HV + h) * 128 + v0) * 128 + kq * 4;
  f32x2 S[VR][8];
#pragma unroll
  for (int j = 0; j < VR; ++j)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(sp + j * 128 + 32 * x);
      S[j][2 * x] = t.x;
      S[j][2 * x + 1] = t.y;
    }
  const float neg_a = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[h];
  const int nbatch = (n + kPfBatch - 1) / kPfBatch;
  float bb_n = 0.f, aa_n = 0.f;          // gate inputs of the batch in flight (threads tid < rows of the batch)
  auto issue = [&](int bi, int buf) {
    const int r0 = bi * kPfBatch, nb = min(kPfBatch, n - r0);
    for (int idx = tid; idx < nb * 64; idx += kThreads) {
      const int r = idx >> 6, c = idx & 63;
      const float* xr = p.qkv + static_cast<size_t>(row0 + r0 + r) * p.C;
      if (c < 32) gdn_cp_async16(&qs[buf][r][4 * c], xr + hk * 128 + 4 * c);
      else gdn_cp_async16(&ks[buf][r][4 * (c - 32)], xr + p.n_q + hk * 128 + 4 * (c - 32));
    }
    for (int idx = tid; idx < nb * 8; idx += kThreads) {
      const int r = idx >> 3, c = idx & 7;
      gdn_cp_async16(&vsm[buf][r][4 * c],
                     p.qkv + static_cast<size_t>(row0 + r0 + r) * p.C + p.n_q + p.n_k + h * 128 + vs * 32 + 4 * c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (tid < nb) {
      const size_t m = static_cast<size_t>(row0 + r0 + tid);
      bb_n = __bfloat162float(p.ba[m * p.ldba + h]);
      aa_n = __bfloat162float(p.ba[m * p.ldba + p.HV + h]);
    }
  };
  issue(0, 0);
  for (int bi = 0; bi < nbatch; ++bi) {
    const int buf = bi & 1;
    const int r0 = bi * kPfBatch, nb = min(kPfBatch, n - r0);
    if (tid < nb) {
      dsm[buf][tid] = __expf(neg_a * gdn_softplus(aa_n + dtb));
      bsm[buf][tid] = 1.f / (1.f + __expf(-bb_n));
    }
    if (bi + 1 < nbatch) {
      issue(bi + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    // The reduction of a row's OUTPUT partial sums is not needed by the next row: it rides with the
    // next row's dot-product reduction (eight independent shuffles per stage instead of four) and
    // the row is stored one step late; the last row of a batch is flushed after the loop.
    float op[VR];
#pragma unroll
    for (int j = 0; j < VR; ++j) op[j] = 0.f;
    for (int r = 0; r < nb; ++r) {
      const float decay = dsm[buf][r], beta = bsm[buf][r];
      const f32x2 dec2 = pack2(decay, decay);
      ulonglong2 kk[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) kk[x] = *reinterpret_cast<const ulonglong2*>(&ks[buf][r][32 * x + 4 * kq]);
      float dot[VR];
#pragma unroll
      for (int j = 0; j < VR; ++j) {
        f32x2 a0 = 0ull, a1 = 0ull;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          S[j][2 * x] = mul2(S[j][2 * x], dec2);
          S[j][2 * x + 1] = mul2(S[j][2 * x + 1], dec2);
          a0 = fma2(S[j][2 * x], kk[x].x, a0);
          a1 = fma2(S[j][2 * x + 1], kk[x].y, a1);
        }
        dot[j] = sum2(a0) + sum2(a1);
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
#pragma unroll
        for (int j = 0; j < VR; ++j) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
#pragma unroll
        for (int j = 0; j < VR; ++j) op[j] += __shfl_xor_sync(0xffffffffu, op[j], o);
      }
      if (r > 0 && kq == 0) {
        float* po = p.out + static_cast<size_t>(row0 + r0 + r - 1) * (static_cast<size_t>(p.HV) * 128) + h * 128 + v0;
#pragma unroll
        for (int j = 0; j < VR; ++j) po[j] = op[j];
      }
      float vj[VR];
#pragma unroll
      for (int j = 0; j < VR; ++j) vj[j] = vsm[buf][r][vg * VR + j];
      ulonglong2 qq[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) qq[x] = *reinterpret_cast<const ulonglong2*>(&qs[buf][r][32 * x + 4 * kq]);
#pragma unroll
      for (int j = 0; j < VR; ++j) {
        const float u = (vj[j] - dot[j]) * beta;
        const f32x2 u2 = pack2(u, u);
        f32x2 o0 = 0ull, o1 = 0ull;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          S[j][2 * x] = fma2(u2, kk[x].x, S[j][2 * x]);
          S[j][2 * x + 1] = fma2(u2, kk[x].y, S[j][2 * x + 1]);
          o0 = fma2(S[j][2 * x], qq[x].x, o0);
          o1 = fma2(S[j][2 * x + 1], qq[x].y, o1);
        }
        op[j] = sum2(o0) + sum2(o1);
      }
    }
#pragma unroll
    for (int s2 = 1; s2 < 8; s2 <<= 1)
#pragma unroll
      for (int j = 0; j < VR; ++j) op[j] += __shfl_xor_sync(0xffffffffu, op[j], s2);
    if (kq == 0) {
      float* po = p.out + static_cast<size_t>(row0 + r0 + nb - 1) * (static_cast<size_t>(p.HV) * 128) + h * 128 + v0;
#pragma unroll
      for (int j = 0; j < VR; ++j) po[j] = op[j];
    }
    __syncthreads();                       // this buffer is refilled by the copies of the next iteration
  }
#pragma unroll
  for (int j = 0; j < VR; ++j)
#pragma unroll
    for (int x = 0; x < 4; ++x)
      *reinterpret_cast<ulonglong2*>(sp + j * 128 + 32 * x) = make_ulonglong2(S[j][2 * x], S[j][2 * x + 1]);
}

}  // namespace saber

extern "C" int saber_gdn_conv_launch(const saber::GdnConvParams* p, int nseq, cudaStream_t stream) {
  using namespace saber;
  if (p->C % 128 || p->n_q % 128 || p->n_k % 128) return static_cast<int>(cudaErrorInvalidValue);
  dim3 grid(p->C / 128, nseq);
  dim3 grid_u(p->C / 128, nseq, (max(1, p->max_rows) + kConvChunk - 1) / kConvChunk);
  saber::launch(gdn_conv_update_kernel, grid_u, dim3(128), 0, stream, 0, *p);
  if (p->commit) saber::launch(gdn_conv_commit_kernel, dim3(grid), dim3(128), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_gdn_recurrent_launch(const saber::GdnRecParams* p, int nseq, int vs,
                                          cudaStream_t stream) {
  using namespace saber;
  if (p->HV % p->HK) return static_cast<int>(cudaErrorInvalidValue);
  if (p->commit && p->prefill_rows) {      // long committing runs: the latency-oriented form
    // two state rows per thread measured 863 us per 2048 rows, four 904 us, the first form (one row per
    // eight threads, synchronous staging) 1071 us
    // (prefill_rows selects the form: 1 = two state rows per thread, 2 = one, 3 = four)
    if (p->prefill_rows == 2) saber::launch(gdn_prefill_rows_kernel<1>, dim3(p->HV * 4, nseq), dim3(256), 0, stream, 0, *p);
    else if (p->prefill_rows == 3) saber::launch(gdn_prefill_rows_kernel<4>, dim3(p->HV * 4, nseq), dim3(64), 0, stream, 0, *p);
    else saber::launch(gdn_prefill_rows_kernel<2>, dim3(p->HV * 4, nseq), dim3(128), 0, stream, 0, *p);
    return static_cast<int>(cudaGetLastError());
  }
  if (vs == 1) saber::launch(gdn_recurrent_kernel<1>, dim3(dim3(p->HV, nseq)), dim3(256), 0, stream, 0, *p);
  else if (vs == 2) saber::launch(gdn_recurrent_kernel<2>, dim3(dim3(p->HV * 2, nseq)), dim3(128), 0, stream, 0, *p);
  else if (vs == 4) saber::launch(gdn_recurrent_kernel<4>, dim3(dim3(p->HV * 4, nseq)), dim3(64), 0, stream, 0, *p);
  else return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}
