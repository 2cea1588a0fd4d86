// Chunked Gated DeltaNet for prefill: the gated delta rule over 64-row chunks instead of one row at a
// time.  Inside a chunk (rows i, cumulative log decay G_i, gamma_i = exp(G_i)):
//   A_ij = beta_i exp(G_i - G_j) (k_i . k_j)  (j < i),   (I + A) W = diag(beta gamma) K,
//   (I + A) U' = diag(beta) V,                 P_ij = exp(G_i - G_j) (q_i . k_j)  (j <= i)
// and, with S0 the state at the chunk's start,
//   U = U' - W S0^T,   O = diag(gamma) Q S0^T + P U,   S = gamma_C S0 + U^T diag(exp(G_C - G_j)) K.
// This is algebraically the row-by-row rule of gdn.cu (S <- S e^g; u = beta (v - S k); S <- S + u k^T;
// o = S q), regrouped so that the state is touched once per 64 rows.
//
// Two launches: `prep` is parallel over (value head, chunk): pair products, the two triangular
// solves (one column per thread, fully unrolled forward substitution) and P; `scan` walks the
// chunks of a sequence in order, one CTA per (value head, 32-row slice of the state), the slice held
// in registers (16 values per thread).  All arithmetic is fp32 on the CUDA cores, so the result
// differs from the row-by-row kernel only by summation order -- and so does the cost: regrouping
// does not remove arithmetic (about 90k FMAs per row and head against 65k row by row), it turns it
// into matrix products.  Measured on 2048 rows x 48 heads: prep 0.44 ms + scan 4.7 ms (before the
// bank-conflict fix) against 1.28 ms row by row, so the engine keeps the row-by-row kernel for
// prefill until the scan's products run on the tensor cores (tf32 `mma.sync`); this file is the
// fp32 statement of the algorithm that version will be checked against.
//
// Parity: crates/saber-kernels/hip/sgdn_chunk.h / `chunk_scan` + `kkt` kernels of the reference's
// prefill path (its published timings on gfx1201: chunk_scan 2048 rows 159.9 us, kkt 43.1 us).
#include "gdn.h"
#include "launch.cuh"
#include <cuda_bf16.h>

namespace saber {

constexpr int kChunk = 64;
constexpr int kKPad = 132;                 // padded row stride (floats) of the K / Q tiles in shared memory
// scratch per (slot, value head): W [64][128] | U' [64][128] | P [64][64] | G [64]
constexpr size_t kChunkScratchFloats = 64 * 128 + 64 * 128 + 64 * 64 + 64;

__device__ __forceinline__ float chunk_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// chunk c of sequence b lives in scratch slot cu_rows[b] / 64 + b + c (disjoint and < M / 64 + nseq)
__device__ __forceinline__ size_t chunk_slot(const int32_t* cu_rows, int b, int c) {
  return static_cast<size_t>(cu_rows[b] / kChunk + b + c);
}

// grid (HV, max_chunks, nseq), block 256, dynamic smem: K | Q (padded) | A
__global__ void __launch_bounds__(256) gdn_chunk_prep_kernel(const GdnRecParams p, float* __restrict__ scratch) {
  pdl_wait();
  extern __shared__ __align__(16) float cs[];
  float* Ks = cs;                          // [64][kKPad]
  float* Qs = Ks + kChunk * kKPad;         // [64][kKPad]
  float* As = Qs + kChunk * kKPad;         // [64][64]  A (strictly lower), later read by the solves
  __shared__ float Gs[kChunk], Bs[kChunk];
  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  if (p.slots[b] < 0) return;
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  const int r0 = c * kChunk;
  if (r0 >= n) return;
  const int m = min(kChunk, n - r0);       // live rows of this chunk
  const int hk = h / (p.HV / p.HK);
  const int t = threadIdx.x;
  const float neg_a = -__expf(p.A_log[h]);
  const float dtb = p.dt_bias[h];

  for (int idx = t; idx < kChunk * 128; idx += 256) {
    const int r = idx >> 7, i = idx & 127;
    float kv = 0.f, qv = 0.f;
    if (r < m) {
      const float* xr = p.qkv + static_cast<size_t>(row0 + r0 + r) * p.C;
      qv = xr[hk * 128 + i];
      kv = xr[p.n_q + hk * 128 + i];
    }
    Ks[r * kKPad + i] = kv;
    Qs[r * kKPad + i] = qv;
  }
  if (t < kChunk) {
    float g = 0.f, be = 0.f;
    if (t < m) {
      const size_t mm = static_cast<size_t>(row0 + r0 + t);
      const float bb = __bfloat162float(p.ba[mm * p.ldba + h]);
      const float aa = __bfloat162float(p.ba[mm * p.ldba + p.HV + h]);
      g = neg_a * chunk_softplus(aa + dtb);
      be = 1.f / (1.f + __expf(-bb));
    }
    Gs[t] = g;
    Bs[t] = be;
  }
  __syncthreads();
  if (t == 0) {                            // cumulative log decay
    float acc = 0.f;
    for (int i = 0; i < kChunk; ++i) { acc += Gs[i]; Gs[i] = acc; }
  }
  __syncthreads();

  float* out = scratch + (chunk_slot(p.cu_rows, b, c) * p.HV + h) * kChunkScratchFloats;
  float* Wo = out, *Uo = out + 64 * 128, *Po = out + 2 * 64 * 128, *Go = Po + 64 * 64;
  // pair products: thread takes pairs (i, j) = (pp / 64, pp % 64)
  for (int pp = t; pp < kChunk * kChunk; pp += 256) {
    const int i = pp >> 6, j = pp & 63;
    float kk = 0.f, qk = 0.f;
    if (j <= i) {
      const float4* ki = reinterpret_cast<const float4*>(Ks + i * kKPad);
      const float4* kj = reinterpret_cast<const float4*>(Ks + j * kKPad);
      const float4* qi = reinterpret_cast<const float4*>(Qs + i * kKPad);
#pragma unroll 8
      for (int x = 0; x < 32; ++x) {
        const float4 a = ki[x], bq = kj[x], q4 = qi[x];
        kk += a.x * bq.x + a.y * bq.y + a.z * bq.z + a.w * bq.w;
        qk += q4.x * bq.x + q4.y * bq.y + q4.z * bq.z + q4.w * bq.w;
      }
    }
    const float d = j <= i ? __expf(Gs[i] - Gs[j]) : 0.f;
    As[i * kChunk + j] = j < i ? Bs[i] * d * kk : 0.f;
    Po[i * kChunk + j] = d * qk;
  }
  if (t < kChunk) Go[t] = Gs[t];
  __syncthreads();

  // forward substitution, one right-hand-side column per thread: W columns for t < 128, U' columns else
  float x[kChunk];
  const bool is_w = t < 128;
  const int col = is_w ? t : t - 128;
#pragma unroll
  for (int i = 0; i < kChunk; ++i) {
    float rhs;
    if (is_w) rhs = Bs[i] * __expf(Gs[i]) * Ks[i * kKPad + col];
    else rhs = (i < m) ? Bs[i] * p.qkv[static_cast<size_t>(row0 + r0 + i) * p.C + p.n_q + p.n_k + h * 128 + col] : 0.f;
    float acc = rhs;
#pragma unroll
    for (int j = 0; j < i; ++j) acc -= As[i * kChunk + j] * x[j];
    x[i] = acc;
  }
  float* dst = is_w ? Wo : Uo;
#pragma unroll
  for (int i = 0; i < kChunk; ++i) dst[i * 128 + col] = x[i];
}

// grid (HV * 4, nseq), block 256: thread = (v row of the 32-row slice, 16-wide k part)
__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(const GdnRecParams p, const float* __restrict__ scratch) {
  pdl_wait();
  extern __shared__ __align__(16) float cs[];
  float* Wc = cs;                          // [64][128]
  float* Qp = Wc + 64 * 128;               // [64][128]  gamma_i q_i
  float* K2 = Qp + 64 * 128;               // [64][128]  exp(G_C - G_j) k_j
  float* Us = K2 + 64 * 128;               // [64][33]   U (this slice)
  float* Os = Us + 64 * 33;                // [64][33]   gamma Q S0^T (this slice)
  float* Ps = Os + 64 * 33;                // [64][64]
  __shared__ float Gs[kChunk];
  const int b = blockIdx.y;
  const int slot = p.slots[b];
  if (slot < 0) return;
  const int h = blockIdx.x >> 2, vs = blockIdx.x & 3;
  const int hk = h / (p.HV / p.HK);
  const int row0 = p.cu_rows[b];
  const int n = p.cu_rows[b + 1] - row0;
  if (n <= 0) return;
  const int t = threadIdx.x;
  const int vr = t >> 3, kp = t & 7;
  const int v = vs * 32 + vr;
  // this thread's 16 state values of row v are k = 32 x + 4 kp + c (x, c < 4): for a fixed x the eight
  // k parts read 128 contiguous bytes of a tile row (no bank conflicts)
  float* sp = p.state + ((static_cast<size_t>(slot) * p.HV + h) * 128 + v) * 128 + kp * 4;
  float S[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 s4 = *reinterpret_cast<const float4*>(sp + 32 * i);
    S[4 * i] = s4.x; S[4 * i + 1] = s4.y; S[4 * i + 2] = s4.z; S[4 * i + 3] = s4.w;
  }
  const int nchunks = (n + kChunk - 1) / kChunk;
  for (int c = 0; c < nchunks; ++c) {
    const int r0 = c * kChunk;
    const int m = min(kChunk, n - r0);
    const float* in = scratch + (chunk_slot(p.cu_rows, b, c) * p.HV + h) * kChunkScratchFloats;
    const float* Wi = in, *Ui = in + 64 * 128, *Pi = in + 2 * 64 * 128, *Gi = Pi + 64 * 64;
    __syncthreads();                       // the previous chunk is done with the tiles
    if (t < kChunk) Gs[t] = Gi[t];
    __syncthreads();
    const float gC = Gs[kChunk - 1];
    for (int idx = t; idx < 64 * 32; idx += 256)   // float4 copies of W
      reinterpret_cast<float4*>(Wc)[idx] = reinterpret_cast<const float4*>(Wi)[idx];
    for (int idx = t; idx < 64 * 64 / 4; idx += 256)
      reinterpret_cast<float4*>(Ps)[idx] = reinterpret_cast<const float4*>(Pi)[idx];
    for (int idx = t; idx < 64 * 32; idx += 256)     // this slice of U'
      Us[(idx >> 5) * 33 + (idx & 31)] = Ui[(idx >> 5) * 128 + vs * 32 + (idx & 31)];
    for (int idx = t; idx < kChunk * 128; idx += 256) {
      const int r = idx >> 7, i = idx & 127;
      float kv = 0.f, qv = 0.f;
      if (r < m) {
        const float* xr = p.qkv + static_cast<size_t>(row0 + r0 + r) * p.C;
        qv = xr[hk * 128 + i];
        kv = xr[p.n_q + hk * 128 + i];
      }
      Qp[idx] = qv * __expf(Gs[r]);
      K2[idx] = kv * __expf(gC - Gs[r]);
    }
    __syncthreads();
    // U = U' - W S0^T and gamma Q S0^T for this thread's v row: partial over its 16 k, reduced over the 8 k parts
    for (int i = 0; i < kChunk; ++i) {
      const float* w4 = Wc + i * 128 + kp * 4;
      const float* q4 = Qp + i * 128 + kp * 4;
      float su = 0.f, so = 0.f;
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float4 a = *reinterpret_cast<const float4*>(w4 + 32 * x), q = *reinterpret_cast<const float4*>(q4 + 32 * x);
        su += a.x * S[4 * x] + a.y * S[4 * x + 1] + a.z * S[4 * x + 2] + a.w * S[4 * x + 3];
        so += q.x * S[4 * x] + q.y * S[4 * x + 1] + q.z * S[4 * x + 2] + q.w * S[4 * x + 3];
      }
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        su += __shfl_xor_sync(0xffffffffu, su, o);
        so += __shfl_xor_sync(0xffffffffu, so, o);
      }
      if (kp == 0) {
        Us[i * 33 + vr] -= su;
        Os[i * 33 + vr] = so;
      }
    }
    __syncthreads();
    // O = gamma Q S0^T + P U: thread = (column vr2 of the slice, rows ig, ig + 8, ...)
    {
      const int vr2 = t & 31, ig = t >> 5;
      for (int i = ig; i < m; i += 8) {
        float acc = Os[i * 33 + vr2];
        for (int j = 0; j <= i; ++j) acc += Ps[i * kChunk + j] * Us[j * 33 + vr2];
        p.out[static_cast<size_t>(row0 + r0 + i) * (static_cast<size_t>(p.HV) * 128) + h * 128 + vs * 32 + vr2] = acc;
      }
    }
    // S = gamma_C S0 + U^T K2
    {
      const float dC = __expf(gC);
#pragma unroll
      for (int x = 0; x < 16; ++x) S[x] *= dC;
      for (int j = 0; j < kChunk; ++j) {
        const float u = Us[j * 33 + vr];
        const float* k4 = K2 + j * 128 + kp * 4;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float4 kk = *reinterpret_cast<const float4*>(k4 + 32 * x);
          S[4 * x] += u * kk.x; S[4 * x + 1] += u * kk.y; S[4 * x + 2] += u * kk.z; S[4 * x + 3] += u * kk.w;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4*>(sp + 32 * i) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
}

}  // namespace saber

extern "C" size_t saber_gdn_chunk_scratch_bytes(int max_rows, int nseq, int HV) {
  // (one scratch serves either form: the tensor-core form's operand images are the larger)
  const size_t a = (static_cast<size_t>(max_rows / saber::kChunk + nseq + 1)) * HV * saber::kChunkScratchFloats * sizeof(float);
  const size_t b = saber_gdn_chunk_tc_scratch_bytes(max_rows, nseq, HV);
  return a > b ? a : b;
}

// Committing (prefill) recurrence over all rows of every sequence.  `max_rows` bounds the rows of one
// sequence (sizes the grid), `scratch` holds saber_gdn_chunk_scratch_bytes(total rows, nseq, HV).
extern "C" int saber_gdn_chunk_launch(const saber::GdnRecParams* p, int nseq, int max_rows, float* scratch,
                                      cudaStream_t stream) {
  using namespace saber;
  if (p->chunk_impl == 1) return saber_gdn_chunk_tc_launch(p, nseq, max_rows, scratch, stream);
  if (p->HV % p->HK || !p->commit || scratch == nullptr || max_rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const int prep_smem = (2 * kChunk * kKPad + kChunk * kChunk) * sizeof(float);
  const int scan_smem = (3 * 64 * 128 + 2 * 64 * 33 + 64 * 64) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem);
    cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, scan_smem);
    configured = true;
  }
  const int max_chunks = (max_rows + kChunk - 1) / kChunk;
  saber::launch(gdn_chunk_prep_kernel, dim3(p->HV, max_chunks, nseq), dim3(256), prep_smem, stream, 0, *p, scratch);
  saber::launch(gdn_chunk_scan_kernel, dim3(p->HV * 4, nseq), dim3(256), scan_smem, stream, 0, *p,
                static_cast<const float*>(scratch));
  return static_cast<int>(cudaGetLastError());
}
