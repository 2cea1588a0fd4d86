// Row producers: every op that feeds a quantised GEMM, one CTA per token row, 16-byte vector
// traffic, and the per-token int8 quantisation fused in so that the GEMM's activation operand is
// written ONCE, already in the tiled/swizzled order the tcgen05 GEMM copies with one bulk copy.
//
// Modes (parity with the reference's activation producers, crates/saber-kernels/hip/
// mxfp4_quant.hip:11-25, macaq_i8.h:1-13, attn_glue.hip attn_gate_quant, saber_gdn_norm.hip):
//   ADD_RMS    s = x + res (fp32); res_out = bf16(s); n = bf16(s * rsqrt(mean s^2 + eps) * (1 + w))
//   SILU_MUL   h = bf16(silu(gate) * up), gate = in[:, :K], up = in[:, K:2K]
//   GATE_SIG   h = bf16(a * sigmoid(b))                          (attention output gate)
//   GDN_NORM   per 128-wide head: h = bf16(rmsnorm(a) * w * silu(b))   (gated RMSNorm, plain w)
//   PLAIN      h = a
// Quantisation law (per token row): amax = max |h|; scale = amax / 127; q = clamp(rint(h * (127 /
// amax)), -127, 127); a zero row stores scale 0.  Rows in [M, M_pad) are written as zeros.
#include "launch.cuh"
#include "rowops.h"
#include "gemm_i8.h"
#include "ptx_sm100.cuh"
#include "rowops_body.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace saber {

constexpr int kRowThreads = 256;

// Quantise the row held in shared memory (bf16, K values) and store it tiled. All threads call.
__device__ __forceinline__ void quant_store_row(const __nv_bfloat16* h, int K, int m, int M_pad,
                                                float amax, int8_t* q, float* scale, int qfmt,
                                                uint8_t* q_sf = nullptr, int sf_m_tiles = 0) {
  if (qfmt == 2) {   // NVFP4: a 16-value chunk is one block
    const float g = amax / (6.f * 448.f);
    if (threadIdx.x == 0) scale[m] = g;
    for (int ch = threadIdx.x; ch < (K >> 4); ch += blockDim.x) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(h[(ch << 4) + i]);
      fp4_store_chunk(v, g, ch, m, M_pad, q, q_sf, sf_m_tiles);
    }
    return;
  }
  const float qmax = qfmt == 1 ? 448.f : 127.f;
  const float inv = amax > 0.f ? qmax / amax : 0.f;
  if (threadIdx.x == 0) scale[m] = amax / qmax;
  const int nchunk = K >> 4;
  for (int ch = threadIdx.x; ch < nchunk; ch += blockDim.x) {
    const int k0 = ch << 4;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = quant4(__bfloat162float(h[k0 + i * 4]), __bfloat162float(h[k0 + i * 4 + 1]),
                    __bfloat162float(h[k0 + i * 4 + 2]), __bfloat162float(h[k0 + i * 4 + 3]), inv, qfmt);
    }
    const int kb = k0 >> 7, c = (k0 & 127) >> 4;
    int8_t* dst = q + (static_cast<size_t>(kb) * M_pad + m) * 128 + (((c ^ (m & 7)) & 7) << 4);
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kRowThreads) row_producer_kernel(const RowOpParams p) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t row_smem[];
  __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(row_smem);  // K bf16
  __shared__ float red[32];
  const int m = blockIdx.x;
  const int K = p.K;
  if (p.m_live != nullptr && m >= *p.m_live) return;   // whole block: rows past the live count
  if (m >= p.M) {  // padding row: zeros
    if (p.q) {
      const int nchunk = p.qfmt == 2 ? (K >> 5) : (K >> 4);    // 16-byte pieces of the row (packed FP4: half as many)
      for (int ch = threadIdx.x; ch < nchunk; ch += blockDim.x) {
        const int k0 = ch << 4;
        const int kb = k0 >> 7, c = (k0 & 127) >> 4;
        int8_t* dst = p.q + (static_cast<size_t>(kb) * p.M_pad + m) * 128 + (((c ^ (m & 7)) & 7) << 4);
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
      if (threadIdx.x == 0) p.scale[m] = 0.f;
    }
    return;
  }
  const int nvec = K >> 3;
  float amax = 0.f;

  uint32_t tp_par = 0;
  if (MODE == kRowAddRms && p.tp_nranks > 1) {
    // wait for the tiles of this row from every rank: one thread per (source rank, feature tile)
    const uint32_t seq = *p.tp_seq_base + static_cast<uint32_t>(p.tp_site) + 1u;
    tp_par = seq & 1u;
    const int nflags = p.tp_nranks * p.tp_tiles_n;
    for (int f = threadIdx.x; f < nflags; f += blockDim.x) {
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
  if (MODE == kRowAddRms) {
    float* s = reinterpret_cast<float*>(row_smem + static_cast<size_t>(K) * 2);  // K fp32 after h
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float x[8];
      if (p.tp_nranks > 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = 0.f;
        for (int src = 0; src < p.tp_nranks; ++src) {   // fixed order: identical sums on every rank
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(
              p.tp_recv + ((static_cast<size_t>(tp_par) * p.tp_nranks + src) * p.tp_rows + m) * p.tp_ld + v * 8));
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            x[2 * i] += f.x;
            x[2 * i + 1] += f.y;
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __bfloat162float(__float2bfloat16(x[i]));  // the all-reduced bf16 value
      } else if (p.a) load8(p.a + static_cast<size_t>(m) * p.lda + v * 8, x);
      else {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = 0.f;
      }
      if (p.res) {
        float r[8];
        load8(p.res + static_cast<size_t>(m) * p.ldres + v * 8, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] += r[i];
        store8(p.res + static_cast<size_t>(m) * p.ldres + v * 8, x);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s[v * 8 + i] = x[i];
        ss += x[i] * x[i];
      }
    }
    ss = block_reduce<false>(ss, red);
    const float rstd = rsqrtf(ss / static_cast<float>(K) + p.eps);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wv = p.w[v * 8 + i] + p.w_offset;
        x[i] = __bfloat162float(__float2bfloat16(s[v * 8 + i] * rstd * wv));
        amax = fmaxf(amax, fabsf(x[i]));
      }
      store8(h + v * 8, x);
      if (p.out) store8(p.out + static_cast<size_t>(m) * p.ldout + v * 8, x);
    }
  } else if (MODE == kRowGdnNorm) {
    // one warp per 128-wide head, heads strided over the warps
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int nheads = K >> 7;
    for (int hd = warp; hd < nheads; hd += nw) {
      const int k0 = hd * 128 + lane * 4;
      float a[4], z[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = p.a_f32 ? p.a_f32[static_cast<size_t>(m) * p.lda + k0 + i]
                       : __bfloat162float(p.a[static_cast<size_t>(m) * p.lda + k0 + i]);
        z[i] = __bfloat162float(p.b[static_cast<size_t>(m) * p.ldb + k0 + i]);
      }
      float ss = a[0] * a[0] + a[1] * a[1] + a[2] * a[2] + a[3] * a[3];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss * (1.f / 128.f) + p.eps);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float wv = p.w[lane * 4 + i] + p.w_offset;
        const float x = __bfloat162float(__float2bfloat16(a[i] * rstd * wv * silu_f(z[i])));
        amax = fmaxf(amax, fabsf(x));
        h[k0 + i] = __float2bfloat16(x);
        if (p.out) p.out[static_cast<size_t>(m) * p.ldout + k0 + i] = __float2bfloat16(x);
      }
    }
  } else {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float x[8];
      if (MODE == kRowSiluMul) {
        float g[8], u[8];
        const int k = v * 8;
        const int kg = p.silu_pair ? ((k >> 7) << 8) + (k & 127) : k;
        const int ku = p.silu_pair ? kg + 128 : K + k;
        load8(p.a + static_cast<size_t>(m) * p.lda + kg, g);
        load8(p.a + static_cast<size_t>(m) * p.lda + ku, u);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = silu_f(g[i]) * u[i];
      } else if (MODE == kRowGateSig) {
        float a[8], b[8];
        load8(p.a + static_cast<size_t>(m) * p.lda + v * 8, a);
        load8(p.b + static_cast<size_t>(m) * p.ldb + v * 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = a[i] * sigmoid_f(b[i]);
      } else {
        load8(p.a + static_cast<size_t>(m) * p.lda + v * 8, x);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] = __bfloat162float(__float2bfloat16(x[i]));
        amax = fmaxf(amax, fabsf(x[i]));
      }
      store8(h + v * 8, x);
      if (p.out) store8(p.out + static_cast<size_t>(m) * p.ldout + v * 8, x);
    }
  }
  amax = block_reduce<true>(amax, red);  // its barriers also publish h to the whole block
  if (p.q) quant_store_row(h, K, m, p.M_pad, amax, p.q, p.scale, p.qfmt, p.q_sf, p.sf_m_tiles);
}

// Register-resident form of ADD_RMS / SILU_MUL / GATE_SIG / PLAIN (body in rowops_body.cuh): a
// thread owns whole 16-value chunks (the unit of the tiled int8 store) and keeps them in registers
// between the passes, so the kernel needs no dynamic shared memory and its CTAs fit beside a
// resident GEMM CTA: the GEMM that follows a row kernel is launched programmatically, gets resident
// while the row kernel runs and streams its first weight tiles meanwhile.  MAXC bounds the chunks
// per thread: K <= MAXC * 4096.
template <int MODE, int MAXC>
__global__ void __launch_bounds__(kRowThreads) row_reg_kernel(const RowOpParams p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int m = blockIdx.x;
  if (p.m_live != nullptr && m >= *p.m_live) return;
  row_reg_body<MODE, MAXC, false>(p, m, red);
}

// The same body for many rows (prefill rungs): as many threads as the row has 16-value chunks (over MAXC),
// so that every thread carries the same load and more bytes per SM are in flight.
template <int MODE, int MAXC>
__global__ void __launch_bounds__(1024) row_reg_wide_kernel(const RowOpParams p) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int m = blockIdx.x;
  if (p.m_live != nullptr && m >= *p.m_live) return;
  row_reg_body<MODE, MAXC, false>(p, m, red);
}

// out[m, :] = table[ids[m], :]   (bf16 rows, 16-byte vectors); ids outside [0, vocab) give zeros.
__global__ void embed_gather_kernel(const __nv_bfloat16* table, const int32_t* ids,
                                    __nv_bfloat16* out, int M, int H, int vocab_lo, int vocab_n,
                                    int ldout) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  if (m >= M) return;
  const int id = ids[m] - vocab_lo;
  const bool ok = id >= 0 && id < vocab_n;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(ok ? id : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * ldout);
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x)
    dst[v] = ok ? src[v] : make_uint4(0, 0, 0, 0);
}

// x[(b * block + j), :] = bf16(ctx[b, :] + tok[b, :] + pos[j, :])   (drafter block input rows)
__global__ void block_expand_kernel(const __nv_bfloat16* ctx, const __nv_bfloat16* tok,
                                    const __nv_bfloat16* pos, __nv_bfloat16* out, int block, int H) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, b = row / block, j = row % block;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
    float c[8], t[8], q[8];
    load8(ctx + static_cast<size_t>(b) * H + v * 8, c);
    load8(tok + static_cast<size_t>(b) * H + v * 8, t);
    load8(pos + static_cast<size_t>(j) * H + v * 8, q);
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] += t[i] + q[i];
    store8(out + static_cast<size_t>(row) * H + v * 8, c);
  }
}

}  // namespace saber

extern "C" int saber_block_expand_launch(const void* ctx, const void* tok, const void* pos, void* out,
                                         int nseq, int block, int H, cudaStream_t stream) {
  if (H & 7) return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(saber::block_expand_kernel, dim3(nseq * block), dim3(128), 0, stream, 0, 
      static_cast<const __nv_bfloat16*>(ctx), static_cast<const __nv_bfloat16*>(tok),
      static_cast<const __nv_bfloat16*>(pos), static_cast<__nv_bfloat16*>(out), block, H);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_row_producer_launch(int mode, const saber::RowOpParams* p, cudaStream_t stream) {
  using namespace saber;
  if ((p->K & 127) || p->M_pad < p->M) return static_cast<int>(cudaErrorInvalidValue);
  const int rows = p->q ? p->M_pad : p->M;
  // many rows (prefill): one thread per chunk (or per two), up to 1024 threads per row
#define SABER_ROW_WIDE(MODE, MAXC)                                                                       \
  if (mode == MODE && rows >= 256 && (p->K >> 4) <= MAXC * 1024 && (MAXC == 1 || (p->K >> 4) > 1024)) {   \
    const int threads = ((((p->K >> 4) + MAXC - 1) / MAXC) + 31) / 32 * 32;                              \
    saber::launch(row_reg_wide_kernel<MODE, MAXC>, dim3(rows), dim3(threads), 0, stream, 0, *p);         \
    return static_cast<int>(cudaGetLastError());                                                         \
  }
  SABER_ROW_WIDE(kRowAddRms, 1)
  SABER_ROW_WIDE(kRowSiluMul, 1)
  SABER_ROW_WIDE(kRowSiluMul, 2)
  SABER_ROW_WIDE(kRowGateSig, 1)
  SABER_ROW_WIDE(kRowPlain, 1)
#undef SABER_ROW_WIDE
  // register-resident forms (no dynamic shared memory) wherever the row fits the chunk budget
#define SABER_ROW_REG(MODE, MAXC)                                                                \
  if (mode == MODE && p->K <= MAXC * 4096) {                                                     \
    static bool carve = false;                                                                   \
    if (!carve) {   /* same shared-memory carve-out as the GEMM, so both can share an SM */      \
      cudaFuncSetAttribute(row_reg_kernel<MODE, MAXC>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                           cudaSharedmemCarveoutMaxShared);                                      \
      carve = true;                                                                              \
    }                                                                                            \
    saber::launch(row_reg_kernel<MODE, MAXC>, dim3(rows), dim3(kRowThreads), 0, stream, 0, *p);  \
    return static_cast<int>(cudaGetLastError());                                                 \
  }
  SABER_ROW_REG(kRowAddRms, 2)
  SABER_ROW_REG(kRowSiluMul, 2)
  SABER_ROW_REG(kRowSiluMul, 5)
  SABER_ROW_REG(kRowGateSig, 2)
  SABER_ROW_REG(kRowPlain, 2)
  SABER_ROW_REG(kRowPlain, 7)
#undef SABER_ROW_REG
  size_t smem = static_cast<size_t>(p->K) * 2 + (mode == kRowAddRms ? static_cast<size_t>(p->K) * 4 : 0);
#define SABER_ROW_CASE(MODE)                                                                     \
  case MODE: {                                                                                   \
    if (smem > 48 * 1024)                                                                        \
      cudaFuncSetAttribute(row_producer_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           static_cast<int>(smem));                                              \
    saber::launch(row_producer_kernel<MODE>, dim3(rows), dim3(kRowThreads), smem, stream, 0, *p);                          \
    break;                                                                                       \
  }
  switch (mode) {
    SABER_ROW_CASE(kRowAddRms)
    SABER_ROW_CASE(kRowSiluMul)
    SABER_ROW_CASE(kRowGateSig)
    SABER_ROW_CASE(kRowGdnNorm)
    SABER_ROW_CASE(kRowPlain)
    default:
      return static_cast<int>(cudaErrorInvalidValue);
  }
#undef SABER_ROW_CASE
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_embed_gather_launch(const void* table, const int32_t* ids, void* out, int M,
                                         int H, int vocab_lo, int vocab_n, int ldout,
                                         cudaStream_t stream) {
  if ((H & 7) || (ldout & 7)) return static_cast<int>(cudaErrorInvalidValue);
  if (ldout == 0) ldout = H;
  saber::launch(saber::embed_gather_kernel, dim3(M), dim3(128), 0, stream, 0, 
      static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), M, H,
      vocab_lo, vocab_n, ldout);
  return static_cast<int>(cudaGetLastError());
}
