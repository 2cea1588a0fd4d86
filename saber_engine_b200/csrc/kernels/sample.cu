// Head-side kernels: argmax over a vocab shard, the top-64 "seam" row (top-k candidates + two
// log-sum-exps) that lets the sampler work on 520 bytes instead of a full logits row, and the
// speculative verify/accept step.
//
// Parity: argmax ordering (value descending, id ascending, NaN never wins) and the seam row are
// the laws of crates/saber-kernels/hip/head.hip:116-145; greedy prefix acceptance is
// crates/saber-exec/src/forward.rs:475 (accept_prefix); the seeded acceptance oracle mirrors the
// reference's RandomAcceptanceExecutor (crates/saber-sched/src/mock.rs:1-20) on the device.
#include "launch.cuh"
#include "sample.h"
#include <cuda_bf16.h>
#include <math.h>

namespace saber {

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// grid = rows, block 1024. out_idx[r] = argmax (global id = local + id_offset), out_val[r] = value.
__global__ void __launch_bounds__(1024) argmax_kernel(const __nv_bfloat16* logits, int ld, int V,
                                                      int id_offset, int32_t* out_idx,
                                                      float* out_val) {
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int r = blockIdx.x;
  const __nv_bfloat16* row = logits + static_cast<size_t>(r) * ld;
  float bv = -INFINITY;
  int bi = V;  // "cols" when nothing finite/non-NaN was seen
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      if (f.x == f.x && better(f.x, v * 8 + 2 * i, bv, bi)) { bv = f.x; bi = v * 8 + 2 * i; }
      if (f.y == f.y && better(f.y, v * 8 + 2 * i + 1, bv, bi)) { bv = f.y; bi = v * 8 + 2 * i + 1; }
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float f = __bfloat162float(row[i]);
    if (f == f && better(f, i, bv, bi)) { bv = f; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? si[lane] : V;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      out_idx[r] = bi + id_offset;
      if (out_val) out_val[r] = bv;
    }
  }
}

// ------------------------------------------------------------------------------- top-k seam
// Order-preserving 16-bit key of a bf16 value (larger key = larger value; NaN sorts lowest).
__device__ __forceinline__ uint32_t bf16_key(uint16_t bits) {
  if ((bits & 0x7FFFu) > 0x7F80u) return 0u;  // NaN
  return (bits & 0x8000u) ? (0xFFFFu ^ bits) & 0xFFFFu : (bits | 0x8000u);
}

// grid = rows, block 1024. Writes per row: ids[kSeamK], vals[kSeamK] (sorted: value desc, id asc),
// lse[2] = log-sum-exp at temperature 1 and at temperature temps[r].
__global__ void __launch_bounds__(1024) topk_seam_kernel(const __nv_bfloat16* logits, int ld, int V,
                                                         int id_offset, const float* temps,
                                                         int32_t* ids, float* vals, float* lse) {
  pdl_wait();
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sel_hi, sel_lo, above_hi, above_lo;
  __shared__ float cand_v[kSeamK];
  __shared__ int cand_i[kSeamK];
  __shared__ uint32_t n_cand, n_tie;
  __shared__ int tie_i[256];
  __shared__ float red[64];
  const int r = blockIdx.x;
  const uint16_t* row = reinterpret_cast<const uint16_t*>(logits + static_cast<size_t>(r) * ld);
  const int tid = threadIdx.x;

  // pass 1: histogram of the high byte of the key, row max for the lse
  if (tid < 256) hist[tid] = 0;
  __syncthreads();
  float mx = -INFINITY;
  for (int i = tid; i < V; i += blockDim.x) {
    const uint16_t bits = row[i];
    atomicAdd(&hist[bf16_key(bits) >> 8], 1u);
    const float f = __bfloat162float(__ushort_as_bfloat16(bits));
    if (f == f) mx = fmaxf(mx, f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  if (tid == 0) {
    uint32_t acc = 0;
    int bin = 255;
    for (; bin > 0; --bin) {
      if (acc + hist[bin] >= kSeamK) break;
      acc += hist[bin];
    }
    sel_hi = bin;
    above_hi = acc;  // elements strictly above the selected high bin
  }
  mx = red[0];
  for (int w = 1; w < 32; ++w) mx = fmaxf(mx, red[w]);   // row maximum, same in every thread
  __syncthreads();
  const uint32_t hi = sel_hi;
  const uint32_t above1 = above_hi;
  __syncthreads();
  if (tid < 256) hist[tid] = 0;
  __syncthreads();
  // pass 2: histogram of the low byte inside the selected high bin
  for (int i = tid; i < V; i += blockDim.x) {
    const uint32_t k = bf16_key(row[i]);
    if ((k >> 8) == hi) atomicAdd(&hist[k & 255u], 1u);
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t acc = above1;
    int bin = 255;
    for (; bin > 0; --bin) {
      if (acc + hist[bin] >= kSeamK) break;
      acc += hist[bin];
    }
    sel_lo = bin;
    above_lo = acc;  // elements with key strictly above the threshold key
    n_cand = 0;
    n_tie = 0;
  }
  __syncthreads();
  const uint32_t thr = (hi << 8) | sel_lo;
  const uint32_t n_above = above_lo;
  // pass 3: collect everything above the threshold key; ties at the threshold by ascending id
  float s1 = 0.f, sT = 0.f;
  const float invT = temps ? 1.f / fmaxf(temps[r], 1e-6f) : 1.f;
  const float mxs = mx == -INFINITY ? 0.f : mx;
  for (int i = tid; i < V; i += blockDim.x) {
    const uint16_t bits = row[i];
    const uint32_t k = bf16_key(bits);
    const float f = __bfloat162float(__ushort_as_bfloat16(bits));
    if (f == f) {
      s1 += __expf(f - mxs);
      sT += __expf((f - mxs) * invT);
    }
    if (k > thr) {
      const uint32_t slot = atomicAdd(&n_cand, 1u);
      if (slot < kSeamK) { cand_v[slot] = f; cand_i[slot] = i; }
    } else if (k == thr) {
      const uint32_t slot = atomicAdd(&n_tie, 1u);
      if (slot < 256) tie_i[slot] = i;
    }
  }
  // block sums for the two log-sum-exps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    sT += __shfl_xor_sync(0xffffffffu, sT, o);
  }
  if ((tid & 31) == 0) { red[tid >> 5] = s1; red[32 + (tid >> 5)] = sT; }
  __syncthreads();
  if (tid == 0) {
    float a = 0.f, bsum = 0.f;
    for (int w = 0; w < 32; ++w) { a += red[w]; bsum += red[32 + w]; }
    lse[r * 2] = mxs + logf(a);
    lse[r * 2 + 1] = mxs * invT + logf(bsum);
    // ties: take the lowest ids (at most 256 ties are remembered; a row with more than 256 equal
    // threshold values keeps an arbitrary 256 of them, lowest ids among those)
    const int need = kSeamK - static_cast<int>(n_above);
    const int nt = min(static_cast<int>(n_tie), 256);
    const float tv = __bfloat162float(__ushort_as_bfloat16(
        static_cast<uint16_t>((thr & 0x8000u) ? (thr & 0x7FFFu) : (0xFFFFu ^ thr))));
    for (int j = 0; j < need; ++j) {
      int best = -1;
      for (int q = 0; q < nt; ++q)
        if (tie_i[q] >= 0 && (best < 0 || tie_i[q] < tie_i[best])) best = q;
      const int slot = static_cast<int>(n_above) + j;
      if (best >= 0) { cand_v[slot] = tv; cand_i[slot] = tie_i[best]; tie_i[best] = -1; }
      else { cand_v[slot] = -INFINITY; cand_i[slot] = V; }
    }
  }
  __syncthreads();
  // sort the kSeamK candidates: value desc, id asc (rank by counting)
  if (tid < kSeamK) {
    const float v = cand_v[tid];
    const int id = cand_i[tid];
    int rank = 0;
    for (int j = 0; j < kSeamK; ++j)
      if (j != tid && better(cand_v[j], cand_i[j], v, id)) ++rank;
    ids[r * kSeamK + rank] = id + id_offset;
    vals[r * kSeamK + rank] = v;
  }
}

// ------------------------------------------------------------------------------- verify / accept
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// One thread per sequence. rows of sequence b are [cu[b], cu[b+1]); row 0 carries the last committed
// token, rows 1.. carry the draft.  target[r] is the model's pick after row r.
//   greedy:  a = longest prefix with draft[r + 1] == target[r]
//   oracle:  a = min(w - 1, G) with G ~ geometric(p_accept) drawn from (seed, seq uid, step)
// Outputs: n_commit[b] = a + 1; out_tokens[b][0..a) = accepted drafts, out_tokens[b][a] = bonus.
__global__ void verify_accept_kernel(const VerifyParams p) {
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= p.nseq) return;
  const int r0 = p.cu_rows[b];
  const int w = p.cu_rows[b + 1] - r0;
  if (w <= 0) {
    p.n_commit[b] = 0;
    if (p.accept_row) p.accept_row[b] = 0;
    if (p.bonus) p.bonus[b] = 0;
    return;
  }
  int a = 0;
  if (p.oracle_p > 0.f) {
    const uint64_t h = splitmix64(p.seed ^ splitmix64(static_cast<uint64_t>(p.seq_uid[b]) * 0x100000001B3ull +
                                                      static_cast<uint64_t>(p.step_no[b])));
    const double u = (static_cast<double>(h >> 11) + 0.5) * (1.0 / 9007199254740992.0);
    // P(G >= k) = p^k  =>  G = floor(log(u) / log(p))
    const int gcount = static_cast<int>(floor(log(u) / log(static_cast<double>(p.oracle_p))));
    a = min(w - 1, max(0, gcount));
  } else {
    while (a < w - 1 && p.draft[r0 + a + 1] == p.target[r0 + a]) ++a;
  }
  for (int j = 0; j < a; ++j) p.out_tokens[b * p.max_w + j] = p.draft[r0 + j + 1];
  p.out_tokens[b * p.max_w + a] = p.target[r0 + a];
  p.n_commit[b] = a + 1;
  if (p.accept_row) p.accept_row[b] = r0 + a;
  if (p.bonus) p.bonus[b] = p.target[r0 + a];
}

}  // namespace saber

extern "C" int saber_argmax_launch(const void* logits, int rows, int ld, int V, int id_offset,
                                   int32_t* out_idx, float* out_val, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (ld & 7) return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(saber::argmax_kernel, dim3(rows), dim3(1024), 0, stream, 0, static_cast<const __nv_bfloat16*>(logits), ld, V,
                                                  id_offset, out_idx, out_val);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_topk_seam_launch(const void* logits, int rows, int ld, int V, int id_offset,
                                      const float* temps, int32_t* ids, float* vals, float* lse,
                                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (V < saber::kSeamK) return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(saber::topk_seam_kernel, dim3(rows), dim3(1024), 0, stream, 0, static_cast<const __nv_bfloat16*>(logits), ld,
                                                     V, id_offset, temps, ids, vals, lse);
  return static_cast<int>(cudaGetLastError());
}

namespace saber {
// out[m] = logits[m][ids[m] - id_offset] as fp32, or -inf when ids[m] lies outside [id_offset, id_offset + V)
// (a row without a successor carries -1).  One thread per row.
__global__ void logit_gather_kernel(const __nv_bfloat16* logits, int ld, int V, int id_offset,
                                    const int32_t* ids, float* out, int rows) {
  pdl_wait();
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= rows) return;
  const int id = ids[m] - id_offset;
  out[m] = (id >= 0 && id < V) ? __bfloat162float(logits[static_cast<size_t>(m) * ld + id]) : -INFINITY;
}
}  // namespace saber

namespace saber {
// Device draw for sampled rows.  The row's 64 candidates arrive sorted (value descending); with
// temperature T the probabilities are softmax(v / T) over the candidates, cut by min-p, top-k and
// top-p in that order (at least one stays), renormalised, and the uniform number u[m] (drawn on the
// host as a function of seed and position) picks the token.  Rows with T <= 0 keep their greedy pick.
// samp: [rows][4] = {T, top_k, top_p, min_p}.  One thread per row.
__global__ void sample_seam_kernel(const int32_t* ids, const float* vals, const float* samp, const float* u,
                                   int32_t* picks, int rows) {
  pdl_wait();
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= rows) return;
  const float T = samp[4 * m];
  if (!(T > 0.f)) return;
  const int top_k = static_cast<int>(samp[4 * m + 1]);
  const float top_p = samp[4 * m + 2], min_p = samp[4 * m + 3];
  const float* v = vals + static_cast<size_t>(m) * kSeamK;
  const int32_t* id = ids + static_cast<size_t>(m) * kSeamK;
  const float inv_t = 1.f / fmaxf(T, 1e-6f), m0 = v[0] * inv_t;
  float z = 0.f;
  for (int j = 0; j < kSeamK; ++j) z += expf(v[j] * inv_t - m0);
  int keep = kSeamK;
  if (min_p > 0.f) {              // p_j >= min_p * p_0  <=>  e_j >= min_p  (e_0 = 1)
    int c = 0;
    for (int j = 0; j < kSeamK; ++j) c += expf(v[j] * inv_t - m0) >= min_p ? 1 : 0;
    keep = min(keep, c);
  }
  if (top_k > 0) keep = min(keep, top_k);
  if (top_p < 1.f) {
    float acc = 0.f;
    int k = 0;
    for (int j = 0; j < keep; ++j) {
      acc += expf(v[j] * inv_t - m0) / z;
      ++k;
      if (acc >= top_p) break;
    }
    keep = min(keep, k);
  }
  keep = max(1, keep);
  float z2 = 0.f;
  for (int j = 0; j < keep; ++j) z2 += expf(v[j] * inv_t - m0) / z;
  const float x = u[m] * z2;
  float acc = 0.f;
  int pick = id[keep - 1];
  for (int j = 0; j < keep; ++j) {
    acc += expf(v[j] * inv_t - m0) / z;
    if (x < acc) { pick = id[j]; break; }
  }
  picks[m] = pick;
}
}  // namespace saber

extern "C" int saber_sample_seam_launch(const int32_t* ids, const float* vals, const float* samp, const float* u,
                                        int32_t* picks, int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  saber::launch(saber::sample_seam_kernel, dim3((rows + 63) / 64), dim3(64), 0, stream, 0, ids, vals, samp, u, picks, rows);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_logit_gather_launch(const void* logits, int rows, int ld, int V, int id_offset,
                                         const int32_t* ids, float* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  saber::launch(saber::logit_gather_kernel, dim3((rows + 127) / 128), dim3(128), 0, stream, 0,
                static_cast<const __nv_bfloat16*>(logits), ld, V, id_offset, ids, out, rows);
  return static_cast<int>(cudaGetLastError());
}

namespace saber {
// one thread per block row
__global__ void draft_index_kernel(const DraftIndexParams p) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int R = p.nseq * p.block;
  if (i >= R) return;
  const int b = i / p.block, j = i - b * p.block;
  const int rows = p.cu_rows[b + 1] - p.cu_rows[b];
  const int r = p.acc_row[b];
  const bool live = rows > 0 && r >= p.cu_rows[b] && r < p.cu_rows[b + 1];
  // sequence index of the committed row: the step's rows end at kv_len - 1
  const int at = live ? p.kv_len[b] - (p.cu_rows[b + 1] - r) : 0;
  const int t = at + 1 + j;
#pragma unroll
  for (int ax = 0; ax < 3; ++ax) p.pos_out[ax * R + i] = live ? p.pos[ax * p.M + r] + 1 + j : 0;
  int slot = -1;
  if (live && t / p.page_tokens < p.max_blocks) {
    const int blk = p.block_table[static_cast<size_t>(b) * p.max_blocks + t / p.page_tokens];
    if (blk > 0) slot = blk * p.page_tokens + t % p.page_tokens;      // block 0 is the null page
  }
  p.slot_out[i] = slot;
  if (j == 0) p.kv_len_out[b] = live ? at + 1 + p.block : 0;
}
}  // namespace saber

extern "C" int saber_draft_index_launch(const saber::DraftIndexParams* p, cudaStream_t stream) {
  const int R = p->nseq * p->block;
  if (R <= 0) return 0;
  saber::launch(saber::draft_index_kernel, dim3((R + 127) / 128), dim3(128), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_verify_launch(const saber::VerifyParams* p, cudaStream_t stream) {
  if (p->nseq <= 0) return 0;
  saber::launch(saber::verify_accept_kernel, dim3((p->nseq + 63) / 64), dim3(64), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}
