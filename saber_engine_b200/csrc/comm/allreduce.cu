// One-shot all-reduce over peer memory (NVLink 5 / NVSwitch), 2..8 ranks, bf16 payload, fp32 sum in
// rank order (every rank adds the same values in the same order, so results are bit-identical
// across ranks).  Block b owns chunk b of the message end to end: push own chunk into every
// peer's receive slot, release a flag per peer, wait (bounded) for every peer's flag, reduce.
#include "../kernels/launch.cuh"
#include "comm.h"
#include <string.h>

namespace saber {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ar_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- race-check helpers (checked twin only)
__device__ __forceinline__ uint32_t chk_mix(uint32_t h) {
  h ^= h >> 15; h *= 0x2c1b3c6du; h ^= h >> 12; h *= 0x297a2d39u; h ^= h >> 15;
  return h;
}
// hash of one pushed 16-byte word, keyed by its position in the message and the call's sequence
__device__ __forceinline__ uint32_t chk_word16(const uint4& w, uint32_t pos, uint32_t seq) {
  uint32_t h = chk_mix(pos * 0x9e3779b9u + seq);
  h = chk_mix(h ^ w.x); h = chk_mix(h ^ w.y); h = chk_mix(h ^ w.z); h = chk_mix(h ^ w.w);
  return h;
}
__device__ __forceinline__ uint32_t block_xor(uint32_t v, uint32_t* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v ^= __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  uint32_t r = 0;
  for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) r ^= sh[i];
  return r;
}

// One block's share of the all-reduce.  kCheck = the checked twin: the pushes, the handshake, the
// reduce and the stores are the served code; the check words and counters ride beside them.
template <bool kCheck>
__device__ __forceinline__ void ar_body(const AllReduceParams& p, const int b) {
  __shared__ uint32_t xsh[17];   // 16 warp words of the block XOR + one decision word
  const int tid = threadIdx.x;
  const uint32_t seq = *p.seq_base + static_cast<uint32_t>(p.site) + 1u;
  const uint32_t par = seq & 1u;
  const int nvec = p.n_elems >> 3;
  const int per = (nvec + kArBlocks - 1) / kArBlocks;
  const int v0 = b * per, v1 = min(nvec, v0 + per);
  const uint4* src = reinterpret_cast<const uint4*>(p.in);
  const size_t slot_vecs = static_cast<size_t>(p.max_elems) >> 3;
  // check word of (slot, block): the slot's last kArBlocks words
  auto chk_at = [&](void* recv, int from_rank) -> uint32_t* {
    return reinterpret_cast<uint32_t*>(reinterpret_cast<uint4*>(recv) + (par * p.nranks + from_rank + 1) * slot_vecs) - kArBlocks + b;
  };

  // push
  uint32_t hx = 0;
  for (int peer = 0; peer < p.nranks; ++peer) {
    if (peer == p.rank) continue;
    uint4* dst = reinterpret_cast<uint4*>(p.peer_recv[peer]) + (par * p.nranks + p.rank) * slot_vecs;
    for (int v = v0 + tid; v < v1; v += blockDim.x) dst[v] = src[v];
  }
  if constexpr (kCheck) {
    for (int v = v0 + tid; v < v1; v += blockDim.x) hx ^= chk_word16(src[v], static_cast<uint32_t>(v), seq);
    hx = block_xor(hx, xsh);
    if (tid < p.nranks && tid != p.rank && !p.chk_fault) *chk_at(p.peer_recv[tid], p.rank) = hx;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.nranks && tid != p.rank)
    st_release_sys(p.peer_flags[tid] + (par * p.nranks + p.rank) * kArBlocks + b, seq);

  // wait (bounded): flag of peer `tid` in this rank's own region
  if (tid < p.nranks && tid != p.rank) {
    const uint32_t* f = p.peer_flags[p.rank] + (par * p.nranks + tid) * kArBlocks + b;
    const unsigned long long limit =
        (p.spin_limit_us ? static_cast<unsigned long long>(p.spin_limit_us) : 1000000ull) * 1000ull;
    const unsigned long long t0 = ar_now_ns();
    bool timed_out = false;
    while (static_cast<int32_t>(ld_acquire_sys(f) - seq) < 0) {
      if (ar_now_ns() - t0 > limit) {
        atomicCAS(p.err, 0u, 5u);
        timed_out = true;
        break;
      }
    }
    if constexpr (kCheck) {
      if (timed_out) {
        atomicAdd(p.diag + kArDTimeout, 1u);
      } else {
        const uint32_t now = ld_acquire_sys(f);      // lockstep: == seq; the peer already in the next call of this parity: ahead
        if (now != seq) atomicAdd(p.diag + (static_cast<int32_t>(now - seq) > 0 ? kArDAhead : kArDDrift), 1u);
      }
    }
  }
  __syncthreads();

  // reduce in rank order
  const uint4* own_recv = reinterpret_cast<const uint4*>(p.peer_recv[p.rank]);
  uint4* dst = reinterpret_cast<uint4*>(p.out);
  uint32_t hr[kMaxRanks];
#pragma unroll
  for (int s = 0; s < kMaxRanks; ++s) hr[s] = 0;
  for (int v = v0 + tid; v < v1; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s) {
      if (s >= p.nranks) break;
      const uint4 raw = (s == p.rank) ? src[v] : __ldcg(own_recv + (par * p.nranks + s) * slot_vecs + v);
      if constexpr (kCheck) {
        if (s != p.rank) hr[s] ^= chk_word16(raw, static_cast<uint32_t>(v), seq);
      }
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    dst[v] = o;
  }
  if constexpr (kCheck) {
    if (tid == 0) {
      atomicAdd(p.diag + kArDBlocks, 1u);
      if (b == 0) p.diag[kArDLastSeq] = seq;
    }
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s) {
      if (s >= p.nranks) break;
      if (s == p.rank) continue;
      const uint32_t got = block_xor(hr[s], xsh);
      const uint32_t* cw = chk_at(p.peer_recv[p.rank], s);
      // ONE thread reads the check word and decides for the block (the word may still be changing:
      // every thread reading it for itself could split the block across the barriers below)
      __syncthreads();
      if (tid == 0) xsh[16] = (got == ld_acquire_sys(cw)) ? 1u : 0u;
      __syncthreads();
      if (xsh[16]) continue;
      if (tid == 0) {
        if (atomicAdd(p.diag + kArDMismatch, 1u) == 0u) {
          p.diag[kArDFirstSeq] = seq; p.diag[kArDFirstBlock] = b; p.diag[kArDFirstSrc] = s;
        }
      }
      // diagnostic re-read at system scope: the reduce already used the first read
      uint32_t conv = 0;
      int polls = 0;
      for (; polls < kArProbeMax && !conv; ++polls) {
        __nanosleep(200);
        uint32_t h2 = 0;
        for (int v = v0 + tid; v < v1; v += blockDim.x) {
          uint4 w;
          const uint4* a = own_recv + (par * p.nranks + s) * slot_vecs + v;
          asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(a) : "memory");
          h2 ^= chk_word16(w, static_cast<uint32_t>(v), seq);
        }
        h2 = block_xor(h2, xsh);
        __syncthreads();
        if (tid == 0) xsh[16] = (h2 == ld_acquire_sys(cw)) ? 1u : 0u;
        __syncthreads();
        conv = xsh[16];
      }
      if (tid == 0) {
        atomicAdd(p.diag + (conv ? kArDConverged : kArDNever), 1u);
        atomicMax(p.diag + kArDPolls, static_cast<uint32_t>(polls));
      }
    }
  }
}

__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const AllReduceParams p) {
  pdl_wait();
  ar_body<false>(p, blockIdx.x);
}

// the checked twin: the served body with the race checks around it
__global__ void __launch_bounds__(512) allreduce_oneshot_chk_kernel(const AllReduceParams p) {
  pdl_wait();
  ar_body<true>(p, blockIdx.x);
}

// Test form for a one-device group: block (rank, b) runs rank's share, all ranks in ONE cooperative
// launch (blocks that wait on one another must be resident together).
__global__ void __launch_bounds__(512) allreduce_emul_kernel(const __grid_constant__ ArEmulParams e) {
  const int r = blockIdx.x / kArBlocks, b = blockIdx.x % kArBlocks;
  if (e.checked) ar_body<true>(e.r[r], b);
  else ar_body<false>(e.r[r], b);
}

__global__ void __launch_bounds__(1024) pick_merge_kernel(const PickMergeParams p) {
  pdl_wait();
  const int tid = threadIdx.x;
  const uint32_t seq = *p.seq_base + static_cast<uint32_t>(p.site) + 1u;
  const uint32_t par = seq & 1u;
  const size_t slot = (static_cast<size_t>(par) * p.nranks + p.rank) * p.rows_max;
  for (int r = tid; r < p.rows; r += blockDim.x) {
    const unsigned long long w = (static_cast<unsigned long long>(__float_as_uint(p.val[r])) << 32) |
                                 static_cast<uint32_t>(p.idx[r]);
    for (int peer = 0; peer < p.nranks; ++peer)
      if (peer != p.rank) static_cast<unsigned long long*>(p.peer_win[peer])[slot + r] = w;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.nranks && tid != p.rank) {
    st_release_sys(p.peer_flags[tid] + par * p.nranks + p.rank, seq);
    const uint32_t* f = p.peer_flags[p.rank] + par * p.nranks + tid;
    const unsigned long long t0 = ar_now_ns();
    while (static_cast<int32_t>(ld_acquire_sys(f) - seq) < 0) {
      if (ar_now_ns() - t0 > 1000000000ull) { atomicCAS(p.err, 0u, 5u); break; }
    }
  }
  __syncthreads();
  const unsigned long long* win = static_cast<const unsigned long long*>(p.peer_win[p.rank]);
  for (int r = tid; r < p.rows; r += blockDim.x) {
    float bv = p.val[r];
    int bi = p.idx[r];
    for (int src = 0; src < p.nranks; ++src) {
      if (src == p.rank) continue;
      const unsigned long long w = __ldcg(win + (static_cast<size_t>(par) * p.nranks + src) * p.rows_max + r);
      const float v = __uint_as_float(static_cast<uint32_t>(w >> 32));
      const int i = static_cast<int>(static_cast<uint32_t>(w));
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    p.val[r] = bv;
    p.idx[r] = bi;
  }
}

// One CTA of 1024 threads per rank.  Push this rank's rows to every peer, raise a flag per peer, wait
// (bounded) for every peer's flag, then merge: 64 x nranks candidates per row, rank by counting (a
// candidate's place = how many beat it: larger value, or equal value and smaller id).
__device__ __forceinline__ void seam_merge_body(const SeamMergeParams& p) {
  __shared__ float cv[kMaxRanks * 64];
  __shared__ int ci[kMaxRanks * 64];
  const int tid = threadIdx.x;
  const uint32_t seq = *p.seq_base + static_cast<uint32_t>(p.site) + 1u;
  const uint32_t par = seq & 1u;
  const size_t slot_words = static_cast<size_t>(p.rows_max) * kSeamWords;
  for (int peer = 0; peer < p.nranks; ++peer) {
    if (peer == p.rank) continue;
    uint32_t* dst = static_cast<uint32_t*>(p.peer_win[peer]) + (par * p.nranks + p.rank) * slot_words;
    for (int i = tid; i < p.rows * kSeamWords; i += blockDim.x) {
      const int r = i / kSeamWords, w = i - r * kSeamWords;
      uint32_t v;
      if (w < 64) v = static_cast<uint32_t>(p.ids[r * 64 + w]);
      else if (w < 128) v = __float_as_uint(p.vals[r * 64 + (w - 64)]);
      else v = __float_as_uint(p.lse[r * 2 + (w - 128)]);
      dst[i] = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.nranks && tid != p.rank) {
    st_release_sys(p.peer_flags[tid] + par * p.nranks + p.rank, seq);
    const uint32_t* f = p.peer_flags[p.rank] + par * p.nranks + tid;
    const unsigned long long t0 = ar_now_ns();
    while (static_cast<int32_t>(ld_acquire_sys(f) - seq) < 0) {
      if (ar_now_ns() - t0 > 1000000000ull) { atomicCAS(p.err, 0u, 5u); break; }
    }
  }
  __syncthreads();
  const uint32_t* win = static_cast<const uint32_t*>(p.peer_win[p.rank]) + par * p.nranks * slot_words;
  const int ncand = p.nranks * 64;
  for (int r = 0; r < p.rows; ++r) {
    for (int c = tid; c < ncand; c += blockDim.x) {
      const int src = c >> 6, j = c & 63;
      if (src == p.rank) {
        cv[c] = p.vals[r * 64 + j];
        ci[c] = p.ids[r * 64 + j];
      } else {
        const uint32_t* w = win + src * slot_words + static_cast<size_t>(r) * kSeamWords;
        ci[c] = static_cast<int>(__ldcg(w + j));
        cv[c] = __uint_as_float(__ldcg(w + 64 + j));
      }
    }
    float l1 = 0.f, lT = 0.f;
    if (tid == 0) {                  // the two log-sum-exps of the whole row, ranks in order
      float m1 = -INFINITY, mT = -INFINITY;
      for (int s2 = 0; s2 < p.nranks; ++s2) {
        const float a = s2 == p.rank ? p.lse[r * 2] : __uint_as_float(__ldcg(win + s2 * slot_words + static_cast<size_t>(r) * kSeamWords + 128));
        const float b = s2 == p.rank ? p.lse[r * 2 + 1] : __uint_as_float(__ldcg(win + s2 * slot_words + static_cast<size_t>(r) * kSeamWords + 129));
        m1 = fmaxf(m1, a);
        mT = fmaxf(mT, b);
      }
      float a1 = 0.f, aT = 0.f;
      for (int s2 = 0; s2 < p.nranks; ++s2) {
        const float a = s2 == p.rank ? p.lse[r * 2] : __uint_as_float(__ldcg(win + s2 * slot_words + static_cast<size_t>(r) * kSeamWords + 128));
        const float b = s2 == p.rank ? p.lse[r * 2 + 1] : __uint_as_float(__ldcg(win + s2 * slot_words + static_cast<size_t>(r) * kSeamWords + 129));
        a1 += expf(a - m1);
        aT += expf(b - mT);
      }
      l1 = m1 + logf(a1);
      lT = mT + logf(aT);
    }
    __syncthreads();                 // candidates staged; every thread has read this row's local values
    for (int c = tid; c < ncand; c += blockDim.x) {
      const float v = cv[c];
      const int id = ci[c];
      int place = 0;
      for (int o = 0; o < ncand; ++o) {
        const float ov = cv[o];
        const int oi = ci[o];
        place += (ov > v || (ov == v && oi < id)) ? 1 : 0;
      }
      if (place < 64) {
        p.vals[r * 64 + place] = v;
        p.ids[r * 64 + place] = id;
      }
    }
    if (tid == 0) { p.lse[r * 2] = l1; p.lse[r * 2 + 1] = lT; }
    __syncthreads();                 // before the next row overwrites the staging arrays
  }
}

__global__ void __launch_bounds__(1024) seam_merge_kernel(const SeamMergeParams p) {
  pdl_wait();
  seam_merge_body(p);
}
__global__ void __launch_bounds__(1024) seam_merge_emul_kernel(const __grid_constant__ SeamEmulParams e) {
  seam_merge_body(e.r[blockIdx.x]);
}

__global__ void comm_advance_kernel(uint32_t* seq_base, uint32_t by) {
  pdl_wait();
  *seq_base += by;
}

}  // namespace saber

extern "C" int saber_allreduce_launch(const saber::AllReduceParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->nranks < 1 || p->nranks > kMaxRanks || (p->n_elems & 7) || p->n_elems > p->max_elems)
    return static_cast<int>(cudaErrorInvalidValue);
  if (p->nranks == 1) {
    if (p->out != p->in)
      return static_cast<int>(cudaMemcpyAsync(p->out, p->in, static_cast<size_t>(p->n_elems) * 2,
                                              cudaMemcpyDeviceToDevice, stream));
    return 0;
  }
  saber::launch(allreduce_oneshot_kernel, dim3(kArBlocks), dim3(512), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_allreduce_chk_launch(const saber::AllReduceParams* p, cudaStream_t stream) {
  using namespace saber;
  // a checked message leaves the slot's last kArBlocks words (16 bf16 each pair of words) to the check words
  if (p->nranks < 2 || p->nranks > kMaxRanks || (p->n_elems & 7) || p->n_elems > p->max_elems - 2 * kArBlocks || !p->diag)
    return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(allreduce_oneshot_chk_kernel, dim3(kArBlocks), dim3(512), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_allreduce_emul_launch(const saber::ArEmulParams* e, cudaStream_t stream) {
  using namespace saber;
  if (e->nranks < 2 || e->nranks > kMaxRanks) return static_cast<int>(cudaErrorInvalidValue);
  for (int r = 0; r < e->nranks; ++r) {
    const AllReduceParams& p = e->r[r];
    if ((p.n_elems & 7) || p.n_elems > p.max_elems - (e->checked ? 2 * kArBlocks : 0) || (e->checked && !p.diag))
      return static_cast<int>(cudaErrorInvalidValue);
  }
  // every block of every rank must be resident: refuse a device that cannot hold the grid at once
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_emul_kernel, 512, 0);
  if (sms * per_sm < e->nranks * kArBlocks) return static_cast<int>(cudaErrorCooperativeLaunchTooLarge);
  saber::launch(allreduce_emul_kernel, dim3(e->nranks * kArBlocks), dim3(512), 0, stream, 1, *e);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_pick_merge_launch(const saber::PickMergeParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->nranks < 1 || p->nranks > kMaxRanks || p->rows > p->rows_max) return static_cast<int>(cudaErrorInvalidValue);
  if (p->nranks == 1) return 0;
  saber::launch(pick_merge_kernel, dim3(1), dim3(1024), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_seam_merge_launch(const saber::SeamMergeParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->nranks < 1 || p->nranks > kMaxRanks || p->rows > p->rows_max) return static_cast<int>(cudaErrorInvalidValue);
  if (p->nranks == 1) return 0;
  saber::launch(seam_merge_kernel, dim3(1), dim3(1024), 0, stream, 0, *p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_seam_merge_emul_launch(const saber::SeamEmulParams* e, cudaStream_t stream) {
  using namespace saber;
  if (e->nranks < 2 || e->nranks > kMaxRanks) return static_cast<int>(cudaErrorInvalidValue);
  for (int r = 0; r < e->nranks; ++r)
    if (e->r[r].rows > e->r[r].rows_max) return static_cast<int>(cudaErrorInvalidValue);
  saber::launch(seam_merge_emul_kernel, dim3(e->nranks), dim3(1024), 0, stream, 1, *e);   // cooperative: the blocks wait on one another
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_comm_advance_launch(uint32_t* seq_base, uint32_t by, cudaStream_t stream) {
  saber::launch(saber::comm_advance_kernel, dim3(1), dim3(1), 0, stream, 0, seq_base, by);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_ipc_get_handle(void* dev_ptr, void* out_handle_64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
  memcpy(out_handle_64, &h, 64);
  return 0;
}
extern "C" int saber_ipc_open_handle(const void* handle_64, void** out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int saber_ipc_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
extern "C" int saber_dev_malloc(void** out, size_t bytes) {
  return static_cast<int>(cudaMalloc(out, bytes));
}
extern "C" int saber_dev_free(void* p) { return static_cast<int>(cudaFree(p)); }
extern "C" int saber_dev_memset(void* p, int value, size_t bytes) {
  cudaError_t e = cudaMemset(p, value, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaDeviceSynchronize());
}
extern "C" int saber_dev_read_u32(const void* p, uint32_t* out) {
  return static_cast<int>(cudaMemcpy(out, p, 4, cudaMemcpyDeviceToHost));
}
