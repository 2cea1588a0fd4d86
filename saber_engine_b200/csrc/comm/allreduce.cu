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

__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const AllReduceParams p) {
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const uint32_t seq = *p.seq_base + static_cast<uint32_t>(p.site) + 1u;
  const uint32_t par = seq & 1u;
  const int nvec = p.n_elems >> 3;
  const int per = (nvec + kArBlocks - 1) / kArBlocks;
  const int v0 = b * per, v1 = min(nvec, v0 + per);
  const uint4* src = reinterpret_cast<const uint4*>(p.in);
  const size_t slot_vecs = static_cast<size_t>(p.max_elems) >> 3;

  // push
  for (int peer = 0; peer < p.nranks; ++peer) {
    if (peer == p.rank) continue;
    uint4* dst = reinterpret_cast<uint4*>(p.peer_recv[peer]) + (par * p.nranks + p.rank) * slot_vecs;
    for (int v = v0 + tid; v < v1; v += blockDim.x) dst[v] = src[v];
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
    while (static_cast<int32_t>(ld_acquire_sys(f) - seq) < 0) {
      if (ar_now_ns() - t0 > limit) {
        atomicCAS(p.err, 0u, 5u);
        break;
      }
    }
  }
  __syncthreads();

  // reduce in rank order
  const uint4* own_recv = reinterpret_cast<const uint4*>(p.peer_recv[p.rank]);
  uint4* dst = reinterpret_cast<uint4*>(p.out);
  for (int v = v0 + tid; v < v1; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < p.nranks; ++s) {
      const uint4 raw = (s == p.rank) ? src[v] : __ldcg(own_recv + (par * p.nranks + s) * slot_vecs + v);
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

extern "C" int saber_pick_merge_launch(const saber::PickMergeParams* p, cudaStream_t stream) {
  using namespace saber;
  if (p->nranks < 1 || p->nranks > kMaxRanks || p->rows > p->rows_max) return static_cast<int>(cudaErrorInvalidValue);
  if (p->nranks == 1) return 0;
  saber::launch(pick_merge_kernel, dim3(1), dim3(1024), 0, stream, 0, *p);
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
