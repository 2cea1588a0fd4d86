// Order-free digest of a device buffer: XOR over all 8-byte words of splitmix64(word ^ mix(index)).
// XOR is commutative, so the digest does not depend on which block or thread gets to which word
// first; it does depend on every word's value AND position.  Enqueued right after a stage inside the
// step program, it records what the stage left in memory at that point of the stream: a kernel
// that raced with its producer, or read a slot a step too early, changes the digest while the
// final tokens may still look plausible.  The digests ride back with the step's result: no extra
// synchronisation.
//
// Parity: crates/saber-kernels/hip/race_digest.hip:1-26 (on-device order-free XOR-splitmix digest of
// every stage, read with the tokens) and crates/saber-engine/src/device/shadow.rs:1-15.
#include "launch.cuh"
#include <cuda_runtime.h>
#include <stdint.h>

namespace saber {

__host__ __device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// grid-stride over 8-byte words; `out` must be zero before the launch (the kernel XORs into it).
__global__ void __launch_bounds__(256) digest_kernel(const uint64_t* __restrict__ buf, size_t n_words,
                                                     unsigned long long* __restrict__ out) {
  pdl_wait();
  uint64_t acc = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_words;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    acc ^= splitmix64(buf[i] ^ splitmix64(i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc ^= __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ uint64_t red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint64_t v = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) v ^= red[w];
    atomicXor(out, static_cast<unsigned long long>(v));
  }
}

__global__ void digest_clear_kernel(unsigned long long* out, int n) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = 0ull;
}

}  // namespace saber

// bytes must be a multiple of 8 and buf 8-byte aligned.
extern "C" int saber_digest_launch(const void* buf, size_t bytes, unsigned long long* out, cudaStream_t stream) {
  if ((bytes & 7) || (reinterpret_cast<uintptr_t>(buf) & 7)) return static_cast<int>(cudaErrorInvalidValue);
  const size_t n = bytes >> 3;
  const int blocks = static_cast<int>(n / 2048 + 1 < 592 ? n / 2048 + 1 : 592);
  saber::launch(saber::digest_kernel, dim3(blocks), dim3(256), 0, stream, 0, static_cast<const uint64_t*>(buf), n, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int saber_digest_clear_launch(unsigned long long* out, int n, cudaStream_t stream) {
  saber::launch(saber::digest_clear_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 0, out, n);
  return static_cast<int>(cudaGetLastError());
}
