// saber_gemm_i8_noalloc: the integer GEMM for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine; it exists for users of THIS
// library who cannot call cudaMalloc where they call the GEMM: inside a stream capture, inside a
// serving loop that must never take the allocator's lock, or in a host process whose device
// memory belongs entirely to another component's pool.  It computes exactly what
// saber_gemm_i8_launch computes (same kernel, same operand layouts, same results bit for bit) but
// takes its split-K scratch from a fixed array inside the library instead of from the caller:
//
//   * capacity: the kernel keeps one block of 128 x 256 int32 partial sums per (split, m tile, n tile),
//     however few of a tile's 128 rows are live, so the limit is
//         splits * ceil(M / nt) * (N_pad / 256) * 32768 <= 4 Mi ints (16 MiB)
//     (for example 8 splits of one m tile reach it at N_pad = 4096) and at most 1024 (m tile, n tile)
//     pairs; larger problems are refused with kNoAllocTooLarge, nothing is launched;
//   * cost: about 16 MiB of device memory on every GPU that loads the library, until exit;
//   * no cudaMalloc / cudaFree / allocating library routine is called, ever;
//   * the first call on a device looks up the array's device address and raises the kernel's
//     shared-memory limit: make that first call outside any stream capture;
//   * every call uses the same array: calls whose kernels can overlap on the GPU (different
//     streams, or graph branches) race on it.  Issue them in one stream, or order them yourself.
//
// `status` may be a device word of the caller's (set to the code of a bounded wait that ran out,
// 0 otherwise; the call clears the library's own word, not the caller's); pass null to use the
// library's, which saber_gemm_i8_noalloc_status() reads back.  Inputs and outputs are the
// caller's, in the layouts gemm_i8.h describes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

enum : int {
  kNoAllocBadArgs = -1,
  kNoAllocTooLarge = -2,   // the problem needs more scratch than the library's fixed array holds
};

extern "C" int saber_gemm_i8_noalloc(const uint8_t* w, const float* w_scale, const int8_t* a,
                                     const float* a_scale, __nv_bfloat16* out, uint32_t* status,
                                     int M, int M_pad, int N, int N_pad, int K, int nt, int splits,
                                     int w4, int ldo, cudaStream_t stream);
// The library's own status word on the current device, after synchronising with `stream`
// (negative: the entry point has not run on this device yet).  Allocates nothing either.
extern "C" int saber_gemm_i8_noalloc_status(cudaStream_t stream);
