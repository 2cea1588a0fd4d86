// Kernel launch helper with programmatic dependent launch (PDL).
//
// Every kernel of the engine starts with pdl_wait(): launched with the programmatic
// stream-serialization attribute, a kernel's CTAs may become resident while its predecessor in the
// stream is still running, and block in pdl_wait() until that predecessor has completed and its
// writes are visible.  Only the light row kernels call pdl_trigger() (at their top): their
// successor is a GEMM, one CTA per SM, which cannot be misplaced by starting early.  Nothing a predecessor produced is read, and nothing is written, before the
// wait, so the result is that of a fully serialised stream; what overlaps is the launch latency,
// the prologue and -- in the GEMM -- the first weight tiles, which no kernel ever writes.
// Captured into a CUDA graph the same launches become programmatic edges.
#pragma once
#include <cuda_runtime.h>

namespace saber {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

int pdl_enabled();   // process-wide switch (launch.cu): 0 off, 1 every kernel, 2 only launches that ask for it

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          int flags, Args... args) {
  const bool cooperative = (flags & 1) != 0;
  const bool wants_pdl = (flags & 2) != 0;     // launch sites that profit from starting early
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cooperative) {
    attr[n].id = cudaLaunchAttributeCooperative;
    attr[n].val.cooperative = 1;
    ++n;
  } else if (pdl_enabled() == 1 || (pdl_enabled() == 2 && wants_pdl)) {
    // (a cooperative grid must be resident as a whole when it starts: it is launched serialised)
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace saber
