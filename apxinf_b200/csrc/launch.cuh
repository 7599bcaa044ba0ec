// Kernel launch helper with programmatic dependent launch (PDL).
//
// Every kernel of the replayed forward is launched with the
// programmatic-stream-serialization attribute: it may start (run its prologue,
// prefetch static weights) while its predecessor in the stream is still
// running, and calls pdl_wait() before it touches anything a predecessor
// writes. Every kernel calls pdl_wait() unconditionally, so completion stays
// transitive along the stream. Captured into a CUDA graph these become
// programmatic dependency edges.
#pragma once

#include <cuda_runtime.h>

#include <utility>

namespace pi05 {

// Process-wide switch (default on); the engine turns it off if a capture with
// programmatic edges is refused by the driver.
bool pdl_enabled();
void set_pdl_enabled(bool enabled);
// Process-wide switch (default on): graphs whose action expert has at most 16 rows plan the
// fused register-streaming launches; off, they plan the same launch list as larger batches.
bool fuse_small_rows_enabled();
void set_fuse_small_rows_enabled(bool enabled);
// With at most 16 action rows: the adaptive RMSNorms as the staging step of the projections
// that read them, or as launches of their own (default).
bool fuse_norms_enabled();
void set_fuse_norms_enabled(bool enabled);
// Diagnostics of the device-timeout path, read when a GEMM plan is built: the poll budget of the
// one-CTA-per-tile kernel's barrier waits (<= 0: the default), and a K block whose A load the
// first CTA announces but never issues (-1: none).
void set_wait_polls(int polls);
void set_drop_load_kb(int kb);
// GEMM plans built afterwards take the kernels compiled for one epilogue where one fits
// (default), or always the general kernel.
void set_single_epilogue_kernels_enabled(bool enabled);

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                       cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

}  // namespace pi05
