// Host side of the persistent denoise kernel (denoise_persistent.cuh): limits of the
// cooperative launch on a device, and the launch itself.
#pragma once

#include <cuda_runtime.h>

#include "denoise_persistent.cuh"

namespace pi05 {

struct DenoisePlan {
  DenoiseParams params{};
  int op = 0;           // OperandType of the projections
  int grid = 0;         // CTAs, one per SM
  int smem_bytes = 0;   // dynamic shared memory of the launch
  void* zero_base = nullptr;  // barrier counter and tile flags: zeroed before every launch
  size_t zero_bytes = 0;
};

// Dynamic shared memory the kernel needs for stages whose own working sets are at most
// `stage_smem_bytes`.
int denoise_smem_bytes(int stage_smem_bytes);

// How many CTAs a cooperative launch of the kernel may have on `device` with that much dynamic
// shared memory; 0 when the device cannot launch cooperatively or the kernel does not fit.
int denoise_max_grid(int op, int smem_bytes, int device);

cudaError_t denoise_plan_launch(const DenoisePlan& plan, cudaStream_t stream);

// Process-wide switch (default off, see denoise_persistent.cu): graphs whose action expert has
// at most 16 rows run the denoise loop as one cooperative launch; off, as one launch per
// projection.
bool persistent_denoise_enabled();
void set_persistent_denoise_enabled(bool enabled);
// Poll budget of the kernel's barrier and flag waits (<= 0: the default, 2^21).
void set_denoise_spin_limit(int polls);
unsigned denoise_spin_limit();
// Diagnostics of the timeout path: plans built afterwards leave out CTA 0's arrival after that
// stage (-1: none), so the barrier never completes and every CTA's bounded wait runs out.
void set_denoise_skip_arrival(int stage);
int denoise_skip_arrival();

}  // namespace pi05
