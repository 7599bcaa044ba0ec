#include "denoise_persistent.h"

namespace pi05 {

namespace {

constexpr int kDenoiseMaxSmem = 226 * 1024;
// Off by default. Measured on the B=1 FP8 forward (10 rows, 920 stages): the kernel is
// bit-identical to the per-projection launches but takes 7.8 ms against 6.5 ms for them. A stage
// is bound by the same dependent L2 round trips either way (barrier arrival + poll, activation
// rows, residual: about 1 us each), so the grid barrier (2-3 us per stage) buys nothing over a
// programmatic dependent launch, while the fused norms cost more than their launches did.
bool g_enabled = false;
unsigned g_spin_limit = 1u << 21;
int g_skip_arrival = -1;

template <int OP>
const void* kernel_ptr() {
  auto kernel = &denoise_persistent_kernel<OP>;
  // the kernel also has a little static shared memory: leave room for it under the 227 KB cap
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDenoiseMaxSmem) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return reinterpret_cast<const void*>(kernel);
}

const void* kernel_of(int op) {
  if (op == kOpBf16) return kernel_ptr<kOpBf16>();
  if (op == kOpE4m3) return kernel_ptr<kOpE4m3>();
  if (op == kOpS8) return kernel_ptr<kOpS8>();
  return nullptr;
}

}  // namespace

bool persistent_denoise_enabled() { return g_enabled; }
void set_persistent_denoise_enabled(bool enabled) { g_enabled = enabled; }
void set_denoise_spin_limit(int polls) { g_spin_limit = polls > 0 ? static_cast<unsigned>(polls) : 1u << 21; }
unsigned denoise_spin_limit() { return g_spin_limit; }
void set_denoise_skip_arrival(int stage) { g_skip_arrival = stage; }
int denoise_skip_arrival() { return g_skip_arrival; }

int denoise_smem_bytes(int stage_smem_bytes) {
  return static_cast<int>((2 * sizeof(DenoiseStage) + 127) / 128 * 128) + stage_smem_bytes;
}

int denoise_max_grid(int op, int smem_bytes, int device) {
  const void* kernel = kernel_of(op);
  if (kernel == nullptr || smem_bytes > kDenoiseMaxSmem) return 0;
  int cooperative = 0, sms = 0, per_sm = 0;
  if (cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kDenoiseThreads, smem_bytes) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (cooperative == 0 || per_sm < 1) return 0;
  return sms;  // one CTA per SM: every stage is planned for at most that many
}

cudaError_t denoise_plan_launch(const DenoisePlan& plan, cudaStream_t stream) {
  const void* kernel = kernel_of(plan.op);
  if (kernel == nullptr || plan.grid <= 0) return cudaErrorInvalidValue;
  cudaError_t err = cudaMemsetAsync(plan.zero_base, 0, plan.zero_bytes, stream);
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(plan.grid));
  config.blockDim = dim3(kDenoiseThreads);
  config.dynamicSmemBytes = plan.smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeCooperative;
  attribute[0].val.cooperative = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  void* args[1] = {const_cast<DenoiseParams*>(&plan.params)};
  return cudaLaunchKernelExC(&config, kernel, args);
}

}  // namespace pi05
