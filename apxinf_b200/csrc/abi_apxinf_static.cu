// Kernel-level entry points under the reference's symbol names
// (include/pi05_apxinf_static.h; crates/apxinf-cuda/adapters/static_bf16_adapter.cu,
// w8a8_adapter.cu, cublaslt_adapter.cu).
#include <mutex>

#include "../../include/pi05_apxinf_static.h"
#include "fmha.h"
#include "gemm.h"
#include "row_kernels.cuh"

namespace {

constexpr int kInvalid = static_cast<int>(cudaErrorInvalidValue);
constexpr int kBlasInvalid = 7;         // CUBLAS_STATUS_INVALID_VALUE
constexpr int kBlasNotInitialized = 1;  // CUBLAS_STATUS_NOT_INITIALIZED
constexpr int kBlasExecutionFailed = 13;

// Device status word of the GEMM launches made through this file (a bounded device
// wait that runs out records a code here); one per GPU, inside the library image.
static __device__ int g_gemm_status;
std::mutex g_mutex;
int* g_status_address[64] = {};

int* status_for_current_device(bool lookup) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status_address[device] == nullptr && lookup) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_gemm_status) != cudaSuccess) return nullptr;
    g_status_address[device] = static_cast<int*>(address);
  }
  return g_status_address[device];
}

pi05::NormArgs norm_args(const void* input, void* output, int rows, int cols, float eps, int kind) {
  pi05::NormArgs a{};
  a.input = input;
  a.output = output;
  a.rows = rows;
  a.cols = cols;
  a.eps = eps;
  a.inv_scale = 1.0f;
  a.kind = kind;
  a.out = pi05::kRowBf16;
  return a;
}

}  // namespace

extern "C" int apxinf_static_rgb_u8_to_patches_bf16(const void* images, void* patches, int views,
                                                    int image_size, int patch_size, int layout,
                                                    void* stream) {
  if (images == nullptr || patches == nullptr || views <= 0 || image_size <= 0 ||
      patch_size <= 0 || image_size % patch_size != 0 || (layout != 0 && layout != 1)) {
    return kInvalid;
  }
  pi05::PatchifyArgs a{};
  a.images = static_cast<const uint8_t*>(images);
  a.patches = patches;
  a.n_images = views;
  a.image_size = image_size;
  a.patch_size = patch_size;
  a.ld = 3 * patch_size * patch_size;
  a.nchw = layout;
  a.out = pi05::kRowBf16;
  a.inv_scale = 1.0f;
  return static_cast<int>(pi05::launch_patchify(a, static_cast<cudaStream_t>(stream)));
}

extern "C" int apxinf_static_rms_norm_bf16(const void* input, const void* weight, void* output,
                                           int rows, int cols, float eps, void* stream) {
  if (input == nullptr || weight == nullptr || output == nullptr) return kInvalid;
  pi05::NormArgs a = norm_args(input, output, rows, cols, eps, pi05::kNormRms);
  a.weight = weight;
  return static_cast<int>(pi05::launch_norm(a, static_cast<cudaStream_t>(stream)));
}

extern "C" int apxinf_static_layer_norm_bf16(const void* input, const void* weight,
                                             const void* bias, void* output, int rows, int cols,
                                             float eps, void* stream) {
  if (input == nullptr || weight == nullptr || bias == nullptr || output == nullptr) return kInvalid;
  pi05::NormArgs a = norm_args(input, output, rows, cols, eps, pi05::kNormLayer);
  a.weight = weight;
  a.bias = bias;
  return static_cast<int>(pi05::launch_norm(a, static_cast<cudaStream_t>(stream)));
}

extern "C" int apxinf_static_ada_rms_norm_bf16(const void* input, const void* style, void* output,
                                               int rows, int cols, float eps, void* stream) {
  if (input == nullptr || style == nullptr || output == nullptr) return kInvalid;
  pi05::NormArgs a = norm_args(input, output, rows, cols, eps, pi05::kNormAda);
  a.style = style;
  return static_cast<int>(pi05::launch_norm(a, static_cast<cudaStream_t>(stream)));
}

extern "C" int apxinf_static_euler_update_bf16(const void* state, const void* velocity,
                                               void* output, int64_t count, float dt,
                                               void* stream) {
  if (state == nullptr || velocity == nullptr || output == nullptr || count <= 0) return kInvalid;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (output != state) {
    const cudaError_t err = cudaMemcpyAsync(output, state, static_cast<size_t>(count) * 2,
                                            cudaMemcpyDeviceToDevice, s);
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  return static_cast<int>(pi05::launch_euler(output, velocity, count, dt, s));
}

extern "C" int apxinf_static_embedding_bf16(const void* table, const void* ids, void* output,
                                            int tokens, int width, int vocab_size, void* stream) {
  return static_cast<int>(pi05::launch_embedding(table, static_cast<const uint32_t*>(ids), output, 1,
                                                 tokens, width, vocab_size, tokens, 0,
                                                 static_cast<cudaStream_t>(stream)));
}

extern "C" int apxinf_static_quantize_rows_bf16_int8(const void* input, void* output, void* scales,
                                                     int rows, int cols, void* stream) {
  return static_cast<int>(pi05::launch_quantize_rows_int8(
      input, static_cast<int8_t*>(output), static_cast<float*>(scales), rows, cols, cols, cols,
      static_cast<cudaStream_t>(stream)));
}

extern "C" int apxinf_static_prepare_bf16_gemm(int m, int n, int k) {
  if (m <= 0 || n <= 0 || k <= 0) return kBlasInvalid;
  return status_for_current_device(true) != nullptr ? 0 : kBlasNotInitialized;
}

extern "C" int apxinf_static_bf16_gemm(const void* activation, const void* weight, void* output,
                                       int m, int n, int k, float alpha, void* stream) {
  if (activation == nullptr || weight == nullptr || output == nullptr || m <= 0 || n <= 0 || k <= 0) {
    return kBlasInvalid;
  }
  int* status = status_for_current_device(false);
  if (status == nullptr) return kBlasNotInitialized;  // prepare was not called on this device
  pi05::GemmProblem q;
  q.op = pi05::kOpBf16;
  q.M = m;
  q.N = n;
  q.K = k;
  q.a = pi05::GemmOperand{activation, m, k, 0, 0};
  q.b = pi05::GemmOperand{weight, k, n, 0, 0};  // [k, n] row-major: MN-major B operand
  q.b_mn_major = true;
  q.out = output;
  q.ldc = n;
  q.alpha = alpha;
  q.status = status;
  pi05::GemmPlan plan;
  const int rc = pi05::gemm_plan_build(q, &plan);
  if (rc != pi05::kPi05Ok) return kBlasInvalid;
  return pi05::gemm_plan_launch(plan, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? 0
             : kBlasExecutionFailed;
}

namespace {

// softmax(q k^T / sqrt(head_dim)) v through the fused attention kernel; strides in elements.
int static_attention(const void* q, long long q_ld, long long q_sb0, long long q_sb1, const void* k,
                     const void* v, long long kv_ld, long long kv_sb0, long long kv_sb1, void* output,
                     int q_rows, int keys, int head_dim, int nb0, int nb1, void* stream) {
  if (q == nullptr || k == nullptr || v == nullptr || output == nullptr || q_rows <= 0 || keys <= 0 ||
      nb0 <= 0 || nb1 <= 0 || !pi05::fmha_supported(q_rows, keys, head_dim)) {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  int* status = status_for_current_device(true);
  if (status == nullptr) return static_cast<int>(cudaErrorInitializationError);
  pi05::FmhaProblem f;
  f.q = q; f.q_ld = q_ld; f.q_sb0 = q_sb0; f.q_sb1 = q_sb1;
  f.k = k; f.k_ld = kv_ld; f.k_sb0 = kv_sb0; f.k_sb1 = kv_sb1;
  f.v = v; f.v_ld = kv_ld; f.v_sb0 = kv_sb0; f.v_sb1 = kv_sb1;
  f.out = output; f.out_ld = q_ld; f.out_sb0 = q_sb0; f.out_sb1 = q_sb1;
  f.q_rows = q_rows; f.keys = keys; f.head_dim = head_dim; f.nb0 = nb0; f.nb1 = nb1;
  f.scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  f.status = status;
  pi05::FmhaPlan plan;
  if (pi05::fmha_plan_build(f, &plan) != pi05::kPi05Ok) return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(pi05::fmha_plan_launch(plan, static_cast<cudaStream_t>(stream)));
}

}  // namespace

extern "C" int apxinf_static_mqa_bf16(const void* q, const void* k, const void* v, void* output,
                                      int query_tokens, int key_tokens, int heads, int head_dim,
                                      void* stream) {
  const long long width = static_cast<long long>(heads) * head_dim;
  return static_attention(q, width, head_dim, 0, k, v, head_dim, 0, 0, output, query_tokens,
                          key_tokens, head_dim, heads, 1, stream);
}

extern "C" int apxinf_static_cublas_mqa_bf16(const void* q, const void* k, const void* v, void* output,
                                             int query_tokens, int key_tokens, int heads,
                                             int head_dim, void* stream) {
  const int rc = apxinf_static_mqa_bf16(q, k, v, output, query_tokens, key_tokens, heads, head_dim, stream);
  return rc == 0 ? 0 : rc == static_cast<int>(cudaErrorInvalidValue) ? kBlasInvalid : kBlasExecutionFailed;
}

extern "C" int apxinf_static_mha_bf16(const void* q, const void* k, const void* v, void* output,
                                      int tokens_per_batch, int batches, int heads, int head_dim,
                                      void* stream) {
  const long long width = static_cast<long long>(heads) * head_dim;
  return static_attention(q, width, head_dim, tokens_per_batch * width, k, v, width, head_dim,
                          tokens_per_batch * width, output, tokens_per_batch, tokens_per_batch,
                          head_dim, heads, batches, stream);
}
