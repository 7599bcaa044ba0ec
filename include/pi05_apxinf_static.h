/*
 * Kernel-level entry points under the reference's own symbol names.
 *
 * `crates/apxinf-cuda/src/ffi/custom.rs` and `ffi/cublaslt.rs` bind `apxinf_static_*`
 * symbols from `libapxinf_kernels.a` (built from crates/apxinf-cuda/adapters/*.cu). The
 * functions below keep those names, argument orders and return conventions
 * (cudaError_t as int: 0 = cudaSuccess, 1 = cudaErrorInvalidValue; the GEMM returns a
 * cublasStatus_t-style int: 0 ok, 7 invalid value, 1 not initialised), so the Rust
 * contracts in crates/apxinf-cuda/src/kernels/*.rs link against this library unchanged
 * for these operators. All pointers are device pointers; `stream` is a cudaStream_t.
 * Nothing here allocates.
 */
#ifndef PI05_APXINF_STATIC_H_
#define PI05_APXINF_STATIC_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* adapters/static_bf16_adapter.cu:28-45 — u8 [views, S, S, 3] (layout 0 = NHWC, 1 = NCHW)
 * -> bf16 [views * (S/ps)^2, 3*ps*ps], (u8/255)*2-1, columns c*ps*ps + dy*ps + dx. */
int apxinf_static_rgb_u8_to_patches_bf16(const void* images, void* patches, int views,
                                         int image_size, int patch_size, int layout, void* stream);
/* adapters/static_bf16_adapter.cu:152-160 — y = x * rsqrt(mean(x^2) + eps) * weight */
int apxinf_static_rms_norm_bf16(const void* input, const void* weight, void* output, int rows,
                                int cols, float eps, void* stream);
/* adapters/static_bf16_adapter.cu:162-171 */
int apxinf_static_layer_norm_bf16(const void* input, const void* weight, const void* bias,
                                  void* output, int rows, int cols, float eps, void* stream);
/* adapters/static_bf16_adapter.cu:203-211 — style = [scale | shift | gate], 3*cols bf16 */
int apxinf_static_ada_rms_norm_bf16(const void* input, const void* style, void* output, int rows,
                                    int cols, float eps, void* stream);
/* adapters/static_bf16_adapter.cu:104-112 — output = state + dt * velocity */
int apxinf_static_euler_update_bf16(const void* state, const void* velocity, void* output,
                                    int64_t count, float dt, void* stream);
/* adapters/static_bf16_adapter.cu:82-90 — table[id] * sqrt(width); id >= vocab -> 0 */
int apxinf_static_embedding_bf16(const void* table, const void* ids, void* output, int tokens,
                                 int width, int vocab_size, void* stream);
/* adapters/w8a8_adapter.cu:18-29 — per-row scale max(absmax/127, 1e-12), round half away */
int apxinf_static_quantize_rows_bf16_int8(const void* input, void* output, void* scales, int rows,
                                          int cols, void* stream);
/* adapters/cublaslt_adapter.cu:9,863-931 — output[m, n] = alpha * activation[m, k] . weight[k, n],
 * bf16 row-major, fp32 accumulate. `prepare` (once per shape, outside graph capture) must
 * precede the first `apxinf_static_bf16_gemm` on a device, as in the reference. */
int apxinf_static_prepare_bf16_gemm(int m, int n, int k);
int apxinf_static_bf16_gemm(const void* activation, const void* weight, void* output, int m, int n,
                            int k, float alpha, void* stream);

/* adapters/static_bf16_adapter.cu:265-278, kernels/custom/attention.cuh:761-812 — multi-query
 * attention softmax(q k^T / sqrt(head_dim)) v: q and output [query_tokens, heads, head_dim], k and v
 * [key_tokens, head_dim], bf16. Here one fused tensor-core launch; key_tokens <= 1024 and head_dim a
 * multiple of 8 up to 256 (cudaErrorInvalidValue otherwise). Returns a cudaError_t value. */
int apxinf_static_mqa_bf16(const void* q, const void* k, const void* v, void* output, int query_tokens,
                           int key_tokens, int heads, int head_dim, void* stream);
/* adapters/cublas_adapter.cu:89-132 — the same contract behind the reference's cuBLAS path
 * (QK^T GEMM, softmax, PV GEMM there); returns a cublasStatus_t value. */
int apxinf_static_cublas_mqa_bf16(const void* q, const void* k, const void* v, void* output,
                                  int query_tokens, int key_tokens, int heads, int head_dim, void* stream);
/* adapters/static_bf16_adapter.cu:280-292, kernels/custom/attention.cuh:814-870 — per-batch
 * multi-head attention: q, k, v and output [batches * tokens_per_batch, heads, head_dim] bf16. */
int apxinf_static_mha_bf16(const void* q, const void* k, const void* v, void* output, int tokens_per_batch,
                           int batches, int heads, int head_dim, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* PI05_APXINF_STATIC_H_ */
