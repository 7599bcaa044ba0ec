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

#include <stddef.h>
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

/*
 * The remaining BF16 row operators of adapters/static_bf16_adapter.cu (all tensors bf16,
 * row-major; `bias` arguments may be NULL; every function returns a cudaError_t value). This
 * library's own PI0.5 engine performs the same arithmetic inside its GEMM epilogues; these
 * entry points serve hosts that bind the reference's operators one by one.
 */
/* :47-80, activation.cuh:244-256 — output = act(input + bias); activation 0 none, 1 GELU(tanh), 2 SiLU */
int apxinf_static_bias_activation_bf16(const void* input, const void* bias, void* output, int rows,
                                       int cols, int activation, void* stream);
/* :92-102 — output = [first; second] along rows */
int apxinf_static_concat_rows_bf16(const void* first, const void* second, void* output, int first_rows,
                                   int second_rows, int cols, void* stream);
/* :114-138, activation.cuh:332-347 — gate_up [rows, 2 * inner] -> gelu(gate) * up [rows, inner] */
int apxinf_static_geglu_bf16(const void* gate_up, void* output, int rows, int inner, void* stream);
/* :140-150, fused.cuh:353-365 — output = projection + residual + bias */
int apxinf_static_bias_residual_bf16(const void* projection, const void* bias, const void* residual,
                                     void* output, int rows, int cols, void* stream);
/* :173-185, fused.cuh:367-391 — hidden = bf16(projection + residual + bias); normalized = RMSNorm(hidden) * weight */
int apxinf_static_bias_residual_rms_norm_bf16(const void* projection, const void* bias, const void* residual,
                                              const void* weight, void* hidden, void* normalized, int rows,
                                              int cols, float eps, void* stream);
/* :187-201, fused.cuh:393-426 — the same with LayerNorm(hidden) * norm_weight + norm_bias */
int apxinf_static_bias_residual_layer_norm_bf16(const void* projection, const void* projection_bias,
                                                const void* residual, const void* norm_weight,
                                                const void* norm_bias, void* hidden, void* normalized,
                                                int rows, int cols, float eps, void* stream);
/* :213-223, fused.cuh:428-441 — output = residual + projection * style[2 * cols + col] (style = scale | shift | gate) */
int apxinf_static_ada_gate_residual_bf16(const void* projection, const void* residual, const void* style,
                                         void* output, int rows, int cols, void* stream);
/* :225-237, fused.cuh:443-469 — hidden as above with gate_style; normalized = adaRMSNorm(hidden; norm_style) */
int apxinf_static_ada_gate_residual_rms_norm_bf16(const void* projection, const void* residual,
                                                  const void* gate_style, const void* norm_style, void* hidden,
                                                  void* normalized, int rows, int cols, float eps, void* stream);
/* :239-252, fused.cuh:471-525 — splits [tokens, (q_heads + 2 kv_heads) * head_dim] (+ bias), rotates q and k
 * (rotate-half, position_offset + token, base theta), writes q [tokens, q_heads, head_dim] and k, v
 * rows at kv_output_offset + token of [*, kv_heads, head_dim] */
int apxinf_static_qkv_rope_bf16(const void* qkv, const void* bias, void* q, void* k, void* v, int tokens,
                                int q_heads, int kv_heads, int head_dim, float theta, int position_offset,
                                int kv_output_offset, void* stream);
/* :254-263, fused.cuh:527-544 — [tokens, 3 * width] (+ bias) -> q, k, v [tokens, width] */
int apxinf_static_qkv_split_bias_bf16(const void* qkv, const void* bias, void* q, void* k, void* v, int tokens,
                                      int projection_width, void* stream);
/* :294-306, elementwise.cuh:168-182 — output = projection + position[token % tokens_per_view] + bias */
int apxinf_static_bias_position_bf16(const void* projection, const void* bias, const void* position,
                                     void* output, int rows, int cols, int tokens_per_view, void* stream);

/*
 * The F16 / E4M3 operators of the reference's FP8 path (crates/apxinf-cuda/src/ffi/custom.rs:34-884,
 * adapters/custom_kernels.cu): activations f16, quantised tensors e4m3 = e4m3(clamp(x / scale,
 * +-448)) computed from the fp32 value, `bias` arguments may be NULL unless noted. Each returns
 * a cudaError_t value.
 */
/* custom_kernels.cu:62-91, quantization.cuh:6-44 */
int apxinf_static_quantize_f16_e4m3(const void* input, void* output, int64_t count, float scale, void* stream);
/* custom_kernels.cu:93-106 — f16(e4m3 * scale) */
int apxinf_static_dequantize_e4m3_f16(const void* input, void* output, int64_t count, float scale, void* stream);
/* custom_kernels.cu:108-134, preprocess.cuh:7-61 — (u8/255)*2-1 rounded to f16, then quantised */
int apxinf_static_rgb_u8_to_patches_e4m3(const void* images, void* patches, int views, int image_size,
                                         int patch_size, int layout, float scale, void* stream);
/* custom_kernels.cu:155-163, normalization.cuh:127-145 */
int apxinf_static_rms_norm_quant_f16_e4m3(const void* input, const void* weight, void* output, int rows,
                                          int cols, float eps, float scale, void* stream);
/* custom_kernels.cu:165-174, normalization.cuh:147-169 */
int apxinf_static_layer_norm_quant_f16_e4m3(const void* input, const void* weight, const void* bias,
                                            void* output, int rows, int cols, float eps, float scale,
                                            void* stream);
/* custom_kernels.cu:345-353, normalization.cuh:171-190 */
int apxinf_static_ada_rms_norm_quant_f16_e4m3(const void* input, const void* style, void* output, int rows,
                                              int cols, float eps, float scale, void* stream);
/* custom_kernels.cu:176-187, activation.cuh:78-89 — bias required */
int apxinf_static_bias_gelu_quant_f16_e4m3(const void* input, const void* bias, void* output, int rows,
                                           int cols, float scale, void* stream);
/* custom_kernels.cu:189-200, activation.cuh:91-103 */
int apxinf_static_bias_silu_quant_f16_e4m3(const void* input, const void* bias, void* output, int rows,
                                           int cols, float scale, void* stream);
/* custom_kernels.cu:202-213 */
int apxinf_static_bias_silu_f16(const void* input, const void* bias, void* output, int rows, int cols,
                                void* stream);
/* custom_kernels.cu:215-226 */
int apxinf_static_bias_f16(const void* input, const void* bias, void* output, int rows, int cols, void* stream);
/* custom_kernels.cu:228-239, embedding.cuh:39-55 */
int apxinf_static_embedding_f16(const void* table, const void* ids, void* output, int tokens, int width,
                                int vocab_size, void* stream);
/* custom_kernels.cu:241-253 */
int apxinf_static_concat_rows_f16(const void* first, const void* second, void* output, int first_rows,
                                  int second_rows, int cols, void* stream);
/* custom_kernels.cu:255-265 */
int apxinf_static_euler_update_f16(const void* state, const void* velocity, void* output, int64_t count,
                                   float dt, void* stream);
/* custom_kernels.cu:267-303, activation.cuh:116-242 */
int apxinf_static_geglu_quant_f16_e4m3(const void* gate_up, void* output, int rows, int inner, float scale,
                                       void* stream);
/* custom_kernels.cu:305-316, fused.cuh:251-261 */
int apxinf_static_bias_residual_f16(const void* projection, const void* bias, const void* residual,
                                    void* output, int rows, int cols, void* stream);
/* custom_kernels.cu:318-329, fused.cuh:112-135 — hidden = f16(projection + residual + bias);
 * normalized = e4m3(RMSNorm(hidden) * weight / scale) */
int apxinf_static_bias_residual_rms_norm_quant_f16_e4m3(const void* projection, const void* bias,
                                                        const void* residual, const void* weight, void* hidden,
                                                        void* normalized, int rows, int cols, float eps,
                                                        float scale, void* stream);
/* custom_kernels.cu:331-343, fused.cuh:137-167 */
int apxinf_static_bias_residual_layer_norm_quant_f16_e4m3(const void* projection, const void* projection_bias,
                                                          const void* residual, const void* norm_weight,
                                                          const void* norm_bias, void* hidden, void* normalized,
                                                          int rows, int cols, float eps, float scale,
                                                          void* stream);
/* custom_kernels.cu:355-366 */
int apxinf_static_ada_gate_residual_f16(const void* projection, const void* residual, const void* style,
                                        void* output, int rows, int cols, void* stream);
/* custom_kernels.cu:368-398, fused.cuh:169-248 */
int apxinf_static_ada_gate_residual_rms_norm_quant_f16_e4m3(const void* projection, const void* residual,
                                                            const void* gate_style, const void* norm_style,
                                                            void* hidden, void* normalized, int rows, int cols,
                                                            float eps, float scale, void* stream);
/* custom_kernels.cu:400-412, fused.cuh:278-332 */
int apxinf_static_qkv_rope_f16(const void* qkv, const void* bias, void* q, void* k, void* v, int tokens,
                               int q_heads, int kv_heads, int head_dim, float theta, int position_offset,
                               int kv_output_offset, void* stream);
/* custom_kernels.cu:414-423, fused.cuh:334-350 */
int apxinf_static_qkv_split_bias_f16(const void* qkv, const void* bias, void* q, void* k, void* v, int tokens,
                                     int projection_width, void* stream);
/* custom_kernels.cu:440-453, elementwise.cuh:132-145 */
int apxinf_static_bias_position_f16(const void* projection, const void* bias, const void* position,
                                    void* output, int rows, int cols, int tokens_per_view, void* stream);
/* custom_kernels.cu:136-153, attention.cuh:642-702 — the suffix rows attend over the cached
 * prefix keys followed by the suffix keys (one shared K/V head, [tokens, head_dim] each) */
int apxinf_static_mqa_flash_f16(const void* q, const void* prefix_k, const void* prefix_v, const void* suffix_k,
                                const void* suffix_v, void* output, int suffix_tokens, int heads, int head_dim,
                                int prefix_tokens, void* stream);
/* custom_kernels.cu:425-438, attention.cuh:706-758 */
int apxinf_static_mha_flash_f16(const void* q, const void* k, const void* v, void* output, int tokens_per_batch,
                                int batches, int heads, int head_dim, void* stream);
/* adapters/cublas_adapter.cu:41-87 — returns a cublasStatus_t value */
int apxinf_static_cublas_mqa_f16(const void* q, const void* k, const void* v, void* output, int query_tokens,
                                 int key_tokens, int heads, int head_dim, void* stream);
/* custom_kernels.cu:47-60 — tuning aid: overwrites `bytes` of `buffer` to displace the L2 contents */
int apxinf_static_evict_l2(void* buffer, size_t bytes, uint32_t seed, void* stream);

/*
 * The FP8 linear layers (adapters/cublaslt_adapter.cu:1092-1294, ffi/cublaslt.rs): activation
 * e4m3 [m, k], weight e4m3 [k, n] row-major, fp32 accumulation, alpha = activation scale x
 * weight scale. As in the reference the prepare_* call of a shape (which may allocate) must
 * come first, outside any stream capture, on the thread that runs the GEMM; the run calls
 * return CUBLAS_STATUS_NOT_INITIALIZED (1) otherwise and never allocate. Returns are
 * cublasStatus_t values (0 ok, 7 invalid value).
 */
int apxinf_static_native_fp8_supported(int device, int* supported); /* cudaError_t value */
int apxinf_static_prepare_fp8_gemm_f16(int m, int n, int k);
int apxinf_static_prepare_fp8_gemm_bias_f16(const void* bias, int m, int n, int k);
int apxinf_static_prepare_fp8_gemm_bias_gelu_e4m3(const void* bias, int m, int n, int k, float output_scale);
int apxinf_static_prepare_fp8_gemm_bias_residual_f16(const void* bias, int m, int n, int k);
/* :1151-1171 — output f16 = alpha * activation . weight */
int apxinf_static_fp8_gemm_f16(const void* activation, const void* weight, void* output, int m, int n, int k,
                               float alpha, void* stream);
/* :1273-1294 — output f16 = alpha * activation . weight + bias */
int apxinf_static_fp8_gemm_bias_f16(const void* activation, const void* weight, const void* bias, void* output,
                                    int m, int n, int k, float alpha, void* stream);
/* :1222-1247 — output e4m3 = gelu_tanh(alpha * activation . weight + bias) / output_scale */
int apxinf_static_fp8_gemm_bias_gelu_e4m3(const void* activation, const void* weight, const void* bias,
                                          void* output, int m, int n, int k, float alpha, float output_scale,
                                          void* stream);
/* :1249-1271 — output f16 = alpha * activation . weight + residual + bias (bias may be NULL) */
int apxinf_static_fp8_gemm_bias_residual_f16(const void* activation, const void* weight, const void* bias,
                                             const void* residual, void* output, int m, int n, int k,
                                             float alpha, void* stream);
/* ffi/cutlass.rs:85-95, adapters/cutlass_fp8_adapter.cu:6-12 — the same product without a
 * prepare step; `tactic` (the reference's tile-shape table, 0..7) is accepted and ignored.
 * Returns the reference's codes: 0 ok, -1 cannot implement, -2 init, -3 run, -5 bad tactic,
 * -6 bad arguments. */
int apxinf_static_cutlass_fp8_gemm_f16(const void* activation, const void* weight, void* output, int m, int n,
                                       int k, float alpha, int tactic, void* stream);
/* adapters/cutlass_w8a8_adapter.cu:6-13 — int8 [m, k] x int8 [n, k] with f32 row and column
 * scales -> bf16 [m, n] (int32 accumulation, exact). cudaError_t value. */
int apxinf_static_cutlass_int8_gemm_bf16(const void* activation, const void* weight_output_major,
                                         const void* row_scales, const void* column_scales, void* output, int m,
                                         int n, int k, void* stream);
/* adapters/w8a8_adapter.cu:31-46 — bf16(acc * row_scale * column_scale) */
int apxinf_static_dequantize_int32_bf16(const void* accumulators, const void* row_scales,
                                        const void* column_scales, void* output, int rows, int cols,
                                        void* stream);

#ifdef __cplusplus
}
#endif

#endif /* PI05_APXINF_STATIC_H_ */
