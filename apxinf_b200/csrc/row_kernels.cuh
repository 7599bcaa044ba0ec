// Row-wise and elementwise kernels of the PI0.5 forward (everything that is not
// a contraction): LayerNorm / RMSNorm / adaptive RMSNorm with fused output
// quantisation, RoPE + KV-cache write, row softmax, uint8 NHWC image -> patch
// rows, token embedding, per-row INT8 / static E4M3 quantisation, Euler update.
//
// All of them are HBM-bound: one global read and one global write per element,
// 16-byte vector accesses, reductions by warp shuffles.
//
// They restate, for sm_100a, the reference kernels in
// crates/apxinf-cuda/kernels/custom/{normalization,fused,attention,preprocess,
// embedding,quantization,elementwise}.cuh; the rounding points are the same.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pi05 {

enum NormKind : int { kNormLayer = 0, kNormRms = 1, kNormAda = 2 };
// kRowInt8: dynamic per-row scale (written to row_scale); kRowInt8Static: one given scale,
// q = clamp(round_half_away(bf16(y) * inv_scale), -128, 127).
enum RowOut : int { kRowBf16 = 0, kRowE4m3 = 1, kRowInt8 = 2, kRowInt8Static = 3 };

struct NormArgs {
  const void* input;    // bf16 [rows, cols]
  void* output;         // bf16 | e4m3 | int8 [rows, cols]
  float* row_scale;     // f32 [rows], written when out == kRowInt8
  const void* weight;   // bf16 [cols] (LayerNorm gamma / RMSNorm scale); may be null (= 1)
  const void* bias;     // bf16 [cols] (LayerNorm beta); may be null (= 0)
  const void* style;    // bf16 [>= 2*cols]: scale | shift (adaptive RMSNorm)
  int rows, cols;
  float eps;
  float inv_scale;      // 1 / activation scale for kRowE4m3 and kRowInt8Static
  int kind, out;
  // != 0: weight / bias / style are written by no kernel of the stream (the engine computes
  // its style vectors once, outside the replayed launch list), so they are read ahead of the
  // programmatic-dependency wait and their round trip overlaps the predecessor's tail
  int static_params;
  // != null (RMSNorm, fewer than 1024 rows): the rows are not read from `input` but formed
  // first, as launch_sum_partials would form them, from `sum_splits` fp32 partial products
  // (`sum_stride` elements apart), the bf16 residual and an optional bf16 bias; they are
  // written to `input` (which may be the residual buffer) and normalised in the same pass.
  const float* sum_partials;
  int sum_splits;
  long long sum_stride;
  const void* sum_residual;
  const void* sum_bias;
};
cudaError_t launch_norm(const NormArgs& args, cudaStream_t stream);

struct RopeArgs {
  const void* qkv;      // bf16 [rows, (q_heads + 2*kv) * head_dim], packed q | k | v
  void* q_out;          // bf16 [rows, q_heads, head_dim]
  void* k_cache;        // bf16 [batch, cache_rows, head_dim]
  void* v_cache;        // bf16 [batch, cache_rows, head_dim]
  const float* cos_table;  // f32 [positions, head_dim/2]
  const float* sin_table;
  int rows;             // batch * tokens
  int tokens;           // tokens per sample
  int q_heads, head_dim;
  int position_offset;  // position of token 0; also its row in the cache
  int cache_rows;       // rows per sample in the caches
};
cudaError_t launch_rope(const RopeArgs& args, cudaStream_t stream);

// In-place softmax over `cols` <= 1024 bf16 scores per row; batch stride and
// leading dimension in elements. Result rounded to bf16.
cudaError_t launch_softmax(void* scores, int rows_per_batch, int batches, long long batch_stride,
                           int cols, long long ld, cudaStream_t stream);

struct PatchifyArgs {
  const uint8_t* images;  // [n_images, size, size, 3] (NHWC) or [n_images, 3, size, size]
  // optional: ready-made patch rows [n_images * pps * pps, 3*ps*ps] fp32 (same column order) to
  // convert instead of reading `images`
  const float* f32_patches;
  void* patches;          // [n_images * pps * pps, ld] bf16 or e4m3, columns c*ps*ps + dy*ps + dx
  int n_images, image_size, patch_size;
  int ld;                 // >= 3*ps*ps, multiple of 16; pad columns are written as zero
  int nchw;
  int out;                // kRowBf16 | kRowE4m3
  float inv_scale;
};
cudaError_t launch_patchify(const PatchifyArgs& args, cudaStream_t stream);

// out[b, row_offset + t, :] = table[ids[b, t], :] * sqrt(width); ids >= vocab give zeros.
cudaError_t launch_embedding(const void* table, const uint32_t* ids, void* out, int batch,
                             int tokens, int width, int vocab, int out_rows_per_batch,
                             int row_offset, cudaStream_t stream);

// Dynamic per-row symmetric INT8: scale = max(absmax/127, 1e-12), round half away.
cudaError_t launch_quantize_rows_int8(const void* input, int8_t* output, float* row_scale, int rows,
                                      int cols, long long ld_in, long long ld_out,
                                      cudaStream_t stream);

// Static per-tensor E4M3: e4m3(clamp(x * inv_scale)).
cudaError_t launch_quantize_e4m3(const void* input, uint8_t* output, long long count,
                                 float inv_scale, cudaStream_t stream);

// Static per-tensor INT8: clamp(round_half_away(x * inv_scale), -128, 127).
cudaError_t launch_quantize_s8(const void* input, int8_t* output, long long count, float inv_scale,
                               cudaStream_t stream);

// out = bf16((bf16(sum_s partials[s]) + residual) + bias): finishes a GEMM whose K range was cut
// into `splits` batches writing fp32 partial products [splits][count] (count = rows * cols,
// cols a multiple of 8; bias bf16 [cols] or null).
cudaError_t launch_sum_partials(const float* partials, int splits, long long count, int cols,
                                const void* residual, const void* bias, void* out,
                                cudaStream_t stream);

// state <- bf16(state + dt * velocity)
cudaError_t launch_euler(void* state, const void* velocity, long long count, float dt,
                         cudaStream_t stream);

}  // namespace pi05
