// Load-time kernels: the reference's synthetic weight generator evaluated on
// the GPU, re-layout of [in, out] matrices into the K-major [out, in] operand
// layout of the GEMM family, and per-output-channel weight quantisation.
// None of this runs inside the replayed graph.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace pi05 {

// dst[i] = bf16 of element (offset + i) of SyntheticRng(seed)
// (crates/apxinf-model/src/pi05/weights.rs:332-357: 64-bit LCG, top 31 bits,
// uniform in [-0.02, 0.02)).
cudaError_t launch_lcg_fill(void* dst_bf16, uint64_t seed, uint64_t offset, long long count,
                            cudaStream_t stream);

// dst[i] = bf16 of element (offset + i) of the seeded N(0, 0.02) stream: a counter-based
// generator (SplitMix64 keyed by the seed, twelve 16-bit fields summed), the distribution the
// benchmark configurations name; same element order as the stream above.
cudaError_t launch_normal_fill(void* dst_bf16, uint64_t seed, uint64_t offset, long long count,
                               cudaStream_t stream);

// bf16 -> f32 (to_f32 != 0) or f32 -> bf16 with round-to-nearest-even, element by element.
cudaError_t launch_convert(const void* src, void* dst, long long count, int to_f32, cudaStream_t stream);

// src [k, n] row-major  ->  dst [*, ldk] rows map(n), columns 0..k-1; both bf16, or both f32
// when f32 != 0.
// map(n) = row_offset + n, or with interleave != 0:
//          (n / 64) * 128 + slot * 64 + n % 64   (gate/up interleave for fused GeGLU).
cudaError_t launch_transpose_pack(const void* src, void* dst, int k, int n, long long ldk,
                                  int row_offset, int interleave, int slot, cudaStream_t stream,
                                  int f32 = 0);

// Per-row (= per output channel) quantisation of a bf16 (f32 when f32 != 0) [rows, ld] matrix.
// E4M3: scale = absmax/448 (1 if the row is zero), q = e4m3(w * (1/scale))
//       (crates/apxinf-model/src/pi05/fp8.rs:88-115).
// INT8: scale = max(absmax/127, 1e-12), q = clamp(round_half_away(w/scale), -128, 127)
//       (crates/apxinf-model/src/pi05/int8_weights.rs:92-123).
cudaError_t launch_quantize_weight_rows(const void* src, void* dst, float* scales, int rows,
                                        int cols, long long ld, int to_int8, cudaStream_t stream,
                                        int f32 = 0);

}  // namespace pi05
