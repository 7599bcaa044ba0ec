// Host-side description, planning and launch of one tcgen05 GEMM.
// A plan (two TMA tensor maps + kernel parameters + launch geometry) is built
// once, on the host, with no device allocation, and can then be launched any
// number of times, also inside a CUDA-graph capture.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_skinny.cuh"
#include "gemm_umma.cuh"

namespace pi05 {

// A K-major operand: `rows` rows of `k` contiguous elements, leading dimension
// `ld`, optionally batched over two outer indices. All strides in elements.
struct GemmOperand {
  const void* ptr = nullptr;
  int rows = 0;
  long long ld = 0;
  long long sb0 = 0, sb1 = 0;
};

struct GemmProblem {
  int op = kOpBf16;  // OperandType of both operands
  int M = 0, N = 0, K = 0;
  int nb0 = 1, nb1 = 1;  // batch extents
  // > 1: the K range of ONE GEMM (nb0 = nb1 = 1) in that many runs of K blocks, run s writing
  // its own product at out + s * out_sb0 (fp32 partial products for a row kernel to add). The
  // runs hold ceil(blocks / k_slices) K blocks each; what the last one lacks reads as zero.
  int k_slices = 1;
  GemmOperand a;         // activations [M, K]
  GemmOperand b;         // weights [N, K]; with b_mn_major: [K, N] row-major, rows = K
  bool b_mn_major = false;
  // output / epilogue (logical [M, N_out]); N_out = N/2 for kEpiGeglu
  void* out = nullptr;
  long long ldc = 0, out_sb0 = 0, out_sb1 = 0;
  int out_type = kOutBf16;
  int mode = kEpiStore;
  const void* residual = nullptr;
  const void* bias = nullptr;
  const float* col_scale = nullptr;
  const float* row_scale = nullptr;
  long long row_scale_sb0 = 0;
  const void* pos = nullptr;
  int pos_rows = 1;
  long long pos_ld = 0;
  const void* gate = nullptr;
  float alpha = 1.0f;
  float out_inv_scale = 1.0f;
  int* status = nullptr;
  // optional split-K scratch (device): raw 32-bit partial tiles and per-tile arrival counters
  // (counters must be zero before the first launch; every launch leaves them zero again)
  void* partials = nullptr;
  size_t partials_bytes = 0;
  int* tile_counters = nullptr;
  int max_tiles = 0;
  int force_split_k = 0;  // 0 = automatic, 1 = off, n = exactly n (clamped to the K blocks)
  // the b operand is a weight matrix no kernel of the stream writes (enables early TMA loads)
  bool b_static = false;
  // b (weights) is stored K-block-major: [ceil(K / kb)][N][kb] with kb = 128 bytes of K
  bool b_blocked = false;
  // ---- launches with at most 16 rows (gemm_skinny.cuh) ----
  // producer fused into the activation staging: `a` then points to bf16 rows [M, K]
  int prologue = kProNone;          // SkinnyPrologue
  const void* style = nullptr;      // kProAdaNorm: bf16 scale | shift, each K long
  float eps = 1e-6f;
  float a_inv_scale = 1.0f;         // static quantisation scale^-1 of the staged activations
  bool a_dynamic_rows = false;      // int8: per-row scales computed in the prologue
  // kEpiRope: q|k|v projection -> rotated Q rows, K/V cache rows
  void* rope_q_out = nullptr;
  void* rope_k_cache = nullptr;
  void* rope_v_cache = nullptr;
  const float* rope_cos = nullptr;
  const float* rope_sin = nullptr;
  int rope_tokens = 0, rope_q_heads = 0, rope_head_dim = 0, rope_position_offset = 0,
      rope_cache_rows = 0;
  float dt = 0.0f;                  // kEpiEuler
  int force_skinny = -1;            // -1 auto, 0 never, 1 always (error if the shape does not fit)
  // tuning overrides (0 / -1 = automatic)
  int force_swap = -1;
  int force_block_n = 0;
  int force_two_per_sm = -1;  // -1 auto, 0 = one deep-ring CTA per SM, 1 = two shallow-ring CTAs
};

struct GemmPlan {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  GemmParams params;
  dim3 grid;
  int smem_bytes = 0;
  int threads = 0;
  const void* kernel = nullptr;
  bool swap = false;
  int block_n = 0;
  int split_k = 1;
  bool skinny = false;      // gemm_skinny_kernel (M <= 16): the tensor maps are unused
  SkinnyParams skinny_params;
  bool persistent = false;  // one CTA per SM walking tiles, double-buffered accumulator
  bool multi_wave_candidate = false;
  int tiles_a = 0, tiles_b = 0, total_tiles = 0;
};

// Error codes of this library's C ABI (negative = rejected before launch).
enum Pi05Error : int {
  kPi05Ok = 0,
  kPi05ErrInvalidValue = -1,
  kPi05ErrUnsupported = -2,
  kPi05ErrDriver = -3,
  kPi05ErrCuda = -4,
  kPi05ErrDeviceTimeout = -5,
  kPi05ErrNotBuilt = -6,
  kPi05ErrScratchLimit = -7,
};

// Rank-4 tiled TMA map {inner, rows, b0, b1} of a K-major operand (element strides),
// 128-byte swizzle, zero fill outside the extents. `op` = OperandType.
int encode_operand_map(CUtensorMap* map, int op, const void* ptr, uint64_t inner, uint64_t rows,
                       uint64_t nb0, uint64_t nb1, long long ld, long long sb0, long long sb1,
                       uint32_t box_inner, uint32_t box_rows, uint32_t box_nb0 = 1,
                       int swizzle_bytes = 128);

int gemm_plan_build(const GemmProblem& problem, GemmPlan* plan);
cudaError_t gemm_plan_launch(const GemmPlan& plan, cudaStream_t stream);

}  // namespace pi05
