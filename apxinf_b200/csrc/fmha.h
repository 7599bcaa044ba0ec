// Host side of the fused attention kernels (fmha_online.cuh, fmha_split.cuh): plan = TMA maps + parameters.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemm.h"

namespace pi05 {

enum FmhaStatus : int { kFmhaTimeout = 201 };

struct FmhaParams {
  int q_rows;      // query rows per batch entry
  int keys;        // keys per batch entry (<= 1024)
  int head_dim;    // 72, 128 or 256 (multiple of 8, <= 256)
  int nb0, nb1;    // batch extents; work items = query tiles x nb0 x nb1
  int pack;        // nb0 when all nb0 query heads share one K/V head (tiles mix heads), else 1
  float scale;
  void* out;       // [.., q_rows, head_dim] bf16 or e4m3
  long long out_ld, out_sb0, out_sb1;
  int out_e4m3;
  float out_inv_scale;
  int* status;
  float rescale_threshold;  // running maximum moves only past this many powers of two (fused kernel)
};


// softmax(scale * q k^T) v, batched over nb0 x nb1. q [q_rows, head_dim], k and v
// [keys, head_dim], all bf16 with contiguous head_dim; leading dimensions and batch strides in
// elements. out [q_rows, head_dim] bf16 or e4m3 (e4m3(clamp(bf16(o) * out_inv_scale))).
struct FmhaProblem {
  const void* q = nullptr;
  long long q_ld = 0, q_sb0 = 0, q_sb1 = 0;
  const void* k = nullptr;
  long long k_ld = 0, k_sb0 = 0, k_sb1 = 0;
  const void* v = nullptr;
  long long v_ld = 0, v_sb0 = 0, v_sb1 = 0;
  void* out = nullptr;
  long long out_ld = 0, out_sb0 = 0, out_sb1 = 0;
  int q_rows = 0, keys = 0, head_dim = 0, nb0 = 1, nb1 = 1;
  float scale = 1.0f;
  bool out_e4m3 = false;
  float out_inv_scale = 1.0f;
  int* status = nullptr;
  // key-split path (fmha_split.cuh): one CTA per (query tile, 64-key slice) plus a combine
  // launch; needs fmha_split_scratch_bytes() of device scratch
  bool key_split = false;
  float* split_scratch = nullptr;
  size_t split_scratch_bytes = 0;
};

// Parameters of the cluster kernel for a handful of query rows (fmha_rows.cuh).
struct FmhaRowsParams;

struct FmhaPlan {
  CUtensorMap tmap_q, tmap_k, tmap_v;
  FmhaParams params;
  dim3 grid;
  bool key_split = false;
  float* split_scratch = nullptr;
  dim3 combine_grid;
  // few query rows: one cluster of 8 CTAs per 16-row tile, no scratch (fmha_rows.cuh)
  bool rows_cluster = false;
  alignas(8) unsigned char rows_params[160];
  int rows_smem = 0;
};

// Process-wide switch (default on): launches with few query rows use the cluster kernel
// instead of the key-split kernel pair.
bool fmha_rows_cluster_enabled();
void set_fmha_rows_cluster_enabled(bool enabled);

bool fmha_supported(int q_rows, int keys, int head_dim);
// Query tiles (CTAs of the unsplit kernel) and scratch bytes of the key-split path.
long long fmha_query_tiles(int q_rows, int nb0, int nb1, bool shared_kv);
size_t fmha_split_scratch_bytes(int q_rows, int keys, int head_dim, int nb0, int nb1, bool shared_kv);
int fmha_plan_build(const FmhaProblem& problem, FmhaPlan* plan);
cudaError_t fmha_plan_launch(const FmhaPlan& plan, cudaStream_t stream);

}  // namespace pi05
