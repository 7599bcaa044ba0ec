#include "fmha.h"

#include <algorithm>
#include <cstring>

#include "fmha_rows.cuh"
#include "fmha_split.cuh"
#include "fmha_online.cuh"

namespace pi05 {

static_assert(sizeof(FmhaRowsParams) <= 160, "FmhaPlan::rows_params is too small");

namespace {
bool g_rows_cluster = true;
}
bool fmha_rows_cluster_enabled() { return g_rows_cluster; }
void set_fmha_rows_cluster_enabled(bool enabled) { g_rows_cluster = enabled; }

namespace {

// Few query rows over one shared K/V head per sample: fill the cluster kernel's parameters.
// Two operand forms reach it: heads as nb0 sharing one K/V head (k_sb0 = v_sb0 = 0, samples
// as nb1), or heads already folded into the rows with one K/V per nb0 entry (nb1 = 1).
bool rows_cluster_fits(const FmhaProblem& q, FmhaRowsParams* r, int* smem) {
  if (!fmha_rows_cluster_enabled() || q.head_dim % 16 != 0 || q.head_dim > 256) return false;
  const bool shared = q.nb0 > 1 && q.k_sb0 == 0 && q.v_sb0 == 0;
  int heads, samples;
  long long q_sample, k_sample, v_sample, o_sample;
  if (shared) {
    heads = q.nb0;
    samples = q.nb1;
    q_sample = q.q_sb1; k_sample = q.k_sb1; v_sample = q.v_sb1; o_sample = q.out_sb1;
  } else if (q.nb1 == 1) {
    heads = 1;
    samples = q.nb0;
    q_sample = q.q_sb0; k_sample = q.k_sb0; v_sample = q.v_sb0; o_sample = q.out_sb0;
  } else {
    return false;
  }
  const int rows = q.q_rows * heads;
  const int tiles = (rows + 15) / 16;
  if (static_cast<long long>(tiles) * samples > 64) return false;  // beyond that the persistent kernel wins
  const int slice = ((q.keys + kRowsCluster - 1) / kRowsCluster + 15) / 16 * 16;
  if (slice > 256) return false;
  auto aligned16 = [](const void* ptr, long long stride_elems) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && (stride_elems * 2) % 16 == 0;
  };
  if (!aligned16(q.q, q.q_ld) || !aligned16(q.k, q.k_ld) || !aligned16(q.v, q.v_ld) ||
      (q.q_sb0 * 2) % 16 != 0 || (q_sample * 2) % 16 != 0 || (k_sample * 2) % 16 != 0 ||
      (v_sample * 2) % 16 != 0) {
    return false;
  }
  // outputs are written as pairs of elements
  const int out_elem = q.out_e4m3 ? 1 : 2;
  if ((reinterpret_cast<uintptr_t>(q.out) % (2 * out_elem)) != 0 || q.out_ld % 2 != 0 || q.out_sb0 % 2 != 0 ||
      o_sample % 2 != 0) {
    return false;
  }
  r->q = static_cast<const __nv_bfloat16*>(q.q);
  r->q_ld = q.q_ld;
  r->q_sb0 = shared ? q.q_sb0 : 0;
  r->q_sb1 = q_sample;
  r->k = static_cast<const __nv_bfloat16*>(q.k);
  r->k_ld = q.k_ld;
  r->k_sb1 = k_sample;
  r->v = static_cast<const __nv_bfloat16*>(q.v);
  r->v_ld = q.v_ld;
  r->v_sb1 = v_sample;
  r->out = q.out;
  r->out_ld = q.out_ld;
  r->out_sb0 = shared ? q.out_sb0 : 0;
  r->out_sb1 = o_sample;
  r->rows = rows;
  r->heads = heads;
  r->keys = q.keys;
  r->head_dim = q.head_dim;
  r->slice_keys = slice;
  r->tiles = tiles;
  r->scale = q.scale;
  r->out_e4m3 = q.out_e4m3 ? 1 : 0;
  r->out_inv_scale = q.out_inv_scale;
  *smem = fmha_rows_smem_bytes(q.head_dim, slice);
  return *smem <= 227 * 1024;
}

}  // namespace

bool fmha_supported(int q_rows, int keys, int head_dim) {
  return q_rows > 0 && keys > 0 && keys <= 1024 && head_dim >= 16 && head_dim <= 256 &&
         head_dim % 8 == 0;
}

long long fmha_query_tiles(int q_rows, int nb0, int nb1, bool shared_kv) {
  const bool packed = shared_kv && nb0 > 1 && 128 % nb0 == 0;
  const int tile_tokens = packed ? 128 / nb0 : 128;
  return (long long)((q_rows + tile_tokens - 1) / tile_tokens) * (packed ? 1 : nb0) * nb1;
}

size_t fmha_split_scratch_bytes(int q_rows, int keys, int head_dim, int nb0, int nb1, bool shared_kv) {
  const long long items = fmha_query_tiles(q_rows, nb0, nb1, shared_kv) * ((keys + kSplitKeys - 1) / kSplitKeys);
  return static_cast<size_t>(items) * fmha_split_item_floats(head_dim) * sizeof(float);
}

int fmha_plan_build(const FmhaProblem& q, FmhaPlan* plan) {
  if (plan == nullptr || q.q == nullptr || q.k == nullptr || q.v == nullptr || q.out == nullptr ||
      q.status == nullptr || q.nb0 <= 0 || q.nb1 <= 0 || 
      !fmha_supported(q.q_rows, q.keys, q.head_dim)) {
    return kPi05ErrInvalidValue;
  }
  // multi-query attention: heads that share one K/V head are packed into the same query tile
  const bool shared_kv = q.nb0 > 1 && q.k_sb0 == 0 && q.v_sb0 == 0 && 128 % q.nb0 == 0;
  const int pack = shared_kv ? q.nb0 : 1;
  int rc;
  if (pack > 1) {
    // dims (head_dim, head, token, nb1), box 64 x pack x 128/pack: row = token * pack + head
    rc = encode_operand_map(&plan->tmap_q, kOpBf16, q.q, q.head_dim, q.nb0, q.q_rows, q.nb1, q.q_sb0,
                            q.q_ld, q.q_sb1, 64, pack, 128 / pack);
  } else {
    rc = encode_operand_map(&plan->tmap_q, kOpBf16, q.q, q.head_dim, q.q_rows, q.nb0, q.nb1, q.q_ld,
                            q.q_sb0, q.q_sb1, 64, 128);
  }
  if (rc != kPi05Ok) return rc;
  rc = encode_operand_map(&plan->tmap_k, kOpBf16, q.k, q.head_dim, q.keys, pack > 1 ? 1 : q.nb0, q.nb1,
                          q.k_ld, q.k_sb0, q.k_sb1, 64,
                          q.key_split ? kSplitKeys : kOnlineKeyBlock);
  if (rc != kPi05Ok) return rc;
  rc = encode_operand_map(&plan->tmap_v, kOpBf16, q.v, q.head_dim, q.keys, pack > 1 ? 1 : q.nb0, q.nb1,
                          q.v_ld, q.v_sb0, q.v_sb1, 64, 64);
  if (rc != kPi05Ok) return rc;
  FmhaParams& p = plan->params;
  p.q_rows = q.q_rows;
  p.keys = q.keys;
  p.head_dim = q.head_dim;
  p.nb0 = q.nb0;
  p.nb1 = q.nb1;
  p.pack = pack;
  p.scale = q.scale;
  p.out = q.out;
  p.out_ld = q.out_ld;
  p.out_sb0 = q.out_sb0;
  p.out_sb1 = q.out_sb1;
  p.out_e4m3 = q.out_e4m3 ? 1 : 0;
  p.out_inv_scale = q.out_inv_scale;
  p.status = q.status;
  p.rescale_threshold = 8.0f;
  const int tile_tokens = 128 / pack;
  const long long items =
      (long long)((q.q_rows + tile_tokens - 1) / tile_tokens) * (pack > 1 ? 1 : q.nb0) * q.nb1;
  int sms = 148, device = 0;
  if (cudaGetDevice(&device) == cudaSuccess) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  }
  plan->key_split = q.key_split;
  if (q.key_split) {
    const int splits = (q.keys + kSplitKeys - 1) / kSplitKeys;
    if (q.split_scratch == nullptr ||
        q.split_scratch_bytes < static_cast<size_t>(items) * splits * fmha_split_item_floats(q.head_dim) * sizeof(float)) {
      return kPi05ErrScratchLimit;
    }
    plan->split_scratch = q.split_scratch;
    FmhaRowsParams rows{};
    int rows_smem = 0;
    plan->rows_cluster = rows_cluster_fits(q, &rows, &rows_smem);
    if (plan->rows_cluster) {
      std::memcpy(plan->rows_params, &rows, sizeof(rows));
      plan->rows_smem = rows_smem;
      const int samples = rows.heads == q.nb0 && q.nb0 > 1 && q.k_sb0 == 0 && q.v_sb0 == 0 ? q.nb1 : q.nb0;
      plan->grid = dim3(static_cast<unsigned>(rows.tiles * samples * kRowsCluster), 1, 1);
      cudaFuncSetAttribute(fmha_rows_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      return kPi05Ok;
    }
    plan->grid = dim3(static_cast<unsigned>(items * splits), 1, 1);
    plan->combine_grid = dim3(static_cast<unsigned>(items * (128 / kCombineRows)), 1, 1);
    cudaFuncSetAttribute(fmha_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSplitSmemBytes);
    return kPi05Ok;
  }
  plan->grid = dim3(static_cast<unsigned>(std::min<long long>(items, sms)), 1, 1);
  cudaFuncSetAttribute(fmha_online_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kOnlineSmemBytes);
  return kPi05Ok;
}

cudaError_t fmha_plan_launch(const FmhaPlan& plan, cudaStream_t stream) {
  if (plan.key_split && plan.rows_cluster) {
    FmhaRowsParams rows;
    std::memcpy(&rows, plan.rows_params, sizeof(rows));
    cudaLaunchConfig_t config = {};
    config.gridDim = plan.grid;
    config.blockDim = dim3(kRowsThreads);
    config.dynamicSmemBytes = plan.rows_smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = kRowsCluster;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&config, fmha_rows_cluster_kernel, rows);
  }
  if (plan.key_split) {
    cudaError_t err = launch_pdl(fmha_split_kernel, plan.grid, dim3(kSplitThreads), kSplitSmemBytes, stream,
                                 plan.tmap_q, plan.tmap_k, plan.tmap_v, plan.params, plan.split_scratch);
    if (err != cudaSuccess) return err;
    return launch_pdl(fmha_combine_kernel, plan.combine_grid, dim3(256), 0, stream, plan.params,
                      static_cast<const float*>(plan.split_scratch));
  }
  return launch_pdl(fmha_online_kernel, plan.grid, dim3(kFmhaThreads), kOnlineSmemBytes, stream,
                    plan.tmap_q, plan.tmap_k, plan.tmap_v, plan.params);
}

}  // namespace pi05
