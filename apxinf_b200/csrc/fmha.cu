#include "fmha.h"

#include <algorithm>

#include "fmha_split.cuh"
#include "fmha_online.cuh"

namespace pi05 {

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
