// Kernel-level extern "C" entry points (declared in include/pi05_b200.h).
#include <string>

#include "../../include/pi05_b200.h"
#include "fmha.h"
#include "gemm.h"

namespace pi05 {

thread_local std::string g_last_cuda_error;

int record_cuda(cudaError_t error) {
  if (error == cudaSuccess) return kPi05Ok;
  g_last_cuda_error = cudaGetErrorString(error);
  return kPi05ErrCuda;
}

}  // namespace pi05

extern "C" const char* pi05_last_cuda_error(void) { return pi05::g_last_cuda_error.c_str(); }

extern "C" const char* pi05_version(void) { return "pi05_b200 sm_100a " __DATE__; }

extern "C" int pi05_gemm(const Pi05GemmArgs* args, void* cuda_stream) {
  using namespace pi05;
  if (args == nullptr) return kPi05ErrInvalidValue;
  GemmProblem q;
  q.op = args->op;
  q.M = args->m;
  q.N = args->n;
  q.K = args->k;
  q.nb0 = args->nb0;
  q.nb1 = args->nb1;
  q.a = GemmOperand{args->a, args->m, args->lda, args->a_sb0, args->a_sb1};
  q.b = GemmOperand{args->b, args->b_mn_major ? args->k : args->n, args->ldb, args->b_sb0,
                    args->b_sb1};
  q.b_mn_major = args->b_mn_major != 0;
  q.out = args->out;
  q.ldc = args->ldc;
  q.out_sb0 = args->out_sb0;
  q.out_sb1 = args->out_sb1;
  q.out_type = args->out_type;
  q.mode = args->mode;
  q.residual = args->residual;
  q.bias = args->bias;
  q.col_scale = args->col_scale;
  q.row_scale = args->row_scale;
  q.pos = args->pos;
  q.pos_rows = args->pos_rows;
  q.pos_ld = args->pos_ld;
  q.gate = args->gate;
  q.alpha = args->alpha;
  q.out_inv_scale = args->out_inv_scale;
  q.status = args->status;
  q.force_swap = args->force_swap;
  q.force_block_n = args->force_block_n;
  q.partials = args->partials;
  q.partials_bytes = args->partials_bytes;
  q.tile_counters = args->tile_counters;
  q.max_tiles = args->max_tiles;
  q.force_split_k = args->force_split_k;
  q.b_blocked = args->b_blocked != 0;
  q.force_skinny = args->force_skinny;
  q.k_slices = args->k_slices > 1 ? args->k_slices : 1;
  q.prologue = args->prologue;
  q.style = args->style;
  q.eps = args->eps;
  q.a_inv_scale = args->a_inv_scale;
  q.a_dynamic_rows = args->a_dynamic_rows != 0;
  q.rope_q_out = args->rope_q_out;
  q.rope_k_cache = args->rope_k_cache;
  q.rope_v_cache = args->rope_v_cache;
  q.rope_cos = args->rope_cos;
  q.rope_sin = args->rope_sin;
  q.rope_tokens = args->rope_tokens;
  q.rope_q_heads = args->rope_q_heads;
  q.rope_head_dim = args->rope_head_dim;
  q.rope_position_offset = args->rope_position_offset;
  q.rope_cache_rows = args->rope_cache_rows;
  q.dt = args->dt;
  GemmPlan plan;
  const int rc = gemm_plan_build(q, &plan);
  if (rc != kPi05Ok) return rc;
  return record_cuda(gemm_plan_launch(plan, static_cast<cudaStream_t>(cuda_stream)));
}

extern "C" int pi05_attention(const Pi05AttentionArgs* args, void* cuda_stream) {
  using namespace pi05;
  if (args == nullptr) return kPi05ErrInvalidValue;
  FmhaProblem f;
  f.q = args->q; f.q_ld = args->q_ld; f.q_sb0 = args->q_sb0; f.q_sb1 = args->q_sb1;
  f.k = args->k; f.k_ld = args->k_ld; f.k_sb0 = args->k_sb0; f.k_sb1 = args->k_sb1;
  f.v = args->v; f.v_ld = args->v_ld; f.v_sb0 = args->v_sb0; f.v_sb1 = args->v_sb1;
  f.out = args->out; f.out_ld = args->out_ld; f.out_sb0 = args->out_sb0; f.out_sb1 = args->out_sb1;
  f.q_rows = args->q_rows; f.keys = args->keys; f.head_dim = args->head_dim;
  f.nb0 = args->nb0; f.nb1 = args->nb1;
  f.scale = args->scale;
  f.out_e4m3 = args->out_e4m3 != 0;
  f.out_inv_scale = args->out_inv_scale;
  f.status = args->status;
  f.key_split = args->key_split != 0;
  f.split_scratch = static_cast<float*>(args->split_scratch);
  f.split_scratch_bytes = static_cast<size_t>(args->split_scratch_bytes);
  FmhaPlan plan;
  const int rc = fmha_plan_build(f, &plan);
  if (rc != kPi05Ok) return rc;
  return record_cuda(fmha_plan_launch(plan, static_cast<cudaStream_t>(cuda_stream)));
}
