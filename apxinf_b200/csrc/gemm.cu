// Host side of the tcgen05 GEMM family: tensor-map encoding, tile-shape
// selection and launch. Nothing here allocates device memory.
#include "gemm.h"

#include <cudaTypedefs.h>

#include <algorithm>
#include <mutex>

namespace pi05 {

namespace {
bool g_pdl_enabled = true;
bool g_fuse_small_rows = true;
uint32_t g_wait_polls = ptx::kSpinLimit;
int g_drop_load_kb = -1;
bool g_single_epilogue = true;
}
void set_wait_polls(int polls) { g_wait_polls = polls > 0 ? static_cast<uint32_t>(polls) : ptx::kSpinLimit; }
void set_drop_load_kb(int kb) { g_drop_load_kb = kb; }
void set_single_epilogue_kernels_enabled(bool enabled) { g_single_epilogue = enabled; }
bool pdl_enabled() { return g_pdl_enabled; }
void set_pdl_enabled(bool enabled) { g_pdl_enabled = enabled; }
bool fuse_small_rows_enabled() { return g_fuse_small_rows; }
void set_fuse_small_rows_enabled(bool enabled) { g_fuse_small_rows = enabled; }
namespace {
// Off: as the staging step of the 80-128 CTAs of the projection that reads it, an adaptive norm
// costs every one of them about 250 dependent instructions per (row, 8-element chunk) item
// (measured: 4.8 us added to the q|k|v and gate|up projections of the B=1 action expert, against
// about 3 us for the 10-CTA norm launch in front of them).
bool g_fuse_norms = false;
}
bool fuse_norms_enabled() { return g_fuse_norms; }
void set_fuse_norms_enabled(bool enabled) { g_fuse_norms = enabled; }

namespace {

using EncodeTiledFn = PFN_cuTensorMapEncodeTiled_v12000;

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) ==
            cudaSuccess &&
        query == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

int elem_bytes(int op) { return op == kOpBf16 ? 2 : 1; }

}  // namespace

// Rank-4 tiled map {inner, rows, b0, b1}, 128-byte swizzle, zero fill outside.
int encode_operand_map(CUtensorMap* map, int op, const void* ptr, uint64_t inner, uint64_t rows,
               uint64_t nb0, uint64_t nb1, long long ld, long long sb0, long long sb1,
               uint32_t box_inner, uint32_t box_rows, uint32_t box_nb0, int swizzle_bytes) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return kPi05ErrDriver;
  const uint64_t es = elem_bytes(op);
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return kPi05ErrInvalidValue;
  if ((ld * es) % 16 != 0) return kPi05ErrInvalidValue;
  uint64_t row_bytes = static_cast<uint64_t>(ld) * es;
  uint64_t s0 = static_cast<uint64_t>(sb0) * es;
  uint64_t s1 = static_cast<uint64_t>(sb1) * es;
  // singleton batch dimensions still need a legal (16-byte multiple) stride
  if (nb0 <= 1) s0 = row_bytes * rows;
  if (nb1 <= 1) s1 = (nb0 <= 1 ? row_bytes * rows : s0 * nb0);
  if (s0 % 16 != 0 || s1 % 16 != 0) return kPi05ErrInvalidValue;
  cuuint64_t dims[4] = {inner, rows, nb0 < 1 ? 1 : nb0, nb1 < 1 ? 1 : nb1};
  cuuint64_t strides[3] = {row_bytes, s0, s1};
  cuuint32_t box[4] = {box_inner, box_rows, box_nb0, 1};
  cuuint32_t estrides[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dtype =
      op == kOpBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult result = encode(map, dtype, 4, const_cast<void*>(ptr), dims, strides, box, estrides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle_bytes == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
                           : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                 : CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return result == CUDA_SUCCESS ? kPi05Ok : kPi05ErrDriver;
}

namespace {

template <int OP, int BLOCK_N, int STAGES, bool SWAP, bool B_MN, int EPI_WARPS = 8, int FIXED_MODE = -1>
const void* kernel_ptr(int* smem, int* threads) {
  auto kernel = &gemm_umma_kernel<OP, BLOCK_N, STAGES, SWAP, B_MN, EPI_WARPS, FIXED_MODE>;
  *threads = gemm_threads(EPI_WARPS);
  *smem = gemm_smem_bytes(BLOCK_N, STAGES);
  // per device and kernel, once: plans may be built while a stream of the thread is capturing
  static bool done[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 64 && !done[device]) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         gemm_smem_bytes(BLOCK_N, STAGES));
    done[device] = true;
  }
  return reinterpret_cast<const void*>(kernel);
}

template <int OP, int BLOCK_N, int STAGES, bool B_MN, int FIXED_MODE = -1>
const void* persistent_ptr(int* smem, int* threads) {
  // Eight epilogue warps. Twelve were a gain while the epilogue was bound by TMEM round trips;
  // measured again on the batched step (three back-to-back pairs on one box: 457.8 / 461.5 /
  // 465.2 against 455.6 / 461.4 / 460.4 action chunks/s, gate|up at 0.887 against 0.868 of the
  // tensor peak) and on the B=1 forward (9.75 against 9.79 ms) eight are level or ahead, with
  // fewer waiting warps to feed under the power cap. Sixteen spill under the register cap.
  constexpr int kEpiWarps = 8;
  auto kernel = &gemm_umma_persistent_kernel<OP, BLOCK_N, STAGES, B_MN, kEpiWarps, FIXED_MODE>;
  *threads = gemm_threads(kEpiWarps);
  *smem = gemm_smem_bytes(BLOCK_N, STAGES);
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       gemm_smem_bytes(BLOCK_N, STAGES));
  return reinterpret_cast<const void*>(kernel);
}

template <int OP, int BLOCK_N, int STAGES>
const void* persistent_lean_ptr(int lean_mode, int* smem, int* threads) {
  {
    if (lean_mode == kEpiStore) return persistent_ptr<OP, BLOCK_N, STAGES, false, kEpiStore>(smem, threads);
    if (lean_mode == kEpiBiasGelu) return persistent_ptr<OP, BLOCK_N, STAGES, false, kEpiBiasGelu>(smem, threads);
    if (lean_mode == kEpiBiasResidual)
      return persistent_ptr<OP, BLOCK_N, STAGES, false, kEpiBiasResidual>(smem, threads);
    if (lean_mode == kEpiGeglu) return persistent_ptr<OP, BLOCK_N, STAGES, false, kEpiGeglu>(smem, threads);
    if (lean_mode == kEpiGateResidual)
      return persistent_ptr<OP, BLOCK_N, STAGES, false, kEpiGateResidual>(smem, threads);
  }
  return persistent_ptr<OP, BLOCK_N, STAGES, false>(smem, threads);
}

template <int OP>
const void* select_persistent(int block_n, bool b_mn, int lean_mode, int* smem, int* threads) {
  if (b_mn) {
    if constexpr (OP == kOpBf16 || OP == kOpE4m3) {
      if (block_n == 128) return persistent_ptr<OP, 128, 6, true>(smem, threads);
      if (block_n == 256) return persistent_ptr<OP, 256, 4, true>(smem, threads);
    }
    return nullptr;
  }
  if (block_n == 64) return persistent_lean_ptr<OP, 64, 8>(lean_mode, smem, threads);
  if (block_n == 128) return persistent_lean_ptr<OP, 128, 6>(lean_mode, smem, threads);
  if (block_n == 256) return persistent_lean_ptr<OP, 256, 4>(lean_mode, smem, threads);
  return nullptr;
}

// The epilogues that SigLIP, the prefix and the batched action expert run in every layer (plain
// store, bias + GELU, bias + residual, gated residual) have kernels of their own for the bf16 and FP8 forward: no other epilogue's code, no
// split-K exchange, one output type (`lean_mode` is the epilogue, or -1 for the general kernel).
// Measured on the FP8 B=1 forward: 9.53 -> 9.05 ms for the shorter instruction stream alone.
template <int OP, int BLOCK_N, int STAGES>
const void* plain_ptr(int mode, int* smem, int* threads) {
  {
    if (mode == kEpiStore) return kernel_ptr<OP, BLOCK_N, STAGES, false, false, 8, kEpiStore>(smem, threads);
    if (mode == kEpiBiasGelu) return kernel_ptr<OP, BLOCK_N, STAGES, false, false, 8, kEpiBiasGelu>(smem, threads);
    if (mode == kEpiBiasResidual)
      return kernel_ptr<OP, BLOCK_N, STAGES, false, false, 8, kEpiBiasResidual>(smem, threads);
    if (mode == kEpiGateResidual)
      return kernel_ptr<OP, BLOCK_N, STAGES, false, false, 8, kEpiGateResidual>(smem, threads);
  }
  return kernel_ptr<OP, BLOCK_N, STAGES, false, false>(smem, threads);
}

template <int OP>
const void* select_kernel(int block_n, bool swap, bool b_mn, bool multi_wave, int lean_mode,
                          int* smem, int* threads) {
  if (b_mn) {
    if constexpr (OP == kOpBf16 || OP == kOpE4m3) {
      if (block_n == 128) return kernel_ptr<OP, 128, 6, false, true>(smem, threads);
      if (block_n == 256) return kernel_ptr<OP, 256, 4, false, true>(smem, threads);
    }
    return nullptr;
  }
  if (swap) {
    if (block_n == 16) return kernel_ptr<OP, 16, 8, true, false>(smem, threads);
    if (block_n == 32) return kernel_ptr<OP, 32, 8, true, false>(smem, threads);
    if (block_n == 64) return kernel_ptr<OP, 64, 8, true, false>(smem, threads);
    return nullptr;
  }
  if (block_n == 64) return plain_ptr<OP, 64, 8>(lean_mode, smem, threads);
  if (block_n == 128) return plain_ptr<OP, 128, 6>(lean_mode, smem, threads);
  if (block_n == 256) return plain_ptr<OP, 256, 4>(lean_mode, smem, threads);
  return nullptr;
}

}  // namespace

namespace {

template <int OP, int NTW, bool PRO>
const void* skinny_ptr_of() {
  auto kernel = &gemm_skinny_kernel<OP, NTW, PRO>;
  // plans of different K share the kernel: allow the largest tile any of them may ask for
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  return reinterpret_cast<const void*>(kernel);
}

// Launches without a fused producer (nearly all) run a kernel that does not contain that code:
// measured on the B=1 forward, 9.75 -> 9.58 ms, for no change but a shorter instruction stream.
template <int OP>
const void* skinny_ptr(int ntw, bool producer) {
  if (producer) return ntw == 2 ? skinny_ptr_of<OP, 2, true>() : skinny_ptr_of<OP, 1, true>();
  return ntw == 2 ? skinny_ptr_of<OP, 2, false>() : skinny_ptr_of<OP, 1, false>();
}

bool needs_skinny(const GemmProblem& q) {
  return q.prologue != kProNone || q.mode == kEpiRope || q.mode == kEpiEuler;
}

// Can the at-most-16-row kernel take this problem? (Everything it cannot take still has the
// tcgen05 path, except the fused prologues and the RoPE / Euler epilogues.)
bool skinny_fits(const GemmProblem& q) {
  const int es = elem_bytes(q.op);
  const bool aligned = (reinterpret_cast<uintptr_t>(q.a.ptr) & 15u) == 0 &&
                       (reinterpret_cast<uintptr_t>(q.b.ptr) & 15u) == 0 &&
                       (q.b.ld * es) % 16 == 0 && ((long long)q.K * es) % 16 == 0 &&
                       (q.a.ld * (q.prologue != kProNone ? 2 : es)) % 16 == 0;
  if (q.M > 16 || q.b_mn_major || q.b_blocked || q.nb0 * q.nb1 != 1 || q.k_slices > 1 || q.mode == kEpiBiasPos || !aligned) {
    return false;
  }
  if (q.prologue != kProNone) {
    // rows are cut into 8-element chunks reduced in segments of 32 (or one power-of-two segment)
    const int chunks = q.K / 8;
    const bool segmentable = chunks % 32 == 0 || (chunks < 32 && (chunks & (chunks - 1)) == 0);
    if (q.K % 8 != 0 || q.K > 4096 || !segmentable) return false;
  }
  if (q.mode == kEpiGeglu && q.N % 128 != 0) return false;
  if (q.mode == kEpiRope &&
      (q.rope_head_dim <= 0 || q.rope_head_dim % 16 != 0 || q.N != (q.rope_q_heads + 2) * q.rope_head_dim ||
       q.rope_q_out == nullptr || q.rope_k_cache == nullptr || q.rope_v_cache == nullptr ||
       q.rope_cos == nullptr || q.rope_sin == nullptr || q.rope_tokens <= 0 || q.M % q.rope_tokens != 0)) {
    return false;
  }
  if (q.prologue == kProAdaNorm && q.style == nullptr) return false;
  return true;
}

int skinny_plan_build(const GemmProblem& q, GemmPlan* plan) {
  const int es = elem_bytes(q.op);
  SkinnyParams& p = plan->skinny_params;
  p = SkinnyParams{};
  p.a = q.a.ptr;
  p.lda = q.a.ld;
  p.w = reinterpret_cast<const uint8_t*>(q.b.ptr);
  p.ldw_bytes = q.b.ld * es;
  p.M = q.M;
  p.N = q.N;
  p.K = q.K;
  p.kbytes = q.K * es;
  p.a_stride = (p.kbytes + 127) / 128 * 128 + 64;
  p.raw_stride = q.prologue != kProNone ? q.K * 2 + 16 : 0;
  p.steps = (p.kbytes + 63) / 64;
  const int ntw = (q.mode == kEpiGeglu || q.mode == kEpiRope) ? 2 : 1;
  p.tile_offset = q.mode == kEpiGeglu ? 64 : q.mode == kEpiRope ? q.rope_head_dim / 2 : 8;
  p.prologue = q.prologue;
  p.style = reinterpret_cast<const __nv_bfloat16*>(q.style);
  p.eps = q.eps;
  p.a_inv_scale = q.a_inv_scale;
  p.dynamic_rows = q.a_dynamic_rows ? 1 : 0;
  p.out = q.out;
  p.ldc = q.ldc;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(q.residual);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(q.bias);
  p.col_scale = q.col_scale;
  p.row_scale = q.row_scale;
  p.gate = reinterpret_cast<const __nv_bfloat16*>(q.gate);
  p.alpha = q.alpha;
  p.out_inv_scale = q.out_inv_scale;
  p.mode = q.mode;
  p.out_type = q.out_type;
  p.dt = q.dt;
  p.q_out = q.rope_q_out;
  p.k_cache = q.rope_k_cache;
  p.v_cache = q.rope_v_cache;
  p.cos_table = q.rope_cos;
  p.sin_table = q.rope_sin;
  p.tokens = q.rope_tokens;
  p.q_heads = q.rope_q_heads;
  p.head_dim = q.rope_head_dim;
  p.position_offset = q.rope_position_offset;
  p.cache_rows = q.rope_cache_rows;
  // K over `ksplit` warps (up to four 64-byte steps in flight each), and as many column groups
  // per CTA as keeps the grid near one CTA per SM: the activation staging (and a fused
  // producer) then runs once per 16-64 columns instead of once per 8-16
  int ksplit = std::max(1, std::min(kSkinnyMaxWarps, (p.steps + kSkinnyUnroll - 1) / kSkinnyUnroll));
  const int total_groups = (q.N + 8 * ntw - 1) / (8 * ntw);
  const int groups = std::max(1, std::min(kSkinnyMaxWarps / ksplit, (total_groups + 147) / 148));
  // a fused producer is spread over the CTA's threads: give it all sixteen warps
  if (q.prologue != kProNone) ksplit = std::max(ksplit, kSkinnyMaxWarps / groups);
  p.groups = groups;
  p.ksplit = ksplit;
  const int warps = groups * ksplit;
  const int smem = skinny_smem_bytes(p.a_stride, warps, ntw, p.raw_stride,
                                     q.prologue == kProAdaNorm ? q.K * 4 : 0);
  if (smem > 227 * 1024) return kPi05ErrUnsupported;
  const void* kernel = nullptr;
  const bool producer = q.prologue != kProNone;
  if (q.op == kOpBf16) kernel = skinny_ptr<kOpBf16>(ntw, producer);
  if (q.op == kOpE4m3) kernel = skinny_ptr<kOpE4m3>(ntw, producer);
  if (q.op == kOpS8) kernel = skinny_ptr<kOpS8>(ntw, producer);
  plan->skinny = true;
  plan->kernel = kernel;
  plan->threads = 32 * warps;
  plan->smem_bytes = smem;
  plan->grid = dim3(static_cast<unsigned>((total_groups + groups - 1) / groups), 1, 1);
  plan->swap = false;
  plan->block_n = 8 * ntw;
  plan->split_k = 1;
  plan->persistent = false;
  return kPi05Ok;
}

}  // namespace

int gemm_plan_build(const GemmProblem& q, GemmPlan* plan) {
  if (plan == nullptr || q.a.ptr == nullptr || q.b.ptr == nullptr || q.out == nullptr ||
      q.M <= 0 || q.N <= 0 || q.K <= 0 || q.nb0 <= 0 || q.nb1 <= 0 || q.status == nullptr) {
    return kPi05ErrInvalidValue;
  }
  plan->skinny = false;
  {
    // at most 16 rows: the register-streaming kernel, unless the caller pins a tcgen05 variant
    const bool pinned = q.force_swap >= 0 || q.force_block_n != 0 || q.force_split_k != 0 ||
                        q.force_two_per_sm >= 0;
    const bool want = q.force_skinny == 1 || needs_skinny(q) || (q.force_skinny < 0 && !pinned);
    if (want && q.force_skinny != 0 && skinny_fits(q)) {
      if (q.op != kOpBf16 && q.op != kOpE4m3 && q.op != kOpS8) return kPi05ErrInvalidValue;
      if (q.out_type < kOutBf16 || q.out_type > kOutF16) return kPi05ErrInvalidValue;
      if (q.out_type == kOutS32 && q.op != kOpS8) return kPi05ErrInvalidValue;
      if ((q.mode == kEpiBiasResidual || q.mode == kEpiGateResidual || q.mode == kEpiEuler) &&
          q.residual == nullptr) {
        return kPi05ErrInvalidValue;
      }
      if (q.mode == kEpiGateResidual && q.gate == nullptr) return kPi05ErrInvalidValue;
      return skinny_plan_build(q, plan);
    }
    if (q.force_skinny == 1 || needs_skinny(q)) return kPi05ErrUnsupported;
  }
  if (q.op != kOpBf16 && q.op != kOpE4m3 && q.op != kOpS8) return kPi05ErrInvalidValue;
  if (q.out_type < kOutBf16 || q.out_type > kOutF16) return kPi05ErrInvalidValue;
  if (q.out_type == kOutS32 && q.op != kOpS8) return kPi05ErrInvalidValue;
  if (q.mode == kEpiGeglu && (q.N % 128 != 0 || q.b_mn_major)) return kPi05ErrInvalidValue;
  if ((q.mode == kEpiBiasResidual || q.mode == kEpiGateResidual) && q.residual == nullptr)
    return kPi05ErrInvalidValue;
  if (q.mode == kEpiGateResidual && q.gate == nullptr) return kPi05ErrInvalidValue;
  if (q.mode == kEpiBiasPos && (q.pos == nullptr || q.pos_rows <= 0)) return kPi05ErrInvalidValue;
  if (q.b_mn_major && q.op == kOpS8) return kPi05ErrUnsupported;
  if (q.b_blocked && (q.b_mn_major || q.nb0 * q.nb1 != 1)) return kPi05ErrUnsupported;
  if (q.k_slices > 1 && (q.nb0 * q.nb1 != 1 || q.b_blocked || q.b_mn_major || q.force_split_k > 1)) {
    return kPi05ErrUnsupported;
  }
  const int k_slices = q.k_slices > 1 ? q.k_slices : 1;

  const int es = elem_bytes(q.op);
  const int block_k = 128 / es;
  bool swap = q.force_swap >= 0 ? q.force_swap != 0 : (q.M <= 64 && !q.b_mn_major);
  if (q.b_mn_major) swap = false;
  int block_n = q.force_block_n;
  if (block_n == 0) {
    if (swap) {
      block_n = q.M <= 16 ? 16 : q.M <= 32 ? 32 : 64;
    } else if (q.b_mn_major) {
      block_n = q.N > 128 ? 256 : 128;
    } else {
      // Measured on B200: a 128-row tcgen05.mma takes ~140 cycles whatever its N, so narrow
      // tiles cost MMA time but buy CTAs. Up to two CTAs share an SM (296 slots): use the
      // widest tile that still fills them, and 256 once there is more than a wave anyway.
      const long long tiles_m = (q.M + 127) / 128;
      const long long batches = (long long)q.nb0 * q.nb1 * k_slices;
      const long long tiles256 = tiles_m * ((q.N + 255) / 256) * batches;
      const long long tiles128 = tiles_m * ((q.N + 127) / 128) * batches;
      // more than a wave of 256-wide tiles that also fills its last wave to four fifths (the
      // batched action q|k|v, 3200 x 2560 x 1024: 250 tiles, 14.7 us against 17.5 us at 128)
      const long long waves256 = (tiles256 + 147) / 148;
      const bool full_waves256 = tiles256 >= 148 && tiles256 * 5 >= waves256 * 148 * 4;
      if (tiles256 >= 2 * 148 || (q.mode == kEpiGeglu && tiles256 >= 148) || full_waves256) {
        block_n = 256;
      } else if (tiles128 >= 120 || q.mode == kEpiGeglu || q.N < 128) {
        block_n = 128;
      } else {
        block_n = 64;
      }
      if (q.mode == kEpiGeglu && block_n < 128) block_n = 128;
      if (q.N % 256 != 0 && q.mode == kEpiGeglu) block_n = 128;
      // a few tiles more than SMs would cost a second, mostly empty wave: one wave of tiles
      // twice as wide is quicker (measured, M = 522, N = 2048, K = 16384: 92 -> 60 us)
      const long long tiles_now = tiles_m * ((q.N + block_n - 1) / block_n) * batches;
      if (block_n < 256 && tiles_now > 148 && tiles_now <= 222 && q.mode != kEpiGeglu) block_n *= 2;
    }
  }
  if (swap && q.M > block_n) return kPi05ErrInvalidValue;

  // more output tiles than SMs: two shallow-ring CTAs per SM overlap epilogue and main loop
  const long long tiles_planned = (long long)((swap ? q.N : q.M) + 127) / 128 *
                                  (((swap ? q.M : q.N) + block_n - 1) / block_n) * q.nb0 * q.nb1 * k_slices;
  // (K slices run the one-CTA-per-tile kernel: the persistent one walks plain batches)
  const bool multi_wave =
      k_slices > 1 ? false : q.force_two_per_sm >= 0 ? q.force_two_per_sm != 0 : tiles_planned > 148;
  int smem = 0, threads = 0;
  const void* kernel = nullptr;
  // the single-epilogue kernels write what the forward writes after that epilogue and never split
  const int act_out = q.op == kOpE4m3 ? kOutE4m3 : q.op == kOpS8 ? kOutS8 : kOutBf16;
  const int lean_out = q.mode == kEpiBiasGelu ? act_out : kOutBf16;
  const bool lean_epilogue =
      q.mode == kEpiStore || q.mode == kEpiBiasGelu || q.mode == kEpiBiasResidual ||
      q.mode == kEpiGateResidual;
  const int lean_mode = (g_single_epilogue && lean_epilogue && !swap && !q.b_mn_major && q.force_split_k <= 1 &&
                         q.out_type == lean_out)
                            ? q.mode
                            : -1;
  if (q.op == kOpBf16) kernel = select_kernel<kOpBf16>(block_n, swap, q.b_mn_major, multi_wave, lean_mode, &smem, &threads);
  if (q.op == kOpE4m3) kernel = select_kernel<kOpE4m3>(block_n, swap, q.b_mn_major, multi_wave, lean_mode, &smem, &threads);
  if (q.op == kOpS8) kernel = select_kernel<kOpS8>(block_n, swap, q.b_mn_major, multi_wave, lean_mode, &smem, &threads);
  if (kernel == nullptr) return kPi05ErrUnsupported;
  plan->threads = threads;
  plan->persistent = false;
  plan->multi_wave_candidate = multi_wave && !swap;

  // A-side map = the operand with 128-row tiles.
  int rc;
  if (!swap) {
    rc = encode_operand_map(&plan->tmap_a, q.op, q.a.ptr, q.K, q.M, q.nb0, q.nb1, q.a.ld, q.a.sb0, q.a.sb1,
                    block_k, 128);
    if (rc != kPi05Ok) return rc;
    if (q.b_mn_major) {
      // [K, N] row-major: boxes of one 128-byte run along N by one K block of rows
      rc = encode_operand_map(&plan->tmap_b, q.op, q.b.ptr, q.N, q.K, q.nb0, q.nb1, q.b.ld, q.b.sb0,
                      q.b.sb1, block_k, block_k);
    } else if (q.b_blocked) {
      rc = encode_operand_map(&plan->tmap_b, q.op, q.b.ptr, block_k, q.N, (q.K + block_k - 1) / block_k, 1,
                      block_k, (long long)q.N * block_k, 0, block_k, block_n);
    } else {
      rc = encode_operand_map(&plan->tmap_b, q.op, q.b.ptr, q.K, q.N, q.nb0, q.nb1, q.b.ld, q.b.sb0,
                      q.b.sb1, block_k, block_n);
    }
    if (rc != kPi05Ok) return rc;
  } else {
    if (q.b_blocked) {
      rc = encode_operand_map(&plan->tmap_a, q.op, q.b.ptr, block_k, q.N, (q.K + block_k - 1) / block_k, 1,
                      block_k, (long long)q.N * block_k, 0, block_k, 128);
    } else {
      rc = encode_operand_map(&plan->tmap_a, q.op, q.b.ptr, q.K, q.N, q.nb0, q.nb1, q.b.ld, q.b.sb0,
                      q.b.sb1, block_k, 128);
    }
    if (rc != kPi05Ok) return rc;
    rc = encode_operand_map(&plan->tmap_b, q.op, q.a.ptr, q.K, q.M, q.nb0, q.nb1, q.a.ld, q.a.sb0, q.a.sb1,
                    block_k, block_n);
    if (rc != kPi05Ok) return rc;
  }

  GemmParams& p = plan->params;
  p.rows_a = swap ? q.N : q.M;
  p.rows_b = swap ? q.M : q.N;
  p.num_kb = (q.K + block_k - 1) / block_k;
  p.nb0 = q.nb0;
  p.k_slice_kb = 0;
  if (k_slices > 1) {
    p.k_slice_kb = (p.num_kb + k_slices - 1) / k_slices;
    p.num_kb = p.k_slice_kb;
    p.nb0 = k_slices;
  }
  p.out = q.out;
  p.ldc = q.ldc;
  p.out_sb0 = q.out_sb0;
  p.out_sb1 = q.out_sb1;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(q.residual);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(q.bias);
  p.col_scale = q.col_scale;
  p.row_scale = q.row_scale;
  p.row_scale_sb0 = q.row_scale_sb0;
  p.pos = reinterpret_cast<const __nv_bfloat16*>(q.pos);
  p.gate = reinterpret_cast<const __nv_bfloat16*>(q.gate);
  p.alpha = q.alpha;
  p.out_inv_scale = q.out_inv_scale;
  p.pos_rows = q.pos_rows;
  p.pos_ld = q.pos_ld;
  p.mode = q.mode;
  p.out_type = q.out_type;
  p.group_a = 1;
  p.status = q.status;
  p.wait_polls = g_wait_polls;
  p.drop_load_kb = g_drop_load_kb;

  const int tiles_x = (p.rows_a + 127) / 128, tiles_y = (p.rows_b + block_n - 1) / block_n;
  const long long tiles = (long long)tiles_x * tiles_y * q.nb0 * q.nb1 * k_slices;
  int split = 1;
  if (q.partials != nullptr && q.tile_counters != nullptr && q.out_type != kOutS32 &&
      q.force_split_k != 1) {
    if (q.force_split_k > 1) {
      split = q.force_split_k;
    } else if (swap) {
      // weight streaming for a handful of rows: spread the K range until ~one CTA per SM
      if (p.num_kb >= 4) split = static_cast<int>(std::min<long long>(p.num_kb / 2, 148 / tiles));
    }
    // (activations on the 128-row side: the last-arrival reduction of 128 x BLOCK_N partial
    // tiles costs more than the shorter K range saves at every shape measured, so the
    // automatic choice never splits there)
    split = std::max(1, std::min(split, p.num_kb));
    const size_t need = static_cast<size_t>(tiles) * split * 128 * block_n * 4;
    if (need > q.partials_bytes || tiles > q.max_tiles) {
      // an explicit split request that does not fit the scratch is an error; the
      // automatic choice quietly stays single-pass
      if (q.force_split_k > 1 && split > 1) return kPi05ErrScratchLimit;
      split = 1;
    }
  }
  p.kb_per_split = (p.num_kb + split - 1) / split;
  split = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  if (lean_mode >= 0 && split != 1) return kPi05ErrInvalidValue;  // by construction; never split
  p.split_k = split;
  p.partials = reinterpret_cast<uint32_t*>(q.partials);
  p.tile_counters = q.tile_counters;
  p.static_a = (swap && q.b_static) ? 1 : 0;
  p.static_b = (!swap && q.b_static) ? 1 : 0;
  p.blocked_a = (swap && q.b_blocked) ? 1 : 0;
  p.blocked_b = (!swap && q.b_blocked) ? 1 : 0;
  plan->split_k = split;
  plan->grid = dim3(tiles_x, tiles_y, q.nb0 * q.nb1 * k_slices * split);
  if (plan->multi_wave_candidate && split == 1) {
    const void* persistent = nullptr;
    // GeGLU too has a kernel of its own here (FP8 out of an FP8 GEMM, bf16 out of a bf16 one)
    const int geglu_out = act_out;
    const int persistent_lean =
        lean_mode >= 0 ? lean_mode
        : (g_single_epilogue && q.mode == kEpiGeglu && !q.b_mn_major && q.out_type == geglu_out)
            ? static_cast<int>(kEpiGeglu)
            : -1;
    if (q.op == kOpBf16) persistent = select_persistent<kOpBf16>(block_n, q.b_mn_major, persistent_lean, &smem, &threads);
    if (q.op == kOpE4m3) persistent = select_persistent<kOpE4m3>(block_n, q.b_mn_major, persistent_lean, &smem, &threads);
    if (q.op == kOpS8) persistent = select_persistent<kOpS8>(block_n, q.b_mn_major, persistent_lean, &smem, &threads);
    if (persistent != nullptr) {
      kernel = persistent;
      plan->persistent = true;
      plan->threads = threads;
      plan->tiles_a = tiles_x;
      plan->tiles_b = tiles_y;
      // row tiles per raster group: about 24 MB of A, which stays in L2 while the group
      // sweeps the column tiles (measured on the batch-64 gate_up launch: HBM reads fell from
      // 1.45 GB, 10 x the operands, when all 261 row tiles formed one group)
      const long long a_tile_bytes = 128LL * q.K * es;
      const long long rows_in_l2 = std::max<long long>(8, (24LL << 20) / std::max<long long>(1, a_tile_bytes));
      plan->params.group_a = static_cast<int>(std::min<long long>(tiles_x, rows_in_l2));
      plan->total_tiles = static_cast<int>(tiles);
      int sms = 148;
      int device = 0;
      if (cudaGetDevice(&device) == cudaSuccess) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
      }
      plan->grid = dim3(static_cast<unsigned>(std::min<long long>(tiles, sms)), 1, 1);
    }
  }
  plan->smem_bytes = smem;
  plan->kernel = kernel;
  plan->swap = swap;
  plan->block_n = block_n;
  return kPi05Ok;
}

cudaError_t gemm_plan_launch(const GemmPlan& plan, cudaStream_t stream) {
  if (plan.skinny) {
    void* skinny_args[1] = {const_cast<SkinnyParams*>(&plan.skinny_params)};
    cudaLaunchConfig_t config = {};
    config.gridDim = plan.grid;
    config.blockDim = dim3(plan.threads);
    config.dynamicSmemBytes = plan.smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelExC(&config, plan.kernel, skinny_args);
  }
  void* args[6] = {const_cast<CUtensorMap*>(&plan.tmap_a), const_cast<CUtensorMap*>(&plan.tmap_b),
                   const_cast<GemmParams*>(&plan.params), const_cast<int*>(&plan.tiles_a),
                   const_cast<int*>(&plan.tiles_b), const_cast<int*>(&plan.total_tiles)};
  cudaLaunchConfig_t config = {};
  config.gridDim = plan.grid;
  config.blockDim = dim3(plan.threads);
  config.dynamicSmemBytes = plan.smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelExC(&config, plan.kernel, args);
}

}  // namespace pi05
