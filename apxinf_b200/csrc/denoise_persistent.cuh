// The B=1 action expert's whole flow-matching loop as ONE cooperative launch.
//
// With at most 16 action rows every launch of the denoise loop is a few microseconds of work
// behind a dependent-launch boundary that costs about as much again; ten flow steps of
// eighteen layers are some 1300 of them. Here the same per-projection and attention bodies
// (gemm_skinny.cuh, fmha_rows.cuh) run as STAGES of one persistent kernel, one CTA per SM:
//
//   * the stage table (one entry per projection / attention of every layer and step, with the
//     very parameter blocks the stand-alone kernels take) lives in global memory; each CTA keeps
//     the current and the next entry in shared memory;
//   * stages are ordered by a grid barrier: a monotonic arrival counter in global memory
//     (zeroed by the host before every launch). A CTA that finished stage s adds one, issues
//     the static part of stage s + 1 (its share of the weight stream into registers, style /
//     scale / bias vectors), and only then waits for the counter to reach (s + 1) * grid; the
//     weight traffic of a stage thus overlaps the tail of the one before it, as it does across
//     programmatic dependent launches, but the hand-over costs an L2 round trip instead of a
//     grid drain and a launch;
//   * the adaptive RMSNorms run as the staging step of the projection that consumes them, so a
//     layer is five stages: q|k|v (+ RoPE, cache write), attention, o (+ gated residual),
//     gate|up (+ GeGLU), down (+ gated residual);
//   * attention splits the keys over eight CTAs per 16-row query tile as the cluster kernel
//     does, and exchanges the partials through a global scratch and a per-tile flag.
//
// Co-residency of all CTAs is guaranteed by launching cooperatively
// (cudaLaunchAttributeCooperative); every wait on the counter or on a flag is bounded: after
// `spin_limit` polls the CTA records kDenoiseTimeout in the status word and leaves the kernel,
// and the others follow when their own waits run out. Nothing here uses tensor memory, TMA or
// clusters, so leaving is always safe once the CTA's own cp.async groups have landed.
//
// Replaces the per-layer launch sequence of the reference's action expert
// (crates/apxinf-model/src/pi05/bf16_executor.rs:89-212, fp8_executor.rs:216-462).
#pragma once

#include "fmha_rows.cuh"
#include "gemm_skinny.cuh"

namespace pi05 {

enum DenoiseStageKind : int { kStageGemm1 = 0, kStageGemm2 = 1, kStageAttention = 2 };

constexpr int kDenoiseThreads = 32 * kSkinnyMaxWarps;  // 512
constexpr int kDenoiseTimeout = 40;                    // status word: a barrier or flag wait ran out

struct alignas(16) DenoiseStage {
  int kind;
  int ctas;     // CTAs 0 .. ctas - 1 take part
  int threads;  // threads 0 .. threads - 1 of those
  int epoch;    // attention: how many attention stages ran before this one
  union {
    SkinnyParams gemm;
    FmhaRowsParams attention;
  };
};
static_assert(sizeof(DenoiseStage) % 16 == 0, "stage entries are copied in 16-byte words");
constexpr int kStageWords = static_cast<int>(sizeof(DenoiseStage) / 16);

struct DenoiseParams {
  const DenoiseStage* stages;
  int count;
  unsigned* barrier;     // arrival counter, zero at launch
  unsigned* tile_flags;  // [query tiles] attention exchange flags, zero at launch
  float* scratch;        // [query tiles][8][rows_partial_floats(head_dim)]
  int* status;           // device status word, 0 = ok
  unsigned spin_limit;   // polls before a wait gives up
  int skip_arrival;      // diagnostics: CTA 0 does not arrive after this stage (-1: none), so
                         // that every wait on the counter runs out
};

namespace denoise_detail {

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Polls until *p >= target; false when `limit` polls were not enough.
__device__ __forceinline__ bool wait_at_least(const unsigned* p, unsigned target, unsigned limit) {
  for (unsigned it = 0; it < limit; ++it) {
    if (ld_acquire(p) >= target) return true;
  }
  return false;
}

struct StageCtx {
  int cta, tid, threads;
  const DenoiseParams* d;
  unsigned barrier_target;  // arrivals that end the previous stage
  int* dead;                // shared: this CTA gave up
  // attention exchange
  float* scratch;
  unsigned* flags;
  unsigned target;

  __device__ __forceinline__ void sync() const {
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
  }
  __device__ __forceinline__ void give_up() const {
    atomicCAS(d->status, 0, kDenoiseTimeout);
    *dead = 1;
  }
  // the producer stage is complete on every CTA
  __device__ __forceinline__ void wait() const {
    if (tid == 0 && barrier_target != 0 && *dead == 0) {
      if (!wait_at_least(d->barrier, barrier_target, d->spin_limit)) give_up();
    }
    sync();
  }

  __device__ __forceinline__ void wait_flag(const unsigned* flag, unsigned value) const {
    if (*dead == 0 && !wait_at_least(flag, value, d->spin_limit)) give_up();
  }
};

}  // namespace denoise_detail

// grid: one CTA per SM (<= the cooperative-launch limit), block: kDenoiseThreads.
// dynamic shared memory: two stage entries + the largest stage's working set.
template <int OP>
__global__ void __launch_bounds__(kDenoiseThreads, 1) denoise_persistent_kernel(const DenoiseParams d) {
  using namespace denoise_detail;
  extern __shared__ __align__(128) uint8_t denoise_smem[];
  __shared__ int s_dead;
  uint4* slots = reinterpret_cast<uint4*>(denoise_smem);  // [2][kStageWords]
  uint8_t* work = denoise_smem + ((2 * sizeof(DenoiseStage) + 127) / 128) * 128;
  const int tid = threadIdx.x;
  const int cta = blockIdx.x;
  const unsigned grid = gridDim.x;

  if (tid == 0) s_dead = 0;
  for (int i = tid; i < kStageWords; i += kDenoiseThreads) {
    slots[i] = __ldg(reinterpret_cast<const uint4*>(d.stages) + i);
  }
  __syncthreads();

  for (int s = 0; s < d.count; ++s) {
    const DenoiseStage& st = *reinterpret_cast<const DenoiseStage*>(slots + (s & 1) * kStageWords);
    // the next entry comes in behind this stage's own work (last warp: it has the fewest roles)
    // (asynchronous copies: the warp goes straight on to its part of the stage)
    if (s + 1 < d.count && tid >= kDenoiseThreads - 32) {
      const uint4* next = reinterpret_cast<const uint4*>(d.stages + s + 1);
      uint4* slot = slots + ((s + 1) & 1) * kStageWords;
      for (int i = tid - (kDenoiseThreads - 32); i < kStageWords; i += 32) {
        rows_detail::cp_async16(slot + i, next + i);
      }
      rows_detail::cp_async_commit();
    }
    StageCtx ctx;
    ctx.cta = cta;
    ctx.tid = tid;
    ctx.threads = st.threads;
    ctx.d = &d;
    ctx.barrier_target = grid * static_cast<unsigned>(s);
    ctx.dead = &s_dead;
    ctx.scratch = d.scratch;
    ctx.flags = d.tile_flags;
    ctx.target = static_cast<unsigned>(kRowsCluster) * static_cast<unsigned>(st.epoch + 1);
    if (cta < st.ctas) {
      if (tid < st.threads) {
        if (st.kind == kStageGemm1) {
          skinny_body<OP, 1, true>(st.gemm, work, ctx);
        } else if (st.kind == kStageGemm2) {
          skinny_body<OP, 2, true>(st.gemm, work, ctx);
        } else {
          fmha_rows_body<false>(st.attention, work, ctx);
        }
      }
    } else if (tid == 0 && ctx.barrier_target != 0 && s_dead == 0) {
      // no part in this stage, but nobody runs ahead of the barrier: arrivals are counted, so a
      // CTA that skipped its way forward would be taken for several
      if (!wait_at_least(d.barrier, ctx.barrier_target, d.spin_limit)) ctx.give_up();
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();  // the stage is done on this CTA and the next entry has landed
    if (s_dead != 0) break;
    if (tid == 0 && !(cta == 0 && s == d.skip_arrival)) {
      __threadfence();
      atomicAdd(d.barrier, 1u);
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
}

}  // namespace pi05
