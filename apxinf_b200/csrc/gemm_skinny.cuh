// Linear layers with at most 16 activation rows (the B=1 action expert: 10 rows per flow
// step and layer). These launches are bound by weight streaming and by latency, not by
// arithmetic: 2.6 MB of weights against 52 MFLOP. The tcgen05 path spends its time on set-up
// (tensor maps, mbarriers, TMEM, a two-phase split-K through global memory); this kernel has
// none of that:
//
//   * every warp issues its whole share of the weight stream as 16-byte global loads straight
//     into registers BEFORE the programmatic-dependency wait (weights are static), so the HBM
//     traffic of a layer overlaps the tail of the previous kernel;
//   * the activations (<= 16 rows) are staged once per CTA in shared memory, and the producer
//     that used to be a kernel of its own runs as that staging step: adaptive RMSNorm (+
//     quantisation to e4m3 / int8), plain quantisation, or the merge of the key-split
//     attention partials;
//   * dot products on mma.sync m16n8k32 (e4m3, s8) / m16n8k16 (bf16) fragments loaded directly
//     from those registers, K split over the warps of a CTA and reduced through shared memory in
//     a fixed order (no atomics, no second launch);
//   * the epilogue pairs two 8-column tiles in one thread, so GeGLU (gate / up features 64
//     packed rows apart) and rotate-half RoPE (features 128 apart) with the K/V-cache write need
//     no exchange.
//
// Same contract and rounding points as the GEMM family of gemm_umma.cuh (see EpilogueMode
// there); replaces for M <= 16 the reference's cuBLAS / cuBLASLt calls plus the row kernels
// around them (crates/apxinf-model/src/pi05/bf16_executor.rs:89-157: adaptive_rms_bf16,
// apply_q_write_kv_bf16, geglu_bf16, adaptive_gate_residual_rms_bf16; fp8_executor.rs:216-314).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "gemm_umma.cuh"
#include "launch.cuh"

namespace pi05 {

enum SkinnyPrologue : int {
  kProNone = 0,      // `a` is already in the operand type
  kProAdaNorm = 1,   // `a` bf16 hidden rows: adaptive RMSNorm with `style`, then to the operand type
  kProQuantize = 2,  // `a` bf16 rows: to the operand type (static scale, or per-row int8)
  kProRmsNorm = 3,   // `a` bf16 hidden rows: RMSNorm (weight = 1), then to the operand type
};

// Extra epilogues of the skinny kernel (continuing EpilogueMode).
constexpr int kEpiRope = 7;   // packed q|k|v projection: rotate-half RoPE, Q out, K/V cache rows
constexpr int kEpiEuler = 8;  // o = extra + dt * rb(rb(v) + bias): velocity head + Euler update

struct SkinnyParams {
  const void* a;          // [M, lda] operand type, or bf16 for the prologues
  long long lda;          // elements
  const uint8_t* w;       // [N, ldw] K-major weights (operand type)
  long long ldw_bytes;    // row pitch in bytes (multiple of 16)
  int M, N, K;            // K in elements
  int kbytes;             // K * element size rounded up to 16
  int a_stride;           // shared-memory row pitch of the staged activations (bytes, = 64 mod 128)
  int raw_stride;         // shared-memory row pitch of the producer's bf16 input (fused prologues)
  int steps;              // 64-byte K steps per weight row
  int tile_offset;        // packed-row distance of the second 8-column tile (NTW == 2)
  int groups;             // column groups per CTA
  int ksplit;             // warps sharing one group's K range
  int prologue;
  const __nv_bfloat16* style;  // adaptive norm: scale | shift, each K long
  float eps;
  float a_inv_scale;      // static quantisation of the staged activations
  int dynamic_rows;       // int8 prologues: per-row scale computed here
  // epilogue (same meaning as GemmParams)
  void* out;
  long long ldc;
  const __nv_bfloat16* residual;
  const __nv_bfloat16* bias;
  const float* col_scale;
  const float* row_scale;  // per-row activation scale of a caller-quantised int8 operand
  const __nv_bfloat16* gate;
  float alpha;
  float out_inv_scale;
  int mode;
  int out_type;
  float dt;                // kEpiEuler
  // kEpiRope
  void* q_out;             // bf16 [rows, q_heads, head_dim]
  void* k_cache;           // bf16 [samples, cache_rows, head_dim]
  void* v_cache;
  const float* cos_table;  // f32 [positions, head_dim / 2]
  const float* sin_table;
  int tokens, q_heads, head_dim, position_offset, cache_rows;
};

namespace skinny {

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 16 bytes that an earlier kernel of the stream may have written: read at L2 (never through a
// line an overlapping predecessor left in L1). As an explicit global load it can also be
// scheduled across the shared-memory stores around it, unlike a generic-pointer load.
__device__ __forceinline__ uint4 ldg_l2(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int OP>
__device__ __forceinline__ void mma(uint32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                    uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (OP == kOpE4m3) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else if constexpr (OP == kOpS8) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(pairs[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}


// Stage one bf16 row (already transformed into y[]) into the activation tile in the operand type.
template <int OP>
__device__ __forceinline__ void store_staged(uint8_t* row_smem, int chunk, const float (&y)[8],
                                             float inv_scale) {
  if constexpr (OP == kOpBf16) {
    uint4 raw;
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
    *reinterpret_cast<uint4*>(row_smem + chunk * 16) = raw;
  } else if constexpr (OP == kOpE4m3) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= static_cast<uint32_t>(to_e4m3(y[i] * inv_scale)) << (8 * i);
      hi |= static_cast<uint32_t>(to_e4m3(y[4 + i] * inv_scale)) << (8 * i);
    }
    *reinterpret_cast<uint2*>(row_smem + chunk * 8) = make_uint2(lo, hi);
  } else {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= static_cast<uint32_t>(to_s8(y[i] * inv_scale)) << (8 * i);
      hi |= static_cast<uint32_t>(to_s8(y[4 + i] * inv_scale)) << (8 * i);
    }
    *reinterpret_cast<uint2*>(row_smem + chunk * 8) = make_uint2(lo, hi);
  }
}

}  // namespace skinny

constexpr int kSkinnyUnroll = 4;      // 64-byte K steps a warp keeps in flight per tile
// Up to 16 warps per CTA: what bounds these launches is how many weight bytes are in flight
// before the dependency wait (capping CTAs at 8 warps, so that a successor's CTAs always fit
// beside them, measured 25 % slower: 13.0 against 10.6 ms for the whole B=1 forward).
constexpr int kSkinnyMaxWarps = 16;
// (row, 8-element chunk) items a thread may hold in registers through a fused producer
constexpr int kSkinnyFastItems = 4;

// `raw_stride`: row pitch of the bf16 copy of the producer's input (fused prologues), else 0;
// `style_bytes`: the adaptive norm's scale | shift vectors (2 K bf16), else 0
__host__ __device__ constexpr int skinny_smem_bytes(int a_stride, int warps, int ntw, int raw_stride,
                                                    int style_bytes) {
  return 16 * a_stride + warps * ntw * 128 * 4 + (kSkinnyMaxWarps * 16 + 16 + 16) * 4 + 16 * raw_stride +
         style_bytes + 16;
}

// A CTA holds `groups` column groups (NTW tiles of 8 packed weight rows each); the `ksplit`
// warps of a group share its K range. grid.x = ceil(column groups / groups),
// block = 32 * groups * ksplit. All warps take part in staging the activations.
//
// The body is shared by two callers through `ctx`: the stand-alone kernel below (one launch per
// projection, ordered by programmatic dependent launch) and the persistent denoise kernel
// (denoise_persistent.cuh: the same projections as stages of one cooperative launch, ordered
// by a grid barrier). `ctx` gives the CTA index, the thread index and count of the threads
// taking part, their barrier, and the wait for the producer of the activations. Everything an
// earlier stage may have written is read at L2 (ld.global.cg), never through L1.
struct SkinnyLaunchCtx {
  int cta, tid, threads;
  __device__ __forceinline__ void sync() const { __syncthreads(); }
  __device__ __forceinline__ void wait() const { pdl_wait(); }
};

// PRO: the fused producers (prologue != kProNone) are compiled in. The projections without one,
// which are nearly all launches, run the variant without that code: fewer registers and a
// shorter instruction stream for launches that are bound by exactly that.
template <int OP, int NTW, bool PRO, class Ctx>
__device__ __forceinline__ void skinny_body(const SkinnyParams& p, uint8_t* skinny_smem, const Ctx& ctx) {
  constexpr int kElem = OP == kOpBf16 ? 2 : 1;
  const int mode = p.mode;  // (a compile-time epilogue on top of PRO measured no further gain)
  const int tid = ctx.tid, nthreads = ctx.threads, cta = ctx.cta;
  const int warps = nthreads >> 5;
  const int ksplit = p.ksplit;
  uint8_t* a_tile = skinny_smem;                                          // [16][a_stride]
  uint32_t* red = reinterpret_cast<uint32_t*>(a_tile + 16 * p.a_stride);  // [warps][NTW][128]
  float* s_part = reinterpret_cast<float*>(red + warps * NTW * 128);      // [kSkinnyMaxWarps][16]
  float* s_stat = s_part + kSkinnyMaxWarps * 16;                          // [16] per-row statistic
  float* s_rowscale = s_stat + 16;                                        // [16]
  uint8_t* raw_tile = reinterpret_cast<uint8_t*>(s_rowscale + 16);        // [M][raw_stride] bf16 (prologues)

  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group_in_cta = warp / ksplit;
  const int kslice = warp - group_in_cta * ksplit;
  const int group = cta * p.groups + group_in_cta;

  // packed weight rows of this warp's tiles
  int n0[NTW];
  if constexpr (NTW == 2) {
    // groups walk the rows that have a partner `tile_offset` further on:
    // [0, off) pairs with [off, 2 off), [2 off, 3 off) with [3 off, 4 off), ...
    const int per_block = p.tile_offset / 8;
    const int block = group / per_block;
    const int in_block = group - block * per_block;
    n0[0] = block * 2 * p.tile_offset + in_block * 8;
    n0[1] = n0[0] + p.tile_offset;
  } else {
    n0[0] = group * 8;
  }

  // ---- weight stream: the first kSkinnyUnroll steps of this warp, before the dependency wait ----
  uint4 wq[NTW][kSkinnyUnroll];
  auto load_weights = [&](int base) {
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int row = n0[j] + g;
#pragma unroll
      for (int u = 0; u < kSkinnyUnroll; ++u) {
        const int step = base + u * ksplit;
        const int byte = step * 64 + t * 16;
        if (row < p.N && step < p.steps && byte < p.kbytes) {
          wq[j][u] = skinny::ldg_stream(p.w + static_cast<long long>(row) * p.ldw_bytes + byte);
        } else {
          wq[j][u] = make_uint4(0, 0, 0, 0);
        }
      }
    }
  };
  load_weights(kslice);

  // Static vectors are fetched ahead of the dependency wait too: the adaptive norm's style
  // (to shared memory) and the per-column scale / bias / gate and RoPE factors of the output
  // element this thread will finish.
  uint8_t* style_tile = raw_tile + 16 * p.raw_stride;  // [2][K] bf16: scale | shift
  if (PRO && p.prologue == kProAdaNorm) {
    const int chunks = (2 * p.K) >> 3;
    for (int i = tid; i < chunks; i += nthreads) {
      *reinterpret_cast<uint4*>(style_tile + i * 16) =
          __ldg(reinterpret_cast<const uint4*>(p.style) + i);
    }
  }
  float pre_scale[NTW], pre_bias[NTW], pre_gate[NTW], pre_cos = 1.0f, pre_sin = 0.0f;
  int en[NTW];         // output columns of the epilogue item this thread finishes first
  bool mine = false;   // ... if it has one
  {
    const int eg = tid >> 7, e = tid & 127;
    const int egroup = cta * p.groups + eg;
    if constexpr (NTW == 2) {
      const int per_block = p.tile_offset / 8;
      const int block = egroup / per_block;
      en[0] = block * 2 * p.tile_offset + (egroup - block * per_block) * 8 + (e & 7);
      en[1] = en[0] + p.tile_offset;
    } else {
      en[0] = egroup * 8 + (e & 7);
    }
    mine = eg < p.groups && (e >> 3) < p.M;
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const bool in = mine && en[j] < p.N;
      pre_scale[j] = p.col_scale != nullptr && in ? __ldg(p.col_scale + en[j]) : 1.0f;
      pre_bias[j] = p.bias != nullptr && in ? __bfloat162float(p.bias[en[j]]) : 0.0f;
      pre_gate[j] = p.gate != nullptr && in ? __bfloat162float(p.gate[en[j]]) : 0.0f;
    }
    if (mode == kEpiRope && mine && en[0] < p.N) {
      const int half = p.head_dim >> 1;
      const int head = en[0] / p.head_dim;
      if (head < p.q_heads + 1) {
        const int token = (e >> 3) % p.tokens;
        const long long at = static_cast<long long>(p.position_offset + token) * half + (en[0] - head * p.head_dim);
        pre_cos = __ldg(p.cos_table + at);
        pre_sin = __ldg(p.sin_table + at);
      }
    }
  }

  ctx.wait();

  // the residual element of the thread's first epilogue item: asked for now, used at the end
  float pre_extra[NTW];
#pragma unroll
  for (int j = 0; j < NTW; ++j) pre_extra[j] = 0.0f;
  if ((mode == kEpiBiasResidual || mode == kEpiGateResidual || mode == kEpiEuler) && mine &&
      !out_is_raw(p.out_type)) {
    const int row = (tid & 127) >> 3;
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      if (en[j] < p.N) {
        pre_extra[j] = __bfloat162float(__ldcg(p.residual + static_cast<long long>(row) * p.ldc + en[j]));
      }
    }
  }

  // ---- activations -> shared memory in the operand type ----
  {
    // Zero what the main loop reads but nothing below writes: the rows beyond M (a NaN pattern in
    // stale shared memory times a zero weight would still poison a sum) and, when K does not end
    // on a 64-byte step, each row's tail. Neither overlaps the rows staged below.
    {
      uint4* beyond = reinterpret_cast<uint4*>(a_tile + p.M * p.a_stride);
      const int words = (16 - p.M) * p.a_stride / 16;
      for (int i = tid; i < words; i += nthreads) beyond[i] = make_uint4(0, 0, 0, 0);
      const int tail = p.steps * 4 - p.kbytes / 16;  // 16-byte chunks between K and the last step's end
      if (tail > 0) {
        for (int i = tid; i < p.M * tail; i += nthreads) {
          const int r = i / tail, c = i - r * tail;
          *reinterpret_cast<uint4*>(a_tile + r * p.a_stride + p.kbytes + c * 16) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    if (tid < 16) s_rowscale[tid] = 1.0f;
    // global -> shared copy of the rows: up to eight 16-byte loads in flight per thread, so the
    // ten rows of the widest projection (4096 e4m3 = 2560 chunks over 512 threads) cost one L2
    // round trip, not two. (row, chunk) of a thread's items are walked, not divided out: these
    // launches are bound by the instructions each warp has to get through.
    constexpr int kCopyDepth = 8;
    auto copy_rows = [&](uint8_t* dst, int dst_stride, int row_bytes, long long src_pitch) {
      const int chunks = row_bytes / 16;
      const int total = p.M * chunks;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.a);
      const int dr = nthreads / chunks, dc = nthreads - dr * chunks;  // one stride of the walk
      int r = tid / chunks, c = tid - r * chunks;
      for (int i0 = tid; i0 < total; i0 += kCopyDepth * nthreads) {
        uint4 v[kCopyDepth];
        int r0 = r, c0 = c;
#pragma unroll
        for (int u = 0; u < kCopyDepth; ++u) {
          if (i0 + u * nthreads < total) v[u] = skinny::ldg_l2(src + r * src_pitch + c * 16);
          r += dr;
          c += dc;
          if (c >= chunks) {
            c -= chunks;
            ++r;
          }
        }
#pragma unroll
        for (int u = 0; u < kCopyDepth; ++u) {
          if (i0 + u * nthreads < total) *reinterpret_cast<uint4*>(dst + r0 * dst_stride + c0 * 16) = v[u];
          r0 += dr;
          c0 += dc;
          if (c0 >= chunks) {
            c0 -= chunks;
            ++r0;
          }
        }
      }
    };
    if (!PRO || p.prologue == kProNone) {
      copy_rows(a_tile, p.a_stride, p.kbytes, p.lda * kElem);
      if (p.row_scale != nullptr && tid < p.M) s_rowscale[tid] = __ldcg(p.row_scale + tid);
    } else if constexpr (!PRO) {
      // unreachable: plans with a fused producer take the PRO variant
    } else if (!(OP == kOpS8 && p.dynamic_rows) && p.M * (p.K >> 3) <= kSkinnyFastItems * nthreads) {
      // Producer fused into the staging, the short way: every thread keeps its (row, 8-element
      // chunk) items in registers from the global load to the operand-type store, so a tile costs
      // one L2 round trip, one barrier (row statistics by shuffles inside 32-chunk segments, the
      // segments' partials through shared memory, added in a fixed order by every thread that
      // needs the row) and a few hundred instructions per thread.
      const int chunks = p.K >> 3;
      const int items = p.M * chunks;
      const bool normed = p.prologue == kProAdaNorm || p.prologue == kProRmsNorm;
      const int seg = chunks >= 32 ? 32 : chunks;
      const int parts = (chunks + 31) >> 5;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(p.a);
      uint4 held[kSkinnyFastItems];
#pragma unroll
      for (int j = 0; j < kSkinnyFastItems; ++j) {
        const int item = tid + j * nthreads;
        held[j] = make_uint4(0, 0, 0, 0);
        if (item < items) {
          const int r = item / chunks, c = item - r * chunks;
          held[j] = skinny::ldg_l2(src + static_cast<long long>(r) * p.lda * 2 + c * 16);
        }
      }
      if (normed) {
#pragma unroll
        for (int j = 0; j < kSkinnyFastItems; ++j) {
          const int item = tid + j * nthreads;
          if (j * nthreads < items) {  // uniform over the CTA: whole warps take the shuffles
            float x[8];
            skinny::unpack8(held[j], x);
            float sq = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += x[e] * x[e];
            for (int o = seg >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            const int r = item / chunks, c = item - r * chunks;
            if (item < items && (c & (seg - 1)) == 0) s_part[r * 16 + (c >> 5)] = sq;
          }
        }
      }
      ctx.sync();  // statistics partials, the style vectors and the zero fill are in place
#pragma unroll
      for (int j = 0; j < kSkinnyFastItems; ++j) {
        const int item = tid + j * nthreads;
        if (item < items) {
          const int r = item / chunks, c = item - r * chunks;
          float inv = 1.0f;
          if (normed) {
            float total = 0.0f;
            for (int part = 0; part < parts; ++part) total += s_part[r * 16 + part];
            inv = rsqrtf(total / static_cast<float>(p.K) + p.eps);
          }
          float y[8];
          skinny::unpack8(held[j], y);
          if (p.prologue == kProAdaNorm) {
            float sc[8], sh[8];
            skinny::unpack8(*reinterpret_cast<const uint4*>(style_tile + c * 16), sc);
            skinny::unpack8(*reinterpret_cast<const uint4*>(style_tile + p.K * 2 + c * 16), sh);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = (y[e] * inv) * (1.0f + sc[e]) + sh[e];
          } else if (normed) {
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = y[e] * inv;
          }
          if constexpr (OP == kOpS8) {
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = round_bf16(y[e]);
          }
          skinny::store_staged<OP>(a_tile + r * p.a_stride, c, y, p.a_inv_scale);
        }
      }
    } else {
      // The producer's bf16 input rows come to shared memory first (one round trip for the whole
      // tile); then one warp per row: statistic by shuffles, transform, operand-type store.
      copy_rows(raw_tile, p.raw_stride, p.K * 2, p.lda * 2);
      ctx.sync();
      const int chunks = p.K >> 3;
      const bool normed = p.prologue == kProAdaNorm || p.prologue == kProRmsNorm;
      // Every thread takes (row, 8-element chunk) items, so the ten rows of a tile are spread
      // over the whole CTA (a warp per row leaves a 700-instruction serial chain per warp: 2.5 us).
      // Row statistics are reduced in two fixed-order levels: shuffles inside a segment of
      // `seg` consecutive chunks, then the row's segment partials from shared memory.
      const int seg = chunks >= 32 ? 32 : chunks;  // chunks is a multiple of 32 or a power of two below it
      const int parts = (chunks + 31) >> 5;
      const int items = p.M * chunks;
      auto transformed = [&](int r, int c, float inv, float (&y)[8]) {
        skinny::unpack8(*reinterpret_cast<const uint4*>(raw_tile + r * p.raw_stride + c * 16), y);
        if (p.prologue == kProAdaNorm) {
          float sc[8], sh[8];
          skinny::unpack8(*reinterpret_cast<const uint4*>(style_tile + c * 16), sc);
          skinny::unpack8(*reinterpret_cast<const uint4*>(style_tile + p.K * 2 + c * 16), sh);
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = (y[e] * inv) * (1.0f + sc[e]) + sh[e];
        } else if (normed) {
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = y[e] * inv;
        }
        if constexpr (OP == kOpS8) {
          // the W8A8 path stores 16-bit activations before it quantises them
#pragma unroll
          for (int e = 0; e < 8; ++e) y[e] = round_bf16(y[e]);
        }
      };
      auto segment_reduce = [&](float v, bool maximum) {
        for (int o = seg >> 1; o > 0; o >>= 1) {
          const float other = __shfl_xor_sync(0xffffffffu, v, o);
          v = maximum ? fmaxf(v, other) : v + other;
        }
        return v;
      };
      // items are laid out so that a warp's 32 lanes cover whole segments: padded to a multiple of 32
      const int padded_items = (items + 31) & ~31;
      if (normed) {
        for (int item = tid; item < padded_items; item += nthreads) {
          float sq = 0.0f;
          const int r = item / chunks, c = item - r * chunks;
          if (item < items) {
            float x[8];
            skinny::unpack8(*reinterpret_cast<const uint4*>(raw_tile + r * p.raw_stride + c * 16), x);
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += x[e] * x[e];
          }
          sq = segment_reduce(sq, false);
          if (item < items && (c & (seg - 1)) == 0) s_part[r * 16 + (c >> 5)] = sq;
        }
        ctx.sync();
        if (tid < p.M) {
          float total = 0.0f;
          for (int part = 0; part < parts; ++part) total += s_part[tid * 16 + part];
          s_stat[tid] = rsqrtf(total / static_cast<float>(p.K) + p.eps);
        }
        ctx.sync();
      }
      if (OP == kOpS8 && p.dynamic_rows) {
        for (int item = tid; item < padded_items; item += nthreads) {
          float amax = 0.0f;
          const int r = item / chunks, c = item - r * chunks;
          if (item < items) {
            float y[8];
            transformed(r, c, normed ? s_stat[r] : 1.0f, y);
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(y[e]));
          }
          amax = segment_reduce(amax, true);
          if (item < items && (c & (seg - 1)) == 0) s_part[r * 16 + (c >> 5)] = amax;
        }
        ctx.sync();
        if (tid < p.M) {
          float amax = 0.0f;
          for (int part = 0; part < parts; ++part) amax = fmaxf(amax, s_part[tid * 16 + part]);
          s_rowscale[tid] = fmaxf(amax / 127.0f, 1.0e-12f);
        }
        ctx.sync();
        for (int item = tid; item < items; item += nthreads) {
          const int r = item / chunks, c = item - r * chunks;
          float y[8];
          transformed(r, c, normed ? s_stat[r] : 1.0f, y);
          const float scale = s_rowscale[r];
          uint32_t lo = 0, hi = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            lo |= static_cast<uint32_t>(to_s8(y[e] / scale)) << (8 * e);
            hi |= static_cast<uint32_t>(to_s8(y[4 + e] / scale)) << (8 * e);
          }
          *reinterpret_cast<uint2*>(a_tile + r * p.a_stride + c * 8) = make_uint2(lo, hi);
        }
      } else {
        for (int item = tid; item < items; item += nthreads) {
          const int r = item / chunks, c = item - r * chunks;
          float y[8];
          transformed(r, c, normed ? s_stat[r] : 1.0f, y);
          skinny::store_staged<OP>(a_tile + r * p.a_stride, c, y, p.a_inv_scale);
        }
      }
    }
    ctx.sync();
  }

  // ---- main loop: fragments from registers (weights) and shared memory (activations) ----
  uint32_t acc[NTW][4];
#pragma unroll
  for (int j = 0; j < NTW; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0u;
  }
  const uint8_t* a_lo = a_tile + g * p.a_stride + t * 16;
  const uint8_t* a_hi = a_lo + 8 * p.a_stride;
  for (int base = kslice; base < p.steps; base += kSkinnyUnroll * ksplit) {
    if (base != kslice) load_weights(base);
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
      const int step = base + u * ksplit;
      if (step < p.steps) {
        const uint4 lo = *reinterpret_cast<const uint4*>(a_lo + step * 64);
        const uint4 hi = *reinterpret_cast<const uint4*>(a_hi + step * 64);
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
          skinny::mma<OP>(acc[j], lo.x, hi.x, lo.y, hi.y, wq[j][u].x, wq[j][u].y);
          skinny::mma<OP>(acc[j], lo.z, hi.z, lo.w, hi.w, wq[j][u].z, wq[j][u].w);
        }
      }
    }
  }

  // ---- K reduction over the warps of a group, in warp order ----
#pragma unroll
  for (int j = 0; j < NTW; ++j) {
    uint32_t* mine = red + (warp * NTW + j) * 128;
    *reinterpret_cast<uint2*>(mine + g * 8 + 2 * t) = make_uint2(acc[j][0], acc[j][1]);
    *reinterpret_cast<uint2*>(mine + (g + 8) * 8 + 2 * t) = make_uint2(acc[j][2], acc[j][3]);
  }
  ctx.sync();
  // ---- epilogue: one (row, column of each tile) per thread; 128 per group cover 16 x 8 ----
  for (int item = tid; item < p.groups * 128; item += nthreads) {
    const int eg = item >> 7, e = item & 127;
    const int row = e >> 3, col = e & 7;
    if (row >= p.M) continue;
    // this item's tiles (the thread's own warp may belong to another group)
    const int egroup = cta * p.groups + eg;
    if constexpr (NTW == 2) {
      const int per_block = p.tile_offset / 8;
      const int block = egroup / per_block;
      n0[0] = block * 2 * p.tile_offset + (egroup - block * per_block) * 8;
      n0[1] = n0[0] + p.tile_offset;
    } else {
      n0[0] = egroup * 8;
    }
    const uint32_t* gred = red + eg * ksplit * NTW * 128;
    float v[NTW];
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      if constexpr (OP == kOpS8) {
        int sum = 0;
        for (int w = 0; w < ksplit; ++w) sum += static_cast<int>(gred[(w * NTW + j) * 128 + e]);
        v[j] = static_cast<float>(sum);
        if (p.out_type == kOutS32 && n0[j] + col < p.N) {
          reinterpret_cast<int*>(p.out)[static_cast<long long>(row) * p.ldc + n0[j] + col] = sum;
        }
      } else {
        float sum = 0.0f;
        for (int w = 0; w < ksplit; ++w) sum += __uint_as_float(gred[(w * NTW + j) * 128 + e]);
        v[j] = sum;
      }
    }
    if (p.out_type == kOutS32) continue;

    const float row_factor = p.alpha * s_rowscale[row];
    const bool preloaded = item == static_cast<int>(tid);
    float bias[NTW], gate[NTW];
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int n = n0[j] + col;
      const bool in = n < p.N;
      if (preloaded) {
        v[j] *= row_factor * pre_scale[j];
        bias[j] = pre_bias[j];
        gate[j] = pre_gate[j];
      } else {
        v[j] *= row_factor * (p.col_scale != nullptr && in ? p.col_scale[n] : 1.0f);
        bias[j] = p.bias != nullptr && in ? __bfloat162float(p.bias[n]) : 0.0f;
        gate[j] = p.gate != nullptr && in ? __bfloat162float(p.gate[n]) : 0.0f;
      }
    }
    auto store = [&](void* base, long long index, float o) {
      if (p.out_type == kOutBf16) {
        reinterpret_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16(o);
      } else if (p.out_type == kOutF16) {
        reinterpret_cast<__half*>(base)[index] = __float2half_rn(o);
      } else if (p.out_type == kOutE4m3) {
        reinterpret_cast<uint8_t*>(base)[index] = to_e4m3(o * p.out_inv_scale);
      } else if (p.out_type == kOutS8) {
        reinterpret_cast<uint8_t*>(base)[index] = to_s8(round_bf16(o) * p.out_inv_scale);
      } else {
        reinterpret_cast<float*>(base)[index] = o;
      }
    };
    if (mode == kEpiGeglu) {
      if constexpr (NTW == 2) {
        const int n = n0[0] + col;  // packed gate row; its feature index is the output column
        if (n < p.N) {
          const int oc = (n / 128) * 64 + (n % 128);
          const float o = gelu_tanh_f(round_bf16(v[0])) * round_bf16(v[1]);
          store(p.out, static_cast<long long>(row) * p.ldc + oc, o);
        }
      }
      continue;
    }
    if (mode == kEpiRope) {
      if constexpr (NTW == 2) {
        // columns n and n + head_dim / 2 of one head: (a, b) -> (a cos - b sin, b cos + a sin)
        const int n = n0[0] + col;
        if (n >= p.N) continue;
        const int half = p.head_dim >> 1;
        const int head = n / p.head_dim;
        const int i = n - head * p.head_dim;  // < half by construction of the tile pairs
        const int sample = row / p.tokens;
        const int token = row - sample * p.tokens;
        const long long cache_row =
            static_cast<long long>(sample) * p.cache_rows + p.position_offset + token;
        const float a = round_bf16(v[0]) + bias[0], b = round_bf16(v[1]) + bias[1];
        if (head < p.q_heads + 1) {
          const int position = p.position_offset + token;
          const float c = preloaded ? pre_cos : p.cos_table[static_cast<long long>(position) * half + i];
          const float sn = preloaded ? pre_sin : p.sin_table[static_cast<long long>(position) * half + i];
          __nv_bfloat16* dst = head < p.q_heads
                                   ? reinterpret_cast<__nv_bfloat16*>(p.q_out) +
                                         (static_cast<long long>(row) * p.q_heads + head) * p.head_dim
                                   : reinterpret_cast<__nv_bfloat16*>(p.k_cache) + cache_row * p.head_dim;
          dst[i] = __float2bfloat16(a * c - b * sn);
          dst[i + half] = __float2bfloat16(b * c + a * sn);
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.v_cache) + cache_row * p.head_dim;
          dst[i] = __float2bfloat16(a);
          dst[i + half] = __float2bfloat16(b);
        }
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int n = n0[j] + col;
      if (n >= p.N) continue;
      const long long index = static_cast<long long>(row) * p.ldc + n;
      float o;
      if (out_is_raw(p.out_type)) {
        o = v[j];
      } else {
        const float extra =
            (mode == kEpiBiasResidual || mode == kEpiGateResidual || mode == kEpiEuler)
                ? (preloaded ? pre_extra[j] : __bfloat162float(__ldcg(p.residual + index)))
                : 0.0f;
        switch (mode) {
          case kEpiBiasGelu: o = gelu_tanh_f(round_bf16(v[j]) + bias[j]); break;
          case kEpiBiasSilu: o = silu_f(round_bf16(v[j]) + bias[j]); break;
          case kEpiBiasResidual: o = (round_bf16(v[j]) + extra) + bias[j]; break;
          case kEpiGateResidual: o = extra + round_bf16(v[j]) * gate[j]; break;
          case kEpiEuler: o = extra + p.dt * round_bf16(round_bf16(v[j]) + bias[j]); break;
          default: o = round_bf16(v[j]) + bias[j]; break;
        }
      }
      store(p.out, index, o);
    }
  }
}

template <int OP, int NTW, bool PRO>
__global__ void __launch_bounds__(32 * kSkinnyMaxWarps)
gemm_skinny_kernel(const SkinnyParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) uint8_t skinny_smem_base[];
  const SkinnyLaunchCtx ctx{static_cast<int>(blockIdx.x), static_cast<int>(threadIdx.x),
                            static_cast<int>(blockDim.x)};
  skinny_body<OP, NTW, PRO>(p, skinny_smem_base, ctx);
}

}  // namespace pi05
