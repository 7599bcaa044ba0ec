// Dense linear layers of the PI0.5 forward as tcgen05 (UMMA) GEMMs with TMEM
// accumulators fed by TMA, for sm_100a only.
//
//   D[i, j] = sum_k A[i, k] * B[j, k]        A: 128-row tile, B: BLOCK_N-row tile
//
// Both operands are K-major in global memory (row = one output index, K
// contiguous) and land in shared memory through 128-byte-swizzled TMA boxes;
// optionally B is "MN-major" (a [K, N] row-major matrix such as an attention
// value matrix). One CTA computes one 128 x BLOCK_N tile:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + single-thread tcgen05.mma issuer
//   warps 2..5  epilogue: tcgen05.ld the accumulator, apply the fused
//               epilogue, store with 16/32-byte accesses
// "Swap" launches put the weight matrix on the 128-row side and the (few)
// activation rows on the BLOCK_N side, so a 10- or 50-row action-expert GEMM
// still fills the 128-lane MMA; the epilogue then writes the transpose.
//
// Replaces, for the PI0.5 path, the reference's cuBLAS / cuBLASLt / CUTLASS
// GEMM dispatch (crates/apxinf-cuda/src/kernels/gemm/{bf16,fp8,w8a8}.rs) and
// the elementwise kernels that follow each GEMM there
// (crates/apxinf-cuda/kernels/custom/{activation,elementwise,fused}.cuh); the
// rounding points of those separate kernels are kept inside the epilogue.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "launch.cuh"
#include "ptx.cuh"

namespace pi05 {

enum OperandType : int { kOpBf16 = 0, kOpE4m3 = 1, kOpS8 = 2 };

// Fused epilogues. "rb" = round to bf16 and back (the reference stores every
// GEMM result as a 16-bit tensor before the next elementwise kernel reads it).
enum EpilogueMode : int {
  kEpiStore = 0,        // o = rb(v); if bias: o = rb(o + bias[c])
  kEpiBiasGelu = 1,     // o = gelu_tanh(rb(v) + bias[c])
  kEpiBiasSilu = 2,     // o = silu(rb(v) + bias[c])
  kEpiBiasResidual = 3, // o = rb(v) + residual[r, c] (+ bias[c])
  kEpiBiasPos = 4,      // o = rb(v) + pos[r % pos_rows, c] (+ bias[c])
  kEpiGateResidual = 5, // o = residual[r, c] + rb(v) * gate[c]
  kEpiGeglu = 6,        // weight rows interleaved 64 gate / 64 up: o = gelu_tanh(rb(g)) * rb(u)
};

enum OutType : int {
  kOutBf16 = 0,  // round-to-nearest-even bf16
  kOutE4m3 = 1,  // e4m3(clamp(o * out_inv_scale, +-448))
  kOutF32 = 2,   // raw scaled accumulator (no epilogue rounding), for tests / partial sums
  kOutS32 = 3,   // raw int32 accumulator (kOpS8 only), for bit-exact checks
  kOutS8 = 4,    // static per-tensor int8: clamp(round_half_away(bf16(o) * out_inv_scale), -128, 127)
  kOutF16 = 5,   // raw scaled accumulator rounded once to f16 (the reference's FP8 GEMM contract)
};

enum GemmStatus : int {
  kGemmOk = 0,
  kGemmTimeoutProducer = 101,
  kGemmTimeoutMma = 102,
  kGemmTimeoutEpilogue = 103,
};

struct GemmParams {
  int rows_a;   // valid rows of the 128-row-side operand
  int rows_b;   // valid rows of the BLOCK_N-side operand
  int num_kb;   // K blocks of 128 bytes
  int nb0;      // blockIdx.z = b0 + nb0 * b1
  // > 0: K slices as a batch. Entry b0 covers K blocks [b0 * k_slice_kb, (b0 + 1) * k_slice_kb)
  // of ONE pair of operands (num_kb = k_slice_kb; blocks past the end of K read as zero) and
  // writes its own output at b0 * out_sb0.
  int k_slice_kb;
  // logical output [M, N] (after un-swapping), element strides
  void* out;
  long long ldc, out_sb0, out_sb1;
  const __nv_bfloat16* residual;  // same geometry as out
  const __nv_bfloat16* bias;      // [N]
  const float* col_scale;         // [N] or null (per-output-channel weight scale)
  const float* row_scale;         // [M] or null (per-row activation scale)
  long long row_scale_sb0;        // batch-0 stride of row_scale
  const __nv_bfloat16* pos;       // [pos_rows, N]
  const __nv_bfloat16* gate;      // [N]
  float alpha;                    // scalar scale applied with row_scale
  float out_inv_scale;            // for kOutE4m3 / kOutS8
  int pos_rows;
  long long pos_ld;
  int mode;
  int out_type;
  int* status;                    // device status word, 0 = ok
  // Diagnostics of the timeout path (one-CTA-per-tile kernel): the poll budget of every
  // barrier wait, and a K block whose A load the first CTA announces (expect_tx) but never
  // issues, so that its stage never fills and the bounded waits run out. -1: none.
  uint32_t wait_polls;
  int drop_load_kb;
  // split-K: blockIdx.z = split + split_k * batch; each split owns kb_per_split K blocks,
  // dumps its raw accumulator tile to `partials`, and the last split to arrive on a tile
  // (per-tile arrival counter, left at zero again) sums them in split order and runs the epilogue.
  int split_k;
  int kb_per_split;
  uint32_t* partials;             // [tiles][split_k][128][BLOCK_N] raw 32-bit accumulators
  int* tile_counters;             // [tiles], zero between launches
  // operands that no kernel of the stream writes (weights): their TMA loads may be issued
  // before the programmatic-dependency wait
  int static_a, static_b;
  // operand stored K-block-major ([K/128B][rows][128 B]): every TMA box is one contiguous
  // 128-row x 128-byte run; its map is {128 B, rows, k-blocks}
  int blocked_a, blocked_b;
  // persistent kernel: row tiles per raster group (>= 1)
  int group_a;
};

__device__ __forceinline__ float round_bf16(float x) {
  return __bfloat162float(__float2bfloat16(x));
}

// gelu_tanh(x) = 0.5 x (1 + tanh(u)), u = 0.79788456 (x + 0.044715 x^3)
// (crates/apxinf-cuda/kernels/custom/math.cuh:8-12), with tanh(u) = 1 - 2 / (1 + e^{2u})
// on the fast exponential: a few 1e-7 of relative error, far below one bf16 ulp.
__device__ __forceinline__ float gelu_tanh_f(float value) {
  constexpr float kAlpha = 0.7978845608028654f;
  const float u = kAlpha * (value + 0.044715f * value * value * value);
  const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
  return 0.5f * value * (1.0f + t);
}

// The same with the hardware tanh (one MUFU operation instead of an exponential and a
// reciprocal; relative error about 2^-11). Used only where the result is quantised to e4m3
// (three mantissa bits) straight away: the activation epilogues are MUFU-bound otherwise.
__device__ __forceinline__ float gelu_tanh_fast(float value) {
  constexpr float kAlpha = 0.7978845608028654f;
  const float u = kAlpha * (value + 0.044715f * value * value * value);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * value * (1.0f + t);
}

__device__ __forceinline__ float silu_f(float value) { return value / (1.0f + expf(-value)); }

__device__ __forceinline__ uint8_t to_e4m3(float scaled) {
  const float clamped = fminf(448.0f, fmaxf(-448.0f, scaled));
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ uint8_t to_s8(float scaled) {
  const float q = fminf(127.0f, fmaxf(-128.0f, roundf(scaled)));
  return static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(q)));
}

template <int OP>
struct OpTraits;
template <>
struct OpTraits<kOpBf16> {
  static constexpr int kElemBytes = 2;
  static constexpr ptx::MmaKind kKind = ptx::MmaKind::kF16;
  static constexpr uint32_t kFormat = 1;   // bf16
  static constexpr uint32_t kCFormat = 1;  // f32
};
template <>
struct OpTraits<kOpE4m3> {
  static constexpr int kElemBytes = 1;
  static constexpr ptx::MmaKind kKind = ptx::MmaKind::kF8F6F4;
  static constexpr uint32_t kFormat = 0;   // e4m3
  static constexpr uint32_t kCFormat = 1;  // f32
};
template <>
struct OpTraits<kOpS8> {
  static constexpr int kElemBytes = 1;
  static constexpr ptx::MmaKind kKind = ptx::MmaKind::kI8;
  static constexpr uint32_t kFormat = 1;   // s8
  static constexpr uint32_t kCFormat = 2;  // s32
};

// TMA warp + MMA warp + EPI_WARPS epilogue warps. Single-wave launches use 8 epilogue warps
// and a deep ring with one CTA per SM; multi-wave launches use 4 epilogue warps and a
// shallow ring so that two CTAs share an SM and one tile's epilogue runs under the other's
// main loop.
__host__ __device__ constexpr int gemm_threads(int epi_warps) { return 64 + 32 * epi_warps; }
constexpr int kTileRowsA = 128;
constexpr int kStageABytes = kTileRowsA * 128;

__host__ __device__ constexpr int gemm_stage_bytes(int block_n) { return kStageABytes + block_n * 128; }
__host__ __device__ constexpr int gemm_smem_bytes(int block_n, int stages) {
  return stages * gemm_stage_bytes(block_n) + 1024 /*alignment slack*/ + 512 /*barriers*/ +
         2 * 3 * 256 * 4 /*epilogue vectors (double-buffered in the persistent kernel)*/;
}
// One accumulator per tile (measured: rotating MMAs over several accumulators does not shorten
// the ~140-cycle issue interval of 128-row MMAs).
__host__ __device__ constexpr uint32_t tmem_cols_for(int block_n) {
  const int cols = block_n;
  return cols <= 32 ? 32u : cols <= 64 ? 64u : cols <= 128 ? 128u : cols <= 256 ? 256u : 512u;
}

// ---------------------------------------------------------------------------
// Epilogue building blocks
// ---------------------------------------------------------------------------

template <int OP>
__device__ __forceinline__ float acc_to_float(uint32_t raw) {
  if constexpr (OP == kOpS8) {
    return static_cast<float>(static_cast<int>(raw));
  } else {
    return __uint_as_float(raw);
  }
}

// One output element before its final rounding (the store converts once).
// `v` = scaled accumulator, `bias` / `gate` = per-column values (0 when absent),
// `extra` = residual or position-embedding element.
template <int MODE>
__device__ __forceinline__ float epi_apply(float v, float bias, float extra, float gate) {
  if constexpr (MODE == kEpiStore) {
    return round_bf16(v) + bias;
  } else if constexpr (MODE == kEpiBiasGelu) {
    return gelu_tanh_f(round_bf16(v) + bias);
  } else if constexpr (MODE == kEpiBiasSilu) {
    return silu_f(round_bf16(v) + bias);
  } else if constexpr (MODE == kEpiBiasResidual || MODE == kEpiBiasPos) {
    return (round_bf16(v) + extra) + bias;
  } else if constexpr (MODE == kEpiGateResidual) {
    return extra + round_bf16(v) * gate;
  } else {
    return v;
  }
}

// One-byte outputs: e4m3 straight from the fp32 value (the FP8 path fuses the quantiser into
// the producer), int8 from the bf16-rounded value (the W8A8 path stores bf16 first).
__device__ __forceinline__ bool out_is_byte(const GemmParams& p) {
  return p.out_type == kOutE4m3 || p.out_type == kOutS8;
}
__device__ __forceinline__ uint8_t out_byte(const GemmParams& p, float o) {
  return p.out_type == kOutS8 ? to_s8(round_bf16(o) * p.out_inv_scale)
                              : to_e4m3(o * p.out_inv_scale);
}
__device__ __forceinline__ uint8_t out_byte_as(int out_type, const GemmParams& p, float o) {
  return out_type == kOutS8 ? to_s8(round_bf16(o) * p.out_inv_scale) : to_e4m3(o * p.out_inv_scale);
}

// outputs that skip the fused epilogue: the scaled accumulator itself
__device__ __forceinline__ bool out_is_raw(int out_type) { return out_type == kOutF32 || out_type == kOutF16; }

__device__ __forceinline__ void store_one(const GemmParams& p, long long index, float o) {
  if (p.out_type == kOutF16) {
    reinterpret_cast<__half*>(p.out)[index] = __float2half_rn(o);
  } else if (p.out_type == kOutBf16) {
    reinterpret_cast<__nv_bfloat16*>(p.out)[index] = __float2bfloat16(o);
  } else if (out_is_byte(p)) {
    reinterpret_cast<uint8_t*>(p.out)[index] = out_byte(p, o);
  } else {
    reinterpret_cast<float*>(p.out)[index] = o;
  }
}

// Store 16 consecutive columns of one row; vectorised when the destination is
// 16-byte aligned and the whole chunk is in range.
template <int OUT = -1>
__device__ __forceinline__ void store_chunk16(const GemmParams& p, long long index, int valid,
                                              const float (&o)[16]) {
  const int out_type = OUT >= 0 ? OUT : p.out_type;  // OUT >= 0: the one type this kernel writes
  if (out_type == kOutBf16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + index;
    if (valid == 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      uint32_t w[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        __nv_bfloat162 pair = __floats2bfloat162_rn(o[2 * t], o[2 * t + 1]);
        w[t] = *reinterpret_cast<uint32_t*>(&pair);
      }
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        if (t < valid) dst[t] = __float2bfloat16(o[t]);
      }
    }
  } else if ((out_type == kOutE4m3 || out_type == kOutS8)) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + index;
    if (valid == 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      uint32_t w[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        w[t] = (uint32_t)out_byte_as(out_type, p, o[4 * t]) |
               ((uint32_t)out_byte_as(out_type, p, o[4 * t + 1]) << 8) |
               ((uint32_t)out_byte_as(out_type, p, o[4 * t + 2]) << 16) |
               ((uint32_t)out_byte_as(out_type, p, o[4 * t + 3]) << 24);
      }
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        if (t < valid) dst[t] = out_byte_as(out_type, p, o[t]);
      }
    }
  } else {
    float* dst = reinterpret_cast<float*>(p.out) + index;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if (t < valid) dst[t] = o[t];
    }
  }
}

// 16 consecutive bf16 of one row as floats (vector loads when aligned).
// Eight consecutive outputs of one row (valid may be <= 0 or > 8).
template <int OUT = -1>
__device__ __forceinline__ void store_chunk8(const GemmParams& p, long long index, int valid,
                                             const float (&o)[8]) {
  if (valid <= 0) return;
  const int out_type = OUT >= 0 ? OUT : p.out_type;  // OUT >= 0: the one type this kernel writes
  if (out_type == kOutBf16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + index;
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      uint32_t w[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        __nv_bfloat162 pair = __floats2bfloat162_rn(o[2 * t], o[2 * t + 1]);
        w[t] = *reinterpret_cast<uint32_t*>(&pair);
      }
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < valid) dst[t] = __float2bfloat16(o[t]);
      }
    }
  } else if ((out_type == kOutE4m3 || out_type == kOutS8)) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + index;
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
      uint32_t w[2];
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        w[t] = (uint32_t)out_byte_as(out_type, p, o[4 * t]) |
               ((uint32_t)out_byte_as(out_type, p, o[4 * t + 1]) << 8) |
               ((uint32_t)out_byte_as(out_type, p, o[4 * t + 2]) << 16) |
               ((uint32_t)out_byte_as(out_type, p, o[4 * t + 3]) << 24);
      }
      *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < valid) dst[t] = out_byte_as(out_type, p, o[t]);
      }
    }
  } else if (out_type == kOutF16) {
    __half* dst = reinterpret_cast<__half*>(p.out) + index;
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      uint32_t w[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const __half2 pair = __floats2half2_rn(o[2 * t], o[2 * t + 1]);
        w[t] = *reinterpret_cast<const uint32_t*>(&pair);
      }
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < valid) dst[t] = __float2half_rn(o[t]);
      }
    }
  } else if (out_type == kOutF32) {
    float* dst = reinterpret_cast<float*>(p.out) + index;
    if (valid >= 8 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        if (t < valid) dst[t] = o[t];
      }
    }
  }
}

__device__ __forceinline__ void load_row16(const __nv_bfloat16* src, int valid, float (&x)[16]) {
  if (valid == 16 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
    const uint4 lo = reinterpret_cast<const uint4*>(src)[0];
    const uint4 hi = reinterpret_cast<const uint4*>(src)[1];
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&lo);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&hi);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 fa = __bfloat1622float2(a[t]);
      const float2 fb = __bfloat1622float2(b[t]);
      x[2 * t] = fa.x;
      x[2 * t + 1] = fa.y;
      x[8 + 2 * t] = fb.x;
      x[8 + 2 * t + 1] = fb.y;
    }
  } else {
#pragma unroll
    for (int t = 0; t < 16; ++t) x[t] = t < valid ? __bfloat162float(src[t]) : 0.0f;
  }
}

// 16 consecutive floats from shared memory with four 16-byte loads.
__device__ __forceinline__ void lds16(const float* src, float (&x)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 v = reinterpret_cast<const float4*>(src)[q];
    x[4 * q] = v.x;
    x[4 * q + 1] = v.y;
    x[4 * q + 2] = v.z;
    x[4 * q + 3] = v.w;
  }
}

// Where the epilogue reads the accumulator from: this CTA's TMEM (one split) or
// the sum over all splits' partial tiles in global memory, added in split order
// so the result does not depend on which split arrived last.
// PARTIAL = false: a kernel that never splits K; only the TMEM path is compiled.
template <int OP, int BLOCK_N, bool PARTIAL = true>
struct AccSource {
  uint32_t taddr_row;
  const uint32_t* partial_row;  // this thread's row in split 0, or null
  long long split_stride;       // elements between splits
  int splits;

  __device__ __forceinline__ void load16(int col0, uint32_t (&raw)[16]) const {
    if (!PARTIAL || partial_row == nullptr) {
      ptx::tmem_ld_16(taddr_row + col0, raw);
      return;
    }
    float facc[16];
    int iacc[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      facc[t] = 0.0f;
      iacc[t] = 0;
    }
    // four splits' loads are issued together (one L2 round trip per group), then added in order
    for (int s0 = 0; s0 < splits; s0 += 4) {
      uint4 v[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < splits) {
          const uint4* src =
              reinterpret_cast<const uint4*>(partial_row + (s0 + u) * split_stride + col0);
#pragma unroll
          for (int q = 0; q < 4; ++q) v[u][q] = __ldcg(src + q);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < splits) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t w[4] = {v[u][q].x, v[u][q].y, v[u][q].z, v[u][q].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if constexpr (OP == kOpS8) {
                iacc[q * 4 + e] += static_cast<int>(w[e]);
              } else {
                facc[q * 4 + e] += __uint_as_float(w[e]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if constexpr (OP == kOpS8) {
        raw[t] = static_cast<uint32_t>(iacc[t]);
      } else {
        raw[t] = __float_as_uint(facc[t]);
      }
    }
  }
  __device__ __forceinline__ void wait() const {
    if (!PARTIAL || partial_row == nullptr) ptx::tmem_ld_wait();
  }
};

// 16 bf16 of one row as two 16-byte words (zero beyond `valid`), kept packed until use.
__device__ __forceinline__ void load_row16_packed(const __nv_bfloat16* src, int valid,
                                                  uint4 (&x)[2]) {
  if (valid == 16 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
    x[0] = reinterpret_cast<const uint4*>(src)[0];
    x[1] = reinterpret_cast<const uint4*>(src)[1];
  } else {
    uint32_t w[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const uint32_t lo = 2 * t < valid ? __bfloat16_as_ushort(src[2 * t]) : 0u;
      const uint32_t hi = 2 * t + 1 < valid ? __bfloat16_as_ushort(src[2 * t + 1]) : 0u;
      w[t] = lo | (hi << 16);
    }
    x[0] = make_uint4(w[0], w[1], w[2], w[3]);
    x[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// Thread = one output row, TMEM columns = output columns. The HALVES warps that share a
// TMEM lane quarter take the 16-column chunks half, half + HALVES, ... (interleaved: giving a
// warp adjacent chunks measured 25 % slower). Two chunks go through each TMEM round trip,
// a bf16 chunk leaves as one 32-byte store, and the residual (or position) values of the next round are
// requested before the current one is processed, the first round's even before the
// accumulator is complete (`wait_acc`), so their latency hides behind the mainloop.
// OUT >= 0 fixes the output type at compile time (the launch's p.out_type must equal it).
template <int OP, int BLOCK_N, int MODE, int HALVES, int OUT = -1, int PER_ROUND = 2, bool PARTIAL,
          typename WaitAcc>
__device__ __forceinline__ void epilogue_normal(const GemmParams& p,
                                                const AccSource<OP, BLOCK_N, PARTIAL>& acc, int r,
                                                int tile_b, long long out_base, float sr, int half,
                                                const float* s_scale, const float* s_bias,
                                                const float* s_gate, WaitAcc&& wait_acc) {
  constexpr bool kExtra =
      MODE == kEpiBiasResidual || MODE == kEpiBiasPos || MODE == kEpiGateResidual;
  constexpr int kChunks = BLOCK_N / 16;
  constexpr int kPerWarp = (kChunks + HALVES - 1) / HALVES;
  // chunks per TMEM round trip
  constexpr int kPerRound = PER_ROUND;
  constexpr int kRounds = (kPerWarp + kPerRound - 1) / kPerRound;
  const int out_type = OUT >= 0 ? OUT : p.out_type;
  const bool row_ok = r < p.rows_a;
  const bool has_scale = p.col_scale != nullptr;
  const __nv_bfloat16* extra_row = nullptr;
  if (kExtra && row_ok) {
    extra_row = MODE == kEpiBiasPos ? p.pos + (long long)(r % p.pos_rows) * p.pos_ld
                                    : p.residual + out_base + (long long)r * p.ldc;
  }
  uint4 ahead[kPerRound][2];  // residual / position values (16 bf16 per chunk) of the round to come
  auto fetch_extra = [&](int round, int u, uint4 (&dst)[2]) {
    const int cc = half + (kPerRound * round + u) * HALVES;
    const int c0 = tile_b * BLOCK_N + cc * 16;
    if (kExtra && row_ok && cc < kChunks && c0 < p.rows_b) {
      load_row16_packed(extra_row + c0, min(16, p.rows_b - c0), dst);
    } else {
      dst[0] = make_uint4(0, 0, 0, 0);
      dst[1] = make_uint4(0, 0, 0, 0);
    }
  };
#pragma unroll
  for (int u = 0; u < kPerRound; ++u) fetch_extra(0, u, ahead[u]);
  wait_acc();
#pragma unroll 1
  for (int round = 0; round < kRounds; ++round) {
    uint32_t raw[kPerRound][16];
#pragma unroll
    for (int u = 0; u < kPerRound; ++u) {
      // always issued (a conditional TMEM load would push the array to local memory); a slot
      // beyond the tile re-reads the last chunk and is ignored below
      acc.load16(min(half + (kPerRound * round + u) * HALVES, kChunks - 1) * 16, raw[u]);
    }
    acc.wait();
#pragma unroll
    for (int u = 0; u < kPerRound; ++u) {
      const int cc = half + (kPerRound * round + u) * HALVES;
      const int c0 = tile_b * BLOCK_N + cc * 16;
      const int valid = row_ok && cc < kChunks ? min(16, p.rows_b - c0) : 0;
      const long long index = out_base + (long long)r * p.ldc + c0;
      if (valid > 0 && out_type == kOutS32) {
        int* dst = reinterpret_cast<int*>(p.out) + index;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          if (t < valid) dst[t] = static_cast<int>(raw[u][t]);
        }
      } else if (valid > 0) {
        uint32_t packed[8];  // bf16 pairs of the 16 columns, for one 32-byte store
        const bool wide = out_type == kOutBf16 && valid == 16 &&
                          ((reinterpret_cast<uintptr_t>(p.out) + 2 * index) & 31u) == 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // eight columns at a time keeps the temporaries in registers
          const int j = cc * 16 + 8 * h;
          float o[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) o[t] = acc_to_float<OP>(raw[u][8 * h + t]) * sr;
          if (has_scale) {
            const float4 s0 = reinterpret_cast<const float4*>(s_scale + j)[0];
            const float4 s1 = reinterpret_cast<const float4*>(s_scale + j)[1];
            o[0] *= s0.x; o[1] *= s0.y; o[2] *= s0.z; o[3] *= s0.w;
            o[4] *= s1.x; o[5] *= s1.y; o[6] *= s1.z; o[7] *= s1.w;
          }
          if (!out_is_raw(out_type)) {
            const float4 b0 = reinterpret_cast<const float4*>(s_bias + j)[0];
            const float4 b1 = reinterpret_cast<const float4*>(s_bias + j)[1];
            const float bias[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            float gate[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if constexpr (MODE == kEpiGateResidual) {
              const float4 g0 = reinterpret_cast<const float4*>(s_gate + j)[0];
              const float4 g1 = reinterpret_cast<const float4*>(s_gate + j)[1];
              gate[0] = g0.x; gate[1] = g0.y; gate[2] = g0.z; gate[3] = g0.w;
              gate[4] = g1.x; gate[5] = g1.y; gate[6] = g1.z; gate[7] = g1.w;
            }
            const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&ahead[u][h]);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const float2 x = __bfloat1622float2(e[t]);
              if (MODE == kEpiBiasGelu && out_type == kOutE4m3) {
                o[2 * t] = gelu_tanh_fast(round_bf16(o[2 * t]) + bias[2 * t]);
                o[2 * t + 1] = gelu_tanh_fast(round_bf16(o[2 * t + 1]) + bias[2 * t + 1]);
              } else {
                o[2 * t] = epi_apply<MODE>(o[2 * t], bias[2 * t], x.x, gate[2 * t]);
                o[2 * t + 1] = epi_apply<MODE>(o[2 * t + 1], bias[2 * t + 1], x.y, gate[2 * t + 1]);
              }
            }
          }
          if (wide) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const __nv_bfloat162 pair = __floats2bfloat162_rn(o[2 * t], o[2 * t + 1]);
              packed[4 * h + t] = *reinterpret_cast<const uint32_t*>(&pair);
            }
          } else {
            store_chunk8<OUT>(p, index + 8 * h, valid - 8 * h, o);
          }
        }
        if (wide) {
          // one 256-bit store per row and chunk: a full 32-byte sector per lane, half the
          // store instructions of two 16-byte ones
          asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(
                           reinterpret_cast<__nv_bfloat16*>(p.out) + index),
                       "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]),
                       "r"(packed[4]), "r"(packed[5]), "r"(packed[6]), "r"(packed[7])
                       : "memory");
        }
      }
      // request the values this slot needs in the next round while the other slot is processed
      if (round + 1 < kRounds) fetch_extra(round + 1, u, ahead[u]);
    }
  }
}

// GeGLU epilogue, thread = one output row: packed columns [128t, 128t+64) are gate features,
// [128t+64, 128t+128) the matching up features.
template <int OP, int BLOCK_N, int HALVES, int OUT = -1, bool PARTIAL>
__device__ __forceinline__ void epilogue_geglu_normal(const GemmParams& p,
                                                      const AccSource<OP, BLOCK_N, PARTIAL>& acc, int r,
                                                      int tile_b, long long out_base, float sr,
                                                      int half, const float* s_scale) {
  const bool fast = (OUT >= 0 ? OUT : p.out_type) == kOutE4m3;
#pragma unroll 1
  for (int it = half; it < BLOCK_N / 32; it += HALVES) {
    const int pair = it >> 2, sub = it & 3;
    uint32_t rg[16], ru[16];
    acc.load16(pair * 128 + sub * 16, rg);
    acc.load16(pair * 128 + 64 + sub * 16, ru);
    const int jg = pair * 128 + sub * 16;
    float sg[16], su[16];
    lds16(s_scale + jg, sg);
    lds16(s_scale + jg + 64, su);
    acc.wait();
    const int cg = tile_b * BLOCK_N + jg;         // packed gate column
    const int oc = (cg / 128) * 64 + (cg % 128);  // output column
    float o[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float g = round_bf16(acc_to_float<OP>(rg[t]) * sr * sg[t]);
      const float u = round_bf16(acc_to_float<OP>(ru[t]) * sr * su[t]);
      o[t] = (fast ? gelu_tanh_fast(g) : gelu_tanh_f(g)) * u;
    }
    if (r < p.rows_a && cg < p.rows_b) {
      store_chunk16<OUT>(p, out_base + (long long)r * p.ldc + oc, 16, o);
    }
  }
}

// Thread = one output column (weight row), TMEM columns = output rows.
template <int OP, int BLOCK_N, int MODE, int HALVES, bool PARTIAL>
__device__ __forceinline__ void epilogue_swapped(const GemmParams& p,
                                                 const AccSource<OP, BLOCK_N, PARTIAL>& acc, int c,
                                                 int tile_b, long long out_base, int half,
                                                 float sc, float bias, float gate,
                                                 const float* s_rowscale) {
  constexpr bool kExtra =
      MODE == kEpiBiasResidual || MODE == kEpiBiasPos || MODE == kEpiGateResidual;
  const bool col_ok = c < p.rows_a;
#pragma unroll 1
  for (int cc = half; cc < BLOCK_N / 16; cc += HALVES) {
    uint32_t raw[16];
    acc.load16(cc * 16, raw);
    const int r0 = tile_b * BLOCK_N + cc * 16;
    const int valid = col_ok ? min(16, p.rows_b - r0) : 0;
    float extra[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      extra[t] = 0.0f;
      if (kExtra && t < valid) {
        const int r = r0 + t;
        extra[t] = MODE == kEpiBiasPos
                       ? __bfloat162float(p.pos[(long long)(r % p.pos_rows) * p.pos_ld + c])
                       : __bfloat162float(p.residual[out_base + (long long)r * p.ldc + c]);
      }
    }
    float rs[16];
    lds16(s_rowscale + cc * 16, rs);
    acc.wait();
    if (valid <= 0) continue;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      if (t < valid) {
        const long long index = out_base + (long long)(r0 + t) * p.ldc + c;
        if (p.out_type == kOutS32) {
          reinterpret_cast<int*>(p.out)[index] = static_cast<int>(raw[t]);
        } else {
          const float v = acc_to_float<OP>(raw[t]) * rs[t] * sc;
          const float o = out_is_raw(p.out_type) ? v : epi_apply<MODE>(v, bias, extra[t], gate);
          store_one(p, index, o);
        }
      }
    }
  }
}

// FIXED_MODE >= 0 compiles the kernel for that one epilogue (the launch's p.mode must equal it):
// the forward's most frequent epilogues get kernels that hold no other epilogue's code.
template <int OP, int BLOCK_N, int STAGES, bool SWAP, bool B_MN, int EPI_WARPS, int FIXED_MODE = -1>
__global__ void __launch_bounds__(gemm_threads(EPI_WARPS), EPI_WARPS == 4 ? 2 : 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using T = OpTraits<OP>;
  static_assert(BLOCK_N % 16 == 0 && BLOCK_N >= 16 && BLOCK_N <= 256, "bad BLOCK_N");
  static_assert(!B_MN || ((OP == kOpBf16 || OP == kOpE4m3) && BLOCK_N % 128 == 0 && !SWAP),
                "MN-major B: bf16 or e4m3, activations on the 128-row side");
  static_assert(EPI_WARPS == 4 || EPI_WARPS == 8, "4 or 8 epilogue warps");
  constexpr int kHalves = EPI_WARPS / 4;
  constexpr int kEpilogueThreads = 32 * EPI_WARPS;
  constexpr int kBlockK = 128 / T::kElemBytes;  // elements per 128-byte K block
  constexpr int kStageBBytes = BLOCK_N * 128;
  constexpr int kStageBytes = kStageABytes + kStageBBytes;
  constexpr uint32_t kTmemCols = tmem_cols_for(BLOCK_N);
  constexpr uint32_t kIdesc =
      ptx::make_idesc(T::kCFormat, T::kFormat, T::kFormat, 0, B_MN ? 1 : 0, 128, BLOCK_N);

  // A kernel compiled for one epilogue also fixes what that epilogue writes in the forward (FP8 /
  // int8 activations after bias + GELU of an FP8 / int8 GEMM, bf16 otherwise) and never splits K.
  constexpr bool kLean = FIXED_MODE >= 0;
  // Chunks per TMEM round trip in the epilogue: the narrow single-epilogue kernels run as one
  // partial wave of CTAs that execute their epilogue once, where a loop body of one chunk (half
  // the code) beat two chunks per round trip (FP8 B=1 forward 8.88 -> 8.82 ms); the 256-wide
  // tiles of the batched step keep two (one was 0.2-2 % slower there).
  constexpr int kPerRound = kLean && BLOCK_N <= 128 ? 1 : 2;
  static_assert(!kLean || !SWAP, "single-epilogue kernels: activations on the 128-row side");
  constexpr int kFixedOut =
      !kLean ? -1 : FIXED_MODE != kEpiBiasGelu ? kOutBf16 : OP == kOpE4m3 ? kOutE4m3 : OP == kOpS8 ? kOutS8 : kOutBf16;
  const int mode = kLean ? FIXED_MODE : p.mode;

  pdl_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  float* s_scale = reinterpret_cast<float*>(smem + STAGES * kStageBytes + 512);
  float* s_bias = s_scale + 256;
  float* s_gate = s_bias + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x;
  const int tile_b = blockIdx.y;
  const int split = blockIdx.z % p.split_k;
  const int batch = blockIdx.z / p.split_k;
  const int b0 = batch % p.nb0;
  const int b1 = batch / p.nb0;
  const int kb_begin = split * p.kb_per_split;
  const int kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
  const int my_kb = kb_end - kb_begin;  // >= 1 by construction

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(accum_bar, 1);
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      bool ok = true;
      int issued = 0;
      const bool first_cta = (blockIdx.x | blockIdx.y | blockIdx.z) == 0;
      // K slices as a batch: the batch index moves the K range, not the operand
      const int kb_slice = p.k_slice_kb > 0 ? b0 * p.k_slice_kb : 0;
      const int c_b0 = p.k_slice_kb > 0 ? 0 : b0;
      auto load_a = [&](int it) {
        if (first_cta && it == p.drop_load_kb) return;
        const int s = it % STAGES;
        if (p.blocked_a) {
          ptx::tma_load_4d(smem + s * kStageBytes, &tmap_a, &full_bar[s], 0, tile_a * kTileRowsA,
                           kb_begin + it, 0);
        } else {
          ptx::tma_load_4d(smem + s * kStageBytes, &tmap_a, &full_bar[s],
                           (kb_slice + kb_begin + it) * kBlockK, tile_a * kTileRowsA, c_b0, b1);
        }
      };
      auto load_b = [&](int it) {
        const int s = it % STAGES;
        uint8_t* sb = smem + s * kStageBytes + kStageABytes;
        const int kb = kb_slice + kb_begin + it;
        if constexpr (B_MN) {
          // MN-major B: 128-byte runs along N (kBlockK elements wide), kBlockK K-rows per chunk
#pragma unroll
          for (int chunk = 0; chunk < BLOCK_N / kBlockK; ++chunk) {
            ptx::tma_load_4d(sb + chunk * (kBlockK * 128), &tmap_b, &full_bar[s],
                             tile_b * BLOCK_N + chunk * kBlockK, kb * kBlockK, b0, b1);
          }
        } else if (p.blocked_b) {
          ptx::tma_load_4d(sb, &tmap_b, &full_bar[s], 0, tile_b * BLOCK_N, kb, 0);
        } else {
          ptx::tma_load_4d(sb, &tmap_b, &full_bar[s], kb * kBlockK, tile_b * BLOCK_N, c_b0, b1);
        }
      };
      // First ring fill: static operands (weights) stream in while the producer of the
      // activations may still be running; the dependent operand follows the wait.
      const int first_fill = min(my_kb, STAGES);
      for (int it = 0; it < first_fill; ++it) {
        ptx::mbar_arrive_expect_tx(&full_bar[it], kStageBytes);
        if (p.static_a) load_a(it);
        if (p.static_b) load_b(it);
      }
      pdl_wait();
      for (int it = 0; it < first_fill; ++it) {
        if (!p.static_a) load_a(it);
        if (!p.static_b) load_b(it);
      }
      issued = first_fill;
      for (int it = first_fill; it < my_kb && ok; ++it) {
        const int s = it % STAGES;
        const uint32_t round = it / STAGES;
        ok = ptx::mbar_wait(&empty_bar[s], (round - 1) & 1, p.wait_polls);
        if (!ok) break;
        ptx::mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
        load_a(it);
        load_b(it);
        ++issued;
      }
      if (!ok) {
        atomicCAS(p.status, 0, kGemmTimeoutProducer);
        // let copies already in flight land before the CTA retires
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int it = first; it < issued; ++it) {
          ptx::mbar_wait(&full_bar[it % STAGES], (it / STAGES) & 1, p.wait_polls);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    pdl_wait();
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < my_kb; ++kb) {
        const int s = kb % STAGES;
        ok = ptx::mbar_wait(&full_bar[s], (kb / STAGES) & 1, p.wait_polls);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t a_addr = ptx::smem_u32(smem + s * kStageBytes);
        const uint32_t b_addr = a_addr + kStageABytes;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t adesc = ptx::make_smem_desc(a_addr + k * 32, 16, 1024);
          const uint64_t bdesc = B_MN ? ptx::make_smem_desc(b_addr + k * (kBlockK / 4) * 128, kBlockK * 128, 1024)
                                      : ptx::make_smem_desc(b_addr + k * 32, 16, 1024);
          ptx::umma<T::kKind>(tmem_base, adesc, bdesc, kIdesc, (kb | k) != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&empty_bar[s]);
      }
      if (!ok) atomicCAS(p.status, 0, kGemmTimeoutMma);
      // Always signal the epilogue so that it never waits on a dead pipeline.
      ptx::umma_commit(accum_bar);
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    const int quarter = warp & 3;           // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;       // which of the quarter's two warps
    const int row_in_tile = quarter * 32 + lane;
    const int ep_tid = threadIdx.x - 64;
    const int gi = tile_a * kTileRowsA + row_in_tile;  // index on the 128-row side
    const long long out_base = (long long)b0 * p.out_sb0 + (long long)b1 * p.out_sb1;
    const float* row_scale =
        p.row_scale != nullptr ? p.row_scale + (long long)b0 * p.row_scale_sb0 : nullptr;

    // Per-column vectors of this tile (scale, bias, gate) go to shared memory while the main
    // loop runs. When the caller declared its weights static (the engine: these vectors are
    // written once, before the replayed stream) they are read ahead of the dependency wait;
    // otherwise an earlier kernel of the stream may have produced them, so the wait comes first.
    if (!(p.static_a | p.static_b)) pdl_wait();
    float sw_scale = 1.0f, sw_bias = 0.0f, sw_gate = 0.0f;
    if constexpr (!SWAP) {
      for (int j = ep_tid; j < BLOCK_N; j += kEpilogueThreads) {
        const int idx = tile_b * BLOCK_N + j;
        const bool in = idx < p.rows_b;
        s_scale[j] = p.col_scale != nullptr && in ? p.col_scale[idx] : 1.0f;
        s_bias[j] = p.bias != nullptr && in ? __bfloat162float(p.bias[idx]) : 0.0f;
        s_gate[j] = p.gate != nullptr && in ? __bfloat162float(p.gate[idx]) : 0.0f;
      }
    } else {
      const bool in = gi < p.rows_a;
      sw_scale = p.col_scale != nullptr && in ? p.col_scale[gi] : 1.0f;
      sw_bias = p.bias != nullptr && in ? __bfloat162float(p.bias[gi]) : 0.0f;
      sw_gate = p.gate != nullptr && in ? __bfloat162float(p.gate[gi]) : 0.0f;
    }
    pdl_wait();  // everything below may read what earlier kernels of the stream wrote
    if constexpr (SWAP) {
      for (int j = ep_tid; j < BLOCK_N; j += kEpilogueThreads) {
        const int idx = tile_b * BLOCK_N + j;
        const bool in = idx < p.rows_b;
        s_scale[j] = p.alpha * (row_scale != nullptr && in ? row_scale[idx] : 1.0f);
      }
    }
    float sr = p.alpha;
    if constexpr (!SWAP) {
      if (row_scale != nullptr && gi < p.rows_a) sr = p.alpha * row_scale[gi];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");

    const bool ok = ptx::mbar_wait(accum_bar, 0, p.wait_polls);
    if (!ok && lane == 0) atomicCAS(p.status, 0, kGemmTimeoutEpilogue);
    ptx::tc_fence_after();
    const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

    AccSource<OP, BLOCK_N, !kLean> acc{taddr_row, nullptr, 0, 1};
    bool run_epilogue = true;
    if (!kLean && p.split_k > 1) {
      const long long tile_id = ((long long)batch * gridDim.y + tile_b) * gridDim.x + tile_a;
      uint32_t* tile_ws = p.partials + tile_id * p.split_k * (128LL * BLOCK_N);
      uint32_t* mine = tile_ws + (long long)split * (128LL * BLOCK_N) + row_in_tile * BLOCK_N;
#pragma unroll 1
      for (int cc = half; cc < BLOCK_N / 16; cc += kHalves) {
        uint32_t raw[16];
        acc.load16(cc * 16, raw);
        acc.wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          __stcg(reinterpret_cast<uint4*>(mine + cc * 16) + q,
                 make_uint4(raw[4 * q], raw[4 * q + 1], raw[4 * q + 2], raw[4 * q + 3]));
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
      int* flag = reinterpret_cast<int*>(tmem_slot + 1);
      if (ep_tid == 0) *flag = atomicAdd(&p.tile_counters[tile_id], 1);
      asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
      run_epilogue = *flag == p.split_k - 1;
      if (run_epilogue) {
        __threadfence();
        if (ep_tid == 0) p.tile_counters[tile_id] = 0;
        acc.partial_row = tile_ws + row_in_tile * BLOCK_N;
        acc.split_stride = 128LL * BLOCK_N;
        acc.splits = p.split_k;
      }
    }

    if (!run_epilogue) {
      // another split finishes this tile
    } else if (mode == kEpiGeglu) {
      if constexpr (!SWAP) {
        epilogue_geglu_normal<OP, BLOCK_N, kHalves>(p, acc, gi, tile_b, out_base, sr, half, s_scale);
      } else {
        // lanes [0,64) hold gate features, lanes [64,128) the matching up features; the up
        // half goes through shared memory (stage 0 is idle once the accumulator is ready).
        float* xchg = reinterpret_cast<float*>(smem);  // [BLOCK_N][64]
        constexpr int kMine = (BLOCK_N / 16 + kHalves - 1) / kHalves;  // 16-column chunks per warp
        float vals[kMine * 16];
#pragma unroll
        for (int i = 0; i < kMine; ++i) {
          const int cc = half + kHalves * i;
          if (cc * 16 < BLOCK_N) {
            uint32_t raw[16];
            acc.load16(cc * 16, raw);
            float rs[16];
            lds16(s_scale + cc * 16, rs);
            acc.wait();
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              vals[i * 16 + t] = round_bf16(acc_to_float<OP>(raw[t]) * rs[t] * sw_scale);
            }
          }
        }
        if (row_in_tile >= 64) {
#pragma unroll
          for (int i = 0; i < kMine; ++i) {
            const int cc = half + kHalves * i;
            if (cc * 16 < BLOCK_N) {
#pragma unroll
              for (int t = 0; t < 16; ++t) {
                xchg[(cc * 16 + t) * 64 + (row_in_tile - 64)] = vals[i * 16 + t];
              }
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
        if (row_in_tile < 64 && gi < p.rows_a) {
          const int oc = tile_a * 64 + row_in_tile;
#pragma unroll
          for (int i = 0; i < kMine; ++i) {
            const int cc = half + kHalves * i;
            if (cc * 16 < BLOCK_N) {
#pragma unroll
              for (int t = 0; t < 16; ++t) {
                const int j = cc * 16 + t;
                const int r = tile_b * BLOCK_N + j;
                if (r < p.rows_b) {
                  const float o = gelu_tanh_f(vals[i * 16 + t]) * xchg[j * 64 + row_in_tile];
                  store_one(p, out_base + (long long)r * p.ldc + oc, o);
                }
              }
            }
          }
        }
      }
    } else if constexpr (!SWAP) {
#define PI05_EPI_CASE(MODE)                                                                       \
  case MODE:                                                                                      \
    epilogue_normal<OP, BLOCK_N, MODE, kHalves, kFixedOut, kPerRound>(                            \
        p, acc, gi, tile_b, out_base, sr, half, s_scale, s_bias, s_gate, [] {});                  \
    break;
      switch (mode) {
        PI05_EPI_CASE(kEpiStore)
        PI05_EPI_CASE(kEpiBiasGelu)
        PI05_EPI_CASE(kEpiBiasSilu)
        PI05_EPI_CASE(kEpiBiasResidual)
        PI05_EPI_CASE(kEpiBiasPos)
        PI05_EPI_CASE(kEpiGateResidual)
        default:
          break;
      }
#undef PI05_EPI_CASE
    } else {
#define PI05_EPI_CASE(MODE)                                                                      \
  case MODE:                                                                                     \
    epilogue_swapped<OP, BLOCK_N, MODE, kHalves>(p, acc, gi, tile_b, out_base, half, sw_scale,   \
                                                 sw_bias, sw_gate, s_scale);                      \
    break;
      switch (mode) {
        PI05_EPI_CASE(kEpiStore)
        PI05_EPI_CASE(kEpiBiasGelu)
        PI05_EPI_CASE(kEpiBiasSilu)
        PI05_EPI_CASE(kEpiBiasResidual)
        PI05_EPI_CASE(kEpiBiasPos)
        PI05_EPI_CASE(kEpiGateResidual)
        default:
          break;
      }
#undef PI05_EPI_CASE
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}


// ---------------------------------------------------------------------------
// Persistent variant for launches with more output tiles than SMs: one CTA per SM walks
// tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the accumulator is double-buffered in TMEM
// (2 x BLOCK_N columns), so the 8 epilogue warps drain tile i while the MMA warp already
// works on tile i+1 and the TMA warp runs ahead through the shared-memory ring.
// Normal orientation only (activations on the 128-row side), no split-K.
// ---------------------------------------------------------------------------
// FIXED_MODE >= 0: compiled for that one epilogue and for the output type the forward writes
// after it (FP8 / int8 after GeGLU or bias + GELU of an FP8 / int8 GEMM, bf16 otherwise).
template <int OP, int BLOCK_N, int STAGES, bool B_MN, int EPI_WARPS, int FIXED_MODE = -1>
__global__ void __launch_bounds__(gemm_threads(EPI_WARPS), 1)
gemm_umma_persistent_kernel(const __grid_constant__ CUtensorMap tmap_a,
                            const __grid_constant__ CUtensorMap tmap_b, const GemmParams p,
                            const int tiles_a, const int tiles_b, const int total_tiles) {
  using T = OpTraits<OP>;
  static_assert(BLOCK_N % 16 == 0 && BLOCK_N >= 16 && BLOCK_N <= 256, "bad BLOCK_N");
  static_assert(EPI_WARPS % 4 == 0 && EPI_WARPS >= 4 && EPI_WARPS <= 16, "whole lane quarters");
  constexpr int kEpilogueThreads = 32 * EPI_WARPS;
  constexpr int kHalves = EPI_WARPS / 4;
  constexpr int kBlockK = 128 / T::kElemBytes;
  constexpr int kStageBBytes = BLOCK_N * 128;
  constexpr int kStageBytes = kStageABytes + kStageBBytes;
  constexpr int kFixedOut = FIXED_MODE < 0 ? -1
                            : !(FIXED_MODE == kEpiBiasGelu || FIXED_MODE == kEpiGeglu) ? kOutBf16
                            : OP == kOpE4m3                                          ? kOutE4m3
                            : OP == kOpS8                                            ? kOutS8
                                                                                     : kOutBf16;
  constexpr uint32_t kTmemCols = 2 * BLOCK_N <= 32    ? 32u
                                 : 2 * BLOCK_N <= 64  ? 64u
                                 : 2 * BLOCK_N <= 128 ? 128u
                                 : 2 * BLOCK_N <= 256 ? 256u
                                                      : 512u;
  constexpr uint32_t kIdesc =
      ptx::make_idesc(T::kCFormat, T::kFormat, T::kFormat, 0, B_MN ? 1 : 0, 128, BLOCK_N);

  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * kStageBytes);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* s_vectors = reinterpret_cast<float*>(smem + STAGES * kStageBytes + 512);  // [2][3][256]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int my_tiles = (total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], EPI_WARPS);  // one arrival per epilogue warp
    }
    ptx::fence_mbar_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  auto decode = [&](int local, int* ta, int* tb, int* b0, int* b1) {
    const int tile = static_cast<int>(blockIdx.x) + local * static_cast<int>(gridDim.x);
    const int per_batch = tiles_a * tiles_b;
    const int batch = tile / per_batch;
    const int in_batch = tile - batch * per_batch;
    // raster order: row tiles in groups of p.group_a; inside a group the row tile runs fastest
    // (CTAs of a wave share the B tile) and every column tile is visited before the next group,
    // so a group's A rows (sized to stay in L2) are fetched from HBM once
    const int group = in_batch / (p.group_a * tiles_b);
    const int in_group = in_batch - group * p.group_a * tiles_b;
    const int group_rows = min(p.group_a, tiles_a - group * p.group_a);
    *tb = in_group / group_rows;
    *ta = group * p.group_a + in_group - *tb * group_rows;
    *b0 = batch % p.nb0;
    *b1 = batch / p.nb0;
  };

  if (warp == 0) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_b);
      bool ok = true;
      long long it = 0;
      for (int local = 0; local < my_tiles && ok; ++local) {
        int ta, tb, b0, b1;
        decode(local, &ta, &tb, &b0, &b1);
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = static_cast<int>(it % STAGES);
          const long long round = it / STAGES;
          if (round > 0) ok = ptx::mbar_wait(&empty_bar[s], static_cast<uint32_t>((round - 1) & 1));
          if (!ok) break;
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kStageABytes;
          ptx::mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
          ptx::tma_load_4d(sa, &tmap_a, &full_bar[s], kb * kBlockK, ta * kTileRowsA, b0, b1);
          if constexpr (B_MN) {
#pragma unroll
            for (int chunk = 0; chunk < BLOCK_N / kBlockK; ++chunk) {
              ptx::tma_load_4d(sb + chunk * (kBlockK * 128), &tmap_b, &full_bar[s],
                               tb * BLOCK_N + chunk * kBlockK, kb * kBlockK, b0, b1);
            }
          } else if (p.blocked_b) {
            ptx::tma_load_4d(sb, &tmap_b, &full_bar[s], 0, tb * BLOCK_N, kb, 0);
          } else {
            ptx::tma_load_4d(sb, &tmap_b, &full_bar[s], kb * kBlockK, tb * BLOCK_N, b0, b1);
          }
        }
      }
      if (!ok) atomicCAS(p.status, 0, kGemmTimeoutProducer);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      long long it = 0;
      for (int local = 0; local < my_tiles; ++local) {
        const int buf = local & 1;
        if (ok && local >= 2) {
          ok = ptx::mbar_wait(&acc_empty[buf], static_cast<uint32_t>(((local >> 1) - 1) & 1));
          ptx::tc_fence_after();
        }
        for (int kb = 0; kb < p.num_kb && ok; ++kb, ++it) {
          const int s = static_cast<int>(it % STAGES);
          ok = ptx::mbar_wait(&full_bar[s], static_cast<uint32_t>((it / STAGES) & 1));
          if (!ok) break;
          ptx::tc_fence_after();
          const uint32_t a_addr = ptx::smem_u32(smem + s * kStageBytes);
          const uint32_t b_addr = a_addr + kStageABytes;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t adesc = ptx::make_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? ptx::make_smem_desc(b_addr + k * (kBlockK / 4) * 128, kBlockK * 128, 1024)
                                        : ptx::make_smem_desc(b_addr + k * 32, 16, 1024);
            ptx::umma<T::kKind>(tmem_base + buf * BLOCK_N, adesc, bdesc, kIdesc,
                                (kb | k) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[s]);
        }
        // signal the epilogue even after a timeout so that it never waits on a dead pipeline
        ptx::umma_commit(&acc_full[buf]);
      }
      if (!ok) atomicCAS(p.status, 0, kGemmTimeoutMma);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const int ep_tid = threadIdx.x - 64;
    for (int local = 0; local < my_tiles; ++local) {
      const int buf = local & 1;
      int ta, tb, b0, b1;
      decode(local, &ta, &tb, &b0, &b1);
      float* s_scale = s_vectors + buf * 768;
      float* s_bias = s_scale + 256;
      float* s_gate = s_bias + 256;
      const int gi = ta * kTileRowsA + row_in_tile;
      const long long out_base = (long long)b0 * p.out_sb0 + (long long)b1 * p.out_sb1;
      const float* row_scale =
          p.row_scale != nullptr ? p.row_scale + (long long)b0 * p.row_scale_sb0 : nullptr;
      for (int j = ep_tid; j < BLOCK_N; j += kEpilogueThreads) {
        const int idx = tb * BLOCK_N + j;
        const bool in = idx < p.rows_b;
        s_scale[j] = p.col_scale != nullptr && in ? p.col_scale[idx] : 1.0f;
        s_bias[j] = p.bias != nullptr && in ? __bfloat162float(p.bias[idx]) : 0.0f;
        s_gate[j] = p.gate != nullptr && in ? __bfloat162float(p.gate[idx]) : 0.0f;
      }
      float sr = p.alpha;
      if (row_scale != nullptr && gi < p.rows_a) sr = p.alpha * row_scale[gi];
      asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");

      auto wait_acc = [&] {
        const bool ok = ptx::mbar_wait(&acc_full[buf], static_cast<uint32_t>((local >> 1) & 1));
        if (!ok && lane == 0) atomicCAS(p.status, 0, kGemmTimeoutEpilogue);
        ptx::tc_fence_after();
      };
      const uint32_t taddr_row =
          tmem_base + buf * BLOCK_N + (static_cast<uint32_t>(quarter * 32) << 16);
      AccSource<OP, BLOCK_N, false> acc{taddr_row, nullptr, 0, 1};
      const int mode = FIXED_MODE >= 0 ? FIXED_MODE : p.mode;
      if (mode == kEpiGeglu) {
        wait_acc();
        epilogue_geglu_normal<OP, BLOCK_N, kHalves, kFixedOut>(p, acc, gi, tb, out_base, sr, half,
                                                               s_scale);
      } else {
#define PI05_EPI_CASE(MODE)                                                                    \
  case MODE:                                                                                   \
    epilogue_normal<OP, BLOCK_N, MODE, kHalves, kFixedOut>(p, acc, gi, tb, out_base, sr, half, \
                                                           s_scale, s_bias, s_gate, wait_acc); \
    break;
        switch (mode) {
          PI05_EPI_CASE(kEpiStore)
          PI05_EPI_CASE(kEpiBiasGelu)
          PI05_EPI_CASE(kEpiBiasSilu)
          PI05_EPI_CASE(kEpiBiasResidual)
          PI05_EPI_CASE(kEpiBiasPos)
          PI05_EPI_CASE(kEpiGateResidual)
          default:
            wait_acc();
            break;
        }
#undef PI05_EPI_CASE
      }
      // this warp has read everything it needs from the accumulator buffer
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[buf]);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace pi05
