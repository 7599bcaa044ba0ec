// Pieces shared by the attention kernels: thread layout and the output store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "fmha.h"

namespace pi05 {

constexpr int kFmhaSoftmaxWarps = 16;  // 4 per TMEM lane quarter, one key-column group each
constexpr int kFmhaSoftmaxThreads = 32 * kFmhaSoftmaxWarps;
constexpr int kFmhaThreads = 64 + kFmhaSoftmaxThreads;
constexpr int kFmhaQBytes = 4 * 16384;        // up to 4 head-dim chunks of [128 x 128 B]
constexpr int kFmhaStageBytes = 256 * 128;    // one ring stage: two K chunks [128 keys x 128 B] or one V sub-block
constexpr int kFmhaExchangeBytes = 3 * 4 * 128 * 4;  // per-row partial maxima (x2) and sums of the 4 column groups

// One 16-column chunk of the output accumulator (fp32 bits in `raw`), normalised by `inv`, to
// global memory as bf16 or as e4m3(clamp(bf16(o) * out_inv_scale)); widest aligned stores.
__device__ __forceinline__ void fmha_store_chunk16(const FmhaParams& p, const uint32_t (&raw)[16],
                                                   float inv, long long out_row, int d0, int hd) {
  const int valid = min(16, hd - d0);
  if (p.out_e4m3) {
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + out_row + d0;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      // the reference rounds the attention output to 16 bits before quantising it
      const float o = __bfloat162float(__float2bfloat16(__uint_as_float(raw[t]) * inv));
      const float clamped = fminf(448.0f, fmaxf(-448.0f, o * p.out_inv_scale));
      const uint32_t byte = static_cast<uint8_t>(__nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3));
      w[t >> 2] |= byte << (8 * (t & 3));
    }
    // head_dim is a multiple of 8, so a row's chunk starts on an 8-byte boundary
    // whenever the head stride and leading dimension do: widest aligned store wins
    const uintptr_t addr = reinterpret_cast<uintptr_t>(dst);
    if (valid == 16 && (addr & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if ((addr & 7u) == 0 && (valid & 7) == 0) {
      *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
      if (valid == 16) *reinterpret_cast<uint2*>(dst + 8) = make_uint2(w[2], w[3]);
    } else {
      for (int t = 0; t < valid; ++t) dst[t] = static_cast<uint8_t>(w[t >> 2] >> (8 * (t & 3)));
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + out_row + d0;
    uint32_t w[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(raw[2 * t]) * inv,
                                                       __uint_as_float(raw[2 * t + 1]) * inv);
      w[t] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    const uintptr_t addr = reinterpret_cast<uintptr_t>(dst);
    if ((addr & 15u) == 0 && (valid & 7) == 0) {
      reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      if (valid == 16) reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
      for (int t = 0; t < valid; ++t) {
        dst[t] = reinterpret_cast<const __nv_bfloat16*>(w)[t];
      }
    }
  }
}

}  // namespace pi05
