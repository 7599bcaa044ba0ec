#include "row_kernels.cuh"

#include <cuda_fp8.h>

#include "launch.cuh"

namespace pi05 {
namespace {

__device__ __forceinline__ float rb(float x) { return __bfloat162float(__float2bfloat16(x)); }

__device__ __forceinline__ uint8_t e4m3_of(float scaled) {
  const float clamped = fminf(448.0f, fmaxf(-448.0f, scaled));
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ uint32_t s8_of(float scaled) {
  const float q = fminf(127.0f, fmaxf(-128.0f, roundf(scaled)));
  return static_cast<uint32_t>(static_cast<int>(q)) & 0xffu;
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

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) pairs[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return raw;
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

// Block-wide reductions; every thread gets the result. `scratch` holds 32 floats.
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < warps ? scratch[lane] : (MAX ? 0.0f : 0.0f);
  r = MAX ? warp_max(r) : warp_sum(r);
  return r;
}

// One CTA per row, one 8-element vector per thread (cols <= 8 * blockDim.x).
template <int KIND, int OUT, bool SUM = false>
__global__ void norm_rows_kernel(NormArgs a) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const int vec = threadIdx.x;
  const int nvec = a.cols >> 3;
  const bool active = vec < nvec;
  // per-column parameters: fetched before the dependency wait when nothing on the stream writes them
  uint4 pw = make_uint4(0, 0, 0, 0), pb = make_uint4(0, 0, 0, 0);
  auto fetch_params = [&]() {
    if (!active) return;
    if (KIND == kNormAda) {
      const __nv_bfloat16* style = reinterpret_cast<const __nv_bfloat16*>(a.style);
      pw = __ldg(reinterpret_cast<const uint4*>(style) + vec);
      pb = __ldg(reinterpret_cast<const uint4*>(style + a.cols) + vec);
    } else {
      if (a.weight != nullptr) pw = __ldg(reinterpret_cast<const uint4*>(a.weight) + vec);
      if (KIND == kNormLayer && a.bias != nullptr) pb = __ldg(reinterpret_cast<const uint4*>(a.bias) + vec);
    }
  };
  if (a.static_params) fetch_params();
  pdl_wait();
  if (!a.static_params) fetch_params();
  const __nv_bfloat16* in = reinterpret_cast<const __nv_bfloat16*>(a.input) + (long long)row * a.cols;
  float x[8];
  if (active) {
    if constexpr (SUM) {
      // the row itself comes first: partial products + residual (+ bias), rounded as the
      // stand-alone adding kernel rounds them, stored, and normalised from the stored values
      const long long base = (long long)row * a.cols + vec * 8;
      float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      for (int s = 0; s < a.sum_splits; ++s) {
        const float4* src = reinterpret_cast<const float4*>(a.sum_partials + s * a.sum_stride + base);
        const float4 lo = __ldcg(src);
        const float4 hi = __ldcg(src + 1);
        acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
        acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
      }
      float r[8], bv[8];
      unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.sum_residual) + base), r);
      if (a.sum_bias != nullptr) {
        unpack8(reinterpret_cast<const uint4*>(a.sum_bias)[vec], bv);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) bv[i] = 0.0f;
      }
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = (rb(acc[i]) + r[i]) + bv[i];
      const uint4 packed = pack8(y);
      reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(in))[vec] = packed;
      unpack8(packed, x);
    } else {
      unpack8(reinterpret_cast<const uint4*>(in)[vec], x);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = 0.0f;
  }
  const float inv_cols = 1.0f / static_cast<float>(a.cols);
  float mean = 0.0f;
  if (KIND == kNormLayer) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += x[i];
    mean = block_reduce<false>(s, scratch) * inv_cols;
  }
  float sq = 0.0f;
  if (active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float c = x[i] - mean;
      sq += c * c;
    }
  }
  const float inv = rsqrtf(block_reduce<false>(sq, scratch) * inv_cols + a.eps);

  float y[8];
  if (active) {
    float w[8], b[8];
    if (KIND == kNormAda) {
      unpack8(pw, w);
      unpack8(pb, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = (x[i] * inv) * (1.0f + w[i]) + b[i];
    } else {
      if (a.weight != nullptr) {
        unpack8(pw, w);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = 1.0f;
      }
      if (KIND == kNormLayer && a.bias != nullptr) {
        unpack8(pb, b);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // operand order of the reference's layer_norm kernel (normalization.cuh:117-121)
        y[i] = KIND == kNormLayer ? w[i] * (x[i] - mean) * inv + b[i] : x[i] * inv * w[i];
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = 0.0f;
  }

  if (OUT == kRowBf16) {
    if (active) {
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.output) + (long long)row * a.cols;
      reinterpret_cast<uint4*>(out)[vec] = pack8(y);
    }
  } else if (OUT == kRowE4m3) {
    if (active) {
      uint8_t* out = reinterpret_cast<uint8_t*>(a.output) + (long long)row * a.cols;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo |= static_cast<uint32_t>(e4m3_of(y[i] * a.inv_scale)) << (8 * i);
        hi |= static_cast<uint32_t>(e4m3_of(y[4 + i] * a.inv_scale)) << (8 * i);
      }
      reinterpret_cast<uint2*>(out)[vec] = make_uint2(lo, hi);
    }
  } else if (OUT == kRowInt8Static) {
    if (active) {
      int8_t* out = reinterpret_cast<int8_t*>(a.output) + (long long)row * a.cols;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo |= s8_of(rb(y[i]) * a.inv_scale) << (8 * i);
        hi |= s8_of(rb(y[4 + i]) * a.inv_scale) << (8 * i);
      }
      reinterpret_cast<uint2*>(out)[vec] = make_uint2(lo, hi);
    }
  } else {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      y[i] = rb(y[i]);
      amax = fmaxf(amax, fabsf(y[i]));
    }
    amax = block_reduce<true>(amax, scratch);
    const float scale = fmaxf(amax / 127.0f, 1.0e-12f);
    if (threadIdx.x == 0) a.row_scale[row] = scale;
    if (active) {
      int8_t* out = reinterpret_cast<int8_t*>(a.output) + (long long)row * a.cols;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float q0 = fminf(127.0f, fmaxf(-128.0f, roundf(y[i] / scale)));
        const float q1 = fminf(127.0f, fmaxf(-128.0f, roundf(y[4 + i] / scale)));
        lo |= (static_cast<uint32_t>(static_cast<int>(q0)) & 0xffu) << (8 * i);
        hi |= (static_cast<uint32_t>(static_cast<int>(q1)) & 0xffu) << (8 * i);
      }
      reinterpret_cast<uint2*>(out)[vec] = make_uint2(lo, hi);
    }
  }
}

// Many rows (the batched forward: tens of thousands of 1152- or 2048-wide rows): one WARP per
// row, eight rows per CTA, VPL 16-byte vectors per lane. All of a row's loads are in flight at
// once, the statistics are warp shuffles (no barrier, no shared memory), and a CTA keeps 18-32 KB
// of reads in flight instead of 2-4 KB, which is what an HBM-bound row kernel needs on this part.
// Same arithmetic per element as norm_rows_kernel; only the order of the row sums differs.
constexpr int kWarpRows = 8;

template <int KIND, int OUT, int VPL>
__global__ void __launch_bounds__(32 * kWarpRows) norm_rows_warp_kernel(NormArgs a) {
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarpRows + warp;
  const int nvec = a.cols >> 3;
  pdl_wait();
  if (row >= a.rows) return;
  const uint4* in = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.input) + row * a.cols);
  float x[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
    if (v < nvec) {
      unpack8(in[v], x[j]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[j][i] = 0.0f;
    }
  }
  const float inv_cols = 1.0f / static_cast<float>(a.cols);
  float mean = 0.0f;
  if (KIND == kNormLayer) {
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s += x[j][i];
    }
    mean = warp_sum(s) * inv_cols;
  }
  float sq = 0.0f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    if (lane + 32 * j < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = x[j][i] - mean;
        sq += c * c;
      }
    }
  }
  const float inv = rsqrtf(warp_sum(sq) * inv_cols + a.eps);

  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
    if (v < nvec) {
      float w[8], b[8];
      if (KIND == kNormAda) {
        const __nv_bfloat16* style = reinterpret_cast<const __nv_bfloat16*>(a.style);
        unpack8(__ldg(reinterpret_cast<const uint4*>(style) + v), w);
        unpack8(__ldg(reinterpret_cast<const uint4*>(style + a.cols) + v), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[j][i] = (x[j][i] * inv) * (1.0f + w[i]) + b[i];
      } else {
        if (a.weight != nullptr) {
          unpack8(__ldg(reinterpret_cast<const uint4*>(a.weight) + v), w);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) w[i] = 1.0f;
        }
        if (KIND == kNormLayer && a.bias != nullptr) {
          unpack8(__ldg(reinterpret_cast<const uint4*>(a.bias) + v), b);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) b[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[j][i] = KIND == kNormLayer ? w[i] * (x[j][i] - mean) * inv + b[i] : x[j][i] * inv * w[i];
        }
      }
      if (OUT == kRowInt8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          x[j][i] = rb(x[j][i]);
          amax = fmaxf(amax, fabsf(x[j][i]));
        }
      }
    }
  }
  float scale = 1.0f;
  if (OUT == kRowInt8) {
    scale = fmaxf(warp_max(amax) / 127.0f, 1.0e-12f);
    if (lane == 0) a.row_scale[row] = scale;
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int v = lane + 32 * j;
    if (v >= nvec) continue;
    const float(&y)[8] = x[j];
    if (OUT == kRowBf16) {
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.output) + row * a.cols)[v] = pack8(y);
    } else {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (OUT == kRowE4m3) {
          lo |= static_cast<uint32_t>(e4m3_of(y[i] * a.inv_scale)) << (8 * i);
          hi |= static_cast<uint32_t>(e4m3_of(y[4 + i] * a.inv_scale)) << (8 * i);
        } else if (OUT == kRowInt8Static) {
          lo |= s8_of(rb(y[i]) * a.inv_scale) << (8 * i);
          hi |= s8_of(rb(y[4 + i]) * a.inv_scale) << (8 * i);
        } else {
          const float q0 = fminf(127.0f, fmaxf(-128.0f, roundf(y[i] / scale)));
          const float q1 = fminf(127.0f, fmaxf(-128.0f, roundf(y[4 + i] / scale)));
          lo |= (static_cast<uint32_t>(static_cast<int>(q0)) & 0xffu) << (8 * i);
          hi |= (static_cast<uint32_t>(static_cast<int>(q1)) & 0xffu) << (8 * i);
        }
      }
      reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(a.output) + row * a.cols)[v] = make_uint2(lo, hi);
    }
  }
}

template <int KIND, int OUT>
cudaError_t launch_norm_warp(const NormArgs& a, cudaStream_t stream) {
  const int vpl = ((a.cols >> 3) + 31) / 32;
  const dim3 grid((a.rows + kWarpRows - 1) / kWarpRows), block(32 * kWarpRows);
  if (vpl <= 4) return launch_pdl(norm_rows_warp_kernel<KIND, OUT, 4>, grid, block, 0, stream, a);
  if (vpl <= 5) return launch_pdl(norm_rows_warp_kernel<KIND, OUT, 5>, grid, block, 0, stream, a);
  return launch_pdl(norm_rows_warp_kernel<KIND, OUT, 8>, grid, block, 0, stream, a);
}

template <int KIND>
cudaError_t launch_norm_kind(const NormArgs& a, int threads, cudaStream_t stream) {
  // a warp per row pays once there are rows enough to fill the SMs with such CTAs
  const bool by_warp = a.rows >= 1024 && (a.cols >> 3) <= 8 * 32;
  if (a.sum_partials != nullptr) {
    if constexpr (KIND == kNormRms) {
      if (by_warp || a.sum_residual == nullptr || a.sum_splits <= 0) return cudaErrorInvalidValue;
      switch (a.out) {
        case kRowBf16:
          return launch_pdl(norm_rows_kernel<KIND, kRowBf16, true>, dim3(a.rows), dim3(threads), 0, stream, a);
        case kRowE4m3:
          return launch_pdl(norm_rows_kernel<KIND, kRowE4m3, true>, dim3(a.rows), dim3(threads), 0, stream, a);
        case kRowInt8:
          return launch_pdl(norm_rows_kernel<KIND, kRowInt8, true>, dim3(a.rows), dim3(threads), 0, stream, a);
        case kRowInt8Static:
          return launch_pdl(norm_rows_kernel<KIND, kRowInt8Static, true>, dim3(a.rows), dim3(threads), 0, stream, a);
        default:
          return cudaErrorInvalidValue;
      }
    } else {
      return cudaErrorInvalidValue;
    }
  }
  if (by_warp) {
    switch (a.out) {
      case kRowBf16: return launch_norm_warp<KIND, kRowBf16>(a, stream);
      case kRowE4m3: return launch_norm_warp<KIND, kRowE4m3>(a, stream);
      case kRowInt8: return launch_norm_warp<KIND, kRowInt8>(a, stream);
      case kRowInt8Static: return launch_norm_warp<KIND, kRowInt8Static>(a, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (a.out) {
    case kRowBf16:
      return launch_pdl(norm_rows_kernel<KIND, kRowBf16>, dim3(a.rows), dim3(threads), 0, stream, a);
    case kRowE4m3:
      return launch_pdl(norm_rows_kernel<KIND, kRowE4m3>, dim3(a.rows), dim3(threads), 0, stream, a);
    case kRowInt8:
      return launch_pdl(norm_rows_kernel<KIND, kRowInt8>, dim3(a.rows), dim3(threads), 0, stream, a);
    case kRowInt8Static:
      return launch_pdl(norm_rows_kernel<KIND, kRowInt8Static>, dim3(a.rows), dim3(threads), 0, stream, a);
    default:
      return cudaErrorInvalidValue;
  }
}

// ---------------------------------------------------------------------------

// One CTA per token row. Work items of 4 rotary pairs (two 8-byte loads):
// q_heads*half/4 for Q, half/4 for K, then head_dim/4 plain copies for V.
__global__ void rope_kv_kernel(RopeArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int sample = row / a.tokens;
  const int token = row - sample * a.tokens;
  const int half = a.head_dim >> 1;
  const int groups_per_head = half >> 2;
  const int q_items = a.q_heads * groups_per_head;
  const int k_items = groups_per_head;
  const int v_items = a.head_dim >> 2;
  const int width = (a.q_heads + 2) * a.head_dim;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(a.qkv) + (long long)row * width;
  const int position = a.position_offset + token;
  const float* cs = a.cos_table + (long long)position * half;
  const float* sn = a.sin_table + (long long)position * half;
  const long long cache_row = (long long)sample * a.cache_rows + a.position_offset + token;
  for (int item = threadIdx.x; item < q_items + k_items + v_items; item += blockDim.x) {
    if (item < q_items + k_items) {
      const bool is_q = item < q_items;
      const int head = is_q ? item / groups_per_head : 0;
      const int group = is_q ? item - head * groups_per_head : item - q_items;
      const __nv_bfloat16* base = src + (is_q ? head * a.head_dim : a.q_heads * a.head_dim);
      const uint2 lo_raw = reinterpret_cast<const uint2*>(base)[group];
      const uint2 hi_raw = reinterpret_cast<const uint2*>(base + half)[group];
      const __nv_bfloat162* lo2 = reinterpret_cast<const __nv_bfloat162*>(&lo_raw);
      const __nv_bfloat162* hi2 = reinterpret_cast<const __nv_bfloat162*>(&hi_raw);
      const float4 c = reinterpret_cast<const float4*>(cs)[group];
      const float4 s = reinterpret_cast<const float4*>(sn)[group];
      const float cc[4] = {c.x, c.y, c.z, c.w};
      const float ss[4] = {s.x, s.y, s.z, s.w};
      float first[4], second[4];
      float2 t0 = __bfloat1622float2(lo2[0]), t1 = __bfloat1622float2(lo2[1]);
      first[0] = t0.x; first[1] = t0.y; first[2] = t1.x; first[3] = t1.y;
      t0 = __bfloat1622float2(hi2[0]); t1 = __bfloat1622float2(hi2[1]);
      second[0] = t0.x; second[1] = t0.y; second[2] = t1.x; second[3] = t1.y;
      float out_lo[4], out_hi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out_lo[i] = first[i] * cc[i] - second[i] * ss[i];
        out_hi[i] = second[i] * cc[i] + first[i] * ss[i];
      }
      uint2 lo_out, hi_out;
      __nv_bfloat162* lo_o = reinterpret_cast<__nv_bfloat162*>(&lo_out);
      __nv_bfloat162* hi_o = reinterpret_cast<__nv_bfloat162*>(&hi_out);
      lo_o[0] = __floats2bfloat162_rn(out_lo[0], out_lo[1]);
      lo_o[1] = __floats2bfloat162_rn(out_lo[2], out_lo[3]);
      hi_o[0] = __floats2bfloat162_rn(out_hi[0], out_hi[1]);
      hi_o[1] = __floats2bfloat162_rn(out_hi[2], out_hi[3]);
      __nv_bfloat16* dst =
          is_q ? reinterpret_cast<__nv_bfloat16*>(a.q_out) +
                     ((long long)row * a.q_heads + head) * a.head_dim
               : reinterpret_cast<__nv_bfloat16*>(a.k_cache) + cache_row * a.head_dim;
      reinterpret_cast<uint2*>(dst)[group] = lo_out;
      reinterpret_cast<uint2*>(dst + half)[group] = hi_out;
    } else {
      const int group = item - q_items - k_items;
      const __nv_bfloat16* base = src + (a.q_heads + 1) * a.head_dim;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.v_cache) + cache_row * a.head_dim;
      reinterpret_cast<uint2*>(dst)[group] = reinterpret_cast<const uint2*>(base)[group];
    }
  }
}

// ---------------------------------------------------------------------------

// One warp per row, up to 1024 columns held in registers.
__global__ void softmax_rows_kernel(__nv_bfloat16* scores, int rows_per_batch, int batches,
                                    long long batch_stride, int cols, long long ld) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= rows_per_batch * batches) return;
  const int batch = warp_global / rows_per_batch;
  const int row = warp_global - batch * rows_per_batch;
  __nv_bfloat16* data = scores + (long long)batch * batch_stride + (long long)row * ld;
  float v[32];
  float maximum = -1.0e30f;
#pragma unroll
  for (int it = 0; it < 32; ++it) {
    const int col = it * 32 + lane;
    v[it] = col < cols ? __bfloat162float(data[col]) : -1.0e30f;
    maximum = fmaxf(maximum, v[it]);
  }
  maximum = warp_max(maximum);
  float sum = 0.0f;
#pragma unroll
  for (int it = 0; it < 32; ++it) {
    v[it] = __expf(v[it] - maximum);
    sum += v[it];
  }
  sum = warp_sum(sum);
  const float inverse = 1.0f / sum;
#pragma unroll
  for (int it = 0; it < 32; ++it) {
    const int col = it * 32 + lane;
    if (col < cols) data[col] = __float2bfloat16(v[it] * inverse);
  }
}

// ---------------------------------------------------------------------------

// One thread per 8 output columns of one patch row.
template <int OUT>
__global__ void patchify_kernel(PatchifyArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = a.ld >> 3;
  const int side = a.image_size / a.patch_size;
  const int area = a.patch_size * a.patch_size;
  const int patch_width = 3 * area;
  const long long total = (long long)a.n_images * side * side * vec_per_row;
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const int vec = static_cast<int>(index % vec_per_row);
  const long long prow = index / vec_per_row;
  const int image = static_cast<int>(prow / (side * side));
  const int in_image = static_cast<int>(prow - (long long)image * side * side);
  const int py = in_image / side, px = in_image - py * side;
  float y[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int col = vec * 8 + i;
    float value = 0.0f;
    if (col < patch_width) {
      const int channel = col / area;
      const int pixel = col - channel * area;
      const int dy = pixel / a.patch_size, dx = pixel - dy * a.patch_size;
      const int yy = py * a.patch_size + dy, xx = px * a.patch_size + dx;
      const long long src =
          a.nchw ? (((long long)image * 3 + channel) * a.image_size + yy) * a.image_size + xx
                 : (((long long)image * a.image_size + yy) * a.image_size + xx) * 3 + channel;
      value = a.f32_patches != nullptr ? a.f32_patches[prow * patch_width + col]
                                       : (static_cast<float>(a.images[src]) / 255.0f) * 2.0f - 1.0f;
    }
    y[i] = value;
  }
  if (OUT == kRowBf16) {
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.patches) + prow * a.ld;
    reinterpret_cast<uint4*>(out)[vec] = pack8(y);
  } else {
    uint8_t* out = reinterpret_cast<uint8_t*>(a.patches) + prow * a.ld;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= static_cast<uint32_t>(e4m3_of(rb(y[i]) * a.inv_scale)) << (8 * i);
      hi |= static_cast<uint32_t>(e4m3_of(rb(y[4 + i]) * a.inv_scale)) << (8 * i);
    }
    reinterpret_cast<uint2*>(out)[vec] = make_uint2(lo, hi);
  }
}

// One thread per output element, for unpadded rows (ld not a multiple of 8).
__global__ void patchify_scalar_kernel(PatchifyArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int side = a.image_size / a.patch_size;
  const int area = a.patch_size * a.patch_size;
  const int patch_width = 3 * area;
  const long long total = (long long)a.n_images * side * side * patch_width;
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const int col = static_cast<int>(index % patch_width);
  const long long prow = index / patch_width;
  const int image = static_cast<int>(prow / (side * side));
  const int in_image = static_cast<int>(prow - (long long)image * side * side);
  const int py = in_image / side, px = in_image - py * side;
  const int channel = col / area;
  const int pixel = col - channel * area;
  const int dy = pixel / a.patch_size, dx = pixel - dy * a.patch_size;
  const int yy = py * a.patch_size + dy, xx = px * a.patch_size + dx;
  const long long src =
      a.nchw ? (((long long)image * 3 + channel) * a.image_size + yy) * a.image_size + xx
             : (((long long)image * a.image_size + yy) * a.image_size + xx) * 3 + channel;
  const float value = a.f32_patches != nullptr
                          ? a.f32_patches[prow * patch_width + col]
                          : (static_cast<float>(a.images[src]) / 255.0f) * 2.0f - 1.0f;
  reinterpret_cast<__nv_bfloat16*>(a.patches)[prow * a.ld + col] = __float2bfloat16(value);
}

__global__ void embedding_kernel(const __nv_bfloat16* table, const uint32_t* ids,
                                 __nv_bfloat16* out, int batch, int tokens, int width, int vocab,
                                 int out_rows_per_batch, int row_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = width >> 3;
  const long long total = (long long)batch * tokens * vec_per_row;
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const int vec = static_cast<int>(index % vec_per_row);
  const long long tok = index / vec_per_row;
  const int sample = static_cast<int>(tok / tokens);
  const int t = static_cast<int>(tok - (long long)sample * tokens);
  const uint32_t id = ids[tok];
  const float normalizer = sqrtf(static_cast<float>(width));
  float y[8];
  if (id < static_cast<uint32_t>(vocab)) {
    unpack8(reinterpret_cast<const uint4*>(table + (long long)id * width)[vec], y);
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] *= normalizer;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = 0.0f;
  }
  __nv_bfloat16* dst = out + ((long long)sample * out_rows_per_batch + row_offset + t) * width;
  reinterpret_cast<uint4*>(dst)[vec] = pack8(y);
}

// One CTA per row; two passes (the row stays in L1/L2 between them).
__global__ void quantize_rows_int8_kernel(const __nv_bfloat16* input, int8_t* output,
                                          float* row_scale, int cols, long long ld_in,
                                          long long ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* in = input + (long long)row * ld_in;
  const int nvec = cols >> 3;
  float amax = 0.0f;
  for (int vec = threadIdx.x; vec < nvec; vec += blockDim.x) {
    float x[8];
    unpack8(reinterpret_cast<const uint4*>(in)[vec], x);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
  }
  amax = block_reduce<true>(amax, scratch);
  const float scale = fmaxf(amax / 127.0f, 1.0e-12f);
  if (threadIdx.x == 0) row_scale[row] = scale;
  int8_t* out = output + (long long)row * ld_out;
  for (int vec = threadIdx.x; vec < nvec; vec += blockDim.x) {
    float x[8];
    unpack8(reinterpret_cast<const uint4*>(in)[vec], x);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float q0 = fminf(127.0f, fmaxf(-128.0f, roundf(x[i] / scale)));
      const float q1 = fminf(127.0f, fmaxf(-128.0f, roundf(x[4 + i] / scale)));
      lo |= (static_cast<uint32_t>(static_cast<int>(q0)) & 0xffu) << (8 * i);
      hi |= (static_cast<uint32_t>(static_cast<int>(q1)) & 0xffu) << (8 * i);
    }
    reinterpret_cast<uint2*>(out)[vec] = make_uint2(lo, hi);
  }
}

__global__ void quantize_e4m3_kernel(const __nv_bfloat16* input, uint8_t* output, long long count,
                                     float inv_scale) {
  pdl_launch_dependents();
  pdl_wait();
  long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)blockDim.x * gridDim.x;
  for (; index < count; index += stride) {
    output[index] = e4m3_of(__bfloat162float(input[index]) * inv_scale);
  }
}

__global__ void quantize_s8_kernel(const __nv_bfloat16* input, int8_t* output, long long count,
                                   float inv_scale) {
  pdl_launch_dependents();
  pdl_wait();
  long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)blockDim.x * gridDim.x;
  for (; index < count; index += stride) {
    output[index] = static_cast<int8_t>(s8_of(__bfloat162float(input[index]) * inv_scale));
  }
}

// One thread per 8 consecutive outputs; the splits' loads are all in flight together.
__global__ void sum_partials_kernel(const float* __restrict__ partials, int splits, long long count,
                                    int cols, const __nv_bfloat16* residual,
                                    const __nv_bfloat16* bias, __nv_bfloat16* out) {
  pdl_launch_dependents();
  pdl_wait();
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long base = vec * 8;
  if (base >= count) return;
  float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  for (int s = 0; s < splits; ++s) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(partials + s * count + base));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(partials + s * count + base) + 1);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
  float r[8], bv[8];
  unpack8(*reinterpret_cast<const uint4*>(residual + base), r);
  if (bias != nullptr) {
    unpack8(*reinterpret_cast<const uint4*>(bias + base % cols), bv);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) bv[i] = 0.0f;
  }
  float y[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) y[i] = (rb(acc[i]) + r[i]) + bv[i];
  *reinterpret_cast<uint4*>(out + base) = pack8(y);
}

__global__ void euler_kernel(__nv_bfloat16* state, const __nv_bfloat16* velocity, long long count,
                             float dt) {
  pdl_launch_dependents();
  pdl_wait();
  long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)blockDim.x * gridDim.x;
  for (; index < count; index += stride) {
    state[index] =
        __float2bfloat16(__bfloat162float(state[index]) + dt * __bfloat162float(velocity[index]));
  }
}

}  // namespace

cudaError_t launch_norm(const NormArgs& a, cudaStream_t stream) {
  if (a.input == nullptr || a.output == nullptr || a.rows <= 0 || a.cols <= 0 ||
      (a.cols & 7) != 0 || a.cols > 8192 || (a.kind == kNormAda && a.style == nullptr) ||
      (a.out == kRowInt8 && a.row_scale == nullptr)) {
    return cudaErrorInvalidValue;
  }
  const int threads = (((a.cols >> 3) + 31) / 32) * 32;
  switch (a.kind) {
    case kNormLayer:
      return launch_norm_kind<kNormLayer>(a, threads, stream);
    case kNormRms:
      return launch_norm_kind<kNormRms>(a, threads, stream);
    case kNormAda:
      return launch_norm_kind<kNormAda>(a, threads, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

cudaError_t launch_rope(const RopeArgs& a, cudaStream_t stream) {
  if (a.qkv == nullptr || a.q_out == nullptr || a.k_cache == nullptr || a.v_cache == nullptr ||
      a.cos_table == nullptr || a.sin_table == nullptr || a.rows <= 0 || a.tokens <= 0 ||
      a.rows % a.tokens != 0 || a.q_heads <= 0 || a.head_dim <= 0 || (a.head_dim & 7) != 0 ||
      a.position_offset < 0 || a.position_offset + a.tokens > a.cache_rows) {
    return cudaErrorInvalidValue;
  }
  return launch_pdl(rope_kv_kernel, dim3(a.rows), dim3(128), 0, stream, a);
}

cudaError_t launch_softmax(void* scores, int rows_per_batch, int batches, long long batch_stride,
                           int cols, long long ld, cudaStream_t stream) {
  if (scores == nullptr || rows_per_batch <= 0 || batches <= 0 || cols <= 0 || cols > 1024 ||
      ld < cols) {
    return cudaErrorInvalidValue;
  }
  const long long warps = (long long)rows_per_batch * batches;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  return launch_pdl(softmax_rows_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0,
                    stream, reinterpret_cast<__nv_bfloat16*>(scores), rows_per_batch, batches,
                    batch_stride, cols, ld);
}

cudaError_t launch_patchify(const PatchifyArgs& a, cudaStream_t stream) {
  if ((a.images == nullptr && a.f32_patches == nullptr) || a.patches == nullptr || a.n_images <= 0 || a.image_size <= 0 ||
      a.patch_size <= 0 || a.image_size % a.patch_size != 0 ||
      a.ld < 3 * a.patch_size * a.patch_size || (a.out != kRowBf16 && a.out != kRowE4m3)) {
    return cudaErrorInvalidValue;
  }
  const int side = a.image_size / a.patch_size;
  if ((a.ld & 15) != 0) {
    if (a.out != kRowBf16) return cudaErrorInvalidValue;
    const long long count = (long long)a.n_images * side * side * 3 * a.patch_size * a.patch_size;
    return launch_pdl(patchify_scalar_kernel, dim3(static_cast<unsigned>((count + 255) / 256)),
                      dim3(256), 0, stream, a);
  }
  const long long total = (long long)a.n_images * side * side * (a.ld >> 3);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  if (a.out == kRowBf16) {
    return launch_pdl(patchify_kernel<kRowBf16>, dim3(blocks), dim3(threads), 0, stream, a);
  }
  return launch_pdl(patchify_kernel<kRowE4m3>, dim3(blocks), dim3(threads), 0, stream, a);
}

cudaError_t launch_embedding(const void* table, const uint32_t* ids, void* out, int batch,
                             int tokens, int width, int vocab, int out_rows_per_batch,
                             int row_offset, cudaStream_t stream) {
  if (table == nullptr || ids == nullptr || out == nullptr || batch <= 0 || tokens <= 0 ||
      width <= 0 || (width & 7) != 0 || vocab <= 0 || row_offset < 0 ||
      row_offset + tokens > out_rows_per_batch) {
    return cudaErrorInvalidValue;
  }
  const long long total = (long long)batch * tokens * (width >> 3);
  const int threads = 256;
  return launch_pdl(embedding_kernel, dim3(static_cast<unsigned>((total + threads - 1) / threads)),
                    dim3(threads), 0, stream, reinterpret_cast<const __nv_bfloat16*>(table), ids,
                    reinterpret_cast<__nv_bfloat16*>(out), batch, tokens, width, vocab,
                    out_rows_per_batch, row_offset);
}

cudaError_t launch_quantize_rows_int8(const void* input, int8_t* output, float* row_scale, int rows,
                                      int cols, long long ld_in, long long ld_out,
                                      cudaStream_t stream) {
  if (input == nullptr || output == nullptr || row_scale == nullptr || rows <= 0 || cols <= 0 ||
      (cols & 7) != 0 || (ld_in & 7) != 0 || (ld_out & 7) != 0) {
    return cudaErrorInvalidValue;
  }
  const int threads = cols >= 2048 ? 256 : 128;
  return launch_pdl(quantize_rows_int8_kernel, dim3(rows), dim3(threads), 0, stream,
                    reinterpret_cast<const __nv_bfloat16*>(input), output, row_scale, cols, ld_in,
                    ld_out);
}

cudaError_t launch_quantize_e4m3(const void* input, uint8_t* output, long long count,
                                 float inv_scale, cudaStream_t stream) {
  if (input == nullptr || output == nullptr || count <= 0) return cudaErrorInvalidValue;
  const int threads = 256;
  const long long blocks = (count + threads - 1) / threads;
  return launch_pdl(quantize_e4m3_kernel, dim3(static_cast<unsigned>(blocks > 1184 ? 1184 : blocks)),
                    dim3(threads), 0, stream, reinterpret_cast<const __nv_bfloat16*>(input), output,
                    count, inv_scale);
}

cudaError_t launch_quantize_s8(const void* input, int8_t* output, long long count, float inv_scale,
                               cudaStream_t stream) {
  if (input == nullptr || output == nullptr || count <= 0) return cudaErrorInvalidValue;
  const int threads = 256;
  const long long blocks = (count + threads - 1) / threads;
  return launch_pdl(quantize_s8_kernel, dim3(static_cast<unsigned>(blocks > 1184 ? 1184 : blocks)),
                    dim3(threads), 0, stream, reinterpret_cast<const __nv_bfloat16*>(input), output,
                    count, inv_scale);
}

cudaError_t launch_sum_partials(const float* partials, int splits, long long count, int cols,
                                const void* residual, const void* bias, void* out,
                                cudaStream_t stream) {
  if (partials == nullptr || residual == nullptr || out == nullptr || splits <= 0 || count <= 0 ||
      cols <= 0 || (cols & 7) != 0 || count % cols != 0) {
    return cudaErrorInvalidValue;
  }
  const int threads = 256;
  const long long vecs = count / 8;
  return launch_pdl(sum_partials_kernel, dim3(static_cast<unsigned>((vecs + threads - 1) / threads)),
                    dim3(threads), 0, stream, partials, splits, count, cols,
                    reinterpret_cast<const __nv_bfloat16*>(residual),
                    reinterpret_cast<const __nv_bfloat16*>(bias), reinterpret_cast<__nv_bfloat16*>(out));
}

cudaError_t launch_euler(void* state, const void* velocity, long long count, float dt,
                         cudaStream_t stream) {
  if (state == nullptr || velocity == nullptr || count <= 0) return cudaErrorInvalidValue;
  const int threads = 256;
  const long long blocks = (count + threads - 1) / threads;
  return launch_pdl(euler_kernel, dim3(static_cast<unsigned>(blocks > 1184 ? 1184 : blocks)),
                    dim3(threads), 0, stream, reinterpret_cast<__nv_bfloat16*>(state),
                    reinterpret_cast<const __nv_bfloat16*>(velocity), count, dt);
}

}  // namespace pi05
