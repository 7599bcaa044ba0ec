#include "weights.cuh"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace pi05 {
namespace {

constexpr uint64_t kLcgA = 6364136223846793005ull;
constexpr uint64_t kLcgC = 1442695040888963407ull;
constexpr uint64_t kSeedXor = 0x9E3779B97F4A7C15ull;
constexpr int kChunk = 64;  // consecutive stream elements per thread

__device__ __forceinline__ void lcg_jump(uint64_t n, uint64_t* a_out, uint64_t* c_out) {
  uint64_t acc_a = 1, acc_c = 0, cur_a = kLcgA, cur_c = kLcgC;
  while (n != 0) {
    if (n & 1) {
      acc_a *= cur_a;
      acc_c = acc_c * cur_a + cur_c;
    }
    cur_c = (cur_a + 1) * cur_c;
    cur_a *= cur_a;
    n >>= 1;
  }
  *a_out = acc_a;
  *c_out = acc_c;
}

__global__ void lcg_fill_kernel(__nv_bfloat16* dst, uint64_t state0, uint64_t offset,
                                long long count) {
  const long long chunk = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long begin = chunk * kChunk;
  if (begin >= count) return;
  uint64_t ja, jc;
  lcg_jump(offset + static_cast<uint64_t>(begin), &ja, &jc);
  uint64_t state = ja * state0 + jc;
  const long long end = begin + kChunk < count ? begin + kChunk : count;
  for (long long i = begin; i < end; ++i) {
    state = state * kLcgA + kLcgC;
    const uint32_t bits = static_cast<uint32_t>(state >> 33);
    const float unit = __fdiv_rn(static_cast<float>(bits), 2147483648.0f);
    const float value = __fmul_rn(__fsub_rn(__fmul_rn(unit, 2.0f), 1.0f), 0.02f);
    dst[i] = __float2bfloat16(value);
  }
}

// Seeded N(0, 0.02): element i = (sum of the twelve 16-bit fields of SplitMix64 outputs at
// counters 3i+1..3i+3, minus 393210) * (0.02 / 65536), an Irwin-Hall sum with unit variance in
// units of 65536. Integer arithmetic and one float multiply, so any host restatement matches
// bit for bit.
__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__global__ void normal_fill_kernel(__nv_bfloat16* dst, uint64_t key, uint64_t offset,
                                   long long count) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)blockDim.x * gridDim.x;
  for (; i < count; i += stride) {
    const uint64_t index = offset + static_cast<uint64_t>(i);
    int total = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const uint64_t z = splitmix64(key + (index * 3ull + static_cast<uint64_t>(j + 1)) * kSeedXor);
      total += static_cast<int>(z & 0xFFFFu) + static_cast<int>((z >> 16) & 0xFFFFu) +
               static_cast<int>((z >> 32) & 0xFFFFu) + static_cast<int>((z >> 48) & 0xFFFFu);
    }
    const float value = __fmul_rn(static_cast<float>(total - 393210), 0.02f / 65536.0f);
    dst[i] = __float2bfloat16(value);
  }
}

__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void transpose_pack_kernel(const T* src, T* dst, int k, int n,
                                      long long ldk, int row_offset, int interleave, int slot) {
  __shared__ T tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int kk = k0 + r, nn = n0 + threadIdx.x;
    tile[r][threadIdx.x] = (kk < k && nn < n) ? src[(long long)kk * n + nn] : T(0.0f);
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int nn = n0 + r, kk = k0 + threadIdx.x;
    if (nn < n && kk < k) {
      const int row = interleave ? (nn / 64) * 128 + slot * 64 + (nn % 64) : row_offset + nn;
      dst[(long long)row * ldk + kk] = tile[threadIdx.x][r];
    }
  }
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < (blockDim.x >> 5) ? scratch[lane] : 0.0f;
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

template <bool INT8, typename T>
__global__ void quantize_weight_rows_kernel(const T* src, uint8_t* dst, float* scales,
                                            int cols, long long ld) {
  __shared__ float scratch[32];
  const int row = blockIdx.x;
  const T* in = src + (long long)row * ld;
  uint8_t* out = dst + (long long)row * ld;
  float amax = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) amax = fmaxf(amax, fabsf(widen(in[c])));
  amax = block_max(amax, scratch);
  float scale;
  if (INT8) {
    scale = fmaxf(__fdiv_rn(amax, 127.0f), 1.0e-12f);
  } else {
    scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
  }
  if (threadIdx.x == 0) scales[row] = scale;
  const float inverse = __fdiv_rn(1.0f, scale);
  for (int c = threadIdx.x; c < ld; c += blockDim.x) {
    const float w = c < cols ? widen(in[c]) : 0.0f;
    if (INT8) {
      const float q = fminf(127.0f, fmaxf(-128.0f, roundf(__fdiv_rn(w, scale))));
      out[c] = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(q)));
    } else {
      const float scaled = fminf(448.0f, fmaxf(-448.0f, __fmul_rn(w, inverse)));
      out[c] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(scaled, __NV_SATFINITE, __NV_E4M3));
    }
  }
}

__global__ void convert_kernel(const void* src, void* dst, long long count, int to_f32) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    if (to_f32) {
      static_cast<float*>(dst)[i] = __bfloat162float(static_cast<const __nv_bfloat16*>(src)[i]);
    } else {
      static_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(static_cast<const float*>(src)[i]);
    }
  }
}

}  // namespace

cudaError_t launch_convert(const void* src, void* dst, long long count, int to_f32, cudaStream_t stream) {
  if (src == nullptr || dst == nullptr || count <= 0) return cudaErrorInvalidValue;
  const int blocks = static_cast<int>(std::min<long long>((count + 255) / 256, 148 * 16));
  convert_kernel<<<blocks, 256, 0, stream>>>(src, dst, count, to_f32);
  return cudaGetLastError();
}

cudaError_t launch_lcg_fill(void* dst_bf16, uint64_t seed, uint64_t offset, long long count,
                            cudaStream_t stream) {
  if (dst_bf16 == nullptr || count <= 0) return cudaErrorInvalidValue;
  const long long chunks = (count + kChunk - 1) / kChunk;
  const int threads = 128;
  lcg_fill_kernel<<<static_cast<unsigned>((chunks + threads - 1) / threads), threads, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16*>(dst_bf16), seed ^ kSeedXor, offset, count);
  return cudaGetLastError();
}

cudaError_t launch_normal_fill(void* dst_bf16, uint64_t seed, uint64_t offset, long long count,
                               cudaStream_t stream) {
  if (dst_bf16 == nullptr || count <= 0) return cudaErrorInvalidValue;
  const int threads = 256;
  const long long blocks = (count + threads - 1) / threads;
  normal_fill_kernel<<<static_cast<unsigned>(blocks > 148 * 16 ? 148 * 16 : blocks), threads, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16*>(dst_bf16), seed ^ 0xD1B54A32D192ED03ull, offset, count);
  return cudaGetLastError();
}

cudaError_t launch_transpose_pack(const void* src, void* dst, int k, int n, long long ldk,
                                  int row_offset, int interleave, int slot, cudaStream_t stream,
                                  int f32) {
  if (src == nullptr || dst == nullptr || k <= 0 || n <= 0 || ldk < k) return cudaErrorInvalidValue;
  if (interleave && (n % 64 != 0)) return cudaErrorInvalidValue;
  dim3 grid((n + 31) / 32, (k + 31) / 32);
  if (f32) {
    transpose_pack_kernel<float><<<grid, dim3(32, 8), 0, stream>>>(
        reinterpret_cast<const float*>(src), reinterpret_cast<float*>(dst), k, n, ldk, row_offset,
        interleave, slot);
  } else {
    transpose_pack_kernel<__nv_bfloat16><<<grid, dim3(32, 8), 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(src), reinterpret_cast<__nv_bfloat16*>(dst), k, n, ldk,
        row_offset, interleave, slot);
  }
  return cudaGetLastError();
}

cudaError_t launch_quantize_weight_rows(const void* src, void* dst, float* scales, int rows,
                                        int cols, long long ld, int to_int8, cudaStream_t stream,
                                        int f32) {
  if (src == nullptr || dst == nullptr || scales == nullptr || rows <= 0 || cols <= 0 || ld < cols) {
    return cudaErrorInvalidValue;
  }
  auto* out = reinterpret_cast<uint8_t*>(dst);
  auto* narrow = reinterpret_cast<const __nv_bfloat16*>(src);
  auto* wide = reinterpret_cast<const float*>(src);
  if (to_int8 && f32) {
    quantize_weight_rows_kernel<true, float><<<rows, 256, 0, stream>>>(wide, out, scales, cols, ld);
  } else if (to_int8) {
    quantize_weight_rows_kernel<true, __nv_bfloat16><<<rows, 256, 0, stream>>>(narrow, out, scales, cols, ld);
  } else if (f32) {
    quantize_weight_rows_kernel<false, float><<<rows, 256, 0, stream>>>(wide, out, scales, cols, ld);
  } else {
    quantize_weight_rows_kernel<false, __nv_bfloat16><<<rows, 256, 0, stream>>>(narrow, out, scales, cols, ld);
  }
  return cudaGetLastError();
}

}  // namespace pi05
