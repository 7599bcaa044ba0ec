// The F16 / E4M3 operator names the reference's FP8 executor binds
// (crates/apxinf-cuda/src/ffi/custom.rs:34-884, adapters/custom_kernels.cu), its FP8 GEMM family
// (ffi/cublaslt.rs, adapters/cublaslt_adapter.cu:1092-1294; ffi/cutlass.rs:85,
// adapters/cutlass_fp8_adapter.cu) and the W8A8 GEMM names (adapters/cutlass_w8a8_adapter.cu,
// w8a8_adapter.cu:31-46), with the reference's storage types: activations F16, quantised
// tensors E4M3, every intermediate in fp32 and one rounding per output.
//
// The PI0.5 engine of this library does not launch the row operators of this file: it keeps
// its activations in BF16 and performs the same arithmetic inside GEMM epilogues and fused row
// kernels. They exist so that a host that links the reference's operators one by one finds
// every name; each is checked against the reference's compiled kernel
// (tests/test_ref_ops_f16_gpu.py). The GEMM names run on the tcgen05 GEMM of this library
// (E4M3 operands with the weight in the reference's [k, n] layout as an MN-major operand).
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "../../include/pi05_apxinf_static.h"
#include "gemm.h"
#include "launch.cuh"

namespace {

constexpr int kInvalid = static_cast<int>(cudaErrorInvalidValue);
constexpr int kThreads = 256;
constexpr int kBlasInvalid = 7;         // CUBLAS_STATUS_INVALID_VALUE
constexpr int kBlasNotInitialized = 1;  // CUBLAS_STATUS_NOT_INITIALIZED
constexpr int kBlasAllocFailed = 3;     // CUBLAS_STATUS_ALLOC_FAILED
constexpr int kBlasExecutionFailed = 13;

__device__ __forceinline__ float h(const __half* p, long long i) { return __half2float(p[i]); }

__device__ __forceinline__ float gelu_tanh_exact(float x) {
  // crates/apxinf-cuda/kernels/custom/math.cuh:8-12
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

__device__ __forceinline__ uint8_t e4m3(float scaled) {
  const float clamped = fminf(448.0f, fmaxf(-448.0f, scaled));
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e4m3_value(uint8_t byte) {
  const __half_raw raw = __nv_cvt_fp8_to_halfraw(byte, __NV_E4M3);
  return __half2float(__half(raw));
}

unsigned blocks_for(long long count) {
  const long long blocks = (count + kThreads - 1) / kThreads;
  return static_cast<unsigned>(blocks < 1 ? 1 : blocks > 148 * 16 ? 148 * 16 : blocks);
}

// ---- elementwise operators: one grid-stride kernel, OP selects the formula -------------------
enum MapOp {
  kQuantize, kDequantize, kBiasGeluQuant, kBiasSiluQuant, kBiasSilu, kBias, kConcat, kEuler, kGegluQuant,
  kBiasResidual, kAdaGateResidual, kBiasPosition
};

struct MapArgs {
  const void* a;  // input / projection / gate_up / first / state
  const void* b;  // bias (may be null) / second / velocity / residual
  const void* c;  // residual / style / position table
  void* out;
  long long count;
  int cols;
  int extra;      // inner | tokens_per_view | rows of `first`
  float scalar;   // 1 / scale | scale | dt
};

template <int OP>
__global__ void map_kernel(MapArgs m) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const __half* a = static_cast<const __half*>(m.a);
  const __half* b = static_cast<const __half*>(m.b);
  const __half* c = static_cast<const __half*>(m.c);
  __half* out16 = static_cast<__half*>(m.out);
  uint8_t* out8 = static_cast<uint8_t*>(m.out);
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < m.count; i += stride) {
    const int col = static_cast<int>(i % m.cols);
    if (OP == kQuantize) {
      out8[i] = e4m3(h(a, i) * m.scalar);
    } else if (OP == kDequantize) {
      out16[i] = __float2half_rn(e4m3_value(static_cast<const uint8_t*>(m.a)[i]) * m.scalar);
    } else if (OP == kBiasGeluQuant) {
      out8[i] = e4m3(gelu_tanh_exact(h(a, i) + h(b, col)) * m.scalar);
    } else if (OP == kBiasSiluQuant || OP == kBiasSilu || OP == kBias) {
      float value = h(a, i);
      if (b != nullptr) value += h(b, col);
      if (OP != kBias) value = value / (1.0f + expf(-value));
      if (OP == kBiasSiluQuant) {
        out8[i] = e4m3(value * m.scalar);
      } else {
        out16[i] = __float2half(value);
      }
    } else if (OP == kConcat) {
      const long long first = static_cast<long long>(m.extra) * m.cols;
      out16[i] = i < first ? a[i] : b[i - first];
    } else if (OP == kEuler) {
      out16[i] = __float2half(h(a, i) + m.scalar * h(b, i));
    } else if (OP == kGegluQuant) {
      // cols = inner: gelu(gate_up[row, col]) * gate_up[row, inner + col]
      const long long row = i / m.cols;
      const __half* in = a + row * 2 * m.cols;
      out8[i] = e4m3(gelu_tanh_exact(h(in, col)) * h(in, m.cols + col) * m.scalar);
    } else if (OP == kBiasResidual) {
      float value = h(a, i) + h(c, i);
      if (b != nullptr) value += h(b, col);
      out16[i] = __float2half(value);
    } else if (OP == kAdaGateResidual) {
      out16[i] = __float2half(h(b, i) + h(a, i) * h(c, 2LL * m.cols + col));  // b = residual, c = style
    } else {
      const int token = static_cast<int>((i / m.cols) % m.extra);
      float value = h(a, i) + h(c, static_cast<long long>(token) * m.cols + col);
      if (b != nullptr) value += h(b, col);
      out16[i] = __float2half(value);
    }
  }
}

template <int OP>
int launch_map(const MapArgs& m, void* stream) {
  if (m.a == nullptr || m.out == nullptr || m.count <= 0 || m.cols <= 0) return kInvalid;
  return static_cast<int>(pi05::launch_pdl(map_kernel<OP>, dim3(blocks_for(m.count)), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), m));
}

// ---- row operators: one CTA per row --------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  __syncthreads();  // scratch may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < kThreads / 32; ++w) total += scratch[w];
  return total;
}

enum NormOp { kRms, kLayer, kAda, kResidualRms, kResidualLayer, kAdaGateRms };

struct NormArgs16 {
  const __half* input;      // input | projection
  const __half* bias;       // projection bias (fused forms, may be null)
  const __half* residual;   // fused forms
  const __half* weight;     // norm weight | style (kAda) | gate style (kAdaGateRms)
  const __half* norm_bias;  // layer-norm bias | norm style (kAdaGateRms)
  __half* hidden;           // fused forms: the new residual stream
  uint8_t* normalized;      // e4m3
  int cols;
  float eps;
  float inverse_scale;
};

template <int OP>
__global__ void __launch_bounds__(kThreads) norm_kernel(NormArgs16 a) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  __shared__ float scratch[kThreads / 32];
  constexpr bool kFused = OP == kResidualRms || OP == kResidualLayer || OP == kAdaGateRms;
  constexpr bool kLayerNorm = OP == kLayer || OP == kResidualLayer;
  const long long base = static_cast<long long>(blockIdx.x) * a.cols;
  // the value the norm sees: the input, or the new hidden state rounded to f16 as it is stored
  auto value_at = [&](int col) {
    if (!kFused) return h(a.input, base + col);
    return h(a.hidden, base + col);  // this thread's own store below
  };
  float acc = 0.0f;
  for (int col = threadIdx.x; col < a.cols; col += kThreads) {
    if (kFused) {
      float value;
      if (OP == kAdaGateRms) {
        value = h(a.residual, base + col) + h(a.input, base + col) * h(a.weight, 2LL * a.cols + col);
      } else {
        value = h(a.input, base + col) + h(a.residual, base + col);
        if (a.bias != nullptr) value += h(a.bias, col);
      }
      a.hidden[base + col] = __float2half(value);
    }
    const float v = value_at(col);
    acc += kLayerNorm ? v : v * v;
  }
  const float first = block_sum(acc, scratch) / a.cols;
  float mean = 0.0f, inverse;
  if (kLayerNorm) {
    mean = first;
    float var = 0.0f;
    for (int col = threadIdx.x; col < a.cols; col += kThreads) {
      const float centered = value_at(col) - mean;
      var += centered * centered;
    }
    inverse = rsqrtf(block_sum(var, scratch) / a.cols + a.eps);
  } else {
    inverse = rsqrtf(first + a.eps);
  }
  for (int col = threadIdx.x; col < a.cols; col += kThreads) {
    float value;
    if (kLayerNorm) {
      value = (value_at(col) - mean) * inverse;
      value = value * h(a.weight, col) + h(a.norm_bias, col);
    } else if (OP == kAda || OP == kAdaGateRms) {
      const __half* style = OP == kAda ? a.weight : a.norm_bias;
      value = value_at(col) * inverse * (1.0f + h(style, col)) + h(style, a.cols + col);
    } else {
      value = value_at(col) * inverse * h(a.weight, col);
    }
    a.normalized[base + col] = e4m3(value * a.inverse_scale);
  }
}

template <int OP>
int launch_norm(const NormArgs16& a, int rows, void* stream) {
  if (a.input == nullptr || a.normalized == nullptr || rows <= 0 || a.cols <= 0 || !(a.inverse_scale > 0.0f)) {
    return kInvalid;
  }
  return static_cast<int>(pi05::launch_pdl(norm_kernel<OP>, dim3(rows), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), a));
}

// ---- q | k | v split (+ bias) with or without rotate-half RoPE ----------------------------------
__global__ void qkv_rope_kernel(const __half* qkv, const __half* bias, __half* q, __half* k, __half* v,
                                int q_heads, int kv_heads, int head_dim, float theta, int position_offset,
                                int kv_output_offset) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const int token = blockIdx.x, head = blockIdx.y;
  const int half_dim = head_dim / 2;
  const int q_width = q_heads * head_dim, kv_width = kv_heads * head_dim;
  const long long row = static_cast<long long>(token) * (q_width + 2 * kv_width);
  for (int pair = threadIdx.x; pair < half_dim; pair += blockDim.x) {
    const float frequency = powf(theta, -static_cast<float>(pair) / half_dim);
    float sine, cosine;
    sincosf((position_offset + token) * frequency, &sine, &cosine);
    const int source = head * head_dim;  // q heads, then k heads, then v heads: all contiguous
    float first = h(qkv, row + source + pair), second = h(qkv, row + source + half_dim + pair);
    if (bias != nullptr) {
      first += h(bias, source + pair);
      second += h(bias, source + half_dim + pair);
    }
    if (head < q_heads) {
      __half* dst = q + (static_cast<long long>(token) * q_heads + head) * head_dim;
      dst[pair] = __float2half(first * cosine - second * sine);
      dst[half_dim + pair] = __float2half(second * cosine + first * sine);
    } else if (head < q_heads + kv_heads) {
      __half* dst = k + (static_cast<long long>(kv_output_offset + token) * kv_heads + (head - q_heads)) * head_dim;
      dst[pair] = __float2half(first * cosine - second * sine);
      dst[half_dim + pair] = __float2half(second * cosine + first * sine);
    } else {
      __half* dst =
          v + (static_cast<long long>(kv_output_offset + token) * kv_heads + (head - q_heads - kv_heads)) * head_dim;
      dst[pair] = __float2half(first);
      dst[half_dim + pair] = __float2half(second);
    }
  }
}

__global__ void qkv_split_kernel(const __half* qkv, const __half* bias, __half* q, __half* k, __half* v, int width) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const long long token = blockIdx.x;
  for (int col = threadIdx.x; col < 3 * width; col += blockDim.x) {
    float value = h(qkv, token * 3 * width + col);
    if (bias != nullptr) value += h(bias, col);
    __half* dst = col < width ? q : col < 2 * width ? k : v;
    dst[token * width + col % width] = __float2half(value);
  }
}

__global__ void embedding_kernel(const __half* table, const uint32_t* ids, __half* out, long long count, int width,
                                 int vocab) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const float normalizer = sqrtf(static_cast<float>(width));
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    const uint32_t id = ids[i / width];
    out[i] = id < static_cast<uint32_t>(vocab)
                 ? __float2half(h(table, static_cast<long long>(id) * width + i % width) * normalizer)
                 : __float2half(0.0f);
  }
}

// u8 image -> patch rows: (u8 / 255) * 2 - 1, rounded to f16, then quantised
// (crates/apxinf-cuda/kernels/custom/preprocess.cuh:7-61)
__global__ void patches_e4m3_kernel(const uint8_t* images, uint8_t* patches, long long count, int image_size,
                                    int patch_size, int nchw, float inverse_scale) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const int side = image_size / patch_size, area = patch_size * patch_size, width = 3 * area;
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    const int col = static_cast<int>(i % width);
    const long long prow = i / width;
    const int image = static_cast<int>(prow / (side * side));
    const int in_image = static_cast<int>(prow - static_cast<long long>(image) * side * side);
    const int py = in_image / side, px = in_image - py * side;
    const int channel = col / area, pixel = col - channel * area;
    const int dy = pixel / patch_size, dx = pixel - dy * patch_size;
    const int yy = py * patch_size + dy, xx = px * patch_size + dx;
    const long long src = nchw ? ((static_cast<long long>(image) * 3 + channel) * image_size + yy) * image_size + xx
                               : ((static_cast<long long>(image) * image_size + yy) * image_size + xx) * 3 + channel;
    const float value =
        __fsub_rn(__fmul_rn(__fdiv_rn(static_cast<float>(images[src]), 255.0f), 2.0f), 1.0f);
    patches[i] = e4m3(__half2float(__float2half_rn(value)) * inverse_scale);
  }
}

// ---- attention on F16 operands: one CTA per (query token, head), scores in shared memory -------
// k / v in up to two segments (a cached prefix and the new suffix rows), each [tokens, kv_stride].
__global__ void __launch_bounds__(kThreads)
attention_f16_kernel(const __half* q, const __half* k0, const __half* v0, int keys0, const __half* k1,
                     const __half* v1, int keys1, __half* out, int heads, int head_dim, long long kv_stride,
                     long long kv_head_stride, long long batch_q, long long batch_kv) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  extern __shared__ float scores[];  // [keys0 + keys1]
  __shared__ float scratch[kThreads / 32];
  const int token = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int keys = keys0 + keys1;
  const __half* qrow = q + batch * batch_q + (static_cast<long long>(token) * heads + head) * head_dim;
  const float scale = rsqrtf(static_cast<float>(head_dim));
  auto key_row = [&](const __half* base0, const __half* base1, int key) {
    const __half* base = key < keys0 ? base0 : base1;
    const int r = key < keys0 ? key : key - keys0;
    return base + batch * batch_kv + static_cast<long long>(r) * kv_stride + head * kv_head_stride;
  };
  float local_max = -3.0e38f;
  for (int key = threadIdx.x; key < keys; key += kThreads) {
    const __half* krow = key_row(k0, k1, key);
    float dot = 0.0f;
    for (int d = 0; d < head_dim; ++d) dot += __half2float(qrow[d]) * __half2float(krow[d]);
    scores[key] = dot * scale;
    local_max = fmaxf(local_max, dot * scale);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, d));
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = local_max;
  __syncthreads();
  float maximum = -3.0e38f;
  for (int w = 0; w < kThreads / 32; ++w) maximum = fmaxf(maximum, scratch[w]);
  float sum = 0.0f;
  for (int key = threadIdx.x; key < keys; key += kThreads) {
    const float e = __expf(scores[key] - maximum);
    scores[key] = e;
    sum += e;
  }
  const float total = block_sum(sum, scratch);
  const float inverse = 1.0f / total;
  for (int d = threadIdx.x; d < head_dim; d += kThreads) {
    float acc = 0.0f;
    for (int key = 0; key < keys; ++key) acc += scores[key] * __half2float(key_row(v0, v1, key)[d]);
    out[batch * batch_q + (static_cast<long long>(token) * heads + head) * head_dim + d] = __float2half(acc * inverse);
  }
}

int launch_attention(const void* q, const void* k0, const void* v0, int keys0, const void* k1, const void* v1,
                     int keys1, void* out, int tokens, int heads, int head_dim, long long kv_stride,
                     long long kv_head_stride, int batches, long long batch_q, long long batch_kv, void* stream) {
  if (q == nullptr || k0 == nullptr || v0 == nullptr || out == nullptr || tokens <= 0 || heads <= 0 ||
      head_dim <= 0 || keys0 < 0 || keys1 < 0 || keys0 + keys1 <= 0 || keys0 + keys1 > 8192 || batches <= 0 ||
      (keys1 > 0 && (k1 == nullptr || v1 == nullptr))) {
    return kInvalid;
  }
  const size_t smem = static_cast<size_t>(keys0 + keys1) * sizeof(float);
  return static_cast<int>(pi05::launch_pdl(
      attention_f16_kernel, dim3(tokens, heads, batches), dim3(kThreads), smem, static_cast<cudaStream_t>(stream),
      static_cast<const __half*>(q), static_cast<const __half*>(k0), static_cast<const __half*>(v0), keys0,
      static_cast<const __half*>(k1), static_cast<const __half*>(v1), keys1, static_cast<__half*>(out), heads,
      head_dim, kv_stride, kv_head_stride, batch_q, batch_kv));
}

// ---- GEMM family -----------------------------------------------------------------------------
// fp32 product [m, n] -> the output contract of one fused form
enum FinishOp { kFinishBias, kFinishBiasGelu, kFinishBiasResidual, kFinishPlain };

template <int OP>
__global__ void finish_kernel(const float* product, const __half* bias, const __half* residual, void* out,
                              long long count, int cols, float inverse_scale) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    float value = product[i];
    if (OP != kFinishPlain && bias != nullptr) value += h(bias, i % cols);
    if (OP == kFinishBiasResidual) value += h(residual, i);
    if (OP == kFinishBiasGelu) {
      static_cast<uint8_t*>(out)[i] = e4m3(gelu_tanh_exact(value) * inverse_scale);
    } else {
      static_cast<__half*>(out)[i] = __float2half_rn(value);
    }
  }
}

__global__ void dequantize_int32_kernel(const int32_t* acc, const float* row_scales, const float* col_scales,
                                        __nv_bfloat16* out, long long count, int cols) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    out[i] = __float2bfloat16(static_cast<float>(acc[i]) * row_scales[i / cols] * col_scales[i % cols]);
  }
}

__global__ void evict_kernel(uint32_t* buffer, size_t words, uint32_t seed) {
  const size_t stride = static_cast<size_t>(blockDim.x) * gridDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride) {
    buffer[i] = buffer[i] * 1664525u + seed + static_cast<uint32_t>(i);
  }
}

// Per-thread set-up state, as the reference keeps it (thread-local plan caches filled by the
// prepare_* entry points, adapters/cublaslt_adapter.cu:128-141): prepared shapes and one fp32
// product buffer per shape for the forms that finish in a second kernel. The execution entry
// points look up only; they never allocate.
struct ShapeKey {
  int m, n, k;
  bool operator==(const ShapeKey& o) const { return m == o.m && n == o.n && k == o.k; }
};
struct ShapeHash {
  size_t operator()(const ShapeKey& s) const {
    return static_cast<size_t>(s.m) * 104729u + static_cast<size_t>(s.n) * 1039u + static_cast<size_t>(s.k) * 31u;
  }
};
thread_local std::unordered_map<ShapeKey, float*, ShapeHash> g_products;  // null = plain form prepared
static __device__ int g_f16_gemm_status;
std::mutex g_status_mutex;
int* g_status_address[64] = {};

int* status_word(bool lookup) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_address[device] == nullptr && lookup) {
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_f16_gemm_status) != cudaSuccess) return nullptr;
    g_status_address[device] = static_cast<int*>(address);
  }
  return g_status_address[device];
}

int prepare_shape(int m, int n, int k, bool with_product) {
  if (m <= 0 || n <= 0 || k <= 0) return kBlasInvalid;
  if (status_word(true) == nullptr) return kBlasNotInitialized;
  auto it = g_products.find(ShapeKey{m, n, k});
  if (it == g_products.end()) it = g_products.emplace(ShapeKey{m, n, k}, nullptr).first;
  if (with_product && it->second == nullptr) {
    float* buffer = nullptr;
    if (cudaMalloc(&buffer, static_cast<size_t>(m) * n * sizeof(float)) != cudaSuccess) return kBlasAllocFailed;
    it->second = buffer;
  }
  return 0;
}

// out (fp32 or f16, row-major [m, n]) = alpha * activation[m, k] (e4m3) . weight[k, n] (e4m3)
int fp8_product(const void* activation, const void* weight, void* out, int out_type, int m, int n, int k,
                float alpha, void* stream) {
  int* status = status_word(false);
  if (status == nullptr) return kBlasNotInitialized;
  pi05::GemmProblem q;
  q.op = pi05::kOpE4m3;
  q.M = m;
  q.N = n;
  q.K = k;
  q.a = pi05::GemmOperand{activation, m, k, 0, 0};
  q.b = pi05::GemmOperand{weight, k, n, 0, 0};  // [k, n] row-major: MN-major B operand
  q.b_mn_major = true;
  q.out = out;
  q.ldc = n;
  q.out_type = out_type;
  q.alpha = alpha;
  q.status = status;
  pi05::GemmPlan plan;
  if (pi05::gemm_plan_build(q, &plan) != pi05::kPi05Ok) return kBlasInvalid;
  return pi05::gemm_plan_launch(plan, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : kBlasExecutionFailed;
}

template <int OP>
int fused_fp8_gemm(const void* activation, const void* weight, const void* bias, const void* residual, void* output,
                   int m, int n, int k, float alpha, float inverse_scale, void* stream) {
  if (activation == nullptr || weight == nullptr || output == nullptr || m <= 0 || n <= 0 || k <= 0) {
    return kBlasInvalid;
  }
  auto it = g_products.find(ShapeKey{m, n, k});
  if (it == g_products.end() || it->second == nullptr) return kBlasNotInitialized;
  const int rc = fp8_product(activation, weight, it->second, pi05::kOutF32, m, n, k, alpha, stream);
  if (rc != 0) return rc;
  const long long count = static_cast<long long>(m) * n;
  const cudaError_t err = pi05::launch_pdl(
      finish_kernel<OP>, dim3(blocks_for(count)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const float*>(it->second), static_cast<const __half*>(bias), static_cast<const __half*>(residual),
      output, count, n, inverse_scale);
  return err == cudaSuccess ? 0 : kBlasExecutionFailed;
}

}  // namespace

// ---- elementwise -----------------------------------------------------------------------------
extern "C" int apxinf_static_quantize_f16_e4m3(const void* input, void* output, int64_t count, float scale,
                                               void* stream) {
  if (!(scale > 0.0f)) return kInvalid;
  return launch_map<kQuantize>(MapArgs{input, nullptr, nullptr, output, count, 1, 0, 1.0f / scale}, stream);
}
extern "C" int apxinf_static_dequantize_e4m3_f16(const void* input, void* output, int64_t count, float scale,
                                                 void* stream) {
  if (!(scale > 0.0f)) return kInvalid;
  return launch_map<kDequantize>(MapArgs{input, nullptr, nullptr, output, count, 1, 0, scale}, stream);
}
extern "C" int apxinf_static_bias_gelu_quant_f16_e4m3(const void* input, const void* bias, void* output, int rows,
                                                      int cols, float scale, void* stream) {
  if (bias == nullptr || rows <= 0 || !(scale > 0.0f)) return kInvalid;
  return launch_map<kBiasGeluQuant>(MapArgs{input, bias, nullptr, output, (long long)rows * cols, cols, 0, 1.0f / scale},
                                    stream);
}
extern "C" int apxinf_static_bias_silu_quant_f16_e4m3(const void* input, const void* bias, void* output, int rows,
                                                      int cols, float scale, void* stream) {
  if (rows <= 0 || !(scale > 0.0f)) return kInvalid;
  return launch_map<kBiasSiluQuant>(MapArgs{input, bias, nullptr, output, (long long)rows * cols, cols, 0, 1.0f / scale},
                                    stream);
}
extern "C" int apxinf_static_bias_silu_f16(const void* input, const void* bias, void* output, int rows, int cols,
                                           void* stream) {
  if (rows <= 0) return kInvalid;
  return launch_map<kBiasSilu>(MapArgs{input, bias, nullptr, output, (long long)rows * cols, cols, 0, 0.0f}, stream);
}
extern "C" int apxinf_static_bias_f16(const void* input, const void* bias, void* output, int rows, int cols,
                                      void* stream) {
  if (rows <= 0) return kInvalid;
  return launch_map<kBias>(MapArgs{input, bias, nullptr, output, (long long)rows * cols, cols, 0, 0.0f}, stream);
}
extern "C" int apxinf_static_concat_rows_f16(const void* first, const void* second, void* output, int first_rows,
                                             int second_rows, int cols, void* stream) {
  if (second == nullptr || first_rows <= 0 || second_rows <= 0) return kInvalid;
  return launch_map<kConcat>(
      MapArgs{first, second, nullptr, output, (long long)(first_rows + second_rows) * cols, cols, first_rows, 0.0f},
      stream);
}
extern "C" int apxinf_static_euler_update_f16(const void* state, const void* velocity, void* output, int64_t count,
                                              float dt, void* stream) {
  if (velocity == nullptr) return kInvalid;
  return launch_map<kEuler>(MapArgs{state, velocity, nullptr, output, count, 1, 0, dt}, stream);
}
extern "C" int apxinf_static_geglu_quant_f16_e4m3(const void* gate_up, void* output, int rows, int inner, float scale,
                                                  void* stream) {
  if (rows <= 0 || !(scale > 0.0f)) return kInvalid;
  return launch_map<kGegluQuant>(MapArgs{gate_up, nullptr, nullptr, output, (long long)rows * inner, inner, 0, 1.0f / scale},
                                 stream);
}
extern "C" int apxinf_static_bias_residual_f16(const void* projection, const void* bias, const void* residual,
                                               void* output, int rows, int cols, void* stream) {
  if (residual == nullptr || rows <= 0) return kInvalid;
  return launch_map<kBiasResidual>(MapArgs{projection, bias, residual, output, (long long)rows * cols, cols, 0, 0.0f},
                                   stream);
}
extern "C" int apxinf_static_ada_gate_residual_f16(const void* projection, const void* residual, const void* style,
                                                   void* output, int rows, int cols, void* stream) {
  if (residual == nullptr || style == nullptr || rows <= 0) return kInvalid;
  return launch_map<kAdaGateResidual>(MapArgs{projection, residual, style, output, (long long)rows * cols, cols, 0, 0.0f},
                                      stream);
}
extern "C" int apxinf_static_bias_position_f16(const void* projection, const void* bias, const void* position,
                                               void* output, int rows, int cols, int tokens_per_view, void* stream) {
  if (position == nullptr || rows <= 0 || tokens_per_view <= 0 || rows % tokens_per_view != 0) return kInvalid;
  return launch_map<kBiasPosition>(
      MapArgs{projection, bias, position, output, (long long)rows * cols, cols, tokens_per_view, 0.0f}, stream);
}
extern "C" int apxinf_static_embedding_f16(const void* table, const void* ids, void* output, int tokens, int width,
                                           int vocab_size, void* stream) {
  if (table == nullptr || ids == nullptr || output == nullptr || tokens <= 0 || width <= 0 || vocab_size <= 0) {
    return kInvalid;
  }
  const long long count = (long long)tokens * width;
  return static_cast<int>(pi05::launch_pdl(embedding_kernel, dim3(blocks_for(count)), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), static_cast<const __half*>(table),
                                           static_cast<const uint32_t*>(ids), static_cast<__half*>(output), count,
                                           width, vocab_size));
}
extern "C" int apxinf_static_rgb_u8_to_patches_e4m3(const void* images, void* patches, int views, int image_size,
                                                    int patch_size, int layout, float scale, void* stream) {
  if (images == nullptr || patches == nullptr || views <= 0 || image_size <= 0 || patch_size <= 0 ||
      image_size % patch_size != 0 || (layout != 0 && layout != 1) || !(scale > 0.0f)) {
    return kInvalid;
  }
  const int side = image_size / patch_size;
  const long long count = (long long)views * side * side * 3 * patch_size * patch_size;
  return static_cast<int>(pi05::launch_pdl(patches_e4m3_kernel, dim3(blocks_for(count)), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), static_cast<const uint8_t*>(images),
                                           static_cast<uint8_t*>(patches), count, image_size, patch_size, layout,
                                           1.0f / scale));
}

// ---- norms -------------------------------------------------------------------------------------
extern "C" int apxinf_static_rms_norm_quant_f16_e4m3(const void* input, const void* weight, void* output, int rows,
                                                     int cols, float eps, float scale, void* stream) {
  if (weight == nullptr || !(scale > 0.0f)) return kInvalid;
  NormArgs16 a{static_cast<const __half*>(input), nullptr, nullptr, static_cast<const __half*>(weight), nullptr,
               nullptr, static_cast<uint8_t*>(output), cols, eps, 1.0f / scale};
  return launch_norm<kRms>(a, rows, stream);
}
extern "C" int apxinf_static_layer_norm_quant_f16_e4m3(const void* input, const void* weight, const void* bias,
                                                       void* output, int rows, int cols, float eps, float scale,
                                                       void* stream) {
  if (weight == nullptr || bias == nullptr || !(scale > 0.0f)) return kInvalid;
  NormArgs16 a{static_cast<const __half*>(input), nullptr, nullptr, static_cast<const __half*>(weight),
               static_cast<const __half*>(bias), nullptr, static_cast<uint8_t*>(output), cols, eps, 1.0f / scale};
  return launch_norm<kLayer>(a, rows, stream);
}
extern "C" int apxinf_static_ada_rms_norm_quant_f16_e4m3(const void* input, const void* style, void* output, int rows,
                                                         int cols, float eps, float scale, void* stream) {
  if (style == nullptr || !(scale > 0.0f)) return kInvalid;
  NormArgs16 a{static_cast<const __half*>(input), nullptr, nullptr, static_cast<const __half*>(style), nullptr,
               nullptr, static_cast<uint8_t*>(output), cols, eps, 1.0f / scale};
  return launch_norm<kAda>(a, rows, stream);
}
extern "C" int apxinf_static_bias_residual_rms_norm_quant_f16_e4m3(const void* projection, const void* bias,
                                                                   const void* residual, const void* weight,
                                                                   void* hidden, void* normalized, int rows, int cols,
                                                                   float eps, float scale, void* stream) {
  if (residual == nullptr || weight == nullptr || hidden == nullptr || !(scale > 0.0f)) return kInvalid;
  NormArgs16 a{static_cast<const __half*>(projection), static_cast<const __half*>(bias),
               static_cast<const __half*>(residual), static_cast<const __half*>(weight), nullptr,
               static_cast<__half*>(hidden), static_cast<uint8_t*>(normalized), cols, eps, 1.0f / scale};
  return launch_norm<kResidualRms>(a, rows, stream);
}
extern "C" int apxinf_static_bias_residual_layer_norm_quant_f16_e4m3(const void* projection,
                                                                     const void* projection_bias, const void* residual,
                                                                     const void* norm_weight, const void* norm_bias,
                                                                     void* hidden, void* normalized, int rows, int cols,
                                                                     float eps, float scale, void* stream) {
  if (residual == nullptr || norm_weight == nullptr || norm_bias == nullptr || hidden == nullptr || !(scale > 0.0f)) {
    return kInvalid;
  }
  NormArgs16 a{static_cast<const __half*>(projection), static_cast<const __half*>(projection_bias),
               static_cast<const __half*>(residual), static_cast<const __half*>(norm_weight),
               static_cast<const __half*>(norm_bias), static_cast<__half*>(hidden),
               static_cast<uint8_t*>(normalized), cols, eps, 1.0f / scale};
  return launch_norm<kResidualLayer>(a, rows, stream);
}
extern "C" int apxinf_static_ada_gate_residual_rms_norm_quant_f16_e4m3(const void* projection, const void* residual,
                                                                       const void* gate_style, const void* norm_style,
                                                                       void* hidden, void* normalized, int rows,
                                                                       int cols, float eps, float scale, void* stream) {
  if (residual == nullptr || gate_style == nullptr || norm_style == nullptr || hidden == nullptr || !(scale > 0.0f)) {
    return kInvalid;
  }
  NormArgs16 a{static_cast<const __half*>(projection), nullptr, static_cast<const __half*>(residual),
               static_cast<const __half*>(gate_style), static_cast<const __half*>(norm_style),
               static_cast<__half*>(hidden), static_cast<uint8_t*>(normalized), cols, eps, 1.0f / scale};
  return launch_norm<kAdaGateRms>(a, rows, stream);
}

// ---- q | k | v ---------------------------------------------------------------------------------
extern "C" int apxinf_static_qkv_rope_f16(const void* qkv, const void* bias, void* q, void* k, void* v, int tokens,
                                          int q_heads, int kv_heads, int head_dim, float theta, int position_offset,
                                          int kv_output_offset, void* stream) {
  if (qkv == nullptr || q == nullptr || k == nullptr || v == nullptr || tokens <= 0 || q_heads <= 0 ||
      kv_heads <= 0 || head_dim <= 0 || head_dim % 2 != 0 || position_offset < 0 || kv_output_offset < 0) {
    return kInvalid;
  }
  return static_cast<int>(pi05::launch_pdl(
      qkv_rope_kernel, dim3(tokens, q_heads + 2 * kv_heads), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __half*>(qkv), static_cast<const __half*>(bias), static_cast<__half*>(q),
      static_cast<__half*>(k), static_cast<__half*>(v), q_heads, kv_heads, head_dim, theta, position_offset,
      kv_output_offset));
}
extern "C" int apxinf_static_qkv_split_bias_f16(const void* qkv, const void* bias, void* q, void* k, void* v,
                                                int tokens, int projection_width, void* stream) {
  if (qkv == nullptr || q == nullptr || k == nullptr || v == nullptr || tokens <= 0 || projection_width <= 0) {
    return kInvalid;
  }
  return static_cast<int>(pi05::launch_pdl(qkv_split_kernel, dim3(tokens), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), static_cast<const __half*>(qkv),
                                           static_cast<const __half*>(bias), static_cast<__half*>(q),
                                           static_cast<__half*>(k), static_cast<__half*>(v), projection_width));
}

// ---- attention ---------------------------------------------------------------------------------
extern "C" int apxinf_static_mqa_flash_f16(const void* q, const void* prefix_k, const void* prefix_v,
                                           const void* suffix_k, const void* suffix_v, void* output,
                                           int suffix_tokens, int heads, int head_dim, int prefix_tokens,
                                           void* stream) {
  return launch_attention(q, prefix_k, prefix_v, prefix_tokens, suffix_k, suffix_v, suffix_tokens, output,
                          suffix_tokens, heads, head_dim, head_dim, 0, 1, 0, 0, stream);
}
extern "C" int apxinf_static_mha_flash_f16(const void* q, const void* k, const void* v, void* output,
                                           int tokens_per_batch, int batches, int heads, int head_dim, void* stream) {
  const long long batch = (long long)tokens_per_batch * heads * head_dim;
  return launch_attention(q, k, v, tokens_per_batch, nullptr, nullptr, 0, output, tokens_per_batch, heads, head_dim,
                          (long long)heads * head_dim, head_dim, batches, batch, batch, stream);
}
extern "C" int apxinf_static_cublas_mqa_f16(const void* q, const void* k, const void* v, void* output,
                                            int query_tokens, int key_tokens, int heads, int head_dim, void* stream) {
  const int rc = launch_attention(q, k, v, key_tokens, nullptr, nullptr, 0, output, query_tokens, heads, head_dim,
                                  head_dim, 0, 1, 0, 0, stream);
  return rc == 0 ? 0 : rc == kInvalid ? kBlasInvalid : kBlasExecutionFailed;
}

// ---- GEMMs -------------------------------------------------------------------------------------
extern "C" int apxinf_static_native_fp8_supported(int device, int* supported) {
  if (device < 0 || supported == nullptr) return kInvalid;
  int major = 0;
  const cudaError_t err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (err != cudaSuccess) return static_cast<int>(err);
  *supported = major >= 10 ? 1 : 0;  // this library is sm_100a code
  return 0;
}
extern "C" int apxinf_static_prepare_fp8_gemm_f16(int m, int n, int k) { return prepare_shape(m, n, k, false); }
extern "C" int apxinf_static_prepare_fp8_gemm_bias_f16(const void* bias, int m, int n, int k) {
  if (bias == nullptr) return kBlasInvalid;
  return prepare_shape(m, n, k, true);
}
extern "C" int apxinf_static_prepare_fp8_gemm_bias_gelu_e4m3(const void* bias, int m, int n, int k,
                                                             float output_scale) {
  if (bias == nullptr || !(output_scale > 0.0f)) return kBlasInvalid;
  return prepare_shape(m, n, k, true);
}
extern "C" int apxinf_static_prepare_fp8_gemm_bias_residual_f16(const void* bias, int m, int n, int k) {
  (void)bias;  // may be null: residual only
  return prepare_shape(m, n, k, true);
}
extern "C" int apxinf_static_fp8_gemm_f16(const void* activation, const void* weight, void* output, int m, int n,
                                          int k, float alpha, void* stream) {
  if (activation == nullptr || weight == nullptr || output == nullptr || m <= 0 || n <= 0 || k <= 0) {
    return kBlasInvalid;
  }
  if (g_products.find(ShapeKey{m, n, k}) == g_products.end()) return kBlasNotInitialized;
  return fp8_product(activation, weight, output, pi05::kOutF16, m, n, k, alpha, stream);
}
extern "C" int apxinf_static_fp8_gemm_bias_f16(const void* activation, const void* weight, const void* bias,
                                               void* output, int m, int n, int k, float alpha, void* stream) {
  if (bias == nullptr) return kBlasInvalid;
  return fused_fp8_gemm<kFinishBias>(activation, weight, bias, nullptr, output, m, n, k, alpha, 1.0f, stream);
}
extern "C" int apxinf_static_fp8_gemm_bias_gelu_e4m3(const void* activation, const void* weight, const void* bias,
                                                     void* output, int m, int n, int k, float alpha,
                                                     float output_scale, void* stream) {
  if (bias == nullptr || !(output_scale > 0.0f)) return kBlasInvalid;
  return fused_fp8_gemm<kFinishBiasGelu>(activation, weight, bias, nullptr, output, m, n, k, alpha,
                                         1.0f / output_scale, stream);
}
extern "C" int apxinf_static_fp8_gemm_bias_residual_f16(const void* activation, const void* weight, const void* bias,
                                                        const void* residual, void* output, int m, int n, int k,
                                                        float alpha, void* stream) {
  if (residual == nullptr) return kBlasInvalid;
  return fused_fp8_gemm<kFinishBiasResidual>(activation, weight, bias, residual, output, m, n, k, alpha, 1.0f, stream);
}
/* ffi/cutlass.rs:85 — the CUTLASS FP8 GEMM name; `tactic` selects among the reference's tile
 * shapes and has no meaning here: 0..7 are accepted, others are -5 as there. Needs no prepare. */
extern "C" int apxinf_static_cutlass_fp8_gemm_f16(const void* activation, const void* weight, void* output, int m,
                                                  int n, int k, float alpha, int tactic, void* stream) {
  if (activation == nullptr || weight == nullptr || output == nullptr || m <= 0 || n <= 0 || k <= 0) return -6;
  if (tactic < 0 || tactic > 7) return -5;
  if (status_word(true) == nullptr) return -2;
  const int rc = fp8_product(activation, weight, output, pi05::kOutF16, m, n, k, alpha, stream);
  return rc == 0 ? 0 : rc == kBlasInvalid ? -1 : -3;
}
/* adapters/cutlass_w8a8_adapter.cu:6-13 — int8 [m, k] x int8 [n, k] (output-major weight) with
 * per-row and per-column f32 scales -> bf16 [m, n], int32 accumulation. */
extern "C" int apxinf_static_cutlass_int8_gemm_bf16(const void* activation, const void* weight_output_major,
                                                    const void* row_scales, const void* column_scales, void* output,
                                                    int m, int n, int k, void* stream) {
  if (activation == nullptr || weight_output_major == nullptr || row_scales == nullptr || column_scales == nullptr ||
      output == nullptr || m <= 0 || n <= 0 || k <= 0) {
    return kInvalid;
  }
  int* status = status_word(true);
  if (status == nullptr) return static_cast<int>(cudaErrorInitializationError);
  pi05::GemmProblem q;
  q.op = pi05::kOpS8;
  q.M = m;
  q.N = n;
  q.K = k;
  q.a = pi05::GemmOperand{activation, m, k, 0, 0};
  q.b = pi05::GemmOperand{weight_output_major, n, k, 0, 0};
  q.out = output;
  q.ldc = n;
  q.row_scale = static_cast<const float*>(row_scales);
  q.col_scale = static_cast<const float*>(column_scales);
  q.status = status;
  pi05::GemmPlan plan;
  if (pi05::gemm_plan_build(q, &plan) != pi05::kPi05Ok) return kInvalid;
  return static_cast<int>(pi05::gemm_plan_launch(plan, static_cast<cudaStream_t>(stream)));
}
extern "C" int apxinf_static_dequantize_int32_bf16(const void* accumulators, const void* row_scales,
                                                   const void* column_scales, void* output, int rows, int cols,
                                                   void* stream) {
  if (accumulators == nullptr || row_scales == nullptr || column_scales == nullptr || output == nullptr ||
      rows <= 0 || cols <= 0) {
    return kInvalid;
  }
  const long long count = (long long)rows * cols;
  return static_cast<int>(pi05::launch_pdl(
      dequantize_int32_kernel, dim3(blocks_for(count)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const int32_t*>(accumulators), static_cast<const float*>(row_scales),
      static_cast<const float*>(column_scales), static_cast<__nv_bfloat16*>(output), count, cols));
}
/* adapters/custom_kernels.cu:47-60 — tuning aid: rewrites `bytes` of `buffer` so that it
 * displaces whatever the L2 held. */
extern "C" int apxinf_static_evict_l2(void* buffer, size_t bytes, uint32_t seed, void* stream) {
  if (buffer == nullptr || bytes < sizeof(uint32_t)) return kInvalid;
  const size_t words = bytes / sizeof(uint32_t);
  evict_kernel<<<blocks_for(static_cast<long long>(words)), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint32_t*>(buffer), words, seed);
  return static_cast<int>(cudaGetLastError());
}
