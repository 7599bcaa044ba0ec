// The remaining BF16 row / elementwise operators of the reference's static path under their
// own symbol names (include/pi05_apxinf_static.h; contracts of
// crates/apxinf-cuda/adapters/static_bf16_adapter.cu). The PI0.5 engine of this library does
// not launch them: it performs the same arithmetic inside the GEMM epilogues and the fused
// row kernels. They exist so that a host that binds these names one by one finds all of them;
// each is checked against the reference's compiled kernel in tests/test_ref_ops_gpu.py.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pi05_apxinf_static.h"
#include "launch.cuh"

namespace {

constexpr int kInvalid = static_cast<int>(cudaErrorInvalidValue);
constexpr int kThreads = 256;

__device__ __forceinline__ float f(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ float gelu_tanh_exact(float x) {
  // crates/apxinf-cuda/kernels/custom/math.cuh:8-12
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

unsigned blocks_for(long long count) {
  const long long blocks = (count + kThreads - 1) / kThreads;
  return static_cast<unsigned>(blocks < 1 ? 1 : blocks > 148 * 16 ? 148 * 16 : blocks);
}

// One grid-stride elementwise kernel; OP selects the formula.
enum MapOp { kBiasActivation, kGeglu, kBiasResidual, kAdaGateResidual, kBiasPosition };

struct MapArgs {
  const __nv_bfloat16* a;  // input / projection / gate_up
  const __nv_bfloat16* b;  // bias (may be null)
  const __nv_bfloat16* c;  // residual / style / position table
  __nv_bfloat16* out;
  long long count;
  int cols;
  int extra;  // activation | inner | tokens_per_view
};

template <int OP>
__global__ void map_kernel(MapArgs m) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < m.count; i += stride) {
    const int col = static_cast<int>(i % m.cols);
    float value;
    if (OP == kBiasActivation) {
      value = f(m.a, i);
      if (m.b != nullptr) value += f(m.b, col);
      if (m.extra == 1) value = gelu_tanh_exact(value);
      if (m.extra == 2) value = value / (1.0f + expf(-value));
    } else if (OP == kGeglu) {
      // cols = inner: out[row, col] = gelu(gate_up[row, col]) * gate_up[row, inner + col]
      const long long row = i / m.cols;
      const __nv_bfloat16* in = m.a + row * 2 * m.cols;
      value = gelu_tanh_exact(f(in, col)) * f(in, m.cols + col);
    } else if (OP == kBiasResidual) {
      value = f(m.a, i) + f(m.c, i);
      if (m.b != nullptr) value += f(m.b, col);
    } else if (OP == kAdaGateResidual) {
      value = f(m.b, i) + f(m.a, i) * f(m.c, 2LL * m.cols + col);  // b = residual, c = style
    } else {
      const int token = static_cast<int>((i / m.cols) % m.extra);
      value = f(m.a, i) + f(m.c, static_cast<long long>(token) * m.cols + col);
      if (m.b != nullptr) value += f(m.b, col);
    }
    m.out[i] = __float2bfloat16(value);
  }
}

template <int OP>
int launch_map(const MapArgs& m, void* stream) {
  if (m.a == nullptr || m.out == nullptr || m.count <= 0 || m.cols <= 0) return kInvalid;
  return static_cast<int>(pi05::launch_pdl(map_kernel<OP>, dim3(blocks_for(m.count)), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), m));
}

// ---- fused "new hidden state, then its norm" row kernels: one CTA per row -------------------

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

enum NormOp { kResidualRms, kResidualLayer, kAdaGateRms };

struct FusedNormArgs {
  const __nv_bfloat16* projection;
  const __nv_bfloat16* bias;      // projection bias (may be null)
  const __nv_bfloat16* residual;
  const __nv_bfloat16* weight;    // norm weight | gate style (kAdaGateRms)
  const __nv_bfloat16* norm_bias; // layer-norm bias | norm style (kAdaGateRms)
  __nv_bfloat16* hidden;
  __nv_bfloat16* normalized;
  int cols;
  float eps;
};

template <int OP>
__global__ void __launch_bounds__(kThreads) fused_norm_kernel(FusedNormArgs a) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  __shared__ float scratch[kThreads / 32];
  const long long base = static_cast<long long>(blockIdx.x) * a.cols;
  // pass 1: the new hidden state, rounded to bf16 as it is stored, and its sum (of squares)
  float acc = 0.0f;
  for (int col = threadIdx.x; col < a.cols; col += kThreads) {
    float value;
    if (OP == kAdaGateRms) {
      value = f(a.residual, base + col) + f(a.projection, base + col) * f(a.weight, 2LL * a.cols + col);
    } else {
      value = f(a.projection, base + col) + f(a.residual, base + col);
      if (a.bias != nullptr) value += f(a.bias, col);
    }
    const __nv_bfloat16 rounded = __float2bfloat16(value);
    a.hidden[base + col] = rounded;
    const float h = __bfloat162float(rounded);
    acc += OP == kResidualLayer ? h : h * h;
  }
  const float first = block_sum(acc, scratch) / a.cols;
  if (OP == kResidualLayer) {
    const float mean = first;
    float var = 0.0f;
    for (int col = threadIdx.x; col < a.cols; col += kThreads) {
      const float centered = f(a.hidden, base + col) - mean;  // this thread's own stores
      var += centered * centered;
    }
    const float inverse_std = rsqrtf(block_sum(var, scratch) / a.cols + a.eps);
    for (int col = threadIdx.x; col < a.cols; col += kThreads) {
      a.normalized[base + col] = __float2bfloat16(
          (f(a.hidden, base + col) - mean) * inverse_std * f(a.weight, col) + f(a.norm_bias, col));
    }
    return;
  }
  const float inverse_rms = rsqrtf(first + a.eps);
  for (int col = threadIdx.x; col < a.cols; col += kThreads) {
    const float value = f(a.hidden, base + col) * inverse_rms;
    a.normalized[base + col] = __float2bfloat16(
        OP == kAdaGateRms ? value * (1.0f + f(a.norm_bias, col)) + f(a.norm_bias, a.cols + col)
                          : value * f(a.weight, col));
  }
}

template <int OP>
int launch_fused_norm(const FusedNormArgs& a, int rows, void* stream) {
  if (a.projection == nullptr || a.residual == nullptr || a.weight == nullptr || a.hidden == nullptr ||
      a.normalized == nullptr || rows <= 0 || a.cols <= 0 ||
      (OP != kResidualRms && a.norm_bias == nullptr)) {
    return kInvalid;
  }
  return static_cast<int>(pi05::launch_pdl(fused_norm_kernel<OP>, dim3(rows), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), a));
}

// ---- q|k|v split with bias, with and without rotary embedding --------------------------------

struct SplitArgs {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* bias;  // may be null
  __nv_bfloat16 *q, *k, *v;
  int tokens, q_heads, kv_heads, head_dim;
  float theta;
  int position_offset, kv_output_offset;
};

// One thread per (token, projection head, rotary pair): q and k rotate-half pairs
// (d, d + head_dim/2) by position * theta^(-d / (head_dim/2)); v is copied. k and v rows land
// at kv_output_offset + token (their place in a cache).
__global__ void qkv_rope_kernel(SplitArgs s) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const int half = s.head_dim >> 1;
  const int heads = s.q_heads + 2 * s.kv_heads;
  const long long total = static_cast<long long>(s.tokens) * heads * half;
  const int q_width = s.q_heads * s.head_dim, kv_width = s.kv_heads * s.head_dim;
  const int fused = q_width + 2 * kv_width;
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int pair = static_cast<int>(i % half);
    const int head = static_cast<int>((i / half) % heads);
    const int token = static_cast<int>(i / (static_cast<long long>(half) * heads));
    const int column = head * s.head_dim;  // heads are laid out q..., k..., v... in the projection
    float first = f(s.qkv, static_cast<long long>(token) * fused + column + pair);
    float second = f(s.qkv, static_cast<long long>(token) * fused + column + half + pair);
    if (s.bias != nullptr) {
      first += f(s.bias, column + pair);
      second += f(s.bias, column + half + pair);
    }
    __nv_bfloat16* dst;
    bool rotate = true;
    if (head < s.q_heads) {
      dst = s.q + (static_cast<long long>(token) * s.q_heads + head) * s.head_dim;
    } else if (head < s.q_heads + s.kv_heads) {
      dst = s.k + (static_cast<long long>(s.kv_output_offset + token) * s.kv_heads + (head - s.q_heads)) * s.head_dim;
    } else {
      dst = s.v + (static_cast<long long>(s.kv_output_offset + token) * s.kv_heads + (head - s.q_heads - s.kv_heads)) * s.head_dim;
      rotate = false;
    }
    if (rotate) {
      const float frequency = powf(s.theta, -static_cast<float>(pair) / half);
      float sine, cosine;
      sincosf((s.position_offset + token) * frequency, &sine, &cosine);
      dst[pair] = __float2bfloat16(first * cosine - second * sine);
      dst[half + pair] = __float2bfloat16(second * cosine + first * sine);
    } else {
      dst[pair] = __float2bfloat16(first);
      dst[half + pair] = __float2bfloat16(second);
    }
  }
}

// projection [tokens, 3 * width] + bias -> q, k, v [tokens, width] each.
__global__ void qkv_split_kernel(SplitArgs s) {
  pi05::pdl_launch_dependents();
  pi05::pdl_wait();
  const int width = s.head_dim;  // reused field: projection width
  const long long total = static_cast<long long>(s.tokens) * 3 * width;
  const long long stride = static_cast<long long>(blockDim.x) * gridDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int col = static_cast<int>(i % (3 * width));
    const long long token = i / (3 * width);
    float value = f(s.qkv, i);
    if (s.bias != nullptr) value += f(s.bias, col);
    __nv_bfloat16* dst = col < width ? s.q : col < 2 * width ? s.k : s.v;
    dst[token * width + col % width] = __float2bfloat16(value);
  }
}

}  // namespace

extern "C" int apxinf_static_bias_activation_bf16(const void* input, const void* bias, void* output,
                                                  int rows, int cols, int activation, void* stream) {
  if (activation < 0 || activation > 2 || rows <= 0) return kInvalid;
  MapArgs m{static_cast<const __nv_bfloat16*>(input), static_cast<const __nv_bfloat16*>(bias), nullptr,
            static_cast<__nv_bfloat16*>(output), static_cast<long long>(rows) * cols, cols, activation};
  return launch_map<kBiasActivation>(m, stream);
}

extern "C" int apxinf_static_concat_rows_bf16(const void* first, const void* second, void* output,
                                              int first_rows, int second_rows, int cols, void* stream) {
  if (first == nullptr || second == nullptr || output == nullptr || first_rows < 0 || second_rows < 0 ||
      cols <= 0) {
    return kInvalid;
  }
  const size_t first_bytes = static_cast<size_t>(first_rows) * cols * 2;
  const size_t second_bytes = static_cast<size_t>(second_rows) * cols * 2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaSuccess;
  if (first_bytes > 0) err = cudaMemcpyAsync(output, first, first_bytes, cudaMemcpyDeviceToDevice, s);
  if (err == cudaSuccess && second_bytes > 0) {
    err = cudaMemcpyAsync(static_cast<uint8_t*>(output) + first_bytes, second, second_bytes,
                          cudaMemcpyDeviceToDevice, s);
  }
  return static_cast<int>(err);
}

extern "C" int apxinf_static_geglu_bf16(const void* gate_up, void* output, int rows, int inner, void* stream) {
  if (rows <= 0) return kInvalid;
  MapArgs m{static_cast<const __nv_bfloat16*>(gate_up), nullptr, nullptr, static_cast<__nv_bfloat16*>(output),
            static_cast<long long>(rows) * inner, inner, 0};
  return launch_map<kGeglu>(m, stream);
}

extern "C" int apxinf_static_bias_residual_bf16(const void* projection, const void* bias, const void* residual,
                                                void* output, int rows, int cols, void* stream) {
  if (residual == nullptr || rows <= 0) return kInvalid;
  MapArgs m{static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(bias),
            static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(output),
            static_cast<long long>(rows) * cols, cols, 0};
  return launch_map<kBiasResidual>(m, stream);
}

extern "C" int apxinf_static_ada_gate_residual_bf16(const void* projection, const void* residual,
                                                    const void* style, void* output, int rows, int cols,
                                                    void* stream) {
  if (residual == nullptr || style == nullptr || rows <= 0) return kInvalid;
  MapArgs m{static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(residual),
            static_cast<const __nv_bfloat16*>(style), static_cast<__nv_bfloat16*>(output),
            static_cast<long long>(rows) * cols, cols, 0};
  return launch_map<kAdaGateResidual>(m, stream);
}

extern "C" int apxinf_static_bias_position_bf16(const void* projection, const void* bias, const void* position,
                                                void* output, int rows, int cols, int tokens_per_view,
                                                void* stream) {
  if (position == nullptr || rows <= 0 || tokens_per_view <= 0) return kInvalid;
  MapArgs m{static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(bias),
            static_cast<const __nv_bfloat16*>(position), static_cast<__nv_bfloat16*>(output),
            static_cast<long long>(rows) * cols, cols, tokens_per_view};
  return launch_map<kBiasPosition>(m, stream);
}

extern "C" int apxinf_static_bias_residual_rms_norm_bf16(const void* projection, const void* bias,
                                                         const void* residual, const void* weight, void* hidden,
                                                         void* normalized, int rows, int cols, float eps,
                                                         void* stream) {
  FusedNormArgs a{static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(bias),
                  static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight), nullptr,
                  static_cast<__nv_bfloat16*>(hidden), static_cast<__nv_bfloat16*>(normalized), cols, eps};
  return launch_fused_norm<kResidualRms>(a, rows, stream);
}

extern "C" int apxinf_static_bias_residual_layer_norm_bf16(const void* projection, const void* projection_bias,
                                                           const void* residual, const void* norm_weight,
                                                           const void* norm_bias, void* hidden, void* normalized,
                                                           int rows, int cols, float eps, void* stream) {
  FusedNormArgs a{static_cast<const __nv_bfloat16*>(projection), static_cast<const __nv_bfloat16*>(projection_bias),
                  static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(norm_weight),
                  static_cast<const __nv_bfloat16*>(norm_bias), static_cast<__nv_bfloat16*>(hidden),
                  static_cast<__nv_bfloat16*>(normalized), cols, eps};
  return launch_fused_norm<kResidualLayer>(a, rows, stream);
}

extern "C" int apxinf_static_ada_gate_residual_rms_norm_bf16(const void* projection, const void* residual,
                                                             const void* gate_style, const void* norm_style,
                                                             void* hidden, void* normalized, int rows, int cols,
                                                             float eps, void* stream) {
  FusedNormArgs a{static_cast<const __nv_bfloat16*>(projection), nullptr, static_cast<const __nv_bfloat16*>(residual),
                  static_cast<const __nv_bfloat16*>(gate_style), static_cast<const __nv_bfloat16*>(norm_style),
                  static_cast<__nv_bfloat16*>(hidden), static_cast<__nv_bfloat16*>(normalized), cols, eps};
  return launch_fused_norm<kAdaGateRms>(a, rows, stream);
}

extern "C" int apxinf_static_qkv_rope_bf16(const void* qkv, const void* bias, void* q, void* k, void* v,
                                           int tokens, int q_heads, int kv_heads, int head_dim, float theta,
                                           int position_offset, int kv_output_offset, void* stream) {
  if (qkv == nullptr || q == nullptr || k == nullptr || v == nullptr || tokens <= 0 || q_heads <= 0 ||
      kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) != 0 || !(theta > 0.0f) || position_offset < 0 ||
      kv_output_offset < 0) {
    return kInvalid;
  }
  SplitArgs s{static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(bias),
              static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
              tokens, q_heads, kv_heads, head_dim, theta, position_offset, kv_output_offset};
  const long long total = static_cast<long long>(tokens) * (q_heads + 2 * kv_heads) * (head_dim / 2);
  return static_cast<int>(pi05::launch_pdl(qkv_rope_kernel, dim3(blocks_for(total)), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), s));
}

extern "C" int apxinf_static_qkv_split_bias_bf16(const void* qkv, const void* bias, void* q, void* k, void* v,
                                                 int tokens, int projection_width, void* stream) {
  if (qkv == nullptr || q == nullptr || k == nullptr || v == nullptr || tokens <= 0 || projection_width <= 0) {
    return kInvalid;
  }
  SplitArgs s{static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(bias),
              static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v),
              tokens, 0, 0, projection_width, 0.0f, 0, 0};
  const long long total = static_cast<long long>(tokens) * 3 * projection_width;
  return static_cast<int>(pi05::launch_pdl(qkv_split_kernel, dim3(blocks_for(total)), dim3(kThreads), 0,
                                           static_cast<cudaStream_t>(stream), s));
}
