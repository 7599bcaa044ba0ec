#include "engine.h"

#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstring>

#include "row_kernels.cuh"
#include "weights.cuh"

namespace pi05 {

#define PI05_CUDA(expr)                                  \
  do {                                                   \
    const cudaError_t pi05_err_ = (expr);                \
    if (pi05_err_ != cudaSuccess) return record_cuda(pi05_err_); \
  } while (0)

#define PI05_TRY(expr)                     \
  do {                                     \
    const int pi05_rc_ = (expr);           \
    if (pi05_rc_ != kPi05Ok) return pi05_rc_; \
  } while (0)

namespace {

constexpr size_t kSplitScratchBytes = 32u << 20;  // split-K partial tiles
constexpr int kSplitMaxTiles = 4096;

uint16_t bf16_bits(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((bits >> 16) | 0x40u);
  const uint32_t rounding = ((bits >> 16) & 1u) + 0x7fffu;
  return static_cast<uint16_t>((bits + rounding) >> 16);
}

float bf16_to_float(uint16_t bits) {
  const uint32_t wide = static_cast<uint32_t>(bits) << 16;
  float value;
  std::memcpy(&value, &wide, 4);
  return value;
}

int elem_size(int prec) { return prec == kPrecBf16 ? 2 : 1; }
int op_of(int prec) { return prec == kPrecBf16 ? kOpBf16 : prec == kPrecFp8 ? kOpE4m3 : kOpS8; }
long long round_up(long long v, long long m) { return (v + m - 1) / m * m; }

}  // namespace

namespace {
cudaError_t launch_op(const Op& op, cudaStream_t stream) {
  if (op.is_gemm) return gemm_plan_launch(op.plan, stream);
  if (op.is_fmha) return fmha_plan_launch(op.fmha, stream);
  return op.launch(stream);
}
}  // namespace

int ModelConfig::validate() const {
  const bool ok =
      action_dim > 0 && action_dim % 8 == 0 && action_horizon > 0 && action_horizon <= 64 &&
      num_flow_steps > 0 && num_views > 0 && image_size > 0 && patch_size > 0 &&
      image_size % patch_size == 0 && vision_width == vision_heads * vision_head_dim &&
      vision_width % 16 == 0 && vision_head_dim % 8 == 0 && vision_mlp_dim % 16 == 0 &&
      vocab_size > 0 && language.width % 16 == 0 && action.width % 16 == 0 &&
      language.mlp_dim % 64 == 0 && action.mlp_dim % 64 == 0 && language.num_kv_heads == 1 &&
      action.num_kv_heads == 1 && language.head_dim == action.head_dim &&
      language.num_heads == action.num_heads && language.depth == action.depth &&
      language.head_dim % 16 == 0 && max_token_len > 0 &&
      num_views * patches_per_view() + max_token_len + action_horizon <= 1024 &&
      patches_per_view() % 8 == 0;
  return ok ? kPi05Ok : kPi05ErrInvalidValue;
}

// ---------------------------------------------------------------------------
// Engine: weights
// ---------------------------------------------------------------------------

namespace {
// Timing events of one call: created on demand, destroyed on every way out.
struct EventSet {
  std::vector<cudaEvent_t> all;
  ~EventSet() {
    for (cudaEvent_t e : all) cudaEventDestroy(e);
  }
  int add(cudaEvent_t* out) {
    const cudaError_t err = cudaEventCreate(out);
    if (err != cudaSuccess) return record_cuda(err);
    all.push_back(*out);
    return kPi05Ok;
  }
};
}  // namespace

Engine::Engine(const ModelConfig& cfg, const EngineOptions& options)
    : cfg_(cfg), prec_(options.precision), device_(options.device), seed_(options.seed),
      act_scale_(options.act_scale), weight_dist_(options.weight_dist),
      int8_static_(options.int8_activations == kInt8Static) {}

namespace {
constexpr long long kConvertChunk = 32ll << 20;  // elements per staged chunk of a converted host tensor
}

// The next tensor, as bf16 (or as f32 when as_f32): from the host table when one was given, else
// the next `count` values of the synthetic stream (bf16 only).
int Engine::fetch(const std::string& name, void* dst, long long count, bool as_f32) {
  if (from_host_) {
    auto it = host_tensors_.find(name);
    if (it == host_tensors_.end() || it->second.data == nullptr ||
        it->second.elements != static_cast<size_t>(count)) {
      missing_tensor_ = name;
      return kPi05ErrInvalidValue;
    }
    const HostTensor& t = it->second;
    const size_t src_size = t.f32 ? 4 : 2, dst_size = as_f32 ? 4 : 2;
    if (t.f32 == as_f32) {
      PI05_CUDA(cudaMemcpyAsync(dst, t.data, static_cast<size_t>(count) * src_size,
                                cudaMemcpyHostToDevice, stream_));
    } else {
      for (long long done = 0; done < count; done += kConvertChunk) {
        const long long n = std::min(kConvertChunk, count - done);
        PI05_CUDA(cudaMemcpyAsync(tmp_convert_, static_cast<const char*>(t.data) + done * src_size,
                                  static_cast<size_t>(n) * src_size, cudaMemcpyHostToDevice, stream_));
        PI05_CUDA(launch_convert(tmp_convert_, static_cast<char*>(dst) + done * dst_size, n,
                                 as_f32 ? 1 : 0, stream_));
        PI05_CUDA(cudaStreamSynchronize(stream_));
      }
    }
    // the destination may be reused by the next tensor; pageable host memory is consumed at once
    PI05_CUDA(cudaStreamSynchronize(stream_));
    return kPi05Ok;
  }
  if (as_f32) return kPi05ErrInvalidValue;
  const cudaError_t err = weight_dist_ == kWeightsNormal
                              ? launch_normal_fill(dst, seed_, cursor_, count, stream_)
                              : launch_lcg_fill(dst, seed_, cursor_, count, stream_);
  cursor_ += static_cast<uint64_t>(count);
  return record_cuda(err);
}

int Engine::fetch_layer_norm(const std::string& prefix, int width, LayerNormParams* out) {
  if (!from_host_ || host_tensors_.find(prefix + ".weight") == host_tensors_.end()) return kPi05Ok;
  out->weight = dmalloc(static_cast<size_t>(width) * 2);
  out->bias = dmalloc(static_cast<size_t>(width) * 2);
  if (out->weight == nullptr || out->bias == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  PI05_TRY(fetch(prefix + ".weight", out->weight, width));
  PI05_TRY(fetch(prefix + ".bias", out->bias, width));
  return kPi05Ok;
}

float Engine::scale_of(const std::string& site) const {
  auto it = site_scales_.find(site);
  return it == site_scales_.end() ? act_scale_ : it->second;
}

int Engine::set_scale(const std::string& site, float value) {
  auto it = site_scales_.find(site);
  if (it == site_scales_.end() || !(value > 0.0f) || !std::isfinite(value)) return kPi05ErrInvalidValue;
  it->second = value;
  return kPi05Ok;
}

Engine::~Engine() {
  cudaSetDevice(device_);
  if (stream_ != nullptr) cudaStreamSynchronize(stream_);
  for (void* p : allocations_) cudaFree(p);
  if (stream_ != nullptr) cudaStreamDestroy(stream_);
}

void* Engine::dmalloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, std::max<size_t>(bytes, 256)) != cudaSuccess) return nullptr;
  allocations_.push_back(p);
  weight_bytes_ += bytes;
  return p;
}

void Engine::release(void* p) {
  if (p == nullptr) return;
  auto it = std::find(allocations_.begin(), allocations_.end(), p);
  if (it != allocations_.end()) allocations_.erase(it);
  cudaFree(p);
}

int Engine::make_linear(const std::string& prefix, const std::vector<std::string>& parts, int k,
                        const std::vector<int>& ns, bool bias, bool interleave, Linear* out) {
  int n_total = 0;
  for (int n : ns) n_total += n;
  const int es = elem_size(prec_);
  const long long ldk = round_up(k, 16);
  out->n = n_total;
  out->k = k;
  out->ldk = ldk;
  out->w = dmalloc(static_cast<size_t>(n_total) * ldk * es);
  if (out->w == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  if (bias) {
    out->bias = dmalloc(static_cast<size_t>(n_total) * 2);
    if (out->bias == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  }
  const bool wide = wide_staging();
  const size_t stage_elem = wide ? 4 : 2;
  void* stage = prec_ == kPrecBf16 ? out->w : tmp_stage_;
  const size_t stage_bytes = static_cast<size_t>(n_total) * ldk * stage_elem;
  if (prec_ != kPrecBf16 && stage_bytes > tmp_stage_bytes_) return kPi05ErrInvalidValue;
  PI05_CUDA(cudaMemsetAsync(stage, 0, stage_bytes, stream_));
  int row_offset = 0;
  for (size_t i = 0; i < parts.size(); ++i) {
    const long long count = static_cast<long long>(k) * ns[i];
    if (static_cast<size_t>(count) * stage_elem > tmp_src_bytes_) return kPi05ErrInvalidValue;
    // part "w": the projection is its own tensor (prefix); else a sibling of the packed name
    const std::string base = parts[i] == "w" ? prefix : prefix.substr(0, prefix.rfind('.') + 1) + parts[i];
    PI05_TRY(fetch(base + ".weight", tmp_src_, count, wide));
    PI05_CUDA(launch_transpose_pack(tmp_src_, stage, k, ns[i], ldk, row_offset,
                                    interleave ? 1 : 0, static_cast<int>(i), stream_, wide ? 1 : 0));
    if (bias) {
      PI05_TRY(fetch(base + ".bias", static_cast<uint16_t*>(out->bias) + row_offset, ns[i]));
    }
    row_offset += ns[i];
  }
  if (prec_ != kPrecBf16) {
    out->col_scale = static_cast<float*>(dmalloc(static_cast<size_t>(n_total) * 4));
    if (out->col_scale == nullptr) return record_cuda(cudaErrorMemoryAllocation);
    PI05_CUDA(launch_quantize_weight_rows(stage, out->w, out->col_scale, n_total, k, ldk,
                                          prec_ == kPrecInt8 ? 1 : 0, stream_, wide ? 1 : 0));
  }
  named_[prefix + ".weight"] = {out->w, static_cast<size_t>(n_total) * ldk * es};
  if (out->col_scale != nullptr) named_[prefix + ".scale"] = {out->col_scale, (size_t)n_total * 4};
  if (out->bias != nullptr) named_[prefix + ".bias"] = {out->bias, (size_t)n_total * 2};
  return kPi05Ok;
}

int Engine::init() {
  PI05_TRY(cfg_.validate());
  if (prec_ < kPrecBf16 || prec_ > kPrecInt8 || !(act_scale_ > 0.0f)) return kPi05ErrInvalidValue;
  if (weight_dist_ != kWeightsLcg && weight_dist_ != kWeightsNormal) return kPi05ErrInvalidValue;
  // every activation-scale site starts at the uniform scale
  site_scales_.clear();
  const char* kLayerSites[4] = {"attention_norm", "attention_output", "mlp_norm", "mlp_activation"};
  auto add_layers = [&](const char* prefix, int depth) {
    for (int i = 0; i < depth; ++i) {
      for (const char* part : kLayerSites) {
        site_scales_[std::string(prefix) + ".layers." + std::to_string(i) + "." + part] = act_scale_;
      }
    }
  };
  add_layers("vision", cfg_.vision_depth);
  add_layers("language", cfg_.language.depth);
  add_layers("action", cfg_.action.depth);
  for (const char* name : {"vision.patch_input", "vision.post_norm", "action.input", "time.input",
                           "time.hidden", "action.conditioning", "action.final_norm"}) {
    site_scales_[name] = act_scale_;
  }
  PI05_CUDA(cudaSetDevice(device_));
  PI05_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  status_ = static_cast<int*>(dmalloc(256));
  if (status_ == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  PI05_CUDA(cudaMemsetAsync(status_, 0, 256, stream_));

  // RoPE tables: float frequency and angle, as the reference's powf / sincosf path computes
  // them (crates/apxinf-cuda/kernels/custom/fused.cuh:471-490), evaluated in double.
  const int half = cfg_.language.head_dim / 2;
  rope_positions = cfg_.num_views * cfg_.patches_per_view() + cfg_.max_token_len + cfg_.action_horizon;
  std::vector<float> host_cos(static_cast<size_t>(rope_positions) * half), host_sin(host_cos.size());
  for (int i = 0; i < half; ++i) {
    const float freq = static_cast<float>(
        std::pow(static_cast<double>(cfg_.rope_theta), -static_cast<double>(i) / half));
    for (int pos = 0; pos < rope_positions; ++pos) {
      const float angle = static_cast<float>(pos) * freq;
      host_cos[static_cast<size_t>(pos) * half + i] = static_cast<float>(std::cos((double)angle));
      host_sin[static_cast<size_t>(pos) * half + i] = static_cast<float>(std::sin((double)angle));
    }
  }
  rope_cos = static_cast<float*>(dmalloc(host_cos.size() * 4));
  rope_sin = static_cast<float*>(dmalloc(host_sin.size() * 4));
  if (rope_cos == nullptr || rope_sin == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  PI05_CUDA(cudaMemcpyAsync(rope_cos, host_cos.data(), host_cos.size() * 4, cudaMemcpyHostToDevice, stream_));
  PI05_CUDA(cudaMemcpyAsync(rope_sin, host_sin.data(), host_sin.size() * 4, cudaMemcpyHostToDevice, stream_));
  PI05_CUDA(cudaStreamSynchronize(stream_));

  // scratch for generation: largest [in, out] source and largest packed staging matrix
  const GemmaDims& lg = cfg_.language;
  const GemmaDims& ac = cfg_.action;
  size_t max_src = 0, max_stage = 0;
  auto consider = [&](long long k, long long n_part, long long n_total) {
    max_src = std::max(max_src, static_cast<size_t>(k * n_part * 2));
    max_stage = std::max(max_stage, static_cast<size_t>(round_up(k, 16) * n_total * 2));
  };
  const int vw = cfg_.vision_width;
  consider(vw, vw, 3 * vw);
  consider(vw, cfg_.vision_mlp_dim, cfg_.vision_mlp_dim);
  consider(cfg_.vision_mlp_dim, vw, vw);
  consider(cfg_.patch_width(), vw, vw);
  consider(vw, lg.width, lg.width);
  for (const GemmaDims* g : {&lg, &ac}) {
    const int qw = g->num_heads * g->head_dim;
    consider(g->width, qw, qw + 2 * g->head_dim);
    consider(qw, g->width, g->width);
    consider(g->width, g->mlp_dim, 2 * g->mlp_dim);
    consider(g->mlp_dim, g->width, g->width);
  }
  consider(ac.width, 3 * ac.width, 3 * ac.width);
  consider(cfg_.action_dim, ac.width, ac.width);
  consider(ac.width, cfg_.action_dim, cfg_.action_dim);
  // generation scratch is tracked like every other allocation, so a failed init frees it
  // with the engine; the success path releases it early (see the end of this function)
  if (wide_staging()) {  // host tensors are staged and quantised as f32
    max_src *= 2;
    max_stage *= 2;
  }
  size_t convert_bytes = 0;
  if (from_host_) {
    convert_bytes = static_cast<size_t>(kConvertChunk) * 4;
    tmp_convert_ = dmalloc(convert_bytes);
    if (tmp_convert_ == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  }
  tmp_src_ = dmalloc(max_src);
  if (tmp_src_ == nullptr) return record_cuda(cudaErrorMemoryAllocation);
  tmp_src_bytes_ = max_src;
  if (prec_ != kPrecBf16) {
    tmp_stage_ = dmalloc(max_stage);
    if (tmp_stage_ == nullptr) return record_cuda(cudaErrorMemoryAllocation);
    tmp_stage_bytes_ = max_stage;
  }
  weight_bytes_ -= max_src + (prec_ != kPrecBf16 ? max_stage : 0) + convert_bytes;

  // Generation order = Pi05Weights::synthetic (crates/apxinf-model/src/pi05/weights.rs:255-330).
  cursor_ = 0;
  vision.resize(cfg_.vision_depth);
  for (int i = 0; i < cfg_.vision_depth; ++i) {
    const std::string p = "vision." + std::to_string(i);
    PI05_TRY(make_linear(p + ".qkv", {"q", "k", "v"}, vw, {vw, vw, vw}, true, false, &vision[i].qkv));
    PI05_TRY(make_linear(p + ".o", {"o"}, vw, {vw}, true, false, &vision[i].o));
    PI05_TRY(make_linear(p + ".fc1", {"fc1"}, vw, {cfg_.vision_mlp_dim}, true, false, &vision[i].fc1));
    PI05_TRY(make_linear(p + ".fc2", {"fc2"}, cfg_.vision_mlp_dim, {vw}, true, false, &vision[i].fc2));
    PI05_TRY(fetch_layer_norm(p + ".norm1", vw, &vision[i].norm1));
    PI05_TRY(fetch_layer_norm(p + ".norm2", vw, &vision[i].norm2));
  }
  PI05_TRY(fetch_layer_norm("vision.post_norm", vw, &vision_post_norm));
  PI05_TRY(make_linear("vision.patch_embedding", {"w"}, cfg_.patch_width(), {vw}, true, false, &patch));
  {
    const long long count = static_cast<long long>(cfg_.patches_per_view()) * vw;
    position_embedding = dmalloc(count * 2);
    if (position_embedding == nullptr) return record_cuda(cudaErrorMemoryAllocation);
    PI05_TRY(fetch("vision.position_embedding", position_embedding, count));
    named_["vision.position_embedding"] = {position_embedding, (size_t)count * 2};
  }
  PI05_TRY(make_linear("vision.projector", {"w"}, vw, {lg.width}, true, false, &projector));
  {
    const long long count = static_cast<long long>(cfg_.vocab_size) * lg.width;
    token_embedding = dmalloc(count * 2);
    if (token_embedding == nullptr) return record_cuda(cudaErrorMemoryAllocation);
    PI05_TRY(fetch("token_embedding", token_embedding, count));
    named_["token_embedding"] = {token_embedding, (size_t)count * 2};
  }
  language.resize(lg.depth);
  for (int i = 0; i < lg.depth; ++i) {
    const std::string p = "language." + std::to_string(i);
    const int qw = lg.num_heads * lg.head_dim;
    PI05_TRY(make_linear(p + ".qkv", {"q", "k", "v"}, lg.width, {qw, lg.head_dim, lg.head_dim}, false, false, &language[i].qkv));
    PI05_TRY(make_linear(p + ".o", {"o"}, qw, {lg.width}, false, false, &language[i].o));
    PI05_TRY(make_linear(p + ".gate_up", {"gate", "up"}, lg.width, {lg.mlp_dim, lg.mlp_dim}, false, true, &language[i].gate_up));
    PI05_TRY(make_linear(p + ".down", {"down"}, lg.mlp_dim, {lg.width}, false, false, &language[i].down));
  }
  action.resize(ac.depth);
  for (int i = 0; i < ac.depth; ++i) {
    const std::string p = "action." + std::to_string(i);
    const int qw = ac.num_heads * ac.head_dim;
    PI05_TRY(make_linear(p + ".input_style", {"w"}, ac.width, {3 * ac.width}, true, false, &action[i].input_style));
    PI05_TRY(make_linear(p + ".qkv", {"q", "k", "v"}, ac.width, {qw, ac.head_dim, ac.head_dim}, false, false, &action[i].qkv));
    PI05_TRY(make_linear(p + ".o", {"o"}, qw, {ac.width}, false, false, &action[i].o));
    PI05_TRY(make_linear(p + ".post_style", {"w"}, ac.width, {3 * ac.width}, true, false, &action[i].post_style));
    PI05_TRY(make_linear(p + ".gate_up", {"gate", "up"}, ac.width, {ac.mlp_dim, ac.mlp_dim}, false, true, &action[i].gate_up));
    PI05_TRY(make_linear(p + ".down", {"down"}, ac.mlp_dim, {ac.width}, false, false, &action[i].down));
  }
  PI05_TRY(make_linear("action.final_style", {"w"}, ac.width, {3 * ac.width}, true, false, &final_style));
  PI05_TRY(make_linear("action_in", {"w"}, cfg_.action_dim, {ac.width}, true, false, &action_in));
  PI05_TRY(make_linear("action_out", {"w"}, ac.width, {cfg_.action_dim}, true, false, &action_out));
  PI05_TRY(make_linear("time_mlp_in", {"w"}, ac.width, {ac.width}, true, false, &time_in));
  PI05_TRY(make_linear("time_mlp_out", {"w"}, ac.width, {ac.width}, true, false, &time_out));
  PI05_CUDA(cudaStreamSynchronize(stream_));
  release(tmp_src_);
  tmp_src_ = nullptr;
  release(tmp_stage_);
  tmp_stage_ = nullptr;
  release(tmp_convert_);
  tmp_convert_ = nullptr;
  host_tensors_.clear();  // the caller's buffers are not referenced after init
  return kPi05Ok;
}

int Engine::read_weight(const char* name, void* host, size_t capacity, size_t* actual) {
  auto it = named_.find(name);
  if (it == named_.end()) return kPi05ErrInvalidValue;
  if (actual != nullptr) *actual = it->second.second;
  if (host == nullptr) return kPi05Ok;
  if (capacity < it->second.second) return kPi05ErrInvalidValue;
  PI05_CUDA(cudaSetDevice(device_));
  PI05_CUDA(cudaMemcpy(host, it->second.first, it->second.second, cudaMemcpyDeviceToHost));
  return kPi05Ok;
}

// ---------------------------------------------------------------------------
// PreparedGraph
// ---------------------------------------------------------------------------

PreparedGraph::PreparedGraph(Engine* engine, int token_count, int image_layout, int batch)
    : e_(engine), T_(token_count), nchw_(image_layout), B_(batch) {
  const ModelConfig& c = e_->cfg();
  V_ = c.num_views * c.patches_per_view();
  P_ = V_ + T_;
  H_ = c.action_horizon;
  S_ = c.num_flow_steps;
}

PreparedGraph::~PreparedGraph() {
  cudaSetDevice(e_->device());
  cudaStreamSynchronize(e_->stream());
  if (exec_ != nullptr) cudaGraphExecDestroy(exec_);
  if (graph_ != nullptr) cudaGraphDestroy(graph_);
  if (arena_base_ != nullptr) cudaFree(arena_base_);
  if (h_out_ != nullptr) cudaFreeHost(h_out_);
}

void PreparedGraph::add_kernel(const char* name, std::function<cudaError_t(cudaStream_t)> fn) {
  if (measuring_) return;
  Op op;
  op.name = name;
  op.stage = stage_;
  op.launch = std::move(fn);
  ops_.push_back(std::move(op));
}

int PreparedGraph::add_gemm(const char* name, const GemmProblem& request) {
  if (measuring_) return kPi05Ok;
  GemmProblem problem = request;
  problem.partials = d_partials_;
  problem.partials_bytes = kSplitScratchBytes;
  problem.tile_counters = d_tile_counters_;
  problem.max_tiles = kSplitMaxTiles;
  Op op;
  op.name = name;
  op.stage = stage_;
  op.is_gemm = true;
  PI05_TRY(gemm_plan_build(problem, &op.plan));
  ops_.push_back(std::move(op));
  return kPi05Ok;
}

Act PreparedGraph::make_act(int rows, long long ld) {
  Act a;
  a.rows = rows;
  a.ld = ld;
  const int prec = e_->precision();
  a.data = arena_.alloc(static_cast<size_t>(rows) * ld * elem_size(prec));
  if (prec == kPrecInt8) {
    a.row_scale = e_->static_int8() ? nullptr
                                    : static_cast<float*>(arena_.alloc(static_cast<size_t>(rows) * 4));
    a.wide = arena_.alloc(static_cast<size_t>(rows) * ld * 2);
  }
  return a;
}

// out = epilogue(in . w^T) with the precision's operand type and scales.
int PreparedGraph::linear(const char* name, const Act& in, int rows, const Linear& w, int mode,
                          void* out, long long ldc, int out_type, const void* residual,
                          const void* gate, const void* pos, int pos_rows, float out_inv_scale,
                          int nb0, long long a_sb0, long long out_sb0) {
  GemmProblem q;
  const int prec = e_->precision();
  q.op = op_of(prec);
  q.M = rows;
  q.N = w.n;
  q.K = static_cast<int>(std::min<long long>(w.ldk, in.ld));
  // A few hundred rows against a very long K (the B=1 language.down: 522 x 2048 x 16384) give
  // too few output tiles for the SMs: the K range goes in as many slices as fill one wave of
  // CTAs (three for that shape: 5 x 8 tiles x 3 = 120), each writing fp32 partial products, and
  // one row kernel adds them and applies the residual.
  {
    const int block_k = 128 / elem_size(prec);
    const long long tiles256 = (long long)((rows + 127) / 128) * ((w.n + 255) / 256);
    const bool long_k = q.K / block_k >= 96;
    const int slices = static_cast<int>(std::max<long long>(2, std::min<long long>(4, 148 / std::max<long long>(1, tiles256))));
    if (nb0 == 1 && mode == kEpiBiasResidual && out_type == kOutBf16 && gate == nullptr && pos == nullptr &&
        rows > 64 && tiles256 <= 74 && long_k && w.n % 8 == 0 && d_k_partials_ != nullptr &&
        (size_t)rows * w.n * slices * sizeof(float) <= k_partials_bytes_) {
      GemmProblem h = q;
      h.k_slices = slices;
      h.a = GemmOperand{in.data, rows, in.ld, 0, 0};
      h.b = GemmOperand{w.w, w.n, w.ldk, 0, 0};
      h.out = d_k_partials_;
      h.ldc = w.n;
      h.out_sb0 = (long long)rows * w.n;
      h.out_type = kOutF32;
      h.mode = kEpiStore;
      h.col_scale = w.col_scale;
      h.row_scale = prec == kPrecInt8 && !e_->static_int8() ? in.row_scale : nullptr;
      h.row_scale_sb0 = 0;
      h.alpha = e_->static_scales() ? in.scale : 1.0f;
      h.status = e_->status();
      h.b_static = true;
      h.force_block_n = 256;
      PI05_TRY(add_gemm(name, h));
      const float* partials = static_cast<const float*>(d_k_partials_);
      const long long count = (long long)rows * w.n;
      const int cols = w.n;
      const void* bias = w.bias;
      add_kernel((std::string(name) + ".sum").c_str(), [=](cudaStream_t s) {
        return launch_sum_partials(partials, slices, count, cols, residual, bias, out, s);
      });
      if (!measuring_) {
        pending_sum_.op_index = ops_.size() - 1;
        pending_sum_.partials = partials;
        pending_sum_.slices = slices;
        pending_sum_.count = count;
        pending_sum_.cols = cols;
        pending_sum_.residual = residual;
        pending_sum_.bias = bias;
        pending_sum_.out = out;
      }
      return kPi05Ok;
    }
  }
  q.nb0 = nb0;
  q.a = GemmOperand{in.data, rows, in.ld, a_sb0, 0};
  q.b = GemmOperand{w.w, w.n, w.ldk, 0, 0};
  q.out = out;
  q.ldc = ldc;
  q.out_sb0 = out_sb0;
  q.out_type = out_type;
  q.mode = mode;
  q.residual = residual;
  q.bias = w.bias;
  q.col_scale = w.col_scale;
  q.row_scale = prec == kPrecInt8 && !e_->static_int8() ? in.row_scale : nullptr;
  q.row_scale_sb0 = nb0 > 1 ? rows : 0;
  q.pos = pos;
  q.pos_rows = pos_rows;
  q.pos_ld = w.n;
  q.gate = gate;
  q.alpha = e_->static_scales() ? in.scale : 1.0f;
  q.out_inv_scale = out_inv_scale;
  q.status = e_->status();
  q.b_static = true;
  return add_gemm(name, q);
}

// GEMM whose result feeds another GEMM: written in the precision's operand form.
int PreparedGraph::linear_to_act(const char* name, const Act& in, int rows, const Linear& w,
                                 int mode, Act* out, const std::string& site) {
  const int prec = e_->precision();
  out->scale = e_->scale_of(site);
  const float inv = 1.0f / out->scale;
  if (prec == kPrecBf16) {
    return linear(name, in, rows, w, mode, out->data, out->ld, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f);
  }
  if (prec == kPrecFp8) {
    return linear(name, in, rows, w, mode, out->data, out->ld, kOutE4m3, nullptr, nullptr, nullptr, 1, inv);
  }
  if (e_->static_int8()) {
    // static scale: the quantiser is part of the epilogue, like the FP8 path's
    return linear(name, in, rows, w, mode, out->data, out->ld, kOutS8, nullptr, nullptr, nullptr, 1, inv);
  }
  PI05_TRY(linear(name, in, rows, w, mode, out->wide, out->ld, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
  const void* wide = out->wide;
  int8_t* data = static_cast<int8_t*>(out->data);
  float* scale = out->row_scale;
  const int cols = static_cast<int>(out->ld);
  add_kernel("quantize_rows_int8", [=](cudaStream_t s) {
    return launch_quantize_rows_int8(wide, data, scale, rows, cols, cols, cols, s);
  });
  return kPi05Ok;
}

// bf16 tensor -> the precision's GEMM-input form (bf16: `out` aliases the source).
void PreparedGraph::quantize_to_act(const char* name, const void* src, int rows, int cols, Act* out,
                                    const std::string& site) {
  const int prec = e_->precision();
  out->scale = e_->scale_of(site);
  const float inv = 1.0f / out->scale;
  const long long count = static_cast<long long>(rows) * cols;
  if (prec == kPrecBf16) {
    out->data = const_cast<void*>(src);
  } else if (prec == kPrecFp8) {
    uint8_t* dst = static_cast<uint8_t*>(out->data);
    add_kernel(name, [=](cudaStream_t s) { return launch_quantize_e4m3(src, dst, count, inv, s); });
  } else if (e_->static_int8()) {
    int8_t* dst = static_cast<int8_t*>(out->data);
    add_kernel(name, [=](cudaStream_t s) { return launch_quantize_s8(src, dst, count, inv, s); });
  } else {
    int8_t* dst = static_cast<int8_t*>(out->data);
    float* rs = out->row_scale;
    add_kernel(name, [=](cudaStream_t s) { return launch_quantize_rows_int8(src, dst, rs, rows, cols, cols, cols, s); });
  }
}

int PreparedGraph::norm_to_act(const char* name, const void* x, int rows, int cols, int kind,
                               const void* style, float eps, Act* out, const std::string& site,
                               const void* weight, const void* bias) {
  out->scale = e_->scale_of(site);
  NormArgs a{};
  a.weight = weight;
  a.bias = bias;
  a.input = x;
  a.output = out->data;
  a.row_scale = out->row_scale;
  a.style = style;
  a.rows = rows;
  a.cols = cols;
  a.eps = eps;
  a.inv_scale = 1.0f / out->scale;
  a.kind = kind;
  a.static_params = 1;  // weights, and the style vectors built once outside the launch list
  const int prec = e_->precision();
  a.out = prec == kPrecBf16 ? kRowBf16
          : prec == kPrecFp8 ? kRowE4m3
          : e_->static_int8() ? kRowInt8Static
                              : kRowInt8;
  // the rows were just formed by the adding launch of a K-sliced GEMM: one launch does both
  const PendingSum& ps = pending_sum_;
  if (!measuring_ && !ops_.empty() && ps.op_index == ops_.size() - 1 && ps.out == x && ps.cols == cols &&
      ps.count == (long long)rows * cols && kind == kNormRms && rows < 1024) {
    a.sum_partials = ps.partials;
    a.sum_splits = ps.slices;
    a.sum_stride = ps.count;
    a.sum_residual = ps.residual;
    a.sum_bias = ps.bias;
    Op& op = ops_.back();
    op.name = op.name + "+" + name;
    op.launch = [a](cudaStream_t s) { return launch_norm(a, s); };
    pending_sum_ = PendingSum{};
    return kPi05Ok;
  }
  add_kernel(name, [a](cudaStream_t s) { return launch_norm(a, s); });
  return kPi05Ok;
}

// softmax(scale * q k^T) v as two tensor-core GEMMs around a row softmax, the
// logits and probabilities held as bf16 like the reference's MQA
// (crates/apxinf-cuda/adapters/cublas_adapter.cu:89-132). v is consumed in its
// natural [keys, head_dim] layout as an MN-major operand.
int PreparedGraph::attention(const char* name, const void* q, long long q_ld, long long q_sb0,
                             long long q_sb1, const void* k, long long k_ld, long long k_sb0,
                             long long k_sb1, const void* v, long long v_ld, long long v_sb0,
                             long long v_sb1, int q_rows, int keys, int head_dim, int nb0, int nb1,
                             float scale, void* logits, Act* out, long long out_ld,
                             long long out_sb0, long long out_sb1) {
  const int prec_now = e_->precision();
  // the fused kernel gives one CTA per 128 query rows: with only a few of them (the B=1
  // action expert) the three-launch path, which spreads keys over more CTAs, is quicker
  const bool shared_kv = nb0 > 1 && k_sb0 == 0 && v_sb0 == 0 && 128 % nb0 == 0;
  const long long fused_ctas = fmha_query_tiles(q_rows, nb0, nb1, shared_kv);
  // a handful of query tiles (B=1 action expert): one CTA per (tile, 64-key slice) and a
  // combine launch keep many more SMs pulling the K/V cache
  const bool key_split = fmha_supported(q_rows, keys, head_dim) && fused_ctas < 32 &&
                         fmha_split_scratch_bytes(q_rows, keys, head_dim, nb0, nb1, shared_kv) <=
                             kSplitScratchBytes;
  if (fmha_supported(q_rows, keys, head_dim) && (fused_ctas >= 8 || key_split)) {
    if (!measuring_) {
      FmhaProblem f;
      f.q = q; f.q_ld = q_ld; f.q_sb0 = q_sb0; f.q_sb1 = q_sb1;
      f.k = k; f.k_ld = k_ld; f.k_sb0 = k_sb0; f.k_sb1 = k_sb1;
      f.v = v; f.v_ld = v_ld; f.v_sb0 = v_sb0; f.v_sb1 = v_sb1;
      f.out = prec_now == kPrecInt8 ? out->wide : out->data;
      f.out_ld = out_ld; f.out_sb0 = out_sb0; f.out_sb1 = out_sb1;
      f.q_rows = q_rows; f.keys = keys; f.head_dim = head_dim; f.nb0 = nb0; f.nb1 = nb1;
      f.scale = scale;
      f.out_e4m3 = prec_now == kPrecFp8;
      f.out_inv_scale = 1.0f / out->scale;
      f.status = e_->status();
      f.key_split = key_split;
      f.split_scratch = static_cast<float*>(d_partials_);
      f.split_scratch_bytes = kSplitScratchBytes;
      Op op;
      op.name = name;
      op.stage = stage_;
      op.is_fmha = true;
      PI05_TRY(fmha_plan_build(f, &op.fmha));
      ops_.push_back(std::move(op));
    }
    if (prec_now == kPrecInt8) quantize_attention_output(out);
    return kPi05Ok;
  }
  const long long ld_s = round_up(keys, 8);
  const long long s_sb0 = static_cast<long long>(q_rows) * ld_s;
  const long long s_sb1 = s_sb0 * nb0;
  GemmProblem s;
  s.op = kOpBf16;
  s.M = q_rows;
  s.N = keys;
  s.K = head_dim;
  s.nb0 = nb0;
  s.nb1 = nb1;
  s.a = GemmOperand{q, q_rows, q_ld, q_sb0, q_sb1};
  s.b = GemmOperand{k, keys, k_ld, k_sb0, k_sb1};
  s.out = logits;
  s.ldc = ld_s;
  s.out_sb0 = s_sb0;
  s.out_sb1 = s_sb1;
  s.alpha = scale;
  s.status = e_->status();
  PI05_TRY(add_gemm((std::string(name) + ".qk").c_str(), s));
  const int batches = nb0 * nb1;
  add_kernel((std::string(name) + ".softmax").c_str(), [=](cudaStream_t st) {
    return launch_softmax(logits, q_rows, batches, s_sb0, keys, ld_s, st);
  });
  GemmProblem pv;
  pv.op = kOpBf16;
  pv.M = q_rows;
  pv.N = head_dim;
  pv.K = keys;
  pv.nb0 = nb0;
  pv.nb1 = nb1;
  pv.a = GemmOperand{logits, q_rows, ld_s, s_sb0, s_sb1};
  pv.b = GemmOperand{v, keys, v_ld, v_sb0, v_sb1};
  pv.b_mn_major = true;
  const int prec = e_->precision();
  pv.out = prec == kPrecInt8 ? out->wide : out->data;
  pv.ldc = out_ld;
  pv.out_sb0 = out_sb0;
  pv.out_sb1 = out_sb1;
  pv.out_type = prec == kPrecFp8 ? kOutE4m3 : kOutBf16;
  pv.out_inv_scale = 1.0f / out->scale;
  pv.status = e_->status();
  PI05_TRY(add_gemm((std::string(name) + ".pv").c_str(), pv));
  if (prec == kPrecInt8) quantize_attention_output(out);
  return kPi05Ok;
}

// INT8: the attention kernels leave bf16 in `wide`; one more launch makes the int8 operand
// (per-row scales, or the tensor's static scale).
void PreparedGraph::quantize_attention_output(Act* out) {
  const void* wide = out->wide;
  int8_t* data = static_cast<int8_t*>(out->data);
  const int rows = out->rows, cols = static_cast<int>(out->ld);
  if (e_->static_int8()) {
    const float inv = 1.0f / out->scale;
    const long long count = static_cast<long long>(rows) * cols;
    add_kernel("quantize_s8", [=](cudaStream_t st) { return launch_quantize_s8(wide, data, count, inv, st); });
  } else {
    float* rs = out->row_scale;
    add_kernel("quantize_rows_int8", [=](cudaStream_t st) {
      return launch_quantize_rows_int8(wide, data, rs, rows, cols, cols, cols, st);
    });
  }
}

int PreparedGraph::build(bool measuring) {
  measuring_ = measuring;
  ops_.clear();
  tensors_.clear();
  const ModelConfig& c = e_->cfg();
  const int prec = e_->precision();
  const GemmaDims& lg = c.language;
  const GemmaDims& ac = c.action;
  const int vw = c.vision_width, pp = c.patches_per_view(), heads_v = c.vision_heads,
            hd_v = c.vision_head_dim;
  const int Rv = B_ * V_, Rp = B_ * P_, Ra = B_ * H_;
  const int n_images = B_ * c.num_views;
  const int cache_rows = P_ + H_;
  const int hd = lg.head_dim, qh = lg.num_heads, qw = qh * hd;
  const long long patch_ld = e_->patch.ldk;

  // ---- inputs / persistent buffers ----
  d_images_ = static_cast<uint8_t*>(arena_.alloc((size_t)n_images * c.image_size * c.image_size * 3));
  if (nchw_ == kLayoutPatches) {
    d_patches_in_ = static_cast<float*>(arena_.alloc(
        (size_t)n_images * c.patches_per_view() * 3 * c.patch_size * c.patch_size * sizeof(float)));
  }
  d_tokens_ = static_cast<uint32_t*>(arena_.alloc((size_t)B_ * T_ * 4));
  d_noise_ = arena_.alloc((size_t)Ra * c.action_dim * 2);
  d_state_ = arena_.alloc((size_t)Ra * c.action_dim * 2);
  d_styles_ = arena_.alloc((size_t)(2 * ac.depth + 1) * S_ * 3 * ac.width * 2);
  d_time_emb_ = arena_.alloc((size_t)S_ * ac.width * 2);
  d_partials_ = arena_.alloc(kSplitScratchBytes);
  // fp32 partial products of a K-halved GEMM (B=1 prefill only: a few hundred rows)
  k_partials_bytes_ = Rp <= 640 ? (size_t)Rp * lg.width * 4 * sizeof(float) : 0;
  d_k_partials_ = k_partials_bytes_ > 0 ? arena_.alloc(k_partials_bytes_) : nullptr;
  d_tile_counters_ = static_cast<int*>(arena_.alloc((size_t)kSplitMaxTiles * 4));
  note("state", d_state_, (size_t)Ra * c.action_dim * 2);
  note("styles", d_styles_, (size_t)(2 * ac.depth + 1) * S_ * 3 * ac.width * 2);
  std::vector<void*> k_cache(lg.depth), v_cache(lg.depth);
  for (int l = 0; l < lg.depth; ++l) {
    k_cache[l] = arena_.alloc((size_t)B_ * cache_rows * hd * 2);
    v_cache[l] = arena_.alloc((size_t)B_ * cache_rows * hd * 2);
    note(("kv." + std::to_string(l) + ".k").c_str(), k_cache[l], (size_t)B_ * cache_rows * hd * 2);
    note(("kv." + std::to_string(l) + ".v").c_str(), v_cache[l], (size_t)B_ * cache_rows * hd * 2);
  }

  // ---- style pre-pass buffers (conditioning is per flow step, not per sample) ----
  Act time_in_act = make_act(S_, ac.width);
  Act time_hidden = make_act(S_, ac.width);
  Act cond = make_act(S_, ac.width);

  if (styles_only_) {
    // time embedding -> conditioning -> 2*depth+1 style vectors, all steps as GEMM rows
    // (crates/apxinf-model/src/pi05/bf16_runtime.rs:258-303).
    stage_ = 3;
    quantize_to_act("quantize_time", d_time_emb_, S_, ac.width, &time_in_act, "time.input");
    PI05_TRY(linear_to_act("time_mlp_in", time_in_act, S_, e_->time_in, kEpiBiasSilu, &time_hidden, "time.hidden"));
    PI05_TRY(linear_to_act("time_mlp_out", time_hidden, S_, e_->time_out, kEpiBiasSilu, &cond, "action.conditioning"));
    for (int idx = 0; idx <= 2 * ac.depth; ++idx) {
      const Linear& w = idx == 2 * ac.depth ? e_->final_style
                        : (idx % 2 == 0 ? e_->action[idx / 2].input_style
                                        : e_->action[idx / 2].post_style);
      void* dst = static_cast<uint16_t*>(d_styles_) + (size_t)idx * S_ * 3 * ac.width;
      PI05_TRY(linear("style", cond, S_, w, kEpiStore, dst, 3 * ac.width, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
    }
    return kPi05Ok;
  }
  auto style_ptr = [&](int idx, int step) -> const void* {
    return static_cast<const uint16_t*>(d_styles_) + ((size_t)idx * S_ + step) * 3 * ac.width;
  };

  // ---- stage 0: preprocessing + SigLIP tower ----
  stage_ = 0;
  Act patches = make_act(Rv, patch_ld);
  void* xv = arena_.alloc((size_t)Rv * vw * 2);
  Act nv = make_act(Rv, vw);
  void* qkv_v = arena_.alloc((size_t)Rv * 3 * vw * 2);
  void* logits_v = arena_.alloc((size_t)n_images * heads_v * pp * round_up(pp, 8) * 2);
  Act attn_v = make_act(Rv, vw);
  Act act_v = make_act(Rv, c.vision_mlp_dim);
  void* xp = arena_.alloc((size_t)Rp * lg.width * 2);
  note("patches", prec == kPrecInt8 ? patches.wide : patches.data, (size_t)Rv * patch_ld * (prec == kPrecFp8 ? 1 : 2));
  note("vision.hidden", xv, (size_t)Rv * vw * 2);
  note("prefix", xp, (size_t)Rp * lg.width * 2);
  {
    patches.scale = e_->scale_of("vision.patch_input");
    PatchifyArgs pa{};
    pa.images = d_images_;
    pa.f32_patches = d_patches_in_;  // null unless the graph takes ready-made patches
    pa.patches = prec == kPrecInt8 ? patches.wide : patches.data;
    pa.n_images = n_images;
    pa.image_size = c.image_size;
    pa.patch_size = c.patch_size;
    pa.ld = static_cast<int>(patch_ld);
    pa.nchw = nchw_ == 1;
    pa.out = prec == kPrecFp8 ? kRowE4m3 : kRowBf16;
    pa.inv_scale = 1.0f / patches.scale;
    add_kernel("patchify", [pa](cudaStream_t s) { return launch_patchify(pa, s); });
    if (prec == kPrecInt8) {
      Act q = patches;
      quantize_to_act("quantize_patches", patches.wide, Rv, static_cast<int>(patch_ld), &q, "vision.patch_input");
    }
  }
  PI05_TRY(linear("vision.patch_embed", patches, Rv, e_->patch, kEpiBiasPos, xv, vw, kOutBf16, nullptr, nullptr, e_->position_embedding, pp, 1.0f));
  auto vsite = [](int i, const char* part) { return "vision.layers." + std::to_string(i) + "." + part; };
  auto lsite = [](int i, const char* part) { return "language.layers." + std::to_string(i) + "." + part; };
  auto asite = [](int i, const char* part) { return "action.layers." + std::to_string(i) + "." + part; };
  {
    const Engine::LayerNormParams& first = c.vision_depth > 0 ? e_->vision[0].norm1 : e_->vision_post_norm;
    PI05_TRY(norm_to_act("vision.ln1", xv, Rv, vw, kNormLayer, nullptr, c.layer_norm_eps, &nv,
                         c.vision_depth > 0 ? vsite(0, "attention_norm") : std::string("vision.post_norm"),
                         first.weight, first.bias));
  }
  const float scale_v = static_cast<float>(1.0 / std::sqrt(static_cast<double>(hd_v)));
  for (int i = 0; i < c.vision_depth; ++i) {
    const Engine::VisionBlock& w = e_->vision[i];
    PI05_TRY(linear("vision.qkv", nv, Rv, w.qkv, kEpiStore, qkv_v, 3 * vw, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
    const uint16_t* base = static_cast<const uint16_t*>(qkv_v);
    attn_v.scale = e_->scale_of(vsite(i, "attention_output"));
    PI05_TRY(attention("vision.attn", base, 3 * vw, hd_v, (long long)pp * 3 * vw, base + vw, 3 * vw, hd_v,
                       (long long)pp * 3 * vw, base + 2 * vw, 3 * vw, hd_v, (long long)pp * 3 * vw, pp, pp,
                       hd_v, heads_v, n_images, scale_v, logits_v, &attn_v, vw, hd_v, (long long)pp * vw));
    PI05_TRY(linear("vision.o", attn_v, Rv, w.o, kEpiBiasResidual, xv, vw, kOutBf16, xv, nullptr, nullptr, 1, 1.0f));
    PI05_TRY(norm_to_act("vision.ln2", xv, Rv, vw, kNormLayer, nullptr, c.layer_norm_eps, &nv, vsite(i, "mlp_norm"),
                         w.norm2.weight, w.norm2.bias));
    PI05_TRY(linear_to_act("vision.fc1", nv, Rv, w.fc1, kEpiBiasGelu, &act_v, vsite(i, "mlp_activation")));
    PI05_TRY(linear("vision.fc2", act_v, Rv, w.fc2, kEpiBiasResidual, xv, vw, kOutBf16, xv, nullptr, nullptr, 1, 1.0f));
    {
      const Engine::LayerNormParams& next = i + 1 < c.vision_depth ? e_->vision[i + 1].norm1 : e_->vision_post_norm;
      PI05_TRY(norm_to_act(i + 1 < c.vision_depth ? "vision.ln1" : "vision.post_ln", xv, Rv, vw, kNormLayer, nullptr, c.layer_norm_eps, &nv,
                           i + 1 < c.vision_depth ? vsite(i + 1, "attention_norm") : std::string("vision.post_norm"),
                           next.weight, next.bias));
    }
  }
  // projector writes the image tokens straight into rows [0, V) of each sample's prefix
  PI05_TRY(linear("vision.projector", nv, V_, e_->projector, kEpiStore, xp, lg.width, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f, B_, (long long)V_ * vw, (long long)P_ * lg.width));
  {
    const void* table = e_->token_embedding;
    const uint32_t* ids = d_tokens_;
    const int batch = B_, tokens = T_, width = lg.width, vocab = c.vocab_size, rows = P_, off = V_;
    add_kernel("embedding", [=](cudaStream_t s) { return launch_embedding(table, ids, xp, batch, tokens, width, vocab, rows, off, s); });
  }

  // ---- stage 1: Gemma prefix prefill into the KV cache ----
  stage_ = 1;
  Act np_ = make_act(Rp, lg.width);
  void* qkv_p = arena_.alloc((size_t)Rp * (qw + 2 * hd) * 2);
  void* qbuf_p = arena_.alloc((size_t)Rp * qw * 2);
  void* logits_p = arena_.alloc((size_t)B_ * qh * P_ * round_up(cache_rows, 8) * 2);
  Act attn_p = make_act(Rp, qw);
  Act act_p = make_act(Rp, lg.mlp_dim);
  const float scale_g = static_cast<float>(1.0 / std::sqrt(static_cast<double>(hd)));
  PI05_TRY(norm_to_act("language.norm", xp, Rp, lg.width, kNormRms, nullptr, c.rms_norm_eps, &np_, lsite(0, "attention_norm")));
  for (int l = 0; l < lg.depth; ++l) {
    const Engine::LanguageLayer& w = e_->language[l];
    PI05_TRY(linear("language.qkv", np_, Rp, w.qkv, kEpiStore, qkv_p, qw + 2 * hd, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
    RopeArgs ra{};
    ra.qkv = qkv_p;
    ra.q_out = qbuf_p;
    ra.k_cache = k_cache[l];
    ra.v_cache = v_cache[l];
    ra.cos_table = e_->rope_cos;
    ra.sin_table = e_->rope_sin;
    ra.rows = Rp;
    ra.tokens = P_;
    ra.q_heads = qh;
    ra.head_dim = hd;
    ra.position_offset = 0;
    ra.cache_rows = cache_rows;
    add_kernel("language.rope", [ra](cudaStream_t s) { return launch_rope(ra, s); });
    if (l + 1 == lg.depth) break;  // the last layer only contributes K/V (bf16_runtime.rs:233)
    attn_p.scale = e_->scale_of(lsite(l, "attention_output"));
    PI05_TRY(attention("language.attn", qbuf_p, hd, (long long)P_ * qw, 0, k_cache[l], hd, (long long)cache_rows * hd, 0,
                       v_cache[l], hd, (long long)cache_rows * hd, 0, P_ * qh, P_, hd, B_, 1, scale_g,
                       logits_p, &attn_p, hd, (long long)P_ * qw, 0));
    PI05_TRY(linear("language.o", attn_p, Rp, w.o, kEpiBiasResidual, xp, lg.width, kOutBf16, xp, nullptr, nullptr, 1, 1.0f));
    PI05_TRY(norm_to_act("language.norm", xp, Rp, lg.width, kNormRms, nullptr, c.rms_norm_eps, &np_, lsite(l, "mlp_norm")));
    PI05_TRY(linear_to_act("language.gate_up", np_, Rp, w.gate_up, kEpiGeglu, &act_p, lsite(l, "mlp_activation")));
    PI05_TRY(linear("language.down", act_p, Rp, w.down, kEpiBiasResidual, xp, lg.width, kOutBf16, xp, nullptr, nullptr, 1, 1.0f));
    PI05_TRY(norm_to_act("language.norm", xp, Rp, lg.width, kNormRms, nullptr, c.rms_norm_eps, &np_, lsite(l + 1, "attention_norm")));
  }

  // ---- stage 2: flow-matching denoise loop of the action expert ----
  stage_ = 2;
  Act state_act = make_act(Ra, c.action_dim);
  void* ha = arena_.alloc((size_t)Ra * ac.width * 2);
  Act na = make_act(Ra, ac.width);
  void* qkv_a = arena_.alloc((size_t)Ra * (qw + 2 * hd) * 2);
  void* qbuf_a = arena_.alloc((size_t)Ra * qw * 2);
  void* logits_a = arena_.alloc((size_t)B_ * qh * H_ * round_up(cache_rows, 8) * 2);
  Act attn_a = make_act(Ra, qw);
  Act act_a = make_act(Ra, ac.mlp_dim);
  void* velocity = arena_.alloc((size_t)Ra * c.action_dim * 2);
  note("action.hidden", ha, (size_t)Ra * ac.width * 2);
  {
    void* dst = d_state_;
    const void* src = d_noise_;
    const size_t bytes = (size_t)Ra * c.action_dim * 2;
    add_kernel("load_noise", [=](cudaStream_t s) { return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s); });
  }
  const float dt = -1.0f / static_cast<float>(S_);
  // At most 16 action rows (B=1, H <= 16): every projection runs on the register-streaming
  // kernel; RoPE + the K/V-cache write are the q|k|v projection's epilogue, the state quantiser
  // the input projection's staging step, and the final norm and the Euler update the prologue
  // and epilogue of the velocity head. Seven launches per layer and step (norm, qkv, attention,
  // o, norm, gate_up, down) instead of nine, and three fewer per step.
  const bool fuse_rows = fuse_small_rows_enabled() && Ra <= 16 && ac.width <= 1024 && ac.width % 8 == 0 && c.action_dim % 8 == 0;
  // ... and the whole loop, all steps and layers, goes into ONE cooperative launch whose stages
  // are these projections and attentions (denoise_persistent.cuh); the adaptive norms then run
  // as the staging step of the projection that reads them. Where the launch list does not
  // qualify (or the device cannot launch cooperatively) the same list runs launch by launch.
  const bool persistent = fuse_rows && persistent_denoise_enabled() && B_ == 1 &&
                          (prec == kPrecFp8 || prec == kPrecBf16);
  // the fused norms need the register-resident staging step: rows x chunks within its budget
  const bool fused_norms = fuse_rows && (persistent || fuse_norms_enabled()) &&
                           !(prec == kPrecInt8 && !e_->static_int8()) &&
                           Ra * (ac.width / 8) <= kSkinnyFastItems * 32 * kSkinnyMaxWarps;
  const int denoise_stage_capacity = S_ * (2 + 5 * ac.depth);
  const int denoise_tiles = (H_ * qh + 15) / 16;
  void* denoise_table = nullptr;
  unsigned* denoise_zero = nullptr;
  float* denoise_scratch = nullptr;
  const size_t denoise_zero_bytes = 256 + static_cast<size_t>(denoise_tiles) * 4;
  if (persistent) {
    denoise_table = arena_.alloc(static_cast<size_t>(denoise_stage_capacity) * sizeof(DenoiseStage));
    denoise_zero = static_cast<unsigned*>(arena_.alloc(denoise_zero_bytes));
    denoise_scratch = static_cast<float*>(arena_.alloc(static_cast<size_t>(denoise_tiles) * kRowsCluster *
                                                       rows_partial_floats(hd) * sizeof(float)));
  }
  const size_t denoise_first_op = ops_.size();
  // GEMM of <= 16 rows whose bf16 input `src` [Ra, k] is normalised / quantised while staged
  auto fused_problem = [&](const Linear& w, const void* src, int k, int prologue, const void* style,
                           const std::string& site) {
    GemmProblem q;
    const float scale = e_->scale_of(site);
    q.op = op_of(prec);
    q.M = Ra;
    q.N = w.n;
    q.K = k;
    q.a = GemmOperand{src, Ra, k, 0, 0};
    q.b = GemmOperand{w.w, w.n, w.ldk, 0, 0};
    q.bias = w.bias;
    q.col_scale = w.col_scale;
    q.alpha = e_->static_scales() ? scale : 1.0f;
    q.status = e_->status();
    q.b_static = true;
    q.force_skinny = 1;
    q.prologue = prec == kPrecBf16 && prologue == kProQuantize ? kProNone : prologue;
    q.style = style;
    q.eps = c.rms_norm_eps;
    q.a_inv_scale = 1.0f / scale;
    q.a_dynamic_rows = prec == kPrecInt8 && !e_->static_int8();
    return q;
  };
  for (int step = 0; step < S_; ++step) {
    if (fuse_rows) {
      {
        GemmProblem q = fused_problem(e_->action_in, d_state_, c.action_dim, kProQuantize, nullptr, "action.input");
        q.out = ha;
        q.ldc = ac.width;
        PI05_TRY(add_gemm("action.in", q));
      }
      // As launches of their own the two adaRMSNorms of a layer stay launches: as a staging step
      // of the 80-128 CTAs of the following projection they cost each of those CTAs what the
      // 10-CTA kernel costs once (measured: 2.5-4 us added to a 3.4 us projection, against about
      // 2 us for the dependent-launched norm kernel). As stages of the persistent kernel they
      // would each cost a grid barrier, so there they are the projections' staging step.
      if (!fused_norms) {
        PI05_TRY(norm_to_act("action.ada_norm", ha, Ra, ac.width, kNormAda, style_ptr(0, step), c.rms_norm_eps, &na, asite(0, "attention_norm")));
      }
      for (int l = 0; l < ac.depth; ++l) {
        const Engine::ActionLayer& w = e_->action[l];
        const uint16_t* attn_style = static_cast<const uint16_t*>(style_ptr(2 * l, step));
        const uint16_t* mlp_style = static_cast<const uint16_t*>(style_ptr(2 * l + 1, step));
        const void* next_style = style_ptr(2 * l + 2, step);
        {
          // q|k|v projection with RoPE, Q rows and the K/V-cache rows written by its epilogue
          GemmProblem q;
          if (fused_norms) {
            q = fused_problem(w.qkv, ha, ac.width, kProAdaNorm, attn_style, asite(l, "attention_norm"));
          } else {
            q.op = op_of(prec);
            q.M = Ra;
            q.N = w.qkv.n;
            q.K = static_cast<int>(std::min<long long>(w.qkv.ldk, na.ld));
            q.a = GemmOperand{na.data, Ra, na.ld, 0, 0};
            q.b = GemmOperand{w.qkv.w, w.qkv.n, w.qkv.ldk, 0, 0};
            q.col_scale = w.qkv.col_scale;
            q.row_scale = prec == kPrecInt8 && !e_->static_int8() ? na.row_scale : nullptr;
            q.alpha = e_->static_scales() ? na.scale : 1.0f;
            q.status = e_->status();
            q.b_static = true;
            q.force_skinny = 1;
          }
          q.out = qkv_a;  // unused by the RoPE epilogue, kept as a valid pointer
          q.ldc = qw + 2 * hd;
          q.mode = kEpiRope;
          q.rope_q_out = qbuf_a;
          q.rope_k_cache = k_cache[l];
          q.rope_v_cache = v_cache[l];
          q.rope_cos = e_->rope_cos;
          q.rope_sin = e_->rope_sin;
          q.rope_tokens = H_;
          q.rope_q_heads = qh;
          q.rope_head_dim = hd;
          q.rope_position_offset = P_;
          q.rope_cache_rows = cache_rows;
          PI05_TRY(add_gemm("action.qkv", q));
        }
        attn_a.scale = e_->scale_of(asite(l, "attention_output"));
        PI05_TRY(attention("action.attn", qbuf_a, hd, (long long)H_ * qw, 0, k_cache[l], hd, (long long)cache_rows * hd, 0,
                           v_cache[l], hd, (long long)cache_rows * hd, 0, H_ * qh, cache_rows, hd, B_, 1, scale_g,
                           logits_a, &attn_a, hd, (long long)H_ * qw, 0));
        PI05_TRY(linear("action.o", attn_a, Ra, w.o, kEpiGateResidual, ha, ac.width, kOutBf16, ha, attn_style + 2 * ac.width, nullptr, 1, 1.0f));
        if (fused_norms) {
          GemmProblem g = fused_problem(w.gate_up, ha, ac.width, kProAdaNorm, mlp_style, asite(l, "mlp_norm"));
          act_a.scale = e_->scale_of(asite(l, "mlp_activation"));
          g.out = act_a.data;
          g.ldc = act_a.ld;
          g.mode = kEpiGeglu;
          g.out_type = prec == kPrecBf16 ? kOutBf16 : prec == kPrecFp8 ? kOutE4m3 : kOutS8;
          g.out_inv_scale = 1.0f / act_a.scale;
          PI05_TRY(add_gemm("action.gate_up", g));
        } else {
          PI05_TRY(norm_to_act("action.ada_norm", ha, Ra, ac.width, kNormAda, mlp_style, c.rms_norm_eps, &na, asite(l, "mlp_norm")));
          PI05_TRY(linear_to_act("action.gate_up", na, Ra, w.gate_up, kEpiGeglu, &act_a, asite(l, "mlp_activation")));
        }
        PI05_TRY(linear("action.down", act_a, Ra, w.down, kEpiGateResidual, ha, ac.width, kOutBf16, ha, mlp_style + 2 * ac.width, nullptr, 1, 1.0f));
        if (l + 1 < ac.depth && !fused_norms) {
          PI05_TRY(norm_to_act("action.ada_norm", ha, Ra, ac.width, kNormAda, next_style, c.rms_norm_eps, &na, asite(l + 1, "attention_norm")));
        }
      }
      {
        // final adaRMSNorm -> velocity head -> Euler update of the state, one launch
        GemmProblem q = fused_problem(e_->action_out, ha, ac.width, kProAdaNorm, style_ptr(2 * ac.depth, step), "action.final_norm");
        q.out = d_state_;
        q.ldc = c.action_dim;
        q.mode = kEpiEuler;
        q.residual = d_state_;
        q.dt = dt;
        PI05_TRY(add_gemm("action.out", q));
      }
      continue;
    }
    quantize_to_act("quantize_state", d_state_, Ra, c.action_dim, &state_act, "action.input");
    PI05_TRY(linear("action.in", state_act, Ra, e_->action_in, kEpiStore, ha, ac.width, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
    PI05_TRY(norm_to_act("action.ada_norm", ha, Ra, ac.width, kNormAda, style_ptr(0, step), c.rms_norm_eps, &na, asite(0, "attention_norm")));
    for (int l = 0; l < ac.depth; ++l) {
      const Engine::ActionLayer& w = e_->action[l];
      const uint16_t* attn_style = static_cast<const uint16_t*>(style_ptr(2 * l, step));
      const uint16_t* mlp_style = static_cast<const uint16_t*>(style_ptr(2 * l + 1, step));
      const void* next_style = style_ptr(2 * l + 2, step);  // next layer's input style or the final style
      PI05_TRY(linear("action.qkv", na, Ra, w.qkv, kEpiStore, qkv_a, qw + 2 * hd, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
      RopeArgs ra{};
      ra.qkv = qkv_a;
      ra.q_out = qbuf_a;
      ra.k_cache = k_cache[l];
      ra.v_cache = v_cache[l];
      ra.cos_table = e_->rope_cos;
      ra.sin_table = e_->rope_sin;
      ra.rows = Ra;
      ra.tokens = H_;
      ra.q_heads = qh;
      ra.head_dim = hd;
      ra.position_offset = P_;
      ra.cache_rows = cache_rows;
      add_kernel("action.rope", [ra](cudaStream_t s) { return launch_rope(ra, s); });
      attn_a.scale = e_->scale_of(asite(l, "attention_output"));
      PI05_TRY(attention("action.attn", qbuf_a, hd, (long long)H_ * qw, 0, k_cache[l], hd, (long long)cache_rows * hd, 0,
                         v_cache[l], hd, (long long)cache_rows * hd, 0, H_ * qh, cache_rows, hd, B_, 1, scale_g,
                         logits_a, &attn_a, hd, (long long)H_ * qw, 0));
      PI05_TRY(linear("action.o", attn_a, Ra, w.o, kEpiGateResidual, ha, ac.width, kOutBf16, ha, attn_style + 2 * ac.width, nullptr, 1, 1.0f));
      PI05_TRY(norm_to_act("action.ada_norm", ha, Ra, ac.width, kNormAda, mlp_style, c.rms_norm_eps, &na, asite(l, "mlp_norm")));
      PI05_TRY(linear_to_act("action.gate_up", na, Ra, w.gate_up, kEpiGeglu, &act_a, asite(l, "mlp_activation")));
      PI05_TRY(linear("action.down", act_a, Ra, w.down, kEpiGateResidual, ha, ac.width, kOutBf16, ha, mlp_style + 2 * ac.width, nullptr, 1, 1.0f));
      PI05_TRY(norm_to_act("action.ada_norm", ha, Ra, ac.width, kNormAda, next_style, c.rms_norm_eps, &na,
                           l + 1 < ac.depth ? asite(l + 1, "attention_norm") : std::string("action.final_norm")));
    }
    PI05_TRY(linear("action.out", na, Ra, e_->action_out, kEpiStore, velocity, c.action_dim, kOutBf16, nullptr, nullptr, nullptr, 1, 1.0f));
    {
      void* st = d_state_;
      const long long count = (long long)Ra * c.action_dim;
      add_kernel("euler", [=](cudaStream_t s) { return launch_euler(st, velocity, count, dt, s); });
    }
  }
  if (persistent && !measuring_) {
    PI05_TRY(fold_denoise(denoise_first_op, denoise_table, denoise_stage_capacity, denoise_zero,
                          denoise_zero_bytes, denoise_scratch, denoise_tiles));
  }
  return kPi05Ok;
}

// Turns ops_[first, end) — the denoise loop planned as one launch per projection / attention —
// into the stage table of the persistent kernel and one op that launches it. Leaves the list as
// it is (every op is a valid launch) when an op is of another kind, a stage wants more CTAs than
// a cooperative launch may have here, or the table does not fit.
int PreparedGraph::fold_denoise(size_t first, void* table, int capacity, unsigned* zero_base,
                                size_t zero_bytes, float* scratch, int tiles) {
  if (first >= ops_.size()) return kPi05Ok;
  std::vector<DenoiseStage> stages;
  int stage_smem = 0, epoch = 0;
  for (size_t i = first; i < ops_.size(); ++i) {
    const Op& op = ops_[i];
    DenoiseStage st{};
    if (op.is_gemm && op.plan.skinny) {
      st.kind = op.plan.block_n == 16 ? kStageGemm2 : kStageGemm1;
      st.ctas = static_cast<int>(op.plan.grid.x);
      st.threads = op.plan.threads;
      st.gemm = op.plan.skinny_params;
      stage_smem = std::max(stage_smem, op.plan.smem_bytes);
    } else if (op.is_fmha && op.fmha.rows_cluster && op.fmha.key_split) {
      FmhaRowsParams rows;
      std::memcpy(&rows, op.fmha.rows_params, sizeof(rows));
      if (rows.tiles > tiles || static_cast<int>(op.fmha.grid.x) != rows.tiles * kRowsCluster) return kPi05Ok;
      st.kind = kStageAttention;
      st.ctas = static_cast<int>(op.fmha.grid.x);
      st.threads = kRowsThreads;
      st.epoch = epoch++;
      st.attention = rows;
      stage_smem = std::max(stage_smem, op.fmha.rows_smem);
    } else {
      return kPi05Ok;
    }
    stages.push_back(st);
  }
  if (static_cast<int>(stages.size()) > capacity) return kPi05Ok;
  DenoisePlan plan;
  plan.op = op_of(e_->precision());
  plan.smem_bytes = denoise_smem_bytes(stage_smem);
  plan.grid = denoise_max_grid(plan.op, plan.smem_bytes, e_->device());
  for (const DenoiseStage& st : stages) {
    if (st.ctas > plan.grid || st.threads > kDenoiseThreads) return kPi05Ok;
  }
  denoise_stages_ = std::move(stages);
  PI05_CUDA(cudaMemcpyAsync(table, denoise_stages_.data(), denoise_stages_.size() * sizeof(DenoiseStage),
                            cudaMemcpyHostToDevice, e_->stream()));
  plan.params.stages = static_cast<const DenoiseStage*>(table);
  plan.params.count = static_cast<int>(denoise_stages_.size());
  plan.params.barrier = zero_base;
  plan.params.tile_flags = zero_base + 64;
  plan.params.scratch = scratch;
  plan.params.status = e_->status();
  plan.params.spin_limit = denoise_spin_limit();
  plan.params.skip_arrival = denoise_skip_arrival();
  plan.zero_base = zero_base;
  plan.zero_bytes = zero_bytes;
  Op folded;
  folded.name = "action.denoise";
  folded.stage = ops_[first].stage;
  folded.launch = [plan](cudaStream_t s) { return denoise_plan_launch(plan, s); };
  ops_.erase(ops_.begin() + static_cast<std::ptrdiff_t>(first), ops_.end());
  ops_.push_back(std::move(folded));
  return kPi05Ok;
}

int PreparedGraph::build_styles() {
  // Runs the style pre-pass once, eagerly, into d_styles_ (outside the replayed graph, as
  // the reference does at capture time: crates/apxinf-model/src/pi05/runtime.rs:691-693).
  const ModelConfig& c = e_->cfg();
  const int aw = c.action.width, half = aw / 2;
  std::vector<uint16_t> emb(static_cast<size_t>(S_) * aw);
  for (int step = 0; step < S_; ++step) {
    const float time = 1.0f - static_cast<float>(step) / static_cast<float>(S_);
    for (int i = 0; i < half; ++i) {
      const double fraction = half == 1 ? 0.0 : static_cast<double>(i) / (half - 1);
      const double period = static_cast<double>(c.time_min_period) *
                            std::pow(static_cast<double>(c.time_max_period) /
                                         static_cast<double>(c.time_min_period),
                                     fraction);
      const double phase = static_cast<double>(time) * 6.283185307179586476925286766559 / period;
      emb[(size_t)step * aw + i] = bf16_bits(static_cast<float>(std::sin(phase)));
      emb[(size_t)step * aw + half + i] = bf16_bits(static_cast<float>(std::cos(phase)));
    }
  }
  PI05_CUDA(cudaMemcpyAsync(d_time_emb_, emb.data(), emb.size() * 2, cudaMemcpyHostToDevice, e_->stream()));
  PI05_CUDA(cudaStreamSynchronize(e_->stream()));
  return kPi05Ok;
}

int PreparedGraph::prepare() {
  const ModelConfig& c = e_->cfg();
  if (T_ <= 0 || T_ > c.max_token_len || B_ <= 0 || P_ + H_ > 1024) return kPi05ErrInvalidValue;
  PI05_CUDA(cudaSetDevice(e_->device()));
  // pass 1: measure the arena; pass 2: styles-only launch list; pass 3: the forward.
  arena_.reset(nullptr, 0);
  styles_only_ = false;
  PI05_TRY(build(true));
  const size_t need = arena_.used() + 4096;
  PI05_CUDA(cudaMalloc(reinterpret_cast<void**>(&arena_base_), need));
  PI05_CUDA(cudaMemsetAsync(arena_base_, 0, need, e_->stream()));
  PI05_CUDA(cudaMallocHost(reinterpret_cast<void**>(&h_out_), (size_t)B_ * H_ * c.action_dim * 2));

  arena_.reset(arena_base_, need);
  styles_only_ = true;
  PI05_TRY(build(false));
  PI05_TRY(build_styles());
  PI05_TRY(run_eager());
  PI05_TRY(sync());

  arena_.reset(arena_base_, need);
  styles_only_ = false;
  PI05_TRY(build(false));
  return kPi05Ok;
}

int PreparedGraph::run_eager() {
  PI05_CUDA(cudaSetDevice(e_->device()));
  for (const Op& op : ops_) {
    PI05_CUDA(launch_op(op, e_->stream()));
  }
  return kPi05Ok;
}

int PreparedGraph::capture() {
  PI05_CUDA(cudaSetDevice(e_->device()));
  if (exec_ != nullptr) return kPi05Ok;
  PI05_CUDA(cudaStreamBeginCapture(e_->stream(), cudaStreamCaptureModeThreadLocal));
  const int rc = run_eager();
  cudaGraph_t graph = nullptr;
  const cudaError_t end = cudaStreamEndCapture(e_->stream(), &graph);
  if (rc != kPi05Ok) {
    if (graph != nullptr) cudaGraphDestroy(graph);
    return rc;
  }
  PI05_CUDA(end);
  graph_ = graph;
  PI05_CUDA(cudaGraphInstantiate(&exec_, graph_, 0));
  return kPi05Ok;
}

int PreparedGraph::replay() {
  if (exec_ == nullptr) return kPi05ErrInvalidValue;
  PI05_CUDA(cudaGraphLaunch(exec_, e_->stream()));
  return kPi05Ok;
}

int PreparedGraph::sync() {
  PI05_CUDA(cudaStreamSynchronize(e_->stream()));
  int status = 0;
  PI05_CUDA(cudaMemcpy(&status, e_->status(), 4, cudaMemcpyDeviceToHost));
  if (status != 0) {
    cudaMemset(e_->status(), 0, 4);
    return kPi05ErrDeviceTimeout;
  }
  return kPi05Ok;
}

int PreparedGraph::update_patch_inputs(const float* patches, const uint32_t* tokens,
                                       const uint16_t* noise_bf16) {
  const ModelConfig& c = e_->cfg();
  if (patches == nullptr || tokens == nullptr || noise_bf16 == nullptr || d_patches_in_ == nullptr) {
    return kPi05ErrInvalidValue;
  }
  PI05_CUDA(cudaSetDevice(e_->device()));
  cudaStream_t s = e_->stream();
  const size_t patch_floats =
      (size_t)B_ * c.num_views * c.patches_per_view() * 3 * c.patch_size * c.patch_size;
  PI05_CUDA(cudaMemcpyAsync(d_patches_in_, patches, patch_floats * sizeof(float), cudaMemcpyHostToDevice, s));
  PI05_CUDA(cudaMemcpyAsync(d_tokens_, tokens, (size_t)B_ * T_ * 4, cudaMemcpyHostToDevice, s));
  PI05_CUDA(cudaMemcpyAsync(d_noise_, noise_bf16, (size_t)B_ * H_ * c.action_dim * 2, cudaMemcpyHostToDevice, s));
  return kPi05Ok;
}

int PreparedGraph::update_inputs(const uint8_t* images, const uint32_t* tokens,
                                 const uint16_t* noise_bf16) {
  const ModelConfig& c = e_->cfg();
  if (images == nullptr || tokens == nullptr || noise_bf16 == nullptr) return kPi05ErrInvalidValue;
  if (d_patches_in_ != nullptr) return kPi05ErrInvalidValue;  // this graph takes patches
  PI05_CUDA(cudaSetDevice(e_->device()));
  cudaStream_t s = e_->stream();
  PI05_CUDA(cudaMemcpyAsync(d_images_, images, (size_t)B_ * c.num_views * c.image_size * c.image_size * 3, cudaMemcpyHostToDevice, s));
  PI05_CUDA(cudaMemcpyAsync(d_tokens_, tokens, (size_t)B_ * T_ * 4, cudaMemcpyHostToDevice, s));
  PI05_CUDA(cudaMemcpyAsync(d_noise_, noise_bf16, (size_t)B_ * H_ * c.action_dim * 2, cudaMemcpyHostToDevice, s));
  return kPi05Ok;
}

int PreparedGraph::output(float* host_f32) {
  const ModelConfig& c = e_->cfg();
  if (host_f32 == nullptr) return kPi05ErrInvalidValue;
  const size_t count = (size_t)B_ * H_ * c.action_dim;
  PI05_CUDA(cudaMemcpyAsync(h_out_, d_state_, count * 2, cudaMemcpyDeviceToHost, e_->stream()));
  PI05_TRY(sync());
  for (size_t i = 0; i < count; ++i) host_f32[i] = bf16_to_float(h_out_[i]);
  return kPi05Ok;
}

int PreparedGraph::time_replays(int iterations, float* ms_each) {
  if (iterations <= 0 || ms_each == nullptr || exec_ == nullptr) return kPi05ErrInvalidValue;
  EventSet events;
  cudaEvent_t begin = nullptr, end = nullptr;
  PI05_TRY(events.add(&begin));
  PI05_TRY(events.add(&end));
  int rc = kPi05Ok;
  for (int i = 0; i < iterations && rc == kPi05Ok; ++i) {
    rc = record_cuda(cudaEventRecord(begin, e_->stream()));
    if (rc == kPi05Ok) rc = replay();
    if (rc == kPi05Ok) rc = record_cuda(cudaEventRecord(end, e_->stream()));
    if (rc == kPi05Ok) rc = record_cuda(cudaEventSynchronize(end));
    if (rc == kPi05Ok) rc = record_cuda(cudaEventElapsedTime(&ms_each[i], begin, end));
  }
  const int status = sync();  // also clears a device-timeout status for the next caller
  return rc != kPi05Ok ? rc : status;
}

int PreparedGraph::stage_times(float* ms3) {
  if (ms3 == nullptr) return kPi05ErrInvalidValue;
  PI05_CUDA(cudaSetDevice(e_->device()));
  EventSet events;
  cudaEvent_t ev[4] = {};
  for (auto& e : ev) PI05_TRY(events.add(&e));
  int stage = 0;
  int rc = record_cuda(cudaEventRecord(ev[0], e_->stream()));
  for (const Op& op : ops_) {
    if (rc != kPi05Ok) break;
    while (op.stage > stage && stage < 2 && rc == kPi05Ok) {
      rc = record_cuda(cudaEventRecord(ev[++stage], e_->stream()));
    }
    if (rc == kPi05Ok) rc = record_cuda(launch_op(op, e_->stream()));
  }
  while (stage < 2 && rc == kPi05Ok) rc = record_cuda(cudaEventRecord(ev[++stage], e_->stream()));
  if (rc == kPi05Ok) rc = record_cuda(cudaEventRecord(ev[3], e_->stream()));
  const int status = sync();
  if (rc == kPi05Ok) rc = status;
  for (int i = 0; i < 3 && rc == kPi05Ok; ++i) {
    rc = record_cuda(cudaEventElapsedTime(&ms3[i], ev[i], ev[i + 1]));
  }
  return rc;
}

int PreparedGraph::time_launches(const char* name, float* mean_ms, int* count) {
  if (name == nullptr || mean_ms == nullptr || count == nullptr) return kPi05ErrInvalidValue;
  *count = 0;
  *mean_ms = 0.0f;
  PI05_CUDA(cudaSetDevice(e_->device()));
  EventSet events;
  std::vector<cudaEvent_t> pairs;
  int rc = kPi05Ok;
  for (const Op& op : ops_) {
    if (rc != kPi05Ok) break;
    const bool timed = op.name == name;
    cudaEvent_t a = nullptr, b = nullptr;
    if (timed) {
      rc = events.add(&a);
      if (rc == kPi05Ok) rc = events.add(&b);
      if (rc == kPi05Ok) rc = record_cuda(cudaEventRecord(a, e_->stream()));
      if (rc != kPi05Ok) break;
    }
    rc = record_cuda(launch_op(op, e_->stream()));
    if (timed && rc == kPi05Ok) {
      rc = record_cuda(cudaEventRecord(b, e_->stream()));
      pairs.push_back(a);
      pairs.push_back(b);
    }
  }
  const int status = sync();
  if (rc == kPi05Ok) rc = status;
  double total = 0.0;
  for (size_t i = 0; i + 1 < pairs.size() && rc == kPi05Ok; i += 2) {
    float ms = 0.0f;
    rc = record_cuda(cudaEventElapsedTime(&ms, pairs[i], pairs[i + 1]));
    total += ms;
  }
  if (rc != kPi05Ok) return rc;
  *count = static_cast<int>(pairs.size() / 2);
  *mean_ms = *count > 0 ? static_cast<float>(total / *count) : 0.0f;
  return rc;
}

int PreparedGraph::read_tensor(const char* name, void* host, size_t capacity, size_t* actual) {
  auto it = tensors_.find(name);
  if (it == tensors_.end()) return kPi05ErrInvalidValue;
  if (actual != nullptr) *actual = it->second.second;
  if (host == nullptr) return kPi05Ok;
  if (capacity < it->second.second) return kPi05ErrInvalidValue;
  PI05_CUDA(cudaSetDevice(e_->device()));
  PI05_CUDA(cudaStreamSynchronize(e_->stream()));
  PI05_CUDA(cudaMemcpy(host, it->second.first, it->second.second, cudaMemcpyDeviceToHost));
  return kPi05Ok;
}

}  // namespace pi05
