// Host side of the PI0.5 policy forward: device weights, the prepared (shape
// fixed) launch list, CUDA-graph capture and replay. One Engine per (GPU, host
// thread); engines share nothing.
//
// Mirrors, in C++, the reference runtimes
//   crates/apxinf-model/src/pi05/bf16_runtime.rs:132-575 (Pi05Bf16CudaRuntime),
//   crates/apxinf-model/src/pi05/runtime.rs:261-818      (Pi05CudaRuntime, FP8),
//   crates/apxinf-model/src/pi05/int8_runtime.rs         (Pi05Int8CudaRuntime),
// their captured-graph objects (bf16_runtime.rs:27-123) and the arena of
//   crates/apxinf-cuda/src/workspace.rs:13-251.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "denoise_persistent.h"
#include "fmha.h"
#include "gemm.h"

namespace pi05 {

enum Precision : int { kPrecBf16 = 0, kPrecFp8 = 1, kPrecInt8 = 2 };

struct GemmaDims {
  int width, depth, mlp_dim, num_heads, num_kv_heads, head_dim;
};

struct ModelConfig {
  int action_dim = 32, action_horizon = 10, max_token_len = 200, num_flow_steps = 10;
  int num_views = 2, image_size = 224, patch_size = 14;
  int vision_width = 1152, vision_depth = 27, vision_mlp_dim = 4304, vision_heads = 16,
      vision_head_dim = 72;
  int vocab_size = 257152;
  float rms_norm_eps = 1e-6f, layer_norm_eps = 1e-6f, rope_theta = 10000.0f;
  float time_min_period = 4e-3f, time_max_period = 4.0f;
  GemmaDims language{2048, 18, 16384, 8, 1, 256};
  GemmaDims action{1024, 18, 4096, 8, 1, 256};

  int patches_per_view() const { return (image_size / patch_size) * (image_size / patch_size); }
  int patch_width() const { return 3 * patch_size * patch_size; }
  int validate() const;
};

// One (possibly packed) projection in GEMM-operand layout.
struct Linear {
  void* w = nullptr;          // [n, ldk] bf16 | e4m3 | int8, K-major
  float* col_scale = nullptr; // [n] (fp8 / int8)
  void* bias = nullptr;       // bf16 [n] or null
  int n = 0, k = 0;
  long long ldk = 0;
};

// A GEMM input as the active precision wants it.
struct Act {
  void* data = nullptr;       // bf16 | e4m3 | int8 [rows, ld]
  float* row_scale = nullptr; // int8 with dynamic scales: one per row
  void* wide = nullptr;       // int8 only: bf16 staging the quantiser reads
  long long ld = 0;
  int rows = 0;
  float scale = 1.0f;         // static activation scale of this tensor (fp8, static int8)
};

struct Op {
  std::string name;
  int stage = 0;
  bool is_gemm = false;
  GemmPlan plan;
  bool is_fmha = false;
  FmhaPlan fmha;
  std::function<cudaError_t(cudaStream_t)> launch;
};

constexpr int kLayoutPatches = 2;

class Arena {
 public:
  void reset(uint8_t* base, size_t capacity) { base_ = base; capacity_ = capacity; used_ = 0; }
  void* alloc(size_t bytes) {
    const size_t aligned = (bytes + 255) & ~static_cast<size_t>(255);
    void* p = base_ == nullptr ? reinterpret_cast<void*>(static_cast<uintptr_t>(256 + used_))
                               : static_cast<void*>(base_ + used_);
    used_ += aligned;
    return p;
  }
  size_t used() const { return used_; }
  size_t capacity() const { return capacity_; }
  bool measuring() const { return base_ == nullptr; }

 private:
  uint8_t* base_ = nullptr;
  size_t capacity_ = 0, used_ = 0;
};

class Engine;

// One prepared inference: fixed token count, image layout and batch.
class PreparedGraph {
 public:
  // image_layout: 0 = NHWC u8 images, 1 = NCHW u8 images, 2 = ready-made fp32 patch rows
  PreparedGraph(Engine* engine, int token_count, int image_layout, int batch);
  ~PreparedGraph();
  int prepare();                       // allocate, plan every launch, compute the styles
  int capture();                       // record the launch list into one CUDA graph
  int run_eager();                     // same launch list, no graph
  int replay();                        // cudaGraphLaunch
  int sync();                          // stream synchronize + device status word
  int update_inputs(const uint8_t* images, const uint32_t* tokens, const uint16_t* noise_bf16);
  // graphs captured with the patch layout: fp32 patch rows instead of images
  int update_patch_inputs(const float* patches, const uint32_t* tokens, const uint16_t* noise_bf16);
  int output(float* host_f32);         // [batch, horizon, action_dim]
  int time_replays(int iterations, float* ms_each);
  int stage_times(float* ms3);
  int time_launches(const char* name, float* mean_ms, int* count);
  int read_tensor(const char* name, void* host, size_t capacity, size_t* actual);
  size_t workspace_bytes() const { return arena_.capacity(); }
  size_t workspace_used() const { return arena_.used(); }
  int num_launches() const { return static_cast<int>(ops_.size()); }
  int batch() const { return B_; }
  const std::vector<Op>& ops() const { return ops_; }

 private:
  friend class Engine;
  int build(bool measuring);
  int build_styles();
  void add_kernel(const char* name, std::function<cudaError_t(cudaStream_t)> fn);
  // The adding launch of a K-sliced GEMM, while it is the newest op: an RMSNorm of the rows it
  // writes takes its place (one launch forms the rows and normalises them).
  struct PendingSum {
    size_t op_index = static_cast<size_t>(-1);
    const float* partials = nullptr;
    int slices = 0;
    long long count = 0;
    int cols = 0;
    const void* residual = nullptr;
    const void* bias = nullptr;
    void* out = nullptr;
  } pending_sum_;
  int add_gemm(const char* name, const GemmProblem& problem);
  int linear(const char* name, const Act& in, int rows, const Linear& w, int mode, void* out,
             long long ldc, int out_type, const void* residual, const void* gate,
             const void* pos, int pos_rows, float out_inv_scale, int nb0 = 1,
             long long a_sb0 = 0, long long out_sb0 = 0);
  // `site` names the static activation scale of the produced tensor (Engine::scale_of)
  int linear_to_act(const char* name, const Act& in, int rows, const Linear& w, int mode,
                    Act* out, const std::string& site);
  int norm_to_act(const char* name, const void* x, int rows, int cols, int kind,
                  const void* style, float eps, Act* out, const std::string& site,
                  const void* weight = nullptr, const void* bias = nullptr);
  // quantises a bf16 tensor (or passes it through) into the precision's operand form
  void quantize_to_act(const char* name, const void* bf16_src, int rows, int cols, Act* out,
                       const std::string& site);
  void quantize_attention_output(Act* out);
  Act make_act(int rows, long long ld);
  int attention(const char* name, const void* q, long long q_ld, long long q_sb0, long long q_sb1,
                const void* k, long long k_ld, long long k_sb0, long long k_sb1, const void* v,
                long long v_ld, long long v_sb0, long long v_sb1, int q_rows, int keys,
                int head_dim, int nb0, int nb1, float scale, void* logits, Act* out,
                long long out_ld, long long out_sb0, long long out_sb1);
  void note(const char* name, void* ptr, size_t bytes) { tensors_[name] = {ptr, bytes}; }

  Engine* e_;
  int T_, nchw_, B_;
  int V_, P_, H_, S_;
  Arena arena_;
  uint8_t* arena_base_ = nullptr;
  std::vector<Op> ops_;
  int stage_ = 0;
  bool measuring_ = false;
  std::vector<DenoiseStage> denoise_stages_;  // host copy of the persistent kernel's stage table
  int fold_denoise(size_t first, void* table, int capacity, unsigned* zero_base, size_t zero_bytes,
                   float* scratch, int tiles);
  bool styles_only_ = false;
  cudaGraph_t graph_ = nullptr;
  cudaGraphExec_t exec_ = nullptr;
  std::unordered_map<std::string, std::pair<void*, size_t>> tensors_;
  // inputs / outputs
  uint8_t* d_images_ = nullptr;
  float* d_patches_in_ = nullptr;  // patch layout only
  uint32_t* d_tokens_ = nullptr;
  void* d_noise_ = nullptr;
  void* d_state_ = nullptr;
  void* d_styles_ = nullptr;
  void* d_time_emb_ = nullptr;
  void* d_partials_ = nullptr;      // split-K scratch shared by every GEMM of the graph
  int* d_tile_counters_ = nullptr;
  void* d_k_partials_ = nullptr;    // fp32 [<= 4][rows][width] of a K-sliced GEMM, or null
  size_t k_partials_bytes_ = 0;
  uint16_t* h_out_ = nullptr;  // pinned
};

enum WeightDist : int { kWeightsLcg = 0, kWeightsNormal = 1 };
enum Int8Activations : int { kInt8Dynamic = 0, kInt8Static = 1 };

// A host tensor handed to the engine instead of the synthetic stream: bf16 bits or f32, linear weights
// in the reference's final [in, out] orientation, named as the synthetic layout names them
// ("vision.3.q.weight", "language.0.gate.weight", "action.2.input_style.bias", "token_embedding",
// ...), plus the LayerNorm parameters "vision.<i>.norm1.weight" / ".bias", "vision.<i>.norm2.*",
// "vision.post_norm.*" (absent = identity).
// f32 tensors (the reference's folded Gemma projections are f32,
// crates/apxinf-model/src/pi05/weights.rs:584-601) are quantised from f32 by the FP8 / INT8
// precisions, as the reference does, and rounded to bf16 (nearest even) where bf16 is stored.
struct HostTensor {
  const void* data = nullptr;
  size_t elements = 0;
  bool f32 = false;
};

struct EngineOptions {
  int precision = kPrecBf16;
  int device = 0;
  uint64_t seed = 0;
  float act_scale = 1.0f;          // uniform static activation scale (sites not set by name)
  int weight_dist = kWeightsLcg;   // reference LCG (uniform +-0.02) | seeded N(0, 0.02)
  int int8_activations = kInt8Dynamic;  // per-row dynamic (reference) | static per-tensor
};

class Engine {
 public:
  Engine(const ModelConfig& cfg, const EngineOptions& options);
  // weights from host tensors instead of the synthetic generator (call before init)
  void set_host_tensors(std::unordered_map<std::string, HostTensor> tensors) {
    host_tensors_ = std::move(tensors);
    from_host_ = true;
  }
  ~Engine();
  int init();  // stream, status word, rope tables, synthetic weights
  const ModelConfig& cfg() const { return cfg_; }
  int precision() const { return prec_; }
  cudaStream_t stream() const { return stream_; }
  int* status() const { return status_; }
  int device() const { return device_; }
  float act_scale() const { return act_scale_; }
  // Static activation scale of a GEMM-input site, named as the reference's calibration table
  // (crates/apxinf-model/src/pi05/runtime.rs:35-81): "vision.patch_input",
  // "vision.layers.<i>.{attention_norm,attention_output,mlp_norm,mlp_activation}",
  // "vision.post_norm", "language.layers.<i>.<...>", "action.input", "time.input",
  // "time.hidden", "action.conditioning", "action.layers.<i>.<...>", "action.final_norm".
  float scale_of(const std::string& site) const;
  int set_scale(const std::string& site, float value);  // before capture; unknown names are refused
  bool static_int8() const { return prec_ == kPrecInt8 && int8_static_; }
  // the precision takes byte operands with one static scale per tensor
  bool static_scales() const { return prec_ == kPrecFp8 || static_int8(); }
  size_t weight_bytes() const { return weight_bytes_; }
  int read_weight(const char* name, void* host, size_t capacity, size_t* actual);

  // LayerNorm gamma / beta (bf16 device vectors; null = 1 / 0, the synthetic weights)
  struct LayerNormParams { void* weight = nullptr; void* bias = nullptr; };
  struct VisionBlock { Linear qkv, o, fc1, fc2; LayerNormParams norm1, norm2; };
  LayerNormParams vision_post_norm;
  struct LanguageLayer { Linear qkv, o, gate_up, down; };
  struct ActionLayer { Linear input_style, qkv, o, post_style, gate_up, down; };
  std::vector<VisionBlock> vision;
  Linear patch, projector;
  void* position_embedding = nullptr;
  void* token_embedding = nullptr;
  std::vector<LanguageLayer> language;
  std::vector<ActionLayer> action;
  Linear final_style, action_in, action_out, time_in, time_out;
  float* rope_cos = nullptr;
  float* rope_sin = nullptr;
  int rope_positions = 0;

 private:
  struct Part { const char* suffix; int k, n; bool bias; };
  int make_linear(const std::string& prefix, const std::vector<std::string>& parts, int k,
                  const std::vector<int>& ns, bool bias, bool interleave, Linear* out);
  void* dmalloc(size_t bytes);
  void release(void* p);  // frees one tracked allocation early
  // the tensor `name` into dst (bf16): the next `count` stream elements, or the host tensor
  int fetch(const std::string& name, void* dst, long long count, bool as_f32 = false);
  int fetch_layer_norm(const std::string& prefix, int width, LayerNormParams* out);
  std::unordered_map<std::string, HostTensor> host_tensors_;
  bool from_host_ = false;
  std::string missing_tensor_;  // name of the host tensor a failed init wanted

 public:
  const std::string& missing_tensor() const { return missing_tensor_; }

 private:
  ModelConfig cfg_;
  int prec_, device_;
  uint64_t seed_;
  float act_scale_;
  int weight_dist_ = kWeightsLcg;
  bool int8_static_ = false;
  std::unordered_map<std::string, float> site_scales_;  // every valid site, current value
  cudaStream_t stream_ = nullptr;
  int* status_ = nullptr;
  uint64_t cursor_ = 0;  // element offset in the synthetic stream
  void* tmp_src_ = nullptr;
  void* tmp_stage_ = nullptr;
  void* tmp_convert_ = nullptr;  // host tensors whose type differs from the staging type, by chunk
  bool wide_staging() const { return from_host_ && prec_ != kPrecBf16; }
  size_t tmp_src_bytes_ = 0, tmp_stage_bytes_ = 0;
  size_t weight_bytes_ = 0;
  std::vector<void*> allocations_;
  std::unordered_map<std::string, std::pair<void*, size_t>> named_;
};

int record_cuda(cudaError_t error);

}  // namespace pi05
