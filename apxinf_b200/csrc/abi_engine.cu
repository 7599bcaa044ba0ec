// Engine-level extern "C" entry points (declared in include/pi05_b200.h).
#include <new>

#include "../../include/pi05_b200.h"
#include <cmath>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "engine.h"

struct Pi05Engine {
  pi05::Engine* impl;
};
struct Pi05Graph {
  pi05::PreparedGraph* impl;
};

namespace {

pi05::ModelConfig to_internal(const Pi05ModelConfig& c) {
  pi05::ModelConfig m;
  m.action_dim = c.action_dim;
  m.action_horizon = c.action_horizon;
  m.max_token_len = c.max_token_len;
  m.num_flow_steps = c.num_flow_steps;
  m.num_views = c.num_views;
  m.image_size = c.image_size;
  m.patch_size = c.patch_size;
  m.vision_width = c.vision_width;
  m.vision_depth = c.vision_depth;
  m.vision_mlp_dim = c.vision_mlp_dim;
  m.vision_heads = c.vision_heads;
  m.vision_head_dim = c.vision_head_dim;
  m.vocab_size = c.vocab_size;
  m.rms_norm_eps = c.rms_norm_eps;
  m.layer_norm_eps = c.layer_norm_eps;
  m.rope_theta = c.rope_theta;
  m.time_min_period = c.time_min_period;
  m.time_max_period = c.time_max_period;
  auto gemma = [](const Pi05Gemma& g) {
    return pi05::GemmaDims{g.width, g.depth, g.mlp_dim, g.num_heads, g.num_kv_heads, g.head_dim};
  };
  m.language = gemma(c.language);
  m.action = gemma(c.action_expert);
  return m;
}

}  // namespace

extern "C" void pi05_default_config(Pi05ModelConfig* c) {
  if (c == nullptr) return;
  const pi05::ModelConfig m;
  c->action_dim = m.action_dim;
  c->action_horizon = m.action_horizon;
  c->max_token_len = m.max_token_len;
  c->num_flow_steps = m.num_flow_steps;
  c->num_views = m.num_views;
  c->image_size = m.image_size;
  c->patch_size = m.patch_size;
  c->vision_width = m.vision_width;
  c->vision_depth = m.vision_depth;
  c->vision_mlp_dim = m.vision_mlp_dim;
  c->vision_heads = m.vision_heads;
  c->vision_head_dim = m.vision_head_dim;
  c->vocab_size = m.vocab_size;
  c->rms_norm_eps = m.rms_norm_eps;
  c->layer_norm_eps = m.layer_norm_eps;
  c->rope_theta = m.rope_theta;
  c->time_min_period = m.time_min_period;
  c->time_max_period = m.time_max_period;
  auto gemma = [](const pi05::GemmaDims& g) {
    return Pi05Gemma{g.width, g.depth, g.mlp_dim, g.num_heads, g.num_kv_heads, g.head_dim};
  };
  c->language = gemma(m.language);
  c->action_expert = gemma(m.action);
}

namespace pi05 {
extern thread_local std::string g_last_cuda_error;
}

namespace {

bool g_force_capture_failure = false;  // test hook of the runtime frontend's eager fallback

int create_engine(const Pi05ModelConfig* config, const Pi05EngineOptions* options,
                  std::unordered_map<std::string, pi05::HostTensor>* tensors, Pi05Engine** out) {
  if (config == nullptr || options == nullptr || out == nullptr || options->device < 0) {
    return pi05::kPi05ErrInvalidValue;
  }
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || options->device >= count) {
    return pi05::record_cuda(cudaErrorNoDevice);
  }
  pi05::EngineOptions o;
  o.precision = options->dtype;
  o.device = options->device;
  o.seed = options->seed;
  o.weight_dist = options->weight_dist;
  o.int8_activations = options->int8_activations;
  // the uniform scale matters to the precisions with static activation scales only
  const bool uses_scale = options->dtype == PI05_DTYPE_FP8 ||
                          (options->dtype == PI05_DTYPE_INT8 &&
                           options->int8_activations == PI05_INT8_ACT_STATIC);
  o.act_scale = uses_scale ? options->act_scale : 1.0f;
  auto* impl = new (std::nothrow) pi05::Engine(to_internal(*config), o);
  if (impl == nullptr) return pi05::kPi05ErrInvalidValue;
  if (tensors != nullptr) impl->set_host_tensors(std::move(*tensors));
  const int rc = impl->init();
  if (rc != pi05::kPi05Ok) {
    if (!impl->missing_tensor().empty()) {
      pi05::g_last_cuda_error = "missing or mis-sized weight tensor `" + impl->missing_tensor() + "`";
    }
    delete impl;
    return rc;
  }
  *out = new Pi05Engine{impl};
  return pi05::kPi05Ok;
}

}  // namespace

extern "C" int pi05_engine_create_ex(const Pi05ModelConfig* config, const Pi05EngineOptions* options,
                                     Pi05Engine** out) {
  return create_engine(config, options, nullptr, out);
}

extern "C" int pi05_engine_create_from_tensors(const Pi05ModelConfig* config,
                                               const Pi05EngineOptions* options,
                                               const Pi05HostTensor* tensors, int32_t count,
                                               Pi05Engine** out) {
  pi05::g_last_cuda_error.clear();  // a message left by this call names the offending tensor
  if (tensors == nullptr || count <= 0) return pi05::kPi05ErrInvalidValue;
  std::unordered_map<std::string, pi05::HostTensor> table;
  for (int32_t i = 0; i < count; ++i) {
    if (tensors[i].name == nullptr || tensors[i].data == nullptr ||
        (tensors[i].dtype != PI05_TENSOR_BF16 && tensors[i].dtype != PI05_TENSOR_F32)) {
      return pi05::kPi05ErrInvalidValue;
    }
    table[tensors[i].name] = pi05::HostTensor{tensors[i].data, static_cast<size_t>(tensors[i].elements),
                                              tensors[i].dtype == PI05_TENSOR_F32};
  }
  return create_engine(config, options, &table, out);
}

extern "C" int pi05_engine_create(const Pi05ModelConfig* config, int32_t dtype, int32_t device,
                                  uint64_t seed, float fp8_act_scale, Pi05Engine** out) {
  Pi05EngineOptions options = {};
  options.dtype = dtype;
  options.device = device;
  options.seed = seed;
  options.act_scale = fp8_act_scale;
  options.weight_dist = PI05_WEIGHTS_LCG;
  options.int8_activations = PI05_INT8_ACT_DYNAMIC;
  return pi05_engine_create_ex(config, &options, out);
}

extern "C" int pi05_set_tuning(const char* name, int32_t value) {
  if (name == nullptr) return pi05::kPi05ErrInvalidValue;
  const std::string key(name);
  if (key == "programmatic_dependent_launch") {
    pi05::set_pdl_enabled(value != 0);
  } else if (key == "fuse_small_rows") {
    pi05::set_fuse_small_rows_enabled(value != 0);
  } else if (key == "attention_cluster") {
    pi05::set_fmha_rows_cluster_enabled(value != 0);
  } else if (key == "fuse_norms") {
    pi05::set_fuse_norms_enabled(value != 0);
  } else if (key == "persistent_denoise") {
    pi05::set_persistent_denoise_enabled(value != 0);
  } else if (key == "denoise_wait_limit_polls") {
    pi05::set_denoise_spin_limit(value);
  } else if (key == "denoise_skip_arrival") {
    pi05::set_denoise_skip_arrival(value);
  } else if (key == "wait_limit_polls") {
    pi05::set_wait_polls(value);
  } else if (key == "drop_one_load") {
    pi05::set_drop_load_kb(value);
  } else if (key == "single_epilogue_kernels") {
    pi05::set_single_epilogue_kernels_enabled(value != 0);
  } else if (key == "force_capture_failure") {
    g_force_capture_failure = value != 0;
  } else {
    return pi05::kPi05ErrInvalidValue;
  }
  return pi05::kPi05Ok;
}

extern "C" int pi05_engine_set_activation_scale(Pi05Engine* engine, const char* site, float scale) {
  if (engine == nullptr || site == nullptr) return pi05::kPi05ErrInvalidValue;
  return engine->impl->set_scale(site, scale);
}

extern "C" float pi05_engine_activation_scale(const Pi05Engine* engine, const char* site) {
  if (engine == nullptr || site == nullptr) return 0.0f;
  return engine->impl->scale_of(site);
}

extern "C" void pi05_engine_destroy(Pi05Engine* engine) {
  if (engine == nullptr) return;
  delete engine->impl;
  delete engine;
}

extern "C" size_t pi05_engine_weight_bytes(const Pi05Engine* engine) {
  return engine == nullptr ? 0 : engine->impl->weight_bytes();
}

extern "C" int pi05_engine_read_weight(Pi05Engine* engine, const char* name, void* host,
                                       size_t capacity, size_t* actual) {
  if (engine == nullptr || name == nullptr) return pi05::kPi05ErrInvalidValue;
  return engine->impl->read_weight(name, host, capacity, actual);
}

extern "C" int pi05_engine_capture(Pi05Engine* engine, int32_t token_count, int32_t image_layout,
                                   int32_t batch, Pi05Graph** out) {
  if (engine == nullptr || out == nullptr) return pi05::kPi05ErrInvalidValue;
  *out = nullptr;
  if (image_layout != PI05_IMAGE_NHWC && image_layout != PI05_IMAGE_NCHW &&
      image_layout != PI05_IMAGE_PATCHES) {
    return pi05::kPi05ErrInvalidValue;
  }
  auto* impl = new (std::nothrow) pi05::PreparedGraph(engine->impl, token_count, image_layout, batch);
  if (impl == nullptr) return pi05::kPi05ErrInvalidValue;
  int rc = impl->prepare();
  if (rc == pi05::kPi05Ok) rc = impl->run_eager();  // warm pass before recording
  if (rc == pi05::kPi05Ok) rc = impl->sync();
  if (rc == pi05::kPi05Ok) rc = impl->capture();
  if (rc != pi05::kPi05Ok) {
    delete impl;
    return rc;
  }
  *out = new Pi05Graph{impl};
  return pi05::kPi05Ok;
}

extern "C" void pi05_graph_destroy(Pi05Graph* graph) {
  if (graph == nullptr) return;
  delete graph->impl;
  delete graph;
}

#define PI05_GRAPH_CALL(expr) (graph == nullptr ? pi05::kPi05ErrInvalidValue : graph->impl->expr)

extern "C" int pi05_graph_update_patch_inputs(Pi05Graph* graph, const float* patches,
                                              const uint32_t* token_ids, const uint16_t* noise_bf16) {
  return PI05_GRAPH_CALL(update_patch_inputs(patches, token_ids, noise_bf16));
}

extern "C" int pi05_graph_update_raw_image_inputs(Pi05Graph* graph, const uint8_t* images,
                                                  const uint32_t* token_ids,
                                                  const uint16_t* noise_bf16) {
  return PI05_GRAPH_CALL(update_inputs(images, token_ids, noise_bf16));
}
extern "C" int pi05_graph_replay(Pi05Graph* graph) { return PI05_GRAPH_CALL(replay()); }
extern "C" int pi05_graph_run_eager(Pi05Graph* graph) { return PI05_GRAPH_CALL(run_eager()); }
extern "C" int pi05_graph_sync(Pi05Graph* graph) { return PI05_GRAPH_CALL(sync()); }
extern "C" int pi05_graph_output(Pi05Graph* graph, float* host_out) {
  return PI05_GRAPH_CALL(output(host_out));
}
extern "C" int pi05_graph_time_replays(Pi05Graph* graph, int32_t iterations, float* ms_each) {
  return PI05_GRAPH_CALL(time_replays(iterations, ms_each));
}
extern "C" int pi05_graph_stage_times(Pi05Graph* graph, float* ms3) {
  return PI05_GRAPH_CALL(stage_times(ms3));
}
extern "C" int pi05_graph_time_launches(Pi05Graph* graph, const char* name, float* mean_ms,
                                        int32_t* count) {
  if (name == nullptr) return pi05::kPi05ErrInvalidValue;
  return PI05_GRAPH_CALL(time_launches(name, mean_ms, count));
}
extern "C" size_t pi05_graph_workspace_bytes(const Pi05Graph* graph) {
  return graph == nullptr ? 0 : graph->impl->workspace_bytes();
}
extern "C" size_t pi05_graph_workspace_used_bytes(const Pi05Graph* graph) {
  return graph == nullptr ? 0 : graph->impl->workspace_used();
}
extern "C" int32_t pi05_graph_num_launches(const Pi05Graph* graph) {
  return graph == nullptr ? 0 : graph->impl->num_launches();
}
extern "C" const char* pi05_graph_launch_name(const Pi05Graph* graph, int32_t index) {
  if (graph == nullptr || index < 0 || index >= graph->impl->num_launches()) return nullptr;
  return graph->impl->ops()[index].name.c_str();
}
extern "C" int pi05_graph_read_tensor(Pi05Graph* graph, const char* name, void* host,
                                      size_t capacity, size_t* actual) {
  if (name == nullptr) return pi05::kPi05ErrInvalidValue;
  return PI05_GRAPH_CALL(read_tensor(name, host, capacity, actual));
}


// ---------------------------------------------------------------------------
// Owning frontend: one cached prepared plan per (token_count, image_layout)
// (crates/apxinf-model/src/pi05/vla_runtime.rs:393-495)
// ---------------------------------------------------------------------------

struct Pi05Runtime {
  pi05::Engine* engine = nullptr;       // borrowed
  pi05::PreparedGraph* plan = nullptr;  // the most recently used shape
  int token_count = 0, image_layout = 0;
  bool graph = false;                   // false: capture was unavailable, the plan runs eagerly
  int builds = 0;
  std::vector<uint16_t> noise_bits;     // host-side dtype normalisation of the noise
};

namespace {

uint16_t to_bf16_bits(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((bits >> 16) | 0x40u);
  return static_cast<uint16_t>((bits + ((bits >> 16) & 1u) + 0x7fffu) >> 16);
}

// build_prepared (vla_runtime.rs:423-473): allocate, try to capture, fall back to eager
int build_plan(Pi05Runtime* rt, int token_count, int image_layout) {
  // the previous plan goes first: its workspace and the new one need not coexist
  delete rt->plan;
  rt->plan = nullptr;
  auto* plan = new (std::nothrow) pi05::PreparedGraph(rt->engine, token_count, image_layout, 1);
  if (plan == nullptr) return pi05::kPi05ErrInvalidValue;
  int rc = plan->prepare();
  if (rc == pi05::kPi05Ok) rc = plan->run_eager();
  if (rc == pi05::kPi05Ok) rc = plan->sync();
  if (rc != pi05::kPi05Ok) {
    delete plan;
    return rc;
  }
  const int capture_rc = g_force_capture_failure ? pi05::kPi05ErrCuda : plan->capture();
  rt->graph = capture_rc == pi05::kPi05Ok;
  rt->plan = plan;
  rt->token_count = token_count;
  rt->image_layout = image_layout;
  ++rt->builds;
  return pi05::kPi05Ok;
}

}  // namespace

extern "C" int pi05_device_sm(int32_t device) {
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return major * 10 + minor;
}

extern "C" int pi05_runtime_create(Pi05Engine* engine, Pi05Runtime** out) {
  if (engine == nullptr || out == nullptr) return pi05::kPi05ErrInvalidValue;
  *out = new Pi05Runtime();
  (*out)->engine = engine->impl;
  return pi05::kPi05Ok;
}

extern "C" void pi05_runtime_destroy(Pi05Runtime* runtime) {
  if (runtime == nullptr) return;
  delete runtime->plan;
  delete runtime;
}

extern "C" int pi05_runtime_infer(Pi05Runtime* rt, const Pi05Observation* obs, float* actions_out) {
  if (rt == nullptr || obs == nullptr || actions_out == nullptr || obs->token_ids == nullptr ||
      obs->noise == nullptr) {
    return pi05::kPi05ErrInvalidValue;
  }
  const pi05::ModelConfig& c = rt->engine->cfg();
  if (obs->token_count <= 0 || obs->token_count > c.max_token_len) return pi05::kPi05ErrInvalidValue;
  const bool patches = obs->image_layout == PI05_IMAGE_PATCHES;
  if (obs->image_layout != PI05_IMAGE_NHWC && obs->image_layout != PI05_IMAGE_NCHW && !patches) {
    return pi05::kPi05ErrInvalidValue;
  }
  if ((patches && obs->patches == nullptr) || (!patches && obs->images == nullptr)) {
    return pi05::kPi05ErrInvalidValue;
  }
  if (obs->noise_dtype != PI05_NOISE_F32 && obs->noise_dtype != PI05_NOISE_BF16) {
    return pi05::kPi05ErrInvalidValue;
  }
  if (rt->plan == nullptr || rt->token_count != obs->token_count || rt->image_layout != obs->image_layout) {
    const int rc = build_plan(rt, obs->token_count, obs->image_layout);
    if (rc != pi05::kPi05Ok) return rc;
  }
  const size_t count = static_cast<size_t>(c.action_horizon) * c.action_dim;
  const uint16_t* noise = static_cast<const uint16_t*>(obs->noise);
  if (obs->noise_dtype == PI05_NOISE_F32) {
    rt->noise_bits.resize(count);
    const float* src = static_cast<const float*>(obs->noise);
    for (size_t i = 0; i < count; ++i) rt->noise_bits[i] = to_bf16_bits(src[i]);
    noise = rt->noise_bits.data();
  }
  int rc = patches ? rt->plan->update_patch_inputs(obs->patches, obs->token_ids, noise)
                   : rt->plan->update_inputs(obs->images, obs->token_ids, noise);
  if (rc != pi05::kPi05Ok) return rc;
  rc = rt->graph ? rt->plan->replay() : rt->plan->run_eager();
  if (rc != pi05::kPi05Ok) return rc;
  return rt->plan->output(actions_out);
}

extern "C" int pi05_runtime_plan_info(const Pi05Runtime* rt, int32_t* token_count, int32_t* image_layout,
                                      int32_t* uses_graph, int32_t* builds) {
  if (rt == nullptr) return pi05::kPi05ErrInvalidValue;
  if (token_count != nullptr) *token_count = rt->plan != nullptr ? rt->token_count : 0;
  if (image_layout != nullptr) *image_layout = rt->image_layout;
  if (uses_graph != nullptr) *uses_graph = rt->plan != nullptr && rt->graph ? 1 : 0;
  if (builds != nullptr) *builds = rt->builds;
  return pi05::kPi05Ok;
}

// Stage signature of a named bf16 intermediate
// (crates/apxinf-model/examples/pi05_integrity_probe.rs:19-51).
extern "C" int pi05_graph_signature(Pi05Graph* graph, const char* name, Pi05Signature* out) {
  if (graph == nullptr || name == nullptr || out == nullptr) return pi05::kPi05ErrInvalidValue;
  size_t bytes = 0;
  int rc = graph->impl->read_tensor(name, nullptr, 0, &bytes);
  if (rc != pi05::kPi05Ok) return rc;
  std::vector<uint16_t> raw(bytes / 2);
  rc = graph->impl->read_tensor(name, raw.data(), bytes, &bytes);
  if (rc != pi05::kPi05Ok) return rc;
  auto value_at = [&](size_t i) {
    const uint32_t wide = static_cast<uint32_t>(raw[i]) << 16;
    float v;
    std::memcpy(&v, &wide, 4);
    return static_cast<double>(v);
  };
  *out = Pi05Signature{};
  out->elements = raw.size();
  double squares = 0.0;
  for (size_t i = 0; i < raw.size(); ++i) {
    const double v = value_at(i);
    out->sum += v;
    out->abs_checksum += v < 0 ? -v : v;
    squares += v * v;
    if ((v < 0 ? -v : v) > out->max_abs) out->max_abs = v < 0 ? -v : v;
  }
  out->l2 = std::sqrt(squares);
  out->sample_count = static_cast<int32_t>(raw.size() < 256 ? raw.size() : 256);
  for (int32_t i = 0; i < out->sample_count; ++i) {
    const size_t source = out->sample_count == 1 ? 0 : static_cast<size_t>(i) * (raw.size() - 1) / (out->sample_count - 1);
    out->sample[i] = static_cast<float>(value_at(source));
  }
  return pi05::kPi05Ok;
}
