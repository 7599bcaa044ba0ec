// pi05_bench — low-level latency benchmark of the PI0.5 policy forward over the C ABI.
//
// Same command line, acceptance gates and JSON report as the reference benchmark
// (crates/apxinf-model/examples/pi05_bench.rs:16-23 flags, :87-121 gates, :562-586 latency
// statistics, :1135-1174 report), so scripts written for it keep working:
//
//   pi05_bench random --dtype {bf16,fp8,int8|w8a8}
//       [--calibration uniform:SCALE] [--tactics <json>] [--views N] [--image-size N]
//       [--action-horizon N] [--action-dim N] [--num-flow-steps N] [--max-token-len N]
//       [--token-count T] [--iterations N] [--seed N] [--image-input patches|nhwc|nchw]
//       [--images-u8 <raw>] [--token-ids-u32le <raw>] [--noise-bf16-u16le <raw>]
//   additive: [--batch N] [--device N]
//
// Only the `random` source is built (synthetic weights need no checkpoint); --tactics is
// accepted and ignored (one kernel per shape class replaces the tactic database);
// `--image-input patches` feeds the same arithmetic image pattern as raw NHWC bytes, the
// patch rows being produced on the device.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "pi05_b200.h"

namespace {

struct Thresholds {
  double eager_graph_max_abs, reference_min_cosine, reference_max_relative_l2;
  bool has_reference_max_abs;
  double reference_max_abs;
};

struct Metrics {
  double cosine, max_abs, mean_abs, rmse, relative_l2;
  bool bitwise_equal;
};

Metrics measure(const std::vector<float>& actual, const std::vector<float>& expected) {
  double dot = 0, aa = 0, bb = 0, max_abs = 0, sum_abs = 0, sum_sq = 0;
  bool equal = true;
  for (size_t i = 0; i < actual.size(); ++i) {
    const double a = actual[i], b = expected[i], d = a - b;
    dot += a * b;
    aa += a * a;
    bb += b * b;
    max_abs = std::max(max_abs, std::fabs(d));
    sum_abs += std::fabs(d);
    sum_sq += d * d;
    equal = equal && std::memcmp(&actual[i], &expected[i], 4) == 0;
  }
  const double n = static_cast<double>(actual.size());
  Metrics m;
  m.cosine = (aa > 0 && bb > 0) ? dot / std::sqrt(aa * bb) : 1.0;
  m.max_abs = max_abs;
  m.mean_abs = sum_abs / n;
  m.rmse = std::sqrt(sum_sq / n);
  m.relative_l2 = std::sqrt(sum_sq) / std::max(std::sqrt(bb), 1e-30);
  m.bitwise_equal = equal;
  return m;
}

std::string latency_json(std::vector<double> ms) {
  std::sort(ms.begin(), ms.end());
  const double n = static_cast<double>(ms.size());
  double mean = 0;
  for (double v : ms) mean += v;
  mean /= n;
  double var = 0;
  for (double v : ms) var += (v - mean) * (v - mean);
  var /= n;
  auto pct = [&](double f) { return ms[static_cast<size_t>(std::llround((ms.size() - 1) * f))]; };
  char buf[512];
  std::snprintf(buf, sizeof buf,
                "{\"min\": %.6f, \"p50\": %.6f, \"p95\": %.6f, \"max\": %.6f, \"mean\": %.6f, "
                "\"standard_deviation\": %.6f}",
                ms.front(), pct(0.50), pct(0.95), ms.back(), mean, std::sqrt(var));
  return buf;
}

bool read_file(const std::string& path, std::vector<uint8_t>* out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  out->assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
  return true;
}

int fail(const std::string& message) {
  std::fprintf(stderr,
               "%s\nusage: pi05_bench <checkpoint-or-index|random> --dtype {bf16,fp8,int8} "
               "[--calibration <json|uniform:SCALE>] [--tactics <json>] [--views N] "
               "[--image-size N] [--action-horizon N] [--action-dim N] [--num-flow-steps N] "
               "[--max-token-len N] [--token-count T] [--iterations N] [--seed N] "
               "[--image-input patches|nhwc|nchw] [--reference <json>] [--min-cosine C] "
               "[--images-u8 <raw>] [--token-ids-u32le <raw>] [--noise-bf16-u16le <raw>] "
               "[--batch N] [--device N]\n",
               message.c_str());
  return 1;
}

std::string json_string_or_null(const std::string& s) { return s.empty() ? "null" : "\"" + s + "\""; }

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) return fail("missing <checkpoint-or-index|random>");
  const std::string source = argv[1];
  std::string dtype_spec, calibration, tactics, reference, image_input, images_u8, token_ids_path,
      noise_path;
  int views = -1, image_size = -1, horizon = -1, action_dim = -1, flow_steps = -1, max_token_len = -1;
  int token_count = 200, iterations = 30, batch = 1, device = 0;
  unsigned long long seed = 0;
  double min_cosine = -1;
  for (int i = 2; i < argc; ++i) {
    const std::string flag = argv[i];
    auto value = [&](std::string* out) -> bool {
      if (i + 1 >= argc) return false;
      *out = argv[++i];
      return true;
    };
    std::string v;
    auto as_int = [&](int* out) -> bool {
      if (!value(&v)) return false;
      char* end = nullptr;
      const long parsed = std::strtol(v.c_str(), &end, 10);
      if (end == v.c_str() || *end != '\0' || parsed < 0) return false;
      *out = static_cast<int>(parsed);
      return true;
    };
    bool ok = true;
    if (flag == "--dtype") ok = value(&dtype_spec);
    else if (flag == "--calibration") ok = value(&calibration);
    else if (flag == "--tactics") ok = value(&tactics);
    else if (flag == "--views") ok = as_int(&views);
    else if (flag == "--image-size") ok = as_int(&image_size);
    else if (flag == "--action-horizon") ok = as_int(&horizon);
    else if (flag == "--action-dim") ok = as_int(&action_dim);
    else if (flag == "--num-flow-steps") ok = as_int(&flow_steps);
    else if (flag == "--max-token-len") ok = as_int(&max_token_len);
    else if (flag == "--token-count") ok = as_int(&token_count);
    else if (flag == "--iterations") ok = as_int(&iterations);
    else if (flag == "--batch") ok = as_int(&batch);
    else if (flag == "--device") ok = as_int(&device);
    else if (flag == "--seed") { ok = value(&v); if (ok) seed = std::strtoull(v.c_str(), nullptr, 10); }
    else if (flag == "--reference") ok = value(&reference);
    else if (flag == "--min-cosine") { ok = value(&v); if (ok) min_cosine = std::atof(v.c_str()); }
    else if (flag == "--image-input") ok = value(&image_input);
    else if (flag == "--images-u8") ok = value(&images_u8);
    else if (flag == "--token-ids-u32le") ok = value(&token_ids_path);
    else if (flag == "--noise-bf16-u16le") ok = value(&noise_path);
    else return fail("unknown argument " + flag);
    if (!ok) return fail("missing or invalid value for " + flag);
  }
  int dtype;
  std::string precision;
  Thresholds th;
  if (dtype_spec == "bf16") { dtype = PI05_DTYPE_BF16; precision = "bf16"; th = {1e-2, 0.999, 0.05, false, 0}; }
  else if (dtype_spec == "fp8") { dtype = PI05_DTYPE_FP8; precision = "fp8"; th = {1e-3, 0.997, 0.10, false, 0}; }
  else if (dtype_spec == "int8" || dtype_spec == "w8a8") { dtype = PI05_DTYPE_INT8; precision = "int8_w8a8"; th = {1e-2, 0.995, 0.10, true, 0.125}; }
  else if (dtype_spec.empty()) return fail("--dtype is required");
  else return fail("--dtype must be bf16, fp8, or int8; got " + dtype_spec);

  if (image_input.empty()) {
    const char* env = std::getenv("APXINF_PI05_IMAGE_INPUT");
    image_input = env != nullptr ? env : "patches";
  }
  int layout = PI05_IMAGE_NHWC;
  std::string input_kind;
  if (image_input == "patches") input_kind = dtype == PI05_DTYPE_FP8 ? "patches_f16" : "patches_bf16";
  else if (image_input == "nhwc") input_kind = "rgb_u8_nhwc";
  else if (image_input == "nchw") { input_kind = "rgb_u8_nchw"; layout = PI05_IMAGE_NCHW; }
  else return fail("image input must be patches, nhwc, or nchw; got " + image_input);
  const bool rgb = image_input != "patches";
  if (!images_u8.empty() && !rgb) return fail("--images-u8 requires --image-input nhwc");
  if (!images_u8.empty() && layout != PI05_IMAGE_NHWC) return fail("--images-u8 currently requires --image-input nhwc");

  const bool random = source == "random";
  const bool has_overrides = views >= 0 || image_size >= 0 || horizon >= 0 || action_dim >= 0 ||
                             flow_steps >= 0 || max_token_len >= 0;
  if (!random && has_overrides)
    return fail("architecture overrides (--views/--image-size/--action-horizon/--action-dim/"
                "--num-flow-steps/--max-token-len) are only valid with the `random` source");
  if (random && !reference.empty())
    return fail("--reference is not valid with the `random` source (no trained weights to match); "
                "eager-vs-graph integrity still runs as a self-test");
  if (dtype != PI05_DTYPE_FP8 && !calibration.empty()) return fail("--calibration only applies to --dtype fp8");
  if (dtype == PI05_DTYPE_INT8 && !tactics.empty()) return fail("--tactics only applies to --dtype bf16 or fp8");
  if (!random) return fail("checkpoint sources are not built in this library: use `random`");
  if (iterations <= 0) return fail("--iterations must be positive");

  float act_scale = 1.0f;  // FP8 without --calibration in random mode: uniform 1.0
  if (!calibration.empty()) {
    if (calibration.rfind("uniform:", 0) != 0) return fail("only --calibration uniform:SCALE is built");
    act_scale = static_cast<float>(std::atof(calibration.c_str() + 8));
    if (!(act_scale > 0.0f) || !std::isfinite(act_scale)) return fail("invalid uniform FP8 scale");
  }

  Pi05ModelConfig cfg;
  pi05_default_config(&cfg);  // two views, horizon 10, 10 flow steps, max 200 tokens
  if (views >= 0) cfg.num_views = views;
  if (image_size >= 0) cfg.image_size = image_size;
  if (horizon >= 0) cfg.action_horizon = horizon;
  if (action_dim >= 0) cfg.action_dim = action_dim;
  if (flow_steps >= 0) cfg.num_flow_steps = flow_steps;
  if (max_token_len >= 0) cfg.max_token_len = max_token_len;
  if (token_count <= 0 || token_count > cfg.max_token_len) {
    return fail("token count must be in 1..=" + std::to_string(cfg.max_token_len) + ", got " +
                std::to_string(token_count));
  }

  std::fprintf(stderr, "building synthetic %s weights (seed %llu) on device %d...\n", precision.c_str(), seed, device);
  Pi05Engine* engine = nullptr;
  int rc = pi05_engine_create(&cfg, dtype, device, seed, act_scale, &engine);
  if (rc != PI05_OK) {
    std::fprintf(stderr, "pi05_engine_create failed: %d (%s)\n", rc, pi05_last_cuda_error());
    return 2;
  }

  // inputs: the reference's arithmetic image pattern, zero ids, zero noise unless fixtures given
  const size_t image_bytes = static_cast<size_t>(cfg.num_views) * cfg.image_size * cfg.image_size * 3;
  std::vector<uint8_t> images(image_bytes * batch);
  std::vector<uint8_t> file;
  if (!images_u8.empty()) {
    if (!read_file(images_u8, &file)) return fail("cannot read " + images_u8);
    if (file.size() != image_bytes)
      return fail("--images-u8 length mismatch: expected " + std::to_string(image_bytes) + ", got " + std::to_string(file.size()));
    for (int b = 0; b < batch; ++b) std::memcpy(images.data() + b * image_bytes, file.data(), image_bytes);
  } else {
    std::vector<uint8_t> nhwc(image_bytes);
    for (size_t i = 0; i < image_bytes; ++i) nhwc[i] = static_cast<uint8_t>((i * 73 + i / 11 + 19) & 0xff);
    if (layout == PI05_IMAGE_NCHW) {
      std::vector<uint8_t> nchw(image_bytes);
      const size_t s = cfg.image_size;
      for (int view = 0; view < cfg.num_views; ++view)
        for (size_t y = 0; y < s; ++y)
          for (size_t x = 0; x < s; ++x)
            for (size_t c = 0; c < 3; ++c)
              nchw[((view * 3 + c) * s + y) * s + x] = nhwc[((view * s + y) * s + x) * 3 + c];
      nhwc.swap(nchw);
    }
    for (int b = 0; b < batch; ++b) std::memcpy(images.data() + b * image_bytes, nhwc.data(), image_bytes);
  }
  std::vector<uint32_t> tokens(static_cast<size_t>(token_count) * batch, 0u);
  if (!token_ids_path.empty()) {
    if (!read_file(token_ids_path, &file)) return fail("cannot read " + token_ids_path);
    if (file.size() != static_cast<size_t>(token_count) * 4)
      return fail("--token-ids-u32le length mismatch: expected " + std::to_string(token_count * 4) + ", got " + std::to_string(file.size()));
    for (int b = 0; b < batch; ++b) std::memcpy(tokens.data() + static_cast<size_t>(b) * token_count, file.data(), file.size());
  }
  const size_t noise_elems = static_cast<size_t>(cfg.action_horizon) * cfg.action_dim;
  std::vector<uint16_t> noise(noise_elems * batch, 0);
  if (!noise_path.empty()) {
    if (!read_file(noise_path, &file)) return fail("cannot read " + noise_path);
    if (file.size() != noise_elems * 2)
      return fail("--noise-bf16-u16le length mismatch: expected " + std::to_string(noise_elems * 2) + ", got " + std::to_string(file.size()));
    for (int b = 0; b < batch; ++b) std::memcpy(noise.data() + b * noise_elems, file.data(), file.size());
  }

  std::fprintf(stderr, "capturing the CUDA graph (token_count %d, batch %d)...\n", token_count, batch);
  Pi05Graph* graph = nullptr;
  rc = pi05_engine_capture(engine, token_count, layout, batch, &graph);
  if (rc != PI05_OK) {
    std::fprintf(stderr, "pi05_engine_capture failed: %d (%s)\n", rc, pi05_last_cuda_error());
    return 2;
  }
  const size_t out_elems = noise_elems * batch;
  std::vector<float> eager(out_elems), captured(out_elems), output(out_elems);
  auto check = [&](int code, const char* what) {
    if (code != PI05_OK) {
      std::fprintf(stderr, "%s failed: %d (%s)\n", what, code, pi05_last_cuda_error());
      std::exit(2);
    }
  };
  check(pi05_graph_update_raw_image_inputs(graph, images.data(), tokens.data(), noise.data()), "update inputs");
  check(pi05_graph_run_eager(graph), "eager pass");
  check(pi05_graph_output(graph, eager.data()), "eager output");
  for (float v : eager)
    if (!std::isfinite(v)) { std::fprintf(stderr, "non-finite action in the eager pass\n"); return 3; }
  if (std::getenv("APXINF_PI05_EAGER_ONLY") != nullptr) {
    std::fprintf(stderr, "APXINF_PI05_EAGER_ONLY set: stopping after the eager integrity pass\n");
    return 0;
  }
  check(pi05_graph_replay(graph), "graph replay");
  check(pi05_graph_output(graph, captured.data()), "graph output");
  const Metrics eg = measure(captured, eager);
  const bool eager_graph_passed = eg.cosine >= 0.999999 && eg.max_abs <= th.eager_graph_max_abs;

  for (int i = 0; i < 10; ++i) check(pi05_graph_replay(graph), "warm-up replay");
  check(pi05_graph_sync(graph), "sync");

  using clock = std::chrono::steady_clock;
  std::vector<double> ms(iterations);
  for (int i = 0; i < iterations; ++i) {
    const auto t0 = clock::now();
    check(pi05_graph_replay(graph), "replay");
    check(pi05_graph_sync(graph), "sync");
    ms[i] = std::chrono::duration<double, std::milli>(clock::now() - t0).count();
  }
  const std::string graph_latency = latency_json(ms);
  std::string update_latency = "null";
  if (rgb) {
    for (int i = 0; i < iterations; ++i) {
      const auto t0 = clock::now();
      check(pi05_graph_update_raw_image_inputs(graph, images.data(), tokens.data(), noise.data()), "update");
      check(pi05_graph_replay(graph), "replay");
      check(pi05_graph_sync(graph), "sync");
      ms[i] = std::chrono::duration<double, std::milli>(clock::now() - t0).count();
    }
    update_latency = latency_json(ms);
  }
  check(pi05_graph_output(graph, output.data()), "output");
  double checksum = 0;
  for (float v : output) checksum += std::fabs(static_cast<double>(v));

  std::printf(
      "{\n"
      "  \"profile\": \"pi05_%dview_h%d_steps%d\",\n"
      "  \"precision\": \"%s\",\n"
      "  \"weights\": \"synthetic\",\n"
      "  \"image_input\": {\n"
      "    \"kind\": \"%s\",\n"
      "    \"graph_includes_cuda_preprocess\": true,\n"
      "    \"graph_latency_includes_h2d\": false,\n"
      "    \"input_update_plus_graph_latency_ms\": %s\n"
      "  },\n"
      "  \"token_count\": %d,\n"
      "  \"batch\": %d,\n"
      "  \"fixture_inputs\": {\"images_u8\": %s, \"token_ids_u32le\": %s, \"noise_bf16_u16le\": %s},\n"
      "  \"iterations\": %d,\n"
      "  \"profile_replay\": false,\n"
      "  \"latency_ms\": %s,\n"
      "  \"launches_per_replay\": %d,\n"
      "  \"workspace\": {\"capacity_bytes\": %zu, \"used_bytes\": %zu},\n"
      "  \"output_abs_checksum\": %.9g,\n"
      "  \"integrity\": {\n"
      "    \"passed\": %s,\n"
      "    \"eager_vs_graph\": {\"cosine\": %.12f, \"max_abs\": %.9g, \"mean_abs\": %.9g, \"rmse\": %.9g, "
      "\"relative_l2\": %.9g, \"bitwise_equal\": %s},\n"
      "    \"reference\": null,\n"
      "    \"thresholds\": {\"eager_graph_min_cosine\": 0.999999, \"eager_graph_max_abs\": %g, "
      "\"reference_min_cosine\": %g, \"reference_max_relative_l2\": %g, \"reference_max_abs\": %s}\n"
      "  }\n"
      "}\n",
      cfg.num_views, cfg.action_horizon, cfg.num_flow_steps, precision.c_str(), input_kind.c_str(),
      update_latency.c_str(), token_count, batch, json_string_or_null(images_u8).c_str(),
      json_string_or_null(token_ids_path).c_str(), json_string_or_null(noise_path).c_str(), iterations,
      graph_latency.c_str(), pi05_graph_num_launches(graph), pi05_graph_workspace_bytes(graph),
      pi05_graph_workspace_used_bytes(graph), checksum, eager_graph_passed ? "true" : "false", eg.cosine,
      eg.max_abs, eg.mean_abs, eg.rmse, eg.relative_l2, eg.bitwise_equal ? "true" : "false",
      th.eager_graph_max_abs, min_cosine >= 0 ? min_cosine : th.reference_min_cosine,
      th.reference_max_relative_l2,
      th.has_reference_max_abs ? std::to_string(th.reference_max_abs).c_str() : "null");
  pi05_graph_destroy(graph);
  pi05_engine_destroy(engine);
  if (!eager_graph_passed) {
    std::fprintf(stderr, "eager/graph integrity failed: cosine %.9f, max_abs %.6f\n", eg.cosine, eg.max_abs);
    return 4;
  }
  return 0;
}
