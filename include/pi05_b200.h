/*
 * pi05_b200 — C ABI of the B200-native PI0.5 policy-forward library.
 *
 * Plain C: device/host pointers, integer sizes, integer status returns. Every
 * entry point returns 0 on success and a negative Pi05Status on failure; no
 * entry point throws, aborts or falls back to a CPU path. Launch functions do
 * not allocate device memory unless their comment says so.
 *
 * Two levels, mirroring the reference (infinigence/ApxInf):
 *   - engine level: what `pi05_bench` and the `apxinf-model` PI0.5 runtime
 *     expose (crates/apxinf-model/src/pi05/{bf16_runtime,runtime,int8_runtime}.rs);
 *   - kernel level: what `crates/apxinf-cuda/src/ffi/*.rs` binds.
 */
#ifndef PI05_B200_H_
#define PI05_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum Pi05Status {
  PI05_OK = 0,
  PI05_ERR_INVALID_VALUE = -1,  /* bad argument, rejected before any launch */
  PI05_ERR_UNSUPPORTED = -2,    /* legal but not built (shape / dtype combination) */
  PI05_ERR_DRIVER = -3,         /* CUDA driver entry point missing or tensor-map encode failed */
  PI05_ERR_CUDA = -4,           /* a CUDA runtime call failed; see pi05_last_cuda_error() */
  PI05_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait ran out (status word != 0) */
  PI05_ERR_NOT_BUILT = -6,
  PI05_ERR_SCRATCH_LIMIT = -7   /* the request needs more split-K scratch than is available */
} Pi05Status;

/* Operand / output element types and fused epilogues of pi05_gemm. */
enum { PI05_OP_BF16 = 0, PI05_OP_E4M3 = 1, PI05_OP_S8 = 2 };
/* PI05_OUT_S8: static per-tensor int8, clamp(round_half_away(bf16(o) * out_inv_scale), -128, 127) */
/* PI05_OUT_F16: the scaled accumulator rounded once to f16, no fused epilogue (as PI05_OUT_F32) */
enum { PI05_OUT_BF16 = 0, PI05_OUT_E4M3 = 1, PI05_OUT_F32 = 2, PI05_OUT_S32 = 3, PI05_OUT_S8 = 4,
       PI05_OUT_F16 = 5 };
enum {
  PI05_EPI_STORE = 0,
  PI05_EPI_BIAS_GELU = 1,
  PI05_EPI_BIAS_SILU = 2,
  PI05_EPI_BIAS_RESIDUAL = 3,
  PI05_EPI_BIAS_POS = 4,
  PI05_EPI_GATE_RESIDUAL = 5,
  PI05_EPI_GEGLU = 6,
  /* m <= 16 only (see "Launches with at most 16 rows" below) */
  PI05_EPI_ROPE = 7,  /* packed q|k|v projection -> rotate-half RoPE, Q rows and K/V cache rows */
  PI05_EPI_EULER = 8  /* out = residual + dt * bf16(bf16(v) + bias): velocity head + Euler step */
};
/* Producers that can run inside a GEMM of at most 16 rows instead of as a kernel before it:
 * `a` is then a bf16 matrix [m, k] and the GEMM stages it in its operand type itself. */
enum {
  PI05_PRO_NONE = 0,
  PI05_PRO_ADA_NORM = 1,  /* adaptive RMSNorm: x rsqrt(mean x^2 + eps) (1 + style[0:k]) + style[k:2k] */
  PI05_PRO_QUANTIZE = 2,  /* conversion only (e4m3 / int8 quantisation of a bf16 tensor) */
  PI05_PRO_RMS_NORM = 3   /* RMSNorm with unit weight */
};

/*
 * One dense linear layer out[M, N] = epilogue(a[M, K] . b[N, K]^T) on the
 * tcgen05 tensor cores. `a` and `b` are K-major device matrices (leading
 * dimensions in elements, rows 16-byte aligned); with b_mn_major != 0, `b` is a
 * row-major [K, N] matrix instead. Batched over nb0 x nb1 with element strides.
 * Replaces the reference GEMM contracts gemm::bf16 / gemm::fp8 / gemm::w8a8 and
 * their fused variants (crates/apxinf-cuda/src/kernels/gemm/bf16.rs:355-453,
 * fp8.rs:457-617, w8a8.rs:30-152, crates/apxinf-cuda/src/kernels/fused.rs:18-119)
 * and the FFI symbols behind them (crates/apxinf-cuda/src/ffi/cublaslt.rs:55,112,
 * ffi/cutlass.rs:85-160).
 */
typedef struct Pi05GemmArgs {
  int32_t op;          /* PI05_OP_* of both operands */
  int32_t m, n, k;
  int32_t nb0, nb1;    /* batch extents (>= 1) */
  const void* a;
  int64_t lda, a_sb0, a_sb1;
  const void* b;
  int64_t ldb, b_sb0, b_sb1;
  int32_t b_mn_major;
  void* out;
  int64_t ldc, out_sb0, out_sb1;
  int32_t out_type;    /* PI05_OUT_* */
  int32_t mode;        /* PI05_EPI_* */
  const void* residual;   /* bf16, same geometry as out */
  const void* bias;       /* bf16 [n] */
  const float* col_scale; /* f32 [n], per-output-channel weight scale, or NULL */
  const float* row_scale; /* f32 [m], per-row activation scale, or NULL */
  const void* pos;        /* bf16 [pos_rows, n] */
  int32_t pos_rows;
  int64_t pos_ld;
  const void* gate;       /* bf16 [n] */
  /* bias, col_scale and gate may be produced by an earlier kernel on the same stream: the
   * kernel reads them after its stream-order dependency is resolved. */
  float alpha;
  float out_inv_scale;
  int32_t* status;        /* device int32, must be 0 before the call; set on device timeouts */
  int32_t force_swap;     /* -1 auto */
  int32_t force_block_n;  /* 0 auto */
  /* Optional split-K scratch, caller-owned device memory: `partials` (partials_bytes) holds
   * raw 32-bit accumulator tiles, `tile_counters` (max_tiles int32, zero before the first
   * call; every call leaves them zero) counts arrivals per output tile. NULL = no split-K. */
  void* partials;
  uint64_t partials_bytes;
  int32_t* tile_counters;
  int32_t max_tiles;
  int32_t force_split_k;  /* 0 auto, 1 off, n = n splits */
  /* != 0: `b` is stored K-block-major, [ceil(k / kb)][n][kb] with kb = 128 bytes of K (64 bf16
   * or 128 one-byte elements, the tail block zero padded), so each tile load is one
   * contiguous run; ldb and the batch strides of b are ignored. */
  int32_t b_blocked;
  /* Launches with at most 16 rows (m <= 16, the B=1 action expert) run on a kernel of their
   * own that streams the weights through registers (crates/apxinf-model/src/pi05/
   * bf16_executor.rs:89-157 is the call list it serves). force_skinny: -1 automatic (taken
   * unless a force_* field above pins a tcgen05 variant), 0 never, 1 required
   * (PI05_ERR_UNSUPPORTED if the problem does not fit). The fields below need that kernel. */
  int32_t force_skinny;
  int32_t prologue;        /* PI05_PRO_*; k <= 1024 and a multiple of 8 */
  const void* style;       /* PI05_PRO_ADA_NORM: bf16 [2 k] */
  float eps;
  float a_inv_scale;       /* 1 / static activation scale of the staged operand (e4m3, int8) */
  int32_t a_dynamic_rows;  /* int8: per-row scales computed by the prologue instead */
  /* PI05_EPI_ROPE (n = (q_heads + 2) * head_dim, one K/V head; replaces
   * apxinf_static_qkv_rope_*, crates/apxinf-cuda/kernels/custom/fused.cuh:471-525): row r is
   * token r % rope_tokens of sample r / rope_tokens at position rope_position_offset + token;
   * q_out bf16 [m, q_heads, head_dim]; K / V go to row position of the sample's
   * [rope_cache_rows, head_dim] cache; cos / sin f32 [positions, head_dim / 2]. */
  void* rope_q_out;
  void* rope_k_cache;
  void* rope_v_cache;
  const float* rope_cos;
  const float* rope_sin;
  int32_t rope_tokens, rope_q_heads, rope_head_dim, rope_position_offset, rope_cache_rows;
  float dt;                /* PI05_EPI_EULER */
  /* > 1: the K range of one GEMM (nb0 = nb1 = 1, no split-K, K-major operands) in that many runs
   * of 128-byte K blocks, run s writing its own product at out + s * out_sb0 elements: partial
   * products (PI05_OUT_F32, PI05_EPI_STORE) for the caller to add. Used for a few hundred rows
   * against a very long K (language.down at B=1), where whole tiles alone would leave most SMs
   * idle. 0 and 1: off. */
  int32_t k_slices;
} Pi05GemmArgs;

int pi05_gemm(const Pi05GemmArgs* args, void* cuda_stream);

/*
 * Split-K pi05_gemm for callers that must not allocate. (No counterpart in the reference,
 * whose launch functions take their workspace from its arena.) Some users of this library
 * cannot call cudaMalloc at the point where they need a GEMM: a control loop that has
 * finished its set-up phase and may not risk an allocation stall or failure, a plugin that was
 * handed a fixed device-memory budget by its host, code running between other people's
 * latency-critical launches. For them the split-K scratch (partial accumulator tiles and the
 * per-tile arrival counters) lives in a fixed array inside the library image instead of in
 * caller memory: PI05_STATIC_SCRATCH_BYTES of partial tiles and PI05_STATIC_SCRATCH_TILES
 * counters per GPU, held by every GPU that loads the library until the process exits.
 *
 * Same arguments and results as pi05_gemm with `force_split_k` >= 2; the `partials`,
 * `partials_bytes`, `tile_counters` and `max_tiles` fields are ignored. Inputs, outputs and the
 * status word are still the caller's. A request whose tiles x splits need more than the fixed
 * scratch is refused with PI05_ERR_SCRATCH_LIMIT before anything is launched (detail text in
 * pi05_last_cuda_error()). The call performs no cudaMalloc / cudaFree and uses no allocating
 * library routine. `cuda_stream` must belong to the current device (PI05_ERR_INVALID_VALUE
 * otherwise). Requests that cannot be split (PI05_OUT_S32 output, or K within one 128-byte
 * block) run as a single pass and leave the scratch untouched.
 *
 * The first call on each device looks up the array's device address (with that device
 * current) and remembers it; make that first call during set-up, before any stream capture.
 * Later calls may be captured into a CUDA graph (the stream's device is then not checked: a
 * capturing stream cannot be queried for it).
 * Every call shares the one array and the counters are cleared on the stream before each
 * launch, so two calls that can overlap on the GPU (different streams, or one stream captured
 * into concurrently running graphs) race on it: serialise them on one stream.
 */
#define PI05_STATIC_SCRATCH_BYTES (8u << 20)
#define PI05_STATIC_SCRATCH_TILES 2048
int pi05_gemm_static_scratch(const Pi05GemmArgs* args, void* cuda_stream);


/*
 * Fused attention out = softmax(scale * q k^T) v on the tcgen05 tensor cores, no mask, at most
 * 1024 keys, head_dim a multiple of 8 up to 256, batched over nb0 x nb1 (element strides).
 * q [q_rows, head_dim], k / v [keys, head_dim] and out [q_rows, head_dim] are bf16 device
 * matrices with contiguous head_dim; with out_e4m3 != 0 the output is
 * e4m3(clamp(bf16(o) * out_inv_scale)). Multi-query attention passes its query heads as nb0
 * with k_sb0 = v_sb0 = 0 (one shared K/V head): when nb0 divides 128 the kernel packs the heads
 * of a token into the same 128-row tile and fetches K/V once for all of them. Replaces the reference attention contracts mha_bf16 /
 * mqa_bf16 / mqa_cached_f16 (crates/apxinf-cuda/src/kernels/attention.rs:627-1261) and the FFI
 * symbols behind them (ffi/cublas.rs:113-134, ffi/cutlass.rs:9-83, ffi/fa2.rs:9-58).
 */
typedef struct Pi05AttentionArgs {
  const void* q;
  int64_t q_ld, q_sb0, q_sb1;
  const void* k;
  int64_t k_ld, k_sb0, k_sb1;
  const void* v;
  int64_t v_ld, v_sb0, v_sb1;
  void* out;
  int64_t out_ld, out_sb0, out_sb1;
  int32_t q_rows, keys, head_dim, nb0, nb1;
  float scale;
  int32_t out_e4m3;
  float out_inv_scale;
  int32_t* status; /* device int32, 0 before the call */
  /* key_split != 0: one CTA per (query tile, 64-key slice) writes partial outputs to
   * split_scratch and a second launch combines them; for calls with few query tiles.
   * split_scratch needs tiles * ceil(keys / 64) * 128 * (head_dim + 2) * 4 bytes
   * (PI05_ERR_SCRATCH_LIMIT if smaller); tiles = ceil(q_rows / 128) * nb0 * nb1, or
   * ceil(q_rows * nb0 / 128) * nb1 for packed multi-query heads. */
  int32_t key_split;
  void* split_scratch;
  int64_t split_scratch_bytes;
} Pi05AttentionArgs;

int pi05_attention(const Pi05AttentionArgs* args, void* cuda_stream);

/* ------------------------------------------------------------------------- */
/* Engine level                                                              */
/* ------------------------------------------------------------------------- */

enum { PI05_DTYPE_BF16 = 0, PI05_DTYPE_FP8 = 1, PI05_DTYPE_INT8 = 2 };
/* PI05_IMAGE_PATCHES: the graph takes ready-made fp32 patch rows (the reference's L0 entry,
 * crates/apxinf-py/src/lib.rs:348-395) instead of u8 images. */
enum { PI05_IMAGE_NHWC = 0, PI05_IMAGE_NCHW = 1, PI05_IMAGE_PATCHES = 2 };

/* Architecture constants; field meaning and defaults follow Pi05Config /
 * GemmaVariantConfig (crates/apxinf-model/src/pi05/config.rs:5-109).
 * pi05_default_config() fills the two-view, horizon-10 bench profile. */
typedef struct Pi05Gemma {
  int32_t width, depth, mlp_dim, num_heads, num_kv_heads, head_dim;
} Pi05Gemma;

typedef struct Pi05ModelConfig {
  int32_t action_dim, action_horizon, max_token_len, num_flow_steps;
  int32_t num_views, image_size, patch_size;
  int32_t vision_width, vision_depth, vision_mlp_dim, vision_heads, vision_head_dim;
  int32_t vocab_size;
  float rms_norm_eps, layer_norm_eps, rope_theta, time_min_period, time_max_period;
  Pi05Gemma language, action_expert;
} Pi05ModelConfig;

typedef struct Pi05Engine Pi05Engine; /* weights + stream of one GPU; one host thread at a time */
typedef struct Pi05Graph Pi05Graph;   /* one prepared (token_count, layout, batch) inference */

void pi05_default_config(Pi05ModelConfig* config);

/* Creates the runtime on `device` with Pi05Weights::synthetic(config, seed) weights
 * (crates/apxinf-model/src/pi05/weights.rs:255-330) generated on the GPU and
 * packed/quantised for `dtype` — the `pi05_bench random --dtype ...` path
 * (crates/apxinf-model/examples/pi05_bench.rs:901-990). `fp8_act_scale` is the
 * uniform static activation scale of Pi05ActivationScales::uniform
 * (crates/apxinf-model/src/pi05/runtime.rs:86-113); ignored unless dtype is FP8.
 * Allocates device memory. Replaces Pi05{Bf16,,Int8}CudaRuntime::new. */
int pi05_engine_create(const Pi05ModelConfig* config, int32_t dtype, int32_t device, uint64_t seed,
                       float fp8_act_scale, Pi05Engine** out);

/* The same with the two choices the benchmark configurations word differently from the
 * reference code:
 *   weight_dist       PI05_WEIGHTS_LCG: the reference generator, uniform in [-0.02, 0.02)
 *                     (weights.rs:332-357); PI05_WEIGHTS_NORMAL: seeded N(0, 0.02) from a
 *                     counter-based generator (SplitMix64 keyed by the seed; element order as
 *                     the reference's tensor order).
 *   int8_activations  PI05_INT8_ACT_DYNAMIC: one scale per activation row, computed on the fly
 *                     (crates/apxinf-cuda/src/kernels/gemm/w8a8.rs:86-98);
 *                     PI05_INT8_ACT_STATIC: one fixed scale per GEMM input, the quantiser
 *                     fused into the norm kernels and GEMM epilogues like the FP8 path's.
 * act_scale is the uniform static activation scale (FP8, static INT8); single sites are set by
 * name with pi05_engine_set_activation_scale. */
enum { PI05_WEIGHTS_LCG = 0, PI05_WEIGHTS_NORMAL = 1 };
enum { PI05_INT8_ACT_DYNAMIC = 0, PI05_INT8_ACT_STATIC = 1 };
typedef struct Pi05EngineOptions {
  int32_t dtype;   /* PI05_DTYPE_* */
  int32_t device;
  uint64_t seed;
  float act_scale;
  int32_t weight_dist;
  int32_t int8_activations;
} Pi05EngineOptions;
int pi05_engine_create_ex(const Pi05ModelConfig* config, const Pi05EngineOptions* options,
                          Pi05Engine** out);
/* The runtime from caller-provided weights instead of the synthetic generator: what the
 * reference builds from a checkpoint (Pi05Weights::from_map, crates/apxinf-model/src/pi05/
 * weights.rs:116-244, then Static*Pi05Weights::from_host). Tensors are host bf16 bit patterns
 * or float32 (the reference's folded Gemma projections are float32: the FP8 and INT8 precisions
 * quantise them from float32 as the reference does, bf16 storage rounds them to nearest even),
 * linear weights in the reference's final [in, out] orientation, named as the reference's
 * synthetic layout orders them: "vision.<i>.{q,k,v,o,fc1,fc2}.{weight,bias}",
 * "vision.patch_embedding.{weight,bias}", "vision.position_embedding",
 * "vision.projector.{weight,bias}", "token_embedding", "language.<i>.{q,k,v,o,gate,up,down}.weight",
 * "action.<i>.{input_style,post_style}.{weight,bias}", "action.<i>.{q,...,down}.weight",
 * "action.final_style.*", "action_in.*", "action_out.*", "time_mlp_in.*", "time_mlp_out.*", and
 * optionally the LayerNorm parameters "vision.<i>.norm1.{weight,bias}", "vision.<i>.norm2.*",
 * "vision.post_norm.*" (absent = 1 / 0). Packing, quantisation and upload are as for the
 * synthetic weights. A missing or mis-sized tensor returns PI05_ERR_INVALID_VALUE and names it
 * in pi05_last_cuda_error(). The host buffers are only read during the call. (apxinf_b200/
 * checkpoint.py reads safetensors checkpoints into this table.) */
enum { PI05_TENSOR_BF16 = 0, PI05_TENSOR_F32 = 1 };
typedef struct Pi05HostTensor {
  const char* name;
  const void* data;
  uint64_t elements;
  int32_t dtype; /* PI05_TENSOR_* */
} Pi05HostTensor;
int pi05_engine_create_from_tensors(const Pi05ModelConfig* config, const Pi05EngineOptions* options,
                                    const Pi05HostTensor* tensors, int32_t count, Pi05Engine** out);

/* Static activation scale of one GEMM-input site, named as the reference's calibration table
 * (Pi05ActivationScales::from_calibration, crates/apxinf-model/src/pi05/runtime.rs:35-81):
 * "vision.patch_input", "vision.layers.<i>.attention_norm" / ".attention_output" / ".mlp_norm" /
 * ".mlp_activation", "vision.post_norm", "language.layers.<i>.<same four>", "action.input",
 * "time.input", "time.hidden", "action.conditioning", "action.layers.<i>.<same four>",
 * "action.final_norm". Takes effect for graphs captured afterwards. Unknown names and
 * non-positive scales return PI05_ERR_INVALID_VALUE. */
int pi05_engine_set_activation_scale(Pi05Engine* engine, const char* site, float scale);
float pi05_engine_activation_scale(const Pi05Engine* engine, const char* site); /* 0 if unknown */
void pi05_engine_destroy(Pi05Engine* engine);
size_t pi05_engine_weight_bytes(const Pi05Engine* engine);
/* Copies a device weight tensor ("language.3.qkv.weight", ".scale", ".bias", ...) to the host;
 * with host == NULL only reports its size. For parity tests. */
int pi05_engine_read_weight(Pi05Engine* engine, const char* name, void* host, size_t capacity,
                            size_t* actual);

/* capture_infer_rgb_u8 (crates/apxinf-model/src/pi05/bf16_runtime.rs:457-575): sizes and
 * allocates the workspace, precomputes the per-step adaRMSNorm styles outside the graph,
 * plans every launch and records them into one CUDA graph. `batch` independent observations
 * share the weights (batch 1 = the reference's only mode). Allocates device memory; no later
 * call on the graph does. */
int pi05_engine_capture(Pi05Engine* engine, int32_t token_count, int32_t image_layout,
                        int32_t batch, Pi05Graph** out);
void pi05_graph_destroy(Pi05Graph* graph);

/* update_raw_image_inputs (bf16_runtime.rs:88-123): queues the host->device copies of
 * images u8 [batch, views, size, size, 3] (or NCHW), token ids u32 [batch, token_count] and
 * noise bf16 bits [batch, horizon, action_dim] on the engine stream. The host buffers must
 * stay valid until the next pi05_graph_sync / pi05_graph_output. */
int pi05_graph_update_raw_image_inputs(Pi05Graph* graph, const uint8_t* images,
                                       const uint32_t* token_ids, const uint16_t* noise_bf16);
/* The same for a graph captured with PI05_IMAGE_PATCHES: patches fp32
 * [batch, views * patches_per_view, 3 * patch_size^2], columns ordered channel, dy, dx
 * (VisionObservation::Patches, crates/apxinf-model/src/vla_runtime.rs). */
int pi05_graph_update_patch_inputs(Pi05Graph* graph, const float* patches,
                                   const uint32_t* token_ids, const uint16_t* noise_bf16);
int pi05_graph_replay(Pi05Graph* graph);     /* cudaGraphLaunch, asynchronous */
int pi05_graph_run_eager(Pi05Graph* graph);  /* the same launch list without the graph */
int pi05_graph_sync(Pi05Graph* graph);       /* waits; PI05_ERR_DEVICE_TIMEOUT if a device wait ran out */
/* Waits, then writes the action chunk [batch, horizon, action_dim] as float32. */
int pi05_graph_output(Pi05Graph* graph, float* host_out);
/* `iterations` replays, each timed with CUDA events on the engine stream (milliseconds). */
int pi05_graph_time_replays(Pi05Graph* graph, int32_t iterations, float* ms_each);
/* One eager pass timed per stage: {vision tower, prefix prefill, denoise loop} in ms. */
int pi05_graph_stage_times(Pi05Graph* graph, float* ms3);
/* One eager pass with a CUDA-event pair around every launch called `name`
 * ("language.gate_up", "action.qkv", ...): mean duration in ms and number of launches. */
int pi05_graph_time_launches(Pi05Graph* graph, const char* name, float* mean_ms, int32_t* count);
size_t pi05_graph_workspace_bytes(const Pi05Graph* graph);
size_t pi05_graph_workspace_used_bytes(const Pi05Graph* graph);
int32_t pi05_graph_num_launches(const Pi05Graph* graph);
/* Name of launch `index` (for launch-list summaries); NULL when out of range. */
const char* pi05_graph_launch_name(const Pi05Graph* graph, int32_t index);
/* Copies a named intermediate ("prefix", "kv.3.k", "state", "vision.hidden", ...) to the host. */
int pi05_graph_read_tensor(Pi05Graph* graph, const char* name, void* host, size_t capacity,
                           size_t* actual);

/*
 * Owning frontend (Pi05VlaRuntime / Pi05PreparedInference,
 * crates/apxinf-model/src/pi05/vla_runtime.rs:393-495): pi05_runtime_infer keeps ONE prepared plan,
 * keyed by (token_count, image_layout); an observation of another shape drops it and builds
 * the new one (a workspace is large: two never coexist). Building tries CUDA-graph capture
 * and falls back to running the same launch list eagerly when capture is unavailable. Noise
 * given as float32 is rounded to the runtime's 16-bit input type on the host. The engine is
 * borrowed and must outlive the runtime; one host thread at a time.
 */
/* Compute capability of a device as major * 10 + minor (100 on B200), -1 when it cannot be
 * read: the input of the reference's automatic precision policy
 * (crates/apxinf-model/src/pi05/vla_runtime.rs:628-639). */
int pi05_device_sm(int32_t device);

enum { PI05_NOISE_F32 = 0, PI05_NOISE_BF16 = 1 };
typedef struct Pi05Observation {
  int32_t token_count;
  int32_t image_layout;       /* PI05_IMAGE_NHWC | PI05_IMAGE_NCHW | PI05_IMAGE_PATCHES */
  const uint8_t* images;      /* u8 [views, S, S, 3] (or NCHW); unused for patches */
  const float* patches;       /* f32 [views * patches_per_view, 3 * patch^2] for PI05_IMAGE_PATCHES */
  const uint32_t* token_ids;  /* [token_count] */
  const void* noise;          /* [horizon, action_dim] */
  int32_t noise_dtype;        /* PI05_NOISE_* */
} Pi05Observation;
typedef struct Pi05Runtime Pi05Runtime;
int pi05_runtime_create(Pi05Engine* engine, Pi05Runtime** out);
void pi05_runtime_destroy(Pi05Runtime* runtime);
/* infer_host_f32 (vla_runtime.rs:491-494): actions_out float32 [horizon, action_dim] on the host. */
int pi05_runtime_infer(Pi05Runtime* runtime, const Pi05Observation* observation, float* actions_out);
/* The cached plan: its shape, whether it replays a CUDA graph (0 = eager fallback) and how many
 * plans this runtime has built so far. Any out pointer may be NULL. */
int pi05_runtime_plan_info(const Pi05Runtime* runtime, int32_t* token_count, int32_t* image_layout,
                           int32_t* uses_graph, int32_t* builds);

/* Signature of a named bf16 intermediate of the last run ("patches", "vision.hidden", "prefix",
 * "kv.<l>.k", "action.hidden", "state", ...): the statistics the reference's integrity probe
 * prints per stage (crates/apxinf-model/examples/pi05_integrity_probe.rs:19-51). */
typedef struct Pi05Signature {
  uint64_t elements;
  double sum, abs_checksum, l2, max_abs;
  int32_t sample_count;  /* min(elements, 256) evenly spaced values */
  float sample[256];
} Pi05Signature;
int pi05_graph_signature(Pi05Graph* graph, const char* name, Pi05Signature* out);

/* Process-wide planning switches, for A/B measurements and tests; they apply to graphs captured
 * afterwards. "programmatic_dependent_launch" (default 1): launches carry the programmatic
 * stream-serialisation attribute. "fuse_small_rows" (default 1): graphs whose action expert has
 * at most 16 rows run its projections on the register-streaming kernel with the row kernels
 * fused in; 0 plans the launch list larger batches use. "attention_cluster" (default 1):
 * key-split attention requests (few query rows) run as one launch of 8-CTA clusters that merge
 * their slices through distributed shared memory; 0 keeps the two-launch form with scratch.
 * "fuse_norms" (default 0): with at most 16 action rows the adaptive RMSNorms run as the staging
 * step of the projections that read them instead of as launches of their own (measured slower).
 * "persistent_denoise" (default 0; measured slower than the launches it replaces): BF16 / FP8 graphs of one observation whose action expert has
 * at most 16 rows run the whole denoise loop (every step, layer, projection and attention) as
 * the stages of one cooperative launch ordered by a grid barrier; 0 keeps one launch per
 * projection. "denoise_wait_limit_polls" (default 0 = 2^21): poll budget of that kernel's
 * barrier waits, after which it records PI05_ERR_DEVICE_TIMEOUT's status and returns.
 * "denoise_skip_arrival" (default -1 = none): diagnostics of that kernel's timeout path, CTA 0
 * leaves out its arrival after that stage, so the barrier never completes and every wait runs out.
 * "wait_limit_polls" (default 0 = 2^24) and "drop_one_load" (default -1 = none) exercise the
 * device-timeout contract without a fault: GEMM plans built afterwards give every barrier wait of
 * the one-CTA-per-tile kernel that poll budget, and their first CTA announces the A load of that
 * K block but never issues it, so the stage never fills, the bounded waits run out, the kernel
 * records its status word, releases its TMEM and returns; the caller sees PI05_ERR_DEVICE_TIMEOUT
 * at the next sync and the context stays usable.
 * "single_epilogue_kernels" (default 1): GEMM plans built afterwards run, where one fits, a
 * tcgen05 kernel compiled for their one epilogue and output type (same arithmetic, a shorter
 * instruction stream); 0 always plans the general kernel.
 * "force_capture_failure" (default 0): plans built by pi05_runtime_infer skip graph capture, as
 * if the driver had refused it (exercises the eager fallback). Unknown names:
 * PI05_ERR_INVALID_VALUE. */
int pi05_set_tuning(const char* name, int32_t value);

/* Last CUDA runtime error string seen by this library on the calling thread. */
const char* pi05_last_cuda_error(void);

/* Library build identification: "pi05_b200 sm_100a <date>". */
const char* pi05_version(void);

#ifdef __cplusplus
}
#endif

#endif /* PI05_B200_H_ */
