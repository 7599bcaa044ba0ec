"""CPU restatement (NumPy) of ApxInf's PI0.5 policy forward — TEST INFRASTRUCTURE ONLY.

This module is the parity oracle: it restates, on the CPU, the arithmetic of the
reference's PI0.5 path with the reference's rounding points. It is imported only
by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs; the product
(libpi05_b200.so and the apxinf_b200 package) never imports or calls it.

Reference files followed (paths inside the ApxInf repository):
  weights / RNG      crates/apxinf-model/src/pi05/weights.rs:255-415
  BF16 graph         crates/apxinf-model/src/pi05/bf16_executor.rs:24-212,
                     crates/apxinf-model/src/pi05/bf16_runtime.rs:158-387
  FP8 graph          crates/apxinf-model/src/pi05/fp8_executor.rs:75-462,
                     crates/apxinf-model/src/pi05/runtime.rs:290-598
  INT8 graph         crates/apxinf-model/src/pi05/int8_executor.rs:24-201
  E4M3 codec         crates/apxinf-model/src/pi05/fp8.rs:128-184
  INT8 quantiser     crates/apxinf-model/src/pi05/int8_weights.rs:92-123,
                     crates/apxinf-cuda/kernels/custom/quantization.cuh:56-88
  time embedding     crates/apxinf-model/src/pi05/math.rs:4-27, runtime.rs:821-838
  per-op math        crates/apxinf-cuda/kernels/custom/{preprocess,normalization,fused,
                     activation,elementwise,embedding,attention,math}.cuh,
                     crates/apxinf-cuda/adapters/cublas_adapter.cu:89-132

Parity pinning: the pieces for which the reference ships known-answer tests are
checked against those vectors in tests/test_oracle_kat.py (E4M3 bytes, INT8
channel quantiser, time-embedding endpoints, Euler sign, patchify layout,
zero-query attention means, W8A8 small case). The reference ships NO end-to-end
golden action vector (its `--reference` JSON comes from an external run on a real
checkpoint), and its host is Rust, which cannot be built here. The per-op math is
therefore pinned one level down, against the reference's own CUDA kernels: the
self-contained adapters (static BF16 operators, F16/E4M3 operators, W8A8 quantiser)
are compiled for sm_100a by oracle/Makefile into oracle/_ref and run on the GPU next
to these restatements in tests/test_ref_ops_gpu.py (patch rows, the three norms,
Euler update, embedding, INT8 row quantiser, MQA / MHA attention, GeGLU,
bias + residual, gated residual, RoPE split, and the E4M3 codec over every finite
half-precision input). What stays unpinned is the ORDER in which the executors
call these ops (restated from the Rust sources by reading) and the cuBLASLt /
CUTLASS GEMMs, which need libraries outside the reference tree.

Declared deltas from the reference, following the benchmark configuration this
repository is measured on: the FP8 path stores activations as BF16 (reference:
FP16; `storage="f16"` reproduces it) and uses one weight scale per output channel
(reference: one per packed matrix; `fp8_weight_scale="tensor"` reproduces it).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Dict, Optional, Tuple

import numpy as np

F32 = np.float32

# ----------------------------------------------------------------------------
# rounding helpers
# ----------------------------------------------------------------------------


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 (round to nearest even) -> float32."""
    x = np.ascontiguousarray(x, dtype=F32)
    bits = x.view(np.uint32)
    rounding = ((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((bits + rounding) & np.uint32(0xFFFF0000)).view(F32)
    return np.where(np.isnan(x), x, out)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    return (round_bf16(x).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bf16_from_bits(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << np.uint32(16)).view(F32)


def round_f16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=F32).astype(np.float16).astype(F32)


E4M3_MAX = F32(448.0)


def e4m3_round(x: np.ndarray) -> np.ndarray:
    """Nearest-even rounding of float32 onto the finite E4M3 grid, saturating (fp8.rs:128-166)."""
    x = np.ascontiguousarray(x, dtype=F32)
    a = np.abs(x)
    bits = a.view(np.uint32)
    rounding = ((bits >> np.uint32(20)) & np.uint32(1)) + np.uint32(0x7FFFF)
    normal = ((bits + rounding) & np.uint32(0xFFF00000)).view(F32)
    sub = np.rint(a * F32(512.0)) / F32(512.0)
    out = np.where(a < F32(2.0 ** -6), sub, normal)
    out = np.minimum(out, E4M3_MAX)
    out = np.where(np.isnan(x), F32(np.nan), out)
    return np.copysign(out, x).astype(F32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 byte ("fn" flavour: no infinities, 0x7f = NaN, max 0x7e = 448)."""
    r = e4m3_round(x)
    a = np.abs(r)
    sign = np.where(np.signbit(r), 0x80, 0).astype(np.uint8)
    bits = a.view(np.uint32)
    exp = ((bits >> np.uint32(23)) & np.uint32(0xFF)).astype(np.int32) - 127
    man = ((bits >> np.uint32(20)) & np.uint32(0x7)).astype(np.int32)
    normal = ((exp + 7) << 3) | man
    with np.errstate(invalid="ignore"):
        sub = np.rint(np.nan_to_num(a) * F32(512.0)).astype(np.int32)
    byte = np.where(a < F32(2.0 ** -6), sub, normal).astype(np.uint8)
    byte = np.where(np.isnan(r), 0x7F, byte | sign).astype(np.uint8)
    return byte


def e4m3_decode(byte: np.ndarray) -> np.ndarray:
    byte = np.asarray(byte, dtype=np.uint8)
    sign = np.where(byte & 0x80, F32(-1.0), F32(1.0))
    exp = ((byte >> 3) & 0x0F).astype(np.int32)
    man = (byte & 0x07).astype(F32)
    sub = man * F32(2.0 ** -9)
    normal = (F32(1.0) + man / F32(8.0)) * np.exp2((exp - 7).astype(F32))
    out = np.where(exp == 0, sub, normal).astype(F32)
    out = np.where((exp == 15) & ((byte & 0x07) == 7), F32(np.nan), out)
    return (sign * out).astype(F32)


def quantize_e4m3_static(x: np.ndarray, scale: float) -> np.ndarray:
    """E4M3 grid value of x / scale (quantization.cuh:6-20): multiply by 1/scale, clamp, RNE."""
    inv = F32(1.0) / F32(scale)
    return e4m3_round(np.clip(np.asarray(x, F32) * inv, -E4M3_MAX, E4M3_MAX))


def quantize_rows_int8(x: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Dynamic per-row symmetric INT8 (quantization.cuh:56-74): half-away rounding."""
    x = np.asarray(x, F32)
    amax = np.max(np.abs(x), axis=1)
    scale = np.maximum(amax / F32(127.0), F32(1.0e-12)).astype(F32)
    t = x / scale[:, None]
    q = np.sign(t) * np.floor(np.abs(t) + F32(0.5))
    q = np.clip(q, -128.0, 127.0).astype(F32)
    return q, scale


def quantize_int8_static(x: np.ndarray, scale: float) -> np.ndarray:
    """Static per-tensor INT8 (the benchmark's W8A8 wording): x * (1/scale), half-away
    rounding, clamp to [-128, 127]."""
    inv = F32(1.0) / F32(scale)
    t = np.asarray(x, F32) * inv
    q = np.sign(t) * np.floor(np.abs(t) + F32(0.5))
    return np.clip(q, -128.0, 127.0).astype(F32)


def quantize_int8_channels(w_in_out: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Per-output-channel INT8 weights of an [in, out] matrix (int8_weights.rs:92-123)."""
    w = np.asarray(w_in_out, F32)
    amax = np.max(np.abs(w), axis=0)
    scale = np.maximum(amax / F32(127.0), F32(1.0e-12)).astype(F32)
    t = w / scale[None, :]
    q = np.sign(t) * np.floor(np.abs(t) + F32(0.5))
    return np.clip(q, -128.0, 127.0).astype(F32), scale


def quantize_e4m3_channels(w_in_out: np.ndarray, per: str = "channel") -> Tuple[np.ndarray, np.ndarray]:
    """E4M3 weights of an [in, out] matrix with absmax/448 scales (fp8.rs:88-115)."""
    w = np.asarray(w_in_out, F32)
    if per == "tensor":
        amax = np.full(w.shape[1], np.max(np.abs(w)), dtype=F32)
    else:
        amax = np.max(np.abs(w), axis=0).astype(F32)
    scale = np.where(amax == 0, F32(1.0), amax / E4M3_MAX).astype(F32)
    inv = (F32(1.0) / scale).astype(F32)
    return e4m3_round(w * inv[None, :]), scale


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """math.cuh:8-12."""
    x = np.asarray(x, F32)
    k = F32(0.7978845608028654)
    inner = k * (x + F32(0.044715) * x * x * x)
    return (F32(0.5) * x * (F32(1.0) + np.tanh(inner).astype(F32))).astype(F32)


def silu(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, F32)
    return (x / (F32(1.0) + np.exp(-x).astype(F32))).astype(F32)


# ----------------------------------------------------------------------------
# configuration
# ----------------------------------------------------------------------------


@dataclass(frozen=True)
class GemmaVariant:
    width: int
    depth: int
    mlp_dim: int
    num_heads: int
    num_kv_heads: int
    head_dim: int


GEMMA_2B = GemmaVariant(2048, 18, 16384, 8, 1, 256)
GEMMA_300M = GemmaVariant(1024, 18, 4096, 8, 1, 256)


@dataclass(frozen=True)
class Pi05Config:
    """config.rs:58-109 (defaults) with the two-view H=10 bench profile as default."""
    action_dim: int = 32
    action_horizon: int = 10
    max_token_len: int = 200
    num_flow_steps: int = 10
    num_views: int = 2
    image_size: int = 224
    patch_size: int = 14
    vision_width: int = 1152
    vision_depth: int = 27
    vision_mlp_dim: int = 4304
    vision_heads: int = 16
    vision_head_dim: int = 72
    vocab_size: int = 257152
    rms_norm_eps: float = 1e-6
    layer_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    time_min_period: float = 4e-3
    time_max_period: float = 4.0
    language: GemmaVariant = GEMMA_2B
    action_expert: GemmaVariant = GEMMA_300M

    @property
    def patches_per_side(self) -> int:
        return self.image_size // self.patch_size

    @property
    def patches_per_view(self) -> int:
        return self.patches_per_side ** 2

    @property
    def patch_width(self) -> int:
        return 3 * self.patch_size * self.patch_size

    @property
    def vision_tokens(self) -> int:
        return self.num_views * self.patches_per_view


def tiny_config(**overrides) -> Pi05Config:
    """A small architecture with every structural feature of PI0.5 (tests only)."""
    base = Pi05Config(
        action_dim=32, action_horizon=5, max_token_len=16, num_flow_steps=3, num_views=2,
        image_size=56, patch_size=14, vision_width=144, vision_depth=2, vision_mlp_dim=320,
        vision_heads=2, vision_head_dim=72, vocab_size=1000,
        language=GemmaVariant(256, 3, 512, 2, 1, 128),
        action_expert=GemmaVariant(128, 3, 256, 2, 1, 128))
    return replace(base, **overrides)


# ----------------------------------------------------------------------------
# synthetic weights (weights.rs:255-415)
# ----------------------------------------------------------------------------

LCG_A = 6364136223846793005
LCG_C = 1442695040888963407
LCG_SEED_XOR = 0x9E3779B97F4A7C15
MASK64 = (1 << 64) - 1
AMPLITUDE = F32(0.02)


def lcg_jump(n: int) -> Tuple[int, int]:
    """(A_n, C_n) with state_{k+n} = A_n * state_k + C_n (mod 2^64)."""
    acc_a, acc_c = 1, 0
    cur_a, cur_c = LCG_A, LCG_C
    while n > 0:
        if n & 1:
            acc_a = (acc_a * cur_a) & MASK64
            acc_c = (acc_c * cur_a + cur_c) & MASK64
        cur_c = ((cur_a + 1) * cur_c) & MASK64
        cur_a = (cur_a * cur_a) & MASK64
        n >>= 1
    return acc_a, acc_c


_LCG_BLOCK = 1 << 20
_lcg_tables: Optional[Tuple[np.ndarray, np.ndarray]] = None


def _lcg_block_tables() -> Tuple[np.ndarray, np.ndarray]:
    global _lcg_tables
    if _lcg_tables is None:
        a = np.empty(_LCG_BLOCK, dtype=np.uint64)
        c = np.empty(_LCG_BLOCK, dtype=np.uint64)
        # doubling construction of (A_j, C_j), j = 1.._LCG_BLOCK
        a[0], c[0] = LCG_A, LCG_C
        filled = 1
        with np.errstate(over="ignore"):
            while filled < _LCG_BLOCK:
                take = min(filled, _LCG_BLOCK - filled)
                aj, cj = a[filled - 1], c[filled - 1]  # jump by `filled`
                a[filled:filled + take] = a[:take] * aj
                c[filled:filled + take] = c[:take] * aj + cj
                filled += take
        _lcg_tables = (a, c)
    return _lcg_tables


def _lcg_block(seed_state: int, start: int, out: np.ndarray) -> None:
    ja, jc = lcg_jump(start)
    state = (ja * seed_state + jc) & MASK64
    ta, tc = _lcg_block_tables()
    take = out.shape[0]
    with np.errstate(over="ignore"):
        s = ta[:take] * np.uint64(state) + tc[:take]
        bits = (s >> np.uint64(33)).astype(np.uint32)
        unit = bits.astype(F32) / F32(2147483648.0)
        out[:] = round_bf16((unit * F32(2.0) - F32(1.0)) * AMPLITUDE)


def lcg_values(seed: int, offset: int, count: int) -> np.ndarray:
    """Elements [offset, offset+count) of SyntheticRng(seed) as bf16-rounded float32.
    Blocks of 2^20 elements are independent (jump-ahead), so they run on a thread pool."""
    state0 = (seed ^ LCG_SEED_XOR) & MASK64
    _lcg_block_tables()
    out = np.empty(count, dtype=F32)
    starts = list(range(0, count, _LCG_BLOCK))
    if len(starts) <= 2:
        for b in starts:
            _lcg_block(state0, offset + b, out[b:b + _LCG_BLOCK])
    else:
        import concurrent.futures
        import os
        with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
            list(pool.map(lambda b: _lcg_block(state0, offset + b, out[b:b + _LCG_BLOCK]), starts))
    return out


# Seeded N(0, 0.02) weights (the benchmark configurations' wording; the reference generator
# above is uniform). Counter-based so that any element can be produced anywhere: element i of
# the stream is the sum of twelve 16-bit fields of three SplitMix64 outputs (counters 3i,
# 3i+1, 3i+2 keyed by the seed) - an Irwin-Hall sum with mean 393210 and standard deviation
# 65536 - centred and scaled by 0.02 / 65536. Integer sums and one float32 multiply: the GPU
# generator (weights.cu, normal_fill_kernel) reproduces it bit for bit.
NORMAL_KEY_XOR = 0xD1B54A32D192ED03
SPLITMIX_GAMMA = 0x9E3779B97F4A7C15


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _normal_block(key: int, start: int, out: np.ndarray) -> None:
    idx = np.arange(start, start + out.shape[0], dtype=np.uint64)
    total = np.zeros(out.shape[0], dtype=np.int64)
    with np.errstate(over="ignore"):
        for j in range(3):
            counter = idx * np.uint64(3) + np.uint64(j + 1)
            z = _splitmix64(np.uint64(key) + counter * np.uint64(SPLITMIX_GAMMA))
            for field in range(4):
                total += ((z >> np.uint64(16 * field)) & np.uint64(0xFFFF)).astype(np.int64)
    centred = (total - 393210).astype(F32)
    out[:] = round_bf16(centred * F32(0.02 / 65536.0))


def normal_values(seed: int, offset: int, count: int) -> np.ndarray:
    """Elements [offset, offset+count) of the seeded N(0, 0.02) stream, bf16-rounded float32."""
    key = (seed ^ NORMAL_KEY_XOR) & MASK64
    out = np.empty(count, dtype=F32)
    starts = list(range(0, count, _LCG_BLOCK))
    if len(starts) <= 2:
        for b in starts:
            _normal_block(key, offset + b, out[b:b + _LCG_BLOCK])
    else:
        import concurrent.futures
        import os
        with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
            list(pool.map(lambda b: _normal_block(key, offset + b, out[b:b + _LCG_BLOCK]), starts))
    return out


def synthetic_layout(cfg: Pi05Config) -> Dict[str, Tuple[int, Tuple[int, ...]]]:
    """name -> (element offset in the LCG stream, shape) in generation order."""
    table: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
    cursor = 0

    def tensor(name, shape):
        nonlocal cursor
        table[name] = (cursor, tuple(shape))
        cursor += int(np.prod(shape))

    def linear(name, fan_in, fan_out, bias):
        tensor(name + ".weight", (fan_in, fan_out))
        if bias:
            tensor(name + ".bias", (fan_out,))

    vw = cfg.vision_width
    for i in range(cfg.vision_depth):
        p = f"vision.{i}"
        linear(p + ".q", vw, vw, True)
        linear(p + ".k", vw, vw, True)
        linear(p + ".v", vw, vw, True)
        linear(p + ".o", vw, vw, True)
        linear(p + ".fc1", vw, cfg.vision_mlp_dim, True)
        linear(p + ".fc2", cfg.vision_mlp_dim, vw, True)
    linear("vision.patch_embedding", cfg.patch_width, vw, True)
    tensor("vision.position_embedding", (cfg.patches_per_view, vw))
    linear("vision.projector", vw, cfg.language.width, True)
    tensor("token_embedding", (cfg.vocab_size, cfg.language.width))

    def attention(p, g):
        linear(p + ".q", g.width, g.num_heads * g.head_dim, False)
        linear(p + ".k", g.width, g.num_kv_heads * g.head_dim, False)
        linear(p + ".v", g.width, g.num_kv_heads * g.head_dim, False)
        linear(p + ".o", g.num_heads * g.head_dim, g.width, False)

    def mlp(p, g):
        linear(p + ".gate", g.width, g.mlp_dim, False)
        linear(p + ".up", g.width, g.mlp_dim, False)
        linear(p + ".down", g.mlp_dim, g.width, False)

    for i in range(cfg.language.depth):
        attention(f"language.{i}", cfg.language)
        mlp(f"language.{i}", cfg.language)
    aw = cfg.action_expert.width
    for i in range(cfg.action_expert.depth):
        linear(f"action.{i}.input_style", aw, 3 * aw, True)
        attention(f"action.{i}", cfg.action_expert)
        linear(f"action.{i}.post_style", aw, 3 * aw, True)
        mlp(f"action.{i}", cfg.action_expert)
    linear("action.final_style", aw, 3 * aw, True)
    linear("action_in", cfg.action_dim, aw, True)
    linear("action_out", aw, cfg.action_dim, True)
    linear("time_mlp_in", aw, aw, True)
    linear("time_mlp_out", aw, aw, True)
    table["__total__"] = (cursor, ())
    return table


class SyntheticWeights:
    """Lazily generated `Pi05Weights::synthetic(config, seed)`; tensors are float32 holding
    bf16 values, linear weights in the reference's [in, out] orientation."""

    def __init__(self, cfg: Pi05Config, seed: int = 0, dist: str = "lcg"):
        assert dist in ("lcg", "normal")
        self.cfg = cfg
        self.seed = seed
        self.dist = dist  # "lcg": the reference's uniform +-0.02 stream; "normal": N(0, 0.02)
        self._values = lcg_values if dist == "lcg" else normal_values
        self.layout = synthetic_layout(cfg)
        self._cache: Dict[str, np.ndarray] = {}
        self.cache_prefixes = ("action", "time_mlp", "vision.patch", "vision.position", "vision.projector")

    def get(self, name: str) -> np.ndarray:
        if name in self._cache:
            return self._cache[name]
        offset, shape = self.layout[name]
        value = self._values(self.seed, offset, int(np.prod(shape))).reshape(shape)
        if name.startswith(self.cache_prefixes):
            self._cache[name] = value
        return value

    def rows(self, name: str, row_ids) -> np.ndarray:
        """Selected rows of a 2-D tensor without generating the rest (token embedding)."""
        offset, shape = self.layout[name]
        width = shape[1]
        return np.stack([self._values(self.seed, offset + int(r) * width, width) for r in row_ids])

    def packed(self, names) -> np.ndarray:
        return np.concatenate([self.get(n + ".weight") for n in names], axis=1)

    def packed_bias(self, names) -> Optional[np.ndarray]:
        if (names[0] + ".bias") not in self.layout:
            return None
        return np.concatenate([self.get(n + ".bias") for n in names])


class TableWeights:
    """The same accessors over a name -> array table (what a checkpoint loader produces):
    float32 arrays holding the values the runtime is given, linear weights [in, out]."""

    def __init__(self, cfg: Pi05Config, table: Dict[str, np.ndarray]):
        self.cfg = cfg
        self.table = {k: np.asarray(v, dtype=F32) for k, v in table.items()}
        self.layout = {k: (0, v.shape) for k, v in self.table.items()}

    def get(self, name: str) -> np.ndarray:
        """Linear weights stay as given (the quantised precisions read them as float32);
        everything else is stored as bf16 by the runtime."""
        value = self.table[name]
        return value if (name.endswith(".weight") and value.ndim == 2) else round_bf16(value)

    def rows(self, name: str, row_ids) -> np.ndarray:
        return round_bf16(self.table[name][np.asarray(list(row_ids), dtype=np.int64)])

    def packed(self, names) -> np.ndarray:
        return np.concatenate([self.get(n + ".weight") for n in names], axis=1)

    def packed_bias(self, names) -> Optional[np.ndarray]:
        if (names[0] + ".bias") not in self.table:
            return None
        return np.concatenate([self.get(n + ".bias") for n in names])

    def layer_norm(self, name: str):
        if (name + ".weight") not in self.table:
            return None
        return round_bf16(self.table[name + ".weight"]), round_bf16(self.table[name + ".bias"])


# ----------------------------------------------------------------------------
# inputs of the bench / tests
# ----------------------------------------------------------------------------


def reference_image_pattern(cfg: Pi05Config) -> np.ndarray:
    """pi05_bench.rs:424-426: ((index*73 + index/11 + 19) & 0xff), NHWC u8."""
    n = cfg.num_views * cfg.image_size * cfg.image_size * 3
    idx = np.arange(n, dtype=np.int64)
    return ((idx * 73 + idx // 11 + 19) & 0xFF).astype(np.uint8).reshape(
        cfg.num_views, cfg.image_size, cfg.image_size, 3)


def synthetic_observation(cfg: Pi05Config, seed: int, token_count: int):
    """Seeded stand-in inputs with the benchmark's shapes and distributions:
    uniform u8 images (NHWC), uniform token ids, N(0,1) noise rounded to bf16."""
    rng = np.random.Generator(np.random.PCG64(seed))
    images = rng.integers(0, 256, size=(cfg.num_views, cfg.image_size, cfg.image_size, 3),
                          dtype=np.uint8)
    tokens = rng.integers(0, cfg.vocab_size, size=(token_count,), dtype=np.uint32)
    noise = round_bf16(rng.standard_normal((cfg.action_horizon, cfg.action_dim)).astype(F32))
    return images, tokens, noise


def sinusoidal_time_embedding(time: float, dimension: int, min_period: float,
                              max_period: float) -> np.ndarray:
    """math.rs:4-27 (float64 phase, float32 result)."""
    half = dimension // 2
    i = np.arange(half, dtype=np.float64)
    fraction = np.zeros(half) if half == 1 else i / (half - 1)
    lo, hi = float(F32(min_period)), float(F32(max_period))
    period = lo * (hi / lo) ** fraction
    phase = float(F32(time)) * (2.0 * math.pi) / period
    return np.concatenate([np.sin(phase), np.cos(phase)]).astype(F32)


def flow_times(steps: int) -> np.ndarray:
    """runtime.rs:821-838: t_s = 1 - s/S in float32."""
    s = np.arange(steps, dtype=F32)
    return (F32(1.0) - s / F32(steps)).astype(F32)


def rope_tables(theta: float, head_dim: int, positions: np.ndarray):
    """cos/sin of position * theta^(-pair/half) with float32 frequency and angle
    (fused.cuh:471-490: powf, float multiply, sincosf)."""
    half = head_dim // 2
    pair = np.arange(half, dtype=np.float64)
    freq = np.power(float(F32(theta)), -(pair / half)).astype(F32)
    angle = (positions.astype(F32)[:, None] * freq[None, :]).astype(F32)
    return np.cos(angle.astype(np.float64)).astype(F32), np.sin(angle.astype(np.float64)).astype(F32)


def patchify(images_u8: np.ndarray, cfg: Pi05Config) -> np.ndarray:
    """preprocess.cuh:65-98: [views*pp, 3*ps*ps] float32 (u8/255)*2-1, channel-major columns."""
    v, hgt, wid, _ = images_u8.shape
    ps, side = cfg.patch_size, cfg.patches_per_side
    x = images_u8.astype(F32) / F32(255.0) * F32(2.0) - F32(1.0)
    x = x.reshape(v, side, ps, side, ps, 3)          # view, py, dy, px, dx, c
    x = x.transpose(0, 1, 3, 5, 2, 4)                # view, py, px, c, dy, dx
    return np.ascontiguousarray(x.reshape(v * side * side, 3 * ps * ps))


# ----------------------------------------------------------------------------
# the forward
# ----------------------------------------------------------------------------


def _chunked_int_matmul(aq: np.ndarray, wq: np.ndarray) -> np.ndarray:
    """Exact integer matmul of int8-valued float32 operands: float32 GEMM per 1024-wide
    K chunk (every partial sum < 2^24, hence exact in any order), chunks summed in float64."""
    k = aq.shape[1]
    total = np.zeros((aq.shape[0], wq.shape[1]), dtype=np.float64)
    for k0 in range(0, k, 1024):
        total += (aq[:, k0:k0 + 1024] @ wq[k0:k0 + 1024]).astype(np.float64)
    return total


@dataclass
class OracleOptions:
    dtype: str = "bf16"               # "bf16" | "fp8" | "int8"
    storage: str = "bf16"             # 16-bit activation storage: "bf16" | "f16"
    act_scale: float = 0.05           # uniform static FP8 activation scale
    fp8_weight_scale: str = "channel"  # "channel" | "tensor"
    vision_round_scores: bool = False  # round SigLIP logits/probabilities to storage
    mqa_round_scores: bool = True      # cublas_adapter.cu:109-130 rounds both
    collect: bool = False              # keep named intermediates
    int8_act: str = "dynamic"          # "dynamic": per-row absmax/127 (w8a8.rs:86-98) | "static"
    # static activation scale per GEMM-input site, named as the reference's calibration table
    # (runtime.rs:35-81: "vision.layers.3.mlp_norm", "action.input", ...); sites not listed use
    # `act_scale`. Applies to FP8 and to INT8 with int8_act == "static".
    act_scales: Optional[Dict[str, float]] = None
    calibrate: bool = False            # record the absmax of every site's input in `amax`


class Pi05Oracle:
    def __init__(self, cfg: Pi05Config, weights: SyntheticWeights, options: OracleOptions):
        self.cfg = cfg
        self.w = weights
        self.o = options
        self.rs = round_bf16 if options.storage == "bf16" else round_f16
        self.trace: Dict[str, np.ndarray] = {}
        self._prepared: Dict[str, tuple] = {}
        self.int32_trace: Dict[str, np.ndarray] = {}
        self.amax: Dict[str, float] = {}

    def site_scale(self, site: Optional[str]) -> float:
        table = self.o.act_scales
        if table is not None and site is not None and site in table:
            return float(table[site])
        return float(self.o.act_scale)

    # ---- linear layers -----------------------------------------------------
    def _prepare(self, key: str, names) -> tuple:
        cacheable = key.startswith(("action", "time_mlp")) or getattr(self, "_prepare_all", False)
        if cacheable and key in self._prepared:
            return self._prepared[key]
        w = self.w.packed(names)
        if self.o.dtype == "bf16":
            prepared = (round_bf16(w), None)  # float32 (folded) checkpoint weights are stored as bf16
        elif self.o.dtype == "fp8":
            prepared = quantize_e4m3_channels(w, self.o.fp8_weight_scale)
        else:
            prepared = quantize_int8_channels(w)
        if cacheable:
            self._prepared[key] = prepared
        return prepared

    def linear(self, pre: np.ndarray, names, *, direct: bool = False, key: Optional[str] = None,
               site: Optional[str] = None):
        """GEMM output rounded to storage (no bias). `pre` is the float32 producer value;
        `direct` says the FP8 path quantises it straight from float32 (fused producer) instead
        of from the storage-rounded tensor. `site` names the input's static activation scale."""
        if isinstance(names, str):
            names = [names]
        key = key or "+".join(names)
        w, ws = self._prepare(key, names)
        if self.o.calibrate and site is not None:
            self.amax[site] = max(self.amax.get(site, 0.0), float(np.max(np.abs(self.rs(pre)))))
        if self.o.dtype == "bf16":
            out = self.rs(pre) @ w
        elif self.o.dtype == "fp8":
            scale = self.site_scale(site)
            src = pre if direct else self.rs(pre)
            xq = quantize_e4m3_static(src, scale)
            acc = xq @ w
            out = (acc * F32(scale)) * ws[None, :]
        elif self.o.int8_act == "static":
            scale = self.site_scale(site)
            xq = quantize_int8_static(self.rs(pre), scale)
            acc = _chunked_int_matmul(xq, w)
            if self.o.collect:
                self.int32_trace[key] = acc.astype(np.int64)
            out = (acc.astype(F32) * F32(scale)) * ws[None, :]
        else:
            xq, rs_ = quantize_rows_int8(self.rs(pre))
            acc = _chunked_int_matmul(xq, w)
            if self.o.collect:
                self.int32_trace[key] = acc.astype(np.int64)
            out = (acc.astype(F32) * rs_[:, None]) * ws[None, :]
        return self.rs(out.astype(F32))

    def bias(self, names):
        if isinstance(names, str):
            names = [names]
        return self.w.packed_bias(names)

    # ---- row ops -----------------------------------------------------------
    def layer_norm(self, x, name: Optional[str] = None):
        """normalization.cuh:96-122: w * (x - mean) * inv_std + b; synthetic weights have
        gamma 1 / beta 0 (weights.rs:262-263), checkpoint tables carry `<name>.weight/.bias`."""
        eps = F32(self.cfg.layer_norm_eps)
        mean = x.mean(axis=1, dtype=F32, keepdims=True)
        centered = x - mean
        var = (centered * centered).mean(axis=1, dtype=F32, keepdims=True)
        inv = F32(1.0) / np.sqrt(var + eps)
        params = self.w.layer_norm(name) if name is not None and hasattr(self.w, "layer_norm") else None
        if params is None:
            return (centered * inv).astype(F32)
        gamma, beta = params
        return ((gamma[None, :] * centered) * inv + beta[None, :]).astype(F32)

    def rms_norm(self, x):
        eps = F32(self.cfg.rms_norm_eps)
        ms = (x * x).mean(axis=1, dtype=F32, keepdims=True)
        return (x * (F32(1.0) / np.sqrt(ms + eps))).astype(F32)

    def ada_rms_norm(self, x, style):
        c = x.shape[1]
        return (self.rms_norm(x) * (F32(1.0) + style[None, :c]) + style[None, c:2 * c]).astype(F32)

    def attention(self, q, k, v, scale, round_scores):
        """q [Tq, heads, d]; k, v [Tk, kv_heads, d] -> [Tq, heads*d] in float32 (unrounded)."""
        tq, heads, d = q.shape
        kv_heads = k.shape[1]
        out = np.empty((tq, heads, d), dtype=F32)
        for h in range(heads):
            kh = k[:, h * kv_heads // heads]
            vh = v[:, h * kv_heads // heads]
            logits = (q[:, h] @ kh.T) * F32(scale)
            if round_scores:
                logits = self.rs(logits)
            m = logits.max(axis=1, keepdims=True)
            e = np.exp(logits - m).astype(F32)
            p = (e * (F32(1.0) / e.sum(axis=1, dtype=F32, keepdims=True))).astype(F32)
            if round_scores:
                p = self.rs(p)
            out[:, h] = p @ vh
        return out.reshape(tq, heads * d)

    def rope_split(self, qkv, g: GemmaVariant, positions):
        """fused.cuh:471-525 (no bias on the Gemma projections)."""
        t = qkv.shape[0]
        qw, kw = g.num_heads * g.head_dim, g.num_kv_heads * g.head_dim
        half = g.head_dim // 2
        cos, sin = rope_tables(self.cfg.rope_theta, g.head_dim, positions)
        q = qkv[:, :qw].reshape(t, g.num_heads, g.head_dim)
        k = qkv[:, qw:qw + kw].reshape(t, g.num_kv_heads, g.head_dim)
        v = qkv[:, qw + kw:].reshape(t, g.num_kv_heads, g.head_dim)

        def rotate(x):
            a, b = x[..., :half], x[..., half:]
            c, s = cos[:, None, :], sin[:, None, :]
            return np.concatenate([a * c - b * s, b * c + a * s], axis=-1).astype(F32)

        return self.rs(rotate(q)), self.rs(rotate(k)), self.rs(v)

    def _keep(self, name, value):
        if self.o.collect:
            self.trace[name] = np.array(value, copy=True)

    # ---- stages --------------------------------------------------------------
    def encode_vision(self, images_u8):
        cfg, rs = self.cfg, self.rs
        patches = patchify(images_u8, cfg)
        self._keep("patches", rs(patches))
        x = self.linear(patches, "vision.patch_embedding", site="vision.patch_input")
        pos = self.w.get("vision.position_embedding")
        reps = cfg.num_views
        x = rs((x + np.tile(pos, (reps, 1))) + self.bias("vision.patch_embedding")[None, :])
        self._keep("vision.embed", x)
        scale = 1.0 / math.sqrt(cfg.vision_head_dim)
        pp, heads, hd = cfg.patches_per_view, cfg.vision_heads, cfg.vision_head_dim
        n = self.layer_norm(x, "vision.0.norm1" if cfg.vision_depth else "vision.post_norm")
        for i in range(cfg.vision_depth):
            p = f"vision.{i}"
            names = [p + ".q", p + ".k", p + ".v"]
            qkv = self.linear(n, names, direct=True, site=f"vision.layers.{i}.attention_norm")
            qkv = rs(qkv + self.bias(names)[None, :])
            vw = cfg.vision_width
            attn = np.empty((x.shape[0], vw), dtype=F32)
            for view in range(cfg.num_views):
                rows = slice(view * pp, (view + 1) * pp)
                q = qkv[rows, :vw].reshape(pp, heads, hd)
                k = qkv[rows, vw:2 * vw].reshape(pp, heads, hd)
                v = qkv[rows, 2 * vw:].reshape(pp, heads, hd)
                attn[rows] = self.attention(q, k, v, scale, self.o.vision_round_scores)
            proj = self.linear(attn, p + ".o", site=f"vision.layers.{i}.attention_output")
            h = rs((proj + x) + self.bias(p + ".o")[None, :])
            n2 = self.layer_norm(h, p + ".norm2")
            f1 = self.linear(n2, p + ".fc1", direct=True, site=f"vision.layers.{i}.mlp_norm")
            act = gelu_tanh(f1 + self.bias(p + ".fc1")[None, :])
            f2 = self.linear(act, p + ".fc2", direct=True, site=f"vision.layers.{i}.mlp_activation")
            x = rs((f2 + h) + self.bias(p + ".fc2")[None, :])
            self._keep(f"vision.{i}.hidden", x)
            n = self.layer_norm(x, f"vision.{i + 1}.norm1" if i + 1 < cfg.vision_depth else "vision.post_norm")
        proj = self.linear(n, "vision.projector", direct=True, site="vision.post_norm")
        out = rs(proj + self.bias("vision.projector")[None, :])
        self._keep("vision.tokens", out)
        return out

    def embed_prefix(self, vision_tokens, token_ids):
        cfg = self.cfg
        width = cfg.language.width
        rows = np.zeros((len(token_ids), width), dtype=F32)
        valid = [i for i, t in enumerate(token_ids) if int(t) < cfg.vocab_size]
        if valid:
            got = self.w.rows("token_embedding", [int(token_ids[i]) for i in valid])
            rows[valid] = got * np.sqrt(F32(width))
        return np.concatenate([vision_tokens, self.rs(rows)], axis=0)

    def prefix_forward(self, prefix):
        cfg, rs, g = self.cfg, self.rs, self.cfg.language
        x = prefix
        ptok = x.shape[0]
        keys, values = [], []
        positions = np.arange(ptok)
        scale = 1.0 / math.sqrt(g.head_dim)
        for i in range(g.depth):
            p = f"language.{i}"
            n = self.rms_norm(x)
            qkv = self.linear(n, [p + ".q", p + ".k", p + ".v"], direct=True,
                              site=f"language.layers.{i}.attention_norm")
            q, k, v = self.rope_split(qkv, g, positions)
            keys.append(k)
            values.append(v)
            if i + 1 < g.depth:
                attn = self.attention(q, k, v, scale, self.o.mqa_round_scores)
                proj = self.linear(attn, p + ".o", site=f"language.layers.{i}.attention_output")
                h = rs(proj + x)
                n2 = self.rms_norm(h)
                gu = self.linear(n2, [p + ".gate", p + ".up"], direct=True,
                                 site=f"language.layers.{i}.mlp_norm")
                act = gelu_tanh(gu[:, :g.mlp_dim]) * gu[:, g.mlp_dim:]
                down = self.linear(act, p + ".down", direct=True,
                                   site=f"language.layers.{i}.mlp_activation")
                x = rs(down + h)
                self._keep(f"language.{i}.hidden", x)
        return keys, values

    def step_styles(self, step_time):
        cfg, rs = self.cfg, self.rs
        aw = cfg.action_expert.width
        emb = sinusoidal_time_embedding(step_time, aw, cfg.time_min_period, cfg.time_max_period)
        emb = rs(emb)[None, :]
        hidden = self.linear(emb, "time_mlp_in", site="time.input")
        hidden = silu(hidden + self.bias("time_mlp_in")[None, :])
        out = self.linear(hidden, "time_mlp_out", direct=True, site="time.hidden")
        cond = silu(out + self.bias("time_mlp_out")[None, :])

        def style(name):
            proj = self.linear(cond, name, direct=True, site="action.conditioning")
            return rs(proj + self.bias(name)[None, :])[0]

        attention = [style(f"action.{i}.input_style") for i in range(cfg.action_expert.depth)]
        mlp = [style(f"action.{i}.post_style") for i in range(cfg.action_expert.depth)]
        return attention, mlp, style("action.final_style")

    def denoise(self, noise, keys, values, prefix_tokens):
        cfg, rs, g = self.cfg, self.rs, self.cfg.action_expert
        aw, hz = g.width, cfg.action_horizon
        x = rs(noise.astype(F32))
        dt = F32(-1.0) / F32(cfg.num_flow_steps)
        positions = prefix_tokens + np.arange(hz)
        scale = 1.0 / math.sqrt(g.head_dim)
        for step, t in enumerate(flow_times(cfg.num_flow_steps)):
            style_attn, style_mlp, style_final = self.step_styles(float(t))
            h = self.linear(x, "action_in", site="action.input")
            h = rs(h + self.bias("action_in")[None, :])
            n = self.ada_rms_norm(h, style_attn[0])
            for i in range(g.depth):
                p = f"action.{i}"
                qkv = self.linear(n, [p + ".q", p + ".k", p + ".v"], direct=True,
                                  site=f"action.layers.{i}.attention_norm")
                q, k, v = self.rope_split(qkv, g, positions)
                kk = np.concatenate([keys[i], k], axis=0)
                vv = np.concatenate([values[i], v], axis=0)
                attn = self.attention(q, kk, vv, scale, self.o.mqa_round_scores)
                proj = self.linear(attn, p + ".o", site=f"action.layers.{i}.attention_output")
                h = rs(h + proj * style_attn[i][None, 2 * aw:])
                n = self.ada_rms_norm(h, style_mlp[i])
                gu = self.linear(n, [p + ".gate", p + ".up"], direct=True,
                                 site=f"action.layers.{i}.mlp_norm")
                act = gelu_tanh(gu[:, :g.mlp_dim]) * gu[:, g.mlp_dim:]
                down = self.linear(act, p + ".down", direct=True,
                                   site=f"action.layers.{i}.mlp_activation")
                h = rs(h + down * style_mlp[i][None, 2 * aw:])
                nxt = style_attn[i + 1] if i + 1 < g.depth else style_final
                n = self.ada_rms_norm(h, nxt)
            vel = self.linear(n, "action_out", direct=True, site="action.final_norm")
            vel = rs(vel + self.bias("action_out")[None, :])
            x = rs(x + dt * vel)
            self._keep(f"action.step{step}", x)
        return x

    def infer(self, images_u8, token_ids, noise):
        vision = self.encode_vision(images_u8)
        prefix = self.embed_prefix(vision, token_ids)
        self._keep("prefix", prefix)
        keys, values = self.prefix_forward(prefix)
        if self.o.collect:
            for i, (k, v) in enumerate(zip(keys, values)):
                self.trace[f"kv.{i}.k"] = k
                self.trace[f"kv.{i}.v"] = v
        return self.denoise(noise, keys, values, prefix.shape[0])


def infer(cfg: Pi05Config, seed: int, images_u8, token_ids, noise, weights_dist: str = "lcg",
          **options) -> np.ndarray:
    """One PI0.5 policy forward with `Pi05Weights::synthetic(cfg, seed)` weights: [H, action_dim]."""
    oracle = Pi05Oracle(cfg, SyntheticWeights(cfg, seed, weights_dist), OracleOptions(**options))
    return oracle.infer(images_u8, token_ids, noise)


# ----------------------------------------------------------------------------
# comparison metrics (pi05_bench.rs:87-121)
# ----------------------------------------------------------------------------


def compare(a: np.ndarray, b: np.ndarray) -> Dict[str, float]:
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    denom = math.sqrt(float(a @ a) * float(b @ b))
    diff = a - b
    return {
        "cosine": float(a @ b) / denom if denom > 0 else 1.0,
        "max_abs": float(np.max(np.abs(diff))),
        "mean_abs": float(np.mean(np.abs(diff))),
        "rmse": float(math.sqrt(np.mean(diff * diff))),
        "relative_l2": float(math.sqrt(diff @ diff) / max(math.sqrt(b @ b), 1e-30)),
        "bitwise_equal": bool(np.array_equal(a, b)),
    }
