"""LeRobot / OpenPI PI0.5 SafeTensors checkpoints -> the engine's host tensor table.

Host-side mirror of the reference's checkpoint path:
  load_path / load_sharded        crates/apxinf-loader/src/safetensors.rs:63-167 (file, directory,
                                  `model.safetensors.index.json`, shard-path and index checks)
  config_from_json                Pi05Config::from_json_str, crates/apxinf-model/src/pi05/config.rs:141-175, 479-493
  tensor_table                    Pi05Weights::from_map, crates/apxinf-model/src/pi05/weights.rs:116-244
                                  (key map, [out, in] -> [in, out] transposes, patch-embedding
                                  reshape, `1 + w` RMSNorm fold into q/k/v and gate/up in float32,
                                  ada-norm `.dense` projections, token-embedding aliases,
                                  shape validation :588-700)
  calibration_scales              StaticFp8Calibration::from_json_str, crates/apxinf-model/src/pi05/fp8.rs:36-69,
                                  Pi05ActivationScales::from_calibration, runtime.rs:34-81
  resolve_precision               crates/apxinf-model/src/pi05/vla_runtime.rs:628-639
This module only prepares host arrays (NumPy); packing, quantisation and all model arithmetic
happen in libpi05_b200.so (`pi05_engine_create_from_tensors`).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import replace
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

from .engine import Pi05Config

ROOT = "paligemma_with_expert"
E4M3_MAX = 448.0


# Pi05Config::default() (config.rs:84-108): three views, 50-step chunks
DEFAULT_CONFIG = Pi05Config(num_views=3, action_horizon=50)


class CheckpointError(RuntimeError):
    pass


# ---------------------------------------------------------------------------------------------
# SafeTensors container
# ---------------------------------------------------------------------------------------------

class HostArray:
    """A tensor as stored: `bits` is uint16 (BF16 / F16 bit patterns) or float32, `kind` says which."""

    __slots__ = ("kind", "data")

    def __init__(self, kind: str, data: np.ndarray):
        assert kind in ("bf16", "f16", "f32")
        self.kind = kind
        self.data = data

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self.data.shape)

    def to_f32(self) -> np.ndarray:
        if self.kind == "f32":
            return self.data
        if self.kind == "f16":
            return self.data.view(np.float16).astype(np.float32)
        return (self.data.astype(np.uint32) << np.uint32(16)).view(np.float32)


_DTYPES = {"BF16": ("bf16", np.uint16), "F16": ("f16", np.uint16), "F32": ("f32", np.float32)}


def load_file(path: str) -> Dict[str, HostArray]:
    """One `.safetensors` file: 8-byte little-endian header length, JSON header, raw data."""
    try:
        size = os.path.getsize(path)
        handle = open(path, "rb")
    except OSError as error:
        raise CheckpointError(f"failed to open {path}: {error}")
    with handle:
        if size < 8:
            raise CheckpointError("file too small to be a SafeTensors file")
        (header_len,) = struct.unpack("<Q", handle.read(8))
        if size < 8 + header_len:
            raise CheckpointError(f"file too small: expected at least {8 + header_len} bytes, got {size}")
        try:
            header = json.loads(handle.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise CheckpointError(f"JSON parse error: {error}")
    body = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + header_len) if size > 8 + header_len \
        else np.zeros(0, np.uint8)
    tensors: Dict[str, HostArray] = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        dtype = entry.get("dtype")
        if dtype not in _DTYPES:
            raise CheckpointError(f"tensor `{name}`: unsupported dtype {dtype}")
        kind, np_type = _DTYPES[dtype]
        shape = tuple(int(d) for d in entry["shape"])
        begin, end = (int(v) for v in entry["data_offsets"])
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if end - begin != count * np.dtype(np_type).itemsize or end > body.size:
            raise CheckpointError(f"tensor `{name}`: data range {begin}..{end} does not match shape {list(shape)}")
        tensors[name] = HostArray(kind, body[begin:end].view(np_type).reshape(shape))
    return tensors


def load_sharded(index_path: str) -> Dict[str, HostArray]:
    try:
        with open(index_path, "r", encoding="utf-8") as handle:
            index = json.load(handle)
    except (OSError, json.JSONDecodeError) as error:
        raise CheckpointError(f"invalid SafeTensors index {index_path}: {error}")
    weight_map = index.get("weight_map") or {}
    if not weight_map:
        raise CheckpointError(f"SafeTensors index {index_path} has an empty weight_map")
    parent = os.path.dirname(index_path) or "."
    tensors: Dict[str, HostArray] = {}
    for shard in sorted(set(weight_map.values())):
        if os.path.isabs(shard) or ".." in shard.replace("\\", "/").split("/"):
            raise CheckpointError(f"unsafe shard path `{shard}` in {index_path}")
        for name, tensor in load_file(os.path.join(parent, shard)).items():
            expected = weight_map.get(name)
            if expected is None:
                continue
            if expected != shard:
                raise CheckpointError(
                    f"tensor `{name}` was found in `{shard}`, index assigns it to `{expected}`")
            if name in tensors:
                raise CheckpointError(f"duplicate indexed tensor `{name}`")
            tensors[name] = tensor
    missing = [name for name in weight_map if name not in tensors][:8]
    if missing:
        raise CheckpointError("SafeTensors shards are missing indexed tensors: " + ", ".join(missing))
    return tensors


def load_path(path: str) -> Dict[str, HostArray]:
    """A file, an index json, or a directory holding either (or exactly one `.safetensors`)."""
    if os.path.isdir(path):
        index = os.path.join(path, "model.safetensors.index.json")
        if os.path.isfile(index):
            return load_sharded(index)
        model = os.path.join(path, "model.safetensors")
        if os.path.isfile(model):
            return load_file(model)
        candidates = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
        if len(candidates) == 1:
            return load_file(os.path.join(path, candidates[0]))
        if not candidates:
            raise CheckpointError(f"no SafeTensors model or index in {path}")
        raise CheckpointError(f"multiple SafeTensors files but no model.safetensors.index.json in {path}")
    if path.endswith(".json"):
        return load_sharded(path)
    return load_file(path)


def save_file(path: str, tensors: Dict[str, HostArray]) -> None:
    """Writer for the same container (used to build test checkpoints and to export)."""
    names = {"bf16": "BF16", "f16": "F16", "f32": "F32"}
    header, offset = {}, 0
    for name, tensor in tensors.items():
        nbytes = tensor.data.size * tensor.data.dtype.itemsize
        header[name] = {"dtype": names[tensor.kind], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(raw)))
        handle.write(raw)
        for tensor in tensors.values():
            handle.write(np.ascontiguousarray(tensor.data).tobytes())


# ---------------------------------------------------------------------------------------------
# config.json
# ---------------------------------------------------------------------------------------------

def _unsigned(v: dict, names: Iterable[str], default: int) -> int:
    for name in names:
        value = v.get(name)
        if isinstance(value, int) and not isinstance(value, bool) and value >= 0:
            return value
    return default


def config_from_json(raw: str) -> Pi05Config:
    """LeRobot's policy config with the OpenPI aliases; architecture constants keep the PI0.5
    values. `discrete_state_input` does not change the policy forward and is not kept."""
    try:
        v = json.loads(raw)
    except json.JSONDecodeError as error:
        raise CheckpointError(f"pi05 config json: {error}")
    base = DEFAULT_CONFIG
    num_views = base.num_views
    if isinstance(v.get("num_views"), int):
        num_views = v["num_views"]
    elif isinstance(v.get("input_features"), dict):
        visual = sum(1 for f in v["input_features"].values()
                     if isinstance(f, dict) and f.get("type") == "VISUAL")
        if visual > 0:
            num_views = visual
    image_size = base.image_size
    resolution = v.get("image_resolution")
    if isinstance(resolution, list) and resolution and isinstance(resolution[0], int):
        image_size = resolution[0]

    def real(name, default):
        value = v.get(name)
        return float(np.float32(value)) if isinstance(value, (int, float)) and not isinstance(value, bool) \
            else default

    cfg = replace(
        base,
        action_dim=_unsigned(v, ("max_action_dim", "action_dim"), base.action_dim),
        action_horizon=_unsigned(v, ("chunk_size", "action_horizon"), base.action_horizon),
        max_token_len=_unsigned(v, ("tokenizer_max_length", "max_token_len"), base.max_token_len),
        num_flow_steps=_unsigned(v, ("num_inference_steps", "num_flow_steps"), base.num_flow_steps),
        num_views=num_views, image_size=image_size,
        time_min_period=real("min_period", base.time_min_period),
        time_max_period=real("max_period", base.time_max_period))
    validate_config(cfg)
    return cfg


def validate_config(cfg: Pi05Config) -> None:
    """Pi05Config::validate (config.rs:433-459), same texts."""
    if cfg.patch_size <= 0 or cfg.image_size % cfg.patch_size != 0:
        raise CheckpointError(f"pi05 image size {cfg.image_size} is not divisible by patch size {cfg.patch_size}")
    if cfg.action_horizon == 0 or cfg.action_horizon > 50:
        raise CheckpointError(f"pi05 action_horizon must be in 1..=50, got {cfg.action_horizon}")
    if cfg.num_flow_steps == 0:
        raise CheckpointError("pi05 num_flow_steps must be non-zero")
    lg, ac = cfg.language, cfg.action_expert
    if (lg.depth, lg.num_heads, lg.num_kv_heads, lg.head_dim) != \
            (ac.depth, ac.num_heads, ac.num_kv_heads, ac.head_dim):
        raise CheckpointError("pi05 language and action experts must share depth/head geometry")


def artifact_root(path: str) -> str:
    return path if os.path.isdir(path) else (os.path.dirname(path) or ".")


def load_config(path: str) -> Pi05Config:
    """`config.json` beside the checkpoint, else the defaults (crates/apxinf-py/src/lib.rs:95-107)."""
    config_path = os.path.join(artifact_root(path), "config.json")
    if os.path.isfile(config_path):
        with open(config_path, "r", encoding="utf-8") as handle:
            return config_from_json(handle.read())
    return DEFAULT_CONFIG


# ---------------------------------------------------------------------------------------------
# key map
# ---------------------------------------------------------------------------------------------

def _bf16_round(x: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((bits + (((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF))) >> np.uint32(16)).astype(np.uint16)


def normalize_lerobot_prefix(tensors: Dict[str, HostArray]) -> Dict[str, HostArray]:
    canonical, wrapped = ROOT + ".", "model." + ROOT + "."
    if any(k.startswith(canonical) for k in tensors) or not any(k.startswith(wrapped) for k in tensors):
        return tensors
    return {(k[len("model."):] if k.startswith("model.") else k): v for k, v in tensors.items()}


class _Taker:
    def __init__(self, tensors: Dict[str, HostArray]):
        self.tensors = dict(tensors)

    def take(self, name: str) -> HostArray:
        if name not in self.tensors:
            raise CheckpointError(f"missing π0.5 weight `{name}`")
        return self.tensors.pop(name)

    def take_any(self, names: List[str]) -> HostArray:
        for name in names:
            if name in self.tensors:
                return self.tensors.pop(name)
        raise CheckpointError("missing π0.5 weight (accepted aliases: " + ", ".join(names) + ")")


def _transpose(tensor: HostArray) -> HostArray:
    if tensor.data.ndim != 2:
        raise CheckpointError(f"π0.5 linear weight must be 2D, got shape {list(tensor.shape)}")
    return HostArray(tensor.kind, np.ascontiguousarray(tensor.data.T))


def _add_one(tensor: HostArray) -> np.ndarray:
    """`1 + w` in the tensor's own type (weights.rs:561-590), returned as float32 values."""
    value = tensor.to_f32() + np.float32(1.0)
    if tensor.kind == "bf16":
        return (_bf16_round(value).astype(np.uint32) << np.uint32(16)).view(np.float32)
    if tensor.kind == "f16":
        return value.astype(np.float16).astype(np.float32)
    return value


def _fold(linear: HostArray, scale: np.ndarray, name: str) -> HostArray:
    """Rows of the [in, out] weight times the per-input multiplier, in float32 (weights.rs:596-612)."""
    if linear.data.ndim != 2 or scale.shape != (linear.shape[0],):
        raise CheckpointError(f"π0.5 input-scale fold mismatch: weight {list(linear.shape)}, "
                              f"scale {list(scale.shape)} ({name})")
    return HostArray("f32", linear.to_f32() * scale[:, None])


def tensor_table(cfg: Pi05Config, tensors: Dict[str, HostArray]) -> Dict[str, HostArray]:
    """Checkpoint tensors -> the engine's names, [in, out] orientation, folds applied, shapes
    checked. F16 tensors are widened to float32 (the engine takes BF16 or float32)."""
    t = _Taker(normalize_lerobot_prefix(tensors))
    out: Dict[str, HostArray] = {}

    def linear(dst: str, src: str, bias: bool, fan_in: int, fan_out: int, fold: Optional[np.ndarray] = None):
        weight = _transpose(t.take(src + ".weight"))
        if fold is not None:
            weight = _fold(weight, fold, src)
        if weight.shape != (fan_in, fan_out):
            raise CheckpointError(f"{dst}: expected weight shape [{fan_in}, {fan_out}], got {list(weight.shape)}")
        out[dst + ".weight"] = weight
        if bias:
            b = t.take(src + ".bias")
            if b.shape != (fan_out,):
                raise CheckpointError(f"{dst}: expected bias shape [{fan_out}], got {list(b.shape)}")
            out[dst + ".bias"] = b

    def layer_norm(dst: str, src: str, width: int):
        for part in ("weight", "bias"):
            value = t.take(f"{src}.{part}")
            if value.shape != (width,):
                raise CheckpointError(f"{dst}.{part}: expected shape [{width}], got {list(value.shape)}")
            out[f"{dst}.{part}"] = value

    vw = cfg.vision_width
    vp = f"{ROOT}.paligemma.model.vision_tower.vision_model"
    for i in range(cfg.vision_depth):
        p, d = f"{vp}.encoder.layers.{i}", f"vision.{i}"
        layer_norm(d + ".norm1", p + ".layer_norm1", vw)
        linear(d + ".q", p + ".self_attn.q_proj", True, vw, vw)
        linear(d + ".k", p + ".self_attn.k_proj", True, vw, vw)
        linear(d + ".v", p + ".self_attn.v_proj", True, vw, vw)
        linear(d + ".o", p + ".self_attn.out_proj", True, vw, vw)
        layer_norm(d + ".norm2", p + ".layer_norm2", vw)
        linear(d + ".fc1", p + ".mlp.fc1", True, vw, cfg.vision_mlp_dim)
        linear(d + ".fc2", p + ".mlp.fc2", True, cfg.vision_mlp_dim, vw)

    patch_name = f"{vp}.embeddings.patch_embedding.weight"
    patch = t.take(patch_name)
    patch_width = 3 * cfg.patch_size * cfg.patch_size
    if patch.data.size != vw * patch_width:
        raise CheckpointError(f"{patch_name}: expected {vw * patch_width} elements, got {patch.data.size}")
    out["vision.patch_embedding.weight"] = _transpose(HostArray(patch.kind, patch.data.reshape(vw, patch_width)))
    out["vision.patch_embedding.bias"] = t.take(f"{vp}.embeddings.patch_embedding.bias")
    position = t.take(f"{vp}.embeddings.position_embedding.weight")
    if position.shape != (cfg.patches_per_view, vw):
        raise CheckpointError(f"position_embedding: expected shape [{cfg.patches_per_view}, {vw}], "
                              f"got {list(position.shape)}")
    out["vision.position_embedding"] = position
    layer_norm("vision.post_norm", f"{vp}.post_layernorm", vw)
    lg, ac = cfg.language, cfg.action_expert
    linear("vision.projector", f"{ROOT}.paligemma.model.multi_modal_projector.linear", True, vw, lg.width)
    embedding = t.take_any([f"{ROOT}.paligemma.model.language_model.embed_tokens.weight",
                            f"{ROOT}.paligemma.lm_head.weight"])
    if embedding.shape != (cfg.vocab_size, lg.width):
        raise CheckpointError(f"token_embedding: expected shape [{cfg.vocab_size}, {lg.width}], "
                              f"got {list(embedding.shape)}")
    out["token_embedding"] = embedding

    def attention(dst, src, g, fold=None):
        qw = g.num_heads * g.head_dim
        kw = g.num_kv_heads * g.head_dim
        linear(dst + ".q", src + ".self_attn.q_proj", False, g.width, qw, fold)
        linear(dst + ".k", src + ".self_attn.k_proj", False, g.width, kw, fold)
        linear(dst + ".v", src + ".self_attn.v_proj", False, g.width, kw, fold)
        linear(dst + ".o", src + ".self_attn.o_proj", False, qw, g.width)

    def mlp(dst, src, g, fold=None):
        linear(dst + ".gate", src + ".mlp.gate_proj", False, g.width, g.mlp_dim, fold)
        linear(dst + ".up", src + ".mlp.up_proj", False, g.width, g.mlp_dim, fold)
        linear(dst + ".down", src + ".mlp.down_proj", False, g.mlp_dim, g.width)

    lp = f"{ROOT}.paligemma.model.language_model"
    for i in range(lg.depth):
        p = f"{lp}.layers.{i}"
        attention_scale = _add_one(t.take(p + ".input_layernorm.weight"))
        mlp_scale = _add_one(t.take(p + ".post_attention_layernorm.weight"))
        attention(f"language.{i}", p, lg, attention_scale)
        mlp(f"language.{i}", p, lg, mlp_scale)
    ap = f"{ROOT}.gemma_expert.model"
    for i in range(ac.depth):
        p = f"{ap}.layers.{i}"
        linear(f"action.{i}.input_style", p + ".input_layernorm.dense", True, ac.width, 3 * ac.width)
        attention(f"action.{i}", p, ac)
        linear(f"action.{i}.post_style", p + ".post_attention_layernorm.dense", True, ac.width, 3 * ac.width)
        mlp(f"action.{i}", p, ac)
    # the language model's final norm is read (and required) by the reference but feeds nothing
    # in the policy forward: the prefix only leaves its keys and values behind
    t.take(f"{lp}.norm.weight")
    linear("action.final_style", f"{ap}.norm.dense", True, ac.width, 3 * ac.width)
    linear("action_in", "action_in_proj", True, cfg.action_dim, ac.width)
    linear("action_out", "action_out_proj", True, ac.width, cfg.action_dim)
    linear("time_mlp_in", "time_mlp_in", True, ac.width, ac.width)
    linear("time_mlp_out", "time_mlp_out", True, ac.width, ac.width)
    return {name: (HostArray("f32", v.to_f32()) if v.kind == "f16" else v) for name, v in out.items()}


# ---------------------------------------------------------------------------------------------
# FP8 calibration and precision policy
# ---------------------------------------------------------------------------------------------

def calibration_from_json(raw: str) -> Dict[str, float]:
    """`{name: scale}`, a nested `scales` object, or entries `{scale: x}` / `{amax: x}`."""
    try:
        root = json.loads(raw)
    except json.JSONDecodeError as error:
        raise CheckpointError(f"π0.5 FP8 calibration JSON: {error}")
    values = root.get("scales", root) if isinstance(root, dict) else root
    if not isinstance(values, dict):
        raise CheckpointError("π0.5 FP8 calibration must be a JSON object")
    scales: Dict[str, float] = {}
    for name, value in values.items():
        scale = None
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            scale = float(value)
        elif isinstance(value, dict):
            if isinstance(value.get("scale"), (int, float)):
                scale = float(value["scale"])
            elif isinstance(value.get("amax"), (int, float)):
                scale = float(value["amax"]) / E4M3_MAX
        if scale is None:
            raise CheckpointError(f"π0.5 FP8 calibration entry `{name}` has no numeric scale or amax")
        scale = float(np.float32(scale))
        if not np.isfinite(scale) or scale <= 0.0:
            raise CheckpointError(f"π0.5 FP8 calibration entry `{name}` has invalid scale {scale}")
        scales[name] = scale
    return scales


def site_names(cfg: Pi05Config) -> List[str]:
    """In the order Pi05ActivationScales::from_calibration resolves them (runtime.rs:39-80)."""
    parts = ("attention_norm", "attention_output", "mlp_norm", "mlp_activation")
    names = [f"vision.layers.{i}.{p}" for i in range(cfg.vision_depth) for p in parts]
    names += [f"language.layers.{i}.{p}" for i in range(cfg.language.depth) for p in parts]
    names += [f"action.layers.{i}.{p}" for i in range(cfg.action_expert.depth) for p in parts]
    names += ["vision.patch_input", "vision.post_norm", "action.input", "time.input", "time.hidden",
              "action.conditioning", "action.final_norm"]
    return names


def calibration_scales(cfg: Pi05Config, calibration: Dict[str, float]) -> Dict[str, float]:
    """Every activation-scale site of the graph from a named table; the first one missing raises."""
    resolved = {}
    for name in site_names(cfg):
        if name not in calibration:
            raise CheckpointError(f"missing π0.5 FP8 activation scale `{name}`")
        resolved[name] = calibration[name]
    return resolved


def resolve_precision(requested: str, sm: int, has_fp8_artifacts: bool) -> str:
    if requested != "auto":
        return requested
    if sm >= 100 and has_fp8_artifacts:
        return "fp8"
    if 80 <= sm < 100:
        return "int8"
    return "bf16"
