"""Host-side mirror of the reference PI0.5 runtime interface over the C ABI.

Names follow the reference so its own call sites read the same:
  Pi05Config / GemmaVariantConfig   crates/apxinf-model/src/pi05/config.rs:5-109
  Pi05Runtime.random(...)           Pi05{Bf16,,Int8}CudaRuntime::new over
                                    Pi05Weights::synthetic (examples/pi05_bench.rs:901-990)
  capture_infer_rgb_u8              crates/apxinf-model/src/pi05/bf16_runtime.rs:457-575
  CapturedGraph.{update_raw_image_inputs, replay, replay_and_synchronize, output,
                 workspace_bytes, workspace_used_bytes}      bf16_runtime.rs:43-123
NumPy arrays are host buffers only; all arithmetic happens in libpi05_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from . import _lib
from ._abi_decls import EngineOptions, Gemma, HostTensor, ModelConfig, Observation, Signature
from ._lib import check, lib

DTYPES = {"bf16": 0, "fp8": 1, "int8": 2, "w8a8": 2}
LAYOUTS = {"nhwc": 0, "nchw": 1}
WEIGHT_DISTS = {"lcg": 0, "normal": 1}
INT8_ACTIVATIONS = {"dynamic": 0, "static": 1}


@dataclass(frozen=True)
class GemmaVariantConfig:
    width: int
    depth: int
    mlp_dim: int
    num_heads: int
    num_kv_heads: int
    head_dim: int


GEMMA_2B = GemmaVariantConfig(2048, 18, 16384, 8, 1, 256)
GEMMA_300M = GemmaVariantConfig(1024, 18, 4096, 8, 1, 256)


@dataclass(frozen=True)
class Pi05Config:
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
    language: GemmaVariantConfig = GEMMA_2B
    action_expert: GemmaVariantConfig = GEMMA_300M

    @property
    def patches_per_view(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    def to_c(self) -> ModelConfig:
        c = ModelConfig()
        for name in ("action_dim", "action_horizon", "max_token_len", "num_flow_steps",
                     "num_views", "image_size", "patch_size", "vision_width", "vision_depth",
                     "vision_mlp_dim", "vision_heads", "vision_head_dim", "vocab_size",
                     "rms_norm_eps", "layer_norm_eps", "rope_theta", "time_min_period",
                     "time_max_period"):
            setattr(c, name, getattr(self, name))
        for name in ("language", "action_expert"):
            g = getattr(self, name)
            setattr(c, name, Gemma(g.width, g.depth, g.mlp_dim, g.num_heads, g.num_kv_heads,
                                   g.head_dim))
        return c

    @staticmethod
    def from_any(other) -> "Pi05Config":
        """Accepts any object with the same attribute names (e.g. the oracle's config)."""
        kwargs = {}
        for name in Pi05Config.__dataclass_fields__:
            value = getattr(other, name)
            if name in ("language", "action_expert"):
                value = GemmaVariantConfig(value.width, value.depth, value.mlp_dim,
                                           value.num_heads, value.num_kv_heads, value.head_dim)
            kwargs[name] = value
        return Pi05Config(**kwargs)


def float_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    rounding = ((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((bits + rounding) >> np.uint32(16)).astype(np.uint16)


class CapturedGraph:
    """One prepared inference (fixed token count, image layout, batch) as a CUDA graph."""

    def __init__(self, runtime: "Pi05Runtime", handle: int, token_count: int, layout: str,
                 batch: int):
        self._rt = runtime
        self._h = handle
        self.token_count = token_count
        self.raw_image_layout = layout
        self.batch = batch
        cfg = runtime.config
        self.output_shape = (batch, cfg.action_horizon, cfg.action_dim)
        self._keep: List[np.ndarray] = []

    def close(self) -> None:
        if self._h:
            lib().pi05_graph_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _host_ptr(buf):
        if isinstance(buf, np.ndarray):
            return buf.ctypes.data
        return int(buf.data_ptr())  # a pinned torch tensor used as a host buffer

    def update_raw_image_inputs(self, images, token_ids, noise) -> None:
        """images u8 [batch, views, S, S, 3] (NHWC) or [batch, views, 3, S, S]; token ids
        u32 [batch, T]; noise float32 (rounded to bf16 here) or uint16 bf16 bits."""
        cfg = self._rt.config
        if isinstance(noise, np.ndarray) and noise.dtype != np.uint16:
            noise = float_to_bf16_bits(noise)
        if isinstance(images, np.ndarray):
            images = np.ascontiguousarray(images, dtype=np.uint8)
            assert images.size == self.batch * cfg.num_views * cfg.image_size ** 2 * 3
        if isinstance(token_ids, np.ndarray):
            token_ids = np.ascontiguousarray(token_ids, dtype=np.uint32)
            assert token_ids.size == self.batch * self.token_count
        if isinstance(noise, np.ndarray):
            noise = np.ascontiguousarray(noise)
            assert noise.size == self.batch * cfg.action_horizon * cfg.action_dim
        self._keep = [images, token_ids, noise]
        check(lib().pi05_graph_update_raw_image_inputs(
            self._h, self._host_ptr(images), self._host_ptr(token_ids), self._host_ptr(noise)),
            "pi05_graph_update_raw_image_inputs")

    def replay(self) -> None:
        check(lib().pi05_graph_replay(self._h), "pi05_graph_replay")

    def run_eager(self) -> None:
        check(lib().pi05_graph_run_eager(self._h), "pi05_graph_run_eager")

    def synchronize(self) -> None:
        check(lib().pi05_graph_sync(self._h), "pi05_graph_sync")

    def replay_and_synchronize(self) -> None:
        self.replay()
        self.synchronize()

    def output(self, out: Optional[np.ndarray] = None) -> np.ndarray:
        if out is None:
            out = np.empty(self.output_shape, dtype=np.float32)
        check(lib().pi05_graph_output(self._h, out.ctypes.data), "pi05_graph_output")
        return out

    def time_replays(self, iterations: int) -> np.ndarray:
        ms = np.zeros(iterations, dtype=np.float32)
        check(lib().pi05_graph_time_replays(self._h, iterations, ms.ctypes.data),
              "pi05_graph_time_replays")
        return ms

    def stage_times(self) -> Dict[str, float]:
        ms = np.zeros(3, dtype=np.float32)
        check(lib().pi05_graph_stage_times(self._h, ms.ctypes.data), "pi05_graph_stage_times")
        return {"vision": float(ms[0]), "prefix": float(ms[1]), "denoise": float(ms[2])}

    def time_launches(self, name: str):
        """(mean ms, count) of the launches called `name`, CUDA events on the engine stream."""
        mean = C.c_float(0.0)
        count = C.c_int32(0)
        check(lib().pi05_graph_time_launches(self._h, name.encode(), C.byref(mean), C.byref(count)),
              "pi05_graph_time_launches")
        return float(mean.value), int(count.value)

    def workspace_bytes(self) -> int:
        return int(lib().pi05_graph_workspace_bytes(self._h))

    def workspace_used_bytes(self) -> int:
        return int(lib().pi05_graph_workspace_used_bytes(self._h))

    def num_launches(self) -> int:
        return int(lib().pi05_graph_num_launches(self._h))

    def launch_names(self) -> List[str]:
        return [lib().pi05_graph_launch_name(self._h, i).decode()
                for i in range(self.num_launches())]

    def read_tensor(self, name: str, dtype=np.uint16) -> np.ndarray:
        size = C.c_size_t(0)
        check(lib().pi05_graph_read_tensor(self._h, name.encode(), None, 0, C.byref(size)),
              f"pi05_graph_read_tensor({name})")
        out = np.empty(size.value // np.dtype(dtype).itemsize, dtype=dtype)
        check(lib().pi05_graph_read_tensor(self._h, name.encode(), out.ctypes.data, size.value,
                                           C.byref(size)), f"pi05_graph_read_tensor({name})")
        return out

    def signature(self, name: str) -> Dict[str, object]:
        """Statistics of a named bf16 intermediate of the last run: the per-stage line of the
        reference's integrity probe (crates/apxinf-model/examples/pi05_integrity_probe.rs:19-51)."""
        sig = Signature()
        check(lib().pi05_graph_signature(self._h, name.encode(), C.byref(sig)),
              f"pi05_graph_signature({name})")
        return {"elements": int(sig.elements), "sum": sig.sum, "abs_checksum": sig.abs_checksum,
                "l2": sig.l2, "max_abs": sig.max_abs,
                "sample": np.array(sig.sample[:sig.sample_count], dtype=np.float32)}

    def update_patch_inputs(self, patches, token_ids, noise) -> None:
        """For graphs captured with `capture_infer_patches`: patches float32
        [batch, views * patches_per_view, 3 * patch_size**2] (VisionObservation::Patches,
        crates/apxinf-model/src/vla/mod.rs:14-19), token ids and noise as above."""
        cfg = self._rt.config
        if isinstance(noise, np.ndarray) and noise.dtype != np.uint16:
            noise = float_to_bf16_bits(noise)
        patches = np.ascontiguousarray(patches, dtype=np.float32)
        assert patches.size == (self.batch * cfg.num_views * cfg.patches_per_view
                                * 3 * cfg.patch_size ** 2)
        token_ids = np.ascontiguousarray(token_ids, dtype=np.uint32)
        assert token_ids.size == self.batch * self.token_count
        noise = np.ascontiguousarray(noise)
        assert noise.size == self.batch * cfg.action_horizon * cfg.action_dim
        self._keep = [patches, token_ids, noise]
        check(lib().pi05_graph_update_patch_inputs(
            self._h, patches.ctypes.data, token_ids.ctypes.data, noise.ctypes.data),
            "pi05_graph_update_patch_inputs")

    def infer_host(self, images, token_ids, noise) -> np.ndarray:
        """Host buffers in, host float32 action chunk out (the call a user makes)."""
        if self.raw_image_layout == "patches":
            self.update_patch_inputs(images, token_ids, noise)
        else:
            self.update_raw_image_inputs(images, token_ids, noise)
        self.replay()
        return self.output()


class Pi05Runtime:
    """Weights + stream on one GPU for one precision ("bf16" | "fp8" | "int8")."""

    def __init__(self, config: Pi05Config, dtype: str, handle: int, device: int):
        self.config = config
        self.dtype = dtype
        self.device = device
        self._h = handle

    @classmethod
    def random(cls, config=None, dtype: str = "bf16", seed: int = 0, device: int = 0,
               fp8_act_scale: float = 1.0, weights_dist: str = "lcg",
               int8_activations: str = "dynamic",
               activation_scales: Optional[Dict[str, float]] = None) -> "Pi05Runtime":
        """Seeded random weights. `weights_dist`: "lcg" (the reference generator, uniform
        +-0.02) or "normal" (N(0, 0.02)); `int8_activations`: "dynamic" (per-row, the
        reference) or "static" (per-tensor); `fp8_act_scale`: the uniform static activation
        scale (FP8, static INT8); `activation_scales`: per-site overrides by the reference's
        calibration names."""
        config = Pi05Config() if config is None else Pi05Config.from_any(config)
        if dtype not in DTYPES:
            raise ValueError(f"--dtype must be bf16, fp8 or int8, got {dtype}")
        if weights_dist not in WEIGHT_DISTS:
            raise ValueError(f"weights_dist must be lcg or normal, got {weights_dist}")
        if int8_activations not in INT8_ACTIVATIONS:
            raise ValueError(f"int8_activations must be dynamic or static, got {int8_activations}")
        c = config.to_c()
        options = EngineOptions(dtype=DTYPES[dtype], device=device, seed=seed,
                                act_scale=fp8_act_scale, weight_dist=WEIGHT_DISTS[weights_dist],
                                int8_activations=INT8_ACTIVATIONS[int8_activations])
        handle = C.c_void_p()
        check(lib().pi05_engine_create_ex(C.byref(c), C.byref(options), C.byref(handle)),
              "pi05_engine_create_ex")
        runtime = cls(config, "int8" if dtype == "w8a8" else dtype, handle.value, device)
        for site, scale in (activation_scales or {}).items():
            runtime.set_activation_scale(site, scale)
        return runtime

    @classmethod
    def from_tensors(cls, config, tensors, dtype: str = "bf16", device: int = 0,
                     fp8_act_scale: float = 1.0, int8_activations: str = "dynamic",
                     activation_scales: Optional[Dict[str, float]] = None) -> "Pi05Runtime":
        """Weights from host arrays instead of the generator: what the reference builds from a
        checkpoint (Static*Pi05Weights::from_host over Pi05Weights::from_map). `tensors` maps
        the synthetic layout's names to uint16 (bf16 bits) or float32 arrays, linear weights
        [in, out]; apxinf_b200.checkpoint.tensor_table produces it."""
        config = Pi05Config.from_any(config)
        if dtype not in DTYPES:
            raise ValueError(f"--dtype must be bf16, fp8 or int8, got {dtype}")
        keep, table = [], (HostTensor * len(tensors))()
        for slot, (name, value) in zip(table, tensors.items()):
            array = value if isinstance(value, np.ndarray) else value.data
            if array.dtype not in (np.uint16, np.float32):
                raise ValueError(f"tensor `{name}` must be uint16 (bf16 bits) or float32, got {array.dtype}")
            array = np.ascontiguousarray(array)
            keep.append(array)
            slot.name = name.encode()
            slot.data = array.ctypes.data
            slot.elements = array.size
            slot.dtype = 1 if array.dtype == np.float32 else 0
        c = config.to_c()
        options = EngineOptions(dtype=DTYPES[dtype], device=device, seed=0, act_scale=fp8_act_scale,
                                weight_dist=0, int8_activations=INT8_ACTIVATIONS[int8_activations])
        handle = C.c_void_p()
        code = lib().pi05_engine_create_from_tensors(C.byref(c), C.byref(options), table, len(tensors),
                                                     C.byref(handle))
        if code != 0:
            # the library names a missing or mis-sized tensor in its message
            detail = (lib().pi05_last_cuda_error() or b"").decode()
            raise _lib.Pi05Error(code, "pi05_engine_create_from_tensors", detail)
        runtime = cls(config, "int8" if dtype == "w8a8" else dtype, handle.value, device)
        for site, scale in (activation_scales or {}).items():
            runtime.set_activation_scale(site, scale)
        return runtime

    def set_activation_scale(self, site: str, scale: float) -> None:
        """Static activation scale of one GEMM-input site (reference calibration names,
        crates/apxinf-model/src/pi05/runtime.rs:35-81); applies to graphs captured afterwards."""
        check(lib().pi05_engine_set_activation_scale(self._h, site.encode(), float(scale)),
              f"pi05_engine_set_activation_scale({site})")

    def activation_scale(self, site: str) -> float:
        return float(lib().pi05_engine_activation_scale(self._h, site.encode()))

    def close(self) -> None:
        if self._h:
            lib().pi05_engine_destroy(self._h)
            self._h = 0

    def weight_bytes(self) -> int:
        return int(lib().pi05_engine_weight_bytes(self._h))

    def read_weight(self, name: str, dtype=np.uint16) -> np.ndarray:
        size = C.c_size_t(0)
        check(lib().pi05_engine_read_weight(self._h, name.encode(), None, 0, C.byref(size)),
              f"pi05_engine_read_weight({name})")
        out = np.empty(size.value // np.dtype(dtype).itemsize, dtype=dtype)
        check(lib().pi05_engine_read_weight(self._h, name.encode(), out.ctypes.data, size.value,
                                            C.byref(size)), f"pi05_engine_read_weight({name})")
        return out

    def capture_infer_rgb_u8(self, token_count: int, layout: str = "nhwc",
                             batch: int = 1) -> CapturedGraph:
        if layout not in LAYOUTS:
            raise ValueError(f"--image-input must be nhwc or nchw, got {layout}")
        handle = C.c_void_p()
        check(lib().pi05_engine_capture(self._h, token_count, LAYOUTS[layout], batch,
                                        C.byref(handle)), "pi05_engine_capture")
        return CapturedGraph(self, handle.value, token_count, layout, batch)

    def capture_infer_patches(self, token_count: int, batch: int = 1) -> CapturedGraph:
        """The same forward from ready-made fp32 patch rows (the reference's L0 entry
        `Model._infer_patches`, crates/apxinf-py/src/lib.rs:348-395)."""
        handle = C.c_void_p()
        check(lib().pi05_engine_capture(self._h, token_count, 2, batch, C.byref(handle)),
              "pi05_engine_capture")
        return CapturedGraph(self, handle.value, token_count, "patches", batch)


class PolicyRuntime:
    """The owning frontend over one Pi05Runtime: `infer` keeps one prepared plan keyed by
    (token count, image layout), rebuilds it when the observation's shape changes and runs
    eagerly when graph capture is unavailable — Pi05VlaRuntime::infer / prepare
    (crates/apxinf-model/src/pi05/vla_runtime.rs:393-495). The cache lives in the library
    (`pi05_runtime_infer`); this class only checks and passes host buffers."""

    def __init__(self, runtime: Pi05Runtime):
        self.runtime = runtime
        handle = C.c_void_p()
        check(lib().pi05_runtime_create(runtime._h, C.byref(handle)), "pi05_runtime_create")
        self._h = handle.value

    def close(self) -> None:
        if self._h:
            lib().pi05_runtime_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def infer(self, layout: str, image, token_ids: np.ndarray, noise: np.ndarray) -> np.ndarray:
        """`layout` "nhwc" | "nchw" (uint8 images) or "patches" (float32 patch rows); `noise`
        float32 or uint16 bf16 bits [horizon, action_dim]. Returns float32 [horizon, action_dim]."""
        c = self.runtime.config
        observation = Observation()
        observation.token_count = int(token_ids.size)
        tokens = np.ascontiguousarray(token_ids, dtype=np.uint32)
        observation.token_ids = tokens.ctypes.data
        if layout == "patches":
            image = np.ascontiguousarray(image, dtype=np.float32)
            expected = c.num_views * c.patches_per_view * 3 * c.patch_size ** 2
            observation.image_layout = 2
            observation.patches = image.ctypes.data
        else:
            if layout not in LAYOUTS:
                raise ValueError(f"--image-input must be nhwc or nchw, got {layout}")
            image = np.ascontiguousarray(image, dtype=np.uint8)
            expected = c.num_views * c.image_size * c.image_size * 3
            observation.image_layout = LAYOUTS[layout]
            observation.images = image.ctypes.data
        if image.size != expected:
            raise ValueError(f"observation image has {image.size} elements, expected {expected}")
        if noise.dtype == np.uint16:
            observation.noise_dtype = 1
        else:
            noise = np.ascontiguousarray(noise, dtype=np.float32)
            observation.noise_dtype = 0
        noise = np.ascontiguousarray(noise)
        if noise.size != c.action_horizon * c.action_dim:
            raise ValueError(f"noise has {noise.size} elements, expected {c.action_horizon * c.action_dim}")
        observation.noise = noise.ctypes.data
        out = np.empty((c.action_horizon, c.action_dim), dtype=np.float32)
        check(lib().pi05_runtime_infer(self._h, C.byref(observation), out.ctypes.data), "pi05_runtime_infer")
        return out

    def plan_info(self) -> Dict[str, int]:
        values = [C.c_int32(0) for _ in range(4)]
        check(lib().pi05_runtime_plan_info(self._h, *[C.byref(v) for v in values]), "pi05_runtime_plan_info")
        return {"token_count": values[0].value, "image_layout": values[1].value,
                "uses_graph": values[2].value, "builds": values[3].value}
