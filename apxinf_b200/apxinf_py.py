"""`apxinf_py.Model` over libpi05_b200: the L0/L1 bare-model interface of the reference's PyO3
extension (crates/apxinf-py/src/lib.rs:196-500, stub crates/apxinf-py/apxinf_py.pyi), same
method names, argument order, shapes, dtypes and error texts, so code written against
`apxinf_py` runs on this library with `from apxinf_b200 import apxinf_py`.

Both constructors end in the same library calls: `Model.random` (seeded weights generated on the
device) and `Model.load` (a LeRobot / OpenPI SafeTensors checkpoint read by
apxinf_b200.checkpoint). Inference goes through the library's owning frontend
(`pi05_runtime_infer`): one cached prepared plan per (token count, input kind), like
Pi05VlaRuntime (crates/apxinf-model/src/pi05/vla_runtime.rs:393-495).
"""
from __future__ import annotations

import os
from dataclasses import replace
from typing import Optional

import numpy as np

from . import checkpoint as _checkpoint
from ._lib import lib as _lib
from .engine import Pi05Config, Pi05Runtime, PolicyRuntime

__version__ = "0.1.0"

_PRECISIONS = {"bf16": "bf16", "fp8": "fp8", "int8": "int8", "w8a8": "int8"}


def _parse_device(device: str) -> int:
    # crates/apxinf-py/src/lib.rs:40-66: "cuda", "cuda:N"; "cpu" is a reference CPU backend
    if device == "cuda":
        return 0
    if device.startswith("cuda:") and device[5:].isdigit():
        return int(device[5:])
    raise ValueError(f"apxinf_py: unsupported device `{device}` (expected `cuda:N`)")


class Model:
    """A pi05 model handle exposing L0/L1 bare-model inference."""

    def __init__(self, runtime: Pi05Runtime, config: Pi05Config, device: int):
        self._rt = runtime
        self._config = config
        self._device = device
        self._frontend = PolicyRuntime(runtime)

    # ---- construction -------------------------------------------------------------------
    @staticmethod
    def load(model: str, path: str, device: str = "cuda:0", precision: str = "auto",
             calibration: Optional[str] = None, tactics: Optional[str] = None,
             action_horizon: Optional[int] = None) -> "Model":
        """A checkpoint directory, `.safetensors` file or index (crates/apxinf-py/src/lib.rs:208-247,
        load_pi05 in crates/apxinf-model/src/pi05/vla_runtime.rs:497-625). `precision` "auto"
        picks fp8 when both a calibration and a tactics file are present (given, or
        `calibration.json` / `tactics.json` beside the checkpoint), else bf16 on this hardware.
        FP8 needs the calibration (one scale per named activation site) and, like the
        reference, refuses to run without a tactics file — whose content is not used here:
        this library plans its own kernels. `action_horizon` overrides `config.json`."""
        if model not in ("pi05", "pi0.5"):
            raise ValueError(f"apxinf_py.load: unknown model `{model}`")
        if precision not in ("auto",) + tuple(_PRECISIONS):
            raise ValueError(f"apxinf_py: unsupported precision `{precision}` "
                             "(expected `auto`, `bf16`, `fp8` or `int8`)")
        index = _parse_device(device)
        path = os.fspath(path)
        try:
            config = _checkpoint.load_config(path)
            if action_horizon is not None:
                config = replace(config, action_horizon=int(action_horizon))
                _checkpoint.validate_config(config)
            root = _checkpoint.artifact_root(path)

            def artifact(given, name):
                if given is not None:
                    return os.fspath(given)
                candidate = os.path.join(root, name)
                return candidate if os.path.isfile(candidate) else None

            calibration_path = artifact(calibration, "calibration.json")
            tactics_path = artifact(tactics, "tactics.json")
            resolved = _checkpoint.resolve_precision(
                precision if precision == "auto" else _PRECISIONS[precision],
                _lib().pi05_device_sm(index), calibration_path is not None and tactics_path is not None)
            scales = None
            if resolved == "fp8":
                if calibration_path is None:
                    raise RuntimeError("FP8 PI0.5 requires LoadOptions.calibration_path or calibration.json")
                with open(calibration_path, "r", encoding="utf-8") as handle:
                    table = _checkpoint.calibration_from_json(handle.read())
                scales = _checkpoint.calibration_scales(config, table)
                if tactics_path is None:
                    raise RuntimeError("FP8 PI0.5 requires LoadOptions.tuning_path or tactics.json")
            tensors = _checkpoint.tensor_table(config, _checkpoint.load_path(path))
        except _checkpoint.CheckpointError as error:
            raise RuntimeError(str(error))
        runtime = Pi05Runtime.from_tensors(config, tensors, dtype=resolved, device=index,
                                           activation_scales=scales)
        return Model(runtime, config, index)

    @staticmethod
    def random(model: str, device: str = "cuda:0", precision: str = "bf16", num_views: int = 2,
               image_size: int = 224, action_horizon: int = 10, action_dim: int = 32,
               num_flow_steps: int = 10, max_token_len: int = 200,
               calibration: Optional[str] = None, tactics: Optional[str] = None,
               seed: int = 0) -> "Model":
        """Synthetic weights from `seed` (crates/apxinf-py/src/lib.rs:265-343). `calibration` may
        be "uniform:<scale>" (one FP8 activation scale everywhere) or the path of a calibration
        json (one scale per named activation site); `tactics` is accepted and ignored (there is
        no tuning database here)."""
        if model not in ("pi05", "pi0.5"):
            raise ValueError(f"apxinf_py.random: unknown model `{model}`")
        if precision not in _PRECISIONS:
            raise ValueError(f"apxinf_py: unsupported precision `{precision}` "
                             "(expected `bf16`, `fp8` or `int8`)")
        index = _parse_device(device)
        scale, scales = 1.0, None
        config = Pi05Config(num_views=num_views, image_size=image_size,
                            action_horizon=action_horizon, action_dim=action_dim,
                            num_flow_steps=num_flow_steps, max_token_len=max_token_len)
        if calibration is not None and calibration.startswith("uniform:"):
            try:
                scale = float(calibration[len("uniform:"):])
            except ValueError:
                raise ValueError(f"apxinf_py.random: invalid uniform FP8 scale in `{calibration}`")
        elif calibration is not None:
            # a calibration json: one scale per named activation site, all of them required
            try:
                with open(calibration, "r", encoding="utf-8") as handle:
                    scales = _checkpoint.calibration_scales(config, _checkpoint.calibration_from_json(handle.read()))
            except (OSError, _checkpoint.CheckpointError) as error:
                raise RuntimeError(str(error))
        runtime = Pi05Runtime.random(config, dtype=_PRECISIONS[precision], seed=seed, device=index,
                                     fp8_act_scale=scale, activation_scales=scales)
        return Model(runtime, config, index)

    # ---- inference ----------------------------------------------------------------------
    def _validate_tokens(self, token_ids) -> np.ndarray:
        if not isinstance(token_ids, np.ndarray) or token_ids.dtype != np.uint32 or \
                not token_ids.flags.c_contiguous or token_ids.ndim != 1:
            raise ValueError("apxinf_py.infer: token_ids must be C-contiguous uint32")
        if token_ids.size == 0:
            raise ValueError("apxinf_py.infer: token_ids must be non-empty")
        if token_ids.size > self._config.max_token_len:
            raise ValueError(f"apxinf_py.infer: token_ids length {token_ids.size} exceeds "
                             f"max_token_len {self._config.max_token_len}")
        return token_ids

    def _validate_noise(self, noise) -> np.ndarray:
        expected = (self._config.action_horizon, self._config.action_dim)
        if not isinstance(noise, np.ndarray) or noise.shape != expected:
            got = list(getattr(noise, "shape", ()))
            raise ValueError(f"apxinf_py.infer: noise expected shape [{expected[0]}, {expected[1]}], "
                             f"got {got}")
        if noise.dtype != np.float32 or not noise.flags.c_contiguous:
            raise ValueError("apxinf_py.infer: noise must be C-contiguous float32")
        return noise

    def _infer_patches(self, patches, token_ids, noise) -> np.ndarray:
        """L0: float32 patches [num_views * patches_per_view, 3 * patch_size^2]; returns the
        normalized-domain action float32 [action_horizon, action_dim]."""
        c = self._config
        expected = (c.num_views * c.patches_per_view, 3 * c.patch_size ** 2)
        if not isinstance(patches, np.ndarray) or patches.shape != expected:
            got = list(getattr(patches, "shape", ()))
            raise ValueError(f"apxinf_py._infer_patches: patches expected shape "
                             f"[{expected[0]}, {expected[1]}], got {got}")
        if patches.dtype != np.float32 or not patches.flags.c_contiguous:
            raise ValueError("apxinf_py._infer_patches: patches must be C-contiguous float32")
        tokens = self._validate_tokens(token_ids)
        noise = self._validate_noise(noise)
        return self._frontend.infer("patches", patches, tokens, noise)

    def infer_rgb(self, rgb_u8, layout: str, token_ids, noise) -> np.ndarray:
        """L1: resized RGB uint8, `layout` "nhwc" or "nchw"; returns the normalized-domain
        action float32 [action_horizon, action_dim]."""
        c = self._config
        if layout not in ("nhwc", "nchw"):
            raise ValueError(f"apxinf_py: unsupported image layout `{layout}` (expected `nhwc` or `nchw`)")
        if not isinstance(rgb_u8, np.ndarray) or rgb_u8.dtype != np.uint8 or \
                not rgb_u8.flags.c_contiguous:
            raise ValueError("apxinf_py.infer_rgb: rgb_u8 must be C-contiguous uint8")
        expected_bytes = c.num_views * c.image_size * c.image_size * 3
        if rgb_u8.size != expected_bytes:
            raise ValueError(f"apxinf_py.infer_rgb: rgb_u8 expected {expected_bytes} bytes "
                             f"({c.num_views} views x {c.image_size}x{c.image_size}x3), got {rgb_u8.size}")
        tokens = self._validate_tokens(token_ids)
        noise = self._validate_noise(noise)
        return self._frontend.infer(layout, rgb_u8, tokens, noise)

    # ---- shape properties ---------------------------------------------------------------
    @property
    def device(self) -> str:
        return f"cuda:{self._device}"

    @property
    def action_dim(self) -> int:
        return self._config.action_dim

    @property
    def action_horizon(self) -> int:
        return self._config.action_horizon

    @property
    def num_views(self) -> int:
        return self._config.num_views

    @property
    def image_size(self) -> int:
        return self._config.image_size

    @property
    def patch_size(self) -> int:
        return self._config.patch_size

    @property
    def patches_per_view(self) -> int:
        return self._config.patches_per_view

    @property
    def max_token_len(self) -> int:
        return self._config.max_token_len

    def __repr__(self) -> str:
        c = self._config
        return (f"Model(device={self.device}, action=[{c.action_horizon}, {c.action_dim}], "
                f"views={c.num_views}, image={c.image_size}, patch={c.patch_size})")

    def close(self) -> None:
        self._frontend.close()
        self._rt.close()
