"""The serving shell around the engine: observation dict -> action chunk, and its websocket
transport. Host-side mirror of the reference's pure-Python layer, same contracts:

  processors        python/apxinf/apxinf/processors/{resize,tokenize,normalize,noise,transforms}.py
                    (image parse + letterbox resize, prompt clean-up / state discretisation /
                    SentencePiece ids, quantile and mean-std (un)normalisation of
                    norm_stats.json, seeded prior noise)
  Pi05Policy        python/apxinf/apxinf/policies/impls/pi05.py:79-476 (pre steps -> bare model
                    `infer_rgb` -> post steps; result keys actions / normalized_actions /
                    token_ids / noise / timing / metadata; `from_random`, `from_pretrained`)
  wire protocol     python/apxinf/apxinf/serving/{websocket,msgpack_numpy}.py (the OpenPI client
                    protocol: metadata frame on connect, one MessagePack frame per observation with
                    NumPy arrays as tagged maps, `actions` + `policy_timing` + `server_timing`
                    back, `/healthz`, traceback text + close 1011 on failure)

Everything here is host glue around `apxinf_py.Model` (this package's, or any object with
`infer_rgb`, `action_horizon`, `action_dim`, `num_views`, `image_size`): no arithmetic of the
model runs in this module.
"""
from __future__ import annotations

import json
import os
import time
import traceback
import warnings
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np

# ---------------------------------------------------------------------------------------------
# MessagePack <-> NumPy (the OpenPI client's tagged maps)
# ---------------------------------------------------------------------------------------------


def encode_numpy(value: Any) -> Any:
    """`default=` hook of msgpack: arrays and NumPy scalars as tagged maps, the rest untouched."""
    if isinstance(value, (np.ndarray, np.generic)) and value.dtype.kind in ("V", "O", "c"):
        raise ValueError(f"unsupported NumPy dtype {value.dtype}")
    if isinstance(value, np.ndarray):
        return {b"__ndarray__": True, b"data": value.tobytes(), b"dtype": value.dtype.str,
                b"shape": value.shape}
    if isinstance(value, np.generic):
        return {b"__npgeneric__": True, b"data": value.item(), b"dtype": value.dtype.str}
    return value


def decode_numpy(value: dict) -> Any:
    """`object_hook=` of msgpack: the inverse of encode_numpy."""
    if b"__ndarray__" in value:
        return np.ndarray(buffer=value[b"data"], dtype=np.dtype(value[b"dtype"]), shape=value[b"shape"])
    if b"__npgeneric__" in value:
        return np.dtype(value[b"dtype"]).type(value[b"data"])
    return value


def pack(message: Any) -> bytes:
    import msgpack
    return msgpack.packb(message, default=encode_numpy)


def unpack(payload: bytes) -> Any:
    import msgpack
    return msgpack.unpackb(payload, object_hook=decode_numpy)


# ---------------------------------------------------------------------------------------------
# processors
# ---------------------------------------------------------------------------------------------


def parse_image(value: Any, name: str = "image") -> np.ndarray:
    """Any rank-3 RGB image (HWC or CHW; uint8, or float in [0, 1] scaled by 255) -> uint8 HWC."""
    image = np.asarray(value)
    if image.ndim != 3:
        raise ValueError(f"{name} must have rank 3, got shape {image.shape}")
    if np.issubdtype(image.dtype, np.floating):
        image = (255 * image).astype(np.uint8)
    if image.shape[0] == 3:
        image = image.transpose(1, 2, 0)
    if image.shape[-1] != 3:
        raise ValueError(f"{name} must have three RGB channels, got shape {image.shape}")
    if image.dtype != np.uint8:
        raise ValueError(f"{name} must be uint8 or floating point, got {image.dtype}")
    return np.ascontiguousarray(image)


def resize_with_pad(image: np.ndarray, size: int = 224) -> np.ndarray:
    """Aspect-preserving bilinear resize onto a black size x size canvas, centred; an image that
    is already size x size is returned as it is."""
    from PIL import Image
    image = np.asarray(image)
    if image.shape[:2] == (size, size):
        return image
    height, width = image.shape[:2]
    ratio = max(width / size, height / size)
    new_height, new_width = int(height / ratio), int(width / ratio)
    resized = Image.fromarray(image).resize((new_width, new_height), resample=Image.Resampling.BILINEAR)
    canvas = Image.new(resized.mode, (size, size), 0)
    canvas.paste(resized, (max(0, int((size - new_width) / 2)), max(0, int((size - new_height) / 2))))
    return np.asarray(canvas)


def discretize_state(state: Sequence[float]) -> np.ndarray:
    """A state in [-1, 1] to bins 0..255: clamp(floor((v + 1) * 128), 0, 255)."""
    values = np.asarray(state, dtype=np.float64)
    return np.clip(np.floor((values + 1.0) * 128.0), 0, 255).astype(np.uint8)


def build_prompt(prompt: str, state: Optional[Sequence[float]] = None, discrete_state: bool = False) -> str:
    """The text given to the tokenizer: the cleaned task, or with state injection
    "Task: {task}, State: {bins};\\nAction: "."""
    task = prompt.strip().replace("_", " ").replace("\n", " ")
    if not discrete_state:
        return task
    if state is None:
        raise ValueError("PromptTokenizer: discrete_state=True requires a state array")
    bins = " ".join(str(int(v)) for v in discretize_state(state))
    return f"Task: {task}, State: {bins};\nAction: "


class PromptTokenizer:
    """Prompt (and optionally state) -> uint32 ids through a SentencePiece model: BOS + text,
    plus the newline token when no state is injected; 1..=max_token_len tokens."""

    def __init__(self, model_path: str, max_token_len: int = 200, discrete_state: bool = False):
        import sentencepiece
        self.max_token_len = int(max_token_len)
        self.discrete_state = bool(discrete_state)
        self._sp = sentencepiece.SentencePieceProcessor(model_file=str(model_path))

    def __call__(self, prompt: str, state: Optional[Sequence[float]] = None) -> np.ndarray:
        if not isinstance(prompt, str):
            raise TypeError(f"PromptTokenizer: prompt must be a string, got {type(prompt)!r}")
        tokens = list(self._sp.encode(build_prompt(prompt, state, self.discrete_state), add_bos=True))
        if not self.discrete_state:
            tokens += list(self._sp.encode("\n"))
        if not 0 < len(tokens) <= self.max_token_len:
            raise ValueError(f"PromptTokenizer: token count must be in 1..={self.max_token_len}, got {len(tokens)}")
        return np.asarray(tokens, dtype=np.uint32)


class SyntheticTokenizer:
    """A fixed-length id ramp for any prompt: the language prefix runs the intended length with
    no tokenizer file on disk (latency measurements with random weights)."""

    discrete_state = False

    def __init__(self, token_count: int, max_token_len: int = 200):
        self.token_count, self.max_token_len = int(token_count), int(max_token_len)
        if not 0 < self.token_count <= self.max_token_len:
            raise ValueError(f"SyntheticTokenizer: token_count must be in 1..={self.max_token_len}, "
                             f"got {self.token_count}")

    def __call__(self, prompt: str, state: Optional[Sequence[float]] = None) -> np.ndarray:
        return (np.arange(self.token_count, dtype=np.uint32) % np.uint32(256)) + np.uint32(1)


class GaussianNoise:
    """Seeded standard-normal [horizon, dim] prior of the flow."""

    def __init__(self, action_horizon: int, action_dim: int, seed: int = 0, dtype=np.float32):
        self.shape = (int(action_horizon), int(action_dim))
        self.seed, self.dtype = int(seed), np.dtype(dtype)
        self._rng = np.random.default_rng(self.seed)

    def __call__(self) -> np.ndarray:
        sample = self._rng.standard_normal(self.shape, dtype=np.float32)
        return sample if self.dtype == np.float32 else sample.astype(self.dtype)

    def reset(self, seed: Optional[int] = None) -> None:
        if seed is not None:
            self.seed = int(seed)
        self._rng = np.random.default_rng(self.seed)


def load_norm_stats(model_dir: str, key: str = "actions") -> dict:
    """The statistics of one key of norm_stats.json (nested under "norm_stats", or flat)."""
    with open(os.path.join(model_dir, "norm_stats.json"), "r", encoding="utf-8") as handle:
        document = json.load(handle)
    stats = document.get("norm_stats", document)
    if key not in stats:
        raise KeyError(f"norm_stats.json has no entry {key!r}; keys: {sorted(stats)}")
    return stats[key]


class _Affine:
    """Quantile ([q01, q99] <-> [-1, 1]) or mean / std statistics over the last axis."""

    def __init__(self, q01=None, q99=None, mean=None, std=None, mode="quantile", dims=None, eps=1e-6):
        if mode not in ("quantile", "mean_std"):
            raise ValueError(f"mode must be 'quantile' or 'mean_std', got {mode!r}")
        first, second = (q01, q99) if mode == "quantile" else (mean, std)
        names = ("q01", "q99") if mode == "quantile" else ("mean", "std")
        if first is None or second is None:
            raise ValueError(f"{mode} mode requires {names[0]} and {names[1]}")
        self.mode, self.eps = mode, float(eps)
        self.lo, self.hi = (self._vector(v, n, dims) for v, n in zip((first, second), names))
        if self.lo.shape != self.hi.shape:
            raise ValueError(f"{names[0]} {self.lo.shape} and {names[1]} {self.hi.shape} must match")

    @staticmethod
    def _vector(values, name, dims) -> np.ndarray:
        vector = np.asarray(values, dtype=np.float32)
        if vector.ndim != 1:
            raise ValueError(f"{name} must be rank 1, got shape {vector.shape}")
        if dims is not None:
            if vector.size < dims:
                raise ValueError(f"{name} has {vector.size} entries, need at least {dims}")
            vector = vector[:int(dims)]
        return np.ascontiguousarray(vector)

    @property
    def width(self) -> int:
        return self.lo.size

    def _checked(self, array, who) -> np.ndarray:
        array = np.asarray(array, dtype=np.float32)
        if array.shape[-1] != self.width:
            raise ValueError(f"{who}: last dim must be {self.width}, got array shape {array.shape}")
        return array

    @staticmethod
    def _finite(array, who) -> np.ndarray:
        if not np.isfinite(array).all():
            raise FloatingPointError(f"{who} produced non-finite values")
        return array.astype(np.float32, copy=False)

    def unnormalize(self, array) -> np.ndarray:
        array = self._checked(array, "Unnormalizer")
        if self.mode == "quantile":
            out = (array + np.float32(1.0)) * ((self.hi - self.lo + np.float32(self.eps)) / np.float32(2.0)) + self.lo
        else:
            out = array * self.hi + self.lo
        return self._finite(out, "Unnormalizer")

    def normalize(self, array) -> np.ndarray:
        array = self._checked(array, "Normalizer")
        if self.mode == "quantile":
            out = np.float32(2.0) * (array - self.lo) / (self.hi - self.lo + np.float32(self.eps)) - np.float32(1.0)
        else:
            out = (array - self.lo) / self.hi
        return self._finite(out, "Normalizer")


class Unnormalizer:
    """Normalized-domain array -> physical units."""

    def __init__(self, **stats):
        self._stats = _Affine(**stats)

    @classmethod
    def from_norm_stats(cls, model_dir, key="actions", mode="quantile", dims=None, eps=1e-6):
        s = load_norm_stats(model_dir, key)
        if mode == "quantile":
            return cls(q01=s["q01"], q99=s["q99"], mode=mode, dims=dims, eps=eps)
        return cls(mean=s["mean"], std=s["std"], mode=mode, dims=dims, eps=eps)

    @property
    def width(self) -> int:
        return self._stats.width

    def __call__(self, array) -> np.ndarray:
        return self._stats.unnormalize(array)


class Normalizer(Unnormalizer):
    """Physical units -> normalized domain (the inverse map over the same statistics)."""

    def __call__(self, array) -> np.ndarray:
        return self._stats.normalize(array)


class Pipeline:
    """Named steps applied in order to one flowing value; steps can be looked up, replaced and
    inserted by name (a custom resize or tokenizer drops in without touching the policy)."""

    def __init__(self, steps: Sequence[Tuple[str, Callable]]):
        self._steps: List[Tuple[str, Callable]] = list(steps)
        if len({name for name, _ in self._steps}) != len(self._steps):
            raise ValueError("Pipeline: step names must be unique")

    @property
    def names(self) -> List[str]:
        return [name for name, _ in self._steps]

    def __getitem__(self, name: str) -> Callable:
        for step_name, step in self._steps:
            if step_name == name:
                return step
        raise KeyError(name)

    def replace(self, name: str, step: Callable) -> "Pipeline":
        self[name]
        self._steps = [(n, step if n == name else s) for n, s in self._steps]
        return self

    def insert_after(self, name: str, new_name: str, step: Callable) -> "Pipeline":
        index = self.names.index(name) if name in self.names else None
        if index is None:
            raise KeyError(name)
        if new_name in self.names:
            raise ValueError(f"Pipeline: step {new_name!r} exists")
        self._steps.insert(index + 1, (new_name, step))
        return self

    def __call__(self, value):
        for _, step in self._steps:
            value = step(value)
        return value


# data-dict keys of the pre / post chains
OBSERVATION, PROMPT, RGB, TOKEN_IDS, NOISE = "observation", "prompt", "rgb", "token_ids", "noise"
NORMALIZED, TRIMMED, ACTIONS = "normalized_actions", "trimmed", "actions"


class Pi05Policy:
    """Raw observation dict + prompt -> unnormalized action chunk: pre chain (stack the cameras,
    tokenize, sample the prior) -> bare model -> post chain (trim, unnormalize)."""

    DEFAULT_IMAGE_KEYS = ("observation/image", "observation/wrist_image")

    def __init__(self, model, *, tokenizer, unnormalizer: Unnormalizer, noise: Optional[GaussianNoise] = None,
                 state_normalizer: Optional[Normalizer] = None, image_pipeline: Optional[Pipeline] = None,
                 image_keys: Sequence[str] = DEFAULT_IMAGE_KEYS, prompt_key: str = "prompt",
                 state_key: str = "observation/state", metadata: Optional[Mapping[str, Any]] = None):
        self.model = model
        self.image_keys, self.prompt_key, self.state_key = tuple(image_keys), prompt_key, state_key
        if len(self.image_keys) != model.num_views:
            raise ValueError(f"Pi05Policy: model expects {model.num_views} camera views but "
                             f"{len(self.image_keys)} image_keys were given: {self.image_keys}. Supply exactly "
                             "the checkpoint's cameras (real views only, no padding).")
        size = model.image_size
        self.image_pipeline = image_pipeline or Pipeline([("parse", parse_image),
                                                          ("resize", lambda image: resize_with_pad(image, size))])
        self.tokenizer, self.state_normalizer = tokenizer, state_normalizer
        self.noise = noise or GaussianNoise(model.action_horizon, model.action_dim)
        self.unnormalizer = unnormalizer
        self.discrete_state = bool(getattr(tokenizer, "discrete_state", False))
        self.input_pipeline = Pipeline([("image_stack", self._stack_images), ("tokenize", self._tokenize),
                                        ("sample_noise", self._sample_noise)])
        self.output_pipeline = Pipeline([("trim", self._trim), ("unnormalize", self._unnormalize)])
        self.metadata = {
            "model_type": "pi05", "action_horizon": model.action_horizon, "action_dim": unnormalizer.width,
            "model_action_dim": model.action_dim, "num_views": model.num_views,
            "image_size": [model.image_size, model.image_size], "image_keys": list(self.image_keys),
            "discrete_state": self.discrete_state, "state_normalized": state_normalizer is not None,
            "input_pipeline": self.input_pipeline.names, "output_pipeline": self.output_pipeline.names,
            **(dict(metadata) if metadata else {}),
        }

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def from_random(cls, model, *, token_count: Optional[int] = None, action_dim: Optional[int] = None,
                    seed: int = 0, image_keys: Optional[Sequence[str]] = None, warn: bool = True,
                    metadata: Optional[Mapping[str, Any]] = None) -> "Pi05Policy":
        """A random-weight model in synthetic processors (fixed-length id ramp, identity
        unnormaliser): end-to-end latency with no file on disk; the actions mean nothing."""
        if warn:
            warnings.warn("Pi05Policy.from_random: synthetic tokenizer + identity unnormalizer; "
                          "actions are latency-only and numerically meaningless.", stacklevel=2)
        max_len = int(getattr(model, "max_token_len", 200))
        tokenizer = SyntheticTokenizer(min(10, max_len) if token_count is None else token_count, max_len)
        width = int(model.action_dim if action_dim is None else action_dim)
        unnormalizer = Unnormalizer(q01=[-1.0] * width, q99=[1.0] * width, dims=width, eps=0.0)
        if image_keys is None:
            image_keys = cls.DEFAULT_IMAGE_KEYS if model.num_views == 2 else \
                tuple(f"observation/image_{i}" for i in range(model.num_views))
        return cls(model, tokenizer=tokenizer, unnormalizer=unnormalizer,
                   noise=GaussianNoise(model.action_horizon, model.action_dim, seed=seed), image_keys=image_keys,
                   metadata={"weights": "synthetic", **(dict(metadata) if metadata else {})})

    @classmethod
    def from_pretrained(cls, model_dir: str, *, model=None, checkpoint: Optional[str] = None,
                        device: str = "cuda:0", precision: str = "auto", calibration: Optional[str] = None,
                        tactics: Optional[str] = None, tokenizer_path: Optional[str] = None,
                        norm_key: str = "actions", action_dim: Optional[int] = None,
                        action_horizon: Optional[int] = None, seed: int = 0, discrete_state: bool = False,
                        state_norm_key: str = "state", image_keys: Sequence[str] = DEFAULT_IMAGE_KEYS,
                        metadata: Optional[Mapping[str, Any]] = None) -> "Pi05Policy":
        """From a checkpoint directory: model.safetensors (+ config / calibration / tactics json),
        the SentencePiece model and norm_stats.json."""
        model_dir = os.fspath(model_dir)
        if model is None:
            from . import apxinf_py
            model = apxinf_py.Model.load("pi05", checkpoint or os.path.join(model_dir, "model.safetensors"),
                                         device=device, precision=precision, calibration=calibration,
                                         tactics=tactics, action_horizon=action_horizon)
        elif action_horizon is not None and int(action_horizon) != int(model.action_horizon):
            raise ValueError(f"Pi05Policy.from_pretrained: action_horizon={action_horizon} conflicts with the "
                             f"supplied model's horizon {model.action_horizon}; pass the override to the model "
                             "constructor instead")
        if tokenizer_path is None:
            candidates = [os.path.join(model_dir, name) for name in
                          ("tokenizer.model", "paligemma_tokenizer.model", os.path.join("tokenizer", "tokenizer.model"))]
            found = [c for c in candidates if os.path.isfile(c)]
            if not found:
                raise FileNotFoundError(f"no SentencePiece model under {model_dir} (tried {candidates}); "
                                        "pass tokenizer_path")
            tokenizer_path = found[0]
        tokenizer = PromptTokenizer(tokenizer_path, max_token_len=getattr(model, "max_token_len", 200),
                                    discrete_state=discrete_state)
        return cls(model, tokenizer=tokenizer,
                   unnormalizer=Unnormalizer.from_norm_stats(model_dir, key=norm_key, dims=action_dim),
                   state_normalizer=Normalizer.from_norm_stats(model_dir, key=state_norm_key) if discrete_state else None,
                   noise=GaussianNoise(model.action_horizon, model.action_dim, seed=seed), image_keys=image_keys,
                   metadata=metadata)

    # ---- steps (dict -> dict) -------------------------------------------------------------
    def _stack_images(self, data: dict) -> dict:
        observation = data[OBSERVATION]
        views = [np.asarray(self.image_pipeline(observation[key])) for key in self.image_keys]
        size = self.model.image_size
        for key, view in zip(self.image_keys, views):
            if view.shape != (size, size, 3) or view.dtype != np.uint8:
                raise ValueError(f"image_stack: {key} came out as {view.dtype} {view.shape}, "
                                 f"expected uint8 ({size}, {size}, 3)")
        data[RGB] = np.ascontiguousarray(np.stack(views))
        return data

    def _tokenize(self, data: dict) -> dict:
        state = None
        if self.discrete_state:
            state = np.asarray(data[OBSERVATION][self.state_key], dtype=np.float32)
            if self.state_normalizer is not None:  # raw state -> [-1, 1] first, then bins
                state = self.state_normalizer(state)
        data[TOKEN_IDS] = np.ascontiguousarray(self.tokenizer(data[PROMPT], state), dtype=np.uint32)
        return data

    def _sample_noise(self, data: dict) -> dict:
        data[NOISE] = np.ascontiguousarray(self.noise(), dtype=np.float32)
        return data

    def _trim(self, data: dict) -> dict:
        data[TRIMMED] = data[NORMALIZED][..., :self.unnormalizer.width]
        return data

    def _unnormalize(self, data: dict) -> dict:
        data[ACTIONS] = self.unnormalizer(data[TRIMMED])
        return data

    # ---- inference ------------------------------------------------------------------------
    def infer(self, observation: Mapping[str, Any]) -> dict:
        started = time.perf_counter()
        if not isinstance(observation, Mapping):
            raise TypeError(f"observation must be a mapping, got {type(observation)!r}")
        required = list(self.image_keys) + [self.prompt_key] + ([self.state_key] if self.discrete_state else [])
        missing = [key for key in required if key not in observation]
        if missing:
            raise KeyError(f"Pi05Policy.infer: missing observation keys: {missing}")
        prompt = observation[self.prompt_key]
        if not isinstance(prompt, str):
            raise TypeError(f"{self.prompt_key} must be a string, got {type(prompt)!r}")
        data = self.input_pipeline({OBSERVATION: observation, PROMPT: prompt})
        model_started = time.perf_counter()
        normalized = np.asarray(self.model.infer_rgb(data[RGB], "nhwc", data[TOKEN_IDS], data[NOISE]), dtype=np.float32)
        model_ms = (time.perf_counter() - model_started) * 1000.0
        expected = (self.model.action_horizon, self.model.action_dim)
        if normalized.shape != expected:
            raise ValueError(f"model returned action shape {normalized.shape}, expected {expected}")
        if not np.isfinite(normalized).all():
            raise FloatingPointError("model returned non-finite normalized actions")
        out = self.output_pipeline({NORMALIZED: normalized, OBSERVATION: data[OBSERVATION]})
        return {"actions": out[ACTIONS], "normalized_actions": normalized, "token_ids": data[TOKEN_IDS],
                "noise": data[NOISE],
                "timing": {"model_ms": model_ms, "total_ms": (time.perf_counter() - started) * 1000.0},
                "metadata": self.metadata}

    __call__ = infer

    @property
    def action_dim(self) -> int:
        return self.unnormalizer.width

    @property
    def action_horizon(self) -> int:
        return self.model.action_horizon

    def close(self) -> None:
        close = getattr(self.model, "close", None)
        if callable(close):
            close()


# ---------------------------------------------------------------------------------------------
# websocket transport
# ---------------------------------------------------------------------------------------------


def wire_response(result: dict) -> dict:
    """What goes on the wire of a policy result: `actions` and `policy_timing` only."""
    timing = result.get("timing", {}) or {}
    policy_timing = {"infer_ms": float(timing.get("model_ms", 0.0))}
    if "total_ms" in timing:
        policy_timing["policy_ms"] = float(timing["total_ms"])
    return {"actions": np.ascontiguousarray(result["actions"], dtype=np.float32), "policy_timing": policy_timing}


class WebsocketPolicyServer:
    """Serves any object with `infer(observation dict) -> result dict` to unmodified OpenPI
    websocket clients. The policy is called on the event-loop thread: the model handle belongs to
    the thread that created it, and a GPU serves one inference at a time anyway."""

    def __init__(self, policy, host: str = "0.0.0.0", port: int = 8000, *, metadata: Optional[dict] = None):
        self._policy, self._host, self._port = policy, host, port
        self._metadata = dict(metadata) if metadata is not None else dict(getattr(policy, "metadata", {}))
        self.bound_port: Optional[int] = None

    async def _handle(self, websocket) -> None:
        import websockets
        await websocket.send(pack(self._metadata))
        previous_total = None
        while True:
            try:
                request_started = time.monotonic()
                payload = await websocket.recv()
                if isinstance(payload, str):
                    raise TypeError("inference requests must be binary MessagePack frames")
                observation = unpack(payload)
                infer_started = time.monotonic()
                result = self._policy.infer(observation)
                response = wire_response(result)
                response["server_timing"] = {"infer_ms": (time.monotonic() - infer_started) * 1000}
                if previous_total is not None:
                    response["server_timing"]["prev_total_ms"] = previous_total * 1000
                await websocket.send(pack(response))
                previous_total = time.monotonic() - request_started
            except websockets.ConnectionClosed:
                break
            except Exception:
                await websocket.send(traceback.format_exc())
                await websocket.close(code=1011, reason="Internal server error. Traceback included in previous frame.")
                break

    @staticmethod
    def _health_check(connection, request):
        import http
        if request.path == "/healthz":
            return connection.respond(http.HTTPStatus.OK, "OK\n")
        return None

    async def run(self, started=None) -> None:
        """Serves until cancelled; `started`, if given, is an asyncio.Event set once listening."""
        import websockets.asyncio.server as server_module
        async with server_module.serve(self._handle, self._host, self._port, compression=None, max_size=None,
                                       process_request=self._health_check) as server:
            self.bound_port = server.sockets[0].getsockname()[1]
            if started is not None:
                started.set()
            await server.serve_forever()

    def serve_forever(self) -> None:
        import asyncio
        asyncio.run(self.run())
