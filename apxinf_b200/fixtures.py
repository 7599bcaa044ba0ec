"""Seeded synthetic observations with the benchmark's shapes and value distributions
(stand-ins for real camera frames and prompts: uniform u8 images in NHWC, uniform token
ids, N(0,1) action noise rounded to bf16), plus the reference bench's arithmetic image
pattern (crates/apxinf-model/examples/pi05_bench.rs:424-426)."""
from __future__ import annotations

import numpy as np

from .engine import Pi05Config, float_to_bf16_bits


def synthetic_observation(cfg: Pi05Config, seed: int, token_count: int):
    """(images u8 [views, S, S, 3], token ids u32 [T], noise f32 [H, action_dim] on the bf16 grid)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    images = rng.integers(0, 256, size=(cfg.num_views, cfg.image_size, cfg.image_size, 3),
                          dtype=np.uint8)
    tokens = rng.integers(0, cfg.vocab_size, size=(token_count,), dtype=np.uint32)
    noise = rng.standard_normal((cfg.action_horizon, cfg.action_dim)).astype(np.float32)
    bits = float_to_bf16_bits(noise).astype(np.uint32) << np.uint32(16)
    return images, tokens, bits.view(np.float32)


def synthetic_batch(cfg: Pi05Config, batch: int, token_count: int, base_seed: int):
    obs = [synthetic_observation(cfg, base_seed + i, token_count) for i in range(batch)]
    return (np.stack([o[0] for o in obs]), np.stack([o[1] for o in obs]),
            np.stack([o[2] for o in obs]))


def reference_image_pattern(cfg: Pi05Config) -> np.ndarray:
    n = cfg.num_views * cfg.image_size * cfg.image_size * 3
    idx = np.arange(n, dtype=np.int64)
    return ((idx * 73 + idx // 11 + 19) & 0xFF).astype(np.uint8).reshape(
        cfg.num_views, cfg.image_size, cfg.image_size, 3)
