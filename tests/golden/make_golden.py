"""Generates tests/golden/pi05_full_*.npz: action chunks (and a few intermediate rows) of the
CPU oracle at the full PI0.5 architecture, for the benchmark configurations:

  cfg2  BF16, 2 views, 10 prompt tokens, H=10, 10 flow steps
  cfg3  FP8 (per-channel E4M3 weights, uniform activation scale 0.05), same shapes
  cfg4  INT8 W8A8, 3 views, 21 prompt tokens, H=50, 10 flow steps
  cfg5  FP8, 2 views, 10 prompt tokens, H=50: three observations with the seeds of the
        throughput benchmark's first three samples (1000, 1001, 1002), for the batched path
  cfg2n cfg2 with seeded N(0, 0.02) weights (the benchmark's wording) instead of the
        reference's uniform generator
  cfg4s cfg4 as the benchmark words it: N(0, 0.02) weights and a STATIC per-tensor INT8
        activation scale per GEMM input. The scales are calibrated here: a first pass with the
        reference's dynamic per-row quantiser records every site's absmax, scale = absmax / 127;
        the table travels in the fixture (sites / scales arrays)

Weights: Pi05Weights::synthetic(seed 0); observation: oracle.synthetic_observation(seed 1234)
(uniform u8 images, uniform token ids, N(0,1) noise rounded to bf16). The GPU parity tests
(tests/test_engine_full_gpu.py) regenerate the same inputs from the seeds and compare.

Run from the repository root:  python tests/golden/make_golden.py [cfg2 cfg3 cfg4]
Takes several minutes per configuration on 8 cores (2.6 G synthetic weights + 2.5-4 TFLOP).
"""
import sys
import time
from dataclasses import replace
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import pi05_oracle as O  # noqa: E402

CASES = {
    "cfg2": dict(dtype="bf16", views=2, tokens=10, horizon=10),
    "cfg3": dict(dtype="fp8", views=2, tokens=10, horizon=10),
    "cfg4": dict(dtype="int8", views=3, tokens=21, horizon=50),
    "cfg5": dict(dtype="fp8", views=2, tokens=10, horizon=50, observation_seeds=(1000, 1001, 1002)),
    "cfg2n": dict(dtype="bf16", views=2, tokens=10, horizon=10, weights="normal"),
    "cfg4s": dict(dtype="int8", views=3, tokens=21, horizon=50, weights="normal", int8_act="static"),
}
WEIGHT_SEED = 0
OBSERVATION_SEED = 1234


def run_batch(name: str) -> None:
    """Several observations through one oracle (weights generated once and kept)."""
    case = CASES[name]
    cfg = replace(O.Pi05Config(), num_views=case["views"], action_horizon=case["horizon"])
    weights = O.SyntheticWeights(cfg, WEIGHT_SEED)
    weights.cache_prefixes = ("",)
    oracle = O.Pi05Oracle(cfg, weights, O.OracleOptions(dtype=case["dtype"], act_scale=0.05,
                                                        vision_round_scores=True, collect=True))
    oracle._prepare_all = True
    last = cfg.language.depth - 2
    actions, hidden, step0 = [], [], []
    start = time.time()
    for seed in case["observation_seeds"]:
        images, tokens, noise = O.synthetic_observation(cfg, seed, case["tokens"])
        actions.append(oracle.infer(images, tokens, noise).astype(np.float32))
        hidden.append(oracle.trace[f"language.{last}.hidden"][[0, 100, -1]].astype(np.float32))
        step0.append(oracle.trace["action.step0"].astype(np.float32))
        print(f"{name} seed {seed}: {time.time() - start:.1f} s", flush=True)
    np.savez_compressed(
        Path(__file__).parent / f"pi05_full_{name}.npz",
        actions=np.stack(actions), hidden_rows=np.stack(hidden), step0=np.stack(step0),
        observation_seeds=np.array(case["observation_seeds"], dtype=np.int64),
        meta=np.array([WEIGHT_SEED, -1, case["views"], case["tokens"], case["horizon"]],
                      dtype=np.int64))


def run(name: str) -> None:
    case = CASES[name]
    if "observation_seeds" in case:
        return run_batch(name)
    cfg = replace(O.Pi05Config(), num_views=case["views"], action_horizon=case["horizon"])
    images, tokens, noise = O.synthetic_observation(cfg, OBSERVATION_SEED, case["tokens"])
    weights = O.SyntheticWeights(cfg, WEIGHT_SEED, case.get("weights", "lcg"))
    extra = {}
    options = O.OracleOptions(dtype=case["dtype"], act_scale=0.05, vision_round_scores=True,
                              collect=True)
    if case.get("int8_act") == "static":
        weights.cache_prefixes = ("",)  # two passes over the same weights
        calib = O.Pi05Oracle(cfg, weights, O.OracleOptions(dtype=case["dtype"], calibrate=True,
                                                           vision_round_scores=True))
        calib._prepare_all = True
        calib.infer(images, tokens, noise)
        table = {site: max(amax, 1e-6) / 127.0 for site, amax in calib.amax.items()}
        options.int8_act = "static"
        options.act_scales = table
        extra = dict(sites=np.array(sorted(table)), scales=np.array([table[k] for k in sorted(table)],
                                                                    dtype=np.float32))
        print(f"{name}: calibrated {len(table)} sites", flush=True)
    oracle = O.Pi05Oracle(cfg, weights, options)
    if case.get("int8_act") == "static":
        oracle._prepared = calib._prepared
        oracle._prepare_all = True
    start = time.time()
    actions = oracle.infer(images, tokens, noise)
    elapsed = time.time() - start
    last = cfg.language.depth - 2
    np.savez_compressed(
        Path(__file__).parent / f"pi05_full_{name}.npz",
        actions=actions.astype(np.float32),
        hidden_rows=oracle.trace[f"language.{last}.hidden"][[0, 100, -1]].astype(np.float32),
        kv0_k_rows=oracle.trace["kv.0.k"][[0, 100, -1], 0].astype(np.float32),
        kv_last_v_rows=oracle.trace[f"kv.{cfg.language.depth - 1}.v"][[0, 100, -1], 0].astype(np.float32),
        step0=oracle.trace["action.step0"].astype(np.float32),
        meta=np.array([WEIGHT_SEED, OBSERVATION_SEED, case["views"], case["tokens"],
                       case["horizon"]], dtype=np.int64), **extra)
    print(f"{name}: {elapsed:.1f} s, |a|max {np.abs(actions).max():.4f}", flush=True)


if __name__ == "__main__":
    for arg in (sys.argv[1:] or list(CASES)):
        run(arg)
