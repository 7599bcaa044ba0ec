"""Whole-model second oracle: the reference's own CUDA kernels and cuBLAS calls, replayed in
the order of its executors (oracle/ref_forward.py over oracle/_ref), against the NumPy oracle
and against this library. Per-op parity is pinned in test_ref_ops_gpu.py; what this file pins
is the ORDER of the ops and the rounding points between them, which the NumPy oracle restates
from the reference's Rust sources."""
from pathlib import Path

import numpy as np
import pytest

from oracle import pi05_oracle as O
from oracle import ref_forward as R

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not R.available(), reason="oracle/_ref was not built")]
GOLDEN = Path(__file__).parent / "golden"


def _bf16(bits):
    return O.bf16_from_bits(np.asarray(bits, dtype=np.uint16))


def test_gpu_weight_stream_equals_the_oracle():
    got = R.lcg_values_gpu(7, 12345, 3 * (1 << 20) + 17).float().cpu().numpy()
    want = O.lcg_values(7, 12345, 3 * (1 << 20) + 17)
    assert np.array_equal(got, want)


def test_tiny_forward_reference_kernels_oracle_and_library_agree():
    from apxinf_b200.engine import Pi05Runtime
    cfg = O.tiny_config()
    token_count = 6
    images, tokens, noise = O.synthetic_observation(cfg, 41, token_count)
    ref = R.RefBf16Forward(cfg, 3)
    got_ref = ref.infer(images, tokens, noise)
    # the reference's SigLIP fallback kernel keeps its scores in fp32; its cuBLAS MQA rounds
    # logits and probabilities to bf16 (cublas_adapter.cu:109-130)
    oracle = O.Pi05Oracle(cfg, O.SyntheticWeights(cfg, 3),
                          O.OracleOptions(dtype="bf16", vision_round_scores=False, mqa_round_scores=True,
                                          collect=True))
    want = oracle.infer(images, tokens, noise)
    m = O.compare(got_ref, want)
    assert m["cosine"] >= 0.9999 and m["max_abs"] <= 2e-2, m
    # intermediates of the reference replay against the oracle's: residual stream after the
    # prefill, first and last layers' cached K/V
    ptok = cfg.vision_tokens + token_count
    hidden = ref.last_hidden.float().cpu().numpy()
    mh = O.compare(hidden, oracle.trace[f"language.{cfg.language.depth - 2}.hidden"])
    assert mh["cosine"] >= 0.9999, mh
    for layer in (0, cfg.language.depth - 1):
        k = ref.keys[layer].float().cpu().numpy()[:ptok]
        mk = O.compare(k, oracle.trace[f"kv.{layer}.k"][:, 0])
        assert mk["cosine"] >= 0.9999, (layer, mk)
    rt = Pi05Runtime.random(cfg, dtype="bf16", seed=3, device=0)
    g = rt.capture_infer_rgb_u8(token_count, "nhwc", 1)
    ours = g.infer_host(images[None], tokens[None], noise[None])[0]
    mo = O.compare(ours, got_ref)
    assert mo["cosine"] >= 0.999 and mo["max_abs"] <= 2e-2, mo
    g.close()
    rt.close()
    ref.close()


def test_full_size_forward_reference_kernels_against_fixture_and_library():
    """cfg2 (BF16, two views, 10 tokens, H=10) at the full architecture: the reference-kernel
    replay against the committed oracle fixture and against this library, with the benchmark's
    BF16 tolerances (cosine >= 0.999, max-abs <= 2e-2)."""
    from apxinf_b200.engine import Pi05Config, Pi05Runtime
    from apxinf_b200.fixtures import synthetic_observation
    gold = np.load(GOLDEN / "pi05_full_cfg2.npz")
    weight_seed, obs_seed, views, tokens_n, horizon = [int(v) for v in gold["meta"]]
    ocfg = O.Pi05Config()
    assert (views, horizon) == (ocfg.num_views, ocfg.action_horizon)
    images, tokens, noise = O.synthetic_observation(ocfg, obs_seed, tokens_n)
    ref = R.RefBf16Forward(ocfg, weight_seed)
    got_ref, times = ref.infer(images, tokens, noise, timed=True)
    assert np.isfinite(got_ref).all() and times["launches"] > 2000
    m = O.compare(got_ref, gold["actions"])
    assert m["cosine"] >= 0.999 and m["max_abs"] <= 2e-2, m
    ptok = views * ocfg.patches_per_view + tokens_n
    hidden = ref.last_hidden.float().cpu().numpy()[[0, 100, -1]]
    assert O.compare(hidden, gold["hidden_rows"])["cosine"] >= 0.999
    k0 = ref.keys[0].float().cpu().numpy()[:ptok][[0, 100, -1]]
    assert O.compare(k0, gold["kv0_k_rows"])["cosine"] >= 0.9999
    ref.close()
    del ref
    import torch
    torch.cuda.empty_cache()
    cfg = Pi05Config(num_views=views, action_horizon=horizon)
    rt = Pi05Runtime.random(cfg, dtype="bf16", seed=weight_seed, device=0)
    g = rt.capture_infer_rgb_u8(tokens_n, "nhwc", 1)
    i2, t2, n2 = synthetic_observation(cfg, obs_seed, tokens_n)
    ours = g.infer_host(i2[None], t2[None], n2[None])[0]
    mo = O.compare(ours, got_ref)
    assert mo["cosine"] >= 0.999 and mo["max_abs"] <= 2e-2, mo
    g.close()
    rt.close()


def test_reference_library_ops_run_at_the_model_shapes():
    """The cuBLASLt FP8 / BF16 linear layers and the cuBLAS MQA of the reference's adapters,
    at two of the model's shapes (the timing legs of bench.py use the same calls)."""
    gemms = R.time_gemms({"vision.fc1": (512, 4304, 1152), "action.qkv": (10, 2560, 1024)}, iters=3)
    for name, entry in gemms.items():
        assert entry["bf16_us"] is not None and entry["bf16_us"] > 0, (name, entry)
    mqa = R.time_mqa({"action": (10, 532, 8, 256)}, iters=3)
    assert mqa["action"]["us"] > 0
