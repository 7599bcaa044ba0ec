"""The denoise loop as one cooperative launch (pi05_set_tuning "persistent_denoise") and the
adaptive norms fused into the projections' staging ("fuse_norms"): both are alternative plans of
the same arithmetic, off by default, and must agree with the default launch list — the persistent
kernel bit for bit with the fused-norm launches (same bodies, same order of every sum), the fused
norms with the separate norm launches within the forward's tolerance (cosine >= 0.999 bf16,
>= 0.99 fp8 against the oracle). A barrier wait that can never complete (CTA 0 leaves out one
arrival) must end as PI05_ERR_DEVICE_TIMEOUT with the context still usable."""
import numpy as np
import pytest

from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu


def _tune(name, value):
    from apxinf_b200._lib import check, lib
    check(lib().pi05_set_tuning(name.encode(), int(value)), f"pi05_set_tuning({name})")


@pytest.fixture()
def defaults():
    yield
    for name, value in (("persistent_denoise", 0), ("fuse_norms", 0), ("denoise_skip_arrival", -1),
                        ("denoise_wait_limit_polls", 0)):
        _tune(name, value)


def _forward(rt, obs, tokens=6):
    g = rt.capture_infer_rgb_u8(tokens, "nhwc", 1)
    out = g.infer_host(*[x[None] for x in obs])[0]
    names = g.launch_names()
    # eager and graph replays of the same launch list agree bit for bit
    g.run_eager()
    assert np.array_equal(g.output()[0], out)
    g.close()
    return out, names


@pytest.mark.parametrize("dtype,min_cos", [("bf16", 0.999), ("fp8", 0.99)])
def test_persistent_kernel_matches_the_launch_list(defaults, dtype, min_cos):
    from apxinf_b200.engine import Pi05Runtime
    cfg = O.tiny_config()
    obs = O.synthetic_observation(cfg, 100, 6)
    rt = Pi05Runtime.random(cfg, dtype=dtype, seed=3, device=0, fp8_act_scale=0.05)
    base, base_names = _forward(rt, obs)
    _tune("fuse_norms", 1)
    fused, fused_names = _forward(rt, obs)
    _tune("persistent_denoise", 1)
    persistent, persistent_names = _forward(rt, obs)
    rt.close()
    assert "action.ada_norm" in base_names and "action.ada_norm" not in fused_names
    assert persistent_names.count("action.denoise") == 1 and "action.qkv" not in persistent_names
    assert len(persistent_names) < len(fused_names) < len(base_names)
    assert np.array_equal(persistent, fused)
    want = O.infer(cfg, 3, *obs, dtype=dtype, act_scale=0.05, vision_round_scores=True)
    for got in (base, fused):
        m = O.compare(got, want)
        assert m["cosine"] >= min_cos, m


def test_a_barrier_that_cannot_complete_times_out_cleanly(defaults):
    from apxinf_b200.engine import Pi05Runtime
    cfg = O.tiny_config()
    obs = O.synthetic_observation(cfg, 100, 6)
    rt = Pi05Runtime.random(cfg, dtype="bf16", seed=3, device=0)
    want, _ = _forward(rt, obs)
    _tune("persistent_denoise", 1)
    _tune("denoise_wait_limit_polls", 1 << 12)
    _tune("denoise_skip_arrival", 7)
    with pytest.raises(RuntimeError, match="PI05_ERR_DEVICE_TIMEOUT"):
        _forward(rt, obs)
    _tune("denoise_skip_arrival", -1)
    _tune("denoise_wait_limit_polls", 0)
    got, names = _forward(rt, obs)  # same engine, same stream, new plan
    assert "action.denoise" in names
    assert O.compare(got, want)["cosine"] >= 0.999
    rt.close()
