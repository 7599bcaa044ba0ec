"""The owning frontend in the library (pi05_runtime_infer): one cached prepared plan keyed by
(token count, image layout), rebuilt when the observation's shape changes, eager fallback when
graph capture is unavailable, host-side noise dtype normalisation — the behaviour of
Pi05VlaRuntime::infer / prepare (crates/apxinf-model/src/pi05/vla_runtime.rs:393-495) — and the
stage signature of the integrity probe."""
import numpy as np
import pytest

from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cfg():
    return O.tiny_config()


@pytest.fixture()
def runtime(cfg):
    from apxinf_b200.engine import Pi05Runtime
    rt = Pi05Runtime.random(cfg, dtype="bf16", seed=3, device=0)
    yield rt
    rt.close()


def _direct(rt, layout, image, tokens, noise):
    g = rt.capture_infer_patches(tokens.size) if layout == "patches" else \
        rt.capture_infer_rgb_u8(tokens.size, layout)
    out = g.infer_host(image[None], tokens[None], noise[None])[0]
    g.close()
    return out


def test_plan_is_cached_by_shape_and_rebuilt_on_change(cfg, runtime):
    from apxinf_b200.engine import PolicyRuntime
    front = PolicyRuntime(runtime)
    assert front.plan_info() == {"token_count": 0, "image_layout": 0, "uses_graph": 0, "builds": 0}
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    first = front.infer("nhwc", images, tokens, noise)
    assert front.plan_info() == {"token_count": 6, "image_layout": 0, "uses_graph": 1, "builds": 1}
    assert np.array_equal(first, _direct(runtime, "nhwc", images, tokens, noise))
    # same shape, other content: the cached plan is replayed
    images2, tokens2, noise2 = O.synthetic_observation(cfg, 101, 6)
    second = front.infer("nhwc", images2, tokens2, noise2)
    assert front.plan_info()["builds"] == 1
    assert np.array_equal(second, _direct(runtime, "nhwc", images2, tokens2, noise2))
    assert not np.array_equal(first, second)
    # other token count: rebuilt; back again: rebuilt again (one plan is kept, not a table)
    images3, tokens3, noise3 = O.synthetic_observation(cfg, 102, 9)
    third = front.infer("nhwc", images3, tokens3, noise3)
    assert front.plan_info() == {"token_count": 9, "image_layout": 0, "uses_graph": 1, "builds": 2}
    assert np.array_equal(third, _direct(runtime, "nhwc", images3, tokens3, noise3))
    assert np.array_equal(front.infer("nhwc", images, tokens, noise), first)
    assert front.plan_info()["builds"] == 3
    # other layout, same token count: a different plan too
    nchw = np.ascontiguousarray(images.transpose(0, 3, 1, 2))
    assert np.array_equal(front.infer("nchw", nchw, tokens, noise), first)
    assert front.plan_info() == {"token_count": 6, "image_layout": 1, "uses_graph": 1, "builds": 4}
    patches = O.patchify(images, cfg)
    assert np.array_equal(front.infer("patches", patches, tokens, noise),
                          _direct(runtime, "patches", patches, tokens, noise))
    assert front.plan_info()["image_layout"] == 2
    front.close()


def test_eager_fallback_when_capture_is_unavailable(cfg, runtime):
    from apxinf_b200._lib import check, lib
    from apxinf_b200.engine import PolicyRuntime
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    want = _direct(runtime, "nhwc", images, tokens, noise)
    check(lib().pi05_set_tuning(b"force_capture_failure", 1), "pi05_set_tuning")
    try:
        front = PolicyRuntime(runtime)
        got = front.infer("nhwc", images, tokens, noise)
        assert front.plan_info() == {"token_count": 6, "image_layout": 0, "uses_graph": 0, "builds": 1}
        assert np.array_equal(got, want)  # the same launch list, run eagerly
        assert np.array_equal(front.infer("nhwc", images, tokens, noise), want)
        assert front.plan_info()["builds"] == 1
    finally:
        check(lib().pi05_set_tuning(b"force_capture_failure", 0), "pi05_set_tuning")
    # the next plan captures again
    images3, tokens3, noise3 = O.synthetic_observation(cfg, 102, 9)
    front.infer("nhwc", images3, tokens3, noise3)
    assert front.plan_info()["uses_graph"] == 1
    front.close()


def test_noise_is_normalised_to_the_runtime_type_on_the_host(cfg, runtime):
    from apxinf_b200.engine import PolicyRuntime
    front = PolicyRuntime(runtime)
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    noise = (noise * np.float32(1.2345)).astype(np.float32)  # not representable in bf16
    from_f32 = front.infer("nhwc", images, tokens, noise)
    from_bits = front.infer("nhwc", images, tokens, O.bf16_bits(noise))
    assert np.array_equal(from_f32, from_bits)
    assert front.plan_info()["builds"] == 1
    front.close()


def test_bad_observations_are_refused(cfg, runtime):
    from apxinf_b200.engine import PolicyRuntime
    front = PolicyRuntime(runtime)
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    with pytest.raises(RuntimeError, match="PI05_ERR_INVALID_VALUE"):
        front.infer("nhwc", images, np.zeros(cfg.max_token_len + 1, np.uint32), noise)
    with pytest.raises(ValueError, match="expected"):
        front.infer("nhwc", images[:1], tokens, noise)
    with pytest.raises(ValueError, match="noise has"):
        front.infer("nhwc", images, tokens, noise[:2])
    assert front.plan_info()["builds"] == 0
    assert np.isfinite(front.infer("nhwc", images, tokens, noise)).all()
    front.close()


def test_stage_signature_matches_the_tensor(cfg, runtime):
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    g = runtime.capture_infer_rgb_u8(6, "nhwc", 1)
    g.infer_host(images[None], tokens[None], noise[None])
    for name in ("patches", "prefix", "kv.0.k"):
        values = O.bf16_from_bits(g.read_tensor(name)).astype(np.float64)
        sig = g.signature(name)
        assert sig["elements"] == values.size
        assert sig["sum"] == pytest.approx(values.sum(), rel=1e-12, abs=1e-9)
        assert sig["abs_checksum"] == pytest.approx(np.abs(values).sum(), rel=1e-12)
        assert sig["l2"] == pytest.approx(np.sqrt((values * values).sum()), rel=1e-12)
        assert sig["max_abs"] == np.abs(values).max()
        count = min(values.size, 256)
        index = np.arange(count) * (values.size - 1) // (count - 1)
        assert np.array_equal(sig["sample"], values[index].astype(np.float32))
    with pytest.raises(RuntimeError, match="PI05_ERR_INVALID_VALUE"):
        g.signature("no.such.tensor")
    g.close()
