"""The `apxinf_py.Model` mirror: L0 (patches) and L1 (RGB) entries agree, as the reference's
python/tests/test_l0_l1_consistency.py requires, and argument checks raise the same errors."""
import numpy as np
import pytest

from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    from apxinf_b200 import apxinf_py
    m = apxinf_py.Model.random("pi05", device="cuda:0", precision="fp8", calibration="uniform:0.05", seed=3)
    yield m
    m.close()


def _inputs(model, seed, tokens=7):
    rng = np.random.default_rng(seed)
    rgb = rng.integers(0, 256, (model.num_views, model.image_size, model.image_size, 3), dtype=np.uint8)
    ids = rng.integers(0, 257152, tokens, dtype=np.uint32)
    noise = rng.standard_normal((model.action_horizon, model.action_dim)).astype(np.float32)
    return rgb, ids, noise


def test_shape_properties_follow_the_config(model):
    assert (model.device, model.action_dim, model.action_horizon, model.num_views) == ("cuda:0", 32, 10, 2)
    assert (model.image_size, model.patch_size, model.patches_per_view, model.max_token_len) == (224, 14, 256, 200)
    assert "views=2" in repr(model)


def test_l0_patches_and_l1_rgb_give_the_same_action(model):
    rgb, ids, noise = _inputs(model, 11)
    l1 = model.infer_rgb(rgb, "nhwc", ids, noise)
    patches = O.patchify(rgb, O.Pi05Config()).astype(np.float32)
    l0 = model._infer_patches(np.ascontiguousarray(patches), ids, noise)
    assert l1.shape == (10, 32) and l1.dtype == np.float32 and np.isfinite(l1).all()
    assert np.array_equal(l0, l1)


def test_nchw_layout_gives_the_same_action_as_nhwc(model):
    rgb, ids, noise = _inputs(model, 12, tokens=5)
    a = model.infer_rgb(rgb, "nhwc", ids, noise)
    b = model.infer_rgb(np.ascontiguousarray(rgb.transpose(0, 3, 1, 2)), "nchw", ids, noise)
    assert np.array_equal(a, b)


def test_argument_errors(model):
    rgb, ids, noise = _inputs(model, 13)
    with pytest.raises(ValueError, match="rgb_u8 expected 301056 bytes"):
        model.infer_rgb(rgb[:1], "nhwc", ids, noise)
    with pytest.raises(ValueError, match="token_ids must be non-empty"):
        model.infer_rgb(rgb, "nhwc", ids[:0], noise)
    with pytest.raises(ValueError, match="exceeds max_token_len 200"):
        model.infer_rgb(rgb, "nhwc", np.zeros(201, dtype=np.uint32), noise)
    with pytest.raises(ValueError, match=r"noise expected shape \[10, 32\]"):
        model.infer_rgb(rgb, "nhwc", ids, noise[:5])
    with pytest.raises(ValueError, match="unsupported image layout"):
        model.infer_rgb(rgb, "hwc", ids, noise)
    with pytest.raises(ValueError, match=r"patches expected shape \[512, 588\]"):
        model._infer_patches(np.zeros((512, 592), dtype=np.float32), ids, noise)


def test_random_model_takes_a_calibration_file(tmp_path):
    """`calibration` is "uniform:<scale>" or a json with one scale per named activation site
    (crates/apxinf-py/src/lib.rs:265-343): a file that sets every site to the uniform value gives
    the same actions bit for bit, a file with a site missing is refused by name."""
    import json
    from apxinf_b200 import apxinf_py, checkpoint
    from apxinf_b200.engine import Pi05Config
    sites = checkpoint.site_names(Pi05Config())
    path = tmp_path / "calibration.json"
    path.write_text(json.dumps({"scales": {name: 0.05 for name in sites}}))
    by_file = apxinf_py.Model.random("pi05", precision="fp8", calibration=str(path), seed=3)
    uniform = apxinf_py.Model.random("pi05", precision="fp8", calibration="uniform:0.05", seed=3)
    rgb, ids, noise = _inputs(uniform, 5)
    assert np.array_equal(by_file.infer_rgb(rgb, "nhwc", ids, noise), uniform.infer_rgb(rgb, "nhwc", ids, noise))
    by_file.close()
    uniform.close()
    path.write_text(json.dumps({name: 0.05 for name in sites[1:]}))
    with pytest.raises(RuntimeError, match="missing π0.5 FP8 activation scale `vision.layers.0.attention_norm`"):
        apxinf_py.Model.random("pi05", precision="fp8", calibration=str(path))
