"""The checkpoint path end to end on the device: a LeRobot-layout SafeTensors checkpoint written
from the synthetic weights must load (file -> key map -> pi05_engine_create_from_tensors) into
exactly the runtime that `random` builds — same packed / quantised weight bytes, same actions —
and a checkpoint with non-trivial norm parameters must match the oracle run on the loader's
tensor table."""
import numpy as np
import pytest

from checkpoint_fixture import expected_table, lerobot_tensors, write_checkpoint
from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cfg():
    return O.tiny_config()


def _load(cfg, path, dtype, **kwargs):
    from apxinf_b200 import checkpoint as ck
    from apxinf_b200.engine import Pi05Runtime
    return Pi05Runtime.from_tensors(cfg, ck.tensor_table(cfg, ck.load_path(path)), dtype=dtype, device=0,
                                    **kwargs)


@pytest.mark.parametrize("dtype", ["bf16", "fp8", "int8"])
@pytest.mark.parametrize("shards", [1, 3])
def test_loaded_checkpoint_equals_the_synthetic_runtime(cfg, dtype, shards, tmp_path):
    from apxinf_b200.engine import Pi05Runtime
    write_checkpoint(str(tmp_path), lerobot_tensors(cfg, 3, wrap_prefix=shards == 3), shards=shards)
    loaded = _load(cfg, str(tmp_path), dtype, fp8_act_scale=0.05)
    random = Pi05Runtime.random(cfg, dtype=dtype, seed=3, device=0, fp8_act_scale=0.05)
    names = ["vision.0.qkv.weight", "vision.1.fc2.weight", "vision.1.qkv.bias", "vision.patch_embedding.weight",
             "vision.position_embedding", "vision.projector.weight", "token_embedding",
             "language.0.qkv.weight", "language.2.gate_up.weight", "language.1.down.weight",
             "action.1.input_style.weight", "action.1.input_style.bias", "action.2.gate_up.weight",
             "action.final_style.weight", "action_in.weight", "action_out.bias", "time_mlp_out.weight"]
    if dtype != "bf16":
        names += ["language.0.qkv.scale", "action.2.gate_up.scale", "vision.1.fc2.scale"]
    for name in names:
        assert np.array_equal(loaded.read_weight(name, np.uint8), random.read_weight(name, np.uint8)), name
    # the loaded runtime also holds the LayerNorm parameters the synthetic one leaves implicit
    layer_norms = 2 * cfg.vision_depth + 1
    assert loaded.weight_bytes() - random.weight_bytes() == layer_norms * 2 * cfg.vision_width * 2
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    outs = []
    for rt in (loaded, random):
        g = rt.capture_infer_rgb_u8(6, "nhwc", 1)
        outs.append(g.infer_host(images[None], tokens[None], noise[None])[0])
        g.close()
        rt.close()
    assert np.isfinite(outs[0]).all()
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype,min_cos,max_abs", [("bf16", 0.999, 2e-2), ("fp8", 0.99, None),
                                                     ("int8", 0.99, None)])
def test_norm_parameters_and_folds_match_the_oracle(cfg, dtype, min_cos, max_abs, tmp_path):
    """LayerNorm gamma / beta and the `1 + w` folds away from their identity values: the device
    forward against the oracle over the same tensor table (tolerances: cosine over the action
    chunk; bf16 also max |difference|, two bf16 ulps at |a| < 4)."""
    tensors = lerobot_tensors(cfg, 5, norm_seed=11)
    write_checkpoint(str(tmp_path), tensors)
    rt = _load(cfg, str(tmp_path), dtype, fp8_act_scale=0.05)
    table = expected_table(cfg, 5, tensors)
    # packed weights of a folded projection: bf16 storage rounds the float32 fold, the quantised
    # precisions quantise it from float32
    want = np.concatenate([table[f"language.1.{p}.weight"] for p in ("q", "k", "v")], axis=1)
    if dtype == "bf16":
        got = O.bf16_from_bits(rt.read_weight("language.1.qkv.weight")).reshape(want.T.shape)
        assert np.array_equal(got, O.round_bf16(want).T)
    elif dtype == "int8":
        q, scale = O.quantize_int8_channels(want)
        assert np.array_equal(rt.read_weight("language.1.qkv.weight", np.int8).reshape(q.T.shape), q.T)
        assert np.array_equal(rt.read_weight("language.1.qkv.scale", np.float32), scale)
    else:
        q, scale = O.quantize_e4m3_channels(want)
        assert np.array_equal(rt.read_weight("language.1.qkv.weight", np.uint8).reshape(q.T.shape),
                              O.e4m3_encode(q).T)
        assert np.array_equal(rt.read_weight("language.1.qkv.scale", np.float32), scale)
    observation = O.synthetic_observation(cfg, 101, 6)
    g = rt.capture_infer_rgb_u8(6, "nhwc", 1)
    got = g.infer_host(*[x[None] for x in observation])[0]
    options = O.OracleOptions(dtype=dtype, act_scale=0.05, vision_round_scores=True, collect=True)
    oracle = O.Pi05Oracle(cfg, O.TableWeights(cfg, table), options)
    want = oracle.infer(*observation)
    m = O.compare(got, want)
    assert m["cosine"] >= min_cos, m
    if max_abs is not None:
        assert m["max_abs"] <= max_abs, m
    # the norm parameters matter where they act: the first layer's keys follow the oracle over the
    # loaded table and are far from what identity norms would give (the tiny model's actions are
    # dominated by the noise input, so this is checked on the cache, not on the chunk)
    plain = O.Pi05Oracle(cfg, O.SyntheticWeights(cfg, 5), options)
    plain.infer(*observation)
    ptok = cfg.vision_tokens + 6
    keys = O.bf16_from_bits(g.read_tensor("kv.0.k")).reshape(ptok + cfg.action_horizon, -1)[:ptok]
    close = O.compare(keys, oracle.trace["kv.0.k"][:, 0])
    far = O.compare(keys, plain.trace["kv.0.k"][:, 0])
    assert close["cosine"] >= min_cos, close
    assert far["max_abs"] > 5 * close["max_abs"] and far["cosine"] < close["cosine"], (close, far)
    g.close()
    rt.close()


def test_missing_and_mis_sized_tensors_are_named(cfg):
    from apxinf_b200 import _lib
    from apxinf_b200 import checkpoint as ck
    from apxinf_b200.engine import Pi05Runtime
    table = ck.tensor_table(cfg, {k: ck.HostArray("bf16", v) for k, v in lerobot_tensors(cfg, 3).items()})
    broken = dict(table)
    del broken["action.1.post_style.bias"]
    with pytest.raises(RuntimeError, match="PI05_ERR_INVALID_VALUE.*action.1.post_style.bias"):
        Pi05Runtime.from_tensors(cfg, broken, dtype="bf16")
    broken = dict(table)
    broken["language.2.down.weight"] = np.zeros(7, np.uint16)
    with pytest.raises(RuntimeError, match="language.2.down.weight"):
        Pi05Runtime.from_tensors(cfg, broken, dtype="fp8")
    with pytest.raises(ValueError, match="uint16 .bf16 bits. or float32"):
        Pi05Runtime.from_tensors(cfg, {"x": np.zeros(3, np.float64)}, dtype="bf16")
    # and a good table still loads afterwards
    Pi05Runtime.from_tensors(cfg, table, dtype="bf16").close()
