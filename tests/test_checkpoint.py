"""Checkpoint path on the host (no GPU): SafeTensors container, LeRobot key map, config.json and
calibration parsing — the cases of the reference's own unit tests for these
(crates/apxinf-model/src/pi05/config.rs:502-580, weights.rs tests, fp8.rs / runtime.rs:850-860,
vla_runtime.rs:774-788, crates/apxinf-loader/src/safetensors.rs) plus round trips."""
import json
import os

import numpy as np
import pytest

from apxinf_b200 import checkpoint as ck
from apxinf_b200.engine import Pi05Config
from checkpoint_fixture import expected_table, lerobot_tensors, write_checkpoint
from oracle import pi05_oracle as O


@pytest.fixture(scope="module")
def cfg():
    return O.tiny_config()  # the loader only reads attributes both config classes have


def test_container_round_trip_and_official_reader(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"a": ck.HostArray("bf16", rng.integers(0, 65536, (3, 5), dtype=np.uint16)),
               "b.c": ck.HostArray("f32", rng.standard_normal((7,)).astype(np.float32)),
               "h": ck.HostArray("f16", rng.standard_normal((2, 2)).astype(np.float16).view(np.uint16))}
    path = str(tmp_path / "x.safetensors")
    ck.save_file(path, tensors)
    back = ck.load_file(path)
    assert set(back) == set(tensors)
    for name in tensors:
        assert back[name].kind == tensors[name].kind and np.array_equal(back[name].data, tensors[name].data)
    torch = pytest.importorskip("torch")
    st = pytest.importorskip("safetensors.torch")
    official = st.load_file(path)
    assert official["a"].dtype == torch.bfloat16
    assert np.array_equal(official["a"].view(torch.uint16).numpy(), tensors["a"].data)
    assert np.array_equal(official["b.c"].numpy(), tensors["b.c"].data)
    # and the other way round: a file written by the official library
    other = str(tmp_path / "y.safetensors")
    st.save_file({"w": torch.arange(12, dtype=torch.float32).reshape(3, 4).to(torch.bfloat16)}, other)
    mine = ck.load_file(other)["w"]
    assert mine.kind == "bf16" and np.array_equal(mine.to_f32(), np.arange(12, dtype=np.float32).reshape(3, 4))


def test_container_rejects_truncated_files(tmp_path):
    path = tmp_path / "t.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(ck.CheckpointError, match="too small"):
        ck.load_file(str(path))
    path.write_bytes((1000).to_bytes(8, "little") + b"{}")
    with pytest.raises(ck.CheckpointError, match="expected at least 1008"):
        ck.load_file(str(path))


def test_directory_index_and_shard_rules(tmp_path, cfg):
    tensors = lerobot_tensors(cfg, 3)
    single, sharded = str(tmp_path / "single"), str(tmp_path / "sharded")
    write_checkpoint(single, tensors)
    write_checkpoint(sharded, tensors, shards=3)
    a, b = ck.load_path(single), ck.load_path(sharded)
    c = ck.load_path(os.path.join(sharded, "model.safetensors.index.json"))
    assert set(a) == set(b) == set(c) == set(tensors)
    assert all(np.array_equal(a[k].data, b[k].data) for k in a)
    # an index that assigns a tensor to another shard than the one holding it
    index_path = os.path.join(sharded, "model.safetensors.index.json")
    index = json.load(open(index_path))
    name = next(iter(index["weight_map"]))
    files = sorted(set(index["weight_map"].values()))
    index["weight_map"][name] = next(f for f in files if f != index["weight_map"][name])
    json.dump(index, open(index_path, "w"))
    with pytest.raises(ck.CheckpointError, match="index assigns it to"):
        ck.load_path(sharded)
    index["weight_map"] = {"x": "../escape.safetensors"}
    json.dump(index, open(index_path, "w"))
    with pytest.raises(ck.CheckpointError, match="unsafe shard path"):
        ck.load_path(sharded)
    json.dump({"weight_map": {}}, open(index_path, "w"))
    with pytest.raises(ck.CheckpointError, match="empty weight_map"):
        ck.load_path(sharded)
    os.remove(index_path)
    with pytest.raises(ck.CheckpointError, match="multiple SafeTensors files"):
        ck.load_path(sharded)
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(ck.CheckpointError, match="no SafeTensors model or index"):
        ck.load_path(str(empty))


def test_config_parses_lerobot_aliases():
    got = ck.config_from_json('''{"max_action_dim": 32, "chunk_size": 10, "tokenizer_max_length": 200,
        "num_inference_steps": 10, "num_views": 2, "image_resolution": [224, 224],
        "discrete_state_input": false}''')
    assert got == Pi05Config(num_views=2, action_horizon=10, num_flow_steps=10)  # the two-view profile
    assert got.patches_per_view == 256
    assert got.num_views * got.patches_per_view + got.max_token_len == 712


def test_config_rejects_invalid_horizon():
    with pytest.raises(ck.CheckpointError, match="action_horizon"):
        ck.config_from_json('{"chunk_size": 0}')
    with pytest.raises(ck.CheckpointError, match="action_horizon"):
        ck.config_from_json('{"chunk_size": 51}')


def test_config_derives_views_from_input_features():
    raw = {"input_features": {"observation.images.image": {"type": "VISUAL", "shape": [3, 256, 256]},
                              "observation.images.image2": {"type": "VISUAL", "shape": [3, 256, 256]},
                              "observation.state": {"type": "STATE", "shape": [8]}},
           "empty_cameras": 1, "chunk_size": 50, "num_inference_steps": 10, "image_resolution": [224, 224]}
    assert ck.config_from_json(json.dumps(raw)).num_views == 2
    raw["num_views"] = 3
    assert ck.config_from_json(json.dumps(raw)).num_views == 3
    assert ck.config_from_json("{}") == ck.DEFAULT_CONFIG
    assert (ck.DEFAULT_CONFIG.num_views, ck.DEFAULT_CONFIG.action_horizon) == (3, 50)


def test_key_map_reproduces_the_synthetic_tensors(cfg):
    tensors = lerobot_tensors(cfg, 3)
    table = ck.tensor_table(cfg, {k: ck.HostArray("bf16", v) for k, v in tensors.items()})
    want = expected_table(cfg, 3, tensors)
    assert set(table) == set(want)
    for name, value in want.items():
        assert table[name].shape == value.shape, name
        assert np.array_equal(table[name].to_f32(), value), name
    # folded projections come out as float32, like the reference's fold; the rest stays bf16
    assert table["language.0.q.weight"].kind == "f32" and table["language.0.gate.weight"].kind == "f32"
    assert table["language.0.o.weight"].kind == "bf16" and table["action.0.q.weight"].kind == "bf16"


def test_key_map_folds_one_plus_w_in_float32(cfg):
    tensors = lerobot_tensors(cfg, 5, norm_seed=11, wrap_prefix=True, embedding_alias=True)
    table = ck.tensor_table(cfg, {k: ck.HostArray("bf16", v) for k, v in tensors.items()})
    want = expected_table(cfg, 5, tensors)
    for name, value in want.items():
        assert np.array_equal(table[name].to_f32(), value), name
    # the fold is not representable in bf16: it must have stayed float32
    q = table["language.1.q.weight"].to_f32()
    assert not np.array_equal(O.round_bf16(q), q)


def test_key_map_errors(cfg):
    tensors = {k: ck.HostArray("bf16", v) for k, v in lerobot_tensors(cfg, 3).items()}
    broken = dict(tensors)
    del broken["time_mlp_in.bias"]
    with pytest.raises(ck.CheckpointError, match="missing π0.5 weight `time_mlp_in.bias`"):
        ck.tensor_table(cfg, broken)
    broken = dict(tensors)
    del broken["paligemma_with_expert.paligemma.model.language_model.embed_tokens.weight"]
    with pytest.raises(ck.CheckpointError, match="accepted aliases"):
        ck.tensor_table(cfg, broken)
    broken = dict(tensors)
    broken["action_in_proj.weight"] = ck.HostArray("bf16", np.zeros((cfg.action_expert.width, 7), np.uint16))
    with pytest.raises(ck.CheckpointError, match="action_in: expected weight shape"):
        ck.tensor_table(cfg, broken)
    broken = dict(tensors)
    broken["time_mlp_out.weight"] = ck.HostArray("bf16", np.zeros((4,), np.uint16))
    with pytest.raises(ck.CheckpointError, match="must be 2D"):
        ck.tensor_table(cfg, broken)


def test_calibration_forms_and_errors(cfg):
    got = ck.calibration_from_json('{"a": 0.5, "b": {"scale": 0.25}, "c": {"amax": 224.0}}')
    assert got == {"a": 0.5, "b": 0.25, "c": 0.5}
    assert ck.calibration_from_json('{"scales": {"x": 2}}') == {"x": 2.0}
    with pytest.raises(ck.CheckpointError, match="`a` has invalid scale"):
        ck.calibration_from_json('{"a": -1}')
    with pytest.raises(ck.CheckpointError, match="no numeric scale or amax"):
        ck.calibration_from_json('{"a": "x"}')
    with pytest.raises(ck.CheckpointError, match="must be a JSON object"):
        ck.calibration_from_json('[1]')
    # the first missing scale is named, in the reference's resolution order
    with pytest.raises(ck.CheckpointError, match=r"vision\.layers\.0\.attention_norm"):
        ck.calibration_scales(cfg, {})
    full = {name: 0.1 for name in ck.site_names(cfg)}
    assert ck.calibration_scales(cfg, full) == full
    depth = cfg.vision_depth + cfg.language.depth + cfg.action_expert.depth
    assert len(full) == 4 * depth + 7


def test_auto_precision_policy():
    assert ck.resolve_precision("auto", 110, True) == "fp8"
    assert ck.resolve_precision("auto", 110, False) == "bf16"
    assert ck.resolve_precision("auto", 87, True) == "int8"
    assert ck.resolve_precision("auto", 100, True) == "fp8"
    assert ck.resolve_precision("bf16", 100, True) == "bf16"


def test_model_load_reports_loader_errors_without_a_device(tmp_path):
    from apxinf_b200 import apxinf_py
    with pytest.raises(ValueError, match="unknown model"):
        apxinf_py.Model.load("llama", str(tmp_path))
    with pytest.raises(ValueError, match="unsupported precision"):
        apxinf_py.Model.load("pi05", str(tmp_path), precision="fp4")
    with pytest.raises(ValueError, match="unsupported device"):
        apxinf_py.Model.load("pi05", str(tmp_path), device="cpu")
    (tmp_path / "config.json").write_text('{"chunk_size": 10, "num_views": 2}')
    with pytest.raises(RuntimeError, match="no SafeTensors model or index"):
        apxinf_py.Model.load("pi05", str(tmp_path), precision="bf16")
    with pytest.raises(RuntimeError, match="action_horizon must be in 1..=50"):
        apxinf_py.Model.load("pi05", str(tmp_path), precision="bf16", action_horizon=64)
    with pytest.raises(RuntimeError, match="requires LoadOptions.calibration_path or calibration.json"):
        apxinf_py.Model.load("pi05", str(tmp_path), precision="fp8")
    (tmp_path / "calibration.json").write_text("{}")
    with pytest.raises(RuntimeError, match=r"missing π0.5 FP8 activation scale `vision\.layers\.0\.attention_norm`"):
        apxinf_py.Model.load("pi05", str(tmp_path), precision="fp8")
