"""No-GPU checks: the shared library loads and exports every symbol the public header
declares; host-side argument validation answers without a device; sharding logic."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b((?:pi05|apxinf_static)_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    from apxinf_b200 import lib
    handle = lib()
    names = _declared_symbols()
    assert len(names) >= 30 and any(n.startswith("apxinf_static_") for n in names)
    for name in names:
        assert hasattr(handle, name), f"{name} declared in include/pi05_b200.h but not exported"
    assert handle.pi05_version().startswith(b"pi05_b200 sm_100a")


def test_default_config_is_the_two_view_profile():
    from apxinf_b200 import lib
    from apxinf_b200._abi_decls import ModelConfig
    c = ModelConfig()
    lib().pi05_default_config(C.byref(c))
    assert (c.num_views, c.action_horizon, c.num_flow_steps, c.max_token_len) == (2, 10, 10, 200)
    assert (c.vision_width, c.vision_depth, c.vision_mlp_dim, c.vision_heads, c.vision_head_dim) == \
        (1152, 27, 4304, 16, 72)
    assert (c.language.width, c.language.mlp_dim, c.action_expert.width, c.action_expert.mlp_dim) == \
        (2048, 16384, 1024, 4096)
    assert c.vocab_size == 257152


def test_null_arguments_are_rejected_without_a_device():
    from apxinf_b200 import lib
    handle = lib()
    assert handle.pi05_gemm(None, None) == -1
    assert handle.pi05_engine_create(None, 0, 0, 0, C.c_float(1.0), None) == -1
    assert handle.pi05_graph_replay(None) == -1
    assert handle.pi05_graph_output(None, None) == -1
    assert handle.pi05_graph_workspace_bytes(None) == 0
    assert handle.pi05_graph_launch_name(None, 0) is None


def test_python_config_mirrors_reference_defaults():
    from apxinf_b200.engine import Pi05Config
    from oracle import pi05_oracle as O
    ours, theirs = Pi05Config(), O.Pi05Config()
    for name in Pi05Config.__dataclass_fields__:
        a, b = getattr(ours, name), getattr(theirs, name)
        if name in ("language", "action_expert"):
            assert (a.width, a.depth, a.mlp_dim, a.num_heads, a.num_kv_heads, a.head_dim) == \
                (b.width, b.depth, b.mlp_dim, b.num_heads, b.num_kv_heads, b.head_dim)
        else:
            assert a == b, name
    assert Pi05Config.from_any(O.tiny_config()).vision_width == 144


def test_fixture_generator_matches_the_oracle_generator():
    from apxinf_b200.engine import Pi05Config, float_to_bf16_bits
    from apxinf_b200.fixtures import reference_image_pattern, synthetic_observation
    from oracle import pi05_oracle as O
    a = synthetic_observation(Pi05Config(), 9, 7)
    b = O.synthetic_observation(O.Pi05Config(), 9, 7)
    assert all(np.array_equal(x, y) for x, y in zip(a, b))
    assert np.array_equal(reference_image_pattern(Pi05Config()), O.reference_image_pattern(O.Pi05Config()))
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5], dtype=np.float32)
    assert np.array_equal(float_to_bf16_bits(x), O.bf16_bits(x))


def test_shard_bounds_cover_the_batch_exactly():
    from apxinf_b200.parallel import shard_bounds
    for batch, world in [(64, 1), (512, 8), (10, 4), (3, 8), (0, 2)]:
        shards = shard_bounds(batch, world)
        assert len(shards) == world
        assert shards[0].start == 0 and shards[-1].stop == batch
        assert all(a.stop == b.start for a, b in zip(shards, shards[1:]))
        sizes = [s.size for s in shards]
        assert max(sizes) - min(sizes) <= 1 and sum(sizes) == batch
    with pytest.raises(ValueError):
        shard_bounds(4, 0)
