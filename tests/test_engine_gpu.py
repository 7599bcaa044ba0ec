"""PI0.5 engine (C ABI: pi05_engine_* / pi05_graph_*) against the CPU oracle on seeded
inputs, at a small architecture the oracle finishes in milliseconds. Integer/byte
artefacts (weights, quantised weights, scales, patch rows) must be bit-exact; floating
point tensors are compared with the tolerances written beside each check."""
import numpy as np
import pytest

from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu


def _runtime(cfg, dtype, seed=3, act_scale=0.05):
    from apxinf_b200.engine import Pi05Runtime
    return Pi05Runtime.random(cfg, dtype=dtype, seed=seed, device=0, fp8_act_scale=act_scale)


def _bf16(bits):
    return O.bf16_from_bits(np.asarray(bits, dtype=np.uint16))


@pytest.fixture(scope="module")
def cfg():
    return O.tiny_config()


def test_synthetic_weights_bit_exact_bf16(cfg):
    rt = _runtime(cfg, "bf16")
    w = O.SyntheticWeights(cfg, 3)
    lg = cfg.language
    # packed q|k|v, K-major [N, K]
    want = w.packed(["language.1.q", "language.1.k", "language.1.v"]).T
    got = _bf16(rt.read_weight("language.1.qkv.weight")).reshape(want.shape)
    assert np.array_equal(got, want)
    # gate/up interleaved in blocks of 64 rows
    gate, up = w.get("action.2.gate.weight").T, w.get("action.2.up.weight").T
    got = _bf16(rt.read_weight("action.2.gate_up.weight")).reshape(-1, 2, 64, gate.shape[1])
    assert np.array_equal(got[:, 0].reshape(gate.shape), gate)
    assert np.array_equal(got[:, 1].reshape(up.shape), up)
    # vision packed qkv with biases interleaved in the generation stream
    names = ["vision.1.q", "vision.1.k", "vision.1.v"]
    assert np.array_equal(_bf16(rt.read_weight("vision.1.qkv.bias")), w.packed_bias(names))
    want = w.packed(names).T
    assert np.array_equal(_bf16(rt.read_weight("vision.1.qkv.weight")).reshape(want.shape), want)
    # padded K (588 -> 592) of the patch embedding, last tensor of the stream
    pe = _bf16(rt.read_weight("vision.patch_embedding.weight")).reshape(cfg.vision_width, -1)
    assert pe.shape[1] == 592
    assert np.array_equal(pe[:, :588], w.get("vision.patch_embedding.weight").T)
    assert not pe[:, 588:].any()
    assert np.array_equal(_bf16(rt.read_weight("time_mlp_out.bias")), w.get("time_mlp_out.bias"))
    assert np.array_equal(_bf16(rt.read_weight("vision.position_embedding")).reshape(-1, cfg.vision_width),
                          w.get("vision.position_embedding"))
    rt.close()


def test_quantised_weights_bit_exact(cfg):
    w = O.SyntheticWeights(cfg, 3)
    names = ["language.0.q", "language.0.k", "language.0.v"]
    packed = w.packed(names)
    rt = _runtime(cfg, "fp8")
    q, scale = O.quantize_e4m3_channels(packed)
    assert np.array_equal(rt.read_weight("language.0.qkv.scale", np.float32), scale)
    got = rt.read_weight("language.0.qkv.weight", np.uint8).reshape(packed.shape[1], -1)
    assert np.array_equal(got, O.e4m3_encode(q).T)
    rt.close()
    rt = _runtime(cfg, "int8")
    q, scale = O.quantize_int8_channels(packed)
    assert np.array_equal(rt.read_weight("language.0.qkv.scale", np.float32), scale)
    got = rt.read_weight("language.0.qkv.weight", np.int8).reshape(packed.shape[1], -1)
    assert np.array_equal(got, q.T.astype(np.int8))
    rt.close()


@pytest.mark.parametrize("dtype,min_cos,max_abs", [("bf16", 0.999, 2e-2), ("fp8", 0.99, None),
                                                     ("int8", 0.99, None)])
@pytest.mark.parametrize("batch", [1, 3])
def test_forward_matches_oracle(cfg, dtype, min_cos, max_abs, batch):
    token_count = 6
    rt = _runtime(cfg, dtype)
    g = rt.capture_infer_rgb_u8(token_count, "nhwc", batch)
    obs = [O.synthetic_observation(cfg, 100 + i, token_count) for i in range(batch)]
    images = np.stack([o[0] for o in obs])
    tokens = np.stack([o[1] for o in obs])
    noise = np.stack([o[2] for o in obs])
    got = g.infer_host(images, tokens, noise)
    assert np.isfinite(got).all()
    for i in range(batch):
        oracle = O.Pi05Oracle(cfg, O.SyntheticWeights(cfg, 3),
                              O.OracleOptions(dtype=dtype, act_scale=0.05, vision_round_scores=True,
                                              collect=True))
        want = oracle.infer(*obs[i])
        m = O.compare(got[i], want)
        assert m["cosine"] >= min_cos, (dtype, i, m)
        if max_abs is not None:
            assert m["max_abs"] <= max_abs, (dtype, i, m)
        if i == 0 and dtype == "bf16":
            # intermediates: the residual stream after the prefix prefill (updated in place
            # from the embedded prefix) and the KV cache of the first / last layer
            width = cfg.language.width
            ptok = cfg.vision_tokens + token_count
            hidden = _bf16(g.read_tensor("prefix")).reshape(batch, ptok, width)[0]
            mp = O.compare(hidden, oracle.trace[f"language.{cfg.language.depth - 2}.hidden"])
            assert mp["cosine"] >= 0.9995, mp
            rows = ptok + cfg.action_horizon
            for layer in (0, cfg.language.depth - 1):
                k = _bf16(g.read_tensor(f"kv.{layer}.k")).reshape(batch, rows, -1)[0, :ptok]
                mk = O.compare(k, oracle.trace[f"kv.{layer}.k"][:, 0])
                assert mk["cosine"] >= 0.999, (layer, mk)
    # eager and graph replays of the same launch list agree bit for bit
    g.update_raw_image_inputs(images, tokens, noise)
    g.run_eager()
    eager = g.output()
    g.replay()
    assert np.array_equal(eager, g.output())
    assert g.workspace_used_bytes() <= g.workspace_bytes()
    g.close()
    rt.close()


def test_patch_rows_bit_exact(cfg):
    rt = _runtime(cfg, "bf16")
    g = rt.capture_infer_rgb_u8(4, "nhwc", 1)
    images, tokens, noise = O.synthetic_observation(cfg, 5, 4)
    g.infer_host(images[None], tokens[None], noise[None])
    got = _bf16(g.read_tensor("patches")).reshape(cfg.vision_tokens, -1)
    want = O.round_bf16(O.patchify(images, cfg))
    assert np.array_equal(got[:, :cfg.patch_width], want)
    assert not got[:, cfg.patch_width:].any()
    # NCHW wire layout gives the same patch rows (crates/apxinf-cuda/src/tests/fp8.rs:238-323)
    g2 = rt.capture_infer_rgb_u8(4, "nchw", 1)
    g2.infer_host(np.ascontiguousarray(images.transpose(0, 3, 1, 2))[None], tokens[None], noise[None])
    assert np.array_equal(_bf16(g2.read_tensor("patches")).reshape(cfg.vision_tokens, -1), got)
    g.close(); g2.close(); rt.close()


def test_capture_rejects_bad_shapes(cfg):
    from apxinf_b200 import Pi05Error
    rt = _runtime(cfg, "bf16")
    with pytest.raises(Pi05Error):
        rt.capture_infer_rgb_u8(0, "nhwc", 1)
    with pytest.raises(Pi05Error):
        rt.capture_infer_rgb_u8(cfg.max_token_len + 1, "nhwc", 1)
    rt.close()


# ---- the benchmark configurations' wording: N(0, 0.02) weights, static INT8 activations ----


def test_normal_weights_bit_exact(cfg):
    """The seeded N(0, 0.02) generator on the GPU equals the oracle's counter-based stream."""
    from apxinf_b200.engine import Pi05Runtime
    rt = Pi05Runtime.random(cfg, dtype="bf16", seed=3, device=0, weights_dist="normal")
    w = O.SyntheticWeights(cfg, 3, "normal")
    want = w.packed(["language.1.q", "language.1.k", "language.1.v"]).T
    got = _bf16(rt.read_weight("language.1.qkv.weight")).reshape(want.shape)
    assert np.array_equal(got, want)
    assert np.array_equal(_bf16(rt.read_weight("time_mlp_out.bias")), w.get("time_mlp_out.bias"))
    assert np.array_equal(_bf16(rt.read_weight("vision.position_embedding")).reshape(-1, cfg.vision_width),
                          w.get("vision.position_embedding"))
    values = w.get("vision.0.fc1.weight")
    assert abs(float(values.std()) - 0.02) < 1e-3 and abs(float(values.mean())) < 1e-3
    rt.close()


@pytest.mark.parametrize("dtype,min_cos,max_abs", [("bf16", 0.999, 2e-2), ("fp8", 0.99, None),
                                                     ("int8", 0.99, None)])
def test_forward_with_normal_weights(cfg, dtype, min_cos, max_abs):
    from apxinf_b200.engine import Pi05Runtime
    token_count = 6
    rt = Pi05Runtime.random(cfg, dtype=dtype, seed=5, device=0, fp8_act_scale=0.05,
                            weights_dist="normal")
    g = rt.capture_infer_rgb_u8(token_count, "nhwc", 1)
    images, tokens, noise = O.synthetic_observation(cfg, 21, token_count)
    got = g.infer_host(images[None], tokens[None], noise[None])[0]
    want = O.infer(cfg, 5, images, tokens, noise, weights_dist="normal", dtype=dtype,
                   act_scale=0.05, vision_round_scores=True)
    m = O.compare(got, want)
    assert m["cosine"] >= min_cos, m
    if max_abs is not None:
        assert m["max_abs"] <= max_abs, m
    g.close()
    rt.close()


@pytest.mark.parametrize("batch", [1, 2])
def test_static_int8_activations_match_oracle(cfg, batch):
    """One fixed scale per GEMM input, the quantiser fused into norms and epilogues. The site
    table is calibrated by the oracle (dynamic pass, absmax / 127) and set by name."""
    from apxinf_b200.engine import Pi05Runtime
    token_count = 6
    obs = [O.synthetic_observation(cfg, 300 + i, token_count) for i in range(batch)]
    weights = O.SyntheticWeights(cfg, 3)
    calib = O.Pi05Oracle(cfg, weights, O.OracleOptions(dtype="int8", calibrate=True,
                                                       vision_round_scores=True))
    for o in obs:
        calib.infer(*o)
    table = {site: max(a, 1e-6) / 127.0 for site, a in calib.amax.items()}
    rt = Pi05Runtime.random(cfg, dtype="int8", seed=3, device=0, fp8_act_scale=0.05,
                            int8_activations="static", activation_scales=table)
    assert abs(rt.activation_scale("action.input") - table["action.input"]) < 1e-9
    g = rt.capture_infer_rgb_u8(token_count, "nhwc", batch)
    # the static path has no per-row quantiser launches
    assert "quantize_rows_int8" not in g.launch_names()
    got = g.infer_host(np.stack([o[0] for o in obs]), np.stack([o[1] for o in obs]),
                       np.stack([o[2] for o in obs]))
    for i in range(batch):
        want = O.Pi05Oracle(cfg, weights, O.OracleOptions(
            dtype="int8", int8_act="static", act_scales=table, vision_round_scores=True)).infer(*obs[i])
        m = O.compare(got[i], want)
        assert m["cosine"] >= 0.99, (i, m)
    g.close()
    rt.close()


def test_activation_scale_sites(cfg):
    """FP8 with two sites set away from the uniform scale follows the oracle given the same
    table; unknown sites and bad values are refused."""
    from apxinf_b200 import Pi05Error
    from apxinf_b200.engine import Pi05Runtime
    table = {"vision.layers.0.mlp_activation": 0.02, "action.layers.1.attention_norm": 0.08,
             "language.layers.0.attention_output": 0.01, "action.input": 0.03}
    rt = Pi05Runtime.random(cfg, dtype="fp8", seed=3, device=0, fp8_act_scale=0.05,
                            activation_scales=table)
    with pytest.raises(Pi05Error):
        rt.set_activation_scale("vision.layers.99.mlp_norm", 0.1)
    with pytest.raises(Pi05Error):
        rt.set_activation_scale("action.input", -1.0)
    assert rt.activation_scale("time.hidden") == pytest.approx(0.05)
    token_count = 6
    g = rt.capture_infer_rgb_u8(token_count, "nhwc", 1)
    images, tokens, noise = O.synthetic_observation(cfg, 9, token_count)
    got = g.infer_host(images[None], tokens[None], noise[None])[0]
    want = O.infer(cfg, 3, images, tokens, noise, dtype="fp8", act_scale=0.05, act_scales=table,
                   vision_round_scores=True)
    uniform = O.infer(cfg, 3, images, tokens, noise, dtype="fp8", act_scale=0.05,
                      vision_round_scores=True)
    m = O.compare(got, want)
    assert m["cosine"] >= 0.99, m
    # the table matters: the engine is closer to the oracle with the table than without
    assert m["rmse"] <= O.compare(got, uniform)["rmse"] + 1e-6
    g.close()
    rt.close()
