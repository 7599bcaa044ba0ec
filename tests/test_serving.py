"""The serving shell on the host (no GPU): wire codec, processors, the policy's layering and the
websocket protocol, with the known answers of the reference's own tests for them
(python/apxinf/tests/test_{tokenize,normalize_golden,resize_golden,policy_layering}.py) and a stub
in place of the model."""
import asyncio
import json

import numpy as np
import pytest

from apxinf_b200 import serving as S


# ---- codec ------------------------------------------------------------------------------------
def test_codec_round_trips_arrays_scalars_and_plain_values():
    message = {"actions": np.arange(12, dtype=np.float32).reshape(3, 4), "step": np.int64(7),
               "prompt": "pick", "nested": {"rgb": np.zeros((2, 2, 3), np.uint8)}, "list": [1, 2.5, None]}
    back = S.unpack(S.pack(message))
    assert back["prompt"] == "pick" and back["list"] == [1, 2.5, None]
    assert back["actions"].dtype == np.float32 and np.array_equal(back["actions"], message["actions"])
    assert isinstance(back["step"], np.int64) and back["step"] == 7
    assert np.array_equal(back["nested"]["rgb"], message["nested"]["rgb"])
    with pytest.raises(ValueError, match="unsupported NumPy dtype"):
        S.pack({"x": np.array([1 + 2j])})
    # the tagged-map layout the OpenPI client reads
    import msgpack
    raw = msgpack.unpackb(S.pack({"a": np.ones(2, np.float32)}))
    assert set(raw["a"]) == {b"__ndarray__", b"data", b"dtype", b"shape"} and raw["a"][b"dtype"] == "<f4"


# ---- images -----------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(224, 224, 3), (256, 320, 3), (480, 640, 3), (100, 50, 3)])
def test_letterbox_resize(shape):
    from PIL import Image
    rng = np.random.default_rng(0)
    image = rng.integers(0, 256, size=shape, dtype=np.uint8)
    got = S.resize_with_pad(S.parse_image(image), 224)
    assert got.shape == (224, 224, 3) and got.dtype == np.uint8
    if shape[:2] == (224, 224):
        assert np.array_equal(got, image)
        return
    h, w = shape[:2]
    ratio = max(w / 224, h / 224)
    nh, nw = int(h / ratio), int(w / ratio)
    top, left = int((224 - nh) / 2), int((224 - nw) / 2)
    inner = np.asarray(Image.fromarray(image).resize((nw, nh), resample=Image.Resampling.BILINEAR))
    assert np.array_equal(got[top:top + nh, left:left + nw], inner)
    mask = np.ones((224, 224), bool)
    mask[top:top + nh, left:left + nw] = False
    assert not got[mask].any()  # black bars


def test_parse_image_forms():
    rng = np.random.default_rng(1)
    chw = rng.random((3, 8, 6)).astype(np.float32)
    got = S.parse_image(chw)
    assert got.shape == (8, 6, 3) and got.dtype == np.uint8
    assert np.array_equal(got, (255 * chw).astype(np.uint8).transpose(1, 2, 0))
    with pytest.raises(ValueError, match="rank 3"):
        S.parse_image(np.zeros((4, 4)))
    with pytest.raises(ValueError, match="three RGB channels"):
        S.parse_image(np.zeros((4, 4, 4), np.uint8))
    with pytest.raises(ValueError, match="uint8 or floating"):
        S.parse_image(np.zeros((4, 4, 3), np.int32))


# ---- prompt -----------------------------------------------------------------------------------
def test_prompt_known_answers():
    assert S.build_prompt("  pick_up the\nblock  ") == "pick up the block"
    assert S.build_prompt("open_drawer", state=[-1.0, 0.0, 1.0], discrete_state=True) == \
        "Task: open drawer, State: 0 128 255;\nAction: "
    with pytest.raises(ValueError):
        S.build_prompt("task", state=None, discrete_state=True)


def test_discretize_state_is_digitize_with_saturation():
    rng = np.random.default_rng(2)
    state = np.concatenate([rng.uniform(-1.5, 1.5, 500), [-1.0, 1.0, 0.0, -2.0, 2.0]])
    edges = np.linspace(-1.0, 1.0, 257)[:-1]
    want = np.clip(np.digitize(state, edges) - 1, 0, 255).astype(np.uint8)
    assert np.array_equal(S.discretize_state(state), want)


@pytest.fixture(scope="module")
def tokenizer_path(tmp_path_factory):
    sentencepiece = pytest.importorskip("sentencepiece")
    folder = tmp_path_factory.mktemp("sp")
    corpus = folder / "corpus.txt"
    words = ["pick", "up", "the", "red", "block", "open", "drawer", "task", "state", "action", "put", "bowl", "on", "plate"]
    rng = np.random.default_rng(3)
    corpus.write_text("\n".join(" ".join(rng.choice(words, 6)) for _ in range(400)))
    prefix = str(folder / "tiny")
    sentencepiece.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=64,
                                             model_type="bpe", bos_id=1, eos_id=2, unk_id=0, pad_id=-1,
                                             user_defined_symbols=["\n"], minloglevel=2)
    return prefix + ".model"


def test_tokenizer_adds_bos_and_newline(tokenizer_path):
    import sentencepiece
    sp = sentencepiece.SentencePieceProcessor(model_file=tokenizer_path)
    prompt = "pick_up the block\n"
    want = list(sp.encode("pick up the block", add_bos=True)) + list(sp.encode("\n"))
    got = S.PromptTokenizer(tokenizer_path)(prompt)
    assert got.dtype == np.uint32 and np.array_equal(got, np.asarray(want, np.uint32))
    with pytest.raises(ValueError, match="token count must be in 1..=1"):
        S.PromptTokenizer(tokenizer_path, max_token_len=1)(prompt)
    with_state = S.PromptTokenizer(tokenizer_path, discrete_state=True)("open drawer", [-1.0, 0.0, 1.0])
    assert np.array_equal(with_state, np.asarray(
        sp.encode("Task: open drawer, State: 0 128 255;\nAction: ", add_bos=True), np.uint32))
    ramp = S.SyntheticTokenizer(10)("anything")
    assert np.array_equal(ramp, np.arange(1, 11, dtype=np.uint32))
    with pytest.raises(ValueError):
        S.SyntheticTokenizer(201)


# ---- normalisation ----------------------------------------------------------------------------
def test_quantile_and_mean_std_maps(tmp_path):
    rng = np.random.default_rng(0)
    q01 = rng.uniform(-2.0, -0.5, 7).astype(np.float32)
    q99 = rng.uniform(0.5, 2.0, 7).astype(np.float32)
    normalized = rng.uniform(-1.0, 1.0, (10, 7)).astype(np.float32)
    got = S.Unnormalizer(q01=q01, q99=q99)(normalized)
    want = ((normalized + 1.0) * (q99 - q01 + np.float32(1.0e-6)) / 2.0 + q01).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-6)
    np.testing.assert_allclose(S.Normalizer(q01=q01, q99=q99)(got), normalized, rtol=0, atol=1e-4)
    mean, std = rng.standard_normal(7).astype(np.float32), rng.uniform(0.5, 2, 7).astype(np.float32)
    np.testing.assert_allclose(S.Unnormalizer(mean=mean, std=std, mode="mean_std")(normalized), normalized * std + mean)
    # norm_stats.json, nested and flat, trimmed to the task's action width
    stats = {"actions": {"q01": q01.tolist() + [0.0], "q99": q99.tolist() + [1.0]}}
    for document in ({"norm_stats": stats}, stats):
        (tmp_path / "norm_stats.json").write_text(json.dumps(document))
        u = S.Unnormalizer.from_norm_stats(str(tmp_path), dims=7)
        assert u.width == 7 and np.allclose(u(normalized), want, atol=1e-6)
    with pytest.raises(KeyError, match="no entry 'state'"):
        S.load_norm_stats(str(tmp_path), "state")
    with pytest.raises(ValueError, match="last dim must be 7"):
        S.Unnormalizer(q01=q01, q99=q99)(np.zeros((2, 8), np.float32))
    with pytest.raises(FloatingPointError):
        S.Unnormalizer(q01=q01, q99=q99)(np.full((1, 7), np.inf, np.float32))


# ---- policy -----------------------------------------------------------------------------------
class StubModel:
    """Stands in for apxinf_py.Model: a deterministic function of its inputs."""
    action_horizon, action_dim, num_views, image_size, max_token_len = 4, 8, 2, 224, 200

    def __init__(self):
        self.calls = []

    def infer_rgb(self, rgb, layout, token_ids, noise):
        assert rgb.dtype == np.uint8 and rgb.shape == (2, 224, 224, 3) and rgb.flags.c_contiguous
        assert layout == "nhwc" and token_ids.dtype == np.uint32 and noise.dtype == np.float32
        self.calls.append((rgb.copy(), token_ids.copy(), noise.copy()))
        return np.tanh(noise + np.float32(rgb.mean() / 255.0) + np.float32(token_ids.sum() % 7) / 10)


def _observation(seed=0):
    rng = np.random.default_rng(seed)
    return {"observation/image": rng.integers(0, 256, (256, 320, 3), dtype=np.uint8),
            "observation/wrist_image": rng.random((3, 224, 224)).astype(np.float32),
            "observation/state": rng.uniform(-1, 1, 8).astype(np.float32), "prompt": "pick_up the block"}


def test_policy_layers_pre_model_post():
    model = StubModel()
    with pytest.warns(UserWarning, match="latency-only"):
        policy = S.Pi05Policy.from_random(model, token_count=12, action_dim=7, seed=5)
    assert policy.metadata["action_dim"] == 7 and policy.metadata["model_action_dim"] == 8
    assert policy.metadata["input_pipeline"] == ["image_stack", "tokenize", "sample_noise"]
    assert policy.metadata["output_pipeline"] == ["trim", "unnormalize"] and policy.metadata["weights"] == "synthetic"
    observation = _observation()
    result = policy.infer(observation)
    rgb, tokens, noise = model.calls[-1]
    assert np.array_equal(rgb[0], S.resize_with_pad(S.parse_image(observation["observation/image"]), 224))
    assert np.array_equal(rgb[1], S.parse_image(observation["observation/wrist_image"]))
    assert np.array_equal(tokens, np.arange(1, 13, dtype=np.uint32))
    assert np.array_equal(noise, np.random.default_rng(5).standard_normal((4, 8), dtype=np.float32))
    # L2 minus unnormalize == L1: identity statistics leave the trimmed model output unchanged
    assert result["actions"].shape == (4, 7) and np.allclose(result["actions"], result["normalized_actions"][:, :7], atol=1e-6)
    assert np.array_equal(result["normalized_actions"], model.infer_rgb(rgb, "nhwc", tokens, noise))
    assert set(result) == {"actions", "normalized_actions", "token_ids", "noise", "timing", "metadata"}
    assert result["timing"]["total_ms"] >= result["timing"]["model_ms"] >= 0
    # the prior advances between calls and restarts on reset
    second = policy.infer(observation)
    assert not np.array_equal(second["noise"], result["noise"])
    policy.noise.reset()
    assert np.array_equal(policy.infer(observation)["noise"], result["noise"])
    with pytest.raises(KeyError, match="observation/wrist_image"):
        policy.infer({k: v for k, v in observation.items() if k != "observation/wrist_image"})
    with pytest.raises(TypeError, match="prompt must be a string"):
        policy.infer({**observation, "prompt": 3})
    with pytest.raises(ValueError, match="expects 2 camera views but 1"):
        S.Pi05Policy.from_random(model, image_keys=("observation/image",), warn=False)
    # a step can be swapped by name
    policy.image_pipeline.replace("resize", lambda image: np.zeros((224, 224, 3), np.uint8))
    policy.infer(observation)
    assert not model.calls[-1][0].any()


def test_policy_from_pretrained_reads_the_directory(tmp_path, tokenizer_path):
    import shutil
    model = StubModel()
    shutil.copy(tokenizer_path, tmp_path / "tokenizer.model")
    q01, q99 = [-2.0] * 8, [3.0] * 8
    (tmp_path / "norm_stats.json").write_text(json.dumps({"norm_stats": {
        "actions": {"q01": q01, "q99": q99}, "state": {"q01": [-4.0] * 8, "q99": [4.0] * 8}}}))
    policy = S.Pi05Policy.from_pretrained(str(tmp_path), model=model, action_dim=7, discrete_state=True, seed=1)
    observation = _observation(1)
    result = policy.infer(observation)
    state = S.Normalizer(q01=[-4.0] * 8, q99=[4.0] * 8)(observation["observation/state"])
    want_tokens = S.PromptTokenizer(str(tmp_path / "tokenizer.model"), discrete_state=True)("pick_up the block", state)
    assert np.array_equal(result["token_ids"], want_tokens)
    want = (result["normalized_actions"][:, :7] + 1.0) * ((3.0 + 2.0 + 1e-6) / 2.0) - 2.0
    assert np.allclose(result["actions"], want, atol=1e-5)
    assert policy.metadata["discrete_state"] and policy.metadata["state_normalized"]
    with pytest.raises(ValueError, match="conflicts with the supplied model's horizon"):
        S.Pi05Policy.from_pretrained(str(tmp_path), model=model, action_horizon=9)


# ---- websocket --------------------------------------------------------------------------------
def test_websocket_protocol_end_to_end():
    websockets = pytest.importorskip("websockets")
    model = StubModel()
    policy = S.Pi05Policy.from_random(model, action_dim=7, seed=2, warn=False)
    server = S.WebsocketPolicyServer(policy, "127.0.0.1", 0)

    async def scenario():
        started = asyncio.Event()
        task = asyncio.create_task(server.run(started))
        await asyncio.wait_for(started.wait(), 10)
        port = server.bound_port
        try:
            # health check over plain HTTP
            reader, writer = await asyncio.open_connection("127.0.0.1", port)
            writer.write(b"GET /healthz HTTP/1.1\r\nHost: x\r\n\r\n")
            await writer.drain()
            reply = await asyncio.wait_for(reader.read(200), 10)
            writer.close()
            assert reply.startswith(b"HTTP/1.1 200") and reply.rstrip().endswith(b"OK")
            async with websockets.connect(f"ws://127.0.0.1:{port}", compression=None, max_size=None) as ws:
                metadata = S.unpack(await ws.recv())
                assert metadata["model_type"] == "pi05" and metadata["action_dim"] == 7
                replies = []
                for seed in (0, 1):
                    await ws.send(S.pack(_observation(seed)))
                    replies.append(S.unpack(await ws.recv()))
                assert set(replies[0]) == {"actions", "policy_timing", "server_timing"}
                assert replies[0]["actions"].shape == (4, 7) and replies[0]["actions"].dtype == np.float32
                assert "prev_total_ms" not in replies[0]["server_timing"] and "prev_total_ms" in replies[1]["server_timing"]
                assert set(replies[0]["policy_timing"]) == {"infer_ms", "policy_ms"}
                # what came over the wire is what the policy computes in process
                policy.noise.reset()
                assert np.array_equal(replies[0]["actions"], policy.infer(_observation(0))["actions"])
                # a text frame is a protocol error: traceback as text, then close 1011
                await ws.send("not msgpack")
                text = await ws.recv()
                assert isinstance(text, str) and "binary MessagePack frames" in text
                with pytest.raises(websockets.ConnectionClosed) as closed:
                    await ws.recv()
                assert closed.value.rcvd.code == 1011
        finally:
            task.cancel()
            try:
                await task
            except asyncio.CancelledError:
                pass

    asyncio.run(scenario())
