"""The serving shell over the real model: the policy's action chunk is the unnormalised, trimmed
output of `apxinf_py.Model.infer_rgb` on the inputs its pre chain built (the layering check of
python/apxinf/tests/test_policy_layering.py), in process and over the websocket."""
import asyncio

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    from apxinf_b200 import apxinf_py
    m = apxinf_py.Model.random("pi05", device="cuda:0", precision="fp8", calibration="uniform:0.05", seed=3)
    yield m
    m.close()


def _observation(seed):
    rng = np.random.default_rng(seed)
    return {"observation/image": rng.integers(0, 256, (256, 320, 3), dtype=np.uint8),
            "observation/wrist_image": rng.integers(0, 256, (224, 224, 3), dtype=np.uint8),
            "prompt": "pick_up the block"}


def test_policy_over_the_engine(model):
    from apxinf_b200 import serving as S
    policy = S.Pi05Policy.from_random(model, token_count=10, action_dim=7, seed=4, warn=False)
    result = policy.infer(_observation(0))
    assert result["actions"].shape == (model.action_horizon, 7) and np.isfinite(result["actions"]).all()
    rgb = np.stack([S.resize_with_pad(S.parse_image(_observation(0)["observation/image"]), model.image_size),
                    _observation(0)["observation/wrist_image"]])
    direct = model.infer_rgb(np.ascontiguousarray(rgb), "nhwc", result["token_ids"], result["noise"])
    assert np.array_equal(result["normalized_actions"], direct)
    assert np.allclose(result["actions"], direct[:, :7], atol=1e-6)  # identity statistics
    assert result["timing"]["model_ms"] < 1000


def test_websocket_round_trip_on_the_gpu(model):
    websockets = pytest.importorskip("websockets")
    from apxinf_b200 import serving as S
    policy = S.Pi05Policy.from_random(model, token_count=10, seed=6, warn=False)
    server = S.WebsocketPolicyServer(policy, "127.0.0.1", 0)

    async def scenario():
        started = asyncio.Event()
        task = asyncio.create_task(server.run(started))
        await asyncio.wait_for(started.wait(), 30)
        try:
            async with websockets.connect(f"ws://127.0.0.1:{server.bound_port}", compression=None, max_size=None) as ws:
                metadata = S.unpack(await ws.recv())
                assert metadata["num_views"] == 2 and metadata["action_horizon"] == model.action_horizon
                times = []
                for seed in range(3):
                    await ws.send(S.pack(_observation(seed)))
                    reply = S.unpack(await ws.recv())
                    assert reply["actions"].shape == (model.action_horizon, model.action_dim)
                    assert np.isfinite(reply["actions"]).all()
                    times.append(reply["policy_timing"]["infer_ms"])
                assert min(times) < 100  # the model call itself is about 10 ms once the plan exists
        finally:
            task.cancel()
            try:
                await task
            except asyncio.CancelledError:
                pass

    asyncio.run(scenario())
