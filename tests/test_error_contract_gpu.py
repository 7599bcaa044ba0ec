"""The device-timeout contract: a bounded barrier wait that runs out makes the kernel record its
status word, release its TMEM and return; the host call reports PI05_ERR_DEVICE_TIMEOUT and the
context stays usable. The wait is made to run out without any fault: the first CTA announces one
operand load (expect_tx) and never issues it, so the stage's barrier simply never completes,
under a small poll budget ("drop_one_load" / "wait_limit_polls" of pi05_set_tuning)."""
import numpy as np
import pytest

from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _tuning(name, value):
    from apxinf_b200._lib import check, lib
    check(lib().pi05_set_tuning(name.encode(), int(value)), f"pi05_set_tuning({name})")


@pytest.fixture()
def dropped_load():
    _tuning("wait_limit_polls", 1 << 14)
    _tuning("drop_one_load", 0)
    yield
    _tuning("drop_one_load", -1)
    _tuning("wait_limit_polls", 0)


def _problem():
    g = torch.Generator(device="cpu").manual_seed(5)
    a = (torch.randn(256, 512, generator=g) * 0.5).to(torch.bfloat16).cuda()
    b = (torch.randn(384, 512, generator=g) * 0.5).to(torch.bfloat16).cuda()
    return a, b, a.float() @ b.float().t()


def test_gemm_wait_runs_out_and_the_next_call_succeeds(dropped_load):
    from apxinf_b200 import _lib, kernels
    a, b, want = _problem()
    out = torch.zeros(256, 384, dtype=torch.bfloat16, device="cuda")
    status = kernels.gemm(a, b, out, op=_lib.OP_BF16)
    torch.cuda.synchronize()  # returns: nothing trapped, nothing hung
    assert status.item() != 0
    # only the first CTA's tile was abandoned; the others finished
    got = out.float()
    assert torch.allclose(got[128:], want[128:], rtol=2e-2, atol=2e-2)
    # the same context, the same problem, without the dropped load
    _tuning("drop_one_load", -1)
    out2 = torch.zeros_like(out)
    status2 = kernels.gemm(a, b, out2, op=_lib.OP_BF16)
    torch.cuda.synchronize()
    assert status2.item() == 0
    assert torch.allclose(out2.float(), want, rtol=2e-2, atol=2e-2)


def test_graph_reports_device_timeout_and_recovers(dropped_load):
    from apxinf_b200.engine import Pi05Runtime
    cfg = O.tiny_config()
    rt = Pi05Runtime.random(cfg, dtype="bf16", seed=3, device=0)
    images, tokens, noise = O.synthetic_observation(cfg, 100, 6)
    batch = (images[None], tokens[None], noise[None])
    # capture runs the launch list once itself: the plan is built with the dropped load baked in
    with pytest.raises(RuntimeError, match="PI05_ERR_DEVICE_TIMEOUT"):
        g = rt.capture_infer_rgb_u8(6, "nhwc", 1)
        g.infer_host(*batch)
    _tuning("drop_one_load", -1)
    _tuning("wait_limit_polls", 0)
    # the engine, its stream and its status word are still good for a new plan
    good = rt.capture_infer_rgb_u8(6, "nhwc", 1)
    got = good.infer_host(*batch)[0]
    want = O.infer(cfg, 3, images, tokens, noise, dtype="bf16", vision_round_scores=True)
    m = O.compare(got, want)
    assert m["cosine"] >= 0.999 and m["max_abs"] <= 2e-2, m
    good.close()
    rt.close()
