"""The at-most-16-row GEMM kernel (weights streamed through registers, producer fused into the
activation staging, paired-tile epilogues) through pi05_gemm, against float64 / the same
rounding points, and against the kernels it replaces (norm + GEMM, GEMM + RoPE kernel)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from apxinf_b200 import _lib as L, kernels as K
    return L, K


def rb(x):
    return x.to(torch.bfloat16).to(torch.float32)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def operand(rows, k, op, gen, scale=1.0):
    L, _ = _lib()
    if op == L.OP_BF16:
        t = (torch.randn(rows, k, generator=gen) * scale).to(torch.bfloat16)
    elif op == L.OP_E4M3:
        t = (torch.randn(rows, k, generator=gen) * scale * 4).clamp(-448, 448).to(torch.float8_e4m3fn)
    else:
        t = torch.randint(-128, 128, (rows, k), generator=gen, dtype=torch.int8)
    return t, t.float()


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("M,N,Kd", [(10, 2560, 1024), (10, 1024, 4096), (1, 3072, 1024), (16, 1024, 2048),
                                     (10, 1024, 32), (10, 32, 1024), (7, 72, 48), (3, 8, 16)])
def test_raw_accumulators(op, M, N, Kd):
    L, K = _lib()
    gen = torch.Generator().manual_seed(M * 7 + N + Kd + op)
    a, af = operand(M, Kd, op, gen)
    b, bf = operand(N, Kd, op, gen)
    want = af.double() @ bf.double().t()
    if op == L.OP_S8:
        out = torch.full((M, N), -7, dtype=torch.int32, device="cuda")
        st = K.gemm(a.cuda(), b.cuda(), out, op=op, out_type=L.OUT_S32, force_skinny=1)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert torch.equal(out.cpu().double(), want), "s32 accumulators must be bit-exact"
    else:
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        K.gemm(a.cuda(), b.cuda(), out, op=op, out_type=L.OUT_F32, force_skinny=1)
        torch.cuda.synchronize()
        scale = math.sqrt(Kd) * (16 if op == L.OP_E4M3 else 1)
        err = (out.cpu().double() - want).abs().max().item()
        assert err <= 2e-5 * scale * (4 if op == L.OP_E4M3 else 1) + 1e-6 * want.abs().max().item(), err


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 5])
@pytest.mark.parametrize("out_type", [0, 1, 4])
def test_epilogues_match_the_tcgen05_kernel(mode, out_type):
    """Same rounding points as the swapped tcgen05 kernel: outputs agree up to accumulation
    order (one step of the output type on a few elements)."""
    L, K = _lib()
    M, N, Kd = 10, 1024, 2048
    gen = torch.Generator().manual_seed(50 + mode)
    a, _ = operand(M, Kd, L.OP_E4M3, gen, 0.25)
    b, _ = operand(N, Kd, L.OP_E4M3, gen, 0.25)
    bias = (torch.randn(N, generator=gen) * 0.1).to(torch.bfloat16).cuda()
    gate = (torch.randn(N, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    residual = torch.randn(M, N, generator=gen).to(torch.bfloat16).cuda()
    scale = (torch.rand(N, generator=gen) * 0.02 + 0.01).cuda()
    dtype = {0: torch.bfloat16, 1: torch.float8_e4m3fn, 4: torch.int8}[out_type]
    kwargs = dict(op=L.OP_E4M3, mode=mode, out_type=out_type, bias=bias, gate=gate if mode == 5 else None,
                  residual=residual if mode in (3, 5) else None, col_scale=scale, alpha=0.05,
                  out_inv_scale=8.0)
    outs = []
    for skinny in (1, 0):
        out = torch.zeros(M, N, dtype=dtype, device="cuda")
        st = K.gemm(a.cuda(), b.cuda(), out, force_skinny=skinny, force_swap=-1 if skinny else 1, **kwargs)
        torch.cuda.synchronize()
        assert st.item() == 0
        outs.append(out.float().cpu())
    diff = (outs[0] - outs[1]).abs()
    assert (diff > 0).float().mean().item() < 0.02
    assert diff.max().item() <= (0.02 if out_type == 0 else 1.0 if out_type == 4 else 0.13) * max(1.0, outs[1].abs().max().item())


@pytest.mark.parametrize("op", [0, 1, 2])
def test_geglu_pairs_gate_and_up_rows(op):
    L, K = _lib()
    M, inner, Kd = 10, 512, 1024
    gen = torch.Generator().manual_seed(3 + op)
    a, af = operand(M, Kd, op, gen, 0.5)
    gate_w, gf = operand(inner, Kd, op, gen, 0.5)
    up_w, uf = operand(inner, Kd, op, gen, 0.5)
    packed = torch.stack([gate_w.view(torch.uint8).view(inner // 64, 64, -1),
                          up_w.view(torch.uint8).view(inner // 64, 64, -1)], dim=1).reshape(2 * inner, -1)
    packed = packed.view(gate_w.dtype)
    alpha = {0: 1.0, 1: 1.0 / 64, 2: 1e-3}[op]
    out = torch.zeros(M, inner, dtype=torch.bfloat16, device="cuda")
    st = K.gemm(a.cuda(), packed.cuda(), out, op=op, mode=L.EPI_GEGLU, alpha=alpha, force_skinny=1)
    torch.cuda.synchronize()
    assert st.item() == 0
    g = rb(((af.double() @ gf.double().t()) * alpha).float())
    u = rb(((af.double() @ uf.double().t()) * alpha).float())
    want = gelu_tanh(g) * u
    err = (out.float().cpu() - want).abs()
    assert (err <= 0.02 + 0.02 * want.abs()).all(), err.max().item()


@pytest.mark.parametrize("op,dynamic", [(0, False), (1, False), (2, False), (2, True)])
def test_adaptive_norm_prologue_equals_norm_kernel_then_gemm(op, dynamic):
    """adaRMSNorm fused into the activation staging against the separate norm launch of this
    library (apxinf_static_ada_rms_norm_bf16 for the bf16 case; the oracle formula otherwise)."""
    from oracle import pi05_oracle as O
    L, K = _lib()
    M, N, Kd = 10, 512, 1024
    gen = torch.Generator().manual_seed(21 + op)
    hidden = (torch.randn(M, Kd, generator=gen) * 2).to(torch.bfloat16)
    style = (torch.randn(3 * Kd, generator=gen) * 0.3).to(torch.bfloat16)
    w, wf = operand(N, Kd, op, gen, 0.5)
    x = hidden.float().numpy()
    oracle = O.Pi05Oracle(O.Pi05Config(), None, O.OracleOptions())
    normed = oracle.ada_rms_norm(x, style.float().numpy())
    act_scale = 0.05
    if op == L.OP_BF16:
        staged, alpha = O.round_bf16(normed), 1.0
        row = np.ones(M, np.float32)
    elif op == L.OP_E4M3:
        staged, alpha = O.quantize_e4m3_static(normed, act_scale), act_scale
        row = np.ones(M, np.float32)
    elif dynamic:
        staged, row = O.quantize_rows_int8(O.round_bf16(normed))
        alpha = 1.0
    else:
        staged, alpha = O.quantize_int8_static(O.round_bf16(normed), act_scale), act_scale
        row = np.ones(M, np.float32)
    want = (staged.astype(np.float64) @ wf.double().numpy().T) * alpha * row[:, None] * 1e-2
    out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    st = K.gemm(hidden.cuda(), w.cuda(), out, op=op, out_type=L.OUT_F32, alpha=alpha * 1e-2, force_skinny=1,
                prologue=L.PRO_ADA_NORM, style=style.cuda(), eps=1e-6, a_inv_scale=1.0 / act_scale,
                a_dynamic_rows=dynamic)
    torch.cuda.synchronize()
    assert st.item() == 0
    got = out.cpu().double().numpy()
    # a normalised value next to a rounding boundary of the operand type may take the other code
    # (rsqrtf and the reduction order differ from NumPy): bounded by a few operand steps per row
    err = np.abs(got - want)
    assert np.median(err) <= 1e-3 * np.abs(want).max() and err.max() <= 0.05 * np.abs(want).max(), (np.median(err), err.max())


def test_rope_epilogue_equals_gemm_then_rope_kernel():
    """q|k|v projection with the RoPE + KV-cache write in the epilogue against the projection
    followed by this library's apxinf_static_qkv_rope_bf16."""
    import ctypes as C
    from apxinf_b200 import lib
    L, K = _lib()
    tokens, heads, hd, Kd, offset, cache_rows = 10, 8, 256, 1024, 522, 532
    N = (heads + 2) * hd
    gen = torch.Generator().manual_seed(77)
    a, _ = operand(tokens, Kd, L.OP_E4M3, gen, 0.25)
    w, _ = operand(N, Kd, L.OP_E4M3, gen, 0.25)
    scale = (torch.rand(N, generator=gen) * 0.02 + 0.01).cuda()
    positions = torch.arange(offset + tokens, dtype=torch.float32)
    pair = torch.arange(hd // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -pair / (hd // 2)).float()
    angle = (positions[:, None] * freq[None, :]).double()
    cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    q_fused = torch.zeros(tokens, heads, hd, dtype=torch.bfloat16, device="cuda")
    k_fused = torch.zeros(cache_rows, hd, dtype=torch.bfloat16, device="cuda")
    v_fused = torch.zeros(cache_rows, hd, dtype=torch.bfloat16, device="cuda")
    dummy = torch.zeros(tokens, N, dtype=torch.bfloat16, device="cuda")
    st = K.gemm(a.cuda(), w.cuda(), dummy, op=L.OP_E4M3, mode=L.EPI_ROPE, col_scale=scale, alpha=0.05,
                force_skinny=1, rope=dict(q_out=q_fused, k_cache=k_fused, v_cache=v_fused, cos=cos, sin=sin,
                                          tokens=tokens, q_heads=heads, head_dim=hd, position_offset=offset,
                                          cache_rows=cache_rows))
    torch.cuda.synchronize()
    assert st.item() == 0
    qkv = torch.zeros(tokens, N, dtype=torch.bfloat16, device="cuda")
    K.gemm(a.cuda(), w.cuda(), qkv, op=L.OP_E4M3, col_scale=scale, alpha=0.05, force_skinny=1)
    q_ref = torch.zeros_like(q_fused)
    k_ref = torch.zeros_like(k_fused)
    v_ref = torch.zeros_like(v_fused)
    rc = lib().apxinf_static_qkv_rope_bf16(
        C.c_void_p(qkv.data_ptr()), None, C.c_void_p(q_ref.data_ptr()), C.c_void_p(k_ref.data_ptr()),
        C.c_void_p(v_ref.data_ptr()), tokens, heads, 1, hd, C.c_float(10000.0), offset, offset,
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.equal(v_fused, v_ref)
    assert not k_fused[:offset].any() and not v_fused[:offset].any()
    for got, want in ((q_fused, q_ref), (k_fused, k_ref)):
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 0.02 * max(1.0, want.float().abs().max().item()), err


def test_euler_epilogue_and_quantize_prologue():
    L, K = _lib()
    M, N, Kd = 10, 32, 1024
    gen = torch.Generator().manual_seed(5)
    a, af = operand(M, Kd, L.OP_BF16, gen)
    w, wf = operand(N, Kd, L.OP_BF16, gen, 0.05)
    bias = (torch.randn(N, generator=gen) * 0.1).to(torch.bfloat16)
    state = torch.randn(M, N, generator=gen).to(torch.bfloat16)
    state_d = state.clone().cuda()
    st = K.gemm(a.cuda(), w.cuda(), state_d, op=L.OP_BF16, mode=L.EPI_EULER, bias=bias.cuda(), residual=state_d,
                dt=-0.1, force_skinny=1)
    torch.cuda.synchronize()
    assert st.item() == 0
    velocity = rb(rb((af.double() @ wf.double().t()).float()) + bias.float())
    want = rb(state.float() + (-0.1) * velocity)
    assert (state_d.float().cpu() - want).abs().max().item() <= 0.02
    # quantise-only prologue: bf16 rows -> e4m3 operand inside the GEMM
    x = torch.randn(M, 32, generator=gen).to(torch.bfloat16)
    w8, w8f = operand(64, 32, L.OP_E4M3, gen, 0.25)
    out = torch.zeros(M, 64, dtype=torch.float32, device="cuda")
    K.gemm(x.cuda(), w8.cuda(), out, op=L.OP_E4M3, out_type=L.OUT_F32, alpha=0.05, force_skinny=1,
           prologue=L.PRO_QUANTIZE, a_inv_scale=20.0)
    torch.cuda.synchronize()
    xq = (x.float() * 20.0).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    want = (xq.double() @ w8f.double().t()) * 0.05
    assert (out.cpu().double() - want).abs().max().item() <= 1e-4 * max(1.0, want.abs().max().item())


def test_more_than_16_rows_is_refused_when_required():
    from apxinf_b200 import Pi05Error
    L, K = _lib()
    a = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(17, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Pi05Error) as info:
        K.gemm(a, b, out, op=L.OP_BF16, force_skinny=1)
    assert info.value.code == -2
