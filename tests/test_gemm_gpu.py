"""tcgen05 GEMM family through the C ABI (pi05_gemm) against an fp32 CPU reference.

Integer (s8 x s8 -> s32) results must be bit-exact; floating-point results are
compared after the same rounding points the epilogue applies.
"""
import math

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


def make_operand(rows, k, op, gen, scale=1.0):
    L, _ = _lib()
    if op == L.OP_BF16:
        t = (torch.randn(rows, k, generator=gen) * scale).to(torch.bfloat16)
        return t, t.float()
    if op == L.OP_E4M3:
        t = (torch.randn(rows, k, generator=gen) * scale * 4).clamp(-448, 448).to(torch.float8_e4m3fn)
        return t, t.float()
    t = torch.randint(-128, 128, (rows, k), generator=gen, dtype=torch.int8)
    return t, t.float()


def check_close(got, want, atol, rtol, what):
    got = got.float().cpu()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{what}: {bad} mismatches, max err {err.max().item():.5f}, max ref {want.abs().max().item():.3f}"


SHAPES_NORMAL = [
    # (M, N, K, block_n)
    (128, 128, 64, 128),
    (256, 256, 256, 128),
    (522, 1152, 592, 128),
    (522, 2560, 2048, 64),
    (300, 512, 4304, 256),
    (130, 72, 256, 128),
    (522, 4304, 1152, 0),
]


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("shape", SHAPES_NORMAL)
def test_gemm_raw_accumulator(op, shape):
    L, K = _lib()
    M, N, Kd, bn = shape
    gen = torch.Generator().manual_seed(1000 + M + N + Kd + op)
    a, af = make_operand(M, Kd, op, gen)
    b, bf = make_operand(N, Kd, op, gen)
    want = af.double() @ bf.double().t()
    ad, bd = a.cuda(), b.cuda()
    if op == L.OP_S8:
        out = torch.full((M, N), -7, dtype=torch.int32, device="cuda")
        st = K.gemm(ad, bd, out, op=op, out_type=L.OUT_S32, force_swap=0, force_block_n=bn)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert torch.equal(out.cpu().double(), want), "s32 accumulators must be bit-exact"
    else:
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        st = K.gemm(ad, bd, out, op=op, out_type=L.OUT_F32, force_swap=0, force_block_n=bn)
        torch.cuda.synchronize()
        assert st.item() == 0
        scale = math.sqrt(Kd) * (16 if op == L.OP_E4M3 else 1)
        check_close(out, want.float(), 2e-3 * scale, 1e-3, f"raw {shape}")


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("shape", [(10, 2560, 1024, 16), (10, 1024, 4096, 16), (1, 3072, 1024, 16),
                                   (50, 8192, 1024, 64), (21, 1024, 2048, 32), (10, 32, 1024, 16),
                                   (10, 1024, 32, 16)])
def test_gemm_swapped_skinny(op, shape):
    L, K = _lib()
    M, N, Kd, bn = shape
    gen = torch.Generator().manual_seed(2000 + M + N + Kd + op)
    a, af = make_operand(M, Kd, op, gen)
    b, bf = make_operand(N, Kd, op, gen)
    want = af.double() @ bf.double().t()
    if op == L.OP_S8:
        out = torch.full((M, N), -7, dtype=torch.int32, device="cuda")
        st = K.gemm(a.cuda(), b.cuda(), out, op=op, out_type=L.OUT_S32, force_swap=1, force_block_n=bn)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert torch.equal(out.cpu().double(), want)
    else:
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        st = K.gemm(a.cuda(), b.cuda(), out, op=op, out_type=L.OUT_F32, force_swap=1, force_block_n=bn)
        torch.cuda.synchronize()
        assert st.item() == 0
        scale = math.sqrt(Kd) * (16 if op == L.OP_E4M3 else 1)
        check_close(out, want.float(), 2e-3 * scale, 1e-3, f"swap {shape}")


def test_gemm_batched_strided_views():
    """Per-(view, head) attention logits out of a packed QKV buffer, as the vision tower uses."""
    L, K = _lib()
    views, heads, tokens, hd = 2, 4, 256, 72
    width = heads * hd
    gen = torch.Generator().manual_seed(7)
    qkv = (torch.randn(views * tokens, 3 * width, generator=gen)).to(torch.bfloat16)
    qkvd = qkv.cuda()
    q4 = qkvd.view(views, tokens, 3, heads, hd)
    qv = q4[:, :, 0].permute(0, 2, 1, 3)  # [views, heads, tokens, hd] strided view
    kv = q4[:, :, 1].permute(0, 2, 1, 3)
    out = torch.zeros(views, heads, tokens, tokens, dtype=torch.bfloat16, device="cuda")
    alpha = 1.0 / math.sqrt(hd)
    st = K.gemm(qv, kv, out, op=L.OP_BF16, alpha=alpha)
    torch.cuda.synchronize()
    assert st.item() == 0
    qf = qkv.float().view(views, tokens, 3, heads, hd)
    want = torch.einsum("vthd,vshd->vhts", qf[:, :, 0], qf[:, :, 1]) * alpha
    check_close(out, rb(want), 2e-2, 1e-2, "batched logits")


@pytest.mark.parametrize("block_n", [128, 256])
def test_gemm_mn_major_b(block_n):
    """P[M, keys] . V[keys, d] with V left row-major (MN-major B operand)."""
    L, K = _lib()
    M, keys, d = 200, 532, 256 if block_n == 256 else 72
    gen = torch.Generator().manual_seed(11)
    ld = 536
    p = torch.zeros(M, ld, dtype=torch.bfloat16)
    p[:, :keys] = torch.rand(M, keys, generator=gen).to(torch.bfloat16)
    v = torch.randn(keys, d, generator=gen).to(torch.bfloat16)
    out = torch.zeros(M, d, dtype=torch.float32, device="cuda")
    pd = p.cuda()[:, :keys]
    st = K.gemm(pd, v.cuda(), out, op=L.OP_BF16, out_type=L.OUT_F32, b_mn_major=True,
                force_block_n=block_n)
    torch.cuda.synchronize()
    assert st.item() == 0
    want = p[:, :keys].float() @ v.float()
    check_close(out, want, 2e-2, 1e-3, "mn-major")


def _epilogue_reference(mode, v, bias, residual, pos, gate, L):
    M, N = v.shape
    if mode == L.EPI_STORE:
        o = rb(v)
        if bias is not None:
            o = rb(o + bias)
        return o
    if mode == L.EPI_BIAS_GELU:
        return gelu_tanh(rb(v) + bias)
    if mode == L.EPI_BIAS_SILU:
        x = rb(v) + bias
        return x / (1.0 + torch.exp(-x))
    if mode == L.EPI_BIAS_RESIDUAL:
        return rb(v) + residual + bias
    if mode == L.EPI_BIAS_POS:
        reps = (M + pos.shape[0] - 1) // pos.shape[0]
        return rb(v) + pos.repeat(reps, 1)[:M] + bias
    if mode == L.EPI_GATE_RESIDUAL:
        return residual + rb(v) * gate
    raise AssertionError(mode)


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("M,swap", [(300, 0), (10, 1), (50, 1)])
@pytest.mark.parametrize("out_type", [0, 1])
def test_gemm_epilogues(mode, M, swap, out_type):
    L, K = _lib()
    N, Kd = 384, 256
    gen = torch.Generator().manual_seed(31 + mode * 7 + M)
    a, af = make_operand(M, Kd, L.OP_BF16, gen)
    b, bf = make_operand(N, Kd, L.OP_BF16, gen, 0.05)
    bias = (torch.randn(N, generator=gen) * 0.1).to(torch.bfloat16)
    residual = torch.randn(M, N, generator=gen).to(torch.bfloat16)
    pos = torch.randn(64, N, generator=gen).to(torch.bfloat16)
    gate = torch.randn(N, generator=gen).to(torch.bfloat16)
    col_scale = torch.rand(N, generator=gen) + 0.5
    v = (af.double() @ bf.double().t()).float() * 0.5 * col_scale
    ref = _epilogue_reference(mode, v, bias.float(), residual.float(), pos.float(), gate.float(), L)
    inv = 8.0
    if out_type == L.OUT_BF16:
        want = rb(ref)
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    else:
        want = (ref * inv).clamp(-448, 448).to(torch.float8_e4m3fn).float()
        out = torch.zeros(M, N, dtype=torch.float8_e4m3fn, device="cuda")
    res_d = residual.cuda()
    if mode in (L.EPI_BIAS_RESIDUAL, L.EPI_GATE_RESIDUAL) and out_type == L.OUT_BF16:
        out.copy_(res_d)  # in-place residual update, as the engine does
        res_arg = out
    else:
        res_arg = res_d
    st = K.gemm(a.cuda(), b.cuda(), out, op=L.OP_BF16, mode=mode, out_type=out_type,
                bias=bias.cuda(), residual=res_arg, pos=pos.cuda(), gate=gate.cuda(),
                col_scale=col_scale.cuda(), alpha=0.5, out_inv_scale=inv, force_swap=swap)
    torch.cuda.synchronize()
    assert st.item() == 0
    got = out.float().cpu()
    # one bf16 / e4m3 ulp of slack for accumulation-order differences
    ulp = want.abs() * (2 ** -7 if out_type == L.OUT_BF16 else 2 ** -2) + (1e-2 if out_type == L.OUT_BF16 else 0.3)
    err = (got - want).abs()
    frac_exact = (err == 0).float().mean().item()
    assert (err <= ulp).all(), f"mode {mode}: max err {err.max().item()}"
    assert frac_exact > 0.97, f"mode {mode}: only {frac_exact:.3f} bit-identical"


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("M,swap,bn", [(300, 0, 128), (300, 0, 256), (10, 1, 16), (50, 1, 64)])
def test_gemm_geglu(op, M, swap, bn):
    """gate|up interleaved in blocks of 64 weight rows; out = gelu(rb(g)) * rb(u)."""
    L, K = _lib()
    inner, Kd = 512, 256
    gen = torch.Generator().manual_seed(77 + op + M)
    a, af = make_operand(M, Kd, op, gen, 0.5 if op != L.OP_S8 else 1.0)
    wg, wgf = make_operand(inner, Kd, op, gen, 0.05 if op != L.OP_S8 else 1.0)
    wu, wuf = make_operand(inner, Kd, op, gen, 0.05 if op != L.OP_S8 else 1.0)
    packed = torch.empty(2 * inner, Kd, dtype=wg.dtype)
    pv = packed.view(inner // 64, 2, 64, Kd)
    pv[:, 0] = wg.view(inner // 64, 64, Kd)
    pv[:, 1] = wu.view(inner // 64, 64, Kd)
    alpha = {0: 1.0, 1: 1.0 / 16, 2: 1e-3}[op]
    g = rb((af.double() @ wgf.double().t()).float() * alpha)
    u = rb((af.double() @ wuf.double().t()).float() * alpha)
    want = rb(gelu_tanh(g) * u)
    out = torch.zeros(M, inner, dtype=torch.bfloat16, device="cuda")
    st = K.gemm(a.cuda(), packed.cuda(), out, op=op, mode=L.EPI_GEGLU, alpha=alpha,
                force_swap=swap, force_block_n=bn)
    torch.cuda.synchronize()
    assert st.item() == 0
    got = out.float().cpu()
    err = (got - want).abs()
    assert (err <= want.abs() * 2 ** -6 + 2e-2).all(), f"max err {err.max().item()}"
    assert (err == 0).float().mean().item() > 0.95


def test_gemm_rejects_bad_arguments():
    L, K = _lib()
    from apxinf_b200 import Pi05Error
    a = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(16, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Pi05Error):  # leading dimension not a multiple of 16 bytes
        K.gemm(a[:, :60][:, :60].contiguous()[:, :52], a[:, :52], out, op=L.OP_BF16)
    with pytest.raises(Pi05Error):  # s32 output only for int8 operands
        K.gemm(a, a, out, op=L.OP_BF16, out_type=L.OUT_S32)


def _scratch():
    partials = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    counters = torch.zeros(1024, dtype=torch.int32, device="cuda")
    return partials, counters


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("M,N,Kd,swap,split", [(10, 1024, 4096, 1, 0), (10, 1024, 4096, 1, 7),
                                                (50, 2560, 1024, 1, 0), (300, 256, 8192, 0, 5),
                                                (522, 384, 4096, 0, 0)])
def test_gemm_split_k_matches_single_pass(op, M, N, Kd, swap, split):
    """K range spread over several CTAs, partial tiles summed in split order by the last
    arrival; two calls in a row share the scratch (the arrival counters return to zero)."""
    L, K = _lib()
    gen = torch.Generator().manual_seed(4000 + M + N + Kd + op)
    if op == L.OP_S8:
        a = torch.randint(-8, 9, (M, Kd), generator=gen, dtype=torch.int8)
        b = torch.randint(-8, 9, (N, Kd), generator=gen, dtype=torch.int8)
        af, bf = a.float(), b.float()
    else:
        a, af = make_operand(M, Kd, op, gen)
        b, bf = make_operand(N, Kd, op, gen)
    want = (af.double() @ bf.double().t()).float()
    partials, counters = _scratch()
    ad, bd = a.cuda(), b.cuda()
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        st = K.gemm(ad, bd, out, op=op, out_type=L.OUT_F32, force_swap=swap, partials=partials,
                    tile_counters=counters, force_split_k=split)
        torch.cuda.synchronize()
        assert st.item() == 0
        assert int(counters.abs().sum().item()) == 0
        if op == L.OP_S8:
            assert torch.equal(out.cpu(), want), "integer partial sums must be exact"
        else:
            scale = math.sqrt(Kd) * (16 if op == L.OP_E4M3 else 1)
            check_close(out, want, 2e-3 * scale, 1e-3, "split-k")


@pytest.mark.parametrize("mode", [0, 3, 5])
def test_gemm_split_k_epilogues(mode):
    L, K = _lib()
    M, N, Kd = 10, 384, 2048
    gen = torch.Generator().manual_seed(91 + mode)
    a, af = make_operand(M, Kd, L.OP_BF16, gen)
    b, bf = make_operand(N, Kd, L.OP_BF16, gen, 0.05)
    bias = (torch.randn(N, generator=gen) * 0.1).to(torch.bfloat16)
    residual = torch.randn(M, N, generator=gen).to(torch.bfloat16)
    gate = torch.randn(N, generator=gen).to(torch.bfloat16)
    v = (af.double() @ bf.double().t()).float()
    ref = _epilogue_reference(mode, v, bias.float(), residual.float(), None, gate.float(), L)
    want = rb(ref)
    partials, counters = _scratch()
    out = residual.cuda().clone()
    st = K.gemm(a.cuda(), b.cuda(), out, op=L.OP_BF16, mode=mode, bias=bias.cuda(), residual=out,
                gate=gate.cuda(), partials=partials, tile_counters=counters, force_split_k=4)
    torch.cuda.synchronize()
    assert st.item() == 0
    err = (out.float().cpu() - want).abs()
    assert (err <= want.abs() * 2 ** -7 + 1e-2).all(), err.max().item()
    assert (err == 0).float().mean().item() > 0.95


@pytest.mark.parametrize("M,swap", [(10, 1), (300, 0)])
def test_gemm_split_k_geglu(M, swap):
    L, K = _lib()
    inner, Kd = 256, 2048
    gen = torch.Generator().manual_seed(55 + M)
    a, af = make_operand(M, Kd, L.OP_BF16, gen, 0.5)
    wg, wgf = make_operand(inner, Kd, L.OP_BF16, gen, 0.05)
    wu, wuf = make_operand(inner, Kd, L.OP_BF16, gen, 0.05)
    packed = torch.empty(2 * inner, Kd, dtype=wg.dtype)
    pv = packed.view(inner // 64, 2, 64, Kd)
    pv[:, 0] = wg.view(inner // 64, 64, Kd)
    pv[:, 1] = wu.view(inner // 64, 64, Kd)
    g = rb((af.double() @ wgf.double().t()).float())
    u = rb((af.double() @ wuf.double().t()).float())
    want = rb(gelu_tanh(g) * u)
    partials, counters = _scratch()
    out = torch.zeros(M, inner, dtype=torch.bfloat16, device="cuda")
    st = K.gemm(a.cuda(), packed.cuda(), out, op=L.OP_BF16, mode=L.EPI_GEGLU, force_swap=swap,
                partials=partials, tile_counters=counters, force_split_k=4)
    torch.cuda.synchronize()
    assert st.item() == 0
    err = (out.float().cpu() - want).abs()
    assert (err <= want.abs() * 2 ** -6 + 2e-2).all(), err.max().item()


@pytest.mark.parametrize("M,N,Kd,batch", [(2560, 2048, 16384, 1), (2000, 1152, 32768, 1), (700, 640, 256, 3)])
def test_persistent_kernel_raster_groups_cover_every_tile(M, N, Kd, batch):
    """More tiles than SMs: the persistent kernel walks row tiles in groups sized to L2 (with
    the long K ranges here the groups are 8 to 12 row tiles, the last one ragged); INT8
    accumulators are exact, so a tile visited twice, skipped or swapped shows up."""
    L, K = _lib()
    gen = torch.Generator().manual_seed(M + N)
    a = torch.randint(-8, 9, (batch, M, Kd), generator=gen, dtype=torch.int8)
    b = torch.randint(-8, 9, (batch, N, Kd), generator=gen, dtype=torch.int8)
    ad, bd = a.cuda(), b.cuda()
    out = torch.full((batch, M, N), -7, dtype=torch.int32, device="cuda")
    st = K.gemm(ad, bd, out, op=L.OP_S8, out_type=L.OUT_S32)
    torch.cuda.synchronize()
    assert st.item() == 0
    want = torch.matmul(ad.float(), bd.float().transpose(1, 2)).round().to(torch.int32)  # exact: |sum| < 2^24
    assert torch.equal(out, want)


def _tuning(name, value):
    from apxinf_b200._lib import lib
    assert lib().pi05_set_tuning(name.encode(), int(value)) == 0


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("mode", [0, 1, 3, 5, 6])
@pytest.mark.parametrize("M,N,Kd", [(300, 200, 320), (522, 1152, 1152), (2600, 1536, 256)])
def test_single_epilogue_kernels_give_the_general_kernel_bits(op, mode, M, N, Kd):
    """Launches that fit a kernel compiled for one epilogue and output type (the default plan)
    against the general kernel planned for the same call: the same arithmetic, so the same
    bits. Covers one wave of tiles with ragged edges, the B=1 SigLIP shape and a multi-wave
    shape that runs the persistent kernel; activation outputs (after GELU / GeGLU) in the
    operand's own 8-bit type."""
    L, K = _lib()
    if mode == L.EPI_GEGLU:
        N = (N + 127) // 128 * 128
    gen = torch.Generator().manual_seed(7000 + 13 * op + mode + M)
    a, _ = make_operand(M, Kd, op, gen, 0.5)
    if op == L.OP_S8:
        a = torch.randint(-20, 21, (M, Kd), generator=gen, dtype=torch.int8)
        b = torch.randint(-20, 21, (N, Kd), generator=gen, dtype=torch.int8)
    else:
        b, _ = make_operand(N, Kd, op, gen, 0.05)
    n_out = N // 2 if mode == L.EPI_GEGLU else N
    bias = (torch.randn(N, generator=gen) * 0.1).to(torch.bfloat16).cuda()
    gate = torch.randn(N, generator=gen).to(torch.bfloat16).cuda()
    residual = torch.randn(M, n_out, generator=gen).to(torch.bfloat16)
    col_scale = (torch.rand(N, generator=gen) * 0.01 + 0.001).cuda()
    activation = mode in (L.EPI_BIAS_GELU, L.EPI_GEGLU)
    if activation and op == L.OP_E4M3:
        out_type, dtype = L.OUT_E4M3, torch.uint8
    elif activation and op == L.OP_S8:
        out_type, dtype = L.OUT_S8, torch.int8
    else:
        out_type, dtype = L.OUT_BF16, torch.bfloat16
    ad, bd = a.cuda(), b.cuda()

    def run():
        if dtype == torch.bfloat16:
            out = residual.cuda().clone()
        else:
            out = torch.zeros(M, n_out, dtype=dtype, device="cuda")
        st = K.gemm(ad, bd, out, op=op, mode=mode, out_type=out_type, bias=None if mode == L.EPI_GEGLU else bias,
                    residual=out if mode in (L.EPI_BIAS_RESIDUAL, L.EPI_GATE_RESIDUAL) else None,
                    gate=gate if mode == L.EPI_GATE_RESIDUAL else None, col_scale=col_scale,
                    alpha=0.5, out_inv_scale=8.0, force_swap=0)
        torch.cuda.synchronize()
        assert st.item() == 0
        return out.cpu()

    single = run()
    _tuning("single_epilogue_kernels", 0)
    try:
        general = run()
    finally:
        _tuning("single_epilogue_kernels", 1)
    assert torch.equal(single.view(torch.uint8), general.view(torch.uint8))
    assert single.view(torch.uint8).float().std().item() > 0  # not all one value


@pytest.mark.parametrize("op", [0, 1, 2])
@pytest.mark.parametrize("M,N,Kd,slices", [(522, 2048, 16384, 3), (300, 256, 1001 * 16, 4), (130, 200, 2048, 2),
                                           (128, 128, 640, 3)])
def test_gemm_k_slices_are_partial_products(op, M, N, Kd, slices):
    """The K range of one GEMM as a batch of K-block runs, each writing its own fp32 product:
    their sum is the whole product. Uneven runs (the last one shorter, or reaching past K, where
    the operands read as zero) and a K that is no multiple of the K block are included."""
    L, K = _lib()
    if op != L.OP_BF16:
        Kd = (Kd + 15) // 16 * 16
    gen = torch.Generator().manual_seed(8100 + M + N + op)
    if op == L.OP_S8:
        a = torch.randint(-8, 9, (M, Kd), generator=gen, dtype=torch.int8)
        b = torch.randint(-8, 9, (N, Kd), generator=gen, dtype=torch.int8)
        af, bf = a.float(), b.float()
    else:
        a, af = make_operand(M, Kd, op, gen)
        b, bf = make_operand(N, Kd, op, gen, 0.05)
    want = (af.double() @ bf.double().t())
    out = torch.full((slices, M, N), float("nan"), dtype=torch.float32, device="cuda")
    st = K.gemm(a.cuda(), b.cuda(), out, op=op, out_type=L.OUT_F32, force_swap=0, k_slices=slices)
    torch.cuda.synchronize()
    assert st.item() == 0
    parts = out.cpu().double()
    assert torch.isfinite(parts).all()
    block = 128 if op != L.OP_BF16 else 64
    run = -(-(-(-Kd // block)) // slices) * block  # K elements per run
    for s in range(slices):
        lo, hi = min(Kd, s * run), min(Kd, (s + 1) * run)
        part = af[:, lo:hi].double() @ bf[:, lo:hi].double().t()
        scale = math.sqrt(max(hi - lo, 1)) * (16 if op == L.OP_E4M3 else 1) * 0.05
        if op == L.OP_S8:
            assert torch.equal(parts[s], part), f"run {s}"
        else:
            check_close(parts[s].float(), part.float(), 2e-3 * scale, 1e-3, f"run {s}")
    if op == L.OP_S8:
        assert torch.equal(parts.sum(0), want)
