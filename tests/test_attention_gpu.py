"""Fused tcgen05 attention (pi05_attention) against a float64 softmax(QK^T)V on the CPU, for
the three attention shapes of PI0.5 and ragged edge cases. Tolerance: the kernel rounds the
scaled logits and the probabilities to bf16 as the reference's MQA does
(crates/apxinf-cuda/adapters/cublas_adapter.cu:109-130), so outputs agree to ~1 bf16 ulp of
the value scale; the reference's own attention test uses |err| < 0.003 on unit-scale data
(crates/apxinf-cuda/src/tests/fp8.rs:1041-1113)."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


class AttentionArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_ld", C.c_int64), ("q_sb0", C.c_int64), ("q_sb1", C.c_int64),
                ("k", C.c_void_p), ("k_ld", C.c_int64), ("k_sb0", C.c_int64), ("k_sb1", C.c_int64),
                ("v", C.c_void_p), ("v_ld", C.c_int64), ("v_sb0", C.c_int64), ("v_sb1", C.c_int64),
                ("out", C.c_void_p), ("out_ld", C.c_int64), ("out_sb0", C.c_int64), ("out_sb1", C.c_int64),
                ("q_rows", C.c_int32), ("keys", C.c_int32), ("head_dim", C.c_int32),
                ("nb0", C.c_int32), ("nb1", C.c_int32), ("scale", C.c_float),
                ("out_e4m3", C.c_int32), ("out_inv_scale", C.c_float), ("status", C.c_void_p),
                ("key_split", C.c_int32), ("split_scratch", C.c_void_p), ("split_scratch_bytes", C.c_int64)]


def run(q, k, v, out, scale, nb0=1, nb1=1, strides=None, e4m3=False, inv=1.0, key_split=False):
    """q/k/v/out: torch CUDA tensors; strides: dict name -> (ld, sb0, sb1) in elements."""
    from apxinf_b200 import lib
    handle = lib()
    handle.pi05_attention.argtypes = [C.POINTER(AttentionArgs), C.c_void_p]
    handle.pi05_attention.restype = C.c_int
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    s = strides
    args = AttentionArgs(
        q=q.data_ptr(), q_ld=s["q"][0], q_sb0=s["q"][1], q_sb1=s["q"][2],
        k=k.data_ptr(), k_ld=s["k"][0], k_sb0=s["k"][1], k_sb1=s["k"][2],
        v=v.data_ptr(), v_ld=s["v"][0], v_sb0=s["v"][1], v_sb1=s["v"][2],
        out=out.data_ptr(), out_ld=s["o"][0], out_sb0=s["o"][1], out_sb1=s["o"][2],
        q_rows=s["rows"], keys=s["keys"], head_dim=s["hd"], nb0=nb0, nb1=nb1, scale=scale,
        out_e4m3=int(e4m3), out_inv_scale=inv, status=status.data_ptr())
    if key_split:
        scratch = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
        args.key_split, args.split_scratch, args.split_scratch_bytes = 1, scratch.data_ptr(), scratch.numel()
    rc = handle.pi05_attention(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, int(status.item())


def reference(q, k, v, scale):
    s = (q.double() @ k.double().transpose(-1, -2)) * scale
    p = torch.softmax(s, dim=-1)
    return (p @ v.double()).float()


@pytest.mark.parametrize("rows,keys,hd", [(80, 532, 256), (4176, 522, 256), (400, 532, 256),
                                            (10, 37, 128), (130, 1000, 256), (7, 1, 64), (256, 256, 72)])
def test_single_batch_shapes(rows, keys, hd):
    gen = torch.Generator().manual_seed(rows + keys + hd)
    q = torch.randn(rows, hd, generator=gen).to(torch.bfloat16)
    k = torch.randn(keys, hd, generator=gen).to(torch.bfloat16)
    v = torch.randn(keys, hd, generator=gen).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    out = torch.full((rows, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc, status = run(q.cuda(), k.cuda(), v.cuda(), out, scale,
                     strides=dict(q=(hd, 0, 0), k=(hd, 0, 0), v=(hd, 0, 0), o=(hd, 0, 0), rows=rows, keys=keys, hd=hd))
    assert rc == 0 and status == 0
    want = reference(q.float(), k.float(), v.float(), scale)
    err = (out.float().cpu() - want).abs().max().item()
    assert err <= 0.02, err


def test_zero_queries_average_the_values():
    # crates/apxinf-cuda/src/tests/fp8.rs:735-778
    rows, keys, hd = 32, 20, 256
    q = torch.zeros(rows, hd, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(keys, hd, dtype=torch.bfloat16, device="cuda")
    v = torch.arange(keys, dtype=torch.float32)[:, None].repeat(1, hd).to(torch.bfloat16).cuda()
    out = torch.zeros(rows, hd, dtype=torch.bfloat16, device="cuda")
    rc, status = run(q, k, v, out, 1 / 16, strides=dict(q=(hd, 0, 0), k=(hd, 0, 0), v=(hd, 0, 0), o=(hd, 0, 0), rows=rows, keys=keys, hd=hd))
    assert rc == 0 and status == 0
    assert (out.float() - 9.5).abs().max().item() < 0.05


def test_siglip_layout_strided_views_and_e4m3_output():
    """Per (image, head) attention read in place from the packed q|k|v projection."""
    images, heads, tokens, hd = 3, 16, 256, 72
    width = heads * hd
    gen = torch.Generator().manual_seed(3)
    qkv = torch.randn(images * tokens, 3 * width, generator=gen).to(torch.bfloat16)
    d = qkv.cuda()
    out = torch.zeros(images * tokens, width, dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    strides = dict(q=(3 * width, hd, tokens * 3 * width), k=(3 * width, hd, tokens * 3 * width),
                   v=(3 * width, hd, tokens * 3 * width), o=(width, hd, tokens * width),
                   rows=tokens, keys=tokens, hd=hd)
    rc, status = run(d, d[:, width:], d[:, 2 * width:], out, scale, nb0=heads, nb1=images, strides=strides)
    assert rc == 0 and status == 0
    x = qkv.float().view(images, tokens, 3, heads, hd)
    want = reference(x[:, :, 0].permute(0, 2, 1, 3), x[:, :, 1].permute(0, 2, 1, 3),
                     x[:, :, 2].permute(0, 2, 1, 3), scale)  # [images, heads, tokens, hd]
    want = want.permute(0, 2, 1, 3).reshape(images * tokens, width)
    assert (out.float().cpu() - want).abs().max().item() <= 0.02
    out8 = torch.zeros(images * tokens, width, dtype=torch.float8_e4m3fn, device="cuda")
    rc, status = run(d, d[:, width:], d[:, 2 * width:], out8, scale, nb0=heads, nb1=images,
                     strides=strides, e4m3=True, inv=20.0)
    assert rc == 0 and status == 0
    got = out8.float().cpu() / 20.0
    assert (got - want).abs().max().item() <= 0.02 + 0.07 * want.abs().max().item()


def test_batched_mqa_over_a_cache_with_row_stride():
    """Each sample attends over its own [cache_rows, 256] cache of which only `keys` rows count."""
    batch, q_rows, keys, cache_rows, hd = 5, 80, 532, 540, 256
    gen = torch.Generator().manual_seed(8)
    q = torch.randn(batch, q_rows, hd, generator=gen).to(torch.bfloat16)
    kc = torch.randn(batch, cache_rows, hd, generator=gen).to(torch.bfloat16)
    vc = torch.randn(batch, cache_rows, hd, generator=gen).to(torch.bfloat16)
    out = torch.zeros(batch, q_rows, hd, dtype=torch.bfloat16, device="cuda")
    rc, status = run(q.cuda(), kc.cuda(), vc.cuda(), out, 1 / 16, nb0=batch,
                     strides=dict(q=(hd, q_rows * hd, 0), k=(hd, cache_rows * hd, 0), v=(hd, cache_rows * hd, 0),
                                  o=(hd, q_rows * hd, 0), rows=q_rows, keys=keys, hd=hd))
    assert rc == 0 and status == 0
    want = reference(q.float(), kc.float()[:, :keys], vc.float()[:, :keys], 1 / 16)
    assert (out.float().cpu() - want).abs().max().item() <= 0.02


@pytest.mark.parametrize("q_rows,keys,batch", [(50, 572, 3), (522, 522, 2), (5, 200, 1)])
def test_multi_query_heads_share_one_kv_head(q_rows, keys, batch):
    """Eight query heads per sample over one K/V head (head stride 0): the kernel packs the
    heads of a token into the same query tile; layout as the engine's [tokens, heads * 256]."""
    heads, hd = 8, 256
    gen = torch.Generator().manual_seed(q_rows + keys)
    q = torch.randn(batch, q_rows, heads, hd, generator=gen).to(torch.bfloat16)
    kc = torch.randn(batch, keys, hd, generator=gen).to(torch.bfloat16)
    vc = torch.randn(batch, keys, hd, generator=gen).to(torch.bfloat16)
    out = torch.full((batch, q_rows, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc, status = run(q.cuda(), kc.cuda(), vc.cuda(), out, 1 / 16, nb0=heads, nb1=batch,
                     strides=dict(q=(heads * hd, hd, q_rows * heads * hd), k=(hd, 0, keys * hd),
                                  v=(hd, 0, keys * hd), o=(heads * hd, hd, q_rows * heads * hd),
                                  rows=q_rows, keys=keys, hd=hd))
    assert rc == 0 and status == 0
    want = reference(q.float().permute(0, 2, 1, 3), kc.float()[:, None], vc.float()[:, None], 1 / 16)
    want = want.permute(0, 2, 1, 3)
    assert (out.float().cpu() - want).abs().max().item() <= 0.02


@pytest.mark.parametrize("q_rows,keys,batch,hd,heads", [(10, 532, 1, 256, 8), (50, 572, 2, 256, 8),
                                                        (7, 1, 1, 64, 1), (130, 200, 1, 72, 3), (3, 1000, 1, 128, 8)])
@pytest.mark.parametrize("e4m3", [False, True])
def test_key_split_path_matches_the_exact_softmax(q_rows, keys, batch, hd, heads, e4m3):
    """One CTA per (query tile, 64-key slice) + combine launch; multi-query when heads == 8."""
    gen = torch.Generator().manual_seed(q_rows * 7 + keys)
    shared = heads == 8
    q = torch.randn(batch, q_rows, heads, hd, generator=gen).to(torch.bfloat16)
    kv_heads = 1 if shared else heads
    kc = torch.randn(batch, kv_heads, keys, hd, generator=gen).to(torch.bfloat16)
    vc = torch.randn(batch, kv_heads, keys, hd, generator=gen).to(torch.bfloat16)
    dtype = torch.float8_e4m3fn if e4m3 else torch.bfloat16
    out = torch.zeros(batch, q_rows, heads, hd, dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    kv_sb0 = 0 if shared else keys * hd
    rc, status = run(q.cuda(), kc.cuda(), vc.cuda(), out, scale, nb0=heads, nb1=batch, e4m3=e4m3, inv=16.0,
                     key_split=True,
                     strides=dict(q=(heads * hd, hd, q_rows * heads * hd), k=(hd, kv_sb0, kv_heads * keys * hd),
                                  v=(hd, kv_sb0, kv_heads * keys * hd), o=(heads * hd, hd, q_rows * heads * hd),
                                  rows=q_rows, keys=keys, hd=hd))
    assert rc == 0 and status == 0
    want = reference(q.float().permute(0, 2, 1, 3), kc.float().expand(batch, heads, keys, hd),
                     vc.float().expand(batch, heads, keys, hd), scale).permute(0, 2, 1, 3)
    got = out.float().cpu() / (16.0 if e4m3 else 1.0)
    tol = 0.02 + (0.07 * want.abs().max().item() if e4m3 else 0.0)
    assert (got - want).abs().max().item() <= tol


@pytest.mark.parametrize("pattern", ["increasing", "decreasing", "some_rows"])
@pytest.mark.parametrize("layout", ["mqa_hd256", "heads_hd72"])
def test_running_maximum_moves_between_key_blocks(pattern, layout):
    """The fused kernel moves its running row maximum only when a 128-key block exceeds it by
    more than 2^8, and then rescales the output accumulator in tensor memory. Random scores
    never do that, so here every block's scores are shifted by a multiple of 8 nats (11.5
    powers of two) through one query/key component: growing from block to block (a rescale at
    every block), falling (never), and growing for every other query row only (rows of one
    warp disagree). Checked against the float64 softmax with a relative tolerance."""
    gen = torch.Generator().manual_seed(11)
    if layout == "mqa_hd256":
        heads, hd, q_rows, keys, shared = 8, 256, 37, 600, True   # packed multi-query tiles
    else:
        heads, hd, q_rows, keys, shared = 3, 72, 200, 300, False  # odd head_dim, ragged last block
    scale = 1.0 / math.sqrt(hd)
    q = torch.randn(1, q_rows, heads, hd, generator=gen)
    kv_heads = 1 if shared else heads
    k = torch.randn(1, kv_heads, keys, hd, generator=gen)
    v = torch.randn(1, kv_heads, keys, hd, generator=gen)
    blocks = (keys + 127) // 128
    step = 8.0 / (4.0 * scale)          # k component that shifts a block's scores by 8 nats
    q[..., 0] = 4.0
    if pattern == "some_rows":
        q[:, 1::2, :, 0] = 0.0
    for j in range(blocks):
        level = j if pattern != "decreasing" else blocks - 1 - j
        k[:, :, j * 128:(j + 1) * 128, 0] = level * step
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    out = torch.full((1, q_rows, heads, hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    kv_sb0 = 0 if shared else keys * hd
    rc, status = run(q.cuda(), k.cuda(), v.cuda(), out, scale, nb0=heads, nb1=1,
                     strides=dict(q=(heads * hd, hd, q_rows * heads * hd), k=(hd, kv_sb0, kv_heads * keys * hd),
                                  v=(hd, kv_sb0, kv_heads * keys * hd), o=(heads * hd, hd, q_rows * heads * hd),
                                  rows=q_rows, keys=keys, hd=hd))
    assert rc == 0 and status == 0
    want = reference(q.float().permute(0, 2, 1, 3), k.float().expand(1, heads, keys, hd),
                     v.float().expand(1, heads, keys, hd), scale).permute(0, 2, 1, 3)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    err = (got - want).abs()
    assert (err <= 0.01 * want.abs() + 0.01).all(), err.max().item()


def test_key_split_needs_scratch():
    q = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    from apxinf_b200 import lib
    st = dict(q=(64, 0, 0), k=(64, 0, 0), v=(64, 0, 0), o=(64, 0, 0), rows=16, keys=100, hd=64)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = AttentionArgs(q=q.data_ptr(), q_ld=64, k=q.data_ptr(), k_ld=64, v=q.data_ptr(), v_ld=64,
                         out=q.data_ptr(), out_ld=64, q_rows=16, keys=16, head_dim=64, nb0=1, nb1=1, scale=1.0,
                         status=status.data_ptr(), key_split=1, split_scratch=None, split_scratch_bytes=0)
    handle = lib()
    handle.pi05_attention.argtypes = [C.POINTER(AttentionArgs), C.c_void_p]
    handle.pi05_attention.restype = C.c_int
    assert handle.pi05_attention(C.byref(args), None) == -7


def test_rejects_unsupported_shapes():
    q = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    rc, _ = run(q, q, q, q, 1.0, strides=dict(q=(64, 0, 0), k=(64, 0, 0), v=(64, 0, 0), o=(64, 0, 0), rows=16, keys=2000, hd=64))
    assert rc == -1
