"""The F16 / E4M3 operator names of the reference's FP8 path exported by this library
(include/pi05_apxinf_static.h, apxinf_b200/csrc/abi_apxinf_static_f16.cu), each run beside the
reference's own compiled kernel (oracle/_ref, built by oracle/Makefile from
crates/apxinf-cuda/adapters/{custom_kernels,cublaslt_adapter,cublas_adapter,w8a8_adapter}.cu)
on the same seeded inputs. Elementwise operators must agree bit for bit; operators with a
block reduction (norms) or a long sum (attention, GEMM) within the stated steps."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import ref_forward as R
from oracle import ref_ops

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (ref_ops.available() and R.available()), reason="oracle/_ref was not built")]


def _ours():
    from apxinf_b200 import lib
    return lib()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _f16(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.float16).cuda()


def _both(name, make_args, outputs):
    """Runs `name` of the reference library and of this library; `make_args(outs)` builds the
    argument list around the given output tensors. Returns ([ref outs], [our outs])."""
    results = []
    for handle in (ref_ops.lib("f16"), _ours()):
        outs = [torch.zeros_like(o) for o in outputs]
        rc = getattr(handle, name)(*make_args(outs), _stream())
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        results.append(outs)
    return results


def _bytes(t):
    return t.view(torch.uint8).cpu().numpy()


def _e4m3_steps(a, b):
    """Distance in e4m3 codes (sign-magnitude order) between two byte tensors."""
    def order(x):
        x = x.astype(np.int32)
        return np.where(x & 0x80, -(x & 0x7F), x & 0x7F)
    return np.abs(order(_bytes(a)) - order(_bytes(b)))


def test_elementwise_operators_are_bit_identical():
    gen = torch.Generator().manual_seed(1)
    rows, cols = 37, 1152
    x, res = _f16(gen, rows, cols), _f16(gen, rows, cols)
    bias = _f16(gen, cols, scale=0.3)
    style = _f16(gen, 3 * cols, scale=0.3)
    e8 = torch.zeros(rows, cols, dtype=torch.uint8, device="cuda")
    h16 = torch.zeros(rows, cols, dtype=torch.float16, device="cuda")
    scale = C.c_float(0.05)
    count = C.c_int64(rows * cols)
    cases = [
        ("apxinf_static_quantize_f16_e4m3", lambda o: (_p(x), _p(o[0]), count, scale), [e8]),
        ("apxinf_static_bias_gelu_quant_f16_e4m3", lambda o: (_p(x), _p(bias), _p(o[0]), rows, cols, scale), [e8]),
        ("apxinf_static_bias_silu_quant_f16_e4m3", lambda o: (_p(x), _p(bias), _p(o[0]), rows, cols, scale), [e8]),
        ("apxinf_static_bias_silu_f16", lambda o: (_p(x), _p(bias), _p(o[0]), rows, cols), [h16]),
        ("apxinf_static_bias_f16", lambda o: (_p(x), None, _p(o[0]), rows, cols), [h16]),
        ("apxinf_static_bias_f16", lambda o: (_p(x), _p(bias), _p(o[0]), rows, cols), [h16]),
        ("apxinf_static_euler_update_f16", lambda o: (_p(x), _p(res), _p(o[0]), count, C.c_float(-0.1)), [h16]),
        ("apxinf_static_bias_residual_f16", lambda o: (_p(x), _p(bias), _p(res), _p(o[0]), rows, cols), [h16]),
        ("apxinf_static_ada_gate_residual_f16", lambda o: (_p(x), _p(res), _p(style), _p(o[0]), rows, cols), [h16]),
        # (the reference wants whole views: rows a multiple of tokens_per_view)
        ("apxinf_static_bias_position_f16",
         lambda o: (_p(x), _p(bias), _p(res), _p(o[0]), 32, cols, 16), [h16]),
        ("apxinf_static_geglu_quant_f16_e4m3",
         lambda o: (_p(x), _p(o[0]), rows, cols // 2, scale), [torch.zeros(rows, cols // 2, dtype=torch.uint8, device="cuda")]),
        ("apxinf_static_concat_rows_f16",
         lambda o: (_p(x), _p(res), _p(o[0]), rows, rows, cols), [torch.zeros(2 * rows, cols, dtype=torch.float16, device="cuda")]),
    ]
    for name, make, outs in cases:
        ref, ours = _both(name, make, outs)
        assert np.array_equal(_bytes(ref[0]), _bytes(ours[0])), name
    # dequantise every e4m3 code
    codes = torch.arange(256, dtype=torch.uint8, device="cuda")
    ref, ours = _both("apxinf_static_dequantize_e4m3_f16",
                      lambda o: (_p(codes), _p(o[0]), C.c_int64(256), C.c_float(0.5)),
                      [torch.zeros(256, dtype=torch.float16, device="cuda")])
    a, b = ref[0].float().cpu().numpy(), ours[0].float().cpu().numpy()
    assert np.array_equal(np.isnan(a), np.isnan(b)) and np.array_equal(a[~np.isnan(a)], b[~np.isnan(b)])


def test_embedding_patches_and_qkv_split():
    gen = torch.Generator().manual_seed(2)
    table = _f16(gen, 64, 256)
    ids = torch.tensor([0, 5, 63, 64, 1000, 17], dtype=torch.int32, device="cuda")
    ref, ours = _both("apxinf_static_embedding_f16", lambda o: (_p(table), _p(ids), _p(o[0]), 6, 256, 64),
                      [torch.zeros(6, 256, dtype=torch.float16, device="cuda")])
    assert np.array_equal(_bytes(ref[0]), _bytes(ours[0]))
    images = torch.randint(0, 256, (2, 224, 224, 3), dtype=torch.uint8, generator=gen).cuda()
    for layout, data in ((0, images), (1, images.permute(0, 3, 1, 2).contiguous())):
        ref, ours = _both("apxinf_static_rgb_u8_to_patches_e4m3",
                          lambda o: (_p(data), _p(o[0]), 2, 224, 14, layout, C.c_float(0.05)),
                          [torch.zeros(512, 588, dtype=torch.uint8, device="cuda")])
        assert np.array_equal(_bytes(ref[0]), _bytes(ours[0])), layout
    tokens, width = 9, 144
    qkv, bias = _f16(gen, tokens, 3 * width), _f16(gen, 3 * width, scale=0.3)
    outs = [torch.zeros(tokens, width, dtype=torch.float16, device="cuda") for _ in range(3)]
    ref, ours = _both("apxinf_static_qkv_split_bias_f16",
                      lambda o: (_p(qkv), _p(bias), _p(o[0]), _p(o[1]), _p(o[2]), tokens, width), outs)
    for a, b in zip(ref, ours):
        assert np.array_equal(_bytes(a), _bytes(b))


@pytest.mark.parametrize("rows,cols", [(7, 1152), (10, 1024), (3, 2048)])
def test_norm_operators_within_one_code(rows, cols):
    gen = torch.Generator().manual_seed(rows + cols)
    x, res = _f16(gen, rows, cols), _f16(gen, rows, cols)
    weight, bias = _f16(gen, cols, scale=0.5), _f16(gen, cols, scale=0.5)
    style, style2 = _f16(gen, 3 * cols, scale=0.3), _f16(gen, 3 * cols, scale=0.3)
    e8 = torch.zeros(rows, cols, dtype=torch.uint8, device="cuda")
    h16 = torch.zeros(rows, cols, dtype=torch.float16, device="cuda")
    eps, scale = C.c_float(1e-6), C.c_float(0.05)
    cases = [
        ("apxinf_static_rms_norm_quant_f16_e4m3", lambda o: (_p(x), _p(weight), _p(o[0]), rows, cols, eps, scale), [e8]),
        ("apxinf_static_layer_norm_quant_f16_e4m3",
         lambda o: (_p(x), _p(weight), _p(bias), _p(o[0]), rows, cols, eps, scale), [e8]),
        ("apxinf_static_ada_rms_norm_quant_f16_e4m3", lambda o: (_p(x), _p(style), _p(o[0]), rows, cols, eps, scale), [e8]),
        ("apxinf_static_bias_residual_rms_norm_quant_f16_e4m3",
         lambda o: (_p(x), _p(bias), _p(res), _p(weight), _p(o[0]), _p(o[1]), rows, cols, eps, scale), [h16, e8]),
        ("apxinf_static_bias_residual_layer_norm_quant_f16_e4m3",
         lambda o: (_p(x), _p(bias), _p(res), _p(weight), _p(bias), _p(o[0]), _p(o[1]), rows, cols, eps, scale), [h16, e8]),
        ("apxinf_static_ada_gate_residual_rms_norm_quant_f16_e4m3",
         lambda o: (_p(x), _p(res), _p(style), _p(style2), _p(o[0]), _p(o[1]), rows, cols, eps, scale), [h16, e8]),
    ]
    for name, make, outs in cases:
        ref, ours = _both(name, make, outs)
        if len(outs) == 2:  # the stored hidden state is elementwise
            assert np.array_equal(_bytes(ref[0]), _bytes(ours[0])), name
        steps = _e4m3_steps(ref[-1], ours[-1])
        # the block reduction order differs: a value next to a rounding boundary may take the next code
        assert steps.max() <= 1 and (steps > 0).mean() < 0.01, (name, steps.max(), (steps > 0).mean())


def test_qkv_rope_and_attention():
    gen = torch.Generator().manual_seed(3)
    tokens, heads, hd, offset = 10, 8, 256, 522
    qkv = _f16(gen, tokens, (heads + 2) * hd)
    outs = [torch.zeros(tokens, heads, hd, dtype=torch.float16, device="cuda"),
            torch.zeros(offset + tokens, hd, dtype=torch.float16, device="cuda"),
            torch.zeros(offset + tokens, hd, dtype=torch.float16, device="cuda")]
    ref, ours = _both("apxinf_static_qkv_rope_f16",
                      lambda o: (_p(qkv), None, _p(o[0]), _p(o[1]), _p(o[2]), tokens, heads, 1, hd,
                                 C.c_float(10000.0), offset, offset), outs)
    for a, b in zip(ref, ours):
        assert (a.float() - b.float()).abs().max().item() <= 2e-3  # powf / sincosf at ~500 rad
    # suffix rows over a cached prefix + the suffix keys
    q = _f16(gen, tokens, heads, hd)
    pk, pv = _f16(gen, 64, hd), _f16(gen, 64, hd)
    sk, sv = _f16(gen, tokens, hd), _f16(gen, tokens, hd)
    ref, ours = _both("apxinf_static_mqa_flash_f16",
                      lambda o: (_p(q), _p(pk), _p(pv), _p(sk), _p(sv), _p(o[0]), tokens, heads, hd, 64),
                      [torch.zeros(tokens, heads, hd, dtype=torch.float16, device="cuda")])
    assert (ref[0].float() - ours[0].float()).abs().max().item() <= 3e-3
    # SigLIP shape: per-view multi-head attention
    tokens_v, heads_v, hd_v, views = 64, 4, 72, 2
    qv, kv, vv = (_f16(gen, views * tokens_v, heads_v, hd_v) for _ in range(3))
    ref, ours = _both("apxinf_static_mha_flash_f16",
                      lambda o: (_p(qv), _p(kv), _p(vv), _p(o[0]), tokens_v, views, heads_v, hd_v),
                      [torch.zeros(views * tokens_v, heads_v, hd_v, dtype=torch.float16, device="cuda")])
    assert (ref[0].float() - ours[0].float()).abs().max().item() <= 3e-3
    # the cuBLAS MQA name (logits and probabilities rounded to f16 there)
    keys = 522
    kk, vk = _f16(gen, keys, hd), _f16(gen, keys, hd)
    out_ref = torch.zeros(tokens, heads, hd, dtype=torch.float16, device="cuda")
    out_ours = torch.zeros_like(out_ref)
    rc = R.lib("cublas_mqa").apxinf_static_cublas_mqa_f16(_p(q), _p(kk), _p(vk), _p(out_ref), tokens, keys, heads, hd,
                                                          _stream())
    assert rc == 0
    rc = _ours().apxinf_static_cublas_mqa_f16(_p(q), _p(kk), _p(vk), _p(out_ours), tokens, keys, heads, hd, _stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert (out_ref.float() - out_ours.float()).abs().max().item() <= 1e-2


@pytest.mark.parametrize("m,n,k", [(522, 2560, 2048), (10, 1024, 4096), (512, 4304, 1152)])
def test_fp8_gemm_family_against_cublaslt(m, n, k):
    """E4M3 x E4M3 -> F16 with the weight in the reference's [k, n] layout: the tcgen05 GEMM of
    this library against the reference's cuBLASLt calls, plain and with the three fused forms."""
    gen = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=gen) * 2).to(torch.float8_e4m3fn).cuda()
    w = (torch.randn(k, n, generator=gen) * 2).to(torch.float8_e4m3fn).cuda()
    bias = _f16(gen, n, scale=0.5)
    residual = _f16(gen, m, n)
    alpha = C.c_float(0.05 * 0.02)
    ref_lib, ours = R.lib("cublaslt"), _ours()

    def run(handle, name, prepare, prep_args, args, out):
        rc = getattr(handle, prepare)(*prep_args)
        assert rc == 0, (prepare, rc)
        rc = getattr(handle, name)(*args, _stream())
        torch.cuda.synchronize()
        assert rc == 0, (name, rc)
        return out

    def compare(name, prepare, prep_args, make_args, dtype, tol):
        outs = []
        for handle in (ref_lib, ours):
            out = torch.zeros(m, n, dtype=dtype, device="cuda")
            outs.append(run(handle, name, prepare, prep_args, make_args(out), out))
        if dtype == torch.uint8:
            steps = _e4m3_steps(outs[0], outs[1])
            assert steps.max() <= 1 and (steps > 0).mean() < 0.02, (name, steps.max(), (steps > 0).mean())
        else:
            ref, got = outs[0].float(), outs[1].float()
            assert (ref - got).abs().max().item() <= tol * max(1.0, ref.abs().max().item()), name

    # run before prepare is refused, as in the reference
    unprepared = torch.zeros(3, 16, dtype=torch.float16, device="cuda")
    assert ours.apxinf_static_fp8_gemm_f16(_p(a), _p(w), _p(unprepared), 3, 16, 32, alpha, _stream()) == 1
    compare("apxinf_static_fp8_gemm_f16", "apxinf_static_prepare_fp8_gemm_f16", (m, n, k),
            lambda o: (_p(a), _p(w), _p(o), m, n, k, alpha), torch.float16, 2e-3)
    compare("apxinf_static_fp8_gemm_bias_f16", "apxinf_static_prepare_fp8_gemm_bias_f16", (_p(bias), m, n, k),
            lambda o: (_p(a), _p(w), _p(bias), _p(o), m, n, k, alpha), torch.float16, 2e-3)
    compare("apxinf_static_fp8_gemm_bias_residual_f16", "apxinf_static_prepare_fp8_gemm_bias_residual_f16",
            (_p(bias), m, n, k), lambda o: (_p(a), _p(w), _p(bias), _p(residual), _p(o), m, n, k, alpha),
            torch.float16, 2e-3)
    compare("apxinf_static_fp8_gemm_bias_gelu_e4m3", "apxinf_static_prepare_fp8_gemm_bias_gelu_e4m3",
            (_p(bias), m, n, k, C.c_float(0.05)),
            lambda o: (_p(a), _p(w), _p(bias), _p(o), m, n, k, alpha, C.c_float(0.05)), torch.uint8, 0)
    # the CUTLASS name: same product, no prepare; bad tactics are refused with the reference's code
    out = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    assert ours.apxinf_static_cutlass_fp8_gemm_f16(_p(a), _p(w), _p(out), m, n, k, alpha, 3, _stream()) == 0
    torch.cuda.synchronize()
    want = (a.float() @ w.float()) * alpha.value
    assert (out.float() - want).abs().max().item() <= 2e-3 * max(1.0, want.abs().max().item())
    assert ours.apxinf_static_cutlass_fp8_gemm_f16(_p(a), _p(w), _p(out), m, n, k, alpha, 9, _stream()) == -5


def test_w8a8_gemm_names():
    gen = torch.Generator().manual_seed(9)
    m, n, k = 50, 1024, 2048
    a = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8).cuda()
    w = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8).cuda()
    rs = (torch.rand(m, generator=gen) * 0.01 + 0.001).cuda()
    cs = (torch.rand(n, generator=gen) * 0.01 + 0.001).cuda()
    acc = (a.cpu().to(torch.int64) @ w.cpu().to(torch.int64).t()).to(torch.int32).cuda()
    want = (acc.float() * rs[:, None] * cs[None, :]).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    rc = _ours().apxinf_static_cutlass_int8_gemm_bf16(_p(a), _p(w), _p(rs), _p(cs), _p(out), m, n, k, _stream())
    torch.cuda.synchronize()
    assert rc == 0
    assert (out.float() - want.float()).abs().max().item() <= 0.01 * want.float().abs().max().item()
    ref = torch.zeros_like(out)
    ours = torch.zeros_like(out)
    for handle, dst in ((ref_ops.lib("w8a8"), ref), (_ours(), ours)):
        rc = handle.apxinf_static_dequantize_int32_bf16(_p(acc), _p(rs), _p(cs), _p(dst), m, n, _stream())
        torch.cuda.synchronize()
        assert rc == 0
    assert torch.equal(ref, ours)
