"""Pins the oracle, and this library's kernels, against the reference's OWN CUDA kernels: the
self-contained adapters of crates/apxinf-cuda/adapters compiled for sm_100a into oracle/_ref
(oracle/Makefile). Every case runs the reference kernel on seeded inputs on the GPU and
compares it with the NumPy restatement the whole-model oracle is made of and, where this
library exports the same entry point, with this library's kernel."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import pi05_oracle as O
from oracle import ref_ops

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_ops.available(), reason="oracle/_ref was not built")]

F32 = np.float32


def _ours():
    from apxinf_b200 import lib
    return lib()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _bf16(rng, *shape, scale=1.0):
    return torch.from_numpy((rng.standard_normal(shape) * scale).astype(F32)).to(torch.bfloat16).cuda()


def _np(t):
    return t.float().cpu().numpy()


def _ulps(got, want, floor=2.0 ** -20):
    """Largest difference in bf16 steps of the expected value's binade (values below `floor`
    are measured in steps of `floor`'s binade: results of cancellations have no relative scale)."""
    got, want = np.asarray(got, F32), np.asarray(want, F32)
    step = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), floor))) - 7)
    return float(np.max(np.abs(got - want) / step))


def _call(handle, name, *args):
    rc = getattr(handle, name)(*args)
    torch.cuda.synchronize()
    assert rc == 0, (name, rc)


def test_patch_rows_reference_oracle_and_ours_are_bit_identical():
    cfg = O.Pi05Config()
    rng = np.random.default_rng(1)
    images = rng.integers(0, 256, (2, 224, 224, 3), dtype=np.uint8)
    d = torch.from_numpy(images).cuda()
    ref = torch.zeros(512, 588, dtype=torch.bfloat16, device="cuda")
    ours = torch.zeros_like(ref)
    _call(ref_ops.lib("bf16"), "apxinf_static_rgb_u8_to_patches_bf16", _p(d), _p(ref), 2, 224, 14, 0, _stream())
    _call(_ours(), "apxinf_static_rgb_u8_to_patches_bf16", _p(d), _p(ours), 2, 224, 14, 0, _stream())
    want = O.round_bf16(O.patchify(images, cfg))
    assert np.array_equal(_np(ref), want)
    assert np.array_equal(_np(ours), _np(ref))


@pytest.mark.parametrize("rows,cols", [(7, 1152), (50, 1024), (3, 2048)])
def test_norms_reference_oracle_and_ours(rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = _bf16(rng, rows, cols)
    weight = _bf16(rng, cols, scale=0.5)
    bias = _bf16(rng, cols, scale=0.5)
    style = _bf16(rng, 3 * cols, scale=0.3)
    oracle = O.Pi05Oracle(O.Pi05Config(), None, O.OracleOptions())
    xs, ws, bs, ss = _np(x), _np(weight), _np(bias), _np(style)
    cases = [
        ("apxinf_static_rms_norm_bf16", (_p(x), _p(weight)), 1e-6,
         oracle.rms_norm(xs) * ws[None]),
        ("apxinf_static_layer_norm_bf16", (_p(x), _p(weight), _p(bias)), 1e-6,
         oracle.layer_norm(xs) * ws[None] + bs[None]),
        ("apxinf_static_ada_rms_norm_bf16", (_p(x), _p(style)), 1e-6,
         oracle.ada_rms_norm(xs, ss)),
    ]
    for name, inputs, eps, want in cases:
        ref = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
        ours = torch.zeros_like(ref)
        _call(ref_ops.lib("bf16"), name, *inputs, _p(ref), rows, cols, C.c_float(eps), _stream())
        _call(_ours(), name, *inputs, _p(ours), rows, cols, C.c_float(eps), _stream())
        # rsqrtf and the block reduction order differ from NumPy by at most one bf16 step
        assert _ulps(_np(ref), O.round_bf16(want)) <= 1.0, name
        assert _ulps(_np(ours), _np(ref)) <= 1.0, name


def test_euler_update_and_embedding():
    rng = np.random.default_rng(4)
    state, velocity = _bf16(rng, 50, 32), _bf16(rng, 50, 32)
    ref = torch.zeros_like(state)
    ours = torch.zeros_like(state)
    for handle, out in ((ref_ops.lib("bf16"), ref), (_ours(), ours)):
        _call(handle, "apxinf_static_euler_update_bf16", _p(state), _p(velocity), _p(out),
              C.c_int64(state.numel()), C.c_float(-0.1), _stream())
    want = O.round_bf16(_np(state) + F32(-0.1) * _np(velocity))
    assert np.array_equal(_np(ref), want) and np.array_equal(_np(ours), want)

    table = _bf16(rng, 64, 256)
    ids = torch.tensor([0, 5, 63, 64, 1000, 17], dtype=torch.int32, device="cuda")  # two beyond the table
    ref = torch.full((6, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    ours = torch.full_like(ref, 7.0)
    for handle, out in ((ref_ops.lib("bf16"), ref), (_ours(), ours)):
        _call(handle, "apxinf_static_embedding_bf16", _p(table), _p(ids), _p(out), 6, 256, 64, _stream())
    assert np.array_equal(_np(ours), _np(ref))


def test_int8_row_quantiser_reference_oracle_and_ours_are_bit_identical():
    rng = np.random.default_rng(5)
    x = _bf16(rng, 33, 1024, scale=3.0)
    x[3] = 0  # an all-zero row takes the 1e-12 floor
    results = []
    for handle in (ref_ops.lib("w8a8"), _ours()):
        codes = torch.zeros(33, 1024, dtype=torch.int8, device="cuda")
        scales = torch.zeros(33, dtype=torch.float32, device="cuda")
        _call(handle, "apxinf_static_quantize_rows_bf16_int8", _p(x), _p(codes), _p(scales), 33, 1024, _stream())
        results.append((codes.cpu().numpy(), scales.cpu().numpy()))
    want_codes, want_scales = O.quantize_rows_int8(_np(x))
    assert np.array_equal(results[0][0], want_codes) and np.array_equal(results[0][1], want_scales.reshape(-1))
    assert np.array_equal(results[1][0], results[0][0]) and np.array_equal(results[1][1], results[0][1])


def test_attention_reference_oracle_and_fused_kernel():
    rng = np.random.default_rng(6)
    tokens, keys, heads, hd = 10, 532, 8, 256
    q, k, v = _bf16(rng, tokens, heads, hd), _bf16(rng, keys, hd), _bf16(rng, keys, hd)
    ref = torch.zeros(tokens, heads, hd, dtype=torch.bfloat16, device="cuda")
    ours = torch.zeros_like(ref)
    args = (_p(q), _p(k), _p(v))
    _call(ref_ops.lib("bf16"), "apxinf_static_mqa_bf16", *args, _p(ref), tokens, keys, heads, hd, _stream())
    _call(_ours(), "apxinf_static_mqa_bf16", *args, _p(ours), tokens, keys, heads, hd, _stream())
    oracle = O.Pi05Oracle(O.Pi05Config(), None, O.OracleOptions())
    want = oracle.attention(_np(q), _np(k)[:, None], _np(v)[:, None], 1.0 / 16.0, False).reshape(tokens, heads, hd)
    assert np.abs(_np(ref) - want).max() <= 0.01       # the restatement against the reference kernel
    assert np.abs(_np(ours) - _np(ref)).max() <= 0.02  # bf16 probabilities in the tensor-core kernel

    images, patches, vh, vd = 2, 256, 16, 72
    shape = (images * patches, vh, vd)
    q, k, v = _bf16(rng, *shape), _bf16(rng, *shape), _bf16(rng, *shape)
    ref = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    ours = torch.zeros_like(ref)
    _call(ref_ops.lib("bf16"), "apxinf_static_mha_bf16", _p(q), _p(k), _p(v), _p(ref), patches, images, vh, vd, _stream())
    _call(_ours(), "apxinf_static_mha_bf16", _p(q), _p(k), _p(v), _p(ours), patches, images, vh, vd, _stream())
    assert np.abs(_np(ours) - _np(ref)).max() <= 0.02


def test_elementwise_epilogues_reference_against_the_oracle_formulas():
    """GeGLU, bias + residual and the gated residual are GEMM epilogues in this library; the
    oracle's formulas for them are the ones checked here against the reference kernels."""
    rng = np.random.default_rng(7)
    rows, inner, cols = 50, 4096, 1024
    gate_up = _bf16(rng, rows, 2 * inner, scale=2.0)
    out = torch.zeros(rows, inner, dtype=torch.bfloat16, device="cuda")
    _call(ref_ops.lib("bf16"), "apxinf_static_geglu_bf16", _p(gate_up), _p(out), rows, inner, _stream())
    g = _np(gate_up)
    want = O.round_bf16(O.gelu_tanh(g[:, :inner]) * g[:, inner:])
    # tanhf; 0.5 x (1 + tanh u) cancels for x << 0, so small products are compared absolutely
    assert _ulps(_np(out), want, floor=2.0 ** -6) <= 1.0

    proj, res, bias = _bf16(rng, rows, cols), _bf16(rng, rows, cols), _bf16(rng, cols)
    out = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    _call(ref_ops.lib("bf16"), "apxinf_static_bias_residual_bf16", _p(proj), _p(bias), _p(res), _p(out), rows, cols, _stream())
    assert np.array_equal(_np(out), O.round_bf16(_np(proj) + _np(res) + _np(bias)[None]))

    style = _bf16(rng, 3 * cols, scale=0.3)
    _call(ref_ops.lib("bf16"), "apxinf_static_ada_gate_residual_bf16", _p(proj), _p(res), _p(style), _p(out), rows, cols, _stream())
    assert np.array_equal(_np(out), O.round_bf16(_np(res) + _np(proj) * _np(style)[None, 2 * cols:]))


def test_rope_split_reference_against_the_oracle():
    rng = np.random.default_rng(8)
    cfg = O.Pi05Config()
    g = cfg.action_expert
    tokens, offset = 10, 522
    qkv = _bf16(rng, tokens, (g.num_heads + 2) * g.head_dim)
    q = torch.zeros(tokens, g.num_heads, g.head_dim, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(offset + tokens, g.head_dim, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    _call(ref_ops.lib("bf16"), "apxinf_static_qkv_rope_bf16", _p(qkv), None, _p(q), _p(k), _p(v), tokens,
          g.num_heads, 1, g.head_dim, C.c_float(cfg.rope_theta), offset, offset, _stream())
    oracle = O.Pi05Oracle(cfg, None, O.OracleOptions())
    wq, wk, wv = oracle.rope_split(_np(qkv), g, np.arange(offset, offset + tokens))
    # powf / sincosf against float64 tables: positions of ~500 rad leave a few 1e-3 absolute
    assert np.abs(_np(q) - wq).max() <= 0.02 and np.abs(_np(k)[offset:] - wk[:, 0]).max() <= 0.02
    assert np.array_equal(_np(v)[offset:], wv[:, 0])


def test_e4m3_codec_reference_kernel_against_the_oracle_for_every_f16_input():
    """Every finite half-precision value through the reference's quantiser
    (kernels/custom/quantization.cuh:6-16) against the oracle's encoder, at two scales."""
    bits = np.arange(65536, dtype=np.uint16)
    values = bits.view(np.float16)
    finite = np.isfinite(values)
    x = torch.from_numpy(values[finite].copy()).cuda()
    for scale in (1.0, 0.05):
        out = torch.zeros(x.numel(), dtype=torch.uint8, device="cuda")
        _call(ref_ops.lib("f16"), "apxinf_static_quantize_f16_e4m3", _p(x), _p(out), C.c_int64(x.numel()),
              C.c_float(scale), _stream())
        scaled = np.clip(values[finite].astype(F32) * F32(1.0 / scale), -448.0, 448.0).astype(F32)
        want = O.e4m3_encode(scaled)
        got = out.cpu().numpy()
        same = got == want
        # +0 and -0 are distinct bytes with the same value
        assert np.all(same | ((got & 0x7F) == 0) & ((want & 0x7F) == 0))


def _both(name, build_args, outputs, tolerance_ulps=0.0):
    """Runs `name` from the reference library and from this one on the same inputs;
    `build_args(outs)` returns the argument tuple for a list of output tensors."""
    results = []
    for handle in (ref_ops.lib("bf16"), _ours()):
        outs = [torch.full_like(o, 3.0) for o in outputs]
        _call(handle, name, *build_args(outs), _stream())
        results.append([_np(o) for o in outs])
    for ref, ours in zip(*results):
        if tolerance_ulps == 0.0:
            assert np.array_equal(ours, ref), name
        else:
            assert _ulps(ours, ref, floor=2.0 ** -6) <= tolerance_ulps, name


def test_remaining_static_row_operators_match_the_reference_kernels():
    rng = np.random.default_rng(9)
    rows, cols, inner = 37, 1152, 512
    x, res = _bf16(rng, rows, cols), _bf16(rng, rows, cols)
    bias, weight, nbias = _bf16(rng, cols), _bf16(rng, cols, scale=0.5), _bf16(rng, cols, scale=0.5)
    style, style2 = _bf16(rng, 3 * cols, scale=0.3), _bf16(rng, 3 * cols, scale=0.3)
    out = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    for activation, ulps in ((0, 0.0), (1, 1.0), (2, 1.0)):
        _both("apxinf_static_bias_activation_bf16",
              lambda o: (_p(x), _p(bias), _p(o[0]), rows, cols, activation), [out], ulps)
    _both("apxinf_static_bias_activation_bf16", lambda o: (_p(x), None, _p(o[0]), rows, cols, 0), [out])
    _both("apxinf_static_bias_residual_bf16", lambda o: (_p(x), _p(bias), _p(res), _p(o[0]), rows, cols), [out])
    _both("apxinf_static_ada_gate_residual_bf16", lambda o: (_p(x), _p(res), _p(style), _p(o[0]), rows, cols), [out])
    pos = _bf16(rng, 16, cols)
    _both("apxinf_static_bias_position_bf16", lambda o: (_p(x), _p(bias), _p(pos), _p(o[0]), rows, cols, 16), [out])
    gate_up = _bf16(rng, rows, 2 * inner, scale=2.0)
    _both("apxinf_static_geglu_bf16", lambda o: (_p(gate_up), _p(o[0]), rows, inner),
          [torch.zeros(rows, inner, dtype=torch.bfloat16, device="cuda")], 1.0)
    second = _bf16(rng, 5, cols)
    _both("apxinf_static_concat_rows_bf16", lambda o: (_p(x), _p(second), _p(o[0]), rows, 5, cols),
          [torch.zeros(rows + 5, cols, dtype=torch.bfloat16, device="cuda")])
    eps = C.c_float(1e-6)
    _both("apxinf_static_bias_residual_rms_norm_bf16",
          lambda o: (_p(x), _p(bias), _p(res), _p(weight), _p(o[0]), _p(o[1]), rows, cols, eps), [out, out], 1.0)
    _both("apxinf_static_bias_residual_layer_norm_bf16",
          lambda o: (_p(x), _p(bias), _p(res), _p(weight), _p(nbias), _p(o[0]), _p(o[1]), rows, cols, eps),
          [out, out], 1.0)
    _both("apxinf_static_ada_gate_residual_rms_norm_bf16",
          lambda o: (_p(x), _p(res), _p(style), _p(style2), _p(o[0]), _p(o[1]), rows, cols, eps), [out, out], 1.0)


def test_remaining_static_split_operators_match_the_reference_kernels():
    rng = np.random.default_rng(10)
    tokens, qh, kvh, hd, offset = 10, 8, 1, 256, 522
    qkv = _bf16(rng, tokens, (qh + 2 * kvh) * hd)
    bias = _bf16(rng, (qh + 2 * kvh) * hd, scale=0.1)
    q = torch.zeros(tokens, qh, hd, dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros(offset + tokens, kvh, hd, dtype=torch.bfloat16, device="cuda")
    for b in (None, bias):
        _both("apxinf_static_qkv_rope_bf16",
              lambda o: (_p(qkv), _p(b), _p(o[0]), _p(o[1]), _p(o[2]), tokens, qh, kvh, hd, C.c_float(10000.0),
                         offset, offset), [q, kv, kv], 1.0)
    width = 1152
    packed = _bf16(rng, 20, 3 * width)
    pb = _bf16(rng, 3 * width)
    third = torch.zeros(20, width, dtype=torch.bfloat16, device="cuda")
    _both("apxinf_static_qkv_split_bias_bf16",
          lambda o: (_p(packed), _p(pb), _p(o[0]), _p(o[1]), _p(o[2]), 20, width), [third, third, third])
