"""Kernel-level entry points under the reference's symbol names (include/pi05_apxinf_static.h)
against the CPU oracle's restatement of the same reference kernels."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import pi05_oracle as O

pytestmark = pytest.mark.gpu


def _lib():
    from apxinf_b200 import lib
    return lib()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bf16(t):
    return t.float().cpu().numpy()


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_rgb_u8_to_patches_bf16_bit_exact_nhwc_and_nchw():
    # crates/apxinf-cuda/src/tests/fp8.rs:238-323: both wire layouts give identical patch rows
    cfg = O.Pi05Config()
    images = O.reference_image_pattern(cfg)
    want = O.round_bf16(O.patchify(images, cfg))
    out = torch.zeros(want.shape, dtype=torch.bfloat16, device="cuda")
    nhwc = torch.from_numpy(images).cuda()
    rc = _lib().apxinf_static_rgb_u8_to_patches_bf16(_p(nhwc), _p(out), 2, 224, 14, 0, _stream())
    torch.cuda.synchronize()
    assert rc == 0 and np.array_equal(_bf16(out), want)
    nchw = torch.from_numpy(np.ascontiguousarray(images.transpose(0, 3, 1, 2))).cuda()
    out2 = torch.zeros_like(out)
    rc = _lib().apxinf_static_rgb_u8_to_patches_bf16(_p(nchw), _p(out2), 2, 224, 14, 1, _stream())
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(out, out2)
    assert _lib().apxinf_static_rgb_u8_to_patches_bf16(None, _p(out), 2, 224, 14, 0, _stream()) == 1


# (the last three take the warp-per-row kernel of the batched forward; row counts off the CTA size)
@pytest.mark.parametrize("rows,cols", [(10, 1024), (522, 2048), (512, 1152), (4100, 1152), (2501, 2048), (1027, 1024)])
def test_norms_match_oracle(rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = O.round_bf16(rng.standard_normal((rows, cols)).astype(np.float32) * 3)
    w = O.round_bf16(1 + 0.1 * rng.standard_normal(cols).astype(np.float32))
    b = O.round_bf16(0.1 * rng.standard_normal(cols).astype(np.float32))
    style = O.round_bf16(0.2 * rng.standard_normal(3 * cols).astype(np.float32))
    xd = torch.from_numpy(x).to(torch.bfloat16).cuda()
    wd = torch.from_numpy(w).to(torch.bfloat16).cuda()
    bd = torch.from_numpy(b).to(torch.bfloat16).cuda()
    sd = torch.from_numpy(style).to(torch.bfloat16).cuda()
    out = torch.zeros_like(xd)
    oracle = O.Pi05Oracle(O.tiny_config(), O.SyntheticWeights(O.tiny_config(), 0), O.OracleOptions())

    def close(got, want):
        err = np.abs(got - want)
        # one bf16 ulp (reduction order and rsqrt differ in the last float bit)
        assert (err <= np.abs(want) * 2.0 ** -7 + 1e-3).all(), err.max()
        assert (err == 0).mean() > 0.98

    assert _lib().apxinf_static_rms_norm_bf16(_p(xd), _p(wd), _p(out), rows, cols, C.c_float(1e-6), _stream()) == 0
    torch.cuda.synchronize()
    close(_bf16(out), O.round_bf16(oracle.rms_norm(x) * w[None, :]))
    assert _lib().apxinf_static_layer_norm_bf16(_p(xd), _p(wd), _p(bd), _p(out), rows, cols, C.c_float(1e-6), _stream()) == 0
    torch.cuda.synchronize()
    close(_bf16(out), O.round_bf16(oracle.layer_norm(x) * w[None, :] + b[None, :]))
    assert _lib().apxinf_static_ada_rms_norm_bf16(_p(xd), _p(sd), _p(out), rows, cols, C.c_float(1e-6), _stream()) == 0
    torch.cuda.synchronize()
    close(_bf16(out), O.round_bf16(oracle.ada_rms_norm(x, style)))


def test_quantize_rows_int8_bit_exact():
    rng = np.random.default_rng(3)
    x = O.round_bf16(rng.standard_normal((50, 4096)).astype(np.float32) * 2)
    x[7] = 0.0  # an all-zero row takes the 1e-12 floor
    xd = torch.from_numpy(x).to(torch.bfloat16).cuda()
    q = torch.zeros(50, 4096, dtype=torch.int8, device="cuda")
    scales = torch.zeros(50, dtype=torch.float32, device="cuda")
    assert _lib().apxinf_static_quantize_rows_bf16_int8(_p(xd), _p(q), _p(scales), 50, 4096, _stream()) == 0
    torch.cuda.synchronize()
    want_q, want_s = O.quantize_rows_int8(x)
    assert np.array_equal(scales.cpu().numpy(), want_s)
    assert np.array_equal(q.cpu().numpy(), want_q.astype(np.int8))


def test_euler_and_embedding():
    rng = np.random.default_rng(4)
    state = O.round_bf16(rng.standard_normal(320).astype(np.float32))
    vel = O.round_bf16(rng.standard_normal(320).astype(np.float32))
    sd = torch.from_numpy(state).to(torch.bfloat16).cuda()
    vd = torch.from_numpy(vel).to(torch.bfloat16).cuda()
    out = torch.zeros_like(sd)
    assert _lib().apxinf_static_euler_update_bf16(_p(sd), _p(vd), _p(out), C.c_int64(320), C.c_float(-0.1), _stream()) == 0
    torch.cuda.synchronize()
    want = O.round_bf16(state + np.float32(-0.1) * vel)
    assert np.abs(_bf16(out) - want).max() <= 2.0 ** -7 * np.abs(want).max()
    assert torch.equal(sd.cpu(), torch.from_numpy(state).to(torch.bfloat16))  # input untouched
    table = O.round_bf16(rng.standard_normal((100, 256)).astype(np.float32))
    ids = np.array([3, 99, 100, 7], dtype=np.uint32)  # 100 is out of vocabulary -> zeros
    td = torch.from_numpy(table).to(torch.bfloat16).cuda()
    idd = torch.from_numpy(ids.view(np.int32)).cuda()
    emb = torch.full((4, 256), 9.0, dtype=torch.bfloat16, device="cuda")
    assert _lib().apxinf_static_embedding_bf16(_p(td), _p(idd), _p(emb), 4, 256, 100, _stream()) == 0
    torch.cuda.synchronize()
    want = O.round_bf16(table[[3, 99, 0, 7]] * np.sqrt(np.float32(256)))
    want[2] = 0
    assert np.array_equal(_bf16(emb), want)


def test_bf16_gemm_row_major_weight():
    # crates/apxinf-cuda/src/tests/bf16.rs:59-74 tolerance: max_abs <= 0.125, rmse <= 0.02
    lib = _lib()
    rng = np.random.default_rng(5)
    m, n, k = 522, 2560, 2048
    a = O.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = O.round_bf16(0.02 * rng.standard_normal((k, n)).astype(np.float32))
    ad = torch.from_numpy(a).to(torch.bfloat16).cuda()
    wd = torch.from_numpy(w).to(torch.bfloat16).cuda()
    out = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    assert lib.apxinf_static_prepare_bf16_gemm(m, n, k) == 0
    assert lib.apxinf_static_bf16_gemm(_p(ad), _p(wd), _p(out), m, n, k, C.c_float(1.0), _stream()) == 0
    torch.cuda.synchronize()
    want = a @ w
    err = _bf16(out) - want
    assert np.abs(err).max() <= 0.125 and np.sqrt((err ** 2).mean()) <= 0.02
    assert lib.apxinf_static_bf16_gemm(None, _p(wd), _p(out), m, n, k, C.c_float(1.0), _stream()) == 7


def _softmax_attention(q, k, v):
    """float64 restatement of kernels/custom/attention.cuh:761-870 (scores * rsqrt(head_dim),
    softmax over keys, probabilities times values)."""
    s = np.einsum("...qd,...kd->...qk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(q.shape[-1])
    s -= s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("...qk,...kd->...qd", p, v.astype(np.float64))


@pytest.mark.parametrize("symbol", ["apxinf_static_mqa_bf16", "apxinf_static_cublas_mqa_bf16"])
def test_mqa_bf16_under_the_reference_names(symbol):
    # crates/apxinf-cuda/src/tests/bf16.rs: MQA over one K/V head, q [tokens, heads, head_dim]
    tokens, keys, heads, hd = 13, 300, 8, 256
    rng = np.random.default_rng(5)
    q = torch.from_numpy(rng.standard_normal((tokens, heads, hd)).astype(np.float32)).to(torch.bfloat16)
    k = torch.from_numpy(rng.standard_normal((keys, hd)).astype(np.float32)).to(torch.bfloat16)
    v = torch.from_numpy(rng.standard_normal((keys, hd)).astype(np.float32)).to(torch.bfloat16)
    out = torch.zeros(tokens, heads, hd, dtype=torch.bfloat16, device="cuda")
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    rc = getattr(_lib(), symbol)(_p(dq), _p(dk), _p(dv), _p(out), tokens, keys, heads, hd, _stream())
    torch.cuda.synchronize()
    assert rc == 0
    want = _softmax_attention(_bf16(q).transpose(1, 0, 2), _bf16(k)[None], _bf16(v)[None]).transpose(1, 0, 2)
    assert np.abs(_bf16(out) - want).max() <= 0.02


def test_mha_bf16_under_the_reference_name():
    tokens, batches, heads, hd = 256, 2, 4, 72
    rng = np.random.default_rng(6)
    shape = (batches * tokens, heads, hd)
    q, k, v = (torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(torch.bfloat16) for _ in range(3))
    out = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    rc = _lib().apxinf_static_mha_bf16(_p(dq), _p(dk), _p(dv), _p(out), tokens, batches, heads, hd, _stream())
    torch.cuda.synchronize()
    assert rc == 0

    def split(t):  # [batches, heads, tokens, hd]
        return _bf16(t).reshape(batches, tokens, heads, hd).transpose(0, 2, 1, 3)

    want = _softmax_attention(split(q), split(k), split(v)).transpose(0, 2, 1, 3).reshape(shape)
    assert np.abs(_bf16(out) - want).max() <= 0.02


def test_static_attention_rejects_what_the_kernel_cannot_do():
    t = torch.zeros(8, 8, 64, dtype=torch.bfloat16, device="cuda")
    assert _lib().apxinf_static_mqa_bf16(_p(t), _p(t), _p(t), _p(t), 8, 5000, 8, 64, _stream()) == 1
    assert _lib().apxinf_static_cublas_mqa_bf16(_p(t), _p(t), _p(t), _p(t), 8, 5000, 8, 64, _stream()) == 7
    assert _lib().apxinf_static_mha_bf16(None, _p(t), _p(t), _p(t), 8, 1, 8, 64, _stream()) == 1
