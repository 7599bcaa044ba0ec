"""Pins the CPU oracle to the known-answer vectors the reference's own tests hold for
the PI0.5 path (file:line of each vector beside the case)."""
import math

import numpy as np

from oracle import pi05_oracle as O

F = np.float32


def test_e4m3_canonical_bytes():
    # crates/apxinf-model/src/pi05/fp8.rs:192-201
    enc = lambda v: int(O.e4m3_encode(np.array([v], dtype=F))[0])
    assert enc(0.0) == 0x00 and enc(-0.0) == 0x80
    assert enc(1.0) == 0x38 and enc(-1.0) == 0xB8 and enc(448.0) == 0x7E
    assert O.e4m3_decode(np.array([0x01], np.uint8))[0] == F(2.0 ** -9)
    assert O.e4m3_decode(np.array([0x7E], np.uint8))[0] == F(448.0)
    assert np.isnan(O.e4m3_decode(np.array([0x7F], np.uint8))[0])


def test_e4m3_saturation_and_ties_to_even():
    # crates/apxinf-model/src/pi05/fp8.rs:203-211
    enc = lambda v: int(O.e4m3_encode(np.array([v], dtype=F))[0])
    assert enc(np.inf) == 0x7E and enc(1000.0) == 0x7E
    assert enc(1.0625) == 0x38
    assert enc(1.1875) == 0x3A
    assert enc(np.nan) == 0x7F


def test_e4m3_round_trip_every_byte():
    finite = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=np.uint8)
    values = O.e4m3_decode(finite)
    assert np.array_equal(O.e4m3_encode(values), finite)
    assert np.array_equal(O.e4m3_round(values), values)


def test_e4m3_absmax_quantisation():
    # crates/apxinf-model/src/pi05/fp8.rs:213-225: [-2,-.5,.5,2] -> scale 2/448, ends saturate
    w = np.array([[-2.0], [-0.5], [0.5], [2.0]], dtype=F)
    q, scale = O.quantize_e4m3_channels(w)
    assert abs(float(scale[0]) - 2.0 / 448.0) < 1e-9
    assert q[0, 0] == -448.0 and q[3, 0] == 448.0


def test_int8_output_channel_quantiser():
    # crates/apxinf-model/src/pi05/int8_weights.rs:142-158
    w = np.array([[1.0, -10.0], [2.0, 0.0], [3.0, 10.0]], dtype=F)   # [in=3, out=2]
    q, scales = O.quantize_int8_channels(w)
    assert q.T.astype(int).ravel().tolist() == [42, 85, 127, -127, 0, 127]  # output-major
    assert abs(float(scales[0]) - 3.0 / 127.0) < 1e-7 and abs(float(scales[1]) - 10.0 / 127.0) < 1e-7
    q, scales = O.quantize_int8_channels(np.zeros((2, 1), dtype=F))
    assert q.ravel().tolist() == [0, 0] and scales.tolist() == [F(1.0e-12)]


def test_w8a8_small_reference_case():
    # crates/apxinf-cuda/src/tests/w8a8.rs:46-80: expected [6, 0, 2, -4] within 0.05
    act = np.array([[1, 2, 3, 4], [-1, 0, 1, 2]], dtype=F)
    w_out_major = np.array([[1, 0, -1, 2], [2, 1, 0, -1]], dtype=F)
    xq, rs = O.quantize_rows_int8(act)
    acc = O._chunked_int_matmul(xq, w_out_major.T)
    out = O.round_bf16((acc.astype(F) * rs[:, None]) * np.ones(2, dtype=F)[None, :])
    assert np.all(np.abs(out.ravel() - np.array([6.0, 0.0, 2.0, -4.0])) <= 0.05)


def test_time_embedding_endpoints_and_euler_sign():
    # crates/apxinf-model/src/pi05/math.rs:65-92
    emb = O.sinusoidal_time_embedding(0.0, 8, 4e-3, 4.0)
    assert np.array_equal(emb[:4], np.zeros(4, F)) and np.array_equal(emb[4:], np.ones(4, F))
    x = np.array([1.0, -1.0], dtype=F)
    v = np.array([2.0, -4.0], dtype=F)
    x = x + (F(-1.0) / F(10)) * v
    assert abs(x[0] - 0.8) < 1e-6 and abs(x[1] + 0.6) < 1e-6
    assert np.array_equal(O.flow_times(4), np.array([1.0, 0.75, 0.5, 0.25], dtype=F))


def test_patchify_matches_kernel_index_formula():
    # crates/apxinf-cuda/kernels/custom/preprocess.cuh:65-98, on the reference's arithmetic
    # image pattern (crates/apxinf-model/examples/pi05_bench.rs:424-426)
    cfg = O.tiny_config(image_size=28, num_views=2)
    images = O.reference_image_pattern(cfg)
    got = O.patchify(images, cfg)
    ps, side, area = cfg.patch_size, cfg.patches_per_side, cfg.patch_size ** 2
    rng = np.random.default_rng(0)
    for _ in range(500):
        row = int(rng.integers(0, got.shape[0]))
        col = int(rng.integers(0, got.shape[1]))
        view, inview = divmod(row, side * side)
        py, px = divmod(inview, side)
        ch, pix = divmod(col, area)
        dy, dx = divmod(pix, ps)
        raw = images[view, py * ps + dy, px * ps + dx, ch]
        assert got[row, col] == F(raw) / F(255.0) * F(2.0) - F(1.0)
    assert images.ravel()[:4].tolist() == [19, 92, 165, 238]


def test_zero_query_attention_averages_values():
    # crates/apxinf-cuda/src/tests/fp8.rs:735-778: 16 prefix + 4 suffix keys, zero q/k,
    # v[token] = token  ->  every output 9.5
    cfg = O.tiny_config()
    oracle = O.Pi05Oracle(cfg, O.SyntheticWeights(cfg, 0), O.OracleOptions())
    q = np.zeros((4, 8, 256), dtype=F)
    k = np.zeros((20, 1, 256), dtype=F)
    v = np.repeat(np.arange(20, dtype=F)[:, None, None], 256, axis=2)
    for rounded in (False, True):
        out = oracle.attention(q, k, v, 1.0 / 16.0, rounded)
        assert np.all(np.abs(out - 9.5) < 0.01 + 0.05 * rounded)


def test_synthetic_stream_matches_scalar_lcg():
    # crates/apxinf-model/src/pi05/weights.rs:332-357, evaluated one element at a time
    seed = 7
    state = (seed ^ O.LCG_SEED_XOR) & O.MASK64
    scalar = []
    for _ in range(2500):
        state = (state * O.LCG_A + O.LCG_C) & O.MASK64
        unit = F(state >> 33) / F(2 ** 31)
        scalar.append((unit * F(2.0) - F(1.0)) * F(0.02))
    scalar = O.round_bf16(np.array(scalar, dtype=F))
    assert np.array_equal(O.lcg_values(seed, 0, 2500), scalar)
    assert np.array_equal(O.lcg_values(seed, 1777, 500), scalar[1777:2277])
    assert np.all(np.abs(scalar) <= 0.0201)  # 0.02 itself rounds up in bf16


def test_synthetic_layout_follows_generation_order():
    # crates/apxinf-model/src/pi05/weights.rs:264-327 and the GEMM table of
    # crates/apxinf-model/src/pi05/schedule.rs:63-200 (full-size architecture)
    cfg = O.Pi05Config()
    layout = O.synthetic_layout(cfg)
    names = [n for n in layout if n != "__total__"]
    assert names[0] == "vision.0.q.weight" and names[1] == "vision.0.q.bias"
    assert names.index("vision.patch_embedding.weight") > names.index("vision.26.fc2.bias")
    assert names.index("token_embedding") < names.index("language.0.q.weight")
    assert names[-1] == "time_mlp_out.bias"
    assert layout["language.0.gate.weight"][1] == (2048, 16384)
    assert layout["action.0.input_style.weight"][1] == (1024, 3072)
    assert layout["vision.patch_embedding.weight"][1] == (588, 1152)
    linear = sum(int(np.prod(s)) for n, (o, s) in layout.items()
                 if n.endswith(".weight") and "style" not in n and "time" not in n)
    # 414.1 M vision + 1,877 M language (last layer's tail included: +~170 M) + 311.5 M action
    assert 2.55e9 < linear < 2.85e9
    offsets = [layout[n][0] for n in names]
    assert offsets == sorted(offsets)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38], dtype=F)
    got = O.round_bf16(x)
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == F(1.015625) and got[3] == -1.0
    assert np.array_equal(O.bf16_from_bits(O.bf16_bits(x)), got)


def test_decoder_layer_with_zero_weights_is_identity():
    # crates/apxinf-model/src/pi05/fp8_executor.rs:499-597: zero projections leave the
    # residual stream bit-exact
    class Zero(O.SyntheticWeights):
        def get(self, name):
            _, shape = self.layout[name]
            return np.zeros(shape, dtype=F)
    cfg = O.tiny_config()
    for dtype in ("bf16", "fp8", "int8"):
        oracle = O.Pi05Oracle(cfg, Zero(cfg, 0), O.OracleOptions(dtype=dtype, collect=True))
        prefix = O.round_bf16(np.random.default_rng(1).standard_normal((12, cfg.language.width)).astype(F))
        oracle.prefix_forward(prefix)
        assert np.array_equal(oracle.trace["language.0.hidden"], prefix)


def test_three_precisions_agree_on_tiny_model():
    cfg = O.tiny_config()
    images, tokens, noise = O.synthetic_observation(cfg, 1, 6)
    ref = O.infer(cfg, 0, images, tokens, noise, dtype="bf16")
    assert np.isfinite(ref).all()
    for dtype in ("fp8", "int8"):
        m = O.compare(O.infer(cfg, 0, images, tokens, noise, dtype=dtype), ref)
        assert m["cosine"] > 0.99, (dtype, m)
    # declared deltas from the reference's FP8 flavour stay inside the FP8 tolerance
    alt = O.infer(cfg, 0, images, tokens, noise, dtype="fp8", storage="f16", fp8_weight_scale="tensor")
    assert O.compare(alt, ref)["cosine"] > 0.99
