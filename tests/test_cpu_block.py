"""The C restatement of the reference's CPU decoder block (BASELINE configuration 1: Gemma-style
block, 8 query heads / 1 KV head, head_dim 256, RoPE base 1e4, GeGLU, pre-RMSNorm eps 1e-6, causal)
against an independent NumPy evaluation, at a size that runs in a second."""
import numpy as np

from oracle import cpu_block


def test_c_block_matches_numpy_small_gemma_shape():
    heads, kv_heads, head_dim = 8, 1, 32
    case = cpu_block.make_case(0, seq=24, hidden=64, heads=heads, kv_heads=kv_heads, head_dim=head_dim, mlp=128)
    got, _ = cpu_block.run_c(case, heads, kv_heads, head_dim)
    want = cpu_block.run_numpy(case, heads, kv_heads, head_dim)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())


def test_c_block_causal_mask_and_silu_variant():
    heads, kv_heads, head_dim = 4, 2, 16
    case = cpu_block.make_case(1, seq=9, hidden=32, heads=heads, kv_heads=kv_heads, head_dim=head_dim, mlp=64)
    for causal in (True, False):
        for gelu in (True, False):
            got, _ = cpu_block.run_c(case, heads, kv_heads, head_dim, causal=causal, gelu=gelu)
            want = cpu_block.run_numpy(case, heads, kv_heads, head_dim, causal=causal, gelu=gelu)
            assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
    # causality: the first token's output does not depend on later tokens
    a, _ = cpu_block.run_c(case, heads, kv_heads, head_dim)
    other = dict(case)
    other["x"] = case["x"].copy()
    other["x"][5:] += 1.0
    b, _ = cpu_block.run_c(other, heads, kv_heads, head_dim)
    assert np.array_equal(a[:5], b[:5]) and not np.array_equal(a[5:], b[5:])
