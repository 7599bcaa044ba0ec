"""ctypes loader for oracle/build/libcpu_block.so and a NumPy twin of the same block
(test infrastructure only). `make -C oracle` builds the library."""
from __future__ import annotations

import ctypes as C
import subprocess
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "build" / "libcpu_block.so"
F = np.float32


def load() -> C.CDLL:
    if not LIB.exists():
        subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    lib = C.CDLL(str(LIB))
    fp = C.POINTER(C.c_float)
    lib.cpu_block_forward.argtypes = [fp] * 10 + [C.c_int] * 6 + [C.c_float, C.c_float, C.c_int, C.c_int, fp]
    lib.cpu_block_forward.restype = C.c_int
    return lib


def make_case(seed: int, seq: int, hidden: int, heads: int, kv_heads: int, head_dim: int, mlp: int):
    """Config-1 style inputs: activations N(0,1) f32, weights N(0, 0.02) rounded to bf16, norms 1."""
    from . import pi05_oracle as O
    rng = np.random.default_rng(seed)
    w = lambda a, b: O.round_bf16((0.02 * rng.standard_normal((a, b))).astype(F))
    qw, kw = heads * head_dim, kv_heads * head_dim
    return dict(x=rng.standard_normal((seq, hidden)).astype(F), attn_norm=np.ones(hidden, F),
                wq=w(hidden, qw), wk=w(hidden, kw), wv=w(hidden, kw), wo=w(qw, hidden),
                ffn_norm=np.ones(hidden, F), w_gate=w(hidden, mlp), w_up=w(hidden, mlp),
                w_down=w(mlp, hidden))


def run_c(case, heads, kv_heads, head_dim, theta=10000.0, eps=1e-6, causal=True, gelu=True):
    lib = load()
    seq, hidden = case["x"].shape
    mlp = case["w_gate"].shape[1]
    out = np.empty((seq, hidden), dtype=F)
    ptr = lambda a: np.ascontiguousarray(a, dtype=F).ctypes.data_as(C.POINTER(C.c_float))
    keep = [np.ascontiguousarray(case[k], dtype=F) for k in
            ("x", "attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "w_gate", "w_up", "w_down")]
    t0 = time.perf_counter()
    rc = lib.cpu_block_forward(*[ptr(a) for a in keep], seq, hidden, heads, kv_heads, head_dim, mlp,
                               C.c_float(theta), C.c_float(eps), int(causal), int(gelu),
                               out.ctypes.data_as(C.POINTER(C.c_float)))
    seconds = time.perf_counter() - t0
    assert rc == 0
    return out, seconds


def run_numpy(case, heads, kv_heads, head_dim, theta=10000.0, eps=1e-6, causal=True, gelu=True):
    from . import pi05_oracle as O
    x = case["x"]
    seq, hidden = x.shape

    def rms(a, w):
        return (a / np.sqrt((a * a).mean(axis=1, keepdims=True, dtype=F) + F(eps))) * w

    def rope(t, n):
        half = head_dim // 2
        freqs = (F(1.0) / np.power(F(theta), F(2.0) * np.arange(half, dtype=F) / F(head_dim))).astype(F)
        ang = (np.arange(seq, dtype=F)[:, None] * freqs[None, :]).astype(F)
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        t = t.reshape(seq, n, head_dim)
        a, b = t[..., :half], t[..., half:]
        return np.concatenate([a * c - b * s, a * s + b * c], axis=-1).astype(F)

    n = rms(x, case["attn_norm"])
    q, k = rope(n @ case["wq"], heads), rope(n @ case["wk"], kv_heads)
    v = (n @ case["wv"]).reshape(seq, kv_heads, head_dim)
    attn = np.zeros((seq, heads, head_dim), dtype=F)
    mask = np.tril(np.ones((seq, seq), dtype=bool)) if causal else np.ones((seq, seq), dtype=bool)
    for h in range(heads):
        kh = h * kv_heads // heads
        s = (q[:, h] @ k[:, kh].T) / np.sqrt(F(head_dim))
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        attn[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, kh]
    h1 = x + attn.reshape(seq, -1) @ case["wo"]
    n2 = rms(h1, case["ffn_norm"])
    gate = n2 @ case["w_gate"]
    gate = O.gelu_tanh(gate) if gelu else O.silu(gate)
    return (h1 + (gate * (n2 @ case["w_up"])) @ case["w_down"]).astype(F)
