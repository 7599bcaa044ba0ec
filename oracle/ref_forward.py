"""The reference's OWN CUDA code run as a whole PI0.5 forward - TEST INFRASTRUCTURE ONLY.

The reference host (Rust) cannot be built in this image, but everything it launches on the
GPU is plain CUDA C++ behind extern "C" adapters, and those compile (oracle/Makefile ->
oracle/_ref). This module replays the executors' call lists over those libraries, op by op
and in the executors' order, on torch-owned device memory:

  BF16 graph  crates/apxinf-model/src/pi05/bf16_executor.rs:24-212 (language / action / vision
              layers) and bf16_runtime.rs:158-387 (encode_vision, embed_prefix, prefix_forward,
              conditioning / styles, denoise steps)
  GEMMs       the default path of kernels/gemm/bf16.rs:439-452 = cublasGemmEx through
              CublasHandle::gemm (src/cublas.rs:228-320): column-major N,N with the weight as
              the first operand, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT
  attention   prefix / action MQA = apxinf_static_cublas_mqa_bf16 (adapters/cublas_adapter.cu:
              89-132, the sm_100 choice of kernels/attention.rs:656-659); SigLIP MHA = the
              fallback kernel apxinf_static_mha_bf16 (the CUTLASS FMHA translation unit is
              left out, see oracle/Makefile)
  row ops     adapters/static_bf16_adapter.cu

Two uses: a second whole-model oracle that pins the ORDER of the ops and the rounding points
between them (tests compare it with oracle/pi05_oracle.py and with this repository's
library), and the "reference kernels on this box" baseline bench.py reports (stage times of
the eager B=1 forward, and single-op times of the FP8 / BF16 GEMMs and the MQA at the model's
shapes through adapters/cublaslt_adapter.cu and cublas_adapter.cu).
torch supplies device memory, streams and events only; no torch operator computes anything
that is compared.
"""
from __future__ import annotations

import ctypes as C
import math
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

from . import pi05_oracle as O

_DIR = Path(__file__).resolve().parent / "_ref"
_LIBS = {
    "bf16": "libref_static_bf16_adapter.so",
    "f16": "libref_custom_kernels.so",
    "cublas_mqa": "libref_cublas_adapter.so",
    "cublaslt": "libref_cublaslt_adapter.so",
}
_handles: Dict[str, C.CDLL] = {}

CUDA_R_16F, CUDA_R_16BF, CUDA_R_32F = 2, 14, 0
CUBLAS_OP_N = 0
CUBLAS_COMPUTE_32F = 68
CUBLAS_GEMM_DEFAULT = -1


def available() -> bool:
    return all((_DIR / name).exists() for name in _LIBS.values())


def lib(which: str) -> C.CDLL:
    if which not in _handles:
        if which == "cublaslt":
            # the cuBLASLt adapter calls the L2-eviction helper defined in the custom-kernel adapter
            C.CDLL(str(_DIR / _LIBS["f16"]), mode=C.RTLD_GLOBAL)
        _handles[which] = C.CDLL(str(_DIR / _LIBS[which]))
    return _handles[which]


def _cublas() -> C.CDLL:
    if "cublas" not in _handles:
        _handles["cublas"] = C.CDLL("libcublas.so.12")
    return _handles["cublas"]


def _p(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# ---------------------------------------------------------------------------
# Pi05Weights::synthetic on the GPU (weights.rs:332-357), in the reference's [in, out] layout
# ---------------------------------------------------------------------------

_lcg_gpu_tables = None


def lcg_values_gpu(seed: int, offset: int, count: int) -> torch.Tensor:
    """Elements [offset, offset + count) of SyntheticRng(seed) as a bf16 CUDA tensor: the
    block jump-ahead of oracle.pi05_oracle.lcg_values with int64 wrap-around on the device."""
    global _lcg_gpu_tables
    block = O._LCG_BLOCK
    if _lcg_gpu_tables is None:
        ta, tc = O._lcg_block_tables()
        _lcg_gpu_tables = (torch.from_numpy(ta.view(np.int64)).cuda(), torch.from_numpy(tc.view(np.int64)).cuda())
    ta, tc = _lcg_gpu_tables
    state0 = (seed ^ O.LCG_SEED_XOR) & O.MASK64
    out = torch.empty(count, dtype=torch.bfloat16, device="cuda")
    for b in range(0, count, block):
        take = min(block, count - b)
        ja, jc = O.lcg_jump(offset + b)
        state = (ja * state0 + jc) & O.MASK64
        signed = state - (1 << 64) if state >= (1 << 63) else state
        s = ta[:take] * signed + tc[:take]  # int64 arithmetic wraps
        bits = (s >> 33) & 0x7FFFFFFF
        unit = bits.to(torch.float32) / 2147483648.0
        out[b:b + take] = ((unit * 2.0 - 1.0) * 0.02).to(torch.bfloat16)
    return out


class RefWeights:
    """Synthetic weights as the reference holds them on the device: BF16, linear weights
    [in, out] row-major, q|k|v and gate|up packed along the output dimension
    (bf16_weights.rs:27-102)."""

    def __init__(self, cfg: O.Pi05Config, seed: int):
        self.cfg, self.seed = cfg, seed
        self.layout = O.synthetic_layout(cfg)
        self._cache: Dict[str, torch.Tensor] = {}

    def get(self, name: str) -> torch.Tensor:
        if name not in self._cache:
            offset, shape = self.layout[name]
            self._cache[name] = lcg_values_gpu(self.seed, offset, int(np.prod(shape))).view(*shape)
        return self._cache[name]

    def packed(self, names: List[str]) -> torch.Tensor:
        key = "+".join(names)
        if key not in self._cache:
            self._cache[key] = torch.cat([self.get(n + ".weight") for n in names], dim=1).contiguous()
            for n in names:
                self._cache.pop(n + ".weight", None)
        return self._cache[key]

    def packed_bias(self, names: List[str]) -> Optional[torch.Tensor]:
        if (names[0] + ".bias") not in self.layout:
            return None
        key = "+".join(names) + ".bias"
        if key not in self._cache:
            self._cache[key] = torch.cat([self.get(n + ".bias") for n in names]).contiguous()
        return self._cache[key]

    def embedding_rows(self, ids) -> torch.Tensor:
        offset, shape = self.layout["token_embedding"]
        width = shape[1]
        return torch.stack([lcg_values_gpu(self.seed, offset + int(i) * width, width) for i in ids])


# ---------------------------------------------------------------------------
# the BF16 forward
# ---------------------------------------------------------------------------


class RefBf16Forward:
    def __init__(self, cfg: O.Pi05Config, seed: int):
        assert available(), "oracle/_ref is not built (make -C oracle)"
        self.cfg = cfg
        self.w = RefWeights(cfg, seed)
        self.ops = lib("bf16")
        self.mqa = lib("cublas_mqa")
        self.blas = _cublas()
        self.handle = C.c_void_p()
        rc = self.blas.cublasCreate_v2(C.byref(self.handle))
        assert rc == 0, rc
        self.launches = 0
        self.ones: Dict[int, torch.Tensor] = {}
        self.zeros: Dict[int, torch.Tensor] = {}

    def close(self):
        if self.handle:
            self.blas.cublasDestroy_v2(self.handle)
            self.handle = C.c_void_p()

    # ---- single ops (names = the Rust wrappers the executors call) ----
    def _new(self, *shape):
        return torch.empty(*shape, dtype=torch.bfloat16, device="cuda")

    def _unit(self, n, value):
        table = self.ones if value == 1 else self.zeros
        if n not in table:
            table[n] = torch.full((n,), float(value), dtype=torch.bfloat16, device="cuda")
        return table[n]

    def _cuda(self, name, *args):
        rc = getattr(self.ops, name)(*args, _stream())
        assert rc == 0, (name, rc)
        self.launches += 1

    def gemm(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """gemm::bf16 default path: CublasHandle::gemm -> cublasGemmEx (cublas.rs:228-320)."""
        m, k = a.shape
        n = w.shape[1]
        assert w.shape[0] == k and a.is_contiguous() and w.is_contiguous()
        out = self._new(m, n)
        alpha, beta = C.c_float(1.0), C.c_float(0.0)
        rc = self.blas.cublasSetStream_v2(self.handle, _stream())
        assert rc == 0, rc
        rc = self.blas.cublasGemmEx(
            self.handle, CUBLAS_OP_N, CUBLAS_OP_N, n, m, k, C.byref(alpha),
            _p(w), CUDA_R_16BF, n, _p(a), CUDA_R_16BF, k, C.byref(beta),
            _p(out), CUDA_R_16BF, n, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT)
        assert rc == 0, ("cublasGemmEx", rc, m, n, k)
        self.launches += 1
        return out

    def bias(self, x, bias, activation=0):
        """elementwise::bias_bf16 / activation::bias_{gelu,silu}_bf16 (activation.rs:133-160);
        activation codes of custom/activation.cuh: 0 identity, 1 GELU-tanh, 2 SiLU."""
        out = self._new(*x.shape)
        self._cuda("apxinf_static_bias_activation_bf16", _p(x), _p(bias), _p(out), x.shape[0], x.shape[1],
                   activation)
        return out

    def layer_norm(self, x):
        cols = x.shape[1]
        out = self._new(*x.shape)
        self._cuda("apxinf_static_layer_norm_bf16", _p(x), _p(self._unit(cols, 1)), _p(self._unit(cols, 0)),
                   _p(out), x.shape[0], cols, C.c_float(self.cfg.layer_norm_eps))
        return out

    def rms_norm(self, x):
        cols = x.shape[1]
        out = self._new(*x.shape)
        self._cuda("apxinf_static_rms_norm_bf16", _p(x), _p(self._unit(cols, 1)), _p(out), x.shape[0], cols,
                   C.c_float(self.cfg.rms_norm_eps))
        return out

    # ---- stages ----
    def encode_vision(self, images_u8: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        views, pp, vw = cfg.num_views, cfg.patches_per_view, cfg.vision_width
        rows = views * pp
        patches = self._new(rows, cfg.patch_width)
        self._cuda("apxinf_static_rgb_u8_to_patches_bf16", _p(images_u8), _p(patches), views, cfg.image_size,
                   cfg.patch_size, 0)
        proj = self.gemm(patches, w.get("vision.patch_embedding.weight"))
        x = self._new(rows, vw)
        self._cuda("apxinf_static_bias_position_bf16", _p(proj), _p(w.get("vision.patch_embedding.bias")),
                   _p(w.get("vision.position_embedding")), _p(x), rows, vw, pp)
        heads, hd = cfg.vision_heads, cfg.vision_head_dim
        eps = C.c_float(cfg.layer_norm_eps)
        for i in range(cfg.vision_depth):
            p = f"vision.{i}"
            names = [p + ".q", p + ".k", p + ".v"]
            n = self.layer_norm(x)
            qkv = self.gemm(n, w.packed(names))
            q, k, v = self._new(rows, vw), self._new(rows, vw), self._new(rows, vw)
            self._cuda("apxinf_static_qkv_split_bias_bf16", _p(qkv), _p(w.packed_bias(names)), _p(q), _p(k),
                       _p(v), rows, vw)
            attn = self._new(rows, vw)
            self._cuda("apxinf_static_mha_bf16", _p(q), _p(k), _p(v), _p(attn), pp, views, heads, hd)
            proj = self.gemm(attn, w.get(p + ".o.weight"))
            hidden, normalized = self._new(rows, vw), self._new(rows, vw)
            self._cuda("apxinf_static_bias_residual_layer_norm_bf16", _p(proj), _p(w.get(p + ".o.bias")), _p(x),
                       _p(self._unit(vw, 1)), _p(self._unit(vw, 0)), _p(hidden), _p(normalized), rows, vw, eps)
            f1 = self.gemm(normalized, w.get(p + ".fc1.weight"))
            act = self.bias(f1, w.get(p + ".fc1.bias"), activation=1)
            f2 = self.gemm(act, w.get(p + ".fc2.weight"))
            x = self._new(rows, vw)
            self._cuda("apxinf_static_bias_residual_bf16", _p(f2), _p(w.get(p + ".fc2.bias")), _p(hidden),
                       _p(x), rows, vw)
        n = self.layer_norm(x)
        proj = self.gemm(n, w.get("vision.projector.weight"))
        return self.bias(proj, w.get("vision.projector.bias"))

    def embed_prefix(self, vision_tokens, token_ids: np.ndarray):
        cfg = self.cfg
        width = cfg.language.width
        # a compact table holding only the rows the ids name (the full table is 1 GB of LCG output);
        # the lookup kernel itself - scaling, out-of-vocabulary zeros - is the reference's
        valid = sorted({int(t) for t in token_ids if int(t) < cfg.vocab_size})
        table = self.w.embedding_rows(valid) if valid else self._new(1, width)
        remap = {t: i for i, t in enumerate(valid)}
        local = np.array([remap.get(int(t), len(valid) + 7) for t in token_ids], dtype=np.uint32)
        ids = torch.from_numpy(local.view(np.int32)).cuda()
        language = self._new(len(token_ids), width)
        self._cuda("apxinf_static_embedding_bf16", _p(table), _p(ids), _p(language), len(token_ids), width,
                   max(len(valid), 1))
        out = self._new(vision_tokens.shape[0] + len(token_ids), width)
        self._cuda("apxinf_static_concat_rows_bf16", _p(vision_tokens), _p(language), _p(out),
                   vision_tokens.shape[0], len(token_ids), width)
        return out

    def _mqa(self, q, k, v, query_tokens, key_tokens, heads, hd):
        out = self._new(query_tokens, heads * hd)
        rc = self.mqa.apxinf_static_cublas_mqa_bf16(_p(q), _p(k), _p(v), _p(out), query_tokens, key_tokens,
                                                    heads, hd, _stream())
        assert rc == 0, ("apxinf_static_cublas_mqa_bf16", rc)
        self.launches += 3
        return out

    def prefix_forward(self, prefix):
        cfg, w, g = self.cfg, self.w, self.cfg.language
        tokens = prefix.shape[0]
        qw = g.num_heads * g.head_dim
        cache_rows = tokens + cfg.action_horizon
        eps = C.c_float(cfg.rms_norm_eps)
        hidden = prefix
        keys, values = [], []
        for i in range(g.depth):
            p = f"language.{i}"
            n = self.rms_norm(hidden)
            qkv = self.gemm(n, w.packed([p + ".q", p + ".k", p + ".v"]))
            q = self._new(tokens, qw)
            # reserve_prefix (kernels/cache.rs:111-161) copies K and V into [P + H, 256] buffers;
            # here the split kernel writes them at rows 0..P of those buffers directly
            kc = torch.zeros(cache_rows, g.head_dim, dtype=torch.bfloat16, device="cuda")
            vc = torch.zeros(cache_rows, g.head_dim, dtype=torch.bfloat16, device="cuda")
            self._cuda("apxinf_static_qkv_rope_bf16", _p(qkv), None, _p(q), _p(kc), _p(vc), tokens, g.num_heads,
                       g.num_kv_heads, g.head_dim, C.c_float(cfg.rope_theta), 0, 0)
            keys.append(kc)
            values.append(vc)
            if i + 1 == g.depth:
                break
            attn = self._mqa(q, kc, vc, tokens, tokens, g.num_heads, g.head_dim)
            proj = self.gemm(attn, w.get(p + ".o.weight"))
            h1, n2 = self._new(tokens, g.width), self._new(tokens, g.width)
            self._cuda("apxinf_static_bias_residual_rms_norm_bf16", _p(proj), None, _p(hidden),
                       _p(self._unit(g.width, 1)), _p(h1), _p(n2), tokens, g.width, eps)
            gu = self.gemm(n2, w.packed([p + ".gate", p + ".up"]))
            act = self._new(tokens, g.mlp_dim)
            self._cuda("apxinf_static_geglu_bf16", _p(gu), _p(act), tokens, g.mlp_dim)
            down = self.gemm(act, w.get(p + ".down.weight"))
            hidden = self._new(tokens, g.width)
            self._cuda("apxinf_static_bias_residual_bf16", _p(down), None, _p(h1), _p(hidden), tokens, g.width)
        self.last_hidden = hidden
        return keys, values

    def step_styles(self, step_time: float):
        cfg, w = self.cfg, self.w
        aw = cfg.action_expert.width
        emb = O.round_bf16(O.sinusoidal_time_embedding(step_time, aw, cfg.time_min_period, cfg.time_max_period))
        emb = torch.from_numpy(emb[None, :]).to(torch.bfloat16).cuda()
        hidden = self.bias(self.gemm(emb, w.get("time_mlp_in.weight")), w.get("time_mlp_in.bias"), activation=2)
        cond = self.bias(self.gemm(hidden, w.get("time_mlp_out.weight")), w.get("time_mlp_out.bias"), activation=2)

        def style(name):
            return self.bias(self.gemm(cond, w.get(name + ".weight")), w.get(name + ".bias")).view(-1)

        depth = cfg.action_expert.depth
        attention = [style(f"action.{i}.input_style") for i in range(depth)]
        mlp = [style(f"action.{i}.post_style") for i in range(depth)]
        return attention, mlp, style("action.final_style")

    def denoise(self, noise: torch.Tensor, keys, values, prefix_tokens, styles):
        cfg, w, g = self.cfg, self.w, self.cfg.action_expert
        hz, aw = cfg.action_horizon, g.width
        qw = g.num_heads * g.head_dim
        eps = C.c_float(cfg.rms_norm_eps)
        dt = C.c_float(-1.0 / cfg.num_flow_steps)
        state = noise
        for step in range(cfg.num_flow_steps):
            style_attn, style_mlp, style_final = styles[step]
            hidden = self.bias(self.gemm(state, w.get("action_in.weight")), w.get("action_in.bias"))
            normalized = None
            for i in range(g.depth):
                p = f"action.{i}"
                if normalized is None:
                    normalized = self._new(hz, aw)
                    self._cuda("apxinf_static_ada_rms_norm_bf16", _p(hidden), _p(style_attn[i]), _p(normalized),
                               hz, aw, eps)
                qkv = self.gemm(normalized, w.packed([p + ".q", p + ".k", p + ".v"]))
                q = self._new(hz, qw)
                self._cuda("apxinf_static_qkv_rope_bf16", _p(qkv), None, _p(q), _p(keys[i]), _p(values[i]), hz,
                           g.num_heads, g.num_kv_heads, g.head_dim, C.c_float(cfg.rope_theta), prefix_tokens,
                           prefix_tokens)
                attn = self._mqa(q, keys[i], values[i], hz, prefix_tokens + hz, g.num_heads, g.head_dim)
                proj = self.gemm(attn, w.get(p + ".o.weight"))
                h1, n1 = self._new(hz, aw), self._new(hz, aw)
                self._cuda("apxinf_static_ada_gate_residual_rms_norm_bf16", _p(proj), _p(hidden), _p(style_attn[i]),
                           _p(style_mlp[i]), _p(h1), _p(n1), hz, aw, eps)
                gu = self.gemm(n1, w.packed([p + ".gate", p + ".up"]))
                act = self._new(hz, g.mlp_dim)
                self._cuda("apxinf_static_geglu_bf16", _p(gu), _p(act), hz, g.mlp_dim)
                down = self.gemm(act, w.get(p + ".down.weight"))
                nxt = style_attn[i + 1] if i + 1 < g.depth else style_final
                hidden, normalized = self._new(hz, aw), self._new(hz, aw)
                self._cuda("apxinf_static_ada_gate_residual_rms_norm_bf16", _p(down), _p(h1), _p(style_mlp[i]),
                           _p(nxt), _p(hidden), _p(normalized), hz, aw, eps)
            vel = self.bias(self.gemm(normalized, w.get("action_out.weight")), w.get("action_out.bias"))
            nxt_state = self._new(hz, cfg.action_dim)
            self._cuda("apxinf_static_euler_update_bf16", _p(state), _p(vel), _p(nxt_state),
                       C.c_int64(state.numel()), dt)
            state = nxt_state
        return state

    def infer(self, images_u8: np.ndarray, token_ids: np.ndarray, noise: np.ndarray, timed: bool = False):
        """One forward; returns float32 [H, action_dim] (and, with `timed`, eager stage times in
        ms measured with CUDA events: vision, prefix, denoise; styles are prepared before, as the
        reference does at capture time)."""
        cfg = self.cfg
        images = torch.from_numpy(np.ascontiguousarray(images_u8)).cuda()
        noise_d = torch.from_numpy(O.round_bf16(noise.astype(np.float32))).to(torch.bfloat16).cuda()
        styles = [self.step_styles(float(t)) for t in O.flow_times(cfg.num_flow_steps)]
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        self.launches = 0
        marks[0].record()
        vision = self.encode_vision(images)
        prefix = self.embed_prefix(vision, token_ids)
        marks[1].record()
        keys, values = self.prefix_forward(prefix)
        marks[2].record()
        state = self.denoise(noise_d, keys, values, prefix.shape[0], styles)
        marks[3].record()
        torch.cuda.synchronize()
        self.keys, self.values = keys, values
        out = state.float().cpu().numpy()
        if timed:
            return out, {"vision": marks[0].elapsed_time(marks[1]), "prefix": marks[1].elapsed_time(marks[2]),
                         "denoise": marks[2].elapsed_time(marks[3]), "launches": self.launches}
        return out


# ---------------------------------------------------------------------------
# single-op timings of the reference's library calls at the model's shapes
# ---------------------------------------------------------------------------


def graph_time_us(launch, iters=20, replays=5):
    """Mean device time of one `launch(i)` in microseconds: `iters` launches are captured into
    one CUDA graph on a side stream (so host launch cost is out of the figure) and the graph
    is replayed `replays` times between CUDA events; the best replay counts. `launch(i)` must
    enqueue on torch's current stream and may rotate its operands with i."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for i in range(3):
            launch(i)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(iters):
            launch(i)
    best = None
    for _ in range(replays):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end)
        best = ms if best is None else min(best, ms)
    del graph
    return best * 1e3 / iters


def weight_copies(weight_bytes: int) -> int:
    """How many copies of a weight matrix a timing loop rotates through so that successive
    launches do not find their weights in the 126 MB L2 (as in the model, where the next
    layer's weights always come from HBM)."""
    return int(min(16, max(2, math.ceil((256 << 20) / max(1, weight_bytes)))))


def time_gemms(shapes, iters=20):
    """shapes: {name: (M, N, K)}. Times, per shape, the reference's FP8 linear
    (apxinf_static_fp8_gemm_f16, adapters/cublaslt_adapter.cu:1110-1171: E4M3 x E4M3 -> F16,
    prepared then run) and BF16 linear (apxinf_static_bf16_gemm, :794-883) on random operands,
    weights rotating through copies larger than L2. Returns {name: {"fp8_us", "bf16_us"}}
    (None where cuBLASLt refuses the problem)."""
    lt = lib("cublaslt")
    results = {}
    for name, (m, n, k) in shapes.items():
        entry = {}
        for label, a_dtype, out_dtype, prepare, run, alpha, elem in (
                ("fp8", torch.float8_e4m3fn, torch.float16, lt.apxinf_static_prepare_fp8_gemm_f16,
                 lt.apxinf_static_fp8_gemm_f16, 0.01, 1),
                ("bf16", torch.bfloat16, torch.bfloat16, lt.apxinf_static_prepare_bf16_gemm,
                 lt.apxinf_static_bf16_gemm, 1.0, 2)):
            copies = weight_copies(n * k * elem)
            a = torch.randn(m, k, device="cuda").to(a_dtype)
            ws = [torch.randn(k, n, device="cuda").to(a_dtype) for _ in range(copies)]
            out = torch.empty(m, n, dtype=out_dtype, device="cuda")
            rc = prepare(m, n, k)
            if rc != 0:
                entry[label + "_us"] = None
                entry[label + "_status"] = rc
                continue

            def launch(i, run=run, a=a, ws=ws, out=out, alpha=alpha):
                status = run(_p(a), _p(ws[i % len(ws)]), _p(out), m, n, k, C.c_float(alpha), _stream())
                if status != 0:
                    raise RuntimeError(f"cuBLASLt status {status}")
            try:
                entry[label + "_us"] = graph_time_us(launch, iters)
            except RuntimeError as error:
                entry[label + "_us"] = None
                entry[label + "_status"] = str(error)
            del a, ws, out
        results[name] = entry
    return results


def time_mqa(shapes, iters=20):
    """shapes: {name: (query_tokens, key_tokens, heads, head_dim)}: the reference's
    three-launch MQA (cuBLAS QK^T, warp softmax, cuBLAS PV; cublas_adapter.cu:89-132)."""
    mqa = lib("cublas_mqa")
    results = {}
    for name, (qt, kt, heads, hd) in shapes.items():
        q = torch.randn(qt, heads * hd, device="cuda").to(torch.bfloat16)
        k = torch.randn(kt, hd, device="cuda").to(torch.bfloat16)
        v = torch.randn(kt, hd, device="cuda").to(torch.bfloat16)
        out = torch.empty(qt, heads * hd, dtype=torch.bfloat16, device="cuda")

        def launch(i):
            status = mqa.apxinf_static_cublas_mqa_bf16(_p(q), _p(k), _p(v), _p(out), qt, kt, heads, hd, _stream())
            if status != 0:
                raise RuntimeError(f"cuBLAS status {status}")
        results[name] = {"us": graph_time_us(launch, iters)}
    return results
