"""Kernel-level operators over the C ABI, taking torch CUDA tensors as device memory.

torch only supplies memory and the stream handle here; every operator is a
hand-written CUDA kernel in libpi05_b200.so.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import GemmArgs, check, lib


def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def _ptr(t) -> int | None:
    return None if t is None else int(t.data_ptr())


def _operand(t: torch.Tensor):
    """(rows, k, ld, nb0, nb1, sb0, sb1) of a [.., rows, k] tensor (innermost contiguous)."""
    assert t.stride(-1) == 1, "innermost dimension must be contiguous"
    rows, k = t.shape[-2], t.shape[-1]
    ld = t.stride(-2)
    nb0 = t.shape[-3] if t.dim() >= 3 else 1
    sb0 = t.stride(-3) if t.dim() >= 3 else 0
    nb1 = t.shape[-4] if t.dim() >= 4 else 1
    sb1 = t.stride(-4) if t.dim() >= 4 else 0
    return rows, k, ld, nb0, nb1, sb0, sb1


def new_status(device="cuda") -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def gemm(a, b, out, *, op, mode=_lib.EPI_STORE, out_type=_lib.OUT_BF16, bias=None,
         residual=None, col_scale=None, row_scale=None, pos=None, gate=None, alpha=1.0,
         out_inv_scale=1.0, b_mn_major=False, status=None, stream=None, force_swap=-1,
         force_block_n=0, partials=None, tile_counters=None, force_split_k=0,
         static_scratch=False, b_blocked=None, force_skinny=-1, prologue=0, style=None, eps=1e-6,
         a_inv_scale=1.0, a_dynamic_rows=False, rope=None, dt=0.0, k_slices=0):
    """out[.., M, N'] = epilogue(a[.., M, K] @ b[.., N, K]^T); see Pi05GemmArgs.
    `rope`: dict(q_out, k_cache, v_cache, cos, sin, tokens, q_heads, head_dim, position_offset,
    cache_rows) for mode EPI_ROPE."""
    m, k, lda, nb0, nb1, a_sb0, a_sb1 = _operand(a)
    if b_blocked is not None:
        # b is [ceil(K / kb), N, kb]; the logical (N, K) comes with it
        n, kb = b_blocked
        ldb, b_sb0, b_sb1 = 0, 0, 0
    elif b_mn_major:
        kb, n, ldb, _, _, b_sb0, b_sb1 = _operand(b)
    else:
        n, kb, ldb, _, _, b_sb0, b_sb1 = _operand(b)
    assert kb == k, (kb, k)
    _, _, ldc, _, _, o_sb0, o_sb1 = _operand(out)
    if status is None:
        status = new_status(a.device)
    args = GemmArgs(
        op=op, m=m, n=n, k=k, nb0=nb0, nb1=nb1,
        a=_ptr(a), lda=lda, a_sb0=a_sb0, a_sb1=a_sb1,
        b=_ptr(b), ldb=ldb, b_sb0=b_sb0, b_sb1=b_sb1, b_mn_major=int(b_mn_major),
        out=_ptr(out), ldc=ldc, out_sb0=o_sb0, out_sb1=o_sb1,
        out_type=out_type, mode=mode,
        residual=_ptr(residual), bias=_ptr(bias), col_scale=_ptr(col_scale),
        row_scale=_ptr(row_scale), pos=_ptr(pos),
        pos_rows=(pos.shape[0] if pos is not None else 1),
        pos_ld=(pos.stride(0) if pos is not None else 0),
        gate=_ptr(gate), alpha=alpha, out_inv_scale=out_inv_scale, status=_ptr(status),
        force_swap=force_swap, force_block_n=force_block_n,
        partials=_ptr(partials),
        partials_bytes=(partials.numel() * partials.element_size() if partials is not None else 0),
        tile_counters=_ptr(tile_counters),
        max_tiles=(tile_counters.numel() if tile_counters is not None else 0),
        force_split_k=force_split_k,
        b_blocked=int(b_blocked is not None), force_skinny=force_skinny, prologue=prologue,
        style=_ptr(style), eps=eps, a_inv_scale=a_inv_scale, a_dynamic_rows=int(a_dynamic_rows), dt=dt,
        k_slices=k_slices)
    if rope is not None:
        args.rope_q_out, args.rope_k_cache, args.rope_v_cache = (_ptr(rope["q_out"]), _ptr(rope["k_cache"]),
                                                                 _ptr(rope["v_cache"]))
        args.rope_cos, args.rope_sin = _ptr(rope["cos"]), _ptr(rope["sin"])
        args.rope_tokens, args.rope_q_heads, args.rope_head_dim = rope["tokens"], rope["q_heads"], rope["head_dim"]
        args.rope_position_offset, args.rope_cache_rows = rope["position_offset"], rope["cache_rows"]
    if static_scratch:
        check(lib().pi05_gemm_static_scratch(C.byref(args), _stream_ptr(stream)),
              "pi05_gemm_static_scratch")
    else:
        check(lib().pi05_gemm(C.byref(args), _stream_ptr(stream)), "pi05_gemm")
    return status
