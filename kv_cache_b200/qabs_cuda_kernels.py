"""Drop-in for the reference's ``qabs_cuda_kernels`` module (littlexi001/kv_cache,
ymluo/projects/qwen3_top2_head_limit3_ppl/src/qabs_cuda_kernels.py = QCK): the same four callables
with the same signatures and tensor layouts (QCK:654-705), served by this package's sm_100a library.

    from kv_cache_b200 import qabs_cuda_kernels            # instead of: import qabs_cuda_kernels

Differences on purpose: nothing is JIT-compiled at first use (QCK:642-651), ``key`` may be the
un-repeated ``[B,Hkv,T,D]`` cache (the reference repeats K/V to the query heads first,
EVAL:6248-6251), and a failure raises instead of being swallowed by the caller's try/except.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _native, ops
from ._native import check


_ELEM_TYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _elem_type(query: torch.Tensor, key: torch.Tensor) -> int:
    """bf16, fp16 or fp32 (the types the reference dispatches over, QCK:430-458); query and key must agree."""
    if query.dtype != key.dtype or query.dtype not in _ELEM_TYPES:
        raise RuntimeError("query and key must both be bfloat16, float16 or float32")
    return _ELEM_TYPES[query.dtype]


def partial_scores(query: torch.Tensor, key_history: torch.Tensor, dim_count: int) -> torch.Tensor:
    """``query [B,H,D]``, ``key_history [B,H|Hkv,T,D]`` (any strides) -> fp32 ``[B,H,T]`` partial scores
    over the ``dim_count`` channels with the largest ``|q|`` per (batch, head) (QCK:654-656)."""
    et = _elem_type(query, key_history)
    q = query.contiguous()
    k = key_history
    B, H, D = q.shape
    Hk, T = k.shape[1], k.shape[2]
    out = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    check(_native.lib().kvb_qabs_partial_scores(
        q.data_ptr(), k.data_ptr(), k.stride(0), k.stride(1), k.stride(2), k.stride(3), None, int(dim_count),
        out.data_ptr(), B, H, Hk, T, D, et, ops._dev(q), ops._stream(q.device)), "kvb_qabs_partial_scores")
    return out


def partial_scores_dim_major(query: torch.Tensor, key_dim_major: torch.Tensor, dim_indices: torch.Tensor) -> torch.Tensor:
    """``key_dim_major [B,H|Hkv,D,T]`` and the channel list ``dim_indices int64 [B,H,S]`` given (QCK:659-665)."""
    et = _elem_type(query, key_dim_major)
    q = query.contiguous()
    k = key_dim_major
    B, H, D = q.shape
    Hk, T = k.shape[1], k.shape[3]
    idx = dim_indices.to(torch.int64).contiguous()
    out = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    check(_native.lib().kvb_qabs_partial_scores(
        q.data_ptr(), k.data_ptr(), k.stride(0), k.stride(1), k.stride(3), k.stride(2), idx.data_ptr(),
        int(idx.shape[-1]), out.data_ptr(), B, H, Hk, T, D, et, ops._dev(q), ops._stream(q.device)),
        "kvb_qabs_partial_scores")
    return out


def candidate_full_scores(query: torch.Tensor, key_history: torch.Tensor, current_candidate: torch.Tensor,
                          previous_candidate: Optional[torch.Tensor], previous_final: Optional[torch.Tensor],
                          protect_sink_tokens: int, protect_recent_tokens: int, scaling: float) -> torch.Tensor:
    """Full ``q.k * scaling`` on ``current | previous_candidate | previous_final | sink | recent``
    (bool ``[B,H,T]`` masks), ``-inf`` elsewhere (QCK:668-691)."""
    et = _elem_type(query, key_history)
    q = query.contiguous()
    k = key_history if key_history.stride(-1) == 1 else key_history.contiguous()
    B, H, D = q.shape
    Hk, T = k.shape[1], k.shape[2]
    as_u8 = lambda m: None if m is None else m.to(torch.uint8).contiguous()  # noqa: E731
    cur, pc, pf = as_u8(current_candidate), as_u8(previous_candidate), as_u8(previous_final)
    out = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    check(_native.lib().kvb_qabs_candidate_full_scores(
        q.data_ptr(), k.data_ptr(), k.stride(0), k.stride(1), k.stride(2), cur.data_ptr(), ops._ptr(pc), ops._ptr(pf),
        int(protect_sink_tokens), int(protect_recent_tokens), float(scaling), out.data_ptr(), B, H, Hk, T, D, et,
        ops._dev(q), ops._stream(q.device)), "kvb_qabs_candidate_full_scores")
    return out


def final_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, indices: torch.Tensor,
                    valid: torch.Tensor, scaling: float) -> torch.Tensor:
    """Gathered attention over ``indices int64 [B,H,S]`` with ``valid`` -> ``[B,1,H,D]`` in the input dtype
    (QCK:694-705). The attention kernel is a bf16 one: fp16 / fp32 inputs are served by gathering the S
    selected rows first (never the whole cache) and rounding those to bf16, which stays inside the
    2e-2 / 1e-2 tolerance of this path; the accumulation is fp32 either way."""
    if key.dtype == torch.bfloat16:
        return ops.sparse_attend(query, key, value, indices, valid, scaling)
    if key.dtype not in _ELEM_TYPES or query.dtype != key.dtype or value.dtype != key.dtype:
        raise RuntimeError("query, key and value must share one of bfloat16, float16, float32")
    q3 = query[:, :, 0, :] if query.dim() == 4 else query
    B, H, D = q3.shape
    Hk, Tk = key.shape[1], key.shape[2]
    S = indices.shape[-1]
    idx = indices.long()
    ok = valid.bool() & (idx >= 0) & (idx < Tk)
    idx = idx.clamp(0, Tk - 1)
    bi = torch.arange(B, device=key.device)[:, None, None]
    hi = (torch.arange(H, device=key.device) // (H // Hk))[None, :, None]
    k_sel = key[bi, hi, idx].to(torch.bfloat16)                  # [B,H,S,D]
    v_sel = value[bi, hi, idx].to(torch.bfloat16)
    local = torch.arange(S, device=key.device).expand(B, H, S).contiguous()
    out = ops.sparse_attend(q3.to(torch.bfloat16), k_sel, v_sel, local, ok, scaling)
    return out.to(query.dtype)
