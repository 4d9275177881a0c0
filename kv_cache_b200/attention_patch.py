"""Drop-in for the reference's patched Qwen3 attention (littlexi001/kv_cache,
ymluo/projects/qwen3_top2_head_limit3_ppl/src/evaluate_qwen3_top2_head_limit3_ppl.py = EVAL).

The reference installs ``_limited_eager_attention_forward`` (EVAL:6236-6931) as the HF "eager"
attention function (``install_qwen3_attention_patch``, EVAL:6934-6944) and steers it with the
``attention_mode(...)`` context manager (EVAL:6947-7075). This module keeps those two entry
points and the mode mini-language for the path this package implements:

    baseline                       dense attention (the original HF eager function)
    qabs{C}cand{P}attn             C partial channels, top ceil(P% * T) tokens  (EVAL:748-754, 4400-4502)
    qabs{C}cand{P}appendattn       same, protected ranges appended instead of filtered (EVAL:2985-3022)

with the int4 scorer and GQA-group selection in place of the reference's fp32 per-head scoring.
Unlike the reference dispatcher, K/V are NOT repeated to the query heads (EVAL:6248-6251 copies
them G times every layer, every step). Any other mode string raises: there is no fallback.
"""
from __future__ import annotations

import math
import re
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from . import ops

_QABS_RE = re.compile(r"qabs(\d+)cand(\d+(?:p\d+)?)(appendattn|attn)")


def parse_qabs_partial_rerank_params(mode: str) -> Optional[tuple[int, float]]:
    """``(channels, candidate_fraction)`` of a ``qabs{C}cand{P}[append]attn`` mode string, else None.
    ``P`` is a percentage with ``p`` as the decimal point (``6p25`` = 6.25 %), as in EVAL:748-754."""
    m = _QABS_RE.fullmatch(mode)
    if not m:
        return None
    return int(m.group(1)), float(m.group(2).replace("p", ".")) / 100.0


def candidate_count(candidate_fraction: float, history_count: int) -> int:
    """EVAL:4423: ``min(T, max(1, ceil(fraction * T)))``."""
    return min(history_count, max(1, math.ceil(candidate_fraction * history_count)))


def mode_for(channels: int, top_k: int, history_count: int, append: bool = False) -> str:
    """Mode string whose candidate count is exactly ``top_k`` at ``history_count`` tokens
    (exact when top_k / history_count is a short binary fraction, e.g. 2048 / 131072)."""
    pct = repr(100.0 * top_k / history_count)
    if "e" in pct:
        raise ValueError("fraction too small for the mode syntax")
    pct = pct.rstrip("0").rstrip(".") if "." in pct else pct
    return f"qabs{channels}cand{pct.replace('.', 'p')}{'appendattn' if append else 'attn'}"


@dataclass
class LayerSideCache:
    """int4 side cache of one layer: derived state, rebuilt from the bf16 K cache when missing."""
    channel_idx: torch.Tensor
    packed: torch.Tensor
    scale: torch.Tensor
    count: int = 0                      # tokens quantized so far
    key_ptr: int = 0                    # identity of the K storage last seen (detects a new sequence)


@dataclass
class SparseDecodeState:
    """Per-model state of the sparse path: one side cache and one fused-step object per layer."""
    layers: dict[int, LayerSideCache] = field(default_factory=dict)
    steps: dict[tuple, ops.DecodeStep] = field(default_factory=dict)
    growth: int = 4096                  # capacity headroom (tokens) when a side cache is (re)allocated

    def reset(self) -> None:
        self.layers.clear()

    def side_cache(self, layer_idx: int, key_states: torch.Tensor, history: int, channels: int) -> LayerSideCache:
        B, Hkv = key_states.shape[0], key_states.shape[1]
        sc = self.layers.get(layer_idx)
        stale = (sc is None or sc.packed.shape[0] != B or sc.packed.shape[1] != Hkv
                 or sc.channel_idx.shape[-1] != channels or sc.count > history
                 or sc.packed.device != key_states.device)
        if stale:
            ch = ops.choose_channels(key_states[:, :, :history], channels)
            packed, scale = ops.alloc_side_cache(B, Hkv, history + 1 + self.growth, channels, key_states.device)
            sc = LayerSideCache(ch, packed, scale, 0)
            self.layers[layer_idx] = sc
        elif sc.packed.shape[2] < history + 1:
            packed, scale = ops.alloc_side_cache(B, Hkv, history + 1 + self.growth, channels, key_states.device)
            packed[:, :, : sc.count].copy_(sc.packed[:, :, : sc.count])
            scale[:, :, : sc.count].copy_(sc.scale[:, :, : sc.count])
            sc.packed, sc.scale = packed, scale
        if sc.count < history:          # first decode step after a prefill: bulk quantize the new rows
            ops.quantize(key_states[:, :, sc.count:history], sc.channel_idx, out=(sc.packed, sc.scale), t_dst=sc.count)
            sc.count = history
        return sc

    def step(self, top_k: int, sink: int, recent: int, keep_self: bool, append: bool) -> ops.DecodeStep:
        key = (top_k, sink, recent, keep_self, append)
        st = self.steps.get(key)
        if st is None:
            st = ops.DecodeStep(top_k, sink, recent, keep_self, append_protected=append, append_self=True)
            self.steps[key] = st
        return st


# Process-global mode, as in the reference (EVAL:55-97): set by attention_mode(), read by the forward.
_ACTIVE_MODE = "baseline"
_ACTIVE_ALWAYS_KEEP_SELF = True
_ACTIVE_PROTECT_SINK_TOKENS = 0
_ACTIVE_PROTECT_RECENT_TOKENS = 0
_ACTIVE_STATE: Optional[SparseDecodeState] = None
_ORIGINAL_EAGER_ATTENTION_FORWARD = None


def sparse_eager_attention_forward(module: torch.nn.Module, query_states: torch.Tensor, key_states: torch.Tensor,
                                   value_states: torch.Tensor, attention_mask: Optional[torch.Tensor],
                                   scaling: Optional[float] = None, dropout: float = 0.0, **kwargs: Any):
    """HF attention-interface function (signature of EVAL:6236-6245): query ``[B,Hq,Tq,D]``, key/value
    ``[B,Hkv,Tk,D]`` (already holding the current token) -> ``(out [B,Tq,Hq,D], weights or None)``."""
    if scaling is None:
        scaling = float(getattr(module, "scaling", 1.0 / math.sqrt(query_states.shape[-1])))
    mode = _ACTIVE_MODE
    if mode == "baseline":
        if _ORIGINAL_EAGER_ATTENTION_FORWARD is None:
            raise RuntimeError("baseline mode needs install_qwen3_attention_patch() to have captured the HF function")
        return _ORIGINAL_EAGER_ATTENTION_FORWARD(module, query_states, key_states, value_states, attention_mask,
                                                 scaling=scaling, dropout=dropout, **kwargs)
    params = parse_qabs_partial_rerank_params(mode)
    if params is None:
        raise RuntimeError(f"kv_cache_b200 implements 'baseline' and 'qabs{{C}}cand{{P}}[append]attn'; got mode {mode!r}")
    channels, fraction = params
    if query_states.shape[2] != 1:
        # same contract as EVAL:4413-4414
        raise RuntimeError("qabs candidate-attention mode requires token-by-token eval; set --eval_chunk_size 1.")
    key_count = key_states.shape[-2]
    if key_count <= 1:                  # EVAL:4415-4417
        out = value_states[:, :, -1:, :].transpose(1, 2)
        rep = query_states.shape[1] // value_states.shape[1]
        return out.repeat_interleave(rep, dim=2).contiguous(), None
    state = _ACTIVE_STATE
    if state is None:
        raise RuntimeError("sparse modes must run inside `with attention_mode(...)`")
    history = key_count - 1
    layer_idx = int(getattr(module, "layer_idx", 0))
    top_k = candidate_count(fraction, history)
    sc = state.side_cache(layer_idx, key_states, history, min(max(2, channels + (channels & 1)), key_states.shape[-1]))
    step = state.step(top_k, _ACTIVE_PROTECT_SINK_TOKENS, _ACTIVE_PROTECT_RECENT_TOKENS, _ACTIVE_ALWAYS_KEEP_SELF,
                      mode.endswith("appendattn"))
    out = step(query_states, key_states, value_states, sc.packed, sc.scale, sc.channel_idx, scaling=scaling,
               attention_mask=attention_mask)
    sc.count = key_count                # the fused step appended the current token's row
    return out, None


def install_qwen3_attention_patch() -> None:
    """Routes HF Qwen3 "eager" attention through this package (EVAL:6934-6944). Load the model with
    ``attn_implementation="eager"``."""
    global _ORIGINAL_EAGER_ATTENTION_FORWARD
    try:
        import transformers.models.qwen3.modeling_qwen3 as modeling_qwen3
    except Exception as exc:
        raise RuntimeError("Could not import transformers.models.qwen3.modeling_qwen3.") from exc
    if _ORIGINAL_EAGER_ATTENTION_FORWARD is None:
        _ORIGINAL_EAGER_ATTENTION_FORWARD = getattr(modeling_qwen3, "eager_attention_forward")
        setattr(modeling_qwen3, "eager_attention_forward", sparse_eager_attention_forward)
        if hasattr(modeling_qwen3, "ALL_ATTENTION_FUNCTIONS"):
            modeling_qwen3.ALL_ATTENTION_FUNCTIONS["eager"] = sparse_eager_attention_forward


def uninstall_qwen3_attention_patch() -> None:
    global _ORIGINAL_EAGER_ATTENTION_FORWARD
    if _ORIGINAL_EAGER_ATTENTION_FORWARD is None:
        return
    import transformers.models.qwen3.modeling_qwen3 as modeling_qwen3

    setattr(modeling_qwen3, "eager_attention_forward", _ORIGINAL_EAGER_ATTENTION_FORWARD)
    if hasattr(modeling_qwen3, "ALL_ATTENTION_FUNCTIONS"):
        modeling_qwen3.ALL_ATTENTION_FUNCTIONS["eager"] = _ORIGINAL_EAGER_ATTENTION_FORWARD
    _ORIGINAL_EAGER_ATTENTION_FORWARD = None


@contextmanager
def attention_mode(mode: str, top_fraction: float = 0.02, max_heads_per_token: int = 3, always_keep_self: bool = True,
                   protect_sink_tokens: int = 0, protect_recent_tokens: int = 0, load_stats: Any = None,
                   sparse_state: Optional[SparseDecodeState] = None, **reference_kwargs: Any):
    """Same leading parameters as the reference's ``attention_mode`` (EVAL:6947-6955). The state
    objects and switches of modes this package does not implement are accepted and ignored so that
    existing call sites keep working; ``sparse_state`` carries the int4 side caches across ``with``
    blocks (a fresh one is created when omitted)."""
    global _ACTIVE_MODE, _ACTIVE_ALWAYS_KEEP_SELF, _ACTIVE_PROTECT_SINK_TOKENS, _ACTIVE_PROTECT_RECENT_TOKENS, _ACTIVE_STATE
    if mode != "baseline" and parse_qabs_partial_rerank_params(mode) is None:
        raise RuntimeError(f"kv_cache_b200 implements 'baseline' and 'qabs{{C}}cand{{P}}[append]attn'; got mode {mode!r}")
    previous = (_ACTIVE_MODE, _ACTIVE_ALWAYS_KEEP_SELF, _ACTIVE_PROTECT_SINK_TOKENS, _ACTIVE_PROTECT_RECENT_TOKENS,
                _ACTIVE_STATE)
    _ACTIVE_MODE = mode
    _ACTIVE_ALWAYS_KEEP_SELF = bool(always_keep_self)
    _ACTIVE_PROTECT_SINK_TOKENS = max(0, int(protect_sink_tokens))
    _ACTIVE_PROTECT_RECENT_TOKENS = max(0, int(protect_recent_tokens))
    _ACTIVE_STATE = sparse_state if sparse_state is not None else SparseDecodeState()
    try:
        yield _ACTIVE_STATE
    finally:
        (_ACTIVE_MODE, _ACTIVE_ALWAYS_KEEP_SELF, _ACTIVE_PROTECT_SINK_TOKENS, _ACTIVE_PROTECT_RECENT_TOKENS,
         _ACTIVE_STATE) = previous
