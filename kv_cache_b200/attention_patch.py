"""Drop-in for the reference's patched Qwen3 attention (littlexi001/kv_cache,
ymluo/projects/qwen3_top2_head_limit3_ppl/src/evaluate_qwen3_top2_head_limit3_ppl.py = EVAL).

The reference installs ``_limited_eager_attention_forward`` (EVAL:6236-6931) as the HF "eager"
attention function (``install_qwen3_attention_patch``, EVAL:6934-6944) and steers it with the
``attention_mode(...)`` context manager (EVAL:6947-7075). This module keeps those two entry
points — ``attention_mode`` with the reference's complete parameter list, so the evaluator's own
call with 29 positional arguments (EVAL:7236-7266) binds — and the mode mini-language for the path
this package implements:

    baseline                       dense attention (the original HF eager function)
    qabs{C}cand{P}attn             C partial channels, top ceil(P% * T) tokens  (EVAL:748-754, 4400-4502)
    qabs{C}cand{P}appendattn       same, protected ranges appended instead of filtered (EVAL:2985-3022)
    qabs{C}cand{P}top2attn         candidates, exact q.k on them, the best ceil(top_fraction * T)  (EVAL:4650-4766)
    qabs{C}cand{P}reuse            candidates + the previous step's candidates and final set, exact q.k on the
      [2set|final][blk{N}]         union, the best ceil(top_fraction * T), protected ranges forced in, optional
                                   widening to aligned blocks of N tokens (EVAL:3991-4397, 1596-1759, 2914-2922)
    sparqfast{C}cand{P}            top ceil(P% * keys) of ALL keys (the decoded token included), exact attention
                                   over them blended with the running mean of V by the softmax mass they carry
                                   under the approximate logits (EVAL:2646-2722, 2006-2016)

with the int4 scorer and GQA-group selection in place of the reference's fp32 per-head scoring: one
candidate list, one exact rerank (maximum of q.k over the group's query heads) and one final list per KV head.
Unlike the reference dispatcher, K/V are NOT repeated to the query heads (EVAL:6248-6251 copies
them G times every layer, every step). Any other mode string raises: there is no fallback.

State. The reference opens one ``with attention_mode(...)`` per decoded token (EVAL:7236), so the
int4 side caches cannot live in the ``with`` block: they live in a module-level
``SparseDecodeState`` (or one the caller passes as ``sparse_state=``) and are extended by one row
per step. A layer's side cache is dropped when the calls that pass through the patched function
stop being a continuation of what it has seen (a new prefill, another batch shape or device), or
by ``reset_sparse_state()``.
"""
from __future__ import annotations

import math
import re
import sys
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from . import ops

_QABS_RE = re.compile(r"qabs(\d+)cand(\d+(?:p\d+)?)(appendattn|top2attn|attn|reuse(?:2set|final)?(?:blk(\d+))?)")


def parse_qabs_partial_rerank_params(mode: str) -> Optional[tuple[int, float]]:
    """``(channels, candidate_fraction)`` of a ``qabs{C}cand{P}...`` mode string this package implements, else
    None. ``P`` is a percentage with ``p`` as the decimal point (``6p25`` = 6.25 %), as in EVAL:748-754."""
    m = _QABS_RE.fullmatch(mode)
    if not m:
        return None
    return int(m.group(1)), float(m.group(2).replace("p", ".")) / 100.0


_SPARQ_RE = re.compile(r"sparqfast(\d+)cand(\d+(?:p\d+)?)")


def parse_sparq_params(mode: str) -> Optional[tuple[int, float]]:
    """``(channels, candidate_fraction)`` of ``sparqfast{C}cand{P}`` (EVAL:892-898), else None."""
    m = _SPARQ_RE.fullmatch(mode)
    if not m:
        return None
    return int(m.group(1)), float(m.group(2).replace("p", ".")) / 100.0


def parse_mode_kind(mode: str) -> Optional[tuple[str, int]]:
    """``(kind, block_size)``: kind is ``attn``, ``appendattn``, ``top2attn`` or ``reuse`` / ``reuse2set`` /
    ``reusefinal`` (EVAL:955-960: which previous sets join the union); block_size from a ``blk{N}`` suffix, else 1."""
    m = _QABS_RE.fullmatch(mode)
    if not m:
        return None
    tail = m.group(3)
    block = int(m.group(4)) if m.group(4) else 1
    if tail.startswith("reuse"):
        tail = tail.split("blk")[0]
    return tail, max(1, block)


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
    count: int = 0                      # rows quantized so far
    seen: int = 0                       # key rows of this sequence that have passed through the patched function
    calibrated_at: int = 0              # history length the channel choice was made from
    fixed_channels: bool = False        # the caller supplied the channel list: never re-chosen


@dataclass
class LayerReuse:
    """What a reuse mode carries from one decode step of a layer to the next (the list form of the two masks in
    ReuseCandidateState.previous_layer, EVAL:1725-1745)."""
    query_token: int
    candidate: torch.Tensor             # int32 [B,Hkv,n]   this step's own candidates
    final: torch.Tensor                 # int32 [B,Hkv,m]   kept set incl. protected ranges, -1 padded
    final_count: torch.Tensor           # int32 [B,Hkv]


@dataclass
class SparseDecodeState:
    """Per-model state of the sparse path: one int4 side cache per layer and one fused-step object
    (with its workspace) per selection policy."""
    layers: dict[int, LayerSideCache] = field(default_factory=dict)
    steps: dict[tuple, ops.DecodeStep] = field(default_factory=dict)
    growth: int = 4096                  # capacity headroom (tokens) when a side cache is (re)allocated
    capacity_hint: int = 0              # allocate side caches for at least this many tokens (the capacity of a
                                        # pre-allocated KV cache): no re-allocation during a decode
    # The static channel set is chosen from the keys that exist at a layer's first sparse call. When that
    # call comes early (token-by-token evaluation from the first token) the choice rests on a handful of
    # rows, so it is made again, once, when the history first reaches this many tokens (the prefix is then
    # re-quantized, a few hundred rows).
    calibration_tokens: int = 256
    channel_lists: dict[int, torch.Tensor] = field(default_factory=dict)    # optional per-layer int32 [Hkv,C] from the caller
    bulk_quantized_rows: int = 0        # rows ever sent through the bulk quantizer (tests read this)
    reuse: dict[int, LayerReuse] = field(default_factory=dict)
    value_means: dict[int, tuple[int, torch.Tensor]] = field(default_factory=dict)    # layer -> (rows, fp32 [B,Hkv,D])

    def reset(self) -> None:
        self.layers.clear()
        self.reuse.clear()
        self.value_means.clear()

    def value_mean(self, layer_idx: int, value_states: torch.Tensor) -> torch.Tensor:
        """Mean of V over all key rows, fp32 ``[B,Hkv,D]``, kept per layer and updated by the one new row when the
        call continues the previous one (SparQMeanState.value_mean, EVAL:2006-2016)."""
        key_count = value_states.shape[2]
        prev = self.value_means.get(layer_idx)
        if prev is not None and prev[0] == key_count - 1 and prev[1].shape[:2] == value_states.shape[:2] \
                and prev[1].device == value_states.device:
            mean = (prev[1] * float(key_count - 1) + value_states[:, :, -1, :].float()) / float(key_count)
        else:
            mean = torch.zeros((*value_states.shape[:2], value_states.shape[-1]), dtype=torch.float32,
                               device=value_states.device)
            for t0 in range(0, key_count, 65536):                        # bounded fp32 temporaries
                mean += value_states[:, :, t0:t0 + 65536].float().sum(dim=2)
            mean /= float(key_count)
        self.value_means[layer_idx] = (key_count, mean)
        return mean

    def observe(self, layer_idx: int, key_count: int, query_count: int) -> None:
        """Called for every attention call that does NOT take the sparse path (baseline mode, prefill
        chunks): keeps a layer's side cache only while those calls continue the sequence it belongs to."""
        sc = self.layers.get(layer_idx)
        if sc is None:
            return
        if key_count - query_count == sc.seen:
            sc.seen = key_count                          # same sequence, rows pending for the next sparse call
        else:
            del self.layers[layer_idx]

    def side_cache(self, layer_idx: int, key_states: torch.Tensor, history: int, channels: int) -> LayerSideCache:
        B, Hkv = key_states.shape[0], key_states.shape[1]
        sc = self.layers.get(layer_idx)
        stale = (sc is None or sc.packed.shape[0] != B or sc.packed.shape[1] != Hkv
                 or sc.channel_idx.shape[-1] != channels or sc.packed.device != key_states.device
                 or sc.seen != history or sc.count > history)
        given = self.channel_lists.get(layer_idx)
        if not stale and not sc.fixed_channels and sc.calibrated_at < self.calibration_tokens <= history:
            stale = True                                 # the one re-calibration (see calibration_tokens)
        if stale:
            if given is not None:
                ch = given.to(device=key_states.device, dtype=torch.int32).contiguous()
            else:
                ch = ops.choose_channels(key_states[:, :, :history], channels)
            packed, scale = ops.alloc_side_cache(B, Hkv, max(history + 1 + self.growth, self.capacity_hint), channels,
                                                 key_states.device)
            sc = LayerSideCache(ch, packed, scale, 0, history, history, given is not None)
            self.layers[layer_idx] = sc
        elif sc.packed.shape[2] < history + 1:
            packed, scale = ops.alloc_side_cache(B, Hkv, history + 1 + self.growth, channels, key_states.device)
            packed[:, :, : sc.count].copy_(sc.packed[:, :, : sc.count])
            scale[:, :, : sc.count].copy_(sc.scale[:, :, : sc.count])
            sc.packed, sc.scale = packed, scale
        if sc.count < history:          # rows that arrived outside the sparse path (prefill): bulk quantize them
            ops.quantize(key_states[:, :, sc.count:history], sc.channel_idx, out=(sc.packed, sc.scale), t_dst=sc.count)
            self.bulk_quantized_rows += history - sc.count
            sc.count = history
        return sc

    def step(self, sink: int, recent: int, keep_self: bool, append: bool) -> ops.DecodeStep:
        """One fused-step object (one workspace) per policy; the candidate count is passed per call."""
        key = (sink, recent, keep_self, append)
        st = self.steps.get(key)
        if st is None:
            st = ops.DecodeStep(1, sink, recent, keep_self, append_protected=append, append_self=True)
            self.steps[key] = st
        return st


# Process-global mode, as in the reference (EVAL:55-97): set by attention_mode(), read by the forward.
_ACTIVE_MODE = "baseline"
_ACTIVE_TOP_FRACTION = 0.02
_ACTIVE_ALWAYS_KEEP_SELF = True
_ACTIVE_PROTECT_SINK_TOKENS = 0
_ACTIVE_PROTECT_RECENT_TOKENS = 0
_ACTIVE_STATE: Optional[SparseDecodeState] = None
_DEFAULT_STATE = SparseDecodeState()
_ORIGINAL_EAGER_ATTENTION_FORWARD = None


def reset_sparse_state() -> None:
    """Drops every int4 side cache of the module-level state (call between unrelated sequences when the
    patched function cannot see the change, e.g. two prompts of which the second is prefilled elsewhere)."""
    _DEFAULT_STATE.reset()


def default_sparse_state() -> SparseDecodeState:
    return _DEFAULT_STATE


def sparse_eager_attention_forward(module: torch.nn.Module, query_states: torch.Tensor, key_states: torch.Tensor,
                                   value_states: torch.Tensor, attention_mask: Optional[torch.Tensor],
                                   scaling: Optional[float] = None, dropout: float = 0.0, **kwargs: Any):
    """HF attention-interface function (signature of EVAL:6236-6245): query ``[B,Hq,Tq,D]``, key/value
    ``[B,Hkv,Tk,D]`` (already holding the current token) -> ``(out [B,Tq,Hq,D], weights or None)``."""
    if scaling is None:
        scaling = float(getattr(module, "scaling", 1.0 / math.sqrt(query_states.shape[-1])))
    mode = _ACTIVE_MODE
    state = _ACTIVE_STATE if _ACTIVE_STATE is not None else _DEFAULT_STATE
    layer_idx = int(getattr(module, "layer_idx", 0))
    key_count = key_states.shape[-2]
    if mode == "baseline":
        if _ORIGINAL_EAGER_ATTENTION_FORWARD is None:
            raise RuntimeError("baseline mode needs install_qwen3_attention_patch() to have captured the HF function")
        state.observe(layer_idx, key_count, query_states.shape[2])
        return _ORIGINAL_EAGER_ATTENTION_FORWARD(module, query_states, key_states, value_states, attention_mask,
                                                 scaling=scaling, dropout=dropout, **kwargs)
    sparq = parse_sparq_params(mode)
    if sparq is not None:
        if query_states.shape[2] != 1:
            raise RuntimeError("SparQ fast mode requires token-by-token eval; set --eval_chunk_size 1.")   # EVAL:6359-6360
        return _sparq_forward(state, layer_idx, sparq, query_states, key_states, value_states, attention_mask, scaling), None
    params = parse_qabs_partial_rerank_params(mode)
    if params is None:
        raise RuntimeError(f"kv_cache_b200 implements 'baseline' and 'qabs{{C}}cand{{P}}' + attn | appendattn | top2attn | reuse[2set|final][blkN], 'sparqfast{{C}}cand{{P}}'; got mode {mode!r}")
    channels, fraction = params
    if query_states.shape[2] != 1:
        # same contract as EVAL:4413-4414
        raise RuntimeError("qabs candidate-attention mode requires token-by-token eval; set --eval_chunk_size 1.")
    if key_count <= 1:                  # EVAL:4415-4417
        state.observe(layer_idx, key_count, 1)
        out = value_states[:, :, -1:, :].transpose(1, 2)
        rep = query_states.shape[1] // value_states.shape[1]
        return out.repeat_interleave(rep, dim=2).contiguous(), None
    history = key_count - 1
    top_k = candidate_count(fraction, history)
    sc = state.side_cache(layer_idx, key_states, history, min(max(2, channels + (channels & 1)), key_states.shape[-1]))
    kind, block = parse_mode_kind(mode)
    if kind == "top2attn" or kind.startswith("reuse"):
        return _rerank_forward(state, layer_idx, sc, kind, block, top_k, query_states, key_states, value_states,
                               attention_mask, scaling), None
    step = state.step(_ACTIVE_PROTECT_SINK_TOKENS, _ACTIVE_PROTECT_RECENT_TOKENS, _ACTIVE_ALWAYS_KEEP_SELF,
                      mode.endswith("appendattn"))
    out = step(query_states, key_states, value_states, sc.packed, sc.scale, sc.channel_idx, scaling=scaling,
               attention_mask=attention_mask, top_k=top_k)
    sc.count = sc.seen = key_count      # the fused step appended the current token's row
    return out, None


def _sparq_forward(state: SparseDecodeState, layer_idx: int, params: tuple[int, float], query_states, key_states,
                   value_states, attention_mask, scaling: float) -> torch.Tensor:
    """``sparqfast{C}cand{P}``: every key row (the decoded token's too) is in the int4 cache; the best
    ceil(P * keys) per KV head are attended exactly and the result is blended with the running mean of V."""
    channels, fraction = params
    key_count = key_states.shape[-2]
    channels = min(max(8, (channels + 7) // 8 * 8), key_states.shape[-1])
    if key_count <= 1:
        state.observe(layer_idx, key_count, 1)
        rep = query_states.shape[1] // value_states.shape[1]
        return value_states[:, :, -1:, :].transpose(1, 2).repeat_interleave(rep, dim=2).contiguous()
    history = key_count - 1
    sc = state.side_cache(layer_idx, key_states, history, channels)
    ops.quantize_append(key_states[:, :, history], sc.channel_idx, sc.packed, sc.scale, history)
    sc.count = sc.seen = key_count
    cand_k = min(key_count, max(1, math.ceil(fraction * key_count)))       # EVAL:2661
    sel = ops.score_select(query_states, sc.packed, sc.scale, sc.channel_idx, key_count, cand_k)
    alpha = ops.sparq_alpha(query_states, sc.packed, sc.scale, sc.channel_idx, key_count, sel, attention_mask=attention_mask)
    vmean = state.value_mean(layer_idx, value_states)
    return ops.attend_selected_blend(query_states, key_states, value_states, sel, key_count, alpha, vmean, keep_self=False,
                                     scaling=scaling, attention_mask=attention_mask)


def _rerank_forward(state: SparseDecodeState, layer_idx: int, sc: LayerSideCache, kind: str, block: int, cand_k: int,
                    query_states, key_states, value_states, attention_mask, scaling: float) -> torch.Tensor:
    """The rerank modes as lists: int4 candidates -> (union with the previous step's lists) -> exact q.k ->
    top ceil(top_fraction * T) -> protected ranges / block widening -> attention over the final list."""
    key_count = key_states.shape[-2]
    history = key_count - 1
    sink, recent = _ACTIVE_PROTECT_SINK_TOKENS, _ACTIVE_PROTECT_RECENT_TOKENS
    cand = ops.score_select(query_states, sc.packed, sc.scale, sc.channel_idx, history, cand_k)
    ops.quantize_append(key_states[:, :, history], sc.channel_idx, sc.packed, sc.scale, history)
    sc.count = sc.seen = key_count
    keep_full = max(1, math.ceil(_ACTIVE_TOP_FRACTION * history))
    if kind == "top2attn":
        keep = min(cand_k, keep_full)                      # EVAL:4676
        kept, cnt = ops.rerank_union(query_states, key_states, [cand], history, keep, scaling=scaling,
                                     attention_mask=attention_mask)
        selected, count = kept, cnt
    else:
        keep = min(history, keep_full)                     # EVAL:4269-4270
        prev = state.reuse.get(layer_idx)
        if prev is not None and (prev.query_token != history - 1 or prev.candidate.shape[:2] != cand.shape[:2]
                                 or prev.candidate.device != cand.device):
            prev = None                                    # not the step before this one (EVAL:1653-1655)
        lists = [cand, prev.candidate if prev is not None and kind != "reusefinal" else None,
                 prev.final if prev is not None and kind != "reuse2set" else None]
        counts = [None, None, prev.final_count if lists[2] is not None else None]
        kept, cnt = ops.rerank_union(query_states, key_states, lists, history, keep, counts=counts, scaling=scaling)
        final, fcnt = ops.expand_final(kept, history, count=cnt, force_sink=sink, force_recent=recent, block_size=block)
        state.reuse[layer_idx] = LayerReuse(history, cand, final, fcnt)
        selected, count = (final, fcnt) if block > 1 else (kept, cnt)
    return ops.attend_selected(query_states, key_states, value_states, selected, history, protect_sink=sink,
                               protect_recent=recent, keep_self=_ACTIVE_ALWAYS_KEEP_SELF, scaling=scaling,
                               attention_mask=attention_mask, selected_count=count.reshape(-1))


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


def install_qabs_cuda_kernels_alias() -> None:
    """Makes ``from qabs_cuda_kernels import ...`` (the top-level import inside the evaluator's
    ``_maybe_cuda_*`` hooks, EVAL:3794, 3826, 3862, 3901) resolve to this package's module with the same four
    callables, so those hooks reach the sm_100a library without an edit of the evaluator."""
    from . import qabs_cuda_kernels

    sys.modules["qabs_cuda_kernels"] = qabs_cuda_kernels


@contextmanager
def attention_mode(mode: str, top_fraction: float = 0.02, max_heads_per_token: int = 3, always_keep_self: bool = True,
                   protect_sink_tokens: int = 0, protect_recent_tokens: int = 0, load_stats: Any = None,
                   obs_state: Any = None, obs_mass_state: Any = None, obs_hybrid_state: Any = None,
                   reuse_state: Any = None, knorm_state: Any = None, block_route_state: Any = None,
                   ksign_state: Any = None, kdom_state: Any = None, brep_state: Any = None,
                   sparq_mean_state: Any = None, candidate_stats: Any = None, reuse_overlap_stats: Any = None,
                   qabs_fast_path: bool = False, qabs_cuda_final_kernel: bool = False,
                   qabs_cuda_candidate_kernel: bool = False, qabs_cuda_reuse_select_kernel: bool = False,
                   qabs_profile_stats: Any = None, qabs_candidate_selection: str = "topk",
                   qabs_threshold_sample_size: int = 256, full_head_map_path: str = "",
                   full_layer_map_path: str = "", layer_budget_map_path: str = "", *,
                   sparse_state: Optional[SparseDecodeState] = None):
    """The reference's ``attention_mode`` with its parameter list in its order (EVAL:6947-6976), so that
    existing call sites — positional or by keyword — keep working. Used here: ``mode``, ``top_fraction``,
    ``always_keep_self``, ``protect_sink_tokens``, ``protect_recent_tokens``; the state objects and switches
    of modes this package does not implement are accepted and ignored (the CUDA-kernel switches are moot:
    the library is always the path). ``sparse_state`` (keyword only, not in the reference) replaces the
    module-level state that carries the int4 side caches from one ``with`` block to the next.
    Yields the state in use."""
    global _ACTIVE_MODE, _ACTIVE_TOP_FRACTION, _ACTIVE_ALWAYS_KEEP_SELF, _ACTIVE_PROTECT_SINK_TOKENS
    global _ACTIVE_PROTECT_RECENT_TOKENS, _ACTIVE_STATE
    if mode != "baseline" and parse_qabs_partial_rerank_params(mode) is None and parse_sparq_params(mode) is None:
        raise RuntimeError(f"kv_cache_b200 implements 'baseline' and 'qabs{{C}}cand{{P}}' + attn | appendattn | top2attn | reuse[2set|final][blkN], 'sparqfast{{C}}cand{{P}}'; got mode {mode!r}")
    previous = (_ACTIVE_MODE, _ACTIVE_TOP_FRACTION, _ACTIVE_ALWAYS_KEEP_SELF, _ACTIVE_PROTECT_SINK_TOKENS,
                _ACTIVE_PROTECT_RECENT_TOKENS, _ACTIVE_STATE)
    _ACTIVE_MODE = mode
    _ACTIVE_TOP_FRACTION = float(top_fraction)
    _ACTIVE_ALWAYS_KEEP_SELF = bool(always_keep_self)
    _ACTIVE_PROTECT_SINK_TOKENS = max(0, int(protect_sink_tokens))
    _ACTIVE_PROTECT_RECENT_TOKENS = max(0, int(protect_recent_tokens))
    _ACTIVE_STATE = sparse_state if sparse_state is not None else _DEFAULT_STATE
    try:
        yield _ACTIVE_STATE
    finally:
        (_ACTIVE_MODE, _ACTIVE_TOP_FRACTION, _ACTIVE_ALWAYS_KEEP_SELF, _ACTIVE_PROTECT_SINK_TOKENS,
         _ACTIVE_PROTECT_RECENT_TOKENS, _ACTIVE_STATE) = previous
