"""A pre-allocated KV cache with the HF ``Cache`` contract, for decode loops that must not copy the cache.

The stock ``DynamicLayer.update`` does ``torch.cat([self.keys, key_states], dim=-2)`` on every call, i.e. it
re-copies a layer's whole K and V for every decoded token (1 GiB per layer per token at batch 8 x 32768
tokens of Qwen3-0.6B shapes) before attention even starts; the reference evaluator inherits that (it feeds
``outputs.past_key_values`` back in, EVAL:7278 of littlexi001/kv_cache,
ymluo/projects/qwen3_top2_head_limit3_ppl/src/evaluate_qwen3_top2_head_limit3_ppl.py). The reference's own
answer to the same problem for its transposed key copy is an incrementally appended buffer with spare
capacity (``SparQMeanState.key_dim_major``, EVAL:2018-2042); this module gives K and V themselves that shape:

* ``PreallocatedLayer``  one layer: K and V live in ``[B, H, capacity, D]`` buffers allocated once;
  ``update`` stores the new rows in place and returns the views ``[:, :, :T]`` (strided: the kernels of
  this package take strides, so nothing is made contiguous). Running out of capacity grows the buffers
  geometrically (one copy per doubling, not per token).
* ``PreallocatedCache``  a ``transformers.Cache`` made of such layers; pass it as ``past_key_values``.

The int4 side caches and fused-step workspaces stay in ``attention_patch.SparseDecodeState``; give it the same
capacity (``state.capacity_hint``) and neither structure is ever re-allocated during a decode.
"""
from __future__ import annotations

from typing import Optional

import torch

try:                                                   # transformers is needed only for the Cache base classes
    from transformers.cache_utils import Cache, CacheLayerMixin
except Exception as exc:                               # pragma: no cover
    raise ImportError("kv_cache_b200.cache needs transformers (Cache, CacheLayerMixin)") from exc


class PreallocatedLayer(CacheLayerMixin):
    """K/V of one layer in buffers of ``capacity`` tokens; ``keys`` / ``values`` are views of the filled part."""

    is_sliding = False

    def __init__(self, capacity: int, growth_factor: float = 2.0):
        super().__init__()
        if capacity <= 0:
            raise ValueError("capacity must be positive")
        self.capacity = int(capacity)
        self.growth_factor = float(growth_factor)
        self.length = 0
        self.key_buffer: Optional[torch.Tensor] = None
        self.value_buffer: Optional[torch.Tensor] = None
        self.reallocations = 0

    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        B, H, _, D = key_states.shape
        self.dtype, self.device = key_states.dtype, key_states.device
        self.key_buffer = torch.empty((B, H, self.capacity, D), dtype=self.dtype, device=self.device)
        self.value_buffer = torch.empty((B, H, self.capacity, value_states.shape[-1]), dtype=value_states.dtype,
                                        device=self.device)
        self.keys, self.values = self.key_buffer[:, :, :0], self.value_buffer[:, :, :0]
        self.is_initialized = True

    def _grow(self, need: int) -> None:
        new_cap = max(need, int(self.capacity * self.growth_factor))
        for name in ("key_buffer", "value_buffer"):
            old = getattr(self, name)
            buf = torch.empty((*old.shape[:2], new_cap, old.shape[-1]), dtype=old.dtype, device=old.device)
            buf[:, :, :self.length].copy_(old[:, :, :self.length])
            setattr(self, name, buf)
        self.capacity = new_cap
        self.reallocations += 1

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
        """Stores the new rows behind the filled part and returns views of everything stored so far."""
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        n = key_states.shape[-2]
        if self.length + n > self.capacity:
            self._grow(self.length + n)
        self.key_buffer[:, :, self.length:self.length + n].copy_(key_states)
        self.value_buffer[:, :, self.length:self.length + n].copy_(value_states)
        self.length += n
        self.keys = self.key_buffer[:, :, :self.length]
        self.values = self.value_buffer[:, :, :self.length]
        return self.keys, self.values

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        return self.get_seq_length() + query_length, 0

    def get_seq_length(self) -> int:
        return self.length if self.is_initialized else 0

    def get_max_cache_shape(self) -> int:
        return -1                                     # grows on demand, like a dynamic layer

    def crop(self, max_length: int) -> None:
        if max_length < 0:
            max_length = self.length - abs(max_length)
        if self.is_initialized and 0 <= max_length < self.length:
            self.length = max_length
            self.keys = self.key_buffer[:, :, :self.length]
            self.values = self.value_buffer[:, :, :self.length]

    def reset(self) -> None:
        self.length = 0
        if self.is_initialized:
            self.keys, self.values = self.key_buffer[:, :, :0], self.value_buffer[:, :, :0]

    def batch_repeat_interleave(self, repeats: int) -> None:
        if self.is_initialized:
            self.key_buffer = self.key_buffer.repeat_interleave(repeats, dim=0)
            self.value_buffer = self.value_buffer.repeat_interleave(repeats, dim=0)
            self.keys, self.values = self.key_buffer[:, :, :self.length], self.value_buffer[:, :, :self.length]

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        if self.is_initialized:
            self.key_buffer = self.key_buffer[indices, ...]
            self.value_buffer = self.value_buffer[indices, ...]
            self.keys, self.values = self.key_buffer[:, :, :self.length], self.value_buffer[:, :, :self.length]

    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        self.batch_select_indices(beam_idx.to(self.key_buffer.device))

    def clone_prefix(self) -> "PreallocatedLayer":
        """A copy with its own buffers of the same capacity (several evaluation modes branching off one
        shared prefill, the use of the reference's ``clone_past_key_values``, EVAL:7114-7130)."""
        other = PreallocatedLayer(self.capacity, self.growth_factor)
        if self.is_initialized:
            other.dtype, other.device = self.dtype, self.device
            other.key_buffer = torch.empty_like(self.key_buffer)
            other.value_buffer = torch.empty_like(self.value_buffer)
            other.key_buffer[:, :, :self.length].copy_(self.key_buffer[:, :, :self.length])
            other.value_buffer[:, :, :self.length].copy_(self.value_buffer[:, :, :self.length])
            other.length = self.length
            other.keys, other.values = other.key_buffer[:, :, :other.length], other.value_buffer[:, :, :other.length]
            other.is_initialized = True
        return other


class PreallocatedCache(Cache):
    """``transformers.Cache`` whose layers are ``PreallocatedLayer``: pass as ``past_key_values``; every
    ``update(k, v, layer_idx)`` writes in place and hands the attention function ``[:, :, :T]`` views."""

    def __init__(self, num_layers: int, capacity: int, growth_factor: float = 2.0):
        super().__init__(layers=[PreallocatedLayer(capacity, growth_factor) for _ in range(num_layers)])
        self.capacity = int(capacity)

    def clone(self) -> "PreallocatedCache":
        other = PreallocatedCache(0, self.capacity)
        other.layers = [layer.clone_prefix() for layer in self.layers]
        return other

    @property
    def reallocations(self) -> int:
        return sum(layer.reallocations for layer in self.layers)


class PagedKV:
    """K/V of a batch of equally long sequences in fixed-size pages of two shared pools: appended rows go into
    the sequence's last page or into a page taken from the free list, and no stored row ever moves. The fused
    decode step reads the pools through ``page_table`` (``ops.DecodeStep(...)(..., kv_pages=(table, history))``);
    the int4 side cache stays contiguous (it is 7 % of the K/V bytes and is read as a stream).

    ``key_pool`` / ``value_pool``: bf16 ``[num_pages, Hkv, page_tokens, D]``; ``page_table``: int32
    ``[B, pages_per_sequence]`` (entries beyond the pages in use are 0, a valid page id that is never read)."""

    def __init__(self, batch: int, kv_heads: int, head_dim: int, page_tokens: int, num_pages: int, device,
                 pages_per_sequence: Optional[int] = None, dtype: torch.dtype = torch.bfloat16,
                 free_order: Optional[torch.Tensor] = None):
        if page_tokens < 1 or page_tokens & (page_tokens - 1):
            raise ValueError("page_tokens must be a power of two")
        self.B, self.Hkv, self.D, self.P = int(batch), int(kv_heads), int(head_dim), int(page_tokens)
        self.key_pool = torch.zeros((num_pages, kv_heads, page_tokens, head_dim), dtype=dtype, device=device)
        self.value_pool = torch.zeros_like(self.key_pool)
        per_seq = pages_per_sequence if pages_per_sequence is not None else num_pages // max(1, batch)
        self.page_table = torch.zeros((batch, per_seq), dtype=torch.int32, device=device)
        order = list(range(num_pages)) if free_order is None else [int(i) for i in free_order.tolist()]
        self.free = order[::-1]                           # pop() hands pages out in `order`
        self.length = 0

    def _ensure_pages(self, upto: int) -> None:
        have = (self.length + self.P - 1) // self.P
        need = (upto + self.P - 1) // self.P
        if need > self.page_table.shape[1]:
            raise RuntimeError("the page table has no room for that many tokens")
        for page in range(have, need):
            if len(self.free) < self.B:
                raise RuntimeError("the pool has no free page left")
            ids = [self.free.pop() for _ in range(self.B)]
            self.page_table[:, page] = torch.tensor(ids, dtype=torch.int32, device=self.page_table.device)

    def reserve(self, tokens: int) -> None:
        """Makes sure pages exist for the next ``tokens`` rows (the fused step stores the decoded token's row itself)."""
        self._ensure_pages(self.length + tokens)

    def append(self, key_rows: torch.Tensor, value_rows: torch.Tensor) -> None:
        """Stores rows ``[B,Hkv,n,D]`` behind the ``length`` rows already there."""
        n = key_rows.shape[2]
        self._ensure_pages(self.length + n)
        done = 0
        while done < n:
            t = self.length + done
            page, row = t // self.P, t % self.P
            take = min(n - done, self.P - row)
            ids = self.page_table[:, page].long()
            self.key_pool[ids, :, row:row + take] = key_rows[:, :, done:done + take]
            self.value_pool[ids, :, row:row + take] = value_rows[:, :, done:done + take]
            done += take
        self.length += n

    def advance(self, tokens: int = 1) -> None:
        """Counts rows that a kernel stored (``new_rows`` of the fused step)."""
        self.length += tokens

    def gather(self, upto: Optional[int] = None) -> tuple[torch.Tensor, torch.Tensor]:
        """The first ``upto`` (default: all) rows as contiguous ``[B,Hkv,T,D]`` tensors (a copy; for checks)."""
        T = self.length if upto is None else int(upto)
        pages = (T + self.P - 1) // self.P
        ids = self.page_table[:, :pages].long()                                     # [B, pages]
        k = self.key_pool[ids].permute(0, 2, 1, 3, 4).reshape(self.B, self.Hkv, pages * self.P, self.D)[:, :, :T]
        v = self.value_pool[ids].permute(0, 2, 1, 3, 4).reshape(self.B, self.Hkv, pages * self.P, self.D)[:, :, :T]
        return k.contiguous(), v.contiguous()
