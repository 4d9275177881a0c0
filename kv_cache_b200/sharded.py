"""Sequence-sharded sparse decode: the KV cache of every sequence is split along the token axis
across the ranks of one node (one process per GPU, torch.distributed for the set-up plumbing).

Rank r owns history tokens [r*T/N, (r+1)*T/N) (bf16 K/V and the int4 side cache); the query, the
channel list and the K/V row of the token being decoded are replicated. One decode step:

  1. local  : int4 score of the shard, exact local top-k per KV head -> (score, GLOBAL token id) lists;
              the best 8192/N entries per row go straight into every rank's exchange buffer
  2. merge  : every rank selects the global top-k from the N lists with the same rule
              (score desc, id asc): identical result on every rank, independent of rank order
  3. attend : each rank attends to the selected ids it owns (the last rank also to the decoded
              token) and sends its un-normalised partial (o, m, l) to every rank
  4. combine: log-sum-exp merge of the N partials on every rank

On GPUs the whole step is ONE library call (kvb_sharded_decode_step): seven kernel launches, no
collective. Data moves between ranks by ordinary stores into peer memory over NVLink (exchange
buffers mapped once at set-up through CUDA IPC) guarded by flags that carry the step number; all
device-side waits are bounded. The call sequence is captured once in a CUDA graph and replayed.

The reference (littlexi001/kv_cache) has no sharded path; the single-GPU operators it composes are
those of kv_cache_b200.ops. Shapes the one-call step does not take (top_k above a shard's length,
non-streaming scorer configurations) and CPU ranks (gloo, with a checker backend standing in for the
device stages) run the same four stages composed from operators around two all-gathers.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _native, ops
from ._native import ShardedStepParams, check


def shard_bounds(total_tokens: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous token range of ``rank``; the first ``total % world`` ranks hold one token more."""
    base, extra = divmod(total_tokens, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def _all_gather(t: torch.Tensor, world: int, group) -> torch.Tensor:
    """``[world, *t.shape]``: one all-gather of a contiguous tensor (flat views: the form every backend takes)."""
    t = t.contiguous()
    out = torch.empty((world * t.numel(),), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.view(-1), group=group)
    return out.view(world, *t.shape)


class PeerExchange:
    """This rank's exchange buffer (zero-filled device memory allocated by the library) and the
    buffers of all peers mapped into this process. ``ptrs[r]`` is rank r's buffer as seen from here."""

    def __init__(self, nbytes: int, device: torch.device, rank: int = 0, world: int = 1, group=None):
        lib = _native.lib()
        self.device = device.index if device.index is not None else torch.cuda.current_device()
        self.nbytes, self.rank, self.world = int(nbytes), rank, world
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        check(lib.kvb_exchange_alloc(self.nbytes, self.device, C.byref(ptr), handle), "kvb_exchange_alloc")
        self.local = ptr.value
        self.ptrs: list[int] = [0] * world
        self.ptrs[rank] = self.local
        if world > 1:
            handles: list = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            for r in range(world):
                if r != rank:
                    peer = C.c_void_p()
                    check(lib.kvb_exchange_open(handles[r], self.device, C.byref(peer)), "kvb_exchange_open")
                    self.ptrs[r] = peer.value
            dist.barrier(group=group)           # nobody steps before every mapping exists

    def close(self) -> None:
        """Unmaps the peers' buffers and frees the local one. Call on every rank, after the last step
        has completed everywhere (the caller synchronises and barriers first)."""
        lib = _native.lib()
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                lib.kvb_exchange_close(p, self.device)
        if self.local:
            lib.kvb_exchange_free(self.local, self.device)
        self.local, self.ptrs = 0, []


def sharded_decode_step(query: torch.Tensor, key_local: torch.Tensor, value_local: torch.Tensor, packed: torch.Tensor,
                        scale: torch.Tensor, channel_idx: torch.Tensor, t_local: int, id_offset: int, total_tokens: int,
                        top_k: int, rank: int, world: int, exchange_ptrs: list[int], exchange_bytes: int,
                        workspace: torch.Tensor, out: Optional[torch.Tensor], selected_out: Optional[torch.Tensor] = None,
                        scaling: Optional[float] = None, phases: int = 7, wait_polls: int = 0) -> int:
    """Thin call of ``kvb_sharded_decode_step`` on the current stream; returns the status code."""
    query = ops._query3(query)
    B, Hq, D = query.shape
    Hkv = key_local.shape[1]
    C_ = int(channel_idx.shape[-1])
    ops._check_side_cache(packed, scale, C_)
    key_local, value_local = ops._rows_contiguous(key_local), ops._rows_contiguous(value_local)
    p = ShardedStepParams()
    p.query, p.q_sb, p.q_sh = query.data_ptr(), query.stride(0), query.stride(1)
    p.key, p.k_sb, p.k_sh, p.k_st = key_local.data_ptr(), key_local.stride(0), key_local.stride(1), key_local.stride(2)
    p.value, p.v_sb, p.v_sh, p.v_st = (value_local.data_ptr(), value_local.stride(0), value_local.stride(1),
                                       value_local.stride(2))
    p.packed, p.packed_sb, p.packed_sh = packed.data_ptr(), packed.stride(0), packed.stride(1)
    p.scale, p.scale_sb, p.scale_sh = scale.data_ptr(), scale.stride(0), scale.stride(1)
    p.channel_idx = channel_idx.data_ptr()
    p.B, p.Hq, p.Hkv, p.D, p.C = B, Hq, Hkv, D, C_
    p.t_local, p.id_offset, p.total_tokens = int(t_local), int(id_offset), int(total_tokens)
    p.top_k, p.rank, p.world = int(top_k), int(rank), int(world)
    p.scaling = float(D) ** -0.5 if scaling is None else float(scaling)
    p.out = ops._ptr(out)
    p.sel_idx_out = ops._ptr(selected_out)
    p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel()
    for r in range(world):
        p.exchange[r] = exchange_ptrs[r]
    p.exchange_bytes = int(exchange_bytes)
    p.phases, p.wait_polls = int(phases), int(wait_polls)
    return _native.lib().kvb_sharded_decode_step(C.byref(p), ops._dev(query), ops._stream(query.device))


class CudaBackend:
    """The four device stages of a sharded step composed from kv_cache_b200.ops (the form used around
    all-gathers when the one-call step does not take the shape)."""

    def local_candidates(self, query, packed, scale, channel_idx, t_local: int, k: int, id_offset: int):
        r = ops.score(query, packed, scale, channel_idx, t_local, want_acc=False, want_deq=False, want_hist=True)
        B, Hkv, _ = r.gmax.shape
        idx, sc = ops.select(r.gmax.view(B * Hkv, t_local), k, idx_offset=id_offset, hist=r.hist,
                             return_scores=True, index_dtype=torch.int32, order="index")
        return sc, idx

    def merge(self, scores, ids, k: int):
        """scores/ids ``[N,R,kk]`` -> global winners int32 ``[R,min(k, N*kk)]`` ascending by id."""
        N, R, kk = scores.shape
        s = scores.permute(1, 0, 2).reshape(R, N * kk).contiguous()
        i = ids.permute(1, 0, 2).reshape(R, N * kk).contiguous()
        return ops.select(s, k, payload=i, index_dtype=torch.int32, order="index")

    def attend_partial(self, query, key, value, selected, t_local: int, id_base: int, keep_self: bool, scaling):
        return ops.attend_selected(query, key, value, selected, t_local, id_base=id_base, keep_self=keep_self,
                                   scaling=scaling, return_partial=True)

    def combine(self, partials):
        return ops.lse_merge(partials)


class ShardedSparseDecode:
    """One layer's sharded decode step. All ranks of ``group`` call ``step`` collectively. Without an
    initialised process group it is a world of one (the same code path, exchange buffers local)."""

    def __init__(self, top_k: int, group: Optional[dist.ProcessGroup] = None, backend=None,
                 total_tokens: Optional[int] = None, wait_polls: int = 0):
        self.top_k = int(top_k)
        self.group = group
        self.backend = backend if backend is not None else CudaBackend()
        on = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if on else 0
        self.world = dist.get_world_size(group) if on else 1
        self.total_tokens = total_tokens      # global history length: needed by the one-call step
        self.wait_polls = int(wait_polls)
        self._fast: Optional[bool] = None     # agreed by all ranks on the first step
        self._ws: Optional[torch.Tensor] = None
        self._out: Optional[torch.Tensor] = None
        self._sel: Optional[torch.Tensor] = None
        self.exchange: Optional[PeerExchange] = None

    def close(self) -> None:
        if self.exchange is not None:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)
            self.exchange.close()
            self.exchange = None

    def _prepare_fast(self, query, key_local, packed, scale, channel_idx, t_local: int, id_offset: int) -> bool:
        """Decides, identically on all ranks, whether the one-call step applies, and sets it up."""
        q3 = ops._query3(query)
        B, Hq, D = q3.shape
        Hkv = key_local.shape[1]
        lib = _native.lib()
        ok = isinstance(self.backend, CudaBackend) and q3.is_cuda and self.total_tokens is not None
        if ok:
            # a dry call of phase 1's checks: kvb_shard_candidates refuses what the front end cannot take
            ok = self.top_k <= t_local and self.world <= 8 and D == 128 and lib.kvb_candidate_capacity(self.top_k) > 0
            ok = ok and ops.shard_candidates(query, packed, scale, channel_idx, t_local, self.top_k, id_offset) is not None
        if self.world > 1:
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=query.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            ok = bool(flag.item())
        if ok:
            dev = q3.device
            need = lib.kvb_sharded_step_workspace_bytes(B, Hq, Hkv, t_local, self.top_k)
            self._ws = torch.empty(need, dtype=torch.uint8, device=dev)
            self._out = torch.empty((B, 1, Hq, D), dtype=torch.bfloat16, device=dev)
            self._sel = torch.empty((B, Hkv, self.top_k), dtype=torch.int32, device=dev)
            xbytes = lib.kvb_sharded_exchange_bytes(B, Hq, Hkv, self.top_k, self.world)
            self.exchange = PeerExchange(xbytes, dev, self.rank, self.world, self.group)
        return ok

    def capture(self, *args, **kwargs):
        """Captures one step into a CUDA graph after two eager warm-up steps; returns ``(graph, outputs)``:
        replaying the graph refreshes ``outputs`` in place. All ranks must capture and replay together."""
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(2):
                self.step(*args, **kwargs)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                outputs = self.step(*args, **kwargs)
        stream.synchronize()
        return graph, outputs

    def step(self, query: torch.Tensor, key_local: torch.Tensor, value_local: torch.Tensor, packed: torch.Tensor,
             scale: torch.Tensor, channel_idx: torch.Tensor, t_local: int, id_offset: int,
             scaling: Optional[float] = None):
        """``key_local`` / ``value_local`` hold this rank's ``t_local`` history rows followed by the
        row of the decoded token (``[B,Hkv,t_local+1,D]``); ``id_offset`` is the global id of local
        row 0. Returns ``(out [B,1,Hq,D] bf16, selected int32 [B,Hkv,k] global ids)``, the same set on
        every rank (ascending from the composed form, in no particular order from the one-call step)."""
        be, N = self.backend, self.world
        B, Hkv = key_local.shape[0], key_local.shape[1]
        if self._fast is None:
            self._fast = self._prepare_fast(query, key_local, packed, scale, channel_idx, t_local, id_offset)
        if self._fast:
            rc = sharded_decode_step(query, key_local, value_local, packed, scale, channel_idx, t_local, id_offset,
                                     self.total_tokens, self.top_k, self.rank, N, self.exchange.ptrs,
                                     self.exchange.nbytes, self._ws, self._out, self._sel, scaling,
                                     wait_polls=self.wait_polls)
            check(rc, "kvb_sharded_decode_step")
            return self._out, self._sel
        sc, idx = be.local_candidates(query, packed, scale, channel_idx, t_local, self.top_k, id_offset)
        R, kk = sc.shape
        # pack (score bits, id) into one buffer so that a single all-gather carries both
        mine = torch.stack((sc.contiguous().view(torch.int32), idx.to(torch.int32)), dim=0).contiguous()
        if N > 1:
            # shards may differ by one token, so kk can differ when k > t_local: pad to the common kk
            kk_all = [None] * N
            if self.top_k > t_local:
                dist.all_gather_object(kk_all, kk, group=self.group)
            else:
                kk_all = [kk] * N
            kk_max = max(kk_all)
            if kk < kk_max:
                # padding entries: the lowest possible score and ids no real token has, distinct within the row
                # (the select requires unique ids) and across ranks
                npad = kk_max - kk
                pad = torch.empty((2, R, npad), dtype=torch.int32, device=mine.device)
                pad[0] = torch.tensor(float("-inf")).view(torch.int32).item()
                top = torch.iinfo(torch.int32).max - self.rank * kk_max
                pad[1] = (top - torch.arange(npad, device=mine.device, dtype=torch.int64)).to(torch.int32)
                mine = torch.cat((mine, pad), dim=2).contiguous()
            gathered = _all_gather(mine, N, self.group)                 # [N, 2, R, kk_max]
            sel = be.merge(gathered[:, 0].view(torch.float32), gathered[:, 1], self.top_k)
            total_real = sum(kk_all)
            if sel.shape[-1] > total_real:               # fewer real candidates than k: drop the padding
                sel = sel[:, :total_real]
        else:
            sel = be.merge(mine[0].view(torch.float32)[None], mine[1][None], self.top_k)
        sel = sel.view(B, Hkv, -1).contiguous()
        keep_self = self.rank == N - 1
        part = be.attend_partial(query, key_local, value_local, sel, t_local, id_offset, keep_self, scaling)
        if N > 1:
            parts = _all_gather(part, N, self.group)
        else:
            parts = part[None]
        return be.combine(parts), sel


def make_shard(w, rank: int, world: int, dev: torch.device):
    """This rank's slice of workload ``w``: K/V rows [t0, t1) plus the decoded token's row, the query, the
    channel list (identical on all ranks: mean |K| summed over the shards) and the int4 side cache."""
    from . import inputs

    B, Hkv, D, T, C_ = w.batch, w.kv_heads, w.head_dim, w.context, w.channels
    t0, t1 = shard_bounds(T, world, rank)
    t_local = t1 - t0
    key = torch.empty((B, Hkv, t_local + 1, D), dtype=torch.bfloat16, device=dev)
    value = torch.empty_like(key)
    for b in range(B):                                           # one batch row at a time: bounded temporaries
        kb, vb = inputs.make_kv(w, dev, t0, t1, batch_rows=range(b, b + 1))
        key[b, :, :t_local], value[b, :, :t_local] = kb[0], vb[0]
        ks, vs = inputs.make_kv(w, dev, T, T + 1, batch_rows=range(b, b + 1))
        key[b, :, t_local:], value[b, :, t_local:] = ks[0], vs[0]
    query = inputs.make_query(w, dev)
    tot = torch.zeros((Hkv, D), dtype=torch.float64, device=dev)
    for s in range(0, t_local, 65536):
        tot += key[:, :, s:min(s + 65536, t_local)].float().abs().sum(dim=(0, 2), dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tot)
    order = torch.sort(tot, dim=-1, descending=True, stable=True).indices[:, :C_]
    ch = torch.sort(order, dim=-1).values.to(torch.int32).contiguous()
    packed, scale = ops.alloc_side_cache(B, Hkv, t_local + 1, C_, dev)
    ops.quantize(key[:, :, :t_local], ch, out=(packed, scale))
    torch.cuda.synchronize()
    return dict(key=key, value=value, query=query, ch=ch, packed=packed, scale=scale, t0=t0, t_local=t_local)
