"""Sequence-sharded sparse decode: the KV cache of every sequence is split along the token axis
across the ranks of one node (one process per GPU, torch.distributed / NCCL).

Rank r owns history tokens [r*T/N, (r+1)*T/N) (bf16 K/V and the int4 side cache); the query, the
channel list and the K/V row of the token being decoded are replicated. One decode step:

  1. local  : int4 score of the shard, local top-k per KV head -> (score, GLOBAL token id) lists
  2. gather : ONE all-gather of the packed (score, id) lists            [N, 2, B*Hkv, kk] int32
  3. merge  : every rank selects the global top-k from the N lists with the same rule
              (score desc, id asc): identical result on every rank, independent of rank order
  4. attend : each rank attends to the selected ids it owns (the last rank also to the decoded
              token) and emits un-normalised partials (o, m, l)
  5. gather : ONE all-gather of the partials [N, B, Hq, D+2], log-sum-exp combine on every rank

Both collectives move at most a few MiB: they are latency-bound, never bandwidth-bound. Remote
data always lands in local memory through the collective before a kernel reads it.

The reference (littlexi001/kv_cache) has no sharded path; the single-GPU operators it composes
are those of kv_cache_b200.ops. The compute backend is pluggable so that the rank/plumbing logic
can be exercised on CPU ranks (gloo) with a checker backend; the default backend is the CUDA one
and has no fallback.
"""
from __future__ import annotations

import json
import os
import statistics
import time
from typing import Optional

import torch
import torch.distributed as dist

from . import ops


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


class CudaBackend:
    """The four device stages of a sharded step on kv_cache_b200.ops."""

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
    """One layer's sharded decode step. All ranks of ``group`` call ``step`` collectively."""

    def __init__(self, top_k: int, group: Optional[dist.ProcessGroup] = None, backend=None,
                 total_tokens: Optional[int] = None):
        self.top_k = int(top_k)
        self.group = group
        self.backend = backend if backend is not None else CudaBackend()
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.total_tokens = total_tokens      # global history length: enables the one-kernel merge (ascending ids)
        self._fast: Optional[bool] = None     # agreed by all ranks on the first step
        self._ws: Optional[torch.Tensor] = None

    def _fast_step(self, query, key_local, value_local, packed, scale, channel_idx, t_local, id_offset, scaling):
        """Front end and merge as single C calls: sampled-threshold candidate scorer -> exact local
        top-k as composites -> ONE all-gather -> one-kernel global merge. Returns None when this
        configuration has no candidate front end."""
        N = self.world
        B, Hkv = key_local.shape[0], key_local.shape[1]
        mark = self._mark
        mark("start")
        # Every shard puts its 8192/N best candidates first: the merge then works on those prefixes alone
        # (all on chip) whenever that is provably the global answer, which it is unless one shard holds far
        # more than its share of the winners.
        prefix = min(self.top_k, 8192 // N) if N > 1 else 0
        comp = ops.shard_candidates(query, packed, scale, channel_idx, t_local, self.top_k, id_offset, self._ws,
                                    split_k=prefix)
        if comp is None:
            return None
        mark("local top-k")
        gathered = _all_gather(comp, N, self.group) if N > 1 else comp[None]
        mark("all-gather candidates")
        # the merge also hands this rank the winners it owns, compacted: the attention walks only those
        sel, owned, owned_count = ops.merge_candidates(gathered, self.top_k, self.total_tokens, prefix_k=prefix,
                                                       own=(id_offset, id_offset + t_local))
        sel = sel.view(B, Hkv, -1)
        mark("global merge")
        part = ops.attend_selected(query, key_local, value_local, owned.view(B, Hkv, -1), t_local, id_base=id_offset,
                                   keep_self=self.rank == N - 1, scaling=scaling, return_partial=True,
                                   selected_count=owned_count)
        mark("attend owned rows")
        parts = _all_gather(part, N, self.group) if N > 1 else part[None]
        mark("all-gather partials")
        out = self.backend.combine(parts)
        mark("LSE combine")
        return out, sel

    def _mark(self, name: str) -> None:
        """Stage timing hook: records a CUDA event when ``self.stage_events`` is a list (eager runs only)."""
        ev = getattr(self, "stage_events", None)
        if ev is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            ev.append((name, e))

    def capture(self, *args, **kwargs):
        """Captures one step (collectives included) into a CUDA graph after two eager warm-up steps;
        returns ``(graph, outputs)``: replaying the graph refreshes ``outputs`` in place. All ranks
        must capture and replay together."""
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
        row 0. Returns ``(out [B,1,Hq,D] bf16, selected int32 [B,Hkv,k] global ids)``, the same on
        every rank."""
        be, N = self.backend, self.world
        B, Hkv = key_local.shape[0], key_local.shape[1]
        if self._fast is None:
            # every rank must take the same path (the paths issue different collectives): agree once
            ok = (isinstance(be, CudaBackend) and self.total_tokens is not None and self.top_k <= t_local
                  and ops.shard_candidates(query, packed, scale, channel_idx, t_local, self.top_k, id_offset) is not None)
            flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=query.device)
            if N > 1:
                dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            self._fast = bool(flag.item())
            if self._fast:
                need = ops._native.lib().kvb_shard_candidates_workspace_bytes(B, Hkv, t_local + 1, self.top_k)
                self._ws = torch.empty(need, dtype=torch.uint8, device=query.device)
        if self._fast:
            return self._fast_step(query, key_local, value_local, packed, scale, channel_idx, t_local, id_offset, scaling)
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
                pad = torch.empty((2, R, kk_max - kk), dtype=torch.int32, device=mine.device)
                pad[0] = torch.tensor(float("-inf")).view(torch.int32).item()
                pad[1] = torch.iinfo(torch.int32).max
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


# ------------------------------------------------------------------------------------------
# benchmark entry (called by bench.py under torchrun for --gpus N > 1)
# ------------------------------------------------------------------------------------------

def bench_main(args, w) -> None:
    from . import inputs

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    B, Hq, Hkv, D, T, C, k = w.batch, w.q_heads, w.kv_heads, w.head_dim, w.context, w.channels, w.top_k
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
    # channel choice must be identical on all ranks: mean |K| summed over the shards
    tot = key[:, :, :t_local].float().abs().sum(dim=(0, 2), dtype=torch.float64) if t_local <= 65536 else sum(
        key[:, :, s:s + 65536].float().abs().sum(dim=(0, 2), dtype=torch.float64) for s in range(0, t_local, 65536))
    dist.all_reduce(tot)
    order = torch.sort(tot, dim=-1, descending=True, stable=True).indices[:, :C]
    ch = torch.sort(order, dim=-1).values.to(torch.int32).contiguous()
    packed, scale = ops.alloc_side_cache(B, Hkv, t_local + 1, C, dev)
    ops.quantize(key[:, :, :t_local], ch, out=(packed, scale))
    torch.cuda.synchronize()

    eng = ShardedSparseDecode(k, total_tokens=T)
    stream = torch.cuda.Stream(dev)

    def run():
        return eng.step(query, key, value, packed, scale, ch, t_local, t0)

    from .benchutil import METRIC, UNIT, ClockSampler, hbm_peak

    # The step is captured into a CUDA graph (kernels and both NCCL all-gathers). A capture failure is
    # fatal on purpose: falling back on one rank only would leave the ranks issuing different collectives.
    graph = None
    if os.environ.get("KVB_SHARDED_EAGER") == "1":
        launch = "eager Python step"
    else:
        graph, (out, sel) = eng.capture(query, key, value, packed, scale, ch, t_local, t0)
        run = graph.replay
        launch = "CUDA graph replay (kernels and both NCCL all-gathers captured)"

    if os.environ.get("KVB_SHARDED_STAGES") == "1":
        # per-stage device times of eager steps (host launch gaps included), printed by rank 0 to stderr
        import sys
        acc: dict = {}
        for it in range(25):
            eng.stage_events = []
            eng.step(query, key, value, packed, scale, ch, t_local, t0)
            torch.cuda.synchronize()
            ev = eng.stage_events
            if it >= 5:
                for (n0, e0), (n1, e1) in zip(ev, ev[1:]):
                    acc.setdefault(n1, []).append(e0.elapsed_time(e1) * 1e3)
        eng.stage_events = None
        if rank == 0:
            print("stage medians (us): " + ", ".join(f"{n}={statistics.median(v):.1f}" for n, v in acc.items()), file=sys.stderr)

    with torch.cuda.stream(stream):
        for _ in range(max(3, args.warmup)):
            run()
        stream.synchronize()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nrep = max(1, int(1000.0 / max(0.3 * args.steps, 1e-3)))     # about a second of timed work
        start.record(stream)
        for _ in range(args.steps * nrep):
            run()
        end.record(stream)
        dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([start.elapsed_time(end) / (args.steps * nrep)], dtype=torch.float64, device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        clocks = sampler.stop() if rank == 0 else None

        # end to end: the step's inputs from pinned host memory, the output back to the host
        h_q = torch.empty_like(query, device="cpu").pin_memory()
        h_q.copy_(query)
        h_kv = torch.empty((2, B, Hkv, 1, D), dtype=torch.bfloat16).pin_memory()
        h_kv[0].copy_(key[:, :, t_local:])
        h_kv[1].copy_(value[:, :, t_local:])
        h_out = torch.empty((B, 1, Hq, D), dtype=torch.bfloat16).pin_memory()
        d_q = torch.empty_like(query)

        def e2e_step():
            d_q.copy_(h_q, non_blocking=True)
            key[:, :, t_local:].copy_(h_kv[0], non_blocking=True)
            value[:, :, t_local:].copy_(h_kv[1], non_blocking=True)
            o, _ = eng.step(d_q, key, value, packed, scale, ch, t_local, t0)
            h_out.copy_(o, non_blocking=True)
            stream.synchronize()

        for _ in range(3):
            e2e_step()
        dist.barrier()
        tw = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        e2e = torch.tensor([(time.perf_counter() - tw) * 1e3 / args.steps], dtype=torch.float64, device=dev)
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)

    if rank == 0:
        ms_step, e2e_ms = float(ms.item()), float(e2e.item())
        tokens = B * T
        alg = w.algorithmic_bytes()
        peak, peak_kind = hbm_peak()
        line = {
            "metric": METRIC, "value": tokens / (ms_step * 1e-3) / 1e3, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "int4xint8->int32 scores, bf16 attention (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": w.name, "batch": B, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": T,
                       "partial_channels": C, "top_k": k, "sharding": f"sequence/{world}",
                       "collectives": "2 NCCL all-gathers per step (candidates, LSE partials)", "launch": launch,
                       "l2": "inputs larger than L2 (scan stream %d MiB per rank)" % ((alg["scan"] // world) >> 20)},
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms * 1e-3) / 1e3, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (h_q.numel() + h_kv.numel()) * 2, "d2h_bytes_per_step": h_out.numel() * 2,
                    "api": "kv_cache_b200.sharded.ShardedSparseDecode.step"},
            "gpu_launches": 9 * args.steps * world,
            "roofline": {"bound": "hbm", "kernel": "whole sharded step, per rank", "achieved":
                         alg["total"] / world / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg["total"] / world / (ms_step * 1e-3) / 1e9 / peak, "peak_source": peak_kind,
                         "traffic": None, "algorithmic_bytes": alg["total"] // world},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    # Teardown: drop the captured graph (it references the communicator) before anything else, and leave
    # without tearing the process group down: destroying a communicator that a captured graph used
    # has been seen to block forever, and the process is about to exit anyway.
    graph = None
    run = None
    torch.cuda.synchronize()
    dist.barrier()
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
