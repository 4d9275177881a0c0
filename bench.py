#!/usr/bin/env python
"""Benchmark of the retrieval-sparse decode attention step (one layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c0|c1|c3|c4]

Metric: K tokens scored+attended per second = B * T * steps / seconds / 1e3 for one layer's
decode step (score all T cached int4 keys, select top-k per KV head, attend over the selected
rows, append the new token to the int4 cache). One JSON line is printed by rank 0.

  value     whole step, inputs resident in HBM, CUDA-graph replay, CUDA events
  e2e       the same step through the Python operator (ops.GraphedDecode / sharded step) with the
            step's inputs (query, new K/V row) copied from pinned host memory and the output
            copied back, every step, inside the timed region. The KV cache itself is device
            state (it is what "cache" means), like weights in a training step.
  roofline  the dominant kernel (the int4 scorer): algorithmic bytes / CUDA-event time of that
            kernel alone, against the measured HBM copy bandwidth in MEASURED_PEAKS.json
  parity    after the timed region (untimed): one seeded (batch row, KV head) of the very outputs
            the timed graph wrote is recomputed by the CPU oracle; ids must be equal, outputs in tolerance
  secondary (--gpus 1, default workload) config 4 on one GPU through the sharded step as a world of
            one, config 3 (chunked-prefill block scoring, both tcgen05 encodings) and the bulk quantizer
  cpu_baseline  the reference's torch CPU op chain for this step (oracle port), timed on this
            box's host cores on one batch row of the same workload

--gpus N > 1 (under torchrun) runs config 4 sequence-sharded over N ranks (strong scaling; the N = 1
point of the same workload is `secondary.c4_n1` of the --gpus 1 line, or `--gpus 1 --workload c4`).
--impl reference times only the CPU chain (all host threads) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from kv_cache_b200.benchutil import METRIC, UNIT, ClockSampler, hbm_peak  # noqa: E402

DTYPE = "int4xint8->int32 scores, bf16 attention (fp32 accumulate)"
# dram__bytes_read.sum + dram__bytes_write.sum of one score_decode_stream_kernel launch at config 2 with
# batch 4 (ncu capture summarised in profiles/): the traffic of a full launch is that times batch / 4
# (the kernel streams every row exactly once, so its traffic is proportional to the rows).
SCORER_DRAM_BYTES_BATCH4_C2 = 151.10e6 + 4.08e6


# ------------------------------------------------------------------------------------------
# CPU arm and the parity checker (the only users of oracle/ outside tests/ and the smoke check)
# ------------------------------------------------------------------------------------------

def cpu_reference_sample(w, steps: int, warmup: int) -> dict:
    """Times the reference's torch CPU chain (EVAL:6248-6251 + EVAL:4400-4502, restated in
    oracle.qabs_candidate_attention) on ONE batch row of the workload, all heads, full context.
    Long contexts are cut to 131072 tokens so that a run stays within minutes."""
    from kv_cache_b200 import inputs
    from oracle import oracle

    torch.set_num_threads(os.cpu_count() or 1)          # torchrun exports OMP_NUM_THREADS=1
    T = min(w.context, 131072)
    ws = inputs.Workload(w.name, 1, w.q_heads, w.kv_heads, w.head_dim, T, w.channels,
                         max(1, round(w.top_k * T / w.context)), w.seed)
    key, value = inputs.make_kv(ws, "cpu", 0, T + 1)
    query = inputs.make_query(ws, "cpu")[:, :, None, :]
    dims, frac = ws.channels, ws.top_k / T
    scaling = ws.head_dim ** -0.5
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.qabs_candidate_attention(query, key, value, None, scaling, dims, frac)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return {
        "value": T / sec / 1e3, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
        "ms_per_step": sec * 1e3, "host_cpus": os.cpu_count(),
        "sample": f"reference torch op chain (repeat KV, fp32 |q|-top-{dims} partial scores, torch.topk {ws.top_k}, "
                  f"gathered bf16 attention) on 1 of {w.batch} batch rows, {ws.q_heads} heads, T={T}; "
                  f"{steps} steps after {warmup} warm-up",
    }


def run_reference_arm(args, w) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    base = cpu_reference_sample(w, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
        "dtype": "fp32 scores / bf16 attention (CPU)", "data": "synthetic",
        "config": {"workload": w.name, "sample": base["sample"]},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def oracle_parity(w, row: tuple[int, int], key_row: torch.Tensor, value_row: torch.Tensor, query: torch.Tensor,
                  ch: torch.Tensor, sel: torch.Tensor, out: torch.Tensor) -> dict:
    """Untimed check of one (batch row, KV head) of the outputs the timed graph wrote against the CPU oracle
    (oracle.decode_step on that row's whole K/V): the selected ids must be the oracle's set, the G output
    heads within 2e-2 relative / 1e-2 absolute. ``key_row`` / ``value_row``: ``[1,1,T+1,D]`` on any device."""
    from oracle import oracle

    b, h = row
    G = w.q_heads // w.kv_heads
    r = oracle.decode_step(query[b:b + 1, h * G:(h + 1) * G].cpu(), key_row.cpu(), value_row.cpu(), ch[h:h + 1].cpu(),
                           w.top_k)
    want = torch.sort(r["selected"][0, 0]).values
    got = torch.sort(sel[b, h].cpu().long()).values
    o = out[b, 0, h * G:(h + 1) * G].float().cpu()
    ref = r["out"][0, 0]
    err = (o - ref).abs()
    return {"row": [b, h], "indices_equal": bool(torch.equal(want, got)), "max_abs_err": float(err.max()),
            "within_tolerance": bool((err <= 1e-2 + 2e-2 * ref.abs()).all()), "tolerance": "2e-2 rel / 1e-2 abs",
            "checker": "oracle.decode_step on the whole row (CPU), against the outputs of the timed graph"}


def parity_row(w) -> tuple[int, int]:
    return (w.seed * 7 + 3) % w.batch, (w.seed * 5 + 1) % w.kv_heads


# ------------------------------------------------------------------------------------------
# GPU arm, one GPU, un-sharded step
# ------------------------------------------------------------------------------------------

def event_time_ms(fn, iters: int, stream) -> float:
    """Average milliseconds of fn() over `iters` back-to-back calls, CUDA events on `stream`."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(iters):
        fn()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def run_single_gpu(args, w, with_secondary: bool) -> None:
    from kv_cache_b200 import _native, inputs, ops

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, Hq, Hkv, D, T, C, k = w.batch, w.q_heads, w.kv_heads, w.head_dim, w.context, w.channels, w.top_k

    t_setup = time.perf_counter()
    key, value = inputs.make_kv(w, dev, 0, T + 1)
    query = inputs.make_query(w, dev)
    ch = ops.choose_channels(key[:, :, :T], C)
    packed, scale = ops.alloc_side_cache(B, Hkv, T + 1, C, dev)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_setup

    # any-order selection: the exact top-k set without the ordering pass (see kvb_decode_step_params)
    step = ops.DecodeStep(k, ordered_selection=False)
    out = torch.empty((B, 1, Hq, D), dtype=torch.bfloat16, device=dev)
    sel = torch.empty((B, Hkv, min(k, T)), dtype=torch.int32, device=dev)
    stream = torch.cuda.Stream(dev)

    def run_step():
        step(query, key, value, packed, scale, ch, out=out, selected_out=sel)

    with torch.cuda.stream(stream):
        for _ in range(3):
            run_step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run_step()
        for _ in range(max(3, args.warmup)):
            graph.replay()
        stream.synchronize()

        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        time.sleep(0.3)
        ms_step = event_time_ms(graph.replay, args.steps, stream)
        # more timed blocks of `steps` replays (about a second in all) so that the clock sampler sees
        # a loaded GPU; the reported step time is the median block
        nrep = max(4, min(400, int(1000.0 / max(ms_step * args.steps, 1e-3))))
        repeats = [ms_step] + [event_time_ms(graph.replay, args.steps, stream) for _ in range(nrep)]
        ms_step = statistics.median(repeats)
        out_timed, sel_timed = out.clone(), sel.clone()         # what the timed graph wrote

        # dominant kernel alone: the scorer in the form the step uses (candidate emission), same stream
        lib = _native.lib()
        cap = lib.kvb_candidate_capacity(k)
        _, _, tau = ops.score_candidates(query, packed, scale, ch, T, k)
        cand = torch.empty((B * Hkv, cap), dtype=torch.int64, device=dev)
        count = torch.zeros((B * Hkv, 32), dtype=torch.int32, device=dev)

        def run_scorer():
            count.zero_()
            rc = lib.kvb_score_candidates(query.data_ptr(), query.stride(0), query.stride(1), packed.data_ptr(),
                                          packed.stride(0), packed.stride(1), scale.data_ptr(), scale.stride(0),
                                          scale.stride(1), ch.data_ptr(), B, Hq, Hkv, T, D, C, tau.data_ptr(),
                                          cand.data_ptr(), count.data_ptr(), cap, dev.index or 0, stream.cuda_stream)
            assert rc == 0, rc

        for _ in range(3):
            run_scorer()
        ms_scorer = event_time_ms(run_scorer, max(args.steps, 20), stream)
        clocks = sampler.stop()

        # end to end through the public graph API with host buffers: every step copies the query and
        # the new K/V row from pinned host memory, scatters the row into the cache at the device-side
        # position, runs the fused step and copies the output back; the host waits for it.
        # (advance=False keeps the history at T so that every timed step is the same workload.)
        gd = ops.GraphedDecode(step, key, value, packed, scale, ch, history=T, q_heads=Hq, advance=False)
        gd.h_query.copy_(query)
        gd.h_key_row.copy_(key[:, :, T:T + 1])
        gd.h_value_row.copy_(value[:, :, T:T + 1])
        for _ in range(3):
            gd()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            h_out = gd()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        h_q, h_k, h_v = gd.h_query, gd.h_key_row, gd.h_value_row
        e2e_equal = bool(torch.equal(h_out.cpu(), out_timed.cpu())) if step.ordered_selection else None

    b_chk, h_chk = parity_row(w)
    parity = oracle_parity(w, (b_chk, h_chk), key[b_chk:b_chk + 1, h_chk:h_chk + 1], value[b_chk:b_chk + 1, h_chk:h_chk + 1],
                           query, ch, sel_timed, out_timed)
    e2e_err = (h_out.float() - out_timed.float().cpu()).abs().max().item()

    tokens = B * T
    peak, peak_kind = hbm_peak()
    alg = w.algorithmic_bytes()
    if alg["total"] > (126 << 20):
        l2_note = "inputs larger than L2 (scan stream %d MiB)" % (alg["scan"] >> 20)
    else:
        l2_note = "working set of %d MiB fits the 126 MB L2: a latency figure, not a bandwidth one" % (alg["total"] >> 20)
    scorer_gbs = alg["scan"] / (ms_scorer * 1e-3) / 1e9
    step_gbs = alg["total"] / (ms_step * 1e-3) / 1e9
    traffic = None
    if w.name.startswith("c2_"):
        traffic = SCORER_DRAM_BYTES_BATCH4_C2 * B / 4.0
    cpu = None
    if not args.no_cpu_baseline:
        cpu = cpu_reference_sample(w, 2, 1)

    secondary = None
    if with_secondary:
        secondary = {}
        w4 = inputs.WORKLOADS["c4"]
        r4 = measure_sharded(w4, max(5, args.steps // 2), 3, dev)
        a4 = w4.algorithmic_bytes()
        secondary["c4_n1"] = {
            "workload": w4.name, "ms_per_step": r4["ms_step"], "value": w4.batch * w4.context / (r4["ms_step"] * 1e-3) / 1e3,
            "unit": UNIT, "e2e_ms_per_step": r4["e2e_ms"], "whole_step_frac": a4["total"] / (r4["ms_step"] * 1e-3) / 1e9 / peak,
            "path": "kvb_sharded_decode_step as a world of one (the code the N >= 2 lines run), CUDA graph replay",
            "parity": r4["parity"]}
        torch.cuda.empty_cache()
        secondary["c3"] = measure_prefill(2, 4096, max(3, args.steps // 4), 3, dev)
        torch.cuda.empty_cache()
        secondary["bulk_quantize"] = measure_quantize(dev)

    line = {
        "metric": METRIC, "value": tokens / (ms_step * 1e-3) / 1e3, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": w.name, "batch": B, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": T,
                   "partial_channels": C, "top_k": k, "l2": l2_note,
                   "launch": "CUDA graph replay of kvb_decode_step (selected ids in any order)", "setup_s": round(setup_s, 1),
                   "timed_blocks": len(repeats), "step_ms_min_med_max": [round(min(repeats), 4), round(ms_step, 4), round(max(repeats), 4)]},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms * 1e-3) / 1e3, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h_q.numel() * 2 + h_k.numel() * 2 + h_v.numel() * 2,
                "d2h_bytes_per_step": h_out.numel() * 2, "max_abs_diff_vs_timed_output": e2e_err,
                "api": "kv_cache_b200.ops.GraphedDecode.__call__ (H2D + kvb_decode_step + D2H in one CUDA graph, device-side history length)"},
        "gpu_launches": 5 * args.steps,      # sample, scorer, final select, attend, merge per replayed step
        "roofline": {"bound": "hbm", "kernel": "score_decode_stream_kernel (candidate form)", "achieved": scorer_gbs, "peak": peak,
                     "unit": "GB/s", "frac": scorer_gbs / peak, "peak_source": peak_kind, "traffic": traffic,
                     "traffic_source": None if traffic is None else "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at batch 4, scaled by batch / 4",
                     "algorithmic_bytes": alg["scan"], "kernel_ms": ms_scorer,
                     "whole_step": {"algorithmic_bytes": alg["total"], "achieved": step_gbs, "frac": step_gbs / peak}},
        "parity": parity,
        "cpu_baseline": cpu,
    }
    if secondary is not None:
        line["secondary"] = secondary
    if e2e_equal is not None:
        line["e2e"]["equal_to_timed_output"] = e2e_equal
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# sequence-sharded step (config 4): N ranks under torchrun, or a world of one
# ------------------------------------------------------------------------------------------

def measure_sharded(w, steps: int, warmup: int, dev: torch.device) -> dict:
    """Times the sharded step of workload ``w`` on the ranks of the default process group (a world of one
    without it): CUDA-graph replays, CUDA events, max over ranks; then the end-to-end form (the step's
    inputs copied from pinned host memory and the output copied back inside one graph, the host waiting
    every step); then, on rank 0, the parity check of the timed outputs against the un-sharded oracle."""
    import torch.distributed as dist
    from kv_cache_b200 import inputs
    from kv_cache_b200.sharded import ShardedSparseDecode, make_shard

    on = dist.is_available() and dist.is_initialized()
    rank = dist.get_rank() if on else 0
    world = dist.get_world_size() if on else 1
    B, Hq, Hkv, D, T, k = w.batch, w.q_heads, w.kv_heads, w.head_dim, w.context, w.top_k
    t_setup = time.perf_counter()
    s = make_shard(w, rank, world, dev)
    setup_s = time.perf_counter() - t_setup
    key, value, query, ch, packed, scale, t0, t_local = (s[n] for n in ("key", "value", "query", "ch", "packed", "scale",
                                                                         "t0", "t_local"))
    eng = ShardedSparseDecode(k, total_tokens=T)
    graph, (out, sel) = eng.capture(query, key, value, packed, scale, ch, t_local, t0)
    one_call = bool(eng._fast)
    stream = torch.cuda.Stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.cuda.stream(stream):
        for _ in range(max(3, warmup)):
            graph.replay()
        stream.synchronize()
        sampler = ClockSampler(dev.index or 0)
        if rank == 0:
            sampler.start()
        barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nrep = max(1, int(800.0 / max(0.3 * steps, 1e-3)))            # the better part of a second of timed work
        start.record(stream)
        for _ in range(steps * nrep):
            graph.replay()
        end.record(stream)
        barrier()
        torch.cuda.synchronize()
        ms_step = max_over_ranks(start.elapsed_time(end) / (steps * nrep))
        clocks = sampler.stop() if rank == 0 else None
        out_timed, sel_timed = out.clone(), sel.clone()

        # end to end: one graph = H2D of the step's inputs, the step, D2H of the output
        nq, nkv = query.numel(), B * Hkv * D
        h_in = torch.empty((nq + 2 * nkv,), dtype=torch.bfloat16).pin_memory()
        h_in[:nq].copy_(query.reshape(-1))
        h_in[nq:nq + nkv].copy_(key[:, :, t_local].reshape(-1))
        h_in[nq + nkv:].copy_(value[:, :, t_local].reshape(-1))
        d_in = torch.empty(h_in.shape, dtype=torch.bfloat16, device=dev)
        d_q = d_in[:nq].view(B, Hq, D)
        h_out = torch.empty((B, 1, Hq, D), dtype=torch.bfloat16).pin_memory()

        def e2e_body():
            d_in.copy_(h_in, non_blocking=True)
            key[:, :, t_local].copy_(d_in[nq:nq + nkv].view(B, Hkv, D))
            value[:, :, t_local].copy_(d_in[nq + nkv:].view(B, Hkv, D))
            o, _ = eng.step(d_q, key, value, packed, scale, ch, t_local, t0)
            h_out.copy_(o, non_blocking=True)

        e2e_body()
        stream.synchronize()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=stream):
            e2e_body()

        def e2e_step():
            g2.replay()
            stream.synchronize()

        for _ in range(3):
            e2e_step()
        barrier()
        tw = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        e2e_ms = max_over_ranks((time.perf_counter() - tw) * 1e3 / steps)

    parity = None
    if rank == 0:
        b_chk, h_chk = parity_row(w)
        kb, vb = inputs.make_kv(w, dev, 0, T + 1, batch_rows=range(b_chk, b_chk + 1))      # the row's shards, all of them
        parity = oracle_parity(w, (b_chk, h_chk), kb[:, h_chk:h_chk + 1], vb[:, h_chk:h_chk + 1], query, ch, sel_timed,
                               out_timed)
        parity["e2e_max_abs_diff_vs_timed_output"] = (h_out.float() - out_timed.float().cpu()).abs().max().item()
        del kb, vb
    barrier()
    graph = g2 = None
    eng.close()
    return dict(ms_step=ms_step, e2e_ms=e2e_ms, clocks=clocks, parity=parity, world=world, rank=rank, one_call=one_call,
                setup_s=setup_s, h2d=h_in.numel() * 2, d2h=h_out.numel() * 2, timed_steps=steps * nrep)


def run_sharded(args, w) -> None:
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    under_torchrun = "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1
    if under_torchrun and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    r = measure_sharded(w, args.steps, args.warmup, dev)
    world = r["world"]
    if rank == 0:
        B, Hq, Hkv, D, T, Cc, k = w.batch, w.q_heads, w.kv_heads, w.head_dim, w.context, w.channels, w.top_k
        ms_step, e2e_ms = r["ms_step"], r["e2e_ms"]
        tokens = B * T
        alg = w.algorithmic_bytes()
        peak, peak_kind = hbm_peak()
        cpu = None if args.no_cpu_baseline else cpu_reference_sample(w, 2, 1)
        line = {
            "metric": METRIC, "value": tokens / (ms_step * 1e-3) / 1e3, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": w.name, "batch": B, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D, "context": T,
                       "partial_channels": Cc, "top_k": k, "sharding": f"sequence/{world}",
                       "exchange": ("no collective in the step: candidate prefixes and LSE partials are stored into "
                                    "peer memory over NVLink under step-numbered flags (kvb_sharded_decode_step)")
                       if r["one_call"] else "2 all-gathers per step (candidates, LSE partials)",
                       "launch": "CUDA graph replay of the 7-kernel step", "timed_steps": r["timed_steps"],
                       "l2": "inputs larger than L2 (scan stream %d MiB per rank)" % ((alg["scan"] // world) >> 20),
                       "setup_s": round(r["setup_s"], 1)},
            "clocks": r["clocks"],
            "e2e": {"value": tokens / (e2e_ms * 1e-3) / 1e3, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"],
                    "api": "kv_cache_b200.sharded.ShardedSparseDecode.step inside one CUDA graph with the H2D copy of "
                           "the step's inputs and the D2H copy of its output; the host waits every step"},
            "gpu_launches": 7 * args.steps * world,
            "roofline": {"bound": "hbm", "kernel": "whole sharded step, per rank", "achieved":
                         alg["total"] / world / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg["total"] / world / (ms_step * 1e-3) / 1e9 / peak, "peak_source": peak_kind,
                         "traffic": None, "algorithmic_bytes": alg["total"] // world},
            "parity": r["parity"],
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# config 3 (chunked-prefill block scoring) and the bulk quantizer
# ------------------------------------------------------------------------------------------

def measure_prefill(B: int, Tq: int, steps: int, warmup: int, dev: torch.device) -> dict:
    """Config 3: Tq queries x 131072 keys, Qwen3-8B shapes. A step = per-token query quantisation + int8 block
    scoring + top-32 blocks per (b, KV head, query); the scorer is also timed alone in both tcgen05 encodings."""
    from kv_cache_b200 import inputs, ops

    Hq, Hkv, D, Tk, C, top_blocks = 32, 8, 128, 131072, 64, 32
    w = inputs.Workload("c3_qwen3-8b_prefill_b%d_tq%d_tk131072_c64_blk64_top32" % (B, Tq), B, Hq, Hkv, D, Tk, C, 0, seed=3)
    key, _ = inputs.make_kv(w, dev, 0, Tk)
    ch = ops.choose_channels(key, C)
    packed, scale = ops.quantize(key, ch)
    del key
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.empty((B, Hq, Tq, D), dtype=torch.bfloat16, device=dev)
    for b in range(B):
        q[b] = inputs.rope(torch.randn(Hq, Tq, D, generator=g, device=dev), torch.arange(Tk, Tk + Tq, device=dev)).to(torch.bfloat16)
    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        def step():
            qc, qs = ops.quantize_query_tokens(q, ch)
            bs = ops.score_prefill_blocks(qc, qs, packed, scale, Tk)
            return ops.block_topk(bs, top_blocks), qc, qs

        for _ in range(max(3, warmup)):
            idx, qc, qs = step()
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        ms_step = event_time_ms(step, steps, stream)
        kernel_ms = {e: event_time_ms(lambda e=e: ops.score_prefill_blocks(qc, qs, packed, scale, Tk, engine=e), steps, stream)
                     for e in ("f16", "i8")}
        wk = ops.WidenedKeys(packed, Tk, "f16")         # operands widened once for all chunks
        kernel_ms["f16w"] = event_time_ms(lambda: ops.score_prefill_blocks(qc, qs, packed, scale, Tk, widened=wk), steps, stream)
        widen_ms = event_time_ms(lambda: wk.update(packed, Tk, 0), steps, stream)
        del wk
        clocks = sampler.stop()
    ops_total = 2.0 * B * Hq * Tq * Tk * C
    best = min(kernel_ms, key=kernel_ms.get)
    return {"workload": w.name, "ms_per_step": ms_step, "tops": ops_total / (ms_step * 1e-3) / 1e12,
            "engine": "f16w (default: key codes widened once per step to fp16 operands in global memory, one bulk copy "
                      "per tile, fp32 accumulators in tensor memory; f16 = widened inside every CTA; i8 = int8 operands, "
                      "int32 accumulators; identical bits)",
            "widen_ms": widen_ms,
            "kernel_ms": kernel_ms, "kernel_tops": {e: ops_total / (v * 1e-3) / 1e12 for e, v in kernel_ms.items()},
            "frac_of_nominal_int8_peak": ops_total / (kernel_ms[best] * 1e-3) / 1e12 / 4500.0, "clocks": clocks,
            "int8_ops": ops_total, "steps": steps}


def run_prefill_gpu(args) -> None:
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B = args.batch or 2
    r = measure_prefill(B, args.queries, args.steps, args.warmup, dev)
    line = {
        "metric": "int8 TOPS, chunked-prefill block scoring", "value": r["tops"],
        "unit": "TOPS", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4->int8, int32 accumulate",
        "data": "synthetic",
        "config": {"workload": r["workload"], "batch": B, "q_heads": 32, "kv_heads": 8, "queries": args.queries,
                   "keys": 131072, "partial_channels": 64, "block": 64, "top_blocks": 32, "engine": r["engine"]},
        "clocks": r["clocks"], "gpu_launches": 4 * args.steps,      # query quantisation, key widening, scorer, block top-k
        "roofline": {"bound": "tensor", "kernel": "score_prefill_tw_kernel (tcgen05, pre-widened operands)",
                     "achieved": max(r["kernel_tops"].values()), "peak": 4500.0, "unit": "TOPS",
                     "frac": r["frac_of_nominal_int8_peak"],
                     "peak_source": "nominal dense int8 (no measured int8 peak on this pool)", "kernel_ms": r["kernel_ms"],
                     "note": "K = 64: every accumulator element is drained from tensor memory after only 64 MACs; the kernel is bound by the per-element scale+max of the epilogue warps, not by the MMAs"},
    }
    print(json.dumps(line), flush=True)


def measure_quantize(dev: torch.device, batch: int = 16) -> dict:
    """Bulk quantize/pack of 4 GiB of bf16 K (config 2's cache of one layer; `batch` scales it), CUDA events."""
    from kv_cache_b200 import ops

    B, Hkv, T, D, C = batch, 8, 131072, 128, 64
    key = torch.empty((B, Hkv, T, D), dtype=torch.bfloat16, device=dev).normal_()
    ch = torch.arange(0, 2 * C, 2, dtype=torch.int32, device=dev).repeat(Hkv, 1)
    packed, scale = ops.alloc_side_cache(B, Hkv, T, C, dev)
    stream = torch.cuda.current_stream(dev)
    for _ in range(3):
        ops.quantize(key, ch, out=(packed, scale))
    ms = event_time_ms(lambda: ops.quantize(key, ch, out=(packed, scale)), 10, stream)
    nbytes = B * Hkv * T * (2 * D + C // 2 + 4)
    peak, _ = hbm_peak()
    return {"ms": ms, "bytes": nbytes, "gb_per_s": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak,
            "what": f"kvb_quantize_pack over bf16 K [{B},8,131072,128] -> int4 codes on 64 channels + fp32 scales"}


def measure_model_decode(steps: int, dev: torch.device, batch: int = 8, context: int = 32768) -> dict:
    """Config 1 as a whole model: the layer stack of Qwen3-0.6B (28 layers, 16 query / 8 KV heads of 128, hidden
    1024, random weights, small vocabulary) decoding one token at a time with `batch` x `context` cached tokens
    per layer. Two arms on the same GPU and the same weights: (a) the patched attention in mode
    qabs32cand3p125attn (32 channels, top 1024 of 32768) over a PreallocatedCache, (b) dense attention over the
    stock DynamicCache, which is what the reference's `baseline` mode runs (EVAL:6602-6604 fed by EVAL:7278).
    The caches are filled with synthetic K/V directly (a 32768-token eager prefill does not fit memory and is
    not what is measured); milliseconds per decoded token, CUDA events, host loop included."""
    from transformers import DynamicCache, Qwen3Config, Qwen3ForCausalLM
    from kv_cache_b200 import attention_patch as ap
    from kv_cache_b200.cache import PreallocatedCache

    torch.manual_seed(1)
    L, Hkv, D = 28, 8, 128
    cfg = Qwen3Config(vocab_size=1024, hidden_size=1024, intermediate_size=3072, num_hidden_layers=L,
                      num_attention_heads=16, num_key_value_heads=Hkv, head_dim=D, max_position_embeddings=40960,
                      rope_theta=1e6, rms_norm_eps=1e-6, attn_implementation="eager")
    model = Qwen3ForCausalLM(cfg).to(dev, torch.bfloat16).eval()
    g = torch.Generator(device=dev).manual_seed(1)
    capacity = context + steps + 8

    def filled_preallocated():
        cache = PreallocatedCache(num_layers=L, capacity=capacity)
        for layer in cache.layers:
            k0 = torch.empty((batch, Hkv, 1, D), dtype=torch.bfloat16, device=dev)
            layer.lazy_initialization(k0, k0)
            layer.key_buffer[:, :, :context].normal_(generator=g)
            layer.value_buffer[:, :, :context].normal_(generator=g)
            layer.length = context
            layer.keys, layer.values = layer.key_buffer[:, :, :context], layer.value_buffer[:, :, :context]
        return cache

    def filled_dynamic():
        cache = DynamicCache(config=cfg)
        for l in range(L):
            k = torch.empty((batch, Hkv, context, D), dtype=torch.bfloat16, device=dev).normal_(generator=g)
            v = torch.empty((batch, Hkv, context, D), dtype=torch.bfloat16, device=dev).normal_(generator=g)
            cache.update(k, v, l)
        return cache

    toks = [torch.randint(0, 1024, (batch, 1), device=dev) for _ in range(steps + 3)]
    pos0 = context

    def run(cache, mode_args, state):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.inference_mode():
            for i, tok in enumerate(toks):
                if i == 3:
                    e0.record()
                position = torch.full((batch, 1), pos0 + i, device=dev, dtype=torch.long)
                with ap.attention_mode(*mode_args, sparse_state=state):
                    model(input_ids=tok, past_key_values=cache, use_cache=True, position_ids=position)
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    ap.install_qwen3_attention_patch()
    try:
        state = ap.SparseDecodeState(capacity_hint=capacity)
        cache = filled_preallocated()
        sparse_ms = run(cache, ("qabs32cand3p125attn", 0.02, 3, True, 0, 0, None), state)
        reallocs = cache.reallocations
        del cache, state
        torch.cuda.empty_cache()
        dense_ms = run(filled_dynamic(), ("baseline",), ap.SparseDecodeState())
    finally:
        ap.uninstall_qwen3_attention_patch()
    torch.cuda.empty_cache()
    return {"workload": f"c1_model_qwen3-0.6b-shaped_28L_b{batch}_t{context}", "decoded_tokens": steps,
            "sparse_ms_per_token": sparse_ms, "dense_dynamic_cache_ms_per_token": dense_ms,
            "tokens_per_s_sparse": batch * 1e3 / sparse_ms, "tokens_per_s_dense": batch * 1e3 / dense_ms,
            "cache_reallocations": reallocs,
            "what": "whole-model decode, host loop and all 28 layers' MLPs included; the int4 side caches of the "
                    "28 layers are built during the first (untimed) token"}


def main() -> None:
    # Only the JSON line belongs on stdout, but native libraries write there too (NCCL prints a version banner at
    # NCCL_DEBUG=VERSION and above): file descriptor 1 is pointed at stderr for the whole run and Python's own
    # sys.stdout keeps the original descriptor.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w", buffering=1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the config 4 / config 3 / quantizer block of the default run")
    ap.add_argument("--queries", type=int, default=4096, help="query chunk length of the prefill workload (c3)")
    ap.add_argument("--context", type=int, default=None,
                    help="override the workload's history length (e.g. the per-rank shard length of a sharded run)")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's batch (smaller device footprint for profiler captures)")
    args = ap.parse_args()

    from kv_cache_b200 import inputs

    name = args.workload or ("c2" if args.gpus == 1 else "c4")
    if name == "quantize":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no int4 quantizer (north-star stage 1)"}))
            return
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        print(json.dumps(measure_quantize(dev, batch=args.batch or 16)), flush=True)
        return
    if name == "c1_model":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "whole-model decode is a secondary measurement; the reference arm times the layer step"}))
            return
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        print(json.dumps(measure_model_decode(max(4, min(args.steps, 32)), dev, batch=args.batch or 8)), flush=True)
        return
    if name == "c3":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no chunked-prefill scorer (query_count must be 1, EVAL:4413)"}))
            return
        run_prefill_gpu(args)
        return
    w = inputs.WORKLOADS[name]
    if args.batch:
        w = dataclasses.replace(w, batch=args.batch, name=f"{w.name}_batch{args.batch}")
    if args.context:
        w = dataclasses.replace(w, context=args.context, name=f"{w.name}_context{args.context}")
    if args.impl == "reference":
        run_reference_arm(args, w)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    if args.gpus == 1 and name != "c4":
        run_single_gpu(args, w, with_secondary=(args.workload is None and not args.batch and not args.no_secondary))
    else:
        run_sharded(args, w)


if __name__ == "__main__":
    main()
