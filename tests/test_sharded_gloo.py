"""The rank/plumbing logic of the sequence-sharded step on CPU ranks (gloo, world size 2 and 3):
candidate packing, the single all-gather of (score, id) lists, the global merge, ownership of the
selected ids, the LSE combine. The device stages are replaced by the CPU oracle through the
backend seam; the sharded result must equal the un-sharded oracle step."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kv_cache_b200 import inputs
from kv_cache_b200.sharded import ShardedSparseDecode, shard_bounds
from oracle import oracle


class OracleBackend:
    """Checker stand-in for kv_cache_b200.sharded.CudaBackend (same four methods, torch CPU)."""

    def local_candidates(self, query, codes, kscale, channel_idx, t_local, k, id_offset):
        qcode, qscale = oracle.quantize_query(query, channel_idx)
        _, _, gmax = oracle.score(qcode, qscale, codes[:, :, :t_local], kscale[:, :, :t_local])
        idx, sc = oracle.select(gmax.reshape(-1, t_local), k)
        return sc, (idx + id_offset).to(torch.int32)

    def merge(self, scores, ids, k):
        sel, _ = oracle.merge_shards(scores, ids.long(), k)
        return torch.sort(sel, dim=-1).values.to(torch.int32)

    def attend_partial(self, query, key, value, selected, t_local, id_base, keep_self, scaling):
        local = selected.long() - id_base
        valid = (local >= 0) & (local < t_local)
        if keep_self:
            local = torch.cat((local, torch.full_like(local[..., :1], t_local)), dim=-1)
            valid = torch.cat((valid, torch.ones_like(valid[..., :1])), dim=-1)
        D = query.shape[-1]
        out, m, l = oracle.attend_fp32(query, key, value, local.clamp(0, t_local), valid,
                                       D ** -0.5 if scaling is None else scaling)
        return torch.cat((out[:, 0] * l[..., None], m[..., None], l[..., None]), dim=-1)

    def combine(self, partials):
        return oracle.lse_merge(partials).to(torch.bfloat16)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, k, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        w = inputs.small_workload(batch=2, q_heads=8, kv_heads=2, context=T, channels=32, top_k=k, seed=21)
        key, value = inputs.make_kv(w, "cpu", 0, T + 1)
        query = inputs.make_query(w, "cpu")
        ch = oracle.choose_channels(key[:, :, :T], 32)
        t0, t1 = shard_bounds(T, world, rank)
        tl = t1 - t0
        k_loc = torch.cat((key[:, :, t0:t1], key[:, :, T:]), dim=2)
        v_loc = torch.cat((value[:, :, t0:t1], value[:, :, T:]), dim=2)
        codes, _, kscale = oracle.quantize_pack(k_loc[:, :, :tl], ch)
        eng = ShardedSparseDecode(k, backend=OracleBackend())
        out, sel = eng.step(query, k_loc, v_loc, codes, kscale, ch, tl, t0)
        want = oracle.decode_step(query, key, value, ch, k)
        assert torch.equal(sel.long(), torch.sort(want["selected"], dim=-1).values), "global selection differs"
        torch.testing.assert_close(out.float(), want["out"], rtol=2e-2, atol=1e-2)
        # every rank holds the same result
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(g, out) for g in gathered)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,k", [(2, 600, 64), (3, 601, 64), (2, 50, 40)])
def test_sharded_step_matches_unsharded_oracle(world, T, k):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, k, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert [ret.get(r) for r in range(world)] == ["ok"] * world


def test_shard_bounds_cover_the_sequence():
    for total, world in ((1048576, 8), (601, 3), (5, 8)):
        spans = [shard_bounds(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1
