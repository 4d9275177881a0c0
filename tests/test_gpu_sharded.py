"""The CUDA backend of the sharded step on one GPU: a world of one, and the per-shard stages run
for every shard of a two-way split inside one process (what each rank would compute), merged
exactly as the ranks would."""
import os
import socket

import pytest
import torch
import torch.distributed as dist

from kv_cache_b200 import ops
from kv_cache_b200.sharded import CudaBackend, ShardedSparseDecode, shard_bounds
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu


def test_two_shards_emulated_in_one_process(cuda_device):
    T, k, N = 3000, 256, 2
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64)
    ch = ops.choose_channels(key[:, :, :T], 64)
    be = CudaBackend()
    scs, ids, shards = [], [], []
    for r in range(N):
        t0, t1 = shard_bounds(T, N, r)
        tl = t1 - t0
        k_loc = torch.cat((key[:, :, t0:t1], key[:, :, T:]), dim=2).contiguous()
        v_loc = torch.cat((value[:, :, t0:t1], value[:, :, T:]), dim=2).contiguous()
        packed, scale = ops.quantize(k_loc[:, :, :tl], ch)
        sc, idx = be.local_candidates(q, packed, scale, ch, tl, k, t0)
        scs.append(sc), ids.append(idx), shards.append((k_loc, v_loc, tl, t0))
    sel = be.merge(torch.stack(scs), torch.stack(ids), k).view(2, 2, -1)
    parts = [be.attend_partial(q, kl, vl, sel, tl, t0, r == N - 1, None) for r, (kl, vl, tl, t0) in enumerate(shards)]
    out = be.combine(torch.stack(parts))
    want = oracle.decode_step(*cpu(q, key, value, ch), k)
    assert torch.equal(sel.cpu().long(), torch.sort(want["selected"], dim=-1).values)
    torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)


def test_world_of_one(cuda_device):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        T, k = 2000, 128
        w, q, key, value = make_case(cuda_device, batch=1, q_heads=4, kv_heads=2, context=T, channels=32)
        ch = ops.choose_channels(key[:, :, :T], 32)
        packed, scale = ops.quantize(key[:, :, :T], ch)
        out, sel = ShardedSparseDecode(k).step(q, key, value, packed, scale, ch, T, 0)
        want = oracle.decode_step(*cpu(q, key, value, ch), k)
        assert torch.equal(sel.cpu().long(), torch.sort(want["selected"], dim=-1).values)
        torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N,T,k", [(2, 24000, 512), (4, 40000, 1024), (8, 80000, 256)])
def test_candidate_front_end_and_one_kernel_merge(cuda_device, N, T, k):
    """kvb_shard_candidates on every shard, concatenated as the all-gather would, then
    kvb_merge_candidates: the global selection must equal the un-sharded oracle top-k."""
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64, seed=N)
    ch = ops.choose_channels(key[:, :, :T], 64)
    lists = []
    for r in range(N):
        t0, t1 = shard_bounds(T, N, r)
        packed, scale = ops.quantize(key[:, :, t0:t1].contiguous(), ch)
        comp = ops.shard_candidates(q, packed, scale, ch, t1 - t0, k, id_offset=t0)
        assert comp is not None and comp.shape == (4, k)
        lists.append(comp)
    sel = ops.merge_candidates(torch.stack(lists), k, id_range=T)
    res = oracle.decode_step(*cpu(q, key, value, ch), k)
    want = res["selected"].reshape(4, k)
    assert torch.equal(torch.sort(sel.cpu().long(), dim=-1).values, torch.sort(want, dim=-1).values)

    # the same with every shard's best entries first, the merge working on those prefixes, and the owned
    # winners of every shard compacted for its attention
    prefix = max(16, min(k, 2 * k // N))
    lists = []
    for r in range(N):
        t0, t1 = shard_bounds(T, N, r)
        packed, scale = ops.quantize(key[:, :, t0:t1].contiguous(), ch)
        comp = ops.shard_candidates(q, packed, scale, ch, t1 - t0, k, id_offset=t0, split_k=prefix)
        plain = ops.shard_candidates(q, packed, scale, ch, t1 - t0, k, id_offset=t0)
        assert torch.equal(torch.sort(comp, dim=-1).values, torch.sort(plain, dim=-1).values)      # same set
        if prefix < k:                                                  # and the prefix is its best part
            u = comp.view(torch.uint8).view(4, k, 8).flip(-1).contiguous().cpu().numpy()       # unsigned order, as bytes
            import numpy as np
            keys = np.ascontiguousarray(u).view(">u8").reshape(4, k)
            assert (keys[:, :prefix].min(axis=1) > keys[:, prefix:].max(axis=1)).all()
        lists.append(comp)
    parts = []
    for r in range(N):
        t0, t1 = shard_bounds(T, N, r)
        sel2, owned, cnt = ops.merge_candidates(torch.stack(lists), k, id_range=T, prefix_k=prefix, own=(t0, t1))
        assert torch.equal(torch.sort(sel2.cpu().long(), dim=-1).values, torch.sort(want, dim=-1).values)
        for row in range(4):
            mine = want[row][(want[row] >= t0) & (want[row] < t1)]
            c = int(cnt[row])
            assert c == mine.numel()
            assert torch.equal(torch.sort(owned[row, :c].cpu().long()).values, torch.sort(mine).values)
        k_loc = torch.cat((key[:, :, t0:t1], key[:, :, T:]), dim=2).contiguous()
        v_loc = torch.cat((value[:, :, t0:t1], value[:, :, T:]), dim=2).contiguous()
        parts.append(ops.attend_selected(q, k_loc, v_loc, owned.view(2, 2, -1), t1 - t0, id_base=t0, keep_self=r == N - 1,
                                         return_partial=True, selected_count=cnt))
    out = ops.lse_merge(torch.stack(parts))
    torch.testing.assert_close(out.float().cpu(), res["out"], rtol=2e-2, atol=1e-2)


def test_prefix_merge_falls_back_when_one_shard_holds_the_winners(cuda_device):
    """All winners live in shard 0, whose prefix is too short to show them: the acceptance test must fail
    and the kernel must redo the select over the whole lists."""
    N, R, kk, prefix = 4, 2, 512, 128
    key_hi, key_lo = 0xC1000000, 0xC0000000
    comp = torch.empty((N, R, kk), dtype=torch.int64, device=cuda_device)
    for r in range(N):
        ids = torch.arange(r * kk, (r + 1) * kk, device=cuda_device)
        # shard 0: every entry beats every entry of the others; inside a list: descending by position
        bits = (key_hi if r == 0 else key_lo) + (kk - torch.arange(kk, device=cuda_device))
        comp[r] = ((bits << 32) | (0xFFFFFFFF - ids)).expand(R, kk)
    sel, owned, cnt = ops.merge_candidates(comp, kk, id_range=N * kk, prefix_k=prefix, own=(0, kk))
    assert torch.equal(torch.sort(sel.cpu(), dim=-1).values, torch.arange(kk, dtype=torch.int32).expand(R, kk))
    assert cnt.tolist() == [kk] * R


def test_merge_candidates_heavy_ties(cuda_device):
    """All scores equal: the segment-minimum filter keeps everything, the refinement path decides by id."""
    N, R, kk = 4, 3, 2048
    ids = torch.arange(N * kk, device=cuda_device).view(N, 1, kk).expand(N, R, kk)
    key_bits = 0xC0000000                                   # any fixed score key
    comp = (torch.full_like(ids, key_bits) << 32) | (0xFFFFFFFF - ids)
    sel = ops.merge_candidates(comp.contiguous(), kk, id_range=N * kk)
    assert torch.equal(sel.cpu(), torch.arange(kk, dtype=torch.int32).expand(R, kk))
