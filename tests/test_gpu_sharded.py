"""The CUDA backend of the sharded step on one GPU: a world of one, and the per-shard stages run
for every shard of a two-way split inside one process (what each rank would compute), merged
exactly as the ranks would."""
import pytest
import torch

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
    """No process group: the one-call step with local exchange buffers (the configuration-4-on-one-GPU path)."""
    T, k = 20000, 128
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=4, kv_heads=2, context=T, channels=32)
    ch = ops.choose_channels(key[:, :, :T], 32)
    packed, scale = ops.quantize(key[:, :, :T], ch)
    eng = ShardedSparseDecode(k, total_tokens=T)
    try:
        want = oracle.decode_step(*cpu(q, key, value, ch), k)
        for _ in range(3):                                      # the step number advances, nothing is cleared in between
            out, sel = eng.step(q, key, value, packed, scale, ch, T, 0)
            assert eng._fast
            assert torch.equal(torch.sort(sel.cpu().long(), dim=-1).values, torch.sort(want["selected"], dim=-1).values)
            torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
    finally:
        eng.close()


def test_world_of_one_composed_form(cuda_device):
    """top_k above the shard length: the step composed from operators (the form used around all-gathers)."""
    T, k = 100, 128
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=4, kv_heads=2, context=T, channels=32)
    ch = ops.choose_channels(key[:, :, :T], 32)
    packed, scale = ops.quantize(key[:, :, :T], ch)
    eng = ShardedSparseDecode(k, total_tokens=T)
    out, sel = eng.step(q, key, value, packed, scale, ch, T, 0)
    assert not eng._fast
    want = oracle.decode_step(*cpu(q, key, value, ch), k)
    assert torch.equal(sel.cpu().long(), torch.sort(want["selected"], dim=-1).values)
    torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)


class _EmulatedRanks:
    """N ranks of the one-call sharded step inside ONE process on one GPU: every rank has its own exchange
    buffer and workspace, and the phases are run rank after rank (all phase 1, then all phase 2, then all
    phase 3), so no kernel ever waits for one queued behind it."""

    def __init__(self, dev, q, key, value, ch, T, k, N, wait_polls=0):
        from kv_cache_b200 import _native
        from kv_cache_b200.sharded import PeerExchange

        lib = _native.lib()
        B, Hq = q.shape[0], q.shape[1]
        Hkv = key.shape[1]
        self.N, self.k, self.T, self.q, self.ch, self.wait_polls = N, k, T, q, ch, wait_polls
        self.xbytes = lib.kvb_sharded_exchange_bytes(B, Hq, Hkv, k, N)
        self.ex = [PeerExchange(self.xbytes, dev) for _ in range(N)]
        self.ptrs = [e.local for e in self.ex]
        self.shards = []
        for r in range(N):
            t0, t1 = shard_bounds(T, N, r)
            tl = t1 - t0
            k_loc = torch.cat((key[:, :, t0:t1], key[:, :, T:]), dim=2).contiguous()
            v_loc = torch.cat((value[:, :, t0:t1], value[:, :, T:]), dim=2).contiguous()
            packed, scale = ops.quantize(k_loc[:, :, :tl], ch)
            ws = torch.empty(lib.kvb_sharded_step_workspace_bytes(B, Hq, Hkv, tl, k), dtype=torch.uint8, device=dev)
            out = torch.zeros((B, 1, Hq, 128), dtype=torch.bfloat16, device=dev)
            sel = torch.zeros((B, Hkv, k), dtype=torch.int32, device=dev)
            self.shards.append(dict(k=k_loc, v=v_loc, packed=packed, scale=scale, tl=tl, t0=t0, ws=ws, out=out, sel=sel))

    def phase(self, r, phases):
        from kv_cache_b200.sharded import sharded_decode_step

        s = self.shards[r]
        return sharded_decode_step(self.q, s["k"], s["v"], s["packed"], s["scale"], self.ch, s["tl"], s["t0"], self.T,
                                   self.k, r, self.N, self.ptrs, self.xbytes, s["ws"], s["out"], s["sel"],
                                   phases=phases, wait_polls=self.wait_polls)

    def step(self):
        for ph in (1, 2, 4):
            for r in range(self.N):
                assert self.phase(r, ph) == 0

    def close(self):
        torch.cuda.synchronize()
        for e in self.ex:
            e.close()


@pytest.mark.parametrize("N,T,k", [(2, 24000, 512), (4, 40000, 1024), (8, 80000, 256), (3, 30001, 4000)])
def test_one_call_step_emulated_ranks(cuda_device, N, T, k):
    """The step that runs across GPUs, with all ranks' buffers on one device: pushed candidate prefixes, flags,
    the merge on the inbox, owned-row attention, pushed partials, the combine. Every rank must hold the
    un-sharded oracle's selection and output, step after step."""
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64, seed=N + 40)
    ch = ops.choose_channels(key[:, :, :T], 64)
    want = oracle.decode_step(*cpu(q, key, value, ch), k)
    want_sel = torch.sort(want["selected"], dim=-1).values
    em = _EmulatedRanks(cuda_device, q, key, value, ch, T, k, N)
    try:
        for it in range(3):
            em.step()
            for r in range(N):
                s = em.shards[r]
                assert torch.equal(torch.sort(s["sel"].cpu().long(), dim=-1).values, want_sel), (it, r)
                torch.testing.assert_close(s["out"].float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
            assert all(torch.equal(em.shards[0]["out"], em.shards[r]["out"]) for r in range(N))     # the same bits everywhere
    finally:
        em.close()


def test_one_call_step_when_one_shard_holds_every_winner(cuda_device):
    """All large keys live in shard 0: the prefixes cannot decide the rows, so the merge must read the ranks'
    whole lists (the path that crosses NVLink with plain loads on a real node)."""
    N, T, k = 8, 64000, 2048
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=8, kv_heads=2, context=T, channels=64, seed=77)
    key = key.clone()
    key[:, :, T // N:T] *= 0.01                                  # shards 1.. are far below shard 0
    ch = ops.choose_channels(key[:, :, :T], 64)
    want = oracle.decode_step(*cpu(q, key, value, ch), k)
    want_sel = torch.sort(want["selected"], dim=-1).values
    assert int((want["selected"] < T // N).sum()) > 2 * (8192 // N)        # more winners in shard 0 than a prefix holds
    em = _EmulatedRanks(cuda_device, q, key, value, ch, T, k, N)
    try:
        em.step()
        for r in range(N):
            assert torch.equal(torch.sort(em.shards[r]["sel"].cpu().long(), dim=-1).values, want_sel)
            torch.testing.assert_close(em.shards[r]["out"].float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
    finally:
        em.close()


def test_bounded_wait_gives_up_cleanly(cuda_device):
    """Rank 1 never runs phase 1, so rank 0's merge waits for a flag that nothing raises: with a poll limit of
    64 the kernels must return, the status word must say KVB_TIMEOUT, and the device must stay usable."""
    import ctypes
    from kv_cache_b200 import _native

    N, T, k = 2, 24000, 256
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=4, kv_heads=2, context=T, channels=32, seed=3)
    ch = ops.choose_channels(key[:, :, :T], 32)
    em = _EmulatedRanks(cuda_device, q, key, value, ch, T, k, N, wait_polls=64)
    lib = _native.lib()
    st = ctypes.c_int(-1)
    try:
        assert lib.kvb_device_status(0, ctypes.byref(st)) == 0 and st.value == 0
        assert em.phase(0, 1) == 0
        assert em.phase(0, 2) == 0                               # waits for rank 1's flag, gives up after 64 polls
        assert em.phase(0, 4) == 0                               # and for rank 1's partial
        torch.cuda.synchronize()
        assert lib.kvb_device_status(0, ctypes.byref(st)) == 0 and st.value == 5          # KVB_TIMEOUT, then cleared
        assert lib.kvb_device_status(0, ctypes.byref(st)) == 0 and st.value == 0
        # the context is alive: bring rank 1 level (its step counter is one behind) and run a full, correct step
        assert em.phase(1, 1) == 0
        em.step()
        torch.cuda.synchronize()
        want = oracle.decode_step(*cpu(q, key, value, ch), k)
        for r in range(N):
            assert torch.equal(torch.sort(em.shards[r]["sel"].cpu().long(), dim=-1).values,
                               torch.sort(want["selected"], dim=-1).values)
            torch.testing.assert_close(em.shards[r]["out"].float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
        assert lib.kvb_device_status(0, ctypes.byref(st)) == 0 and st.value == 0
    finally:
        em.close()


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
