"""The rerank modes as lists: kvb_score_select, kvb_rerank_union, kvb_expand_final and the mode strings
built on them, against (a) what the REFERENCE recorded over three consecutive reuse steps and a top-2 % step
(tests/golden, produced by its own code) and (b) the oracle for the int4 / GQA-group form."""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from kv_cache_b200 import attention_patch as ap
from kv_cache_b200 import ops
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2
GOLD = np.load(Path(__file__).parent / "golden" / "reference_golden.npz")


def bf16(a):
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def _lists_from_mask(mask: torch.Tensor) -> torch.Tensor:
    """bool [B,H,T] -> int32 [B,H,n] ascending ids, -1 padded."""
    n = max(1, int(mask.sum(-1).max()))
    ids = torch.full((*mask.shape[:2], n), -1, dtype=torch.int32)
    for b in range(mask.shape[0]):
        for h in range(mask.shape[1]):
            nz = torch.nonzero(mask[b, h]).flatten()
            ids[b, h, :nz.numel()] = nz.to(torch.int32)
    return ids


def test_rerank_on_the_references_recorded_candidates(cuda_device):
    """Per query head, as the reference does it: its recorded candidate masks of three consecutive steps go in
    as lists; the kept ids plus the protected ranges must be exactly the final masks it stored, and the
    attention over them must equal its recorded outputs."""
    dev = cuda_device
    q, k, v = bf16(GOLD["ru_q"]).to(dev), bf16(GOLD["ru_k"]).to(dev), bf16(GOLD["ru_v"]).to(dev)
    top, sink, recent, T0 = GOLD["ru_params"].tolist()
    sink, recent, T0 = int(sink), int(recent), int(T0)
    for step in range(3):
        hist = T0 + step
        keep = min(hist, max(1, math.ceil(top * hist)))
        lists = [_lists_from_mask(torch.from_numpy(GOLD[f"ru_{step}_candidate"])).to(dev)]
        if step:
            lists += [_lists_from_mask(torch.from_numpy(GOLD[f"ru_{step - 1}_candidate"])).to(dev),
                      _lists_from_mask(torch.from_numpy(GOLD[f"ru_{step - 1}_final"])).to(dev)]
        kept, cnt = ops.rerank_union(q[step][:, :, 0], k[:, :, :hist], lists, hist, keep)
        assert kept.shape == (2, 8, keep) and int(cnt.min()) == keep
        final, fcnt = ops.expand_final(kept, hist, count=cnt, force_sink=sink, force_recent=recent)
        want = torch.from_numpy(GOLD[f"ru_{step}_final"])
        for b in range(2):
            for h in range(8):
                got = final[b, h, :int(fcnt[b, h])].cpu().tolist()
                assert got == torch.nonzero(want[b, h]).flatten().tolist(), (step, b, h)
        fidx, fvalid = ops.build_final_indices(kept, None, hist, hist + 1, sink, recent, True)
        out = ops.sparse_attend(q[step], k[:, :, :hist + 1], v[:, :, :hist + 1], fidx, fvalid)
        torch.testing.assert_close(out.float().cpu(), torch.from_numpy(GOLD[f"ru_{step}_out"]), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("G,Hi_is_q", [(4, False), (4, True), (1, False), (8, False), (2, False)])
def test_rerank_union_matches_oracle(cuda_device, G, Hi_is_q):
    T, Hkv = 3000, 2
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=Hkv * G, kv_heads=Hkv, context=T, channels=32, seed=G)
    Hi = Hkv * G if Hi_is_q else Hkv
    g = torch.Generator(device=cuda_device).manual_seed(5)
    l0 = torch.randint(0, T, (2, Hi, 200), generator=g, device=cuda_device, dtype=torch.int32)
    l1 = torch.randint(-5, T + 40, (2, Hi, 150), generator=g, device=cuda_device, dtype=torch.int32)     # stale / padding ids
    l2 = torch.randint(0, T, (2, Hi, 90), generator=g, device=cuda_device, dtype=torch.int32)
    c2 = torch.randint(0, 91, (2, Hi), generator=g, device=cuda_device, dtype=torch.int32)
    mask = torch.zeros((2, 1, 1, T + 1), dtype=torch.bfloat16, device=cuda_device)
    mask[1, 0, 0, :300] = -1e4
    for keep, lists, counts, msk, fs, fr in ((64, [l0, l1, l2], [None, None, c2], None, 0, 0),
                                            (1000, [l0], None, None, 0, 0),              # keep > |union|
                                            (50, [l0, None, l2], None, mask, 7, 9)):
        kept, cnt = ops.rerank_union(q, key, lists, T, keep, counts=counts, attention_mask=msk, force_sink=fs, force_recent=fr)
        want, wcnt = oracle.rerank_union(q.cpu(), key.cpu(), [None if l is None else l.cpu() for l in lists], T, keep,
                                         128 ** -0.5, counts=None if counts is None else [None if c is None else c.cpu() for c in counts],
                                         mask_rows=None if msk is None else msk[:, 0, 0].float().cpu(), force_sink=fs, force_recent=fr)
        assert torch.equal(cnt.cpu().long(), wcnt)
        assert torch.equal(kept.cpu().long(), want)


def test_rerank_union_ties_go_to_the_lower_id(cuda_device):
    T = 500
    key = torch.zeros((1, 1, T, 128), dtype=torch.bfloat16, device=cuda_device)
    key[0, 0, 100:120, 0] = 1.0                                 # twenty equal best scores
    q = torch.zeros((1, 1, 128), dtype=torch.bfloat16, device=cuda_device)
    q[0, 0, 0] = 1.0
    ids = torch.arange(90, 130, dtype=torch.int32, device=cuda_device).flip(0).view(1, 1, -1)
    kept, cnt = ops.rerank_union(q, key, [ids], T, 5)
    assert kept[0, 0].tolist() == [100, 101, 102, 103, 104] and int(cnt) == 5
    kept, cnt = ops.rerank_union(q, key, [ids], T, 25)        # all twenty, then the lowest ids among the zeros
    assert kept[0, 0].tolist() == list(range(90, 95)) + list(range(100, 120))


@pytest.mark.parametrize("block", [1, 16, 64])
def test_expand_final_matches_the_reference_rule(cuda_device, block):
    T = 1000 + block // 2                                        # a partial last block
    g = torch.Generator(device=cuda_device).manual_seed(block)
    ids = torch.randint(-3, T + 10, (3, 2, 40), generator=g, device=cuda_device, dtype=torch.int32)
    cnt = torch.tensor([[40, 0], [13, 40], [1, 39]], dtype=torch.int32, device=cuda_device)
    out, n = ops.expand_final(ids, T, count=cnt, force_sink=5, force_recent=3, block_size=block)
    want = oracle.expand_final(ids.cpu(), T, counts=cnt.cpu(), force_sink=5, force_recent=3, block_size=block)
    for r, wl in enumerate(want):
        b, h = divmod(r, 2)
        assert int(n[b, h]) == len(wl)
        assert out[b, h, :len(wl)].cpu().tolist() == wl
        assert (out[b, h, len(wl):] == -1).all()
    # and against the reference's own mask helper (restated in the oracle)
    keep = torch.zeros((1, 1, T), dtype=torch.bool)
    keep[0, 0, [3, 500, T - 1]] = True
    exp = oracle.expand_keep_to_aligned_blocks(keep, block)
    one, n1 = ops.expand_final(torch.tensor([[[3, 500, T - 1]]], dtype=torch.int32, device=cuda_device), T, block_size=block)
    assert one[0, 0, :int(n1)].cpu().tolist() == torch.nonzero(exp[0, 0]).flatten().tolist()


@pytest.mark.parametrize("T,k", [(5000, 200), (20000, 700), (70000, 2048)])
def test_score_select_gives_the_oracle_candidates(cuda_device, T, k):
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64, seed=T % 97)
    ch = ops.choose_channels(key[:, :, :T], 64)
    packed, scale = ops.quantize(key[:, :, :T], ch)
    got = ops.score_select(q, packed, scale, ch, T, k)
    want = oracle.decode_step(*cpu(q, key, value, ch), k)["selected"]
    assert torch.equal(got.cpu().long(), torch.sort(want, dim=-1).values)        # ascending ids


class _Layer(torch.nn.Module):
    def __init__(self, idx):
        super().__init__()
        self.layer_idx = idx
        self.scaling = 128 ** -0.5


@pytest.mark.parametrize("mode,block", [("qabs32cand12p5reuse", 1), ("qabs32cand12p5reuse2set", 1),
                                        ("qabs32cand12p5reusefinal", 1), ("qabs32cand12p5reuseblk16", 16)])
def test_reuse_modes_through_the_patched_attention(cuda_device, mode, block):
    """Three decode steps, one `with` block each: the int4 candidates, the union with the previous step's lists,
    the exact rerank, the protected ranges and the block widening must follow the oracle's reuse step, step
    after step (the state carried between steps included)."""
    T0, top, sink, recent = 1500, 0.03, 4, 6
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T0 + 3, channels=32, seed=19)
    layer = _Layer(1)
    state = ap.SparseDecodeState()
    pc = pf = None
    for i in range(3):
        kc = T0 + 1 + i
        qi = (q.float() * (1.0 + 0.1 * i)).to(torch.bfloat16)
        with ap.attention_mode(mode, top, 3, True, sink, recent, None, sparse_state=state):
            out, _ = ap.sparse_eager_attention_forward(layer, qi[:, :, None, :], key[:, :, :kc], value[:, :, :kc], None)
        ch = state.layers[1].channel_idx
        hist = kc - 1
        want = oracle.reuse_decode_step(qi.cpu(), key[:, :, :kc].cpu(), value[:, :, :kc].cpu(), ch.cpu(),
                                        ap.candidate_count(0.125, hist), min(hist, max(1, math.ceil(top * hist))),
                                        prev_candidate=None if mode.endswith("reusefinal") else pc,
                                        prev_final=None if mode.endswith("reuse2set") else pf,
                                        protect_sink=sink, protect_recent=recent, block_size=block)
        rec = state.reuse[1]
        assert rec.query_token == hist
        assert torch.equal(rec.candidate.cpu().long(), torch.sort(want["candidates"], dim=-1).values)
        for r, f in enumerate(want["final"]):
            b, g = divmod(r, 2)
            assert rec.final[b, g, :int(rec.final_count[b, g])].cpu().tolist() == f, (i, b, g)
        torch.testing.assert_close(out.float().cpu(), want["out"], rtol=RTOL, atol=ATOL)
        pc = want["candidates"]
        pf = torch.full((2, 2, max(len(f) for f in want["final"])), -1, dtype=torch.long)
        for r, f in enumerate(want["final"]):
            pf[r // 2, r % 2, :len(f)] = torch.tensor(f)
    assert state.layers[1].count == T0 + 3


def test_top2_mode_through_the_patched_attention(cuda_device):
    T, top = 4000, 0.02
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64, seed=23)
    state = ap.SparseDecodeState()
    with ap.attention_mode("qabs64cand6p25top2attn", top, 3, True, 3, 5, None, sparse_state=state):
        out, _ = ap.sparse_eager_attention_forward(_Layer(0), q[:, :, None, :], key, value, None)
    ch = state.layers[0].channel_idx
    cand_k = ap.candidate_count(0.0625, T)
    keep = min(cand_k, max(1, math.ceil(top * T)))
    res = oracle.decode_step(*cpu(q, key, value, ch), cand_k)
    kept, cnt = oracle.rerank_union(q.cpu(), key.cpu(), [res["selected"]], T, keep, 128 ** -0.5)
    fidx, fvalid = oracle.final_indices_from_selected(kept, kept >= 0, T, T + 1, True, 3, 5)
    want, _, _ = oracle.attend_fp32(q.cpu(), key.cpu(), value.cpu(), fidx, fvalid, 128 ** -0.5)
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)
