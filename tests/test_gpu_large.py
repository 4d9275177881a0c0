"""Parity at the sizes the benchmarks run, where the kernels take branches that small cases never
reach: rows longer than 262144 tokens switch the threshold sampler to 16 tokens per thread, and the
sequence-sharded configuration hands such rows to kvb_shard_candidates. Selected ids must equal the
oracle's bit for bit, outputs within 2e-2 relative / 1e-2 absolute."""
import numpy as np
import pytest
import torch

from kv_cache_b200 import inputs, ops
from oracle import oracle
from tests.gpu_util import cpu

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2


def _long_case(dev, T, seed):
    w = inputs.Workload("long", 1, 8, 2, 128, T, 64, 4096, seed)
    key, value = inputs.make_kv(w, dev, 0, T + 1)
    query = inputs.make_query(w, dev)
    ch = ops.choose_channels(key[:, :, :T], 64)
    packed, scale = ops.alloc_side_cache(1, 2, T + 1, 64, dev)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    return w, query, key, value, ch, packed, scale


@pytest.mark.parametrize("T", [262144, 262145, 524288, 1048576])
def test_decode_step_and_shard_candidates_on_long_rows(cuda_device, T):
    k = 4096
    w, q, key, value, ch, packed, scale = _long_case(cuda_device, T, seed=T % 1000)
    want = oracle.decode_step(*cpu(q, key, value, ch), k)
    want_sorted = torch.sort(want["selected"], dim=-1).values
    assert torch.equal(packed[:, :, :T].cpu(), want["packed"])

    # the fused step, in both selection orders
    for ordered in (True, False):
        sel = torch.empty((1, 2, k), dtype=torch.int32, device=cuda_device)
        out = ops.DecodeStep(k, ordered_selection=ordered, append_self=False)(q, key, value, packed, scale, ch,
                                                                             selected_out=sel)
        got = sel.cpu().long()
        assert torch.equal(got if ordered else torch.sort(got, dim=-1).values, want_sorted)
        torch.testing.assert_close(out.float().cpu(), want["out"], rtol=RTOL, atol=ATOL)

    # the shard front end: composites (score key << 32 | ~global id), with and without the best-first split
    offset = 1000003
    order = torch.sort(want["selected"], dim=-1)
    want_scores = torch.gather(want["selected_scores"], -1, order.indices).reshape(2, k).numpy()
    for split in (0, 1024):
        comp = ops.shard_candidates(q, packed, scale, ch, T, k, id_offset=offset, split_k=split)
        assert comp is not None and comp.shape == (2, k)
        u = comp.cpu().numpy().view(np.uint64)
        ids = (0xFFFFFFFF - (u & np.uint64(0xFFFFFFFF))).astype(np.int64)
        by_id = np.argsort(ids, axis=1)
        assert (np.take_along_axis(ids, by_id, 1) - offset == want_sorted.reshape(2, k).numpy()).all()
        # the upper half of a composite is the order-preserving key of the fp32 group maximum
        bits = (np.take_along_axis(u, by_id, 1) >> np.uint64(32)).astype(np.uint32)
        raw = np.where(bits & np.uint32(0x80000000), bits & np.uint32(0x7FFFFFFF), ~bits)
        assert (raw.view(np.float32) == want_scores).all()
        if split:                                   # the first `split` entries are the `split` best composites
            best = np.sort(u, axis=1)[:, ::-1][:, :split]
            assert (np.sort(u[:, :split], axis=1)[:, ::-1] == best).all()


def test_choose_channels_matches_oracle(cuda_device):
    w = inputs.small_workload(batch=2, q_heads=8, kv_heads=2, context=70000, channels=64, seed=31)
    key, _ = inputs.make_kv(w, cuda_device, 0, w.context)
    for c in (32, 64, 128):
        assert torch.equal(ops.choose_channels(key, c).cpu(), oracle.choose_channels(key.cpu(), c))


def test_choose_channels_near_ties(cuda_device):
    """Two channels whose mean |K| differs by one bf16 step of one token among 40000, and two that are
    exactly equal: the larger mean wins, equal means go to the lower channel, on both sides."""
    T = 40000
    key = torch.zeros((1, 1, T, 128), dtype=torch.bfloat16)
    key[..., 10] = 1.0
    key[..., 11] = 1.0
    key[0, 0, 777, 11] = 1.0078125          # one step above 1.0 in bf16
    key[..., 20] = -0.5
    key[..., 90] = 0.5                      # |.| equal to channel 20
    key[..., 5] = 0.25
    want = oracle.choose_channels(key, 3)
    assert want.tolist() == [[10, 11, 20]]
    assert oracle.choose_channels(key, 1).tolist() == [[11]]
    dev_key = key.to(cuda_device)
    for c in (1, 2, 3, 4, 5):
        assert torch.equal(ops.choose_channels(dev_key, c).cpu(), oracle.choose_channels(key, c))


@pytest.fixture(scope="module")
def prefill_case(cuda_device):
    """Config-3 inputs on the device plus the oracle's block scores for 64 seeded query rows (computed once
    for the three engines)."""
    B, Hq, Hkv, D, Tq, Tk, C = 2, 32, 8, 128, 4096, 131072, 64
    dev = cuda_device
    w = inputs.Workload("c3", B, Hq, Hkv, D, Tk, C, 0, seed=3)
    key, _ = inputs.make_kv(w, dev, 0, Tk)
    ch = ops.choose_channels(key, C)
    packed, scale = ops.quantize(key, ch)
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.empty((B, Hq, Tq, D), dtype=torch.bfloat16, device=dev)
    for b in range(B):
        q[b] = inputs.rope(torch.randn(Hq, Tq, D, generator=g, device=dev),
                           torch.arange(Tk, Tk + Tq, device=dev)).to(torch.bfloat16)
    qcode, qscale = ops.quantize_query_tokens(q, ch)
    rows = torch.randperm(Tq, generator=torch.Generator().manual_seed(17))[:64].sort().values
    rows[0], rows[-1] = 0, Tq - 1                                     # the edges of the chunk too
    codes_o, packed_o, kscale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    assert torch.equal(packed.cpu(), packed_o)
    del key
    qc_o, qs_o = oracle.quantize_query_tokens(q[:, :, rows.to(dev)].cpu(), ch.cpu())
    assert torch.equal(qcode[:, :, rows.to(dev)].cpu(), qc_o) and torch.equal(qscale[:, :, rows.to(dev)].cpu(), qs_o)
    want = oracle.prefill_block_scores(qc_o, qs_o, codes_o, kscale_o)          # [B,Hkv,64,2048]
    want_idx, _ = oracle.select(want, 32)
    return dict(qcode=qcode, qscale=qscale, packed=packed, scale=scale, Tk=Tk, rows=rows.to(dev), want=want,
                want_idx=want_idx)


@pytest.mark.parametrize("engine", ["mma", "i8", "f16", "i8w", "f16w"])
def test_prefill_block_scores_at_full_key_length(prefill_case, engine):
    """The chunked-prefill configuration at its real size (4096 queries x 131072 keys, batch 2, 32 query
    heads over 8 KV heads): 64 seeded query rows per batch row are recomputed by the oracle over all
    131072 keys; block scores and the selected blocks must be identical."""
    c = prefill_case
    bs = ops.score_prefill_blocks(c["qcode"], c["qscale"], c["packed"], c["scale"], c["Tk"], engine=engine)
    idx = ops.block_topk(bs, 32)
    got = bs[:, :, c["rows"]].cpu()
    assert torch.equal(got.view(torch.int32), c["want"].view(torch.int32))
    assert torch.equal(idx[:, :, c["rows"]].cpu().long(), c["want_idx"])
