"""Chunked-prefill block scoring: per-token query codes, block scores and selected block ids
bit-exact against the oracle (parity unpinned by the reference, which has no prefill scorer)."""
import pytest
import torch

from kv_cache_b200 import inputs, ops
from oracle import oracle
from tests.gpu_util import cpu

pytestmark = pytest.mark.gpu


def _case(dev, B, Hq, Hkv, Tq, Tk, C, seed=3):
    w = inputs.small_workload(batch=B, q_heads=Hq, kv_heads=Hkv, context=Tk, channels=C, seed=seed)
    key, _ = inputs.make_kv(w, dev, 0, Tk)
    g = torch.Generator(device=dev).manual_seed(seed)
    q = inputs.rope(torch.randn(B, Hq, Tq, 128, generator=g, device=dev), torch.arange(Tk, Tk + Tq, device=dev))
    return key, q.to(torch.bfloat16)


@pytest.mark.parametrize("B,Hq,Hkv,Tq,Tk,C", [
    (1, 8, 2, 128, 4096, 64),       # the full small case of the specification
    (2, 4, 2, 150, 1000, 64),       # ragged query tile and a short last key block
    (1, 2, 2, 16, 64, 32),          # G = 1, one block
    (1, 16, 2, 40, 700, 32),        # G = 8
    (1, 4, 2, 33, 2048 + 70, 128),  # C = 128, G = 2
])
def test_block_scores_and_topk_bit_exact(cuda_device, B, Hq, Hkv, Tq, Tk, C):
    key, q = _case(cuda_device, B, Hq, Hkv, Tq, Tk, C)
    ch = ops.choose_channels(key, C)
    packed, scale = ops.quantize(key, ch)
    qcode, qscale = ops.quantize_query_tokens(q, ch)
    qcode_o, qscale_o = oracle.quantize_query_tokens(q.cpu(), ch.cpu())
    assert torch.equal(qcode.cpu(), qcode_o) and torch.equal(qscale.cpu(), qscale_o)
    bs = ops.score_prefill_blocks(qcode, qscale, packed, scale, Tk)
    codes_o, _, kscale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    want = oracle.prefill_block_scores(qcode_o, qscale_o, codes_o, kscale_o)
    assert torch.equal(bs.cpu().view(torch.int32), want.view(torch.int32))
    idx, val = ops.block_topk(bs, 32, return_scores=True)
    want_i, want_v = oracle.select(want, 32)
    assert torch.equal(idx.cpu().long(), want_i) and torch.equal(val.cpu(), want_v)
    idx2, _ = ops.prefill_select_blocks(q, packed, scale, ch, Tk, 32)
    assert torch.equal(idx2, idx)


@pytest.mark.parametrize("engine", ["mma", "i8", "f16", "i8w", "f16w"])
@pytest.mark.parametrize("B,Hq,Hkv,Tq,Tk,C", [
    (1, 8, 2, 128, 4096, 64),       # 32 key tiles, two query tiles per CTA, G = 4
    (2, 4, 2, 150, 1000, 64),       # ragged query tile, short last block, odd number of blocks
    (1, 2, 2, 300, 64 * 9, 32),     # G = 1: 256 queries per CTA, nine blocks (half-filled last key tile)
    (1, 16, 2, 40, 700, 32),        # G = 8
    (1, 4, 2, 33, 2048 + 70, 128),  # C = 128, G = 2
])
def test_every_prefill_engine_gives_the_same_bits(cuda_device, engine, B, Hq, Hkv, Tq, Tk, C):
    key, q = _case(cuda_device, B, Hq, Hkv, Tq, Tk, C, seed=5)
    ch = ops.choose_channels(key, C)
    packed, scale = ops.quantize(key, ch)
    qcode, qscale = ops.quantize_query_tokens(q, ch)
    bs = ops.score_prefill_blocks(qcode, qscale, packed, scale, Tk, engine=engine)
    codes_o, _, kscale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    want = oracle.prefill_block_scores(qcode.cpu(), qscale.cpu(), codes_o, kscale_o)
    assert torch.equal(bs.cpu().view(torch.int32), want.view(torch.int32))


@pytest.mark.parametrize("engine", ["mma", "i8", "f16", "i8w", "f16w"])
def test_prefill_engines_at_the_largest_accumulator(cuda_device, engine):
    """Every code at its extreme (|q| = 127, |k| = 7, C = 128): |acc| reaches 127 * 7 * 128 = 113792, the
    largest integer any accumulator of this path can hold; it must come out exact in every encoding."""
    B, Hq, Hkv, Tq, Tk, C = 1, 4, 2, 64, 512, 128
    g = torch.Generator(device=cuda_device).manual_seed(9)
    sign = lambda *shape: torch.randint(0, 2, shape, generator=g, device=cuda_device) * 2 - 1  # noqa: E731
    key = (sign(B, Hkv, Tk, 128) * 3.0).to(torch.bfloat16)
    key[..., :8, :] = 3.0                                       # a run of all-positive rows: the extreme sum
    ch = torch.arange(C, dtype=torch.int32, device=cuda_device).repeat(Hkv, 1)
    packed, scale = ops.quantize(key, ch)
    qcode = (sign(B, Hq, Tq, C) * 127).to(torch.int8)
    qcode[:, :, :4, :] = 127
    qscale = torch.rand(B, Hq, Tq, generator=g, device=cuda_device) + 0.5
    bs = ops.score_prefill_blocks(qcode, qscale, packed, scale, Tk, engine=engine)
    codes_o, _, kscale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    assert int(codes_o.abs().min()) == 7
    want = oracle.prefill_block_scores(qcode.cpu(), qscale.cpu(), codes_o, kscale_o)
    assert torch.equal(bs.cpu().view(torch.int32), want.view(torch.int32))
    assert float(want.max()) >= 113792 * float(kscale_o.min()) * 0.5


def test_block_topk_ties_and_short_rows(cuda_device):
    s = torch.tensor([[1.0, 5.0, 5.0, -0.0, 0.0, 5.0]], device=cuda_device)
    assert ops.block_topk(s, 4).tolist() == [[1, 2, 5, 0]]
    assert ops.block_topk(s, 100).tolist() == [[1, 2, 5, 0, 3, 4]]
    g = torch.Generator(device=cuda_device).manual_seed(1)
    big = torch.randint(-3, 4, (70, 2048), generator=g, device=cuda_device).float()
    want, _ = oracle.select(big.cpu(), 32)
    assert torch.equal(ops.block_topk(big, 32).cpu().long(), want)


@pytest.mark.parametrize("engine", ["i8", "f16"])
def test_widened_keys_kept_across_chunks_and_grown(cuda_device, engine):
    """One widened operand buffer with spare capacity serves several query chunks; keys appended later are
    widened from the tile of the first new token on and the scores still equal the oracle's."""
    B, Hq, Hkv, Tq, C = 1, 8, 2, 70, 64
    T0, T1, cap = 1000, 1000 + 300, 2048
    key, q = _case(cuda_device, B, Hq, Hkv, Tq, T1, C, seed=11)
    ch = ops.choose_channels(key, C)
    packed, scale = ops.quantize(key, ch)
    qcode, qscale = ops.quantize_query_tokens(q, ch)
    codes_o, _, kscale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    wk = ops.WidenedKeys(packed, T0, engine, capacity=cap)
    for Tk in (T0, T1):
        if Tk > wk.key_count:
            wk.update(packed, Tk, first_token=wk.key_count)
        for _ in range(2):                              # two chunks against the same operands
            bs = ops.score_prefill_blocks(qcode, qscale, packed, scale, Tk, widened=wk)
            want = oracle.prefill_block_scores(qcode.cpu(), qscale.cpu(), codes_o[:, :, :Tk], kscale_o[:, :, :Tk])
            assert torch.equal(bs.cpu().view(torch.int32), want.view(torch.int32))
