"""Stage 2 parity: int32 partial scores, dequantised scores and group max bit-exact."""
import pytest
import torch

from kv_cache_b200 import ops
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu


def _check(cuda_device, B, Hq, Hkv, T, C, want_hist=False, seed=7):
    w, q, key, _ = make_case(cuda_device, batch=B, q_heads=Hq, kv_heads=Hkv, context=T, channels=C, seed=seed)
    hist_k = key[:, :, :T]
    ch = ops.choose_channels(hist_k, C)
    packed, scale = ops.quantize(hist_k, ch)
    r = ops.score(q, packed, scale, ch, T, want_hist=want_hist)
    codes_o, _, scale_o = oracle.quantize_pack(*cpu(hist_k, ch))
    qcode, qscale = oracle.quantize_query(q.cpu(), ch.cpu())
    acc_o, deq_o, gmax_o = oracle.score(qcode, qscale, codes_o, scale_o)
    assert torch.equal(r.acc.cpu(), acc_o)
    assert torch.equal(r.deq.cpu().view(torch.int32), deq_o.view(torch.int32))
    assert torch.equal(r.gmax.cpu().view(torch.int32), gmax_o.view(torch.int32))
    if want_hist:
        keys = gmax_o.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        keys = torch.where(keys >= 2**31, (~keys) & 0xFFFFFFFF, keys | 2**31)
        want = torch.stack([torch.bincount(row >> 20, minlength=4096) for row in keys.reshape(-1, T)])
        assert torch.equal(r.hist.cpu().to(torch.int64), want)
    return r


@pytest.mark.parametrize("C", [32, 64, 128])
@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_stream_kernel_all_shapes(cuda_device, C, G):
    # T spans several warp tiles and leaves a ragged tail
    _check(cuda_device, B=2, Hq=2 * G, Hkv=2, T=3 * 1024 + 77, C=C)


@pytest.mark.parametrize("T", [1, 31, 63, 64, 65, 255, 256, 257, 4096])
def test_edge_lengths(cuda_device, T):
    _check(cuda_device, B=1, Hq=4, Hkv=2, T=T, C=64)


@pytest.mark.parametrize("C,G", [(16, 2), (34, 4), (64, 3), (32, 16), (6, 1)])
def test_generic_kernel(cuda_device, C, G):
    _check(cuda_device, B=2, Hq=2 * G, Hkv=2, T=777, C=C)


@pytest.mark.parametrize("C", [32, 64])
def test_fused_histogram(cuda_device, C):
    _check(cuda_device, B=2, Hq=8, Hkv=2, T=5000, C=C, want_hist=True)
    _check(cuda_device, B=2, Hq=6, Hkv=2, T=700, C=C, want_hist=True)   # generic kernel's histogram


def test_many_rows_more_ctas_than_units(cuda_device):
    _check(cuda_device, B=16, Hq=32, Hkv=8, T=300, C=64)


def test_config0_shapes(cuda_device):
    _check(cuda_device, B=1, Hq=16, Hkv=8, T=4096, C=32, seed=0, want_hist=True)


def test_gmax_only_and_strided_side_cache(cuda_device):
    w, q, key, _ = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=1500, channels=64)
    ch = ops.choose_channels(key[:, :, :1500], 64)
    packed, scale = ops.alloc_side_cache(2, 2, 4000, 64, cuda_device)       # capacity > T
    ops.quantize(key[:, :, :1500], ch, out=(packed, scale))
    r = ops.score(q, packed, scale, ch, 1500, want_acc=False, want_deq=False)
    full = ops.score(q, packed, scale, ch, 1500)
    assert r.acc is None and r.deq is None
    assert torch.equal(r.gmax, full.gmax)
    assert torch.equal(full.gmax, full.deq.view(2, 2, 4, -1).amax(2) + 0.0)


@pytest.mark.parametrize("T,k,C,G", [(40000, 1024, 64, 4), (20000, 256, 32, 2), (5000, 300, 64, 4)])
def test_candidate_form_contains_the_exact_top_k(cuda_device, T, k, C, G):
    """The scorer's candidate lists: every entry is (key of the exact group max, token), the count is
    within [k, capacity] on this data, and the exact top-k is a subset."""
    w, q, key, _ = make_case(cuda_device, batch=2, q_heads=2 * G, kv_heads=2, context=T, channels=C)
    ch = ops.choose_channels(key[:, :, :T], C)
    packed, scale = ops.quantize(key[:, :, :T], ch)
    cand, count, tau = ops.score_candidates(q, packed, scale, ch, T, k)
    full = ops.score(q, packed, scale, ch, T, want_acc=False, want_deq=False).gmax.view(-1, T)
    want, _ = oracle.select(full.cpu(), k)
    cap = cand.shape[1]
    for r in range(full.shape[0]):
        n = int(count[r])
        assert k <= n <= cap
        c = cand[r, :n].cpu()
        tok = 0xFFFFFFFF - (c & 0xFFFFFFFF)
        keybits = (c >> 32) & 0xFFFFFFFF
        g = full[r].cpu()[tok]
        gk = g.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        gk = torch.where(gk >= 2**31, (~gk) & 0xFFFFFFFF, gk | 2**31)
        assert torch.equal(keybits, gk)                                   # composites carry the exact score keys
        assert len(set(tok.tolist())) == n                                # no token twice
        assert (g >= tau[r].cpu()).all()
        assert int((full[r] >= tau[r]).sum()) == n                        # and none missed
        assert set(want[r].tolist()) <= set(tok.tolist())
