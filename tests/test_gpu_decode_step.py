"""The fused per-layer step against the oracle chain: selected ids bit-exact, output in tolerance,
side cache extended by the decoded token."""
import pytest
import torch

from kv_cache_b200 import ops
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2


@pytest.mark.parametrize("B,Hq,Hkv,T,C,k,sink,recent", [
    (1, 16, 8, 4096, 32, 256, 0, 0),        # config 0 shapes
    (2, 8, 2, 1000, 64, 64, 0, 0),
    (2, 8, 2, 1000, 64, 64, 10, 10),
    (2, 4, 4, 300, 32, 512, 3, 2),          # k > T
    (1, 8, 1, 70, 128, 16, 0, 0),
    (2, 8, 2, 20000, 64, 512, 0, 0),        # longer than the candidate capacity: sampled threshold path
    (1, 4, 2, 40000, 32, 2048, 5, 5),
    (2, 16, 2, 9000, 64, 100, 0, 0),        # small k: the rank floor of the sample decides tau
    (1, 2, 2, 33000, 128, 3000, 0, 0),      # G = 1, C = 128, k above 8192 / 3
])
def test_step_matches_oracle(cuda_device, B, Hq, Hkv, T, C, k, sink, recent):
    w, q, key, value = make_case(cuda_device, batch=B, q_heads=Hq, kv_heads=Hkv, context=T, channels=C, seed=B + T)
    ch = ops.choose_channels(key[:, :, :T], C)
    packed, scale = ops.alloc_side_cache(B, Hkv, T + 1, C, cuda_device)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    step = ops.DecodeStep(k, protect_sink=sink, protect_recent=recent)
    sel = torch.empty((B, Hkv, min(k, T)), dtype=torch.int32, device=cuda_device)
    out = step(q, key, value, packed, scale, ch, selected_out=sel)
    r = oracle.decode_step(*cpu(q, key, value, ch), k, protect_sink=sink, protect_recent=recent)
    assert torch.equal(sel.cpu().long(), torch.sort(r["selected"], dim=-1).values)   # fused step emits ascending ids
    torch.testing.assert_close(out.float().cpu(), r["out"], rtol=RTOL, atol=ATOL)
    # the decoded token's row joined the int4 cache
    _, packed_o, scale_o = oracle.quantize_pack(key.cpu(), ch.cpu())
    assert torch.equal(packed[:, :, :T + 1].cpu(), packed_o)
    assert torch.equal(scale[:, :, :T + 1].cpu(), scale_o)
    # running it again (now stale workspace contents) gives the same answer
    out2 = step(q, key, value, packed, scale, ch)
    assert torch.equal(out, out2)
    # any-order selection: the same exact set, the same output within the tolerance
    sel3 = torch.empty_like(sel)
    out3 = ops.DecodeStep(k, protect_sink=sink, protect_recent=recent, ordered_selection=False)(
        q, key, value, packed, scale, ch, selected_out=sel3)
    assert torch.equal(torch.sort(sel3, dim=-1).values, sel)
    torch.testing.assert_close(out3.float().cpu(), r["out"], rtol=RTOL, atol=ATOL)


def test_step_equals_operator_chain(cuda_device):
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=5000, channels=64)
    T = 5000
    ch = ops.choose_channels(key[:, :, :T], 64)
    packed, scale = ops.alloc_side_cache(2, 2, T + 1, 64, cuda_device)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    r = ops.score(q, packed, scale, ch, T)
    sel = ops.select(r.gmax, 128, order="index")
    fidx, fvalid = ops.build_final_indices(sel, None, T, T + 1, 4, 4, True)
    chain = ops.sparse_attend(q, key, value, fidx, fvalid)
    fused = ops.DecodeStep(128, 4, 4)(q, key, value, packed, scale, ch)
    assert torch.equal(chain, fused)


def test_device_status_is_clean(cuda_device):
    import ctypes
    from kv_cache_b200 import _native

    st = ctypes.c_int(-1)
    assert _native.lib().kvb_device_status(0, ctypes.byref(st)) == 0
    assert st.value == 0


@pytest.mark.parametrize("T,k", [(30000, 512), (12000, 4000), (300000, 1024)])      # the last: the long-row sampler
def test_heavy_ties_take_the_rescue_path(cuda_device, T, k):
    """Keys quantised from a handful of distinct rows: scores tie massively, the sampled threshold
    admits far more candidates than fit, and the exact refinement over the re-scored row must take over."""
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64, seed=5)
    key = key.clone()
    key[:, :, :T] = key[:, :, :3].repeat(1, 1, (T + 2) // 3, 1)[:, :, :T]
    ch = ops.choose_channels(key[:, :, :T], 64)
    packed, scale = ops.alloc_side_cache(2, 2, T + 1, 64, cuda_device)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    sel = torch.empty((2, 2, k), dtype=torch.int32, device=cuda_device)
    out = ops.DecodeStep(k)(q, key, value, packed, scale, ch, selected_out=sel)
    r = oracle.decode_step(*cpu(q, key, value, ch), k)
    assert torch.equal(sel.cpu().long(), torch.sort(r["selected"], dim=-1).values)
    torch.testing.assert_close(out.float().cpu(), r["out"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("T", [10000, 270000])          # the second: the long-row sampler, every sample value equal
def test_all_zero_keys(cuda_device, T):
    k = 256
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=4, kv_heads=2, context=T, channels=32)
    key = torch.zeros_like(key)
    ch = torch.arange(32, dtype=torch.int32, device=cuda_device).repeat(2, 1)
    packed, scale = ops.alloc_side_cache(1, 2, T + 1, 32, cuda_device)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    sel = torch.empty((1, 2, k), dtype=torch.int32, device=cuda_device)
    ops.DecodeStep(k)(q, key, value, packed, scale, ch, selected_out=sel)
    assert torch.equal(sel.cpu(), torch.arange(k, dtype=torch.int32).expand(1, 2, k))     # all tie: lowest indices win


@pytest.mark.parametrize("zero_copy", [False, True])     # True: kernels read the new rows from / write the output to pinned host memory
def test_graphed_decode_loop_with_device_side_history(cuda_device, zero_copy):
    """One captured graph replayed for consecutive tokens: the history length lives on the device and
    advances by one per replay; every replay must equal the oracle step at that length."""
    T0, k, steps = 12000, 256, 3
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T0 + steps, channels=64, seed=9)
    ch = ops.choose_channels(key[:, :, :T0], 64)
    cache_k = torch.zeros((2, 2, T0 + steps + 4, 128), dtype=torch.bfloat16, device=cuda_device)
    cache_v = torch.zeros_like(cache_k)
    cache_k[:, :, :T0], cache_v[:, :, :T0] = key[:, :, :T0], value[:, :, :T0]
    packed, scale = ops.alloc_side_cache(2, 2, T0 + steps + 4, 64, cuda_device)
    ops.quantize(key[:, :, :T0], ch, out=(packed, scale))
    g = ops.GraphedDecode(ops.DecodeStep(k), cache_k, cache_v, packed, scale, ch, history=T0, q_heads=8, zero_copy=zero_copy)
    for i in range(steps):
        T = T0 + i
        g.h_query.copy_(q)
        g.h_key_row.copy_(key[:, :, T:T + 1])
        g.h_value_row.copy_(value[:, :, T:T + 1])
        out = g().clone()
        assert int(g.history.item()) == T + 1
        want = oracle.decode_step(*cpu(q, key[:, :, :T + 1], value[:, :, :T + 1], ch), k)
        torch.testing.assert_close(out.float(), want["out"], rtol=RTOL, atol=ATOL)
    # the cache and the int4 side cache were extended by the three decoded tokens
    assert torch.equal(cache_k[:, :, :T0 + steps], key[:, :, :T0 + steps])
    _, packed_o, scale_o = oracle.quantize_pack(key[:, :, :T0 + steps].cpu(), ch.cpu())
    assert torch.equal(packed[:, :, :T0 + steps].cpu(), packed_o)
    assert torch.equal(scale[:, :, :T0 + steps].cpu(), scale_o)


def test_paged_kv_pools_give_the_same_step(cuda_device):
    """K and V in pages of 256 tokens scattered over a pool in a shuffled order: the fused step through the page
    table returns the bits it returns on contiguous caches (same selection, same attention order), stores the
    decoded token's rows at their paged place, and appends the same int4 row."""
    from kv_cache_b200.cache import PagedKV

    T, k, P = 20000, 512, 256
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=64, seed=21)
    ch = ops.choose_channels(key[:, :, :T], 64)
    packed, scale = ops.alloc_side_cache(2, 2, T + 1, 64, cuda_device)
    ops.quantize(key[:, :, :T], ch, out=(packed, scale))
    packed2, scale2 = packed.clone(), scale.clone()
    sel = torch.empty((2, 2, k), dtype=torch.int32, device=cuda_device)
    want = ops.DecodeStep(k, protect_sink=4, protect_recent=8)(q, key, value, packed, scale, ch, selected_out=sel)

    pages_per_seq = (T + 1 + P - 1) // P
    order = torch.randperm(2 * pages_per_seq + 5, generator=torch.Generator().manual_seed(3))
    kv = PagedKV(2, 2, 128, P, 2 * pages_per_seq + 5, cuda_device, pages_per_sequence=pages_per_seq, free_order=order)
    kv.append(key[:, :, :T], value[:, :, :T])
    gk, gv = kv.gather()
    assert torch.equal(gk, key[:, :, :T]) and torch.equal(gv, value[:, :, :T])
    kv.reserve(1)
    sel2 = torch.empty_like(sel)
    new_k, new_v = key[:, :, T].contiguous(), value[:, :, T].contiguous()
    got = ops.DecodeStep(k, protect_sink=4, protect_recent=8)(
        q, kv.key_pool, kv.value_pool, packed2, scale2, ch, selected_out=sel2, new_rows=(new_k, new_v),
        kv_pages=(kv.page_table, T))
    kv.advance(1)
    assert torch.equal(sel2, sel)
    assert torch.equal(got, want)
    gk, gv = kv.gather()
    assert torch.equal(gk, key[:, :, :T + 1]) and torch.equal(gv, value[:, :, :T + 1])
    assert torch.equal(packed2[:, :, :T + 1], packed[:, :, :T + 1]) and torch.equal(scale2[:, :, :T + 1], scale[:, :, :T + 1])
