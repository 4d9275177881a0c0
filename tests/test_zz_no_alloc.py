"""The allocation-free select entry point (kvb_select_topk_static).

It exists for hosts that must not allocate device memory where they call the library (inside a
stream-ordered region, under an embedding runtime that owns all allocation, with the memory budget
already spent): its workspace is a fixed array inside the library image. The test drives it through
the C ABI twice in a row — the array keeps the previous call's contents, so the second call proves
that stale scratch does no harm — and checks every output bit for bit against kvb_select_topk
and against the CPU oracle's select. Collected last on purpose; it must pass on its own and after the rest of the suite."""
import ctypes

import pytest
import torch

from kv_cache_b200 import _native
from oracle import oracle

pytestmark = pytest.mark.gpu


def _reference(lib, scores, k, order, dev):
    R, T = scores.shape
    kk = min(k, T)
    ws_bytes = lib.kvb_select_topk_workspace_bytes(R, T, kk)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    idx32 = torch.empty((R, kk), dtype=torch.int32, device=dev)
    idx64 = torch.empty((R, kk), dtype=torch.int64, device=dev)
    val = torch.empty((R, kk), dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.kvb_select_topk(scores.data_ptr(), scores.stride(0), None, R, T, k, 7, order, idx32.data_ptr(),
                             idx64.data_ptr(), val.data_ptr(), None, ws.data_ptr(), ws_bytes, dev.index, st)
    assert rc == 0
    return idx32, idx64, val


def _static(lib, scores, k, order, dev):
    R, T = scores.shape
    kk = min(k, T)
    idx32 = torch.full((R, kk), -1, dtype=torch.int32, device=dev)
    idx64 = torch.full((R, kk), -1, dtype=torch.int64, device=dev)
    val = torch.full((R, kk), float("nan"), dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.kvb_select_topk_static(scores.data_ptr(), scores.stride(0), R, T, k, 7, order, idx32.data_ptr(),
                                    idx64.data_ptr(), val.data_ptr(), dev.index, st)
    assert rc == 0, _native.STATUS_NAMES.get(rc, rc)
    return idx32, idx64, val


def test_static_select_matches_workspace_select_on_two_calls_in_a_row(cuda_device):
    lib = _native.lib()
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(99)
    first = torch.randn(16, 50000, generator=g, device=dev)
    # second call: other shape, heavy ties (takes the refinement path) and k > T on a short row set
    second = torch.randint(-2, 3, (8, 30000), generator=g, device=dev).float()
    third = torch.randn(3, 100, generator=g, device=dev)
    for scores, k in ((first, 2048), (second, 4096), (third, 500)):
        for order in (0, 1):
            want = _reference(lib, scores, k, order, dev)
            got = _static(lib, scores, k, order, dev)
            torch.cuda.synchronize()
            for a, b in zip(got, want):
                assert torch.equal(a, b)
            # and against the oracle: (score desc, index asc) order, or the same set by ascending index
            o_idx, o_val = oracle.select(scores.cpu(), k)
            if order == 1:
                by_index = torch.sort(o_idx, dim=-1)
                o_idx, o_val = by_index.values, torch.gather(o_val, -1, by_index.indices)
            assert torch.equal(got[1].cpu(), o_idx + 7)
            assert torch.equal(got[2].cpu(), o_val)


def test_static_select_refuses_what_does_not_fit(cuda_device):
    lib = _native.lib()
    dev = cuda_device
    limit = lib.kvb_select_topk_static_limit_bytes()
    assert limit == 4 << 20
    R, T, k = 512, 4096, 256
    assert lib.kvb_select_topk_workspace_bytes(R, T, k) > limit
    scores = torch.zeros((R, T), dtype=torch.float32, device=dev)
    out = torch.empty((R, k), dtype=torch.int32, device=dev)
    rc = lib.kvb_select_topk_static(scores.data_ptr(), T, R, T, k, 0, 0, out.data_ptr(), None, None, dev.index,
                                    torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 8 and lib.kvb_status_string(rc) == b"problem exceeds the built-in scratch"
