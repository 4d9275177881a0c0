"""The drop-in ``qabs_cuda_kernels`` module: the reference's four callables (QCK:654-705) against
outputs recorded from the reference's own torch code (golden vectors) and against the oracle."""
from pathlib import Path

import numpy as np
import pytest
import torch

from kv_cache_b200 import qabs_cuda_kernels as qck
from oracle import oracle

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "reference_golden.npz")


def bf16(a):
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def test_partial_scores_match_the_reference_expression(cuda_device):
    """Inputs and fp32 scores recorded from EVAL:4428 + 4443-4446 (32 channels by |q|)."""
    q = bf16(GOLD["ds_q"])[:, :, 0, :].to(cuda_device)                    # [B,Hq,D]
    k = bf16(GOLD["ds_k"]).to(cuda_device)                                # [B,Hkv,Tk,D], not repeated
    want = torch.from_numpy(GOLD["ps_scores"])
    got = qck.partial_scores(q, k[:, :, :-1, :], 32)                      # sliced view, KV heads not repeated
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-4)     # same fp32 products, other summation order
    rep = k.repeat_interleave(q.shape[1] // k.shape[1], dim=1)
    got_rep = qck.partial_scores(q, rep[:, :, :-1, :], 32)                # the layout the reference passes
    assert torch.equal(got_rep, got)
    # channel list given + dim-major K (the second reference entry point)
    qdim = torch.from_numpy(GOLD["ps_qdim"]).to(cuda_device)
    kdm = rep[:, :, :-1, :].transpose(2, 3).contiguous()                  # [B,H,D,T]
    got_dm = qck.partial_scores_dim_major(q, kdm, qdim)
    torch.testing.assert_close(got_dm.cpu(), want, rtol=1e-5, atol=1e-4)


def test_channel_choice_ties_go_to_the_lower_channel(cuda_device):
    q = torch.zeros(1, 1, 128, dtype=torch.bfloat16, device=cuda_device)
    q[0, 0, [5, 9, 70]] = torch.tensor([2.0, -2.0, 2.0], dtype=torch.bfloat16, device=cuda_device)
    k = torch.zeros(1, 1, 3, 128, dtype=torch.bfloat16, device=cuda_device)
    k[0, 0, 0, 5] = 1.0
    k[0, 0, 1, 9] = 1.0
    k[0, 0, 2, 70] = 1.0
    assert qck.partial_scores(q, k, 2)[0, 0].tolist() == [2.0, -2.0, 0.0]   # channels 5 and 9 chosen, 70 not


def test_candidate_full_scores_and_final_attention(cuda_device):
    g = torch.Generator(device=cuda_device).manual_seed(4)
    B, H, T, D = 2, 4, 300, 128
    q = torch.randn(B, H, D, generator=g, device=cuda_device).to(torch.bfloat16)
    k = torch.randn(B, H, T, D, generator=g, device=cuda_device).to(torch.bfloat16)
    v = torch.randn(B, H, T, D, generator=g, device=cuda_device).to(torch.bfloat16)
    cur = torch.rand(B, H, T, generator=g, device=cuda_device) > 0.9
    prev = torch.rand(B, H, T, generator=g, device=cuda_device) > 0.95
    got = qck.candidate_full_scores(q, k, cur, prev, None, 4, 6, D ** -0.5)
    want = oracle.qabs_candidate_full_scores(q.cpu(), k.cpu(), cur.cpu(), prev.cpu(), None, 4, 6, D ** -0.5)
    assert torch.equal(torch.isinf(got.cpu()), torch.isinf(want))
    fin = ~torch.isinf(want)
    torch.testing.assert_close(got.cpu()[fin], want[fin], rtol=1e-5, atol=1e-4)
    idx = torch.randint(0, T, (B, H, 40), generator=g, device=cuda_device)
    valid = torch.rand(B, H, 40, generator=g, device=cuda_device) > 0.2
    out = qck.final_attention(q, k, v, idx, valid, D ** -0.5)
    ref = oracle.attention_from_final_indices(q.cpu()[:, :, None, :], k.cpu(), v.cpu(), None, idx.cpu(), valid.cpu(), D ** -0.5)
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_the_four_callables_take_fp32_and_fp16_like_the_reference(cuda_device, dtype):
    """The reference's extension is compiled for float, half and bfloat16 (QCK:430-458)."""
    g = torch.Generator(device=cuda_device).manual_seed(8)
    B, H, Hk, T, D = 2, 4, 2, 257, 128
    q = torch.randn(B, H, D, generator=g, device=cuda_device).to(dtype)
    k = torch.randn(B, Hk, T, D, generator=g, device=cuda_device).to(dtype)
    v = torch.randn(B, Hk, T, D, generator=g, device=cuda_device).to(dtype)
    rep = k.repeat_interleave(H // Hk, dim=1)
    want, qdim = oracle.qabs_partial_scores(q.cpu(), rep.cpu(), 16)
    got = qck.partial_scores(q, k, 16)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-3)
    got_dm = qck.partial_scores_dim_major(q, rep.transpose(2, 3).contiguous(), qdim.to(cuda_device))
    torch.testing.assert_close(got_dm.cpu(), want, rtol=1e-4, atol=1e-3)
    cur = torch.rand(B, H, T, generator=g, device=cuda_device) > 0.8
    full = qck.candidate_full_scores(q, k, cur, None, None, 2, 3, D ** -0.5)
    want_full = oracle.qabs_candidate_full_scores(q.cpu(), rep.cpu(), cur.cpu(), None, None, 2, 3, D ** -0.5)
    fin = ~torch.isinf(want_full)
    assert torch.equal(torch.isinf(full.cpu()), ~fin)
    torch.testing.assert_close(full.cpu()[fin], want_full[fin], rtol=1e-4, atol=1e-3)
    idx = torch.randint(0, T, (B, H, 33), generator=g, device=cuda_device)
    valid = torch.rand(B, H, 33, generator=g, device=cuda_device) > 0.2
    out = qck.final_attention(q, k, v, idx, valid, D ** -0.5)
    assert out.dtype == dtype and out.shape == (B, 1, H, D)
    ref, _, _ = oracle.attend_fp32(q.cpu().to(torch.bfloat16), k.cpu().to(torch.bfloat16), v.cpu().to(torch.bfloat16),
                                   idx.cpu(), valid.cpu(), D ** -0.5)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2e-2, atol=1e-2)
