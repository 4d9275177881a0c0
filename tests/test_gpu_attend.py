"""Stage 4 parity: sparse attention within 2e-2 relative / 1e-2 absolute of the fp32 oracle and
of the reference's own bf16 torch form (golden vectors produced by the reference)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from kv_cache_b200 import ops
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2
GOLD = np.load(Path(__file__).parent / "golden" / "reference_golden.npz")


def bf16(a):
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("S", [1, 31, 32, 33, 200, 2049])
def test_against_fp32_oracle(cuda_device, G, S):
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=2 * G, kv_heads=2, context=3000)
    g = torch.Generator(device=cuda_device).manual_seed(S)
    idx = torch.randint(0, 3001, (2, 2, S), generator=g, device=cuda_device)
    valid = torch.rand(2, 2, S, generator=g, device=cuda_device) > 0.1
    out = ops.sparse_attend(q, key, value, idx, valid)
    want, _, _ = oracle.attend_fp32(*cpu(q, key, value, idx, valid), 128 ** -0.5)
    assert out.shape == (2, 1, 2 * G, 128) and out.dtype == torch.bfloat16
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)


def test_per_query_head_lists_int32_and_partials(cuda_device):
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=500)
    g = torch.Generator(device=cuda_device).manual_seed(1)
    idx = torch.randint(0, 501, (2, 8, 70), generator=g, device=cuda_device, dtype=torch.int32)
    out = ops.sparse_attend(q, key, value, idx)
    want, m, l = oracle.attend_fp32(*cpu(q, key, value, idx), None, 128 ** -0.5)
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)
    part = ops.sparse_attend(q, key, value, idx, return_partial=True).cpu()
    torch.testing.assert_close(part[..., -2], m, rtol=1e-3, atol=1e-3)
    o_norm = part[..., :-2] / part[..., -1:]
    torch.testing.assert_close(o_norm[:, None], want, rtol=RTOL, atol=ATOL)
    merged = ops.lse_merge(part[None].to(cuda_device))
    torch.testing.assert_close(merged.float().cpu(), want, rtol=RTOL, atol=ATOL)


def test_invalid_out_of_range_and_empty_lists(cuda_device):
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=4, kv_heads=2, context=100)
    idx = torch.tensor([[[5, -1, 1000, 7], [1, 2, 3, 4]]], device=cuda_device)
    valid = torch.tensor([[[True, True, True, False], [False, False, False, False]]], device=cuda_device)
    out = ops.sparse_attend(q, key, value, idx, valid)
    want, _, _ = oracle.attend_fp32(*cpu(q, key, value, idx, valid), 128 ** -0.5)
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)
    assert (out[0, 0, 2:] == 0).all()                       # no valid entry -> zeros (QCK:388,404)
    torch.testing.assert_close(out[0, 0, 0].float(), value[0, 0, 5].float(), rtol=RTOL, atol=ATOL)


def test_additive_mask_and_strided_kv(cuda_device):
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=4, kv_heads=2, context=400)
    key_v, value_v = key[:, :, :300], value[:, :, :300]     # sliced views of a longer cache
    g = torch.Generator(device=cuda_device).manual_seed(2)
    idx = torch.randint(0, 300, (2, 2, 90), generator=g, device=cuda_device)
    mask = torch.zeros(2, 1, 1, 300, dtype=torch.bfloat16, device=cuda_device)
    mask[1, 0, 0, :150] = torch.finfo(torch.bfloat16).min
    out = ops.sparse_attend(q, key_v, value_v, idx, attention_mask=mask)
    want, _, _ = oracle.attend_fp32(*cpu(q, key_v, value_v, idx), None, 128 ** -0.5, mask[:, 0, 0].float().cpu())
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("masked", [False, True])
def test_reference_golden_vectors(cuda_device, masked):
    """Inputs and outputs recorded from the reference's _qabs_attention_from_final_indices."""
    q, k, v = (bf16(GOLD[n]).to(cuda_device) for n in ("at_q", "at_k", "at_v"))
    idx = torch.from_numpy(GOLD["at_idx"]).to(cuda_device)
    val = torch.from_numpy(GOLD["at_valid"]).to(cuda_device)
    mask = bf16(GOLD["at_mask"]).to(cuda_device) if masked else None
    out = ops.sparse_attend(q, k, v, idx, val, attention_mask=mask)      # Hkv == Hq here (repeated KV)
    want = bf16(GOLD["at_out_mask" if masked else "at_out_nomask"]).float()
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("case", range(len(GOLD["fi_cases"])))
def test_final_index_builder_matches_reference(cuda_device, case):
    B, H, history, key_count, kk = GOLD["fi_shape"].tolist()
    sink, recent, keep = GOLD["fi_cases"][case].tolist()
    sel = torch.from_numpy(GOLD["fi_selected"]).to(cuda_device)
    val = torch.from_numpy(GOLD["fi_selected_valid"]).to(cuda_device)
    for app, tag in ((False, ""), (True, "_app")):
        idx, v = ops.build_final_indices(sel, val, history, key_count, sink, recent, bool(keep), app)
        assert torch.equal(idx.cpu().long(), torch.from_numpy(GOLD[f"fi_{case}{tag}_idx"]))
        assert torch.equal(v.cpu(), torch.from_numpy(GOLD[f"fi_{case}{tag}_valid"]))
