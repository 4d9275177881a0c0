"""Pins the oracle's restatements of reference code against outputs of the reference itself
(tests/golden/reference_golden.npz, produced by tests/golden/make_reference_golden.py)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

GOLD = np.load(Path(__file__).parent / "golden" / "reference_golden.npz")


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("case", range(len(GOLD["fi_cases"])))
def test_final_indices_match_reference(case):
    B, H, history, key_count, kk = GOLD["fi_shape"].tolist()
    sink, recent, keep = GOLD["fi_cases"][case].tolist()
    sel = torch.from_numpy(GOLD["fi_selected"])
    val = torch.from_numpy(GOLD["fi_selected_valid"])
    idx, v = oracle.final_indices_from_selected(sel, val, history, key_count, bool(keep), sink, recent)
    assert torch.equal(idx, torch.from_numpy(GOLD[f"fi_{case}_idx"]))
    assert torch.equal(v, torch.from_numpy(GOLD[f"fi_{case}_valid"]))
    idx, v = oracle.final_indices_from_selected(sel, val, history, key_count, bool(keep), sink, recent,
                                                append_protected=True)
    assert torch.equal(idx, torch.from_numpy(GOLD[f"fi_{case}_app_idx"]))
    assert torch.equal(v, torch.from_numpy(GOLD[f"fi_{case}_app_valid"]))


@pytest.mark.parametrize("masked", [False, True])
def test_attention_from_final_indices_matches_reference_bitwise(masked):
    q, k, v = bf16(GOLD["at_q"]), bf16(GOLD["at_k"]), bf16(GOLD["at_v"])
    idx = torch.from_numpy(GOLD["at_idx"])
    val = torch.from_numpy(GOLD["at_valid"])
    mask = bf16(GOLD["at_mask"]) if masked else None
    out = oracle.attention_from_final_indices(q, k, v, mask, idx, val, q.shape[-1] ** -0.5)
    want = bf16(GOLD["at_out_mask" if masked else "at_out_nomask"])
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("masked", [False, True])
def test_fp32_attention_within_tolerance_of_reference(masked):
    """The fp32-accumulate oracle (what the CUDA kernel is held to) against the reference's bf16 form."""
    q, k, v = bf16(GOLD["at_q"]), bf16(GOLD["at_k"]), bf16(GOLD["at_v"])
    idx = torch.from_numpy(GOLD["at_idx"])
    val = torch.from_numpy(GOLD["at_valid"])
    mask_rows = bf16(GOLD["at_mask"])[:, 0, 0, :].float() if masked else None
    out, _, _ = oracle.attend_fp32(q[:, :, 0, :], k, v, idx, val, q.shape[-1] ** -0.5, mask_rows)
    want = bf16(GOLD["at_out_mask" if masked else "at_out_nomask"]).float()
    torch.testing.assert_close(out, want, rtol=2e-2, atol=1e-2)


def test_partial_scores_match_reference():
    q, k = bf16(GOLD["ds_q"]), bf16(GOLD["ds_k"])
    G = q.shape[1] // k.shape[1]
    kr = k.repeat_interleave(G, dim=1)
    scores, qdim = oracle.qabs_partial_scores(q[:, :, 0, :], kr[:, :, :-1, :], 32)
    assert torch.equal(qdim, torch.from_numpy(GOLD["ps_qdim"]))
    assert torch.equal(scores, torch.from_numpy(GOLD["ps_scores"]))


@pytest.mark.parametrize("case", range(3))
def test_reference_decode_step_restated(case):
    q, k, v = bf16(GOLD["ds_q"]), bf16(GOLD["ds_k"]), bf16(GOLD["ds_v"])
    mode = str(GOLD["ds_modes"][case])
    sink, recent = GOLD["ds_protect"][case].tolist()
    dims, frac = GOLD[f"ds_{case}_params"].tolist()
    out = oracle.qabs_candidate_attention(q, k, v, None, q.shape[-1] ** -0.5, int(dims), frac, True, sink, recent,
                                          append_protected=mode.endswith("appendattn"))
    want = bf16(GOLD[f"ds_{case}_out"])
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))


def test_candidate_count_rule():
    assert oracle.candidate_count(0.0625, 4096) == 256
    assert oracle.candidate_count(0.015625, 131072) == 2048
    assert oracle.candidate_count(0.5, 1) == 1
    assert oracle.candidate_count(0.0, 10) == 1
