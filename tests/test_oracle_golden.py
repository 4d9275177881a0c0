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


def _f32(a):
    return bf16(a).float()


def test_reuse_steps_restated_against_the_reference():
    """Three consecutive steps of the reference's rerank + reuse mode (EVAL:3991-4397): the masks it stores for
    the next step and its outputs, from the oracle's restatement fed with its own previous masks."""
    q, k, v = _f32(GOLD["ru_q"]), _f32(GOLD["ru_k"]), _f32(GOLD["ru_v"])
    top, sink, recent, T0 = GOLD["ru_params"].tolist()
    sink, recent, T0 = int(sink), int(recent), int(T0)
    dims, frac = 16, 0.125
    assert str(GOLD["ru_mode"][0]) == "qabs16cand12p5reuse"
    pc = pf = None
    for step in range(3):
        kc = T0 + 1 + step
        out, cur, fin = oracle.qabs_reuse_step(q[step], k[:, :, :kc], v[:, :, :kc], 128 ** -0.5, dims, frac, top, pc, pf,
                                               sink, recent)
        assert torch.equal(cur, torch.from_numpy(GOLD[f"ru_{step}_candidate"]))
        assert torch.equal(fin, torch.from_numpy(GOLD[f"ru_{step}_final"]))
        torch.testing.assert_close(out, torch.from_numpy(GOLD[f"ru_{step}_out"]), rtol=1e-5, atol=1e-6)
        pc, pf = cur, fin


def test_top2_step_restated_against_the_reference():
    q, k, v = _f32(GOLD["ru_q"]), _f32(GOLD["ru_k"]), _f32(GOLD["ru_v"])
    top, sink, recent = GOLD["t2_params"].tolist()
    T0 = int(GOLD["ru_params"][3])
    out, sel = oracle.qabs_top2_step(q[0], k[:, :, :T0 + 1], v[:, :, :T0 + 1], None, 128 ** -0.5, 16, 0.125, top,
                                     int(sink), int(recent))
    torch.testing.assert_close(out, torch.from_numpy(GOLD["t2_out"]), rtol=1e-5, atol=1e-6)
    assert sel.shape[-1] == 9                                            # min(38 candidates, ceil(0.03 * 300))


def test_list_rerank_equals_the_mask_form():
    """oracle.rerank_union (lists, this project's tie rule) against the reference's mask form on the recorded
    steps: per query head, the kept ids plus the protected ranges are exactly the reference's final mask."""
    q, k = _f32(GOLD["ru_q"]), _f32(GOLD["ru_k"])
    top, sink, recent, T0 = GOLD["ru_params"].tolist()
    sink, recent, T0 = int(sink), int(recent), int(T0)
    import math
    for step in range(3):
        hist = T0 + step
        keep = min(hist, max(1, math.ceil(top * hist)))
        masks = [torch.from_numpy(GOLD[f"ru_{step}_candidate"])]
        if step:
            masks += [torch.from_numpy(GOLD[f"ru_{step - 1}_candidate"]), torch.from_numpy(GOLD[f"ru_{step - 1}_final"])]
        lists = []
        for m in masks:
            n = int(m.sum(-1).max())
            ids = torch.full((*m.shape[:2], n), -1, dtype=torch.long)
            for b in range(m.shape[0]):
                for h in range(m.shape[1]):
                    nz = torch.nonzero(m[b, h]).flatten()
                    ids[b, h, :nz.numel()] = nz
            lists.append(ids)
        kept, cnt = oracle.rerank_union(q[step][:, :, 0], k[:, :, :hist], lists, hist, keep, 128 ** -0.5)
        final = oracle.expand_final(kept, hist, counts=cnt, force_sink=sink, force_recent=recent)
        want = torch.from_numpy(GOLD[f"ru_{step}_final"])
        for r, f in enumerate(final):
            b, h = divmod(r, want.shape[1])
            assert f == torch.nonzero(want[b, h]).flatten().tolist()


def test_sparq_fast_steps_restated_against_the_reference():
    """Two consecutive steps of the reference's SparQ fast mode with its running mean of V (EVAL:2646-2722,
    2006-2016): the oracle's restatement, fed the incrementally updated mean, reproduces the recorded outputs."""
    q, k, v = _f32(GOLD["ru_q"]), _f32(GOLD["ru_k"]), _f32(GOLD["ru_v"])
    T0 = int(GOLD["ru_params"][3])
    G = q.shape[2] // k.shape[1]
    mean = None
    for step in range(2):
        kc = T0 + 1 + step
        vr = v[:, :, :kc].repeat_interleave(G, dim=1)
        if mean is None:
            mean = vr.float().mean(dim=2, keepdim=True)                                   # EVAL:2014
        else:
            mean = (mean * float(kc - 1) + vr[:, :, -1:, :].float()) / float(kc)           # EVAL:2011-2012
        torch.testing.assert_close(mean, torch.from_numpy(GOLD[f"sq_{step}_vmean"]), rtol=1e-6, atol=1e-7)
        out = oracle.sparq_fast_step(q[step], k[:, :, :kc], v[:, :, :kc], None, 128 ** -0.5, 16, 0.125, value_mean=mean)
        torch.testing.assert_close(out, torch.from_numpy(GOLD[f"sq_{step}_out"]), rtol=1e-5, atol=1e-6)
