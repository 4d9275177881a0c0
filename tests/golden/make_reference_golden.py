"""Generates tests/golden/reference_golden.npz by IMPORTING the reference (littlexi001/kv_cache)
and running its own torch code on small seeded inputs. Only runs where the reference checkout
is present; the produced file is committed and is what the oracle is pinned against.

    python tests/golden/make_reference_golden.py [/path/to/reference]

Functions exercised (EVAL = ymluo/projects/qwen3_top2_head_limit3_ppl/src/
evaluate_qwen3_top2_head_limit3_ppl.py):
  _qabs_final_indices_from_selected   EVAL:2938-2982
  _qabs_final_indices_append_protected EVAL:2985-3022
  _qabs_attention_from_final_indices  EVAL:4612-4647 (torch branch)
  _limited_eager_attention_forward    EVAL:6236 -> _qabs_candidate_attention_forward EVAL:4400-4502
  parse_qabs_partial_rerank_params    EVAL:748-754
  _qabs_reuse_fast_attention_forward  EVAL:3991-4397 with ReuseCandidateState EVAL:1596-1759 (three consecutive
                                      decode steps; fp32 tensors holding bf16-representable values)
  _qabs_candidate_top2_attention_forward EVAL:4650-4766
  _sparq_fast_attention_output_for_query EVAL:2646-2722 with SparQMeanState.value_mean EVAL:2006-2016 (two steps)
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_reference_golden.py <checkout of littlexi001/kv_cache>")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "ymluo/projects/qwen3_top2_head_limit3_ppl/src"))
import evaluate_qwen3_top2_head_limit3_ppl as ref  # noqa: E402

OUT = Path(__file__).resolve().parent / "reference_golden.npz"


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit pattern (npz has no bf16)."""
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def mode(name, sink, recent, keep_self=True):
    return ref.attention_mode(name, 0.02, 3, keep_self, sink, recent, None, qabs_fast_path=True)


def main() -> None:
    torch.manual_seed(1234)
    torch.set_num_threads(1)
    out: dict[str, np.ndarray] = {}

    # ---- final index builders ----------------------------------------------------------
    B, H, history, kk = 2, 3, 97, 12
    key_count = history + 1
    sel = torch.stack([torch.stack([torch.randperm(history)[:kk] for _ in range(H)]) for _ in range(B)])
    sel_valid = torch.rand(B, H, kk) > 0.2
    out["fi_selected"] = sel.numpy()
    out["fi_selected_valid"] = sel_valid.numpy()
    out["fi_shape"] = np.array([B, H, history, key_count, kk])
    cases = [(0, 0, 1), (4, 0, 1), (0, 5, 1), (4, 5, 1), (4, 5, 0), (200, 0, 1), (0, 200, 1), (60, 60, 1)]
    out["fi_cases"] = np.array(cases)
    for ci, (sink, recent, keep) in enumerate(cases):
        with mode("qabs32cand6p25attn", sink, recent, bool(keep)):
            idx, val = ref._qabs_final_indices_from_selected(sel, sel_valid, history, key_count, bool(keep))
            idx2, val2 = ref._qabs_final_indices_append_protected(sel, sel_valid, history, key_count, bool(keep))
        out[f"fi_{ci}_idx"], out[f"fi_{ci}_valid"] = idx.numpy(), val.numpy()
        out[f"fi_{ci}_app_idx"], out[f"fi_{ci}_app_valid"] = idx2.numpy(), val2.numpy()

    # ---- attention from final indices (K/V repeated to the query heads, bf16) ------------
    B, Hq, Tk, D, S = 2, 4, 130, 128, 24
    q = torch.randn(B, Hq, 1, D).to(torch.bfloat16)
    k = (torch.randn(B, Hq, Tk, D) * 1.5).to(torch.bfloat16)
    v = torch.randn(B, Hq, Tk, D).to(torch.bfloat16)
    idx = torch.randint(0, Tk, (B, Hq, S))
    val = torch.rand(B, Hq, S) > 0.15
    mask = torch.zeros(B, 1, 1, Tk, dtype=torch.bfloat16)
    mask[1, 0, 0, :7] = torch.finfo(torch.bfloat16).min
    scaling = D ** -0.5
    with mode("qabs32cand6p25attn", 0, 0):
        o_nomask = ref._qabs_attention_from_final_indices(q, k, v, None, idx, val, scaling)
        o_mask = ref._qabs_attention_from_final_indices(q, k, v, mask, idx, val, scaling)
    out["at_q"], out["at_k"], out["at_v"] = bits(q), bits(k), bits(v)
    out["at_idx"], out["at_valid"], out["at_mask"] = idx.numpy(), val.numpy(), bits(mask)
    out["at_out_nomask"], out["at_out_mask"] = bits(o_nomask), bits(o_mask)

    # ---- whole reference decode step through the dispatcher (un-repeated KV in) ----------
    B, Hq, Hkv, Tk, D = 2, 8, 2, 257, 128
    q = torch.randn(B, Hq, 1, D).to(torch.bfloat16)
    k = (torch.randn(B, Hkv, Tk, D) * torch.exp(torch.randn(1, Hkv, 1, D))).to(torch.bfloat16)
    v = torch.randn(B, Hkv, Tk, D).to(torch.bfloat16)
    out["ds_q"], out["ds_k"], out["ds_v"] = bits(q), bits(k), bits(v)
    step_cases = [("qabs32cand6p25attn", 0, 0), ("qabs16cand12p5attn", 3, 4), ("qabs8cand25appendattn", 2, 2)]
    out["ds_modes"] = np.array([m for m, _, _ in step_cases])
    out["ds_protect"] = np.array([[s, r] for _, s, r in step_cases])

    class _M(torch.nn.Module):
        layer_idx = 0
        scaling = D ** -0.5

    for ci, (m, sink, recent) in enumerate(step_cases):
        with mode(m, sink, recent):
            o, w = ref._limited_eager_attention_forward(_M(), q, k, v, None, scaling=D ** -0.5)
        assert w is None
        out[f"ds_{ci}_out"] = bits(o)
        dims, frac = ref.parse_qabs_partial_rerank_params(m)
        out[f"ds_{ci}_params"] = np.array([dims, frac])

    # partial-score expression alone (EVAL:4428, 4443-4446), K repeated like the dispatcher does
    kr = k.repeat_interleave(Hq // Hkv, dim=1)
    q_raw = q[:, :, 0, :]
    k_hist = kr[:, :, : Tk - 1, :]
    qdim = torch.topk(q_raw.float().abs(), k=32, dim=-1, largest=True).indices
    q_sel = torch.gather(q_raw.float(), -1, qdim)
    k_sel = torch.gather(k_hist.float(), -1, qdim[:, :, None, :].expand(-1, -1, Tk - 1, -1))
    out["ps_scores"] = (k_sel * q_sel[:, :, None, :]).sum(-1).numpy()
    out["ps_qdim"] = qdim.numpy()

    # ---- rerank + reuse over three consecutive steps (EVAL:3991-4397) and the top-2 % mode (EVAL:4650-4766) ----
    # fp32 tensors whose values are exactly representable in bf16: the reference then forms its exact scores in
    # fp32 (no bf16 rounding of q.k, hence no rounding ties at the cut), and a bf16 kernel sees the same numbers.
    B, Hq, Hkv, D, T0 = 2, 8, 2, 128, 300
    G = Hq // Hkv
    rq = torch.randn(3, B, Hq, 1, D).to(torch.bfloat16).float()
    rk = (torch.randn(B, Hkv, T0 + 3, D) * torch.exp(0.7 * torch.randn(1, Hkv, 1, D))).to(torch.bfloat16).float()
    rv = torch.randn(B, Hkv, T0 + 3, D).to(torch.bfloat16).float()
    out["ru_q"], out["ru_k"], out["ru_v"] = bits(rq.to(torch.bfloat16)), bits(rk.to(torch.bfloat16)), bits(rv.to(torch.bfloat16))
    ru_mode, ru_top, ru_sink, ru_recent = "qabs16cand12p5reuse", 0.05, 2, 3
    out["ru_mode"] = np.array([ru_mode])
    out["ru_params"] = np.array([ru_top, ru_sink, ru_recent, T0])
    state = ref.ReuseCandidateState()
    for step in range(3):
        kc = T0 + 1 + step
        with ref.attention_mode(ru_mode, ru_top, 3, True, ru_sink, ru_recent, None, reuse_state=state, qabs_fast_path=True):
            o, w = ref._limited_eager_attention_forward(_M(), rq[step], rk[:, :, :kc], rv[:, :, :kc], None, scaling=D ** -0.5)
        assert w is None
        rec = state.previous_layer[0]
        assert rec["query_token"] == kc - 1
        out[f"ru_{step}_candidate"] = rec["candidate"].numpy()          # bool [B,Hq,history]: this step's own candidates
        out[f"ru_{step}_final"] = rec["final"].numpy()                  # bool [B,Hq,history]: kept set incl. protected ranges
        out[f"ru_{step}_out"] = o.numpy()
        # the cut must not sit on a near-tie (summation order differs between implementations)
        hist = kc - 1
        kr_ = rk[:, :, :hist].repeat_interleave(G, dim=1)
        exact = torch.einsum("bhd,bhtd->bht", rq[step][:, :, 0], kr_) * D ** -0.5
        keep = min(hist, max(1, __import__("math").ceil(ru_top * hist)))
        union = torch.from_numpy(out[f"ru_{step}_candidate"]).clone()
        if step > 0:
            pc = torch.from_numpy(out[f"ru_{step - 1}_candidate"])
            pf = torch.from_numpy(out[f"ru_{step - 1}_final"])
            union[..., : pc.shape[-1]] |= pc | pf
        srt = torch.sort(exact.masked_fill(~union, float("-inf")), dim=-1, descending=True).values
        assert float((srt[..., keep - 1] - srt[..., keep]).min()) > 1e-4, "near-tie at the cut: change the seed"

    t2_mode, t2_top = "qabs16cand12p5top2attn", 0.03
    kc = T0 + 1
    with ref.attention_mode(t2_mode, t2_top, 3, True, 2, 3, None, qabs_fast_path=True):
        o, w = ref._limited_eager_attention_forward(_M(), rq[0], rk[:, :, :kc], rv[:, :, :kc], None, scaling=D ** -0.5)
    out["t2_mode"] = np.array([t2_mode])
    out["t2_params"] = np.array([t2_top, 2, 3])
    out["t2_out"] = o.numpy()

    # ---- SparQ fast mode with its running mean of V, two consecutive steps (EVAL:2646-2722, 2006-2016) ----
    sq_mode = "sparqfast16cand12p5"
    out["sq_mode"] = np.array([sq_mode])
    sq_state = ref.SparQMeanState()
    for step in range(2):
        kc = T0 + 1 + step
        with ref.attention_mode(sq_mode, 0.02, 3, True, 0, 0, None, sparq_mean_state=sq_state, qabs_fast_path=True):
            o, w = ref._limited_eager_attention_forward(_M(), rq[step], rk[:, :, :kc], rv[:, :, :kc], None, scaling=D ** -0.5)
        out[f"sq_{step}_out"] = o.numpy()
        out[f"sq_{step}_vmean"] = sq_state.previous_layer[0]["mean"].numpy()

    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.1f} KiB), {len(out)} arrays")


if __name__ == "__main__":
    main()
