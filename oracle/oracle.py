"""CPU oracle for the retrieval-sparse decode attention path — TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this file; tests, the smoke check and the CPU-baseline leg of
the benchmark use it as the checker. It is written with torch CPU ops (and a little numpy).

Two kinds of functions live here.

(1) Restatements of code that exists in the reference (littlexi001/kv_cache); each cites the
    lines it follows. These are pinned by the golden vectors in tests/golden/ that were produced
    by importing the reference itself (tests/golden/make_reference_golden.py):
      EVAL = ymluo/projects/qwen3_top2_head_limit3_ppl/src/evaluate_qwen3_top2_head_limit3_ppl.py
      QCK  = ymluo/projects/qwen3_top2_head_limit3_ppl/src/qabs_cuda_kernels.py
(2) The int4 stages the reference does not have (quantize/pack, integer scoring, GQA-group
    max, tie-broken top-k, block scoring, shard merge). PARITY UNPINNED for these: no reference
    code, test or golden vector exists; the semantics below are this project's own pinned
    specification, stated once here and implemented independently by the CUDA kernels.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

TWO_M24 = 2.0 ** -24


# ==========================================================================================
# (2) int4 path — project specification (parity unpinned by the reference)
# ==========================================================================================

def choose_channels(key: torch.Tensor, num_channels: int) -> torch.Tensor:
    """Per KV head the C channels with the largest mean |K| over (B, T); ties -> lower channel;
    ascending int32 [Hkv, C]. The mean is taken in fp64: a sum of bf16 magnitudes is exact there for
    any realistic cache (8-bit mantissas, 53-bit accumulator), so the result does not depend on the
    order of summation and "equal means" is a well-defined notion."""
    B, Hkv, T, D = key.shape
    total = torch.zeros((Hkv, D), dtype=torch.float64)
    for t0 in range(0, T, 65536):                                      # bounded temporaries
        total += key[:, :, t0:t0 + 65536].to(torch.float64).abs().sum(dim=(0, 2))
    mean_abs = total / max(1, B * T)
    order = torch.sort(mean_abs, dim=-1, descending=True, stable=True).indices[:, :num_channels]
    return torch.sort(order, dim=-1).values.to(torch.int32)


def _div(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """IEEE fp32 division, done by numpy so that no library rewrites x / c as x * (1 / c)."""
    return torch.from_numpy(np.divide(a.numpy().astype(np.float32), b.numpy().astype(np.float32), dtype=np.float32))


def quantize_pack(key: torch.Tensor, channel_idx: torch.Tensor):
    """key bf16 [B,Hkv,T,D], channel_idx [Hkv,C] -> codes int8 [B,Hkv,T,C] in [-7,7],
    packed uint8 [B,Hkv,T,C/2] (byte j: low nibble = code 2j, high nibble = code 2j+1, two's
    complement), scale fp32 [B,Hkv,T] = max(absmax, 2^-24) / 7 (IEEE), code = clamp(round_half_even(x / scale))."""
    B, Hkv, T, D = key.shape
    C = channel_idx.shape[-1]
    idx = channel_idx.long()[None, :, None, :].expand(B, Hkv, T, C)
    ksel = torch.gather(key.float(), -1, idx)
    absmax = ksel.abs().amax(-1)
    scale = _div(absmax.clamp_min(TWO_M24), torch.full_like(absmax, 7.0))
    codes = torch.round(_div(ksel, scale[..., None].expand_as(ksel))).clamp(-7, 7).to(torch.int8)
    u = codes.to(torch.int16) & 0xF
    packed = (u[..., 0::2] | (u[..., 1::2] << 4)).to(torch.uint8)
    return codes, packed, scale


def unpack(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [..., C/2] -> int8 codes [..., C]."""
    p = packed.to(torch.int16)
    lo = p & 0xF
    hi = (p >> 4) & 0xF
    lo = torch.where(lo >= 8, lo - 16, lo)
    hi = torch.where(hi >= 8, hi - 16, hi)
    return torch.stack((lo, hi), dim=-1).flatten(-2).to(torch.int8)


def quantize_query(query: torch.Tensor, channel_idx: torch.Tensor):
    """query bf16 [B,Hq,D] -> qcode int8 [B,Hq,C] in [-127,127], qscale fp32 [B,Hq] =
    max(absmax, 2^-24) / 127, over the channels of the head's KV head."""
    B, Hq, D = query.shape
    Hkv, C = channel_idx.shape
    G = Hq // Hkv
    idx = channel_idx.long().repeat_interleave(G, dim=0)[None].expand(B, Hq, C)
    qsel = torch.gather(query.float(), -1, idx)
    absmax = qsel.abs().amax(-1)
    qscale = _div(absmax.clamp_min(TWO_M24), torch.full_like(absmax, 127.0))
    qcode = torch.round(_div(qsel, qscale[..., None].expand_as(qsel))).clamp(-127, 127).to(torch.int8)
    return qcode, qscale


def score(qcode: torch.Tensor, qscale: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor):
    """acc int32 [B,Hq,T] = sum_c qcode*code (exact); deq = (float(acc) * scale[b,h/G,t]) * qscale[b,h]
    with two separately rounded fp32 products in this order; gmax [B,Hkv,T] = max over the group,
    -0 folded into +0."""
    B, Hq, C = qcode.shape
    Hkv, T = codes.shape[1], codes.shape[2]
    G = Hq // Hkv
    # exact: |acc| <= 128 * 127 * 7 < 2^24, so an fp32 (or fp64) matmul of small integers is exact
    qf = qcode.to(torch.float64).view(B, Hkv, G, C)
    cf = codes.to(torch.float64)                                   # [B,Hkv,T,C]
    acc = torch.einsum("bgqc,bgtc->bgqt", qf, cf).round().to(torch.int32).reshape(B, Hq, T)
    ks = scale.repeat_interleave(G, dim=1)                         # [B,Hq,T]
    deq = (acc.to(torch.float32) * ks) * qscale[..., None]
    gmax = deq.view(B, Hkv, G, T).amax(dim=2) + 0.0
    return acc, deq, gmax


def select(gmax: torch.Tensor, k: int, index: Optional[torch.Tensor] = None):
    """Per row: order (score desc, index asc), first min(k, T). Stable descending sort, never
    torch.topk (which leaves the order of ties unspecified). With ``index`` (same shape as gmax,
    unique per row) the tie-break and the returned ids use it instead of the column number."""
    T = gmax.shape[-1]
    kk = min(k, T)
    g = gmax + 0.0
    if index is None:
        order = torch.sort(g, dim=-1, descending=True, stable=True).indices[..., :kk]
        return order, torch.gather(g, -1, order)
    # sort by index ascending first, then stable by score descending
    by_idx = torch.sort(index, dim=-1, stable=True).indices
    g1 = torch.gather(g, -1, by_idx)
    o2 = torch.sort(g1, dim=-1, descending=True, stable=True).indices[..., :kk]
    pos = torch.gather(by_idx, -1, o2)
    return torch.gather(index, -1, pos), torch.gather(g, -1, pos)


def attend_fp32(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, indices: torch.Tensor,
                valid: Optional[torch.Tensor], scaling: float, mask_rows: Optional[torch.Tensor] = None):
    """fp32-accumulate form of the sparse attention on UN-repeated K/V: query [B,Hq,D] bf16,
    key/value [B,Hkv,Tk,D] bf16, indices [B,Hkv|Hq,S]. Returns (out fp32 [B,1,Hq,D], m, l)."""
    B, Hq, D = query.shape
    Hkv, Tk = key.shape[1], key.shape[2]
    G = Hq // Hkv
    Hi = indices.shape[1]
    idx = indices.long()
    if valid is None:
        valid = torch.ones_like(idx, dtype=torch.bool)
    ok = valid.bool() & (idx >= 0) & (idx < Tk)
    idx = idx.clamp(0, Tk - 1)
    if Hi == Hkv:
        idx = idx.repeat_interleave(G, dim=1)
        ok = ok.repeat_interleave(G, dim=1)
    # rows are gathered from the un-repeated cache (head h reads KV head h // G): same values as
    # repeating K/V to the query heads first, without the G-fold copy of the whole cache
    bi = torch.arange(B)[:, None, None]
    hi = (torch.arange(Hq) // G)[None, :, None]
    ks = key[bi, hi, idx].float()                                   # [B,Hq,S,D]
    vs = value[bi, hi, idx].float()
    s = torch.einsum("bhd,bhsd->bhs", query.float(), ks) * scaling
    if mask_rows is not None:
        s = s + torch.gather(mask_rows.float()[:, None, :].expand(-1, Hq, -1), -1, idx)
    s = s.masked_fill(~ok, float("-inf"))
    m = s.amax(-1)
    mu = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - mu[..., None])
    p = torch.where(ok, p, torch.zeros_like(p))
    l = p.sum(-1)
    o = torch.einsum("bhs,bhsd->bhd", p, vs)
    out = torch.where(l[..., None] > 0, o / l.clamp_min(1e-30)[..., None], torch.zeros_like(o))
    return out[:, None, :, :], m, l


def decode_step(query, key, value, channel_idx, top_k, *, protect_sink=0, protect_recent=0, keep_self=True,
                append_protected=False, scaling=None):
    """The whole int4 path on CPU for key/value holding history+1 rows. Returns a dict."""
    B, Hq, D = query.shape
    Tk = key.shape[2]
    T = Tk - 1
    scaling = D ** -0.5 if scaling is None else scaling
    codes, packed, kscale = quantize_pack(key[:, :, :T], channel_idx)
    qcode, qscale = quantize_query(query, channel_idx)
    acc, deq, gmax = score(qcode, qscale, codes, kscale)
    sel, sel_scores = select(gmax, top_k)
    fidx, fvalid = final_indices_from_selected(sel, torch.ones_like(sel, dtype=torch.bool), T, Tk, keep_self,
                                               protect_sink, protect_recent, append_protected)
    out, m, l = attend_fp32(query, key, value, fidx, fvalid, scaling)
    return dict(codes=codes, packed=packed, kscale=kscale, qcode=qcode, qscale=qscale, acc=acc, deq=deq, gmax=gmax,
                selected=sel, selected_scores=sel_scores, final_indices=fidx, final_valid=fvalid, out=out, m=m, l=l)


def reuse_decode_step(query, key, value, channel_idx, candidate_k, keep, *, prev_candidate=None, prev_final=None,
                      protect_sink=0, protect_recent=0, keep_self=True, block_size=1, scaling=None, mask_rows=None):
    """The rerank / reuse step of this project on the int4 path (parity unpinned for the int4 part; the union /
    exact-score / top-keep / protected-range / block stages follow the reference, see rerank_union and
    qabs_reuse_step): per KV head, candidates = int4 group-max top-candidate_k; union with the previous step's
    candidate and final lists; exact rerank with the group maximum of q.k; keep the best `keep`; final set =
    kept + protected ranges, widened to blocks; attention over final + self. Lists are int tensors [B,Hkv,n]
    (-1 padded). Returns dict(candidates, kept, kept_count, final (list of lists per row), out)."""
    B, Hq, D = query.shape
    Hkv, Tk = key.shape[1], key.shape[2]
    T = Tk - 1
    scaling = D ** -0.5 if scaling is None else scaling
    codes, _, kscale = quantize_pack(key[:, :, :T], channel_idx)
    qcode, qscale = quantize_query(query, channel_idx)
    _, _, gmax = score(qcode, qscale, codes, kscale)
    cand, _ = select(gmax, candidate_k)
    kept, kept_count = rerank_union(query, key, [cand, prev_candidate, prev_final], T, keep, scaling, mask_rows=mask_rows)
    final = expand_final(kept, T, counts=kept_count, force_sink=protect_sink, force_recent=protect_recent,
                         block_size=block_size)
    S = max(len(f) for f in final) + (1 if keep_self else 0)
    idx = torch.zeros((B, Hkv, S), dtype=torch.long)
    valid = torch.zeros((B, Hkv, S), dtype=torch.bool)
    for r, f in enumerate(final):
        b, g = divmod(r, Hkv)
        row = f + ([T] if keep_self else [])
        idx[b, g, :len(row)] = torch.tensor(row, dtype=torch.long)
        valid[b, g, :len(row)] = True
    out, _, _ = attend_fp32(query, key, value, idx, valid, scaling, mask_rows)
    return dict(candidates=cand, kept=kept, kept_count=kept_count, final=final, out=out)


def sparq_alpha(query, deq, selected, channel_idx, mask_rows=None):
    """alpha[b,h] = softmax mass, over all T tokens, of the ids in selected[b, h // G] under the logits
    deq[b,h,t] / sqrt(D * |q_sel|_1 / |q|_1) (+ mask): the blend weight of EVAL:2683-2686, 2720-2722 with the
    dequantised int4 partial score as the approximate logit."""
    B, Hq, D = query.shape
    Hkv = channel_idx.shape[0]
    G = Hq // Hkv
    T = deq.shape[-1]
    qf = query.float()
    idx = channel_idx.long().repeat_interleave(G, dim=0)[None].expand(B, Hq, -1)
    sel_abs = torch.gather(qf, -1, idx).abs().sum(-1).clamp_min(1.0e-6)
    all_abs = qf.abs().sum(-1).clamp_min(1.0e-6)
    ds = torch.sqrt(D * sel_abs / all_abs)
    logits = deq.double() / ds[..., None].double()
    if mask_rows is not None:
        logits = logits + mask_rows[:, None, :T].double()
    w = torch.softmax(logits, dim=-1)
    alpha = torch.zeros((B, Hq), dtype=torch.float64)
    for b in range(B):
        for h in range(Hq):
            ids = [int(x) for x in selected[b, h // G].tolist() if 0 <= int(x) < T]
            alpha[b, h] = w[b, h, sorted(set(ids))].sum()
    return alpha.float()


def sparq_decode_step(query, key, value, channel_idx, top_k, *, scaling=None, mask_rows=None):
    """The mean-value-corrected step of this project on the int4 path (parity unpinned for the int4 part): ALL
    key rows (the decoded token's included) are quantized and scored, the top-k per KV head (group max, lower
    id on ties) are attended exactly, alpha from sparq_alpha, out = mean(V) + alpha * (exact - mean(V)) with the
    mean over all key rows in fp32 (EVAL:2646-2722 with the int4 logits). Returns dict(selected, alpha, vmean, out)."""
    B, Hq, D = query.shape
    Tk = key.shape[2]
    scaling = D ** -0.5 if scaling is None else scaling
    codes, _, kscale = quantize_pack(key, channel_idx)
    qcode, qscale = quantize_query(query, channel_idx)
    _, deq, gmax = score(qcode, qscale, codes, kscale)
    sel, _ = select(gmax, top_k)
    alpha = sparq_alpha(query, deq, sel, channel_idx, mask_rows)
    exact, _, _ = attend_fp32(query, key, value, sel, None, scaling, mask_rows)
    G = Hq // key.shape[1]
    vmean = value.float().mean(dim=2)                                   # [B,Hkv,D]
    vm = vmean.repeat_interleave(G, dim=1)[:, None]                     # [B,1,Hq,D]
    out = vm + alpha[:, None, :, None] * (exact - vm)
    return dict(selected=sel, alpha=alpha, vmean=vmean, out=out)


def sparq_fast_step(query_states, key_states, value_states, attention_mask, scaling, dim_count, candidate_fraction,
                    value_mean=None):
    """EVAL:2646-2722 (_sparq_fast_attention_output_for_query, torch branches, one query token) after the K/V
    repeat of the dispatcher (EVAL:6248-6251): approximate logits from the dim_count channels with the largest
    |q| per head, softmax over all keys, exact attention over the top ceil(fraction * keys) of them, blended
    with the mean of V by the approximate mass they carry. query [B,H,1,D] -> [B,1,H,D]."""
    if key_states.shape[1] != query_states.shape[1]:
        rep = query_states.shape[1] // key_states.shape[1]
        key_states = key_states.repeat_interleave(rep, dim=1)
        value_states = value_states.repeat_interleave(rep, dim=1)
    B, H, _, D = query_states.shape
    key_count = key_states.shape[-2]
    d_s = min(max(1, dim_count), D)
    cc = min(key_count, max(1, math.ceil(candidate_fraction * key_count)))
    q = query_states[:, :, 0:1, :]
    abs_q = q.float().abs()
    abs_q_hat, dim_indices = torch.topk(abs_q, k=d_s, dim=-1, largest=True, sorted=False)
    q_sel = torch.gather(q.float(), -1, dim_indices)
    k_sel = torch.gather(key_states.float(), -1, dim_indices.expand(B, H, key_count, d_s))
    approx = torch.matmul(q_sel, k_sel.transpose(2, 3))
    divscale = torch.sqrt(torch.tensor(float(D)) * abs_q_hat.sum(-1, keepdim=True).clamp_min(1.0e-6)
                          / abs_q.sum(-1, keepdim=True).clamp_min(1.0e-6))
    approx = approx / divscale
    mask_row = None
    if attention_mask is not None:
        mask_row = attention_mask[:, :, 0:1, :key_count]
        if mask_row.shape[1] == 1 and H != 1:
            mask_row = mask_row.expand(-1, H, -1, -1)
        approx = approx + mask_row
    w = F.softmax(approx, dim=-1, dtype=torch.float32)
    mass, top = torch.topk(w, k=cc, dim=-1, largest=True, sorted=False)
    gi = top[..., None].expand(B, H, 1, cc, D).squeeze(2)
    sk, sv = torch.gather(key_states, 2, gi), torch.gather(value_states, 2, gi)
    exact_scores = torch.matmul(q, sk.transpose(2, 3)) * scaling
    if mask_row is not None:
        exact_scores = exact_scores + torch.gather(mask_row, -1, top)
    exact = torch.matmul(F.softmax(exact_scores, dim=-1, dtype=torch.float32).to(q.dtype), sv)
    if value_mean is None:
        value_mean = value_states.float().mean(dim=2, keepdim=True).to(value_states.dtype)
    alpha = mass.sum(-1, keepdim=True).to(q.dtype)
    return torch.lerp(value_mean, exact, alpha).transpose(1, 2).contiguous()


def quantize_query_tokens(query: torch.Tensor, channel_idx: torch.Tensor):
    """query bf16 [B,Hq,Tq,D] -> per-token qcode int8 [B,Hq,Tq,C], qscale fp32 [B,Hq,Tq]."""
    B, Hq, Tq, D = query.shape
    qc, qs = quantize_query(query.permute(0, 2, 1, 3).reshape(B * Tq, Hq, D), channel_idx)
    C = qc.shape[-1]
    return qc.view(B, Tq, Hq, C).permute(0, 2, 1, 3).contiguous(), qs.view(B, Tq, Hq).permute(0, 2, 1).contiguous()


def prefill_block_scores(qcode: torch.Tensor, qscale: torch.Tensor, codes: torch.Tensor, kscale: torch.Tensor,
                         block: int = 64):
    """blk[b,g,i,j] = max over the G heads of g and the tokens of block j of
    (float(acc) * kscale[b,g,t]) * qscale[b,h,i]; the last block may be short; -0 -> +0.
    Every query sees every key (no causal term inside the chunk)."""
    B, Hq, Tq, C = qcode.shape
    Hkv, Tk = codes.shape[1], codes.shape[2]
    G = Hq // Hkv
    nblk = (Tk + block - 1) // block
    out = torch.empty((B, Hkv, Tq, nblk), dtype=torch.float32)
    cf = codes.to(torch.float64)
    for b in range(B):
        for g in range(Hkv):
            qf = qcode[b, g * G:(g + 1) * G].to(torch.float64)                       # [G,Tq,C]
            acc = torch.einsum("hic,tc->hit", qf, cf[b, g]).round().to(torch.float32)  # exact small integers
            deq = (acc * kscale[b, g][None, None, :]) * qscale[b, g * G:(g + 1) * G][:, :, None]
            gm = deq.amax(0)                                                          # [Tq,Tk]
            pad = nblk * block - Tk
            if pad:
                gm = torch.cat((gm, torch.full((Tq, pad), float("-inf"))), dim=1)
            out[b, g] = gm.view(Tq, nblk, block).amax(-1) + 0.0
    return out


def merge_shards(cand_scores: torch.Tensor, cand_idx: torch.Tensor, k: int):
    """Global top-k from per-shard candidate lists [N,R,kk] (scores, global ids): concatenated
    along the shard axis and selected with the same (score desc, id asc) rule."""
    N, R, kk = cand_scores.shape
    s = cand_scores.permute(1, 0, 2).reshape(R, N * kk)
    i = cand_idx.permute(1, 0, 2).reshape(R, N * kk)
    return select(s, k, index=i)


def lse_merge(partials: torch.Tensor) -> torch.Tensor:
    """partials fp32 [N,B,Hq,D+2] = (o scaled to m, m, l) -> fp32 [B,1,Hq,D]."""
    o, m, l = partials[..., :-2], partials[..., -2], partials[..., -1]
    m = torch.where(l > 0, m, torch.full_like(m, float("-inf")))
    M = m.amax(0)
    Mu = torch.where(torch.isinf(M), torch.zeros_like(M), M)
    w = torch.where(l > 0, torch.exp(m - Mu[None]), torch.zeros_like(m))
    L = (l * w).sum(0)
    O = (o * w[..., None]).sum(0)
    out = torch.where(L[..., None] > 0, O / L.clamp_min(1e-30)[..., None], torch.zeros_like(O))
    return out[:, None, :, :]


def rerank_union(query, key, lists, history_count, keep, scaling, counts=None, mask_rows=None, force_sink=0,
                 force_recent=0):
    """List form of the reference's exact rerank (the candidate union of EVAL:4186-4214, the exact scores of
    QCK:160-216 / EVAL:4287-4295, the top-keep of EVAL:4297-4302) with the tie rule of this project:
    per list row, the union of the ids in ``lists`` (int [B,Hi,n_i], entries outside [0, history_count)
    ignored, optional per-row counts) and of the forced ranges; score = max over the query heads sharing the
    list of fp32 q.k, times scaling, plus mask; the min(keep, |union|) best by (score desc, id asc), returned
    ascending and -1 padded with their count. query [B,Hq,D], key [B,Hkv,>=history_count,D]."""
    B, Hq, D = query.shape
    Hkv = key.shape[1]
    Hi = lists[0].shape[1]
    GG, G = Hq // Hi, Hq // Hkv
    out = torch.full((B, Hi, keep), -1, dtype=torch.int64)
    cnt = torch.zeros((B, Hi), dtype=torch.int64)
    qf, kf = query.float(), key.float()
    for b in range(B):
        for hi in range(Hi):
            ids = set()
            for li, l in enumerate(lists):
                if l is None:
                    continue
                n = l.shape[2] if counts is None or counts[li] is None else int(counts[li][b, hi])
                ids.update(int(x) for x in l[b, hi, :n].tolist() if 0 <= int(x) < history_count)
            ids.update(range(min(force_sink, history_count)))
            ids.update(range(max(0, history_count - force_recent), history_count) if force_recent > 0 else ())
            if not ids:
                continue
            u = torch.tensor(sorted(ids), dtype=torch.long)
            heads = range(hi * GG, (hi + 1) * GG)
            kv = (hi * GG) // G
            sc = torch.stack([kf[b, kv, u] @ qf[b, h] for h in heads]).amax(0) * scaling
            if mask_rows is not None:
                sc = sc + mask_rows[b, u].float()
            order = torch.sort(sc + 0.0, descending=True, stable=True).indices[:keep]          # u ascending: ties -> lower id
            win = torch.sort(u[order]).values
            out[b, hi, :win.numel()] = win
            cnt[b, hi] = win.numel()
    return out, cnt


def expand_final(ids, history_count, counts=None, force_sink=0, force_recent=0, block_size=1):
    """ids (any int tensor [..., n], out-of-range ignored) plus the protected ranges (EVAL:4306-4311), widened to
    aligned blocks (EVAL:2914-2922): list of sorted python lists, one per leading row."""
    flat = ids.reshape(-1, ids.shape[-1])
    res = []
    for r in range(flat.shape[0]):
        n = flat.shape[1] if counts is None else int(counts.reshape(-1)[r])
        keep = torch.zeros(history_count, dtype=torch.bool)
        good = [int(x) for x in flat[r, :n].tolist() if 0 <= int(x) < history_count]
        keep[good] = True
        if force_sink > 0:
            keep[:min(force_sink, history_count)] = True
        if force_recent > 0:
            keep[max(0, history_count - force_recent):] = True
        if block_size > 1:
            pad = (-history_count) % block_size
            padded = F.pad(keep, (0, pad), value=False)
            blk = padded.view(-1, block_size).any(dim=-1, keepdim=True).expand(-1, block_size).reshape(-1)
            keep = blk[:history_count]
        res.append(torch.nonzero(keep).flatten().tolist())
    return res


# ==========================================================================================
# (1) restatements of reference code (pinned by tests/golden/reference_*.npz)
# ==========================================================================================

def final_indices_from_selected(selected: torch.Tensor, selected_valid: torch.Tensor, history_count: int,
                                key_count: int, always_keep_self: bool, protect_sink: int, protect_recent: int,
                                append_protected: bool = False):
    """EVAL:2938-2982 (_qabs_final_indices_from_selected) and, with append_protected,
    EVAL:2985-3022 (_qabs_final_indices_append_protected): selected || sink || recent || self.
    The reference reads the protect counts from module globals; here they are arguments."""
    lead = selected.shape[:-1]
    sel = selected.long()
    valid = selected_valid.clone()
    sink_end = min(protect_sink, history_count) if protect_sink > 0 else 0
    idx_parts, valid_parts = [sel], None
    recent_from = None
    if append_protected:
        if protect_recent > 0:
            rs = max(max(0, history_count - protect_recent), sink_end)
            if rs < history_count:
                recent_from = rs
    else:
        recent_start = history_count
        if protect_recent > 0:
            recent_start = max(0, history_count - protect_recent)
            valid &= ~((sel >= recent_start) & (sel < history_count))
        if sink_end > 0:
            valid &= sel >= sink_end
        if protect_recent > 0 and recent_start < history_count:
            rs = max(recent_start, sink_end)
            if rs < history_count:
                recent_from = rs
    valid_parts = [valid]
    if sink_end > 0:
        part = torch.arange(sink_end, dtype=torch.long).expand(*lead, -1)
        idx_parts.append(part)
        valid_parts.append(torch.ones_like(part, dtype=torch.bool))
    if recent_from is not None:
        part = torch.arange(recent_from, history_count, dtype=torch.long).expand(*lead, -1)
        idx_parts.append(part)
        valid_parts.append(torch.ones_like(part, dtype=torch.bool))
    if always_keep_self:
        part = torch.full((*lead, 1), key_count - 1, dtype=torch.long)
        idx_parts.append(part)
        valid_parts.append(torch.ones_like(part, dtype=torch.bool))
    return torch.cat(idx_parts, dim=-1), torch.cat(valid_parts, dim=-1)


def attention_from_final_indices(query_states, key_states, value_states, attention_mask, final_indices, final_valid,
                                 scaling):
    """EVAL:4612-4647 (_qabs_attention_from_final_indices), torch branch: K/V already repeated to
    the query heads, bf16 matmul, fp32 softmax cast to the input dtype, weighted sum in the input
    dtype. query [B,H,1,D]; returns [B,1,H,D]."""
    _, head_count, _, head_dim = query_states.shape
    key_count = key_states.shape[-2]
    gather = final_indices[:, :, :, None].expand(-1, -1, -1, head_dim)
    sel_k = torch.gather(key_states, 2, gather)
    sel_v = torch.gather(value_states, 2, gather)
    scores = torch.matmul(query_states[:, :, 0:1, :], sel_k.transpose(2, 3)).squeeze(2) * scaling
    if attention_mask is not None:
        mask_row = attention_mask[:, :, 0, :key_count]
        if mask_row.shape[1] == 1 and head_count != 1:
            mask_row = mask_row.expand(-1, head_count, -1)
        scores = scores + torch.gather(mask_row, -1, final_indices)
    scores = scores.masked_fill(~final_valid, torch.finfo(scores.dtype).min)
    weights = F.softmax(scores, dim=-1, dtype=torch.float32).to(query_states.dtype)
    out = torch.sum(weights[:, :, :, None] * sel_v, dim=2)
    return out[:, None, :, :].contiguous()


def qabs_partial_scores(q_raw: torch.Tensor, k_history: torch.Tensor, dim_count: int):
    """EVAL:4428 + EVAL:4443-4446: per (b, head) the dim_count channels with the largest |q|, then
    fp32 sum over those channels of q * K. q_raw [B,H,D], k_history [B,H,T,D]. Returns
    (scores fp32 [B,H,T], channel indices [B,H,dim_count])."""
    T = k_history.shape[2]
    qdim = torch.topk(q_raw.float().abs(), k=dim_count, dim=-1, largest=True).indices
    q_sel = torch.gather(q_raw.float(), -1, qdim)
    k_idx = qdim[:, :, None, :].expand(-1, -1, T, -1)
    k_sel = torch.gather(k_history.float(), -1, k_idx)
    return (k_sel * q_sel[:, :, None, :]).sum(-1), qdim


def candidate_count(candidate_fraction: float, history_count: int) -> int:
    """EVAL:4423: min(T, max(1, ceil(fraction * T)))."""
    return min(history_count, max(1, math.ceil(candidate_fraction * history_count)))


def qabs_candidate_attention(query_states, key_states, value_states, attention_mask, scaling, dim_count,
                             candidate_fraction, always_keep_self=True, protect_sink=0, protect_recent=0,
                             append_protected=False):
    """EVAL:4400-4502 (_qabs_candidate_attention_forward, torch branches) preceded by the K/V
    repeat of the dispatcher (EVAL:6248-6251): the reference's own CPU path for one decode step.
    ``append_protected`` is the ``...appendattn`` form of the mode (EVAL:4451-4458).
    query [B,Hq,1,D], key/value [B,Hkv,Tk,D] -> [B,1,Hq,D]."""
    if key_states.shape[1] != query_states.shape[1]:
        rep = query_states.shape[1] // key_states.shape[1]
        key_states = key_states.repeat_interleave(rep, dim=1)
        value_states = value_states.repeat_interleave(rep, dim=1)
    head_dim = query_states.shape[-1]
    key_count = key_states.shape[-2]
    if key_count <= 1:
        return value_states[:, :, -1:, :].transpose(1, 2).contiguous()
    history = key_count - 1
    d_s = min(max(1, dim_count), head_dim)
    requested = candidate_count(candidate_fraction, history)
    q_raw = query_states[:, :, 0, :]
    partial, _ = qabs_partial_scores(q_raw, key_states[:, :, :history, :], d_s)
    _, cand = torch.topk(partial, k=requested, dim=-1, largest=True)
    fidx, fvalid = final_indices_from_selected(cand, torch.ones_like(cand, dtype=torch.bool), history, key_count,
                                               always_keep_self, protect_sink, protect_recent, append_protected)
    return attention_from_final_indices(query_states, key_states, value_states, attention_mask, fidx, fvalid, scaling)


def indices_from_keep_mask(keep: torch.Tensor):
    """EVAL:2896-2911 (_indices_from_keep_mask): bool [B,H,T] -> padded indices (DESCENDING positions, as the
    reference's topk over positions yields) and their validity."""
    counts = keep.sum(dim=-1)
    max_selected = int(counts.max().item()) if counts.numel() else 0
    if max_selected <= 0:
        empty = torch.zeros((*keep.shape[:-1], 0), dtype=torch.long)
        return empty, torch.zeros_like(empty, dtype=torch.bool)
    positions = torch.arange(keep.shape[-1], dtype=torch.long).view(1, 1, -1).expand_as(keep)
    masked = torch.where(keep, positions, torch.full_like(positions, -1))
    indices = torch.topk(masked, k=max_selected, dim=-1, largest=True).values
    return indices.clamp_min(0), indices >= 0


def expand_keep_to_aligned_blocks(keep: torch.Tensor, block_size: Optional[int]) -> torch.Tensor:
    """EVAL:2914-2922 (_expand_history_keep_to_aligned_blocks)."""
    if block_size is None or block_size <= 1 or keep.shape[-1] <= 1:
        return keep
    history_count = int(keep.shape[-1])
    pad = (-history_count) % int(block_size)
    padded = F.pad(keep, (0, pad), value=False) if pad else keep
    blk = padded.view(*padded.shape[:-1], -1, int(block_size)).any(dim=-1, keepdim=True)
    return blk.expand(*blk.shape[:-1], int(block_size)).reshape(*padded.shape[:-1], padded.shape[-1])[..., :history_count]


def _pad_mask(mask: Optional[torch.Tensor], history_count: int) -> Optional[torch.Tensor]:
    """EVAL:1603-1624 (ReuseCandidateState.previous_layer_masks): cut or zero-pad a stored mask to the new length."""
    if mask is None:
        return None
    if mask.shape[-1] > history_count:
        mask = mask[..., :history_count]
    if mask.shape[-1] < history_count:
        mask = F.pad(mask, (0, history_count - mask.shape[-1]), value=False)
    return mask


def qabs_reuse_step(query_states, key_states, value_states, scaling, dim_count, candidate_fraction, top_fraction,
                    prev_candidate=None, prev_final=None, protect_sink=0, protect_recent=0, always_keep_self=True,
                    use_prev_candidate=True, use_prev_final=True, block_size=None):
    """EVAL:3991-4397 (_qabs_reuse_fast_attention_forward, torch branches, 'qabs{D}cand{C}reuse[2set|final][blkN]')
    preceded by the K/V repeat of the dispatcher (EVAL:6248-6251): per head, current candidates = partial score
    >= the requested-th largest (EVAL:3987-3989), union with the previous step's candidate and final masks
    (EVAL:4186-4196), exact q.k on the union (EVAL:4287-4295), top ceil(top_fraction * T) (EVAL:4297-4302),
    protected ranges forced in (EVAL:4306-4311), optional block widening (EVAL:4314-4316), attention over the
    final list (EVAL:4364-4396). Returns (out [B,1,Hq,D], current candidate mask, final mask), the two masks being
    what the reference stores for the next step (EVAL:4352-4362)."""
    if key_states.shape[1] != query_states.shape[1]:
        rep = query_states.shape[1] // key_states.shape[1]
        key_states = key_states.repeat_interleave(rep, dim=1)
        value_states = value_states.repeat_interleave(rep, dim=1)
    B, H, _, D = query_states.shape
    key_count = key_states.shape[-2]
    history = key_count - 1
    q_raw = query_states[:, :, 0, :]
    k_history = key_states[:, :, :history, :]
    d_s = min(max(1, dim_count), D)
    requested = candidate_count(candidate_fraction, history)
    partial, _ = qabs_partial_scores(q_raw, k_history, d_s)
    threshold = torch.topk(partial, k=requested, dim=-1, largest=True).values[:, :, -1:]
    current = partial >= threshold
    union = current.clone()
    pc, pf = _pad_mask(prev_candidate, history), _pad_mask(prev_final, history)
    if pc is not None and use_prev_candidate:
        union |= pc
    if pf is not None and use_prev_final:
        union |= pf
    cand_idx, cand_valid = indices_from_keep_mask(union)
    gather = cand_idx[:, :, :, None].expand(-1, -1, -1, D)
    cand_keys = torch.gather(k_history, 2, gather)
    cand_scores = torch.matmul(query_states[:, :, 0:1, :], cand_keys.transpose(2, 3)).squeeze(2) * scaling
    cand_scores = cand_scores.masked_fill(~cand_valid, torch.finfo(cand_scores.dtype).min)
    keep_count = min(min(history, max(1, math.ceil(top_fraction * history))), cand_scores.shape[-1])
    _, pos = torch.topk(cand_scores, k=keep_count, dim=-1, largest=True)
    sel_idx = torch.gather(cand_idx, -1, pos)
    sel_valid = torch.gather(cand_valid, -1, pos)
    final = torch.zeros_like(current)
    final.scatter_(-1, sel_idx, sel_valid)
    if protect_sink > 0:
        final[:, :, :min(protect_sink, history)] = True
    if protect_recent > 0:
        final[:, :, max(0, history - protect_recent):history] = True
    if block_size is not None:
        final = expand_keep_to_aligned_blocks(final, block_size)
        sel_idx, sel_valid = indices_from_keep_mask(final)
    fidx, fvalid = final_indices_from_selected(sel_idx, sel_valid, history, key_count, always_keep_self, protect_sink,
                                               protect_recent)
    out = attention_from_final_indices(query_states, key_states, value_states, None, fidx, fvalid, scaling)
    return out, current, final


def qabs_top2_step(query_states, key_states, value_states, attention_mask, scaling, dim_count, candidate_fraction,
                   top_fraction, protect_sink=0, protect_recent=0, always_keep_self=True):
    """EVAL:4650-4766 (_qabs_candidate_top2_attention_forward, plain 'qabs{D}cand{C}top2attn') after the K/V repeat
    of the dispatcher: top candidates by partial score, exact q.k (+ mask) on them, the best
    min(candidates, ceil(top_fraction * T)) per head, attention over the final list. Returns (out, selected ids)."""
    if key_states.shape[1] != query_states.shape[1]:
        rep = query_states.shape[1] // key_states.shape[1]
        key_states = key_states.repeat_interleave(rep, dim=1)
        value_states = value_states.repeat_interleave(rep, dim=1)
    B, H, _, D = query_states.shape
    key_count = key_states.shape[-2]
    history = key_count - 1
    cc = candidate_count(candidate_fraction, history)
    final_per_head = min(cc, max(1, math.ceil(top_fraction * history)))
    q_raw = query_states[:, :, 0, :]
    k_history = key_states[:, :, :history, :]
    partial, _ = qabs_partial_scores(q_raw, k_history, min(max(1, dim_count), D))
    _, cand = torch.topk(partial, k=cc, dim=-1, largest=True)
    cand_keys = torch.gather(k_history, 2, cand[:, :, :, None].expand(-1, -1, -1, D))
    scores = torch.matmul(query_states[:, :, 0:1, :], cand_keys.transpose(2, 3)).squeeze(2) * scaling
    if attention_mask is not None:
        mask_row = attention_mask[:, :, 0, :history]
        if mask_row.shape[1] == 1 and H != 1:
            mask_row = mask_row.expand(-1, H, -1)
        scores = scores + torch.gather(mask_row, -1, cand)
    _, pos = torch.topk(scores, k=final_per_head, dim=-1, largest=True)
    sel = torch.gather(cand, -1, pos)
    fidx, fvalid = final_indices_from_selected(sel, torch.ones_like(sel, dtype=torch.bool), history, key_count,
                                               always_keep_self, protect_sink, protect_recent)
    out = attention_from_final_indices(query_states, key_states, value_states, attention_mask, fidx, fvalid, scaling)
    return out, sel


def qabs_candidate_full_scores(query, key_history, current, previous_candidate, previous_final, protect_sink,
                               protect_recent, scaling):
    """QCK:160-216 (qabs_candidate_full_scores_kernel) restated: fp32 q.k over all channels times scaling
    on current | previous_candidate | previous_final | [0, sink) | [T - recent, T); -inf elsewhere.
    query [B,H,D], key_history [B,H,T,D], masks bool [B,H,T]."""
    T = key_history.shape[2]
    sel = current.clone()
    if previous_candidate is not None:
        sel |= previous_candidate
    if previous_final is not None:
        sel |= previous_final
    if protect_sink > 0:
        sel[..., :protect_sink] = True
    if protect_recent > 0:
        sel[..., max(0, T - protect_recent):] = True
    scores = torch.einsum("bhd,bhtd->bht", query.float(), key_history.float()) * scaling
    return torch.where(sel, scores, torch.full_like(scores, float("-inf")))
