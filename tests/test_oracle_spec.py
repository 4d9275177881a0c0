"""Checks the int4 part of the oracle (this project's own specification — parity unpinned by the
reference) against slow, obviously-correct Python/numpy restatements on small cases."""
import numpy as np
import torch

from oracle import oracle


def _inputs(seed=0, B=2, Hq=4, Hkv=2, T=50, D=128, C=32):
    g = torch.Generator().manual_seed(seed)
    key = (torch.randn(B, Hkv, T, D, generator=g) * torch.exp(torch.randn(1, Hkv, 1, D, generator=g))).to(torch.bfloat16)
    val = torch.randn(B, Hkv, T, D, generator=g).to(torch.bfloat16)
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16)
    return q, key, val, oracle.choose_channels(key, C)


def test_choose_channels_ties_go_to_lower_index():
    key = torch.zeros(1, 1, 4, 8, dtype=torch.bfloat16)
    key[..., 5] = 2.0
    key[..., 1] = 1.0
    key[..., 6] = 1.0
    key[..., 3] = 1.0
    assert oracle.choose_channels(key, 3).tolist() == [[1, 3, 5]]


def test_quantize_matches_scalar_loop():
    q, key, _, ch = _inputs(T=9)
    codes, packed, scale = oracle.quantize_pack(key, ch)
    kf = key.float().numpy()
    for b in range(key.shape[0]):
        for h in range(key.shape[1]):
            for t in range(key.shape[2]):
                x = kf[b, h, t, ch[h].numpy()]
                s = np.float32(max(np.abs(x).max(), np.float32(2.0 ** -24))) / np.float32(7.0)
                assert np.float32(s) == scale[b, h, t].item()
                c = np.clip(np.rint(x.astype(np.float32) / np.float32(s)), -7, 7).astype(np.int8)
                assert (c == codes[b, h, t].numpy()).all()
                for j in range(len(c) // 2):
                    assert packed[b, h, t, j].item() == ((int(c[2 * j]) & 0xF) | ((int(c[2 * j + 1]) & 0xF) << 4))
    assert torch.equal(oracle.unpack(packed), codes)
    assert codes.abs().max() <= 7


def test_zero_row_quantizes_to_zero_codes():
    key = torch.zeros(1, 1, 3, 128, dtype=torch.bfloat16)
    ch = torch.arange(32, dtype=torch.int32)[None]
    codes, packed, scale = oracle.quantize_pack(key, ch)
    assert (codes == 0).all() and (packed == 0).all()
    assert scale.flatten().tolist() == [2.0 ** -24 / 7.0] * 3 or torch.allclose(scale, torch.full_like(scale, 2.0 ** -24 / 7.0))


def test_score_matches_integer_loop_and_group_max():
    q, key, _, ch = _inputs(T=17)
    codes, _, scale = oracle.quantize_pack(key, ch)
    qcode, qscale = oracle.quantize_query(q, ch)
    acc, deq, gmax = oracle.score(qcode, qscale, codes, scale)
    B, Hq = q.shape[:2]
    G = Hq // key.shape[1]
    for b in range(B):
        for h in range(Hq):
            want = (codes[b, h // G].to(torch.int32) * qcode[b, h].to(torch.int32)[None]).sum(-1)
            assert torch.equal(acc[b, h], want)
            d = (want.float() * scale[b, h // G]) * qscale[b, h]
            assert torch.equal(deq[b, h], d)
    assert torch.equal(gmax, deq.view(B, key.shape[1], G, -1).amax(2) + 0.0)


def test_select_is_score_desc_then_index_asc():
    s = torch.tensor([[1.0, 3.0, 3.0, -0.0, 0.0, 3.0, 2.0]])
    idx, val = oracle.select(s, 5)
    assert idx.tolist() == [[1, 2, 5, 6, 0]]
    idx, _ = oracle.select(s, 100)
    assert idx.tolist() == [[1, 2, 5, 6, 0, 3, 4]]          # -0 and +0 tie, lower index first
    payload = torch.tensor([[70, 60, 50, 40, 30, 20, 10]])
    idx, _ = oracle.select(s, 3, index=payload)
    assert idx.tolist() == [[20, 50, 60]]


def test_shard_merge_equals_global_select():
    torch.manual_seed(3)
    R, T, N, k = 3, 64, 4, 8
    s = torch.randint(-3, 4, (R, T)).float()                  # many ties
    want, _ = oracle.select(s, k)
    per = T // N
    cs, ci = [], []
    for r in range(N):
        i, v = oracle.select(s[:, r * per:(r + 1) * per], k)
        cs.append(v)
        ci.append(i + r * per)
    got, _ = oracle.merge_shards(torch.stack(cs), torch.stack(ci), k)
    assert torch.equal(got, want)


def test_lse_merge_equals_single_pass():
    q, key, val, ch = _inputs(T=40)
    B, Hq, D = q.shape
    idx = torch.arange(40)[None, None].expand(B, key.shape[1], -1)
    full, _, _ = oracle.attend_fp32(q, key, val, idx, None, D ** -0.5)
    parts = []
    for lo, hi in ((0, 13), (13, 14), (14, 40)):
        o, m, l = oracle.attend_fp32(q, key, val, idx[..., lo:hi], None, D ** -0.5)
        parts.append(torch.cat((o[:, 0] * l[..., None], m[..., None], l[..., None]), dim=-1))
    got = oracle.lse_merge(torch.stack(parts))
    torch.testing.assert_close(got, full, rtol=1e-5, atol=1e-6)


def test_decode_step_runs_and_selects_k_plus_self():
    q, key, val, ch = _inputs(T=65)
    r = oracle.decode_step(q, key, val, ch, 16)
    assert r["selected"].shape == (2, 2, 16)
    assert r["final_indices"].shape == (2, 2, 17)
    assert (r["final_indices"][..., -1] == 64).all()
    assert r["out"].shape == (2, 1, 4, 128)
