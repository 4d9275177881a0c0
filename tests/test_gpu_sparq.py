"""SparQ-style mean-value correction on the int4 path: alpha (the softmax mass of the selected tokens under the
approximate logits), the blended attention output, and the `sparqfast{C}cand{P}` mode with its running mean of
V over consecutive steps, against the oracle (whose reference-side restatement is pinned by the golden vectors)."""
import math

import pytest
import torch

from kv_cache_b200 import attention_patch as ap
from kv_cache_b200 import ops
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2


@pytest.mark.parametrize("G,C,T", [(4, 64, 20000), (1, 32, 700), (8, 32, 9000), (2, 128, 3000)])
def test_alpha_matches_oracle(cuda_device, G, C, T):
    Hkv = 2
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=Hkv * G, kv_heads=Hkv, context=T, channels=C, seed=G + 50)
    ch = ops.choose_channels(key[:, :, :T], C)
    packed, scale = ops.quantize(key[:, :, :T], ch)
    codes, _, kscale = oracle.quantize_pack(key[:, :, :T].cpu(), ch.cpu())
    qcode, qscale = oracle.quantize_query(q.cpu(), ch.cpu())
    _, deq, gmax = oracle.score(qcode, qscale, codes, kscale)
    sel, _ = oracle.select(gmax, max(1, T // 16))
    mask = torch.zeros((2, 1, 1, T), dtype=torch.bfloat16, device=cuda_device)
    mask[0, 0, 0, : T // 3] = -30.0
    for m in (None, mask):
        got = ops.sparq_alpha(q, packed, scale, ch, T, sel.to(cuda_device), attention_mask=m)
        want = oracle.sparq_alpha(q.cpu(), deq, sel, ch.cpu(), None if m is None else m[:, 0, 0].float().cpu())
        torch.testing.assert_close(got.cpu(), want, rtol=2e-3, atol=2e-4)
        assert float(got.min()) >= 0.0 and float(got.max()) <= 1.0
    # every token selected: the whole mass
    everything = torch.arange(T, dtype=torch.int32, device=cuda_device).expand(2, Hkv, T).contiguous()
    full = ops.sparq_alpha(q, packed, scale, ch, T, everything)
    torch.testing.assert_close(full.cpu(), torch.ones(2, Hkv * G), rtol=1e-3, atol=1e-3)
    # a per-row count cuts the list
    cnt = torch.tensor([[0, 5], [T // 16, 1]], dtype=torch.int32, device=cuda_device)
    part = ops.sparq_alpha(q, packed, scale, ch, T, sel.to(cuda_device), selected_count=cnt)
    sel_cut = sel.clone()
    for b in range(2):
        for g in range(Hkv):
            sel_cut[b, g, int(cnt[b, g]):] = -1
    torch.testing.assert_close(part.cpu(), oracle.sparq_alpha(q.cpu(), deq, sel_cut, ch.cpu()), rtol=2e-3, atol=2e-4)


def test_blend_is_the_lerp_of_mean_and_attention(cuda_device):
    T = 1500
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T, channels=32, seed=61)
    g = torch.Generator(device=cuda_device).manual_seed(3)
    sel = torch.randint(0, T, (2, 2, 100), generator=g, device=cuda_device, dtype=torch.int32)
    alpha = torch.rand(2, 8, generator=g, device=cuda_device)
    vmean = value[:, :, :T].float().mean(dim=2)
    out = ops.attend_selected_blend(q, key[:, :, :T], value[:, :, :T], sel, T, alpha, vmean)
    exact, _, _ = oracle.attend_fp32(q.cpu(), key[:, :, :T].cpu(), value[:, :, :T].cpu(), sel.cpu(), None, 128 ** -0.5)
    vm = vmean.cpu().repeat_interleave(4, dim=1)[:, None]
    want = vm + alpha.cpu()[:, None, :, None] * (exact - vm)
    torch.testing.assert_close(out.float().cpu(), want, rtol=RTOL, atol=ATOL)
    zero = ops.attend_selected_blend(q, key[:, :, :T], value[:, :, :T], sel, T, torch.zeros_like(alpha), vmean)
    torch.testing.assert_close(zero.float().cpu(), vm.expand(2, 1, 8, 128).to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


class _Layer(torch.nn.Module):
    def __init__(self, idx):
        super().__init__()
        self.layer_idx = idx
        self.scaling = 128 ** -0.5


def test_sparqfast_mode_over_consecutive_steps(cuda_device):
    T0 = 2500
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T0 + 2, channels=32, seed=67)
    state = ap.SparseDecodeState()
    for i in range(3):
        kc = T0 + 1 + i
        qi = (q.float() * (1.0 + 0.2 * i)).to(torch.bfloat16)
        with ap.attention_mode("sparqfast32cand6p25", 0.02, 3, True, 0, 0, None, sparse_state=state):
            out, _ = ap.sparse_eager_attention_forward(_Layer(4), qi[:, :, None, :], key[:, :, :kc], value[:, :, :kc], None)
        ch = state.layers[4].channel_idx
        want = oracle.sparq_decode_step(qi.cpu(), key[:, :, :kc].cpu(), value[:, :, :kc].cpu(), ch.cpu(),
                                        min(kc, max(1, math.ceil(0.0625 * kc))))
        rows, mean = state.value_means[4]
        assert rows == kc
        torch.testing.assert_close(mean.cpu(), want["vmean"], rtol=1e-4, atol=1e-5)      # incremental update == full mean
        torch.testing.assert_close(out.float().cpu(), want["out"], rtol=RTOL, atol=ATOL)
        assert state.layers[4].count == kc
    assert state.bulk_quantized_rows == T0
