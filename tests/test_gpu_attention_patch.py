"""The drop-in attention function on the GPU: against the oracle step for one layer call, and
through a small random-init HF Qwen3 model where selecting every token must reproduce dense
attention (prefill under 'baseline', decode under the sparse mode, as the reference runs it)."""
import pytest
import torch

from kv_cache_b200 import attention_patch as ap
from oracle import oracle
from tests.gpu_util import cpu, make_case

pytestmark = pytest.mark.gpu


class _Layer(torch.nn.Module):
    def __init__(self, idx):
        super().__init__()
        self.layer_idx = idx
        self.scaling = 128 ** -0.5


def test_forward_matches_oracle_and_keeps_the_side_cache_growing(cuda_device):
    T = 700
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T + 1, channels=32)
    layer = _Layer(3)
    with ap.attention_mode("qabs32cand12p5attn", 0.02, 3, True, 4, 4, None) as state:
        out, weights = ap.sparse_eager_attention_forward(layer, q[:, :, None, :], key[:, :, :T + 1], value[:, :, :T + 1], None)
        assert weights is None and out.shape == (2, 1, 8, 128)
        sc = state.layers[3]
        assert sc.count == T + 1
        ch = sc.channel_idx
        want = oracle.decode_step(*cpu(q, key[:, :, :T + 1], value[:, :, :T + 1], ch), ap.candidate_count(0.125, T),
                                  protect_sink=4, protect_recent=4)
        torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
        # next decode step: one more row, the side cache is extended, not rebuilt
        packed_before = sc.packed
        out2, _ = ap.sparse_eager_attention_forward(layer, q[:, :, None, :], key, value, None)
        assert state.layers[3].packed is packed_before and state.layers[3].count == T + 2
        want2 = oracle.decode_step(*cpu(q, key, value, ch), ap.candidate_count(0.125, T + 1), protect_sink=4, protect_recent=4)
        torch.testing.assert_close(out2.float().cpu(), want2["out"], rtol=2e-2, atol=1e-2)


def test_tiny_qwen3_decode_equals_dense_when_everything_is_selected(cuda_device):
    transformers = pytest.importorskip("transformers")
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      rope_theta=1e6, attn_implementation="eager")
    model = Qwen3ForCausalLM(cfg).to(cuda_device, torch.bfloat16).eval()
    ap.install_qwen3_attention_patch()
    try:
        ids = torch.randint(0, 512, (2, 300), device=cuda_device)
        nxt = torch.randint(0, 512, (2, 1), device=cuda_device)
        with torch.inference_mode():
            with ap.attention_mode("baseline"):
                pre = model(input_ids=ids, use_cache=True)
                import copy
                dense = model(input_ids=nxt, past_key_values=copy.deepcopy(pre.past_key_values), use_cache=True)
            with ap.attention_mode("qabs64cand100attn", 0.02, 3, True, 0, 0, None) as state:
                sparse = model(input_ids=nxt, past_key_values=pre.past_key_values, use_cache=True)
                assert sorted(state.layers) == [0, 1] and state.layers[0].count == 301
        torch.testing.assert_close(sparse.logits.float(), dense.logits.float(), rtol=5e-2, atol=5e-2)
    finally:
        ap.uninstall_qwen3_attention_patch()


def test_qwen3_0p6b_shaped_model_decodes_through_all_28_layers(cuda_device):
    """The layer stack of Qwen3-0.6B (28 layers, 16 query / 8 KV heads of 128, hidden 1024; small vocabulary,
    random weights): prefill under 'baseline', then decode steps under the sparse mode. With every token
    selected the logits must match dense attention; at 6.25 % the step must run, stay finite, and extend
    the int4 side cache of every layer by one row per step."""
    pytest.importorskip("transformers")
    from transformers import Qwen3Config, Qwen3ForCausalLM
    import copy

    torch.manual_seed(1)
    cfg = Qwen3Config(vocab_size=1024, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                      num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                      rope_theta=1e6, rms_norm_eps=1e-6, attn_implementation="eager")
    model = Qwen3ForCausalLM(cfg).to(cuda_device, torch.bfloat16).eval()
    ap.install_qwen3_attention_patch()
    try:
        ids = torch.randint(0, 1024, (2, 1536), device=cuda_device)
        nxt = torch.randint(0, 1024, (2, 1), device=cuda_device)
        with torch.inference_mode():
            with ap.attention_mode("baseline"):
                pre = model(input_ids=ids, use_cache=True)
                dense = model(input_ids=nxt, past_key_values=copy.deepcopy(pre.past_key_values), use_cache=True)
            with ap.attention_mode("qabs32cand100attn", 0.02, 3, True, 0, 0, None) as state:
                full = model(input_ids=nxt, past_key_values=copy.deepcopy(pre.past_key_values), use_cache=True)
                assert sorted(state.layers) == list(range(28))
            torch.testing.assert_close(full.logits.float(), dense.logits.float(), rtol=5e-2, atol=5e-2)
            with ap.attention_mode("qabs32cand6p25attn", 0.02, 3, True, 4, 16, None) as state:
                past = pre.past_key_values
                for step in range(3):
                    out = model(input_ids=nxt, past_key_values=past, use_cache=True)
                    past = out.past_key_values
                    assert torch.isfinite(out.logits.float()).all()
                    assert all(state.layers[l].count == 1537 + step for l in range(28))
            # a sparse step stays close to the dense one on this random model (most attention mass is kept)
            assert (out.logits.float() - dense.logits.float()).abs().mean() < 1.0
    finally:
        ap.uninstall_qwen3_attention_patch()
