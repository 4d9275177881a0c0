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
    with ap.attention_mode("qabs32cand12p5attn", 0.02, 3, True, 4, 4, None, sparse_state=ap.SparseDecodeState()) as state:
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
            with ap.attention_mode("qabs64cand100attn", 0.02, 3, True, 0, 0, None,
                                   sparse_state=ap.SparseDecodeState()) as state:
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
    ap.reset_sparse_state()
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


def test_one_with_block_per_token_quantizes_the_prefix_once(cuda_device):
    """The reference opens one `with attention_mode(...)` per decoded token (EVAL:7236): the int4 side cache
    must survive from block to block (same storage, one more row each), the prefix must go through the bulk
    quantizer exactly once, and every step must equal the oracle."""
    T = 900
    w, q, key, value = make_case(cuda_device, batch=2, q_heads=8, kv_heads=2, context=T + 3, channels=32, seed=12)
    layer = _Layer(5)
    ap.reset_sparse_state()
    state = ap.default_sparse_state()
    rows_before = state.bulk_quantized_rows
    args = ("qabs32cand12p5attn", 0.02, 3, True, 0, 0, None, None, None, None, None, None, None, None, None, None, None,
            None, None, True, False, False, False, None, "topk", 256, "", "", "")           # the call of EVAL:7236-7266
    packed = None
    for i in range(3):
        kc = T + 1 + i
        with ap.attention_mode(*args):
            out, _ = ap.sparse_eager_attention_forward(layer, q[:, :, None, :], key[:, :, :kc], value[:, :, :kc], None)
        sc = state.layers[5]
        if packed is None:
            packed = sc.packed
        assert sc.packed is packed and sc.count == kc
        want = oracle.decode_step(*cpu(q, key[:, :, :kc], value[:, :, :kc], sc.channel_idx), ap.candidate_count(0.125, kc - 1))
        torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
    assert state.bulk_quantized_rows - rows_before == T           # the prefix, once; the decoded rows came from the steps
    _, packed_o, scale_o = oracle.quantize_pack(key[:, :, :T + 3].cpu(), state.layers[5].channel_idx.cpu())
    assert torch.equal(state.layers[5].packed[:, :, :T + 3].cpu(), packed_o)
    ap.reset_sparse_state()
    assert not state.layers


def test_second_longer_sequence_does_not_reuse_the_first_ones_rows(cuda_device):
    """Sequence A is decoded to 1000+ rows; sequence B (other keys) then arrives with a LONGER prefix through
    the same state. Its selection must come from its own keys (the side cache is rebuilt), not from A's rows."""
    layer = _Layer(2)
    wa, qa, ka, va = make_case(cuda_device, batch=1, q_heads=8, kv_heads=2, context=1003, channels=32, seed=1)
    wb, qb, kb, vb = make_case(cuda_device, batch=1, q_heads=8, kv_heads=2, context=2003, channels=32, seed=2)
    state = ap.SparseDecodeState()
    with ap.attention_mode("qabs32cand12p5attn", sparse_state=state):
        for kc in (1001, 1002):
            ap.sparse_eager_attention_forward(layer, qa[:, :, None, :], ka[:, :, :kc], va[:, :, :kc], None)
        assert state.layers[2].count == 1002
        outb, _ = ap.sparse_eager_attention_forward(layer, qb[:, :, None, :], kb[:, :, :2001], vb[:, :, :2001], None)
    sc = state.layers[2]
    assert sc.count == 2001
    _, packed_o, _ = oracle.quantize_pack(kb[:, :, :2001].cpu(), sc.channel_idx.cpu())
    assert torch.equal(sc.packed[:, :, :2001].cpu(), packed_o)
    want = oracle.decode_step(*cpu(qb, kb[:, :, :2001], vb[:, :, :2001], sc.channel_idx), ap.candidate_count(0.125, 2000))
    torch.testing.assert_close(outb.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)


def test_token_by_token_from_the_first_token_recalibrates_the_channels(cuda_device):
    """Decoding from an empty cache: the channel set first rests on one key row; when the history reaches the
    calibration length it is chosen again from all rows (and the prefix re-quantized), after which the int4
    selection recalls most of the exact group-max top-k and the step equals the oracle for the new channels."""
    T_end, C = 400, 32
    w, q, key, value = make_case(cuda_device, batch=1, q_heads=8, kv_heads=2, context=T_end, channels=C, seed=33)
    layer = _Layer(0)
    state = ap.SparseDecodeState(calibration_tokens=256)
    first_choice = None
    for kc in range(1, T_end + 1):
        with ap.attention_mode("qabs32cand25attn", sparse_state=state):
            out, _ = ap.sparse_eager_attention_forward(layer, q[:, :, None, :], key[:, :, :kc], value[:, :, :kc], None)
        if kc == 2:
            first_choice = state.layers[0].channel_idx.clone()
            assert state.layers[0].calibrated_at == 1
        if kc == 300:
            sc = state.layers[0]
            assert sc.calibrated_at == 256
            assert torch.equal(sc.channel_idx.cpu(), oracle.choose_channels(key[:, :, :256].cpu(), C))
            assert not torch.equal(sc.channel_idx, first_choice)
    sc = state.layers[0]
    assert sc.count == T_end
    k = ap.candidate_count(0.25, T_end - 1)
    want = oracle.decode_step(*cpu(q, key[:, :, :T_end], value[:, :, :T_end], sc.channel_idx), k)
    torch.testing.assert_close(out.float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
    # recall of the int4 selection against the exact (all 128 channels, fp32) group-max top-k
    exact = torch.einsum("bhd,bgtd->bhgt", q.float().cpu(), key[:, :, :T_end - 1].float().cpu())
    G = 4
    exact_g = torch.stack([exact[:, g * G:(g + 1) * G, g].amax(1) for g in range(2)], dim=1)        # [B,Hkv,T]
    top_exact = torch.topk(exact_g, k, dim=-1).indices
    hit = sum(len(set(want["selected"][0, g].tolist()) & set(top_exact[0, g].tolist())) for g in range(2)) / (2 * k)
    assert hit > 0.5, hit


def test_config_1_sized_step_all_28_layers_resident(cuda_device):
    """Batch 8, 16 query / 8 KV heads, 32768 cached tokens, 32 channels, top-1024, the K/V caches of all 28
    layers resident (about 30 GiB): one decode token through the patched attention function of every layer
    under the reference's mode string; per layer, one seeded batch row is recomputed by the oracle."""
    from kv_cache_b200 import inputs
    import dataclasses

    base = inputs.WORKLOADS["c1"]
    B, Hq, Hkv, T, C, k, L = base.batch, base.q_heads, base.kv_heads, base.context, base.channels, base.top_k, base.layers
    mode = ap.mode_for(C, k, T)
    assert mode == "qabs32cand3p125attn"
    caches = []
    for layer in range(L):
        w = dataclasses.replace(base, seed=100 + layer)
        key, value = inputs.make_kv(w, cuda_device, 0, T + 1)
        caches.append((w, key, value, inputs.make_query(w, cuda_device)))
    state = ap.SparseDecodeState()
    outs = []
    with ap.attention_mode(mode, 0.02, 3, True, 0, 0, None, sparse_state=state):
        for layer, (w, key, value, q) in enumerate(caches):
            out, _ = ap.sparse_eager_attention_forward(_Layer(layer), q[:, :, None, :], key, value, None)
            outs.append(out)
    torch.cuda.synchronize()
    assert sorted(state.layers) == list(range(L)) and all(state.layers[l].count == T + 1 for l in range(L))
    for layer, (w, key, value, q) in enumerate(caches):
        b = (5 * layer + 3) % B
        ch = state.layers[layer].channel_idx
        want = oracle.decode_step(q[b:b + 1].cpu(), key[b:b + 1].cpu(), value[b:b + 1].cpu(), ch.cpu(), k)
        torch.testing.assert_close(outs[layer][b:b + 1].float().cpu(), want["out"], rtol=2e-2, atol=1e-2)
        assert torch.equal(state.layers[layer].packed[b:b + 1, :, :T].cpu(), want["packed"])


def test_preallocated_cache_decodes_without_copying_the_cache(cuda_device):
    """A Qwen3-0.6B-shaped model (28 layers) decoded token by token through PreallocatedCache under the sparse
    mode, one `with` block per token as the reference's loop does: K/V buffers, int4 side caches and the step
    workspace keep their storage for the whole decode, the prefix is quantized once, and the logits equal
    those of the same decode through the stock DynamicCache."""
    pytest.importorskip("transformers")
    from transformers import DynamicCache, Qwen3Config, Qwen3ForCausalLM
    from kv_cache_b200.cache import PreallocatedCache

    torch.manual_seed(2)
    cfg = Qwen3Config(vocab_size=1024, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                      num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                      rope_theta=1e6, rms_norm_eps=1e-6, attn_implementation="eager")
    model = Qwen3ForCausalLM(cfg).to(cuda_device, torch.bfloat16).eval()
    ap.install_qwen3_attention_patch()
    try:
        ids = torch.randint(0, 1024, (2, 1200), device=cuda_device)
        steps = [torch.randint(0, 1024, (2, 1), device=cuda_device) for _ in range(4)]
        mode = "qabs32cand6p25attn"

        def decode(cache, state):
            logits = []
            with torch.inference_mode():
                with ap.attention_mode("baseline", sparse_state=state):
                    out = model(input_ids=ids, past_key_values=cache, use_cache=True)
                for tok in steps:
                    with ap.attention_mode(mode, 0.02, 3, True, 4, 16, None, sparse_state=state):
                        out = model(input_ids=tok, past_key_values=out.past_key_values, use_cache=True)
                    logits.append(out.logits.float().clone())
            return logits

        ref_logits = decode(DynamicCache(config=cfg), ap.SparseDecodeState())
        state = ap.SparseDecodeState(capacity_hint=2048)
        cache = PreallocatedCache(num_layers=28, capacity=2048)
        got = decode(cache, state)
        for a, b in zip(got, ref_logits):
            torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-3)
        assert cache.reallocations == 0 and cache.get_seq_length() == 1204
        assert state.bulk_quantized_rows == 28 * 1200                      # every layer's prefix, once
        assert all(state.layers[l].packed.shape[2] >= 2048 and state.layers[l].count == 1204 for l in range(28))
        assert len(state.steps) == 1                                       # one step object (one workspace) for the policy
    finally:
        ap.uninstall_qwen3_attention_patch()
