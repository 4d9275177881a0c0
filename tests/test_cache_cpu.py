"""The pre-allocated KV cache on CPU tensors: the HF Cache contract (update returns views of everything
stored so far), in-place storage, growth, crop, clone — and a tiny HF Qwen3 model that decodes through it to the
same logits as through DynamicCache."""
import pytest
import torch

pytest.importorskip("transformers")
from kv_cache_b200.cache import PreallocatedCache, PreallocatedLayer  # noqa: E402


def test_update_writes_in_place_and_returns_views():
    cache = PreallocatedCache(num_layers=2, capacity=16)
    k0 = torch.randn(2, 3, 5, 8)
    v0 = torch.randn(2, 3, 5, 8)
    keys, values = cache.update(k0, v0, 0)
    assert keys.shape == (2, 3, 5, 8) and torch.equal(keys, k0) and torch.equal(values, v0)
    base = cache.layers[0].key_buffer.data_ptr()
    assert keys.data_ptr() == base and keys.stride(1) == 16 * 8          # a view of the capacity-sized buffer
    k1, v1 = torch.randn(2, 3, 1, 8), torch.randn(2, 3, 1, 8)
    keys, values = cache.update(k1, v1, 0)
    assert keys.shape[2] == 6 and keys.data_ptr() == base                 # no re-allocation, no concatenation
    assert torch.equal(keys[:, :, :5], k0) and torch.equal(keys[:, :, 5:], k1)
    assert cache.get_seq_length(0) == 6 and cache.get_seq_length(1) == 0
    assert cache.layers[0].get_mask_sizes(1) == (7, 0)
    assert cache.reallocations == 0


def test_growth_crop_reset_and_clone():
    layer = PreallocatedLayer(capacity=4)
    a = torch.arange(2 * 1 * 3 * 2, dtype=torch.float32).view(2, 1, 3, 2)
    layer.update(a, a + 100)
    layer.update(a, a + 100)                                              # 6 rows > capacity 4: one growth
    assert layer.reallocations == 1 and layer.capacity >= 6 and layer.get_seq_length() == 6
    assert torch.equal(layer.keys, torch.cat((a, a), dim=2)) and torch.equal(layer.values, torch.cat((a, a), dim=2) + 100)
    layer.crop(4)
    assert layer.get_seq_length() == 4 and torch.equal(layer.keys, torch.cat((a, a), dim=2)[:, :, :4])
    layer.crop(-1)
    assert layer.get_seq_length() == 3
    other = layer.clone_prefix()
    other.update(a[:, :, :1], a[:, :, :1])
    assert layer.get_seq_length() == 3 and other.get_seq_length() == 4
    assert other.key_buffer.data_ptr() != layer.key_buffer.data_ptr()
    layer.reset()
    assert layer.get_seq_length() == 0 and layer.keys.shape[2] == 0


def test_tiny_qwen3_decodes_to_the_same_logits_as_with_dynamic_cache():
    from transformers import DynamicCache, Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=16, max_position_embeddings=256, attn_implementation="eager")
    model = Qwen3ForCausalLM(cfg).eval()
    ids = torch.randint(0, 128, (2, 12))
    with torch.inference_mode():
        pre_a = model(input_ids=ids, past_key_values=DynamicCache(config=cfg), use_cache=True)
        cache = PreallocatedCache(num_layers=2, capacity=64)
        pre_b = model(input_ids=ids, past_key_values=cache, use_cache=True)
        torch.testing.assert_close(pre_b.logits, pre_a.logits)
        past_a = pre_a.past_key_values
        ptrs = [layer.key_buffer.data_ptr() for layer in cache.layers]
        for _ in range(4):
            nxt = torch.randint(0, 128, (2, 1))
            out_a = model(input_ids=nxt, past_key_values=past_a, use_cache=True)
            out_b = model(input_ids=nxt, past_key_values=cache, use_cache=True)
            torch.testing.assert_close(out_b.logits, out_a.logits)
            past_a = out_a.past_key_values
            assert out_b.past_key_values is cache
    assert cache.get_seq_length() == 16 and cache.reallocations == 0
    assert [layer.key_buffer.data_ptr() for layer in cache.layers] == ptrs


def test_paged_kv_bookkeeping_on_cpu():
    """Pages are handed out in the given order, rows never move, gather() returns what was appended."""
    from kv_cache_b200.cache import PagedKV

    g = torch.Generator().manual_seed(0)
    B, H, D, P = 2, 2, 128, 8
    order = torch.randperm(20, generator=g)
    kv = PagedKV(B, H, D, P, 20, "cpu", pages_per_sequence=6, dtype=torch.float32, free_order=order)
    k = torch.randn(B, H, 37, D, generator=g)
    v = torch.randn(B, H, 37, D, generator=g)
    kv.append(k[:, :, :5], v[:, :, :5])
    first_pages = kv.page_table[:, 0].clone()
    kv.append(k[:, :, 5:30], v[:, :, 5:30])
    kv.append(k[:, :, 30:], v[:, :, 30:])
    assert kv.length == 37 and torch.equal(kv.page_table[:, 0], first_pages)
    gk, gv = kv.gather()
    assert torch.equal(gk, k) and torch.equal(gv, v)
    used = kv.page_table[:, :5].flatten().tolist()
    assert len(set(used)) == 10 and used[:2] != used[2:4]                 # ten distinct pages for 2 x 5
    assert sorted(used) == sorted(int(i) for i in order[:10].tolist())     # taken in the order given
    with pytest.raises(RuntimeError):
        kv.append(k[:, :, :20], v[:, :, :20])                             # 57 tokens need 8 pages per sequence, the table has 6
