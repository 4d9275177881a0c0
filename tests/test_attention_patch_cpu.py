"""Host logic of the drop-in attention patch that needs no GPU: the mode mini-language
(EVAL:748-754), the candidate count rule (EVAL:4423), the context manager's save/restore of the
process-global mode (EVAL:6947-7075) and the loud failure on modes that are not implemented."""
import pytest
import torch

from kv_cache_b200 import attention_patch as ap


def test_mode_strings_parse_like_the_reference():
    assert ap.parse_qabs_partial_rerank_params("qabs32cand6p25attn") == (32, 0.0625)
    assert ap.parse_qabs_partial_rerank_params("qabs64cand1p5625attn") == (64, 0.015625)
    assert ap.parse_qabs_partial_rerank_params("qabs8cand25appendattn") == (8, 0.25)
    assert ap.parse_qabs_partial_rerank_params("qabs8cand3reuse") is None
    assert ap.parse_qabs_partial_rerank_params("baseline") is None


def test_candidate_count_and_mode_for_round_trip():
    assert ap.candidate_count(0.0625, 4096) == 256
    assert ap.candidate_count(0.015625, 131072) == 2048
    assert ap.candidate_count(0.5, 1) == 1
    for c, k, t in ((32, 256, 4096), (32, 1024, 32768), (64, 2048, 131072), (64, 4096, 1048576)):
        mode = ap.mode_for(c, k, t)
        ch, frac = ap.parse_qabs_partial_rerank_params(mode)
        assert ch == c and ap.candidate_count(frac, t) == k
    assert ap.mode_for(64, 2048, 131072) == "qabs64cand1p5625attn"


def test_attention_mode_restores_globals_and_rejects_unknown_modes():
    assert ap._ACTIVE_MODE == "baseline"
    with ap.attention_mode("qabs32cand6p25attn", 0.02, 3, False, 7, 9, None, reuse_state=None,
                           qabs_fast_path=True) as state:
        assert ap._ACTIVE_MODE == "qabs32cand6p25attn"
        assert (ap._ACTIVE_ALWAYS_KEEP_SELF, ap._ACTIVE_PROTECT_SINK_TOKENS, ap._ACTIVE_PROTECT_RECENT_TOKENS) == (False, 7, 9)
        assert isinstance(state, ap.SparseDecodeState) and ap._ACTIVE_STATE is state
        with ap.attention_mode("baseline"):
            assert ap._ACTIVE_MODE == "baseline"
        assert ap._ACTIVE_MODE == "qabs32cand6p25attn"
    assert ap._ACTIVE_MODE == "baseline" and ap._ACTIVE_STATE is None
    with pytest.raises(RuntimeError, match="implements"):
        with ap.attention_mode("qabs8cand3reuse"):
            pass


def test_forward_contract_errors_without_a_gpu():
    class M(torch.nn.Module):
        layer_idx = 0

    q = torch.zeros(1, 4, 3, 128, dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 9, 128, dtype=torch.bfloat16)
    with ap.attention_mode("qabs32cand50attn"):
        with pytest.raises(RuntimeError, match="token-by-token"):       # same message as EVAL:4413-4414
            ap.sparse_eager_attention_forward(M(), q, k, k, None)
        # a single key row short-circuits to the value row (EVAL:4415-4417)
        out, w = ap.sparse_eager_attention_forward(M(), q[:, :, :1], k[:, :, :1], k[:, :, :1] + 1, None)
        assert out.shape == (1, 1, 4, 128) and w is None and (out == 1).all()
        # CPU tensors reach the operators and fail loudly: no fallback path exists
        with pytest.raises(RuntimeError):
            ap.sparse_eager_attention_forward(M(), q[:, :, :1], k, k, None)
