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
    assert ap.parse_qabs_partial_rerank_params("qabs8cand3reuse") == (8, 0.03)
    assert ap.parse_qabs_partial_rerank_params("qabs8cand3keep") is None
    assert ap.parse_qabs_partial_rerank_params("baseline") is None
    assert ap.parse_mode_kind("qabs8cand3reuse") == ("reuse", 1)
    assert ap.parse_mode_kind("qabs8cand3reuse2setblk16") == ("reuse2set", 16)
    assert ap.parse_mode_kind("qabs8cand3reusefinal") == ("reusefinal", 1)
    assert ap.parse_mode_kind("qabs8cand3top2attn") == ("top2attn", 1)
    assert ap.parse_mode_kind("qabs8cand3appendattn") == ("appendattn", 1)
    assert ap.parse_mode_kind("qabs8cand3attn") == ("attn", 1)


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
        assert state is ap.default_sparse_state() and ap._ACTIVE_STATE is state      # the module-level state by default
        with ap.attention_mode("baseline"):
            assert ap._ACTIVE_MODE == "baseline"
        assert ap._ACTIVE_MODE == "qabs32cand6p25attn"
    assert ap._ACTIVE_MODE == "baseline" and ap._ACTIVE_STATE is None
    own = ap.SparseDecodeState()
    with ap.attention_mode("qabs32cand6p25attn", sparse_state=own) as state:
        assert state is own
    with pytest.raises(RuntimeError, match="implements"):
        with ap.attention_mode("qabs8cand3keep"):
            pass


def test_attention_mode_binds_the_reference_call_with_29_positionals():
    """The evaluator's hot loop (EVAL:7236-7266) passes every parameter of EVAL:6947-6976 by position."""
    import inspect

    names = ["mode", "top_fraction", "max_heads_per_token", "always_keep_self", "protect_sink_tokens",
             "protect_recent_tokens", "load_stats", "obs_state", "obs_mass_state", "obs_hybrid_state", "reuse_state",
             "knorm_state", "block_route_state", "ksign_state", "kdom_state", "brep_state", "sparq_mean_state",
             "candidate_stats", "reuse_overlap_stats", "qabs_fast_path", "qabs_cuda_final_kernel",
             "qabs_cuda_candidate_kernel", "qabs_cuda_reuse_select_kernel", "qabs_profile_stats",
             "qabs_candidate_selection", "qabs_threshold_sample_size", "full_head_map_path", "full_layer_map_path",
             "layer_budget_map_path"]
    sig = inspect.signature(ap.attention_mode)
    positional = [n for n, p in sig.parameters.items() if p.kind == p.POSITIONAL_OR_KEYWORD]
    assert positional == names                                   # same names, same order
    assert sig.parameters["sparse_state"].kind == inspect.Parameter.KEYWORD_ONLY
    args = ("qabs8cand3attn", 0.02, 3, True, 10, 10, None, None, None, None, None, None, None, None, None, None, None,
            None, None, True, False, False, False, None, "topk", 256, "", "", "")
    assert len(args) == 29
    with ap.attention_mode(*args):
        assert ap._ACTIVE_MODE == "qabs8cand3attn" and ap._ACTIVE_PROTECT_SINK_TOKENS == 10
    assert ap._ACTIVE_MODE == "baseline"


def test_qabs_cuda_kernels_alias_serves_the_top_level_import():
    import sys

    saved = sys.modules.pop("qabs_cuda_kernels", None)
    try:
        ap.install_qabs_cuda_kernels_alias()
        from qabs_cuda_kernels import candidate_full_scores, final_attention, partial_scores, partial_scores_dim_major  # noqa: F401
        import kv_cache_b200.qabs_cuda_kernels as mine
        assert partial_scores is mine.partial_scores and final_attention is mine.final_attention
    finally:
        sys.modules.pop("qabs_cuda_kernels", None)
        if saved is not None:
            sys.modules["qabs_cuda_kernels"] = saved


def test_side_cache_continuity_rule():
    """A layer's int4 rows survive only while the calls seen by the patched function continue its sequence."""
    st = ap.SparseDecodeState()
    t = torch.zeros(1)
    st.layers[0] = ap.LayerSideCache(t, t, t, count=100, seen=100)
    st.observe(0, 101, 1)                      # a dense decode step of the same sequence: kept, one row pending
    assert st.layers[0].seen == 101 and st.layers[0].count == 100
    st.observe(0, 140, 39)                     # a prefill chunk that continues it
    assert st.layers[0].seen == 140
    st.observe(0, 2000, 2000)                  # a new sequence is prefilled (longer than the old one): dropped
    assert 0 not in st.layers
    st.layers[1] = ap.LayerSideCache(t, t, t, count=50, seen=50)
    st.observe(1, 50, 1)                       # a step that re-decodes an old position: not a continuation
    assert 1 not in st.layers
    st.observe(7, 10, 10)                      # unknown layer: nothing to do


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
