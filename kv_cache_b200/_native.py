"""ctypes binding of the C-ABI library (include/kvcache_b200.h).

The library is the product: there is no Python or CPU fallback. If it is missing and cannot be
built, or an entry point returns a non-zero status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

from . import build as _build

STATUS_NAMES = {
    0: "KVB_OK",
    1: "KVB_BAD_SHAPE",
    2: "KVB_BAD_ALIGN",
    3: "KVB_BAD_DEVICE",
    4: "KVB_WORKSPACE_TOO_SMALL",
    5: "KVB_TIMEOUT",
    6: "KVB_CUDA_ERROR",
    7: "KVB_BAD_ARG",
    8: "KVB_SCRATCH_LIMIT",
}

_i, _i64, _p, _sz, _f = C.c_int, C.c_int64, C.c_void_p, C.c_size_t, C.c_float


class DecodeStepParams(C.Structure):
    """Mirror of struct kvb_decode_step_params."""

    _fields_ = [
        ("query", _p), ("q_sb", _i64), ("q_sh", _i64),
        ("key", _p), ("k_sb", _i64), ("k_sh", _i64), ("k_st", _i64),
        ("value", _p), ("v_sb", _i64), ("v_sh", _i64), ("v_st", _i64),
        ("packed", _p), ("packed_sb", _i64), ("packed_sh", _i64),
        ("scale", _p), ("scale_sb", _i64), ("scale_sh", _i64),
        ("channel_idx", _p),
        ("mask", _p), ("mask_sb", _i64),
        ("B", _i), ("Hq", _i), ("Hkv", _i), ("D", _i), ("C", _i),
        ("history_count", _i),
        ("top_k", _i),
        ("protect_sink", _i), ("protect_recent", _i), ("keep_self", _i), ("append_protected", _i),
        ("append_self", _i),
        ("scaling", _f),
        ("out", _p),
        ("sel_idx_out", _p),
        ("workspace", _p), ("workspace_bytes", _sz),
        ("history_count_dev", _p), ("advance_history", _i),
        ("new_key_row", _p), ("new_value_row", _p),
        ("selected_any_order", _i),
        ("kv_page_table", _p),
        ("kv_page_table_stride", _i64),
        ("kv_page_tokens", _i),
    ]


class ShardedStepParams(C.Structure):
    """Mirror of struct kvb_sharded_step_params."""

    _fields_ = [
        ("query", _p), ("q_sb", _i64), ("q_sh", _i64),
        ("key", _p), ("k_sb", _i64), ("k_sh", _i64), ("k_st", _i64),
        ("value", _p), ("v_sb", _i64), ("v_sh", _i64), ("v_st", _i64),
        ("packed", _p), ("packed_sb", _i64), ("packed_sh", _i64),
        ("scale", _p), ("scale_sb", _i64), ("scale_sh", _i64),
        ("channel_idx", _p),
        ("B", _i), ("Hq", _i), ("Hkv", _i), ("D", _i), ("C", _i),
        ("t_local", _i), ("id_offset", _i64), ("total_tokens", _i64),
        ("top_k", _i), ("rank", _i), ("world", _i),
        ("scaling", _f),
        ("out", _p), ("sel_idx_out", _p),
        ("workspace", _p), ("workspace_bytes", _sz),
        ("exchange", _p * 8), ("exchange_bytes", _sz),
        ("phases", _i), ("wait_polls", C.c_uint),
    ]


# name -> (restype, argtypes); every symbol declared in include/kvcache_b200.h
SIGNATURES = {
    "kvb_version": (_i, []),
    "kvb_status_string": (C.c_char_p, [_i]),
    "kvb_device_status": (_i, [_i, C.POINTER(_i)]),
    "kvb_quantize_pack": (_i, [_p, _i64, _i64, _i64, _p, _p, _i64, _i64, _p, _i64, _i64,
                               _i, _i, _i, _i, _i, _i64, _i, _p]),
    "kvb_quantize_append": (_i, [_p, _i64, _i64, _p, _p, _i64, _i64, _p, _i64, _i64,
                                 _i, _i, _i, _i, _i64, _i, _p]),
    "kvb_score_decode": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p,
                              _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _i, _p]),
    "kvb_candidate_capacity": (_i, [_i]),
    "kvb_sample_thresholds": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p,
                                   _i, _i, _i, _i, _i, _i, _i, _p, _i, _p]),
    "kvb_score_candidates": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p,
                                  _i, _i, _i, _i, _i, _i, _p, _p, _p, _i, _i, _p]),
    "kvb_select_topk_workspace_bytes": (_sz, [_i, _i, _i]),
    "kvb_select_topk": (_i, [_p, _i64, _p, _i, _i, _i, _i64, _i, _p, _p, _p, _p, _p, _sz, _i, _p]),
    "kvb_select_topk_static_limit_bytes": (_sz, []),
    "kvb_select_topk_static": (_i, [_p, _i64, _i, _i, _i, _i64, _i, _p, _p, _p, _i, _p]),
    "kvb_final_index_count": (_i, [_i, _i, _i, _i, _i]),
    "kvb_build_final_indices": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _i, _p]),
    "kvb_sparse_attend_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "kvb_sparse_attend": (_i, [_p, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _i64, _i64,
                               _p, _i, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _f,
                               _p, _p, _p, _sz, _i, _p]),
    "kvb_attend_selected": (_i, [_p, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _i64, _i64,
                                 _p, _i, _p, _i64, _i, _i, _i, _i, _i, _p, _i64,
                                 _i, _i, _i, _i, _i, _f, _p, _p, _p, _sz, _i, _p]),
    "kvb_shard_candidates_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "kvb_shard_candidates": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p,
                                  _i, _i, _i, _i, _i, _i, _i, _i, _i64, _p, _p, _sz, _i, _p]),
    "kvb_merge_candidates": (_i, [_p, _i, _i, _i, _i, _i64, _i, _p, _i64, _i64, _p, _p, _i, _p]),
    "kvb_score_select": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p,
                              _i, _i, _i, _i, _i, _i, _i, _i, _p, _p, _sz, _i, _p]),
    "kvb_rerank_union_workspace_bytes": (_sz, [_i, _i]),
    "kvb_rerank_union": (_i, [_p, _i64, _i64, _p, _i64, _i64, _i64, _p, _i, _p, _p, _i, _p, _p, _i, _p, _i, _i,
                              _p, _i64, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p, _sz, _i, _p]),
    "kvb_sparq_alpha_workspace_bytes": (_sz, [_i, _i, _i]),
    "kvb_sparq_alpha": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _p, _p, _i64, _p, _i, _p,
                             _i, _i, _i, _i, _i, _i, _p, _p, _sz, _i, _p]),
    "kvb_attend_selected_blend": (_i, [_p, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _i64, _i64, _p, _i, _p,
                                       _i, _i, _p, _i64, _p, _p, _i, _i, _i, _i, _i, _f, _p, _p, _sz, _i, _p]),
    "kvb_expand_final": (_i, [_p, _i, _p, _i, _i, _i, _i, _i, _p, _i, _p, _i, _p]),
    "kvb_sharded_exchange_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "kvb_sharded_step_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "kvb_exchange_alloc": (_i, [_sz, _i, C.POINTER(_p), _p]),
    "kvb_exchange_open": (_i, [_p, _i, C.POINTER(_p)]),
    "kvb_exchange_close": (_i, [_p, _i]),
    "kvb_exchange_free": (_i, [_p, _i]),
    "kvb_sharded_decode_step": (_i, [C.POINTER(ShardedStepParams), _i, _p]),
    "kvb_lse_merge": (_i, [_p, _i, _i, _i, _i, _p, _i, _p]),
    "kvb_quantize_query_tokens": (_i, [_p, _i64, _i64, _i64, _p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "kvb_score_prefill_blocks": (_i, [_p, _p, _p, _i64, _i64, _p, _i64, _i64, _i, _i, _i, _i, _i, _i, _i, _p, _i, _p]),
    "kvb_score_prefill_blocks_engine": (_i, [_p, _p, _p, _i64, _i64, _p, _i64, _i64, _i, _i, _i, _i, _i, _i, _i, _p, _i,
                                             _i, _p]),
    "kvb_prefill_operand_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "kvb_widen_keys": (_i, [_p, _i64, _i64, _i, _i, _i, _i, _i, _i, _i, _p, _sz, _i, _p]),
    "kvb_score_prefill_blocks_widened": (_i, [_p, _p, _p, _sz, _i, _p, _i64, _i64, _i, _i, _i, _i, _i, _i, _i, _p, _i,
                                              _i, _p]),
    "kvb_block_topk": (_i, [_p, _i64, _i64, _i, _i, _p, _p, _i, _p]),
    "kvb_qabs_partial_scores": (_i, [_p, _p, _i64, _i64, _i64, _i64, _p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "kvb_qabs_candidate_full_scores": (_i, [_p, _p, _i64, _i64, _i64, _p, _p, _p, _i, _i, _f, _p,
                                            _i, _i, _i, _i, _i, _i, _i, _p]),
    "kvb_decode_step_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i, _i]),
    "kvb_decode_step": (_i, [C.POINTER(DecodeStepParams), _i, _p]),
}


def library_path() -> Path:
    return _build.LIB_PATH


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    """Loads (building first when stale) the shared library and declares every prototype."""
    path = _build.LIB_PATH
    if _build.is_stale():
        try:
            _build.build()
        except Exception as exc:  # no nvcc on this machine and no prebuilt library
            if not path.exists():
                raise RuntimeError(
                    f"kv_cache_b200: the CUDA library {path} is missing and could not be built ({exc}); "
                    "there is no fallback path"
                ) from exc
    handle = C.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(handle, name)  # AttributeError if the library does not export it
        fn.restype = restype
        fn.argtypes = argtypes
    return handle


def check(status: int, what: str) -> None:
    if status != 0:
        name = STATUS_NAMES.get(status, str(status))
        raise RuntimeError(f"kv_cache_b200: {what} failed with {name}")
