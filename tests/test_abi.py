"""The C-ABI library builds for sm_100a, loads without a GPU, and exports every symbol that
include/kvcache_b200.h declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

from kv_cache_b200 import _native, build

HEADER = Path(__file__).resolve().parents[1] / "include" / "kvcache_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(kvb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("kvb_quantize_pack", "kvb_quantize_append", "kvb_score_decode", "kvb_select_topk",
                 "kvb_sparse_attend", "kvb_decode_step", "kvb_select_topk_workspace_bytes",
                 "kvb_sparse_attend_workspace_bytes"):
        assert must in names


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    assert path.exists()
    handle = ctypes.CDLL(str(path))
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert sorted(_native.SIGNATURES) == declared_symbols()
    lib = _native.lib()
    assert lib.kvb_version() >= 100
    assert lib.kvb_status_string(0) == b"ok"
    assert lib.kvb_status_string(4) == b"workspace too small"


def test_size_queries_need_no_gpu():
    lib = _native.lib()
    assert lib.kvb_final_index_count(2048, 131072, 0, 0, 1) == 2049
    assert lib.kvb_final_index_count(16, 100, 4, 5, 1) == 16 + 4 + 5 + 1
    assert lib.kvb_final_index_count(16, 100, 200, 0, 0) == 16 + 100
    assert lib.kvb_select_topk_workspace_bytes(128, 131072, 2048) > 128 * 8192 * 8
    assert lib.kvb_sparse_attend_workspace_bytes(16, 32, 8, 2049) > 0
    assert lib.kvb_sparse_attend_workspace_bytes(16, 32, 5, 2049) == 0
    assert lib.kvb_decode_step_workspace_bytes(16, 32, 8, 131072, 2048, 0, 0, 1) > 16 * 8 * 131072 * 4


def test_exchange_buffer_size_follows_the_documented_layout():
    """step counter | full candidate lists [R, k] of 8-byte composites | inbox [N, R, prefix] of 16-byte tagged
    pairs | flags [N, R] | partial inbox [N, B*Hq, D+2] of 8-byte tagged pairs, each area rounded to 256 bytes."""
    lib = _native.lib()
    D = 128
    for B, Hq, Hkv, k, N in [(4, 32, 8, 4096, 1), (4, 32, 8, 4096, 2), (4, 32, 8, 4096, 8), (2, 8, 2, 64, 3),
                             (16, 32, 8, 2048, 4)]:
        R = B * Hkv
        prefix = min(k, 8192 // N)
        assert N * prefix >= k                                    # the prefixes alone can hold a full answer
        areas = [4, 8 * R * k, 16 * N * R * prefix, 4 * N * R, 8 * N * B * Hq * (D + 2)]
        got = lib.kvb_sharded_exchange_bytes(B, Hq, Hkv, k, N)
        assert sum(areas) <= got <= sum(areas) + 256 * len(areas)
        assert got % 256 == 0


def test_bad_arguments_are_rejected_before_any_launch():
    lib = _native.lib()
    # null pointers / impossible shapes return a status without touching a device
    assert lib.kvb_quantize_pack(None, 0, 0, 0, None, None, 0, 0, None, 0, 0, 1, 1, 1, 128, 32, 0, 0, None) == 7
    assert lib.kvb_select_topk(None, 0, None, 1, 1, 1, 0, 0, None, None, None, None, None, 0, 0, None) == 7
    assert lib.kvb_lse_merge(None, 1, 1, 1, 128, None, 0, None) == 7
