"""Helpers shared by the GPU parity tests (inputs come from kv_cache_b200.inputs, the checker
from oracle/)."""
import torch

from kv_cache_b200 import inputs


def make_case(device, **kw):
    """Small seeded workload: query [B,Hq,D], key/value [B,Hkv,T+1,D] (last row = decoded token)."""
    w = inputs.small_workload(**kw)
    key, value = inputs.make_kv(w, device, 0, w.context + 1)
    query = inputs.make_query(w, device)
    return w, query, key, value


def cpu(*ts):
    return [None if t is None else t.detach().cpu() for t in ts]
