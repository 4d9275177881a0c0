"""Seeded synthetic K/V/query tensors with the shapes and value distributions of the benchmark
configurations (they stand in for the natural-text caches the reference measured on).

K and V are N(0,1); K is multiplied per (KV head, channel) by lognormal(0,1) factors to emulate
outlier channels; RoPE (theta 1e6, HF rotate-half pairing i <-> i + D/2) is applied to K at
absolute positions and to the query at position T; everything is cast to bf16 once. Values are
generated per (seed, batch row, 4096-token chunk), so any token range of any sequence can be
produced on its own (a sequence shard, or a slice handed to a CPU checker).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

TOKEN_CHUNK = 4096
ROPE_THETA = 1.0e6


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    head_dim: int
    context: int          # history tokens T (the decode query sits at position T)
    channels: int         # int4 partial channels C
    top_k: int
    seed: int
    layers: int = 1

    @property
    def group(self) -> int:
        return self.q_heads // self.kv_heads

    def algorithmic_bytes(self) -> dict:
        """Bytes one layer-step must move: packed K + scales read once, selected K/V rows once per KV head."""
        rows = self.batch * self.kv_heads
        scan = rows * self.context * (self.channels // 2 + 4)
        k_eff = min(self.top_k, self.context)
        gather = rows * (k_eff + 1) * self.head_dim * 2 * 2
        return {"scan": scan, "gather": gather, "total": scan + gather}


# BASELINE configurations (decode ones); c1 is one layer of the 28-layer model's shapes.
WORKLOADS = {
    "c0": Workload("c0_qwen3-0.6b_b1_t4096_c32_k256", 1, 16, 8, 128, 4096, 32, 256, seed=0),
    "c1": Workload("c1_qwen3-0.6b_b8_t32768_c32_k1024", 8, 16, 8, 128, 32768, 32, 1024, seed=1, layers=28),
    "c2": Workload("c2_qwen3-8b_b16_t131072_c64_k2048", 16, 32, 8, 128, 131072, 64, 2048, seed=2, layers=36),
    "c4": Workload("c4_qwen3-8b_b4_t1048576_c64_k4096", 4, 32, 8, 128, 1048576, 64, 4096, seed=4),
}


def _seed_for(seed: int, what: int, b: int, chunk: int) -> int:
    return (seed * 1_000_003 + what * 15_485_863 + b * 7_919 + chunk * 104_729 + 12_345) % (2**62)


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def channel_multipliers(kv_heads: int, head_dim: int, seed: int, device) -> torch.Tensor:
    """lognormal(0,1) factor per (KV head, channel), fp32 ``[Hkv, D]``; generated on the CPU so that
    every device and every shard sees the same outlier channels."""
    g = _gen("cpu", _seed_for(seed, 1, 0, 0))
    return torch.exp(torch.randn((kv_heads, head_dim), generator=g, dtype=torch.float32)).to(device)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float = ROPE_THETA) -> torch.Tensor:
    """HF rotary embedding of fp32 ``x[..., T, D]`` at integer ``positions[T]``."""
    D = x.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    cos, sin = emb.cos(), emb.sin()
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return x * cos + torch.cat((-x2, x1), dim=-1) * sin


def make_kv(w: Workload, device, t_begin: int = 0, t_end: Optional[int] = None,
            batch_rows: Optional[range] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``K, V [B', Hkv, t_end - t_begin, D]`` for absolute token positions ``[t_begin, t_end)``
    (``t_end`` may be ``context + 1`` to include the row of the token being decoded)."""
    t_end = w.context if t_end is None else t_end
    rows = list(range(w.batch) if batch_rows is None else batch_rows)
    n = t_end - t_begin
    K = torch.empty((len(rows), w.kv_heads, n, w.head_dim), dtype=torch.bfloat16, device=device)
    V = torch.empty_like(K)
    mult = channel_multipliers(w.kv_heads, w.head_dim, w.seed, device)
    first_chunk = t_begin // TOKEN_CHUNK
    last_chunk = (t_end - 1) // TOKEN_CHUNK if n > 0 else first_chunk - 1
    for bi, b in enumerate(rows):
        for ch in range(first_chunk, last_chunk + 1):
            c0, c1 = ch * TOKEN_CHUNK, (ch + 1) * TOKEN_CHUNK
            g = _gen(device, _seed_for(w.seed, 2, b, ch))
            kf = torch.randn((w.kv_heads, TOKEN_CHUNK, w.head_dim), generator=g, dtype=torch.float32, device=device)
            vf = torch.randn((w.kv_heads, TOKEN_CHUNK, w.head_dim), generator=g, dtype=torch.float32, device=device)
            pos = torch.arange(c0, c1, device=device)
            kf = rope(kf * mult[:, None, :], pos)
            lo, hi = max(c0, t_begin), min(c1, t_end)
            K[bi, :, lo - t_begin: hi - t_begin] = kf[:, lo - c0: hi - c0].to(torch.bfloat16)
            V[bi, :, lo - t_begin: hi - t_begin] = vf[:, lo - c0: hi - c0].to(torch.bfloat16)
    return K, V


def make_query(w: Workload, device, position: Optional[int] = None) -> torch.Tensor:
    """bf16 decode query ``[B, Hq, D]`` with RoPE at ``position`` (default: the context length)."""
    position = w.context if position is None else position
    g = _gen("cpu", _seed_for(w.seed, 3, 0, 0))
    q = torch.randn((w.batch, w.q_heads, 1, w.head_dim), generator=g, dtype=torch.float32)
    q = rope(q, torch.tensor([position]))
    return q[:, :, 0, :].to(torch.bfloat16).to(device)


def small_workload(name: str = "small", batch: int = 2, q_heads: int = 8, kv_heads: int = 2, context: int = 1000,
                   channels: int = 32, top_k: int = 64, seed: int = 7, head_dim: int = 128) -> Workload:
    return Workload(name, batch, q_heads, kv_heads, head_dim, context, channels, top_k, seed)
