"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

Generator rule: every per-token tensor is drawn in chunks of 4096 tokens, chunk c of tensor number j
from `manual_seed(seed * 1_000_003 + 1009 * j + c)` in fp32 and then cast; small replicated parameters
(norm weight, router bias, smooth scales, cos/sin table) come from `manual_seed(seed)`.  A rank that owns
tokens [t0, t1) therefore generates exactly the rows a single-GPU run would hold there, and a CPU run
(`gen_device="cpu"`) yields the same bits for the parity tests.  A CUDA generator gives a different
(equally seeded) stream and is only used where values do not matter (throughput runs).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

CHUNK = 4096


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def per_token(kind: str, j: int, t0: int, t1: int, width: int, dtype, seed: int = 0, gen_device="cpu",
              out_device=None, high: int = 0) -> torch.Tensor:
    """Rows [t0, t1) of per-token tensor number j ([tokens, width]).  kind: "randn" | "randint"."""
    out_device = out_device or gen_device
    out = torch.empty((t1 - t0, width) if width else (t1 - t0,), dtype=dtype, device=out_device)
    c0, c1 = t0 // CHUNK, (max(t1, t0 + 1) - 1) // CHUNK
    for c in range(c0, c1 + 1):
        lo, hi = c * CHUNK, (c + 1) * CHUNK
        g = _gen(seed * 1_000_003 + 1009 * j + c, gen_device)
        shape = (CHUNK, width) if width else (CHUNK,)
        if kind == "randn":
            chunk = torch.randn(shape, generator=g, device=gen_device, dtype=torch.float32)
        else:
            chunk = torch.randint(0, high, shape, generator=g, device=gen_device, dtype=torch.int64)
        a, b = max(lo, t0), min(hi, t1)
        if b > a:
            out[a - t0:b - t0] = chunk[a - lo:b - lo].to(dtype)
    return out


def norm_weight(hidden: int, dtype, seed: int = 0, device="cpu") -> torch.Tensor:
    g = _gen(seed, "cpu")
    return (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).to(device)


def cos_sin_cache(max_pos: int, rot_dim: int, theta: float, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """[max_pos, rot_dim] = cos || sin with inv_freq = theta^(-2i/rot_dim)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    ang = torch.arange(max_pos, dtype=torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
    return torch.cat([ang.cos(), ang.sin()], dim=-1).to(dtype).to(device)


# ----------------------------------------------------------------------------------------------
# Part 1: add + RMSNorm + per-token int8 quant
# ----------------------------------------------------------------------------------------------
def norm_quant_inputs(tokens: int, hidden: int, t0: int = 0, seed: int = 0, gen_device="cpu", device=None,
                      dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    device = device or gen_device
    return {
        "x": per_token("randn", 0, t0, t0 + tokens, hidden, dtype, seed, gen_device, device),
        "residual": per_token("randn", 1, t0, t0 + tokens, hidden, dtype, seed, gen_device, device),
        "weight": norm_weight(hidden, dtype, seed, device),
        "eps": 1e-6,
    }


def norm_quant_bytes(tokens: int, hidden: int, elem: int = 2) -> int:
    """x and residual read, residual and int8 codes written, weight read once, one fp32 scale per token."""
    return tokens * hidden * (2 * elem + elem + 1) + hidden * elem + 4 * tokens


# ----------------------------------------------------------------------------------------------
# Part 2: NeoX RoPE + int8 paged KV store
# ----------------------------------------------------------------------------------------------
def rope_kv_inputs(tokens: int, q_heads: int, kv_heads: int, head_dim: int, max_pos: int, theta: float = 500000.0,
                   block_size: int = 16, num_blocks: int = 2048, t0: int = 0, seed: int = 0, gen_device="cpu",
                   device=None, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """slot_mapping is a random permutation of the first `tokens` slots of this rank's own cache;
    scales are NOT filled in here (they depend on the rotated K): see `kv_scales`."""
    device = device or gen_device
    assert tokens <= block_size * num_blocks
    g = _gen(seed * 1_000_003 + 7919 + t0, "cpu")
    return {
        "query": per_token("randn", 10, t0, t0 + tokens, q_heads * head_dim, dtype, seed, gen_device, device),
        "key": per_token("randn", 11, t0, t0 + tokens, kv_heads * head_dim, dtype, seed, gen_device, device),
        "value": per_token("randn", 12, t0, t0 + tokens, kv_heads * head_dim, dtype, seed, gen_device, device),
        "positions": per_token("randint", 13, t0, t0 + tokens, 0, torch.int64, seed, gen_device, device, high=max_pos),
        "cos_sin_cache": cos_sin_cache(max_pos, head_dim, theta, torch.float32, device),
        "slot_mapping": torch.randperm(tokens, generator=g).to(torch.int64).to(device),
        "key_cache": torch.zeros(num_blocks, block_size, kv_heads, head_dim, dtype=torch.int8, device=device),
        "value_cache": torch.zeros(num_blocks, block_size, kv_heads, head_dim, dtype=torch.int8, device=device),
        "head_size": head_dim,
    }


def kv_scales(rotated_key: torch.Tensor, value: torch.Tensor, kv_heads: int, head_dim: int):
    """Per-head dequantisation scales absmax/127 of the (bf16-rounded) rotated K and of V."""
    n = rotated_key.shape[0]
    k = rotated_key.reshape(n, kv_heads, head_dim).float().abs().amax(dim=(0, 2)) / 127.0
    v = value.reshape(n, kv_heads, head_dim).float().abs().amax(dim=(0, 2)) / 127.0
    return k.contiguous(), v.contiguous()


def rope_kv_bytes(tokens: int, q_heads: int, kv_heads: int, head_dim: int, elem: int = 2) -> int:
    """q, k, v read; q, k written; two int8 cache rows written; position, slot and the cos/sin row read."""
    q = tokens * q_heads * head_dim * elem
    kv = tokens * kv_heads * head_dim * elem
    return 2 * q + 2 * kv + kv + 2 * (tokens * kv_heads * head_dim) + tokens * (16 + head_dim * 4)


# ----------------------------------------------------------------------------------------------
# Part 3: routing + dispatch + combine
# ----------------------------------------------------------------------------------------------
def router_inputs(tokens: int, experts: int, t0: int = 0, seed: int = 0, gen_device="cpu", device=None):
    device = device or gen_device
    g = _gen(seed, "cpu")
    return {
        "logits": per_token("randn", 20, t0, t0 + tokens, experts, torch.float32, seed, gen_device, device),
        "bias": (0.01 * torch.randn(experts, generator=g)).to(device),
    }


def dispatch_inputs(tokens: int, hidden: int, experts: int, topk: int, t0: int = 0, seed: int = 0, gen_device="cpu",
                    device=None, with_hidden: bool = True):
    """hidden states (seed), smooth scales = 1.0, and the synthetic expert outputs y (seed + 1)."""
    device = device or gen_device
    d = {
        "smooth": torch.ones(experts, hidden, dtype=torch.float32, device=device),
        "y": per_token("randn", 22, t0 * topk, (t0 + tokens) * topk, hidden, torch.bfloat16, seed + 1, gen_device, device),
    }
    if with_hidden:
        d["hidden"] = per_token("randn", 21, t0, t0 + tokens, hidden, torch.bfloat16, seed, gen_device, device)
    return d


def gate_bytes(tokens: int, experts: int, topk: int) -> int:
    return tokens * experts * 4 + experts * 4 + tokens * topk * 8


def scatter_bytes(tokens: int, hidden: int, experts: int, topk: int) -> int:
    """token rows read once, smooth table once, int8 rows + scale + row2tok written, ids + weights read."""
    rows = tokens * topk
    return tokens * hidden * 2 + experts * hidden * 4 + rows * hidden + 8 * rows + 8 * tokens * topk


def gather_bytes(tokens: int, hidden: int, topk: int, accumulate: bool) -> int:
    rows = tokens * topk
    return rows * hidden * 2 + 4 * rows + tokens * hidden * 2 * (2 if accumulate else 1)


# ----------------------------------------------------------------------------------------------
# The five benchmark configurations
# ----------------------------------------------------------------------------------------------
CONFIGS = {
    1: dict(name="norm_quant_256x4096", tokens=256, hidden=4096),
    2: dict(name="rope_kv_4096", tokens=4096, q_heads=32, kv_heads=8, head_dim=128, max_pos=8192, block_size=16, num_blocks=2048),
    3: dict(name="deepseek_route_dispatch_8192", tokens=8192, experts=256, groups=8, topk_group=4, topk=8, scaling=2.5, hidden=7168),
    4: dict(name="llama70b_prefill_chunk_32768", tokens=32768, hidden=8192, q_heads=64, kv_heads=8, head_dim=128, max_pos=131072,
            block_size=16, num_blocks=2048),
    5: dict(name="token_sharded_chain_262144", tokens=262144, hidden=7168, experts=8, topk=2),
}


def chain5_bytes(tokens: int, hidden: int = 7168, experts: int = 8, topk: int = 2) -> Dict[str, int]:
    """Algorithmic bytes of the four kernels of configuration 5 for `tokens` tokens."""
    return {
        "norm_quant": norm_quant_bytes(tokens, hidden),
        "softmax_topk": gate_bytes(tokens, experts, topk) - experts * 4,
        "scatter": scatter_bytes(tokens, hidden, experts, topk),
        "gather": gather_bytes(tokens, hidden, topk, False),
    }
