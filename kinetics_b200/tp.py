"""Tensor-parallel partition of the layer by KV head.

Rank r of `world` owns KV heads [r*Hkv/world, (r+1)*Hkv/world) with their query groups, the
matching rows of the fused QKV projection and columns of the output projection, and its slice of
the KV pages and page summaries.  Append, scoring, selection and attention never cross ranks.  The
layer has two exchanges: the sum of the o_proj partial results and, with the MLP split by
`shard_mlp`, the sum of the down_proj partial results; the residual is added once, after each sum.
Follows the weight split of LiteSys litesys/models/qwen_layer.py:354-379 and the two all-reduces of
litesys/models/qwen3_dist.py:111-112 and :120-121.
"""
from __future__ import annotations

import torch


def shard_range(num_kv_heads: int, rank: int, world: int):
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads do not split over {world} ranks")
    per = num_kv_heads // world
    return rank * per, (rank + 1) * per


def shard_wqkv(weight, bias, num_heads: int, num_kv_heads: int, head_dim: int, rank: int, world: int):
    """Rows of the fused [q | k | v] projection that belong to `rank` (bias may be None)."""
    g = num_heads // num_kv_heads
    lo, hi = shard_range(num_kv_heads, rank, world)
    q0, k0, v0 = 0, num_heads * head_dim, (num_heads + num_kv_heads) * head_dim
    rows = torch.cat([
        torch.arange(q0 + lo * g * head_dim, q0 + hi * g * head_dim),
        torch.arange(k0 + lo * head_dim, k0 + hi * head_dim),
        torch.arange(v0 + lo * head_dim, v0 + hi * head_dim),
    ])
    return weight[rows].contiguous(), (None if bias is None else bias[rows].contiguous())


def shard_wo(weight, num_heads: int, head_dim: int, rank: int, world: int):
    """Columns of the output projection that multiply this rank's heads."""
    per = num_heads // world * head_dim
    return weight[:, rank * per:(rank + 1) * per].contiguous()


def shard_mlp(up, gate, down, rank: int, world: int):
    """Column split of up/gate, row split of down (litesys/models/qwen_layer.py:366-379)."""
    per = up.shape[0] // world
    sl = slice(rank * per, (rank + 1) * per)
    return up[sl].contiguous(), gate[sl].contiguous(), down[:, sl].contiguous()
