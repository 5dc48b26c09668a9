"""Attention without softmax over a sliding window plus pooled blocks of older keys.

A query at position i sees the keys j with 0 <= i - j < window and, beside them, ONE key and value for every block
of `pool` positions that lies wholly before the window (block b = positions b pool .. b pool + pool - 1 is seen iff
b pool + pool - 1 <= i - window); the block's key and value are the means of its cached keys and values.  Tokens
that have left the window while their block is not yet complete enough to be seen are not seen at all.  The weight
of a visible key is not normalised over the keys:
    s = (q . k) scale;   s <- cap tanh(s / cap) when there is a cap;   weight = sigmoid(s + bias_h)
with one learned bias per query head (`<prefix>pb`).  Queries and keys are rotated by position on their first
`rot_dims` values (value i with value i + rot_dims / 2, angle p base^(-2i / rot_dims)).  With `rotate_values` the
values are rotated too, over their whole size (value m with m + value_dim / 2, angle j base^(-2m / value_dim)), are
cached so, and every head's output is turned back by the query's own position, so that a value contributes as
rotated by its distance from the query.

Cache: keys and values of single tokens in pages that go back to the pool once neither the window nor an incomplete
block can reach them, and a second, strided entry with one row per complete block.  Scores, weights and angles are
32-bit."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache import KVNeed
from ..weights import COMPUTE, FLOAT32, WeightSpec
from .feed_forward import scaled_matrix
from .registry import register_part


def half_frequencies(dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2: computed in 64-bit, kept in 32-bit."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(torch.float32).contiguous()


class PooledWindowAttention:
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 softcap: Optional[float] = None, window: Optional[int] = None, pool: Optional[int] = None,
                 rot_dims: int = 0, rot_base: float = 10000.0, rotate_values: bool = False, out_scale: float = 1.0,
                 shares_cache: bool = False):
        if shares_cache:
            raise ValueError("this attention does not read another layer call's cache")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads evenly")
        if rot_dims % 2 or rot_dims > key_dim:
            raise ValueError(f"{rot_dims} rotated values must be even and at most the key size {key_dim}")
        if rotate_values and value_dim % 2:
            raise ValueError(f"rotated values need an even value size, not {value_dim}")
        if pool is not None and window is None:
            raise ValueError("pooled blocks stand for keys behind a window; without a window every key is seen itself")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.softcap = float(scale), (None if softcap is None else float(softcap))
        self.window, self.pool = window, pool
        self.rot_dims, self.rot_base, self.rotate_values = rot_dims, float(rot_base), rotate_values
        self.out_scale = float(out_scale)
        self.q_dim, self.k_dim, self.v_dim = num_heads * key_dim, num_kv_heads * key_dim, num_kv_heads * value_dim
        self.w_qkv = self.w_o = self.head_bias = self.freq_k = self.freq_v = None

    def cache_need(self):
        # a token's page must outlive its block's completion as well as the window
        keep = None if self.window is None else max(self.window, self.pool or 1)
        tokens = KVNeed(self.num_kv_heads, self.key_dim, keep, value_dim=self.value_dim)
        if self.pool is None:
            return tokens
        return (tokens, KVNeed(self.num_kv_heads, self.key_dim, None, value_dim=self.value_dim, stride=self.pool))

    def weight_specs(self, prefix: str):
        h = self.hidden_size
        return [WeightSpec(prefix + "q", (self.q_dim, h), COMPUTE), WeightSpec(prefix + "k", (self.k_dim, h), COMPUTE),
                WeightSpec(prefix + "v", (self.v_dim, h), COMPUTE),
                WeightSpec(prefix + "pb", (self.num_heads,), FLOAT32, init=("normal", 1.0)),
                WeightSpec(prefix + "o", (h, self.num_heads * self.value_dim), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.w_qkv = torch.cat([weights[prefix + n] for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.head_bias = weights[prefix + "pb"]
        dev = self.w_o.device
        self.freq_k = half_frequencies(self.rot_dims, self.rot_base).to(dev) if self.rot_dims else None
        self.freq_v = half_frequencies(self.value_dim, self.rot_base).to(dev) if self.rotate_values else None

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        nh, nkv, kd, vd = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        tokens, blocks = cache if self.pool is not None else (cache, None)
        qkv = ctx.workspace.get("qkv", (t, self.q_dim + self.k_dim + self.v_dim), ctx.dtype)
        ops.linear(h, self.w_qkv, qkv, cluster_slices=True)
        ops.rope_halves_kv_write(qkv, ctx.batch.positions, self.freq_k, self.rot_dims, self.freq_v, nh, nkv, nkv, kd, vd,
                                 tokens.k, tokens.v, tokens.slot_mapping)
        if blocks is not None:
            ops.pool_kv_blocks(tokens.k, tokens.v, tokens.block_table, blocks.k, blocks.v, blocks.slot_mapping,
                               ctx.batch, self.pool)
        out = ctx.workspace.get("attn_out", (t, nh * vd), ctx.dtype)
        ops.window_pool_attention(qkv, nh, nkv, kd, vd, tokens.k, tokens.v, tokens.block_table,
                                  None if blocks is None else blocks.k, None if blocks is None else blocks.v,
                                  None if blocks is None else blocks.block_table, ctx.batch, out, self.scale,
                                  self.softcap, self.head_bias, self.window, self.pool, self.freq_v, workspace=ctx.workspace)
        ops.linear(out, self.w_o, resid, accumulate=True)


register_part("mixer", "pooled_window_attention", PooledWindowAttention)
