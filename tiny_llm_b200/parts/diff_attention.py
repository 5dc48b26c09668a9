"""Differential attention over the paged cache.

Every head has two score maps, each a softmax attention of its own (own queries, own keys) over the SAME values;
the head's output is their difference, normalised:
    a_m = softmax(q_m k_m^T * scale, visible keys) v          m = 1, 2
    lam = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff    one number per layer
    o   = a_1 - lam * a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)     per head, no weight
The query matrix has heads * 2 * dim rows laid out head by head as [map 1, map 2], the key matrix
kv_heads * 2 * dim rows in the same way, the value matrix kv_heads * vdim rows; query head h reads key/value head
h // (heads / kv_heads).  The first `rot_dims` values of every query and key row are rotated pairwise (value 2i with
2i + 1) by position * f_i, with the frequencies of `RotaryPairs` below.  A key at position j is visible to a query
at position p iff j <= p, and, with `chunk`, iff both lie in the same chunk of that many positions counted from 0.

The cache holds two key rows per key/value head and token and one value row, whose size may differ from the key's.
Scores, softmax, lam, the difference and the norm are 32-bit; the two maps leave attention as float32 rows."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache import KVNeed
from ..weights import COMPUTE, FLOAT32, WeightSpec
from .feed_forward import scaled_matrix
from .registry import register_part


def scaled_pair_frequencies(rot_dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = base^(-2i / rot_dims), i < rot_dims / 2, in 32-bit.  `scaling` (factor, low, high, original) stretches
    the slow rotations as Llama 3.1 does: with the wavelength L = 2 pi / f, f stays where L < original / high,
    becomes f / factor where L > original / low, and between the two is the blend (1 - s) f / factor + s f with
    s = (original / L - low) / (high - low)."""
    i = torch.arange(rot_dims // 2, dtype=torch.float32)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float32), -2.0 * i / rot_dims)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        wavelength = 2.0 * math.pi / f
        s = (orig / wavelength - low) / (high - low)
        f = torch.where(wavelength < orig / high, f,
                        torch.where(wavelength > orig / low, f / factor, (1.0 - s) * f / factor + s * f))
    return f.contiguous()


class DiffAttention:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    MAPS = 2   # score maps per head; the difference of two is what the design is

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, scale: float,
                 diff: float, eps: float, rot_dims: int = 0, rot_base: float = 10000.0, rot_scaling: Optional[dict] = None,
                 chunk: Optional[int] = None, out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("differential attention does not read another layer call's cache")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads evenly")
        if rot_dims % 2 or rot_dims > key_dim:
            raise ValueError(f"{rot_dims} rotated values must be even and at most the key size {key_dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.rot_dims, self.rot_base, self.rot_scaling = rot_dims, float(rot_base), rot_scaling
        self.chunk = chunk
        self.out_scale = float(out_scale)
        self.q_dim = num_heads * self.MAPS * key_dim
        self.k_dim = num_kv_heads * self.MAPS * key_dim
        self.v_dim = num_kv_heads * value_dim
        self.w_qkv = self.w_o = self.freq = None
        self.lam = None

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.key_dim, None, value_dim=self.value_dim, key_rows=self.MAPS,
                      chunk=self.chunk)

    def weight_specs(self, prefix: str):
        h, kd = self.hidden_size, self.key_dim
        small = ("normal", 0.1)
        return [WeightSpec(prefix + "q", (self.q_dim, h), COMPUTE), WeightSpec(prefix + "k", (self.k_dim, h), COMPUTE),
                WeightSpec(prefix + "v", (self.v_dim, h), COMPUTE),
                WeightSpec(prefix + "lq1", (kd,), FLOAT32, init=small), WeightSpec(prefix + "lk1", (kd,), FLOAT32, init=small),
                WeightSpec(prefix + "lq2", (kd,), FLOAT32, init=small), WeightSpec(prefix + "lk2", (kd,), FLOAT32, init=small),
                WeightSpec(prefix + "o", (h, self.num_heads * self.value_dim), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.w_qkv = torch.cat([weights[prefix + n] for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)
        self.lam = [weights[prefix + n] for n in ("lq1", "lk1", "lq2", "lk2")]
        self.freq = scaled_pair_frequencies(self.rot_dims, self.rot_base, self.rot_scaling).to(self.w_o.device) \
            if self.rot_dims else None

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        maps, nh, nkv, kd, vd = self.MAPS, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        qkv = ctx.workspace.get("qkv", (t, self.q_dim + self.k_dim + self.v_dim), ctx.dtype)
        ops.linear(h, self.w_qkv, qkv, cluster_slices=True)
        ops.rope_pairs_kv_write(qkv, ctx.batch.positions, self.freq, self.rot_dims, nh * maps, nkv * maps, nkv, kd, vd,
                                cache.k, cache.v, cache.slot_mapping)
        per_map = ctx.workspace.get("attn_maps", (t, nh * maps * vd), torch.float32)
        ops.paged_attention_maps(qkv, nh, nkv, maps, kd, vd, cache.k, cache.v, cache.block_table, ctx.batch, per_map,
                                 self.scale, None, self.chunk)
        out = ctx.workspace.get("attn_out", (t, nh * vd), ctx.dtype)
        ops.diff_combine(per_map.view(t, nh, maps, vd), *self.lam, self.diff, self.eps, out)
        ops.linear(out, self.w_o, resid, accumulate=True)


register_part("mixer", "diff_attention", DiffAttention)
