"""Recurrent mixers: a state of fixed size per request instead of keys and values.

minGRU.  A gated recurrence whose gates read the current token only, so all gates of a portion come from one
matrix product and only the element-wise recurrence walks the tokens:
    z_t = sigmoid(Wz h_t + bz)                      how much of the candidate enters
    u_t = Wx h_t + bx;  c_t = u_t + 1/2 (u_t >= 0), sigmoid(u_t) (u_t < 0)      the candidate, always positive
    S_t = (1 - z_t) S_(t-1) + z_t c_t               element by element, S_(-1) = 0
    y_t = Wo (S_t * silu(Wg h_t))
The three input matrices are fused into one at load ([z | u | g] rows); the state is a float32 vector of `width`
values in the request's state slot, carried from step to step; biases, sigmoids and the recurrence are 32-bit."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateNeed
from ..weights import COMPUTE, FLOAT32, WeightSpec
from .feed_forward import scaled_matrix
from .registry import register_part


class MinGRU:
    graph_safe = True   # launches kernels only: a step through this part can be captured in a CUDA graph

    def __init__(self, hidden_size: int, width: int, out_scale: float = 1.0, shares_cache: bool = False):
        if shares_cache:
            raise ValueError("a recurrent mixer's state cannot be read by another layer call")
        self.hidden_size = hidden_size
        self.width = width
        self.out_scale = float(out_scale)
        self.w_in = self.w_o = self.bias_z = self.bias_u = None

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def weight_specs(self, prefix: str):
        w, h = self.width, self.hidden_size
        return [WeightSpec(prefix + "z", (w, h), COMPUTE), WeightSpec(prefix + "z.b", (w,), FLOAT32, init=("normal", 0.5)),
                WeightSpec(prefix + "x", (w, h), COMPUTE), WeightSpec(prefix + "x.b", (w,), FLOAT32, init=("normal", 0.5)),
                WeightSpec(prefix + "g", (w, h), COMPUTE), WeightSpec(prefix + "o", (h, w), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.w_in = torch.cat([weights[prefix + n] for n in ("z", "x", "g")], dim=0).contiguous()
        self.bias_z = weights[prefix + "z.b"]
        self.bias_u = weights[prefix + "x.b"]
        self.w_o = scaled_matrix(weights[prefix + "o"], self.out_scale)

    def forward(self, ctx, h, resid, cache) -> None:
        t = h.shape[0]
        zug = ctx.workspace.get("gru_in", (t, 3 * self.width), ctx.dtype)
        ops.linear(h, self.w_in, zug, cluster_slices=True)
        y = ctx.workspace.get("gru_out", (t, self.width), ctx.dtype)
        ops.min_gru_scan(zug, self.bias_z, self.bias_u, cache.state, ctx.batch, y, ctx.workspace)
        ops.linear(y, self.w_o, resid, accumulate=True)


register_part("mixer", "min_gru", MinGRU)
