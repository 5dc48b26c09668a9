"""Hooks: parts that rewrite the float32 stream right after the embedding, or the logits."""
from __future__ import annotations

from .. import ops
from ..weights import COMPUTE, WeightSpec
from .registry import register_part


class LearnedPositions:
    """A learned vector per position, added to the stream after the embedding: x_t += table[position_t].  The table
    is stored under the hook's own name with `max_positions` rows."""
    graph_safe = True

    def __init__(self, size: int, max_positions: int):
        self.size, self.max_positions = size, max_positions
        self.table = None

    def weight_specs(self, prefix: str):
        return [WeightSpec(prefix, (self.max_positions, self.size), COMPUTE)]

    def load(self, prefix: str, weights) -> None:
        self.table = weights[prefix]

    def forward(self, ctx, x) -> None:
        ops.embedding(ctx.batch.positions, self.table, x, accumulate=True)


register_part("hook", "learned_positions", LearnedPositions)
