"""Learned positions: a vector per position, added to the embeddings before the first block
(``ModelSpec.embedding_position``).  Positions count from 0 in every sequence; the table bounds
the length of a sequence, and a position outside it is reported through the status words."""
from __future__ import annotations

from ..kernels import ops
from .base import ParamSpec, PositionEncoding, register_position_encoding


class LearnedPositions(PositionEncoding):
    capturable = True

    def __init__(self, max_positions, hidden_size):
        super().__init__()
        self.max_positions, self.hidden_size = int(max_positions), int(hidden_size)

    def param_specs(self):
        return {"weight": ParamSpec((self.max_positions, self.hidden_size))}

    def add_to_embeddings(self, residual, ctx) -> None:
        ops.add_position_rows_(residual, self.w["weight"], ctx.positions)


register_position_encoding("learned_positions", LearnedPositions)
