"""Operations on the residual stream between blocks.

``InputInjection``: before pass t of a group of layers that runs several times with the same
weights, the stream is mixed with the embedding output again, r <- W [r; r0] + step[t]
(W [hidden, 2 hidden], the stream's columns first; step [times, hidden]).  The product takes
[r; r0] in the compute dtype and leaves the new stream in 32-bit.

``InputAdd``: the plain form of the same idea, r <- r + r0: the embedding output is added to the
stream, in 32-bit, together with whatever the block before left pending."""
from __future__ import annotations

from ..kernels import ops
from .base import ParamSpec, StreamOp, register_stream_op


class InputInjection(StreamOp):
    capturable = True
    needs_first = True

    def __init__(self, hidden_size, times):
        super().__init__()
        self.hidden_size, self.times = hidden_size, int(times)

    def param_specs(self):
        return {"in.weight": ParamSpec((self.hidden_size, 2 * self.hidden_size)),
                "step.weight": ParamSpec((self.times, self.hidden_size), role="vector", init="normal")}

    def forward(self, residual, pending, first, ctx, arg):
        if not 0 <= arg < self.times:
            raise ValueError(f"input injection: pass {arg} of {self.times}")
        both = ops.stream_concat(residual, pending, first, ctx.dtype)
        # (the pass's vector rides as the product's bias: added in 32-bit in its epilogue, or by a
        # kernel of its own behind the library's product)
        return ops.linear(both, self.w["in.weight"], self.w["step.weight"][arg], out_float32=True), None


register_stream_op("input_injection", InputInjection)


class InputAdd(StreamOp):
    capturable = True
    needs_first = True

    def __init__(self, hidden_size):
        super().__init__()
        self.hidden_size = hidden_size

    def forward(self, residual, pending, first, ctx, arg):
        return ops.stream_add_(residual, pending, first), None


register_stream_op("input_add", InputAdd)
