"""What opens a pass of a span of layers that runs several times in a row.

``mix_in``: ``x <- W_in [x; x0] + step[n]`` with x the stream as the pass finds it, x0 the stream as it entered the
model's first layer (the token rows), ``W_in`` [width, 2 width] (x's columns first) and ``step`` [passes, width] a
learned vector per pass, n = 0, 1, ...  The product reads both streams rounded to the activation dtype and keeps its
float32 sums, to which the pass's vector is added in float32: the result is the new stream.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import PASS_ENTRIES, BuildContext, PassEntry, TensorSpec


@PASS_ENTRIES.register("mix_in")
class MixIn(PassEntry):
    graph_safe = True

    def __init__(self, ctx: BuildContext, width: int, passes: int, names: dict | None = None):
        self.ctx, self.width, self.passes = ctx, width, passes
        self.names = {"in": "in", "step": "step", **(names or {})}
        self.w_in = self.step32 = None

    def tensor_specs(self):
        return {self.names["in"]: TensorSpec((self.width, 2 * self.width)),
                self.names["step"]: TensorSpec((self.passes, self.width))}

    def bind(self, tensors):
        self.w_in = tensors[self.names["in"]].contiguous()
        self.step32 = tensors[self.names["step"]].to(torch.float32).contiguous()

    def forward(self, resid32, entered32, pass_index, inputs):
        if not (0 <= pass_index < self.passes):
            raise ValueError(f"pass {pass_index} of {self.passes}")
        both = ops.pair_rows(resid32, entered32, self.ctx.dtype)
        y32 = ops.linear(both, self.w_in, out_dtype=torch.float32)
        return ops.add_row(y32, self.step32[pass_index])
