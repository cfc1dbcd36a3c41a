"""A token's own side rows added to the stream inside a layer, as a layer extra.

A side table holds for every token of the vocabulary a row of ``layers * dim`` entries; layer ``index`` owns
columns ``index * dim .. (index + 1) * dim`` of it.  With x the stream after the layer's other sublayers:
    e = table[token, index * dim : (index + 1) * dim]
    g = gelu_tanh(W_gate x) * e                      (the tanh form of gelu)
    y = W_proj g;     x += y / sqrt(mean(y^2) + eps) * norm
The table is one tensor shared by all layers (its name is given whole); gate, proj and norm are the layer's
own.  A layer that runs several times uses the same columns every time.  The norm and the sum are float32.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import LAYER_EXTRAS, BuildContext, LayerExtra, TensorSpec


@LAYER_EXTRAS.register("token_side")
class TokenSide(LayerExtra):
    graph_safe = True

    def __init__(self, ctx: BuildContext, hidden_size: int, vocab_size: int, dim: int, index: int, table_width: int,
                 eps: float, table: str, names: dict):
        """``table``: the side table's whole name; ``names``: whole names of the layer's gate, proj and norm."""
        if dim < 1 or index < 0 or (index + 1) * dim > table_width:
            raise ValueError(f"token side: columns {index * dim}..{(index + 1) * dim} lie outside a table of {table_width}")
        self.ctx, self.hidden_size, self.vocab_size = ctx, hidden_size, vocab_size
        self.dim, self.index, self.table_width, self.eps = dim, index, table_width, float(eps)
        self.table_name, self.names = table, dict(names)
        self.table = self.w_gate = self.w_proj = self.norm32 = None

    def tensor_specs(self):
        return {self.table_name: TensorSpec((self.vocab_size, self.table_width)),
                self.names["gate"]: TensorSpec((self.dim, self.hidden_size)),
                self.names["proj"]: TensorSpec((self.hidden_size, self.dim)),
                self.names["norm"]: TensorSpec((self.hidden_size,), "norm")}

    def bind(self, tensors):
        self.table = tensors[self.table_name].contiguous()
        self.w_gate = tensors[self.names["gate"]].contiguous()
        self.w_proj = tensors[self.names["proj"]].contiguous()
        self.norm32 = tensors[self.names["norm"]].to(torch.float32).contiguous()

    def forward(self, resid32, rows, inputs, defer: bool = False):
        """``defer``: the normed sum is not taken here but handed back (``ops.NormedPending``) for the kernel of
        the norm that follows."""
        dt = self.ctx.dtype
        g = ops.side_gate_linear(rows, self.w_gate, inputs.token_ids, self.table, self.index * self.dim)
        y = ops.linear(g, self.w_proj, out_dtype=dt)
        pending = ops.NormedPending(y, self.norm32, self.eps)
        if defer:
            return pending
        pending.settle(resid32)
        return None
