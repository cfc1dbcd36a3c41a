"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` in float32, one rounding at the end (``one_plus``: the stored
weight is the distance of ``w`` from one); and LayerNorm with
weight and bias: ``(x - mean) * rsqrt(var + eps) * w + b``, var the mean of the squared deviations.

Reference: ``RMSNorm`` in ``acorninfer/models/qwen3.py:50-60`` (the weight multiplies in
float32 before the cast) and the fused residual-add form in ``acorninfer/ops/rmsnorm.py:15-36``.
Here the residual stream itself stays in float32, so the fused form adds the incoming
delta to it without rounding.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, BuildContext, Norm, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, ctx: BuildContext, width: int, eps: float, tensor: str = "weight", one_plus: bool = False):
        """``tensor``: the weight's name relative to the part's prefix ("" where the prefix is the
        whole name).  ``one_plus``: the tensor holds ``w - 1`` (values around zero); the norm multiplies by
        ``1 + tensor``, the sum taken once, in float32, when the weight is bound."""
        self.ctx = ctx
        self.width = width
        self.eps = float(eps)
        self.tensor = tensor
        self.one_plus = bool(one_plus)
        self.weight32: torch.Tensor | None = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.width,), "norm_offset" if self.one_plus else "norm")}

    def bind(self, tensors):
        # Norm weights are held in float32 whatever they were stored as (widening is exact).
        w = tensors[self.tensor].to(torch.float32)
        self.weight32 = (w + 1.0 if self.one_plus else w).contiguous()

    def normed_add_norm(self, resid32, y, next_norm: "RMSNorm"):
        """resid32 += norm(y) (in place), and ``next_norm`` of the new stream in the activation dtype: this
        sublayer's output norm and the next sublayer's input norm in one kernel."""
        return ops.rmsnorm_add_norm(resid32, y, self.weight32, self.eps, next_norm.weight32, next_norm.eps)

    def normed_add(self, resid32, y, rounded=True):
        """resid32 += norm(y) (in place): the norm of a sublayer's *output*, added to the stream.
        Returns the new stream rounded to the activation dtype (None under a float32 engine, where the
        stream itself is read, or if ``rounded`` is off)."""
        return ops.rmsnorm_add(resid32, y, self.weight32, self.eps, rounded=rounded)

    def as_epilogue(self, resid32):
        return ops.AddNormEpilogue(resid32, self.weight32, self.eps)

    def forward(self, x32, out=None, rows=None):
        return ops.add_rmsnorm(x32, None, self.weight32, self.eps, self.ctx.dtype, row_idx=rows, out=out)

    def add_forward(self, resid32, delta, out=None, rows=None):
        return ops.add_rmsnorm(resid32, delta, self.weight32, self.eps, self.ctx.dtype, row_idx=rows, out=out)


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``(x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b`` in float32, one rounding.  ``tensor`` names
    the weight relative to the part's prefix and ``bias_tensor`` the bias (None: no bias)."""

    graph_safe = True
    accepts_pair = True           # add_forward takes an ``ops.DeltaPair`` (two results to add) as well

    def __init__(self, ctx: BuildContext, width: int, eps: float, tensor: str = "weight", bias_tensor: str | None = "bias"):
        self.ctx = ctx
        self.width = width
        self.eps = float(eps)
        self.tensor, self.bias_tensor = tensor, bias_tensor
        self.weight32: torch.Tensor | None = None
        self.bias32: torch.Tensor | None = None

    def tensor_specs(self):
        specs = {self.tensor: TensorSpec((self.width,), "norm")}
        if self.bias_tensor is not None:
            specs[self.bias_tensor] = TensorSpec((self.width,), "bias")
        return specs

    def bind(self, tensors):
        self.weight32 = tensors[self.tensor].to(torch.float32).contiguous()
        if self.bias_tensor is not None:
            self.bias32 = tensors[self.bias_tensor].to(torch.float32).contiguous()

    def forward(self, x32, out=None, rows=None):
        return ops.add_layernorm(x32, None, self.weight32, self.bias32, self.eps, self.ctx.dtype, row_idx=rows, out=out)

    def add_forward(self, resid32, delta, out=None, rows=None):
        return ops.add_layernorm(resid32, delta, self.weight32, self.bias32, self.eps, self.ctx.dtype, row_idx=rows, out=out)
