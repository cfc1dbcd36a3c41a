"""A routed mixture of small SwiGLU experts, some of which are the identity, as a feed-forward.

Router logits ``z = W_router h`` over ``experts + identity`` outputs, in float32; scores
``s = softmax(z)``; experts are ranked by ``s + correction``.  Neighbouring outputs form ``groups`` groups of
equal size; a group is ranked by the best ranking value inside it, and outputs outside the ``keep`` best
groups are out of the running whatever their value.  The ``top`` best-ranked outputs are taken, each
weighted by its own ``s`` (the correction only ranks; the weights are left as they are, not rescaled to
sum to one).  The last ``identity`` outputs own no tensors and pass their input through.  A real expert is ``down(silu(gate h) * (up h))``.  The result is the weighted
sum over the chosen.

Options: no correction (``correction`` false: experts are ranked by their scores alone); the chosen outputs'
scores divided by their sum (``normalize``); experts of the capped form (``activation="capped_swish"`` with
``limit`` L: ``g = min(gate h, L), u = clamp(up h, -L, L), down(g sigmoid(1.702 g) (u + 1))``); a shared expert of
the same form (``shared_size``, ``shared_limit``; tensors ``shared.gate`` / ``up`` / ``down``) that every token
takes, added to the weighted sum.

On the device: the router's choice (one kernel), the (token, choice) pairs grouped by expert (one
kernel), one product per expert over its own rows for gate/up (SwiGLU in its epilogue on the tensor-core
kernel) and for down (a kernel each, walking the per-expert offsets on the device: nothing of the routing
is read on the host), and the weighted sum in the order of the choices, which also norms the result and
adds it to the stream when the block asks.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, BuildContext, FeedForward, TensorSpec


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, ctx: BuildContext, hidden_size: int, expert_size: int, num_experts: int, num_identity: int,
                 top: int, groups: int = 1, keep: int = 1, correction: bool = True, normalize: bool = False,
                 activation: str = "silu", limit: float = 0.0, shared_size: int | None = None,
                 shared_limit: float | None = None):
        if activation not in ("silu", "capped_swish"):
            raise ValueError(f"expert activation must be 'silu' or 'capped_swish', got {activation!r}")
        self.correction, self.normalize, self.activation, self.limit = bool(correction), bool(normalize), activation, float(limit)
        self.shared_size, self.shared_limit = shared_size, float(shared_limit if shared_limit is not None else limit)
        self.w_shared_gu = self.w_shared_down = None
        n = num_experts + num_identity
        if n < 1 or n % groups or not (1 <= keep <= groups) or top > keep * (n // groups):
            raise ValueError(f"{n} router outputs do not split into {groups} groups of which {keep} hold {top} choices")
        self.ctx = ctx
        self.hidden_size, self.ff = hidden_size, expert_size
        self.E, self.I, self.top, self.groups, self.keep = num_experts, num_identity, top, groups, keep
        self.w_router = self.correction32 = self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        n = self.E + self.I
        specs = {"router": TensorSpec((n, self.hidden_size))}
        if self.correction:
            specs["correction"] = TensorSpec((n,), "bias")
        if self.shared_size:
            specs["shared.gate"] = TensorSpec((self.shared_size, self.hidden_size))
            specs["shared.up"] = TensorSpec((self.shared_size, self.hidden_size))
            specs["shared.down"] = TensorSpec((self.hidden_size, self.shared_size))
        for e in range(self.E):
            specs[f"e{e}.gate"] = TensorSpec((self.ff, self.hidden_size))
            specs[f"e{e}.up"] = TensorSpec((self.ff, self.hidden_size))
            specs[f"e{e}.down"] = TensorSpec((self.hidden_size, self.ff))
        return specs

    def bind(self, tensors):
        t = tensors
        # Under a bfloat16 engine the router's matrix stays as stored: a product of two bfloat16 numbers is
        # exact in float32, so the tensor-core product with float32 accumulation is the float32 computation
        # on the rounded input, up to the order of the sum.
        self.w_router = t["router"].contiguous()
        self.correction32 = t["correction"].to(torch.float32).contiguous() if self.correction else \
            torch.zeros(self.E + self.I, dtype=torch.float32, device=self.w_router.device)
        if self.shared_size:
            g, u = t["shared.gate"], t["shared.up"]
            dtype = g.dtype if g.dtype == u.dtype else torch.float32
            self.w_shared_gu = torch.cat([g.to(dtype), u.to(dtype)], dim=0).contiguous()       # [gate | up]
            self.w_shared_down = t["shared.down"].contiguous()
        if self.E:
            mats = [t[f"e{e}.{n}"] for e in range(self.E) for n in ("gate", "up", "down")]
            dtype = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
            # gate and up rows in turns (row 2i: gate of output i, row 2i + 1: its up row): a thread of the grouped
            # product's epilogue then holds both and applies SwiGLU itself
            self.w_gate_up = torch.stack([torch.stack([t[f"e{e}.gate"].to(dtype), t[f"e{e}.up"].to(dtype)], dim=1)
                                          .reshape(2 * self.ff, self.hidden_size) for e in range(self.E)]).contiguous()
            self.w_down = torch.stack([t[f"e{e}.down"].to(dtype) for e in range(self.E)]).contiguous()   # [E, width, ff]

    adds_normed_residual = True     # ``forward(..., add_normed=(resid32, norm))`` adds the normed result to the stream itself

    def forward(self, x, inputs, add_normed=None):
        T = x.shape[0]
        z = ops.linear(x, self.w_router, out_dtype=torch.float32)
        idx, wts = ops.moe_route(z, self.correction32, self.top, self.groups, self.keep, normalize=self.normalize)
        offsets, slot_of, slot_token = ops.moe_plan(idx, self.E + self.I)
        slots = T * self.top
        if self.E:
            w_gu = self.w_gate_up if self.w_gate_up.dtype == x.dtype else self.w_gate_up.to(x.dtype)
            w_dn = self.w_down if self.w_down.dtype == x.dtype else self.w_down.to(x.dtype)
            hidden = ops.grouped_gemm(x, slot_token, w_gu, offsets, slots, swiglu_pairs=True, activation=self.activation,
                                      limit=self.limit)
            y = ops.grouped_gemm(hidden, None, w_dn, offsets, slots)
        else:
            y = x
        shared = None
        if self.shared_size:
            gu = ops.linear(x, self.w_shared_gu, out_dtype=self.ctx.dtype)
            shared = ops.linear(ops.swiglu(gu, activation=self.activation, limit=self.shared_limit), self.w_shared_down,
                                out_dtype=self.ctx.dtype)
        if add_normed is not None:
            resid32, norm = add_normed
            return ops.moe_combine(y, x, slot_of, idx, wts, self.E, resid32=resid32, weight32=norm.weight32, eps=norm.eps,
                                   extra=shared)
        return ops.moe_combine(y, x, slot_of, idx, wts, self.E, extra=shared)
