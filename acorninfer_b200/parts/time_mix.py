"""Time mixing with a matrix state per head (the RWKV kind), as a mixer with per-request state.

Per token, from the mixer's input h and the input h' of the token before it in its request (zeros for a
request's first token), with a learned share ``mu_s`` per channel for each of s in r, k, v, g, w:
    x_s = h + (h' - h) * mu_s
    r, k, v = W_r x_r, W_k x_k, W_v x_v   (heads x dim each);   gate = silu(W_g x_g)
    decay = exp(-exp(W_w2 tanh(W_w1 x_w) + w0))                 per head and key channel, in (0, 1)
Per head, on a state S [dim, dim] that starts at zero, with a bonus u per key channel for the token itself:
    o = (S + diag(u) k v^T)^T r;      S = diag(decay) S + k v^T
then o / rms(o) per head, the heads side by side times ``norm`` times the gate, and the output projection.
Decays, gate, recurrence and the norm are float32, and so is the state: S of every head and the last input
row h' live in the request's state slot (one float32 vector).

The recurrence is the form of the delta rule's kernel that reads the state before the token's decay and
write (``ops.delta_rule(bonus32=...)``); the input row is kept by the convolution-memory kernel with two taps
(for rows of a single token by the blending kernel itself).  The one host-side value of a step that is read is
its longest row, which is 1 in every captured step.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, BuildContext, CacheNeeds, Mixer, StateNeeds, TensorSpec

_BLENDS = ("r", "k", "v", "g", "w")


@MIXERS.register("time_mix")
class TimeMix(Mixer):
    graph_safe = True

    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, dim: int, norm_eps: float,
                 decay_rank: int | None = None):
        """``decay_rank``: inner size of the decay's low-rank projection; None: taken from the checkpoint's
        tensors (give it when writing a model)."""
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.H, self.dim, self.eps, self.decay_rank = num_heads, dim, float(norm_eps), decay_rank
        self.state_s = num_heads * dim * dim                      # floats of S; the last input row follows

    def tensor_specs(self):
        C, W = self.H * self.dim, self.hidden_size
        specs = {f"mu.{s}": TensorSpec((W,), "blend") for s in _BLENDS}
        specs.update({s: TensorSpec((C, W)) for s in ("r", "k", "v", "g")})
        specs.update({"w1": TensorSpec((self.decay_rank, W)), "w2": TensorSpec((C, self.decay_rank)),
                      "w0": TensorSpec((C,), "decay_log"), "u": TensorSpec((self.H, self.dim), "bias"),
                      "norm": TensorSpec((C,), "norm"), "o": TensorSpec((W, C))})
        return specs

    def bind(self, tensors):
        t = tensors
        f32 = lambda x: x.to(torch.float32).contiguous()
        self.mu32 = f32(torch.stack([t[f"mu.{s}"] for s in _BLENDS]))
        self.w = {s: t[s].contiguous() for s in ("w1", "w2", "o")}
        # r, k, v, g read a blend each and are as large as one another: one grouped product, a blend's rows to its matrix
        self.w_rkvg = torch.stack([t[s] for s in ("r", "k", "v", "g")]).contiguous()
        self.w0_32, self.u32, self.norm32 = f32(t["w0"]), f32(t["u"]), f32(t["norm"])

    def cache_needs(self):
        return CacheNeeds(state=StateNeeds((self.state_s + self.hidden_size,)))

    def step_arrays(self):
        # where each blend's rows start among the rows of all blends: [0, T, 2T, 3T, 4T]
        import numpy as np
        return {"time_mix.blend_rows": lambda plan: (np.arange(5, dtype=np.int64) * plan.num_tokens).astype(np.int32)}

    def forward(self, x, inputs, cache):
        dt, w = self.ctx.dtype, self.w
        mixes = ops.token_shift(x, self.mu32, cache.state, self.state_s, inputs.token_row, inputs.row_start,
                                inputs.row_slot, update_single=True)
        if inputs.plan.max_q_len > 1:       # rows of one token had their row kept by the kernel above
            ops.conv_state_update(x, cache.state, self.state_s, inputs.row_start, inputs.row_slot, inputs.num_rows,
                                  self.hidden_size, 2, skip_single=True)
        T = x.shape[0]
        r, k, v, g = ops.grouped_gemm(mixes[:4].view(4 * T, self.hidden_size), None, self.w_rkvg,
                                      inputs.extra["time_mix.blend_rows"], 4 * T).view(4, T, -1).unbind(0)
        z = ops.linear(ops.linear(mixes[4], w["w1"], out_dtype=dt, act="tanh"), w["w2"], out_dtype=torch.float32)
        r32, k32, v32, decay, gate = ops.wkv_prep(r, k, v, g, z, self.w0_32, self.H)
        o = ops.delta_rule(r32, k32, v32, None, decay, cache.state, inputs.row_start, inputs.row_slot,
                           inputs.num_rows, bonus32=self.u32, longest_row=inputs.plan.max_q_len)
        y = ops.delta_out(o, gate, self.norm32, self.eps, dt)
        return ops.linear(y, w["o"], out_dtype=dt)
