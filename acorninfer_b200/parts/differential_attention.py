"""Differential attention over the paged cache, as a mixer.

A query head holds two score maps side by side, ``[map 1 | map 2]`` of ``dim`` entries each, and so does a key
head; value heads (``value_dim`` wide) are shared by both maps.  With ``a1``, ``a2`` the two maps' attention
outputs (each an ordinary softmax over the visible keys of ``softcap tanh(q_a . k_a scale / softcap)``),

    lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff          (one number for the layer)
    o = unit_rms(a1 - lambda a2) * (1 - diff)                           (per head, over its value entries)
    out = W_o (o * sigmoid(W_g x))                                      (a gate per output entry, from the mixer's input)

The q, k, v projections have biases; positions do not enter the scores; a query reads the last ``window``
positions (or all).  Query head h uses key/value head ``h // (heads / kv_heads)``.

On the device: one product gives ``[q | k | v | gate]``; the kernel between projection and cache adds the biases
and writes k and v into the pages (a key head is a row of ``2 dim``); the attention kernels run the ``2 heads``
(head, map) pairs as heads of their own over key rows of ``2 dim`` (a pair is scored against its map's half of
the key row), which gives a1 and a2 side by side; one kernel forms ``o``, norms and gates it; the output product
follows.  ``lambda`` is evaluated once, in float64, when the weights are bound.

Key rows of 128 under bfloat16 (``spread``): the query matrix is bound with a pair's rows laid out over the whole
key row, zeros outside its map's half, so that the product itself yields the pairs' queries as heads of 128 and
the tcgen05 prefill kernel, which takes its queries by TMA, serves the layer (the query product doubles: about a
fortieth of a layer's multiply-adds at these sizes).
"""

from __future__ import annotations

import math

import torch

from ..kernels import attention as attn_kernels
from ..kernels import ops
from .base import MIXERS, BuildContext, CacheNeeds, KVNeeds, Mixer, TensorSpec

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
          "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    graph_safe = True
    supports_epilogue = True
    adds_residual = True

    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, value_dim: int,
                 scale: float, diff: float, norm_eps: float, softcap: float | None = None, window: int | None = None,
                 bias: bool = True, names: dict | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if window is not None and window < 1:
            raise ValueError(f"window must be >= 1 or None, got {window}")
        if softcap is not None and not softcap > 0:
            raise ValueError(f"softcap must be > 0 or None, got {softcap}")
        self.ctx, self.hidden_size = ctx, hidden_size
        self.H, self.G, self.d, self.dv = num_heads, num_kv_heads, dim, value_dim
        self.scale, self.diff, self.eps, self.softcap, self.window = float(scale), float(diff), float(norm_eps), softcap, window
        self.bias = bool(bias)
        self.names = {**_NAMES, **(names or {})}
        self.w_in = self.w_o = self.bias32 = None
        self.lam = None
        # the pairs' queries laid out over the whole key row by the product itself: where the tcgen05 kernel can take them
        self.spread = ctx.dtype == torch.bfloat16 and 2 * dim == 128 and value_dim == 128
        self.q_cols = (2 if self.spread else 1) * self.H * 2 * dim

    def tensor_specs(self):
        n, W = self.names, self.hidden_size
        specs = {n["q"]: TensorSpec((self.H * 2 * self.d, W)), n["k"]: TensorSpec((self.G * 2 * self.d, W)),
                 n["v"]: TensorSpec((self.G * self.dv, W)), n["gate"]: TensorSpec((self.H * self.dv, W)),
                 n["o"]: TensorSpec((W, self.H * self.dv))}
        for which in ("lq1", "lk1", "lq2", "lk2"):
            specs[n[which]] = TensorSpec((self.d,), "lambda_part")
        if self.bias:
            specs[n["q_bias"]] = TensorSpec((self.H * 2 * self.d,), "bias")
            specs[n["k_bias"]] = TensorSpec((self.G * 2 * self.d,), "bias")
            specs[n["v_bias"]] = TensorSpec((self.G * self.dv,), "bias")
        return specs

    def bind(self, tensors):
        n = self.names
        parts = [tensors[n[w]] for w in ("q", "k", "v", "gate")]
        dtype = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        biases = [tensors[n[w + "_bias"]].to(torch.float32) for w in ("q", "k", "v")] if self.bias else None
        if self.spread:
            parts[0] = self._spread_rows(parts[0])
            if biases:
                biases[0] = self._spread_rows(biases[0])
        self.w_in = torch.cat([p.to(dtype) for p in parts], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if biases:
            self.bias32 = torch.cat(biases).contiguous()
        l64 = {w: tensors[n[w]].to(torch.float64).cpu() for w in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((l64["lq1"] * l64["lk1"]).sum())) - math.exp(float((l64["lq2"] * l64["lk2"]).sum())) + self.diff

    def _spread_rows(self, t):
        """Rows [H, 2, dim] of a query tensor as [H, 2, 2 dim]: pair (h, a) keeps its rows at a dim .. and zeros elsewhere."""
        d = self.d
        src = t.reshape(self.H, 2, d, *t.shape[1:])
        out = src.new_zeros((self.H, 2, 2 * d, *t.shape[1:]))
        for a in range(2):
            out[:, a, a * d:(a + 1) * d] = src[:, a]
        return out.reshape(self.H * 2 * 2 * d, *t.shape[1:])

    def cache_needs(self):
        return CacheNeeds(kv=KVNeeds(self.G, 2 * self.d, self.window, value_dim=None if self.dv == 2 * self.d else self.dv))

    def step_arrays(self):
        return attn_kernels.STEP_ARRAYS

    def fusable(self, num_rows):
        widths = (self.w_in.shape[0], self.hidden_size)                         # of the first and of the output product
        return (ops.fused_rows_ok(num_rows, self.ctx.dtype, widths, ops.device_sms(self.ctx.device))
                and self.w_in.dtype == torch.bfloat16 and self.w_o.dtype == torch.bfloat16
                and self.hidden_size % 8 == 0 and (self.H * self.dv) % 8 == 0)

    def forward(self, x, inputs, cache, epilogue=None, residual32=None):
        if not cache.write:
            raise ValueError("differential attention keeps a cache of its own")
        g = inputs.groups[cache.group]
        D = 2 * self.d
        proj = ops.linear(x, self.w_in, out_dtype=self.ctx.dtype)
        nq = 2 * self.H if self.spread else self.H          # query heads of a key row's width in a projected row
        q = torch.empty((proj.shape[0], nq * D), dtype=self.ctx.dtype, device=proj.device)
        ops.qk_rope_kv(proj, None, None, _no_freq(self.ctx.device), inputs.positions, inputs.token_row, g.block_table,
                       g.page_base, cache.k_pages, cache.v_pages, nq, self.G, D, 0, False, 0.0, write_kv=True,
                       value_dim=self.dv, bias32=self.bias32, q_out=q)
        # the 2 H (head, map) pairs as heads over key rows of 2 dim: a1 and a2 of every head side by side
        pairs = attn_kernels.paged_attention(q, inputs, g, cache, 2 * self.H, self.G, D, self.scale, self.window,
                                             value_dim=self.dv, softcap=self.softcap, maps=1 if self.spread else 2)
        gate_col = self.q_cols + self.G * (D + self.dv)
        o = ops.diff_combine(pairs, proj[:, gate_col:], self.H, self.dv, self.lam, 1.0 - self.diff, self.eps)
        return ops.linear(o, self.w_o, out_dtype=self.ctx.dtype, epilogue=epilogue,
                          residual32=residual32 if epilogue is None else None)


_NO_FREQ: dict = {}


def _no_freq(device):
    if device not in _NO_FREQ:
        _NO_FREQ[device] = torch.zeros(0, dtype=torch.float32, device=device)
    return _NO_FREQ[device]
