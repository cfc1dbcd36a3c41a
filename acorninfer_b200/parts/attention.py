"""Grouped-query attention over the paged cache, as a mixer.

Per token: q/k/v projections (no bias), optional per-head RMSNorm of q and k (one weight
of head size shared by all heads), position encoding, K/V written to the request's
pages, causal attention of every query over the keys of its own request, output projection.
Reference: ``Qwen3Attention`` in
``acorninfer/models/qwen3.py:106-152`` and its decode form ``:154-233``; scale
``head_dim ** -0.5`` (``acorninfer/ops/paged_attention.py:147``); query head h uses kv head
``h // (nq / nkv)`` (``acorninfer/models/qwen3.py:98-103``).

Which earlier keys a query reads: all of them; the last ``window`` positions; those of its own
block of ``chunk`` positions (blocks counted from position 0 of the request); and, whatever the
rule, the request's first ``keep_first`` keys.  Options: value heads of a width of their own
(``value_dim``); values that are the keys as projected, before norm and rotation
(``values_from_keys``: no value matrix); a gate per head on the heads' outputs,
``sigmoid(W_g x)_h``, a function of the mixer's input (``head_gate``); biases on the q, k, v projections
(``bias``); a short causal convolution over time on every channel of q, k and v, directly after the
projection and before the norm (``conv_taps``; the last ``conv_taps - 1`` projected rows of a request
are its state, float32, in its state slot); a penalty on the distance to the key,
``score = q . k * scale - slope_h * (i - j)`` with ``slope_h = 2^(-slope_exponent * (h + 1) / heads)``
(``slope_exponent``); the q/k norm applied after the rotation instead of before it (``norm_after_rotation``) and
without weights (``qk_norm_weights`` false: the heads are only brought to unit root mean square); a learned sink per
head, a term ``exp(sink_h)`` in the softmax denominator that has no key and no value (``sink``); a cap on the scaled
scores, ``cap tanh(score / cap)`` (``softcap``).  A position encoding's factor on cos and sin (``magnitude``) is applied.

All sizes are parameters.  The q, k, v (and gate) matrices are concatenated when bound so that one
matrix product yields a token's whole row.  A run that reads another run's
cache (``cache.write`` false) computes queries only.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels import attention as attn_kernels
from .base import MIXERS, BuildContext, CacheNeeds, KVNeeds, Mixer, StateNeeds, TensorSpec

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
          "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "gate": "g_proj.weight",
          "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
          "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight", "sink": "sink"}


@MIXERS.register("attention")
class Attention(Mixer):
    graph_safe = True
    supports_epilogue = True
    adds_residual = True

    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: str | None, scale: float, qk_norm_eps: float | None = None,
                 window: int | None = None, chunk: int | None = None, keep_first: int = 0,
                 value_dim: int | None = None, values_from_keys: bool = False, head_gate: bool = False,
                 names: dict | None = None, bias: bool = False, conv_taps: int | None = None,
                 slope_exponent: float | None = None, norm_after_rotation: bool = False, qk_norm_weights: bool = True,
                 sink: bool = False, softcap: float | None = None):
        """``names``: the tensors' names relative to the part's prefix (keys q, k, v, o, q_norm, k_norm, gate,
        q_bias, k_bias, v_bias, q_conv, k_conv, v_conv, sink)."""
        if (norm_after_rotation or not qk_norm_weights) and (qk_norm_eps is None or conv_taps or bias):
            raise ValueError("a q/k norm after the rotation or without weights needs qk_norm_eps and plain projections")
        if not qk_norm_weights and not norm_after_rotation:
            raise ValueError("a q/k norm without weights is built for the norm after the rotation only")
        if softcap is not None and (not softcap > 0 or slope_exponent is not None):
            raise ValueError("softcap must be > 0 and does not go with a distance penalty")
        if conv_taps is not None and (conv_taps < 1 or values_from_keys):
            raise ValueError("conv_taps must be >= 1 or None, and needs value columns of their own")
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        for what, n in (("window", window), ("chunk", chunk)):
            if n is not None and n < 1:
                raise ValueError(f"{what} must be >= 1 or None, got {n}")
        if keep_first < 0:
            raise ValueError(f"keep_first must be >= 0, got {keep_first}")
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.nq, self.nkv, self.d = num_heads, num_kv_heads, head_dim
        self.dv = head_dim if value_dim is None else value_dim
        if values_from_keys and self.dv != head_dim:
            raise ValueError(f"values taken from the keys have the keys' width {head_dim}, not {self.dv}")
        self.values_from_keys, self.head_gate = values_from_keys, head_gate
        self.scale = float(scale)
        self.qk_norm_eps = qk_norm_eps
        self.window, self.chunk, self.keep_first = window, chunk, keep_first
        self.names = {**_NAMES, **(names or {})}
        self.position = ctx.positions[position] if position is not None else None
        if self.position is not None and self.position.head_dim != head_dim:
            raise ValueError("position encoding was built for another head size")
        # the plain arrangement [q | k | v] of equal head sizes, which the fused products take
        self.bias, self.taps = bool(bias), conv_taps
        self.slopes32 = None
        if slope_exponent is not None:
            self.slopes32 = torch.tensor([2.0 ** (-float(slope_exponent) * (h + 1) / num_heads) for h in range(num_heads)],
                                         dtype=torch.float64).to(torch.float32)
        self.channels = (num_heads + num_kv_heads) * head_dim + (0 if values_from_keys else num_kv_heads * self.dv)
        self.bias32 = self.conv32 = None
        self.norm_after, self.norm_weights, self.sink, self.softcap = bool(norm_after_rotation), bool(qk_norm_weights), bool(sink), softcap
        self.sink32 = None
        magnitude = getattr(self.position, "magnitude", 1.0) if self.position is not None else 1.0
        self.plain = (not (values_from_keys or head_gate or bias or conv_taps or self.norm_after or self.sink or softcap)
                      and self.norm_weights and magnitude == 1.0 and self.dv == head_dim)
        self.gate_col = (self.nq + self.nkv) * self.d + (0 if values_from_keys else self.nkv * self.dv)
        self.w_qkv = self.w_o = self.q_norm32 = self.k_norm32 = None

    def tensor_specs(self):
        n = self.names
        specs = {
            n["q"]: TensorSpec((self.nq * self.d, self.hidden_size)),
            n["k"]: TensorSpec((self.nkv * self.d, self.hidden_size)),
            n["o"]: TensorSpec((self.hidden_size, self.nq * self.dv)),
        }
        if not self.values_from_keys:
            specs[n["v"]] = TensorSpec((self.nkv * self.dv, self.hidden_size))
        if self.head_gate:
            specs[n["gate"]] = TensorSpec((self.nq, self.hidden_size))
        if self.qk_norm_eps is not None and self.norm_weights:
            specs[n["q_norm"]] = TensorSpec((self.d,), "norm")
            specs[n["k_norm"]] = TensorSpec((self.d,), "norm")
        if self.sink:
            specs[n["sink"]] = TensorSpec((self.nq,), "sink")
        rows = {"q": self.nq * self.d, "k": self.nkv * self.d, **({} if self.values_from_keys else {"v": self.nkv * self.dv})}
        for which, size in rows.items():
            if self.bias:
                specs[n[which + "_bias"]] = TensorSpec((size,), "bias")
            if self.taps:
                specs[n[which + "_conv"]] = TensorSpec((size, self.taps), "conv")
        return specs

    def bind(self, tensors):
        n = self.names
        parts = [tensors[n["q"]], tensors[n["k"]]]
        if not self.values_from_keys:
            parts.append(tensors[n["v"]])
        if self.head_gate:
            # padded with zero rows to a multiple of 8, so that a token's row keeps 16-byte alignment
            g = tensors[n["gate"]]
            pad = (-self.nq) % 8
            parts.append(torch.cat([g, g.new_zeros((pad, g.shape[1]))], dim=0) if pad else g)
        dtype = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        self.w_qkv = torch.cat([p.to(dtype) for p in parts], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.qk_norm_eps is not None and self.norm_weights:
            self.q_norm32 = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm32 = tensors[n["k_norm"]].to(torch.float32).contiguous()
        if self.sink:
            self.sink32 = tensors[n["sink"]].to(torch.float32).contiguous()
        which = ("q", "k") + (() if self.values_from_keys else ("v",))
        if self.bias:
            self.bias32 = torch.cat([tensors[n[w + "_bias"]].to(torch.float32) for w in which]).contiguous()
        if self.taps:
            self.conv32 = torch.cat([tensors[n[w + "_conv"]].to(torch.float32) for w in which], dim=0).contiguous()
        if self.slopes32 is not None:
            self.slopes32 = self.slopes32.to(self.w_o.device)

    def cache_needs(self):
        kv = KVNeeds(self.nkv, self.d, self.window, chunk=self.chunk, keep_first=self.keep_first,
                     value_dim=None if self.dv == self.d else self.dv)
        # the convolutions' memory: the last taps - 1 rows as projected (with their biases), float32
        state = StateNeeds(((self.taps - 1) * self.channels,)) if self.taps and self.taps > 1 and self.channels else None
        return CacheNeeds(kv=kv, state=state)

    def step_arrays(self):
        return attn_kernels.STEP_ARRAYS

    def fusable(self, num_rows):
        # (the options only change what runs between the two products, which take the fused forms either way)
        return (self._rows_fuse(num_rows) and self.w_qkv.dtype == torch.bfloat16
                and self.w_o.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and (self.nq * self.d) % 8 == 0)

    def _rows_fuse(self, num_rows):
        widths = ((self.nq + 2 * self.nkv) * self.d, self.hidden_size)         # of the q/k/v product and of the o product
        return ops.fused_rows_ok(num_rows, self.ctx.dtype, widths, ops.device_sms(self.ctx.device))

    def inner(self, x, inputs, cache, out_scale: float = 1.0, out=None):
        """Everything before the output projection: the heads' outputs [T, nq * dv] (gated, times ``out_scale``),
        into ``out`` if given (rows of a wider buffer)."""
        g = inputs.groups[cache.group]
        pos = self.position
        rows = x.x.shape[0] if isinstance(x, ops.NormedRows) else x.shape[0]
        proj = None                 # the projected rows where the queries do not stay among them
        if (self.plain and pos is not None and self.w_qkv.dtype == torch.bfloat16 and ops.gemm_tc_supported(
                x.x if isinstance(x, ops.NormedRows) else x, self.w_qkv)
                and self._rows_fuse(rows)
                and ops.rope_kv_fusable(rows, self.ctx.dtype, self.d, pos.rotary_dim, pos.interleaved)):
            # few rows or very many, head size 128: norm, rotation and the cache write are the epilogue of the product
            qkv = ops.gemm_tc_qkv_rope(x, self.w_qkv, ops.RopeKvEpilogue(
                inputs.positions, inputs.token_row, g.block_table, g.page_base,
                cache.k_pages if cache.write else None, cache.v_pages if cache.write else None,
                self.q_norm32, self.k_norm32, pos.inv_freq, self.nq, self.nkv,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                cos_sin=pos.table(inputs) if rows > ops.GEMM_TC_MAX_ROWS and hasattr(pos, "table") else None))
        elif self.bias or self.taps:
            if not cache.write:
                raise ValueError("attention: biased or convolved projections need a cache of the run's own")
            proj = ops.linear(x, self.w_qkv, out_dtype=self.ctx.dtype)
            qkv = torch.empty((rows, self.nq * self.d), dtype=self.ctx.dtype, device=proj.device)      # the queries
            conv = None
            if self.taps:
                conv = ops.ShortConv(self.conv32, cache.state if self.taps > 1 else proj.new_zeros((1, 0), dtype=torch.float32),
                                     0, inputs.row_start, inputs.row_slot, update_single=True)
            ops.qk_rope_kv(proj, self.q_norm32, self.k_norm32,
                           pos.inv_freq if pos is not None else _no_freq(self.ctx.device),
                           inputs.positions, inputs.token_row, g.block_table, g.page_base,
                           cache.k_pages, cache.v_pages, self.nq, self.nkv, self.d,
                           pos.rotary_dim if pos is not None else 0, pos.interleaved if pos is not None else False,
                           self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_kv=True,
                           value_dim=self.dv, bias32=self.bias32, conv=conv, q_out=qkv,
                           magnitude=getattr(pos, "magnitude", 1.0) if pos is not None else 1.0)
            if self.taps and self.taps > 1 and inputs.plan.max_q_len > 1:     # rows of one token shifted their memory above
                ops.conv_state_update(proj, cache.state, 0, inputs.row_start, inputs.row_slot, inputs.num_rows,
                                      self.channels, self.taps, bias32=self.bias32, skip_single=True)
        else:
            qkv = ops.linear(x, self.w_qkv, out_dtype=self.ctx.dtype)
            ops.qk_rope_kv(qkv, self.q_norm32, self.k_norm32,
                           pos.inv_freq if pos is not None else _no_freq(self.ctx.device),
                           inputs.positions, inputs.token_row, g.block_table, g.page_base,
                           cache.k_pages, cache.v_pages, self.nq, self.nkv, self.d,
                           pos.rotary_dim if pos is not None else 0, pos.interleaved if pos is not None else False,
                           self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_kv=cache.write,
                           value_dim=self.dv, values_from_keys=self.values_from_keys,
                           magnitude=getattr(pos, "magnitude", 1.0) if pos is not None else 1.0,
                           norm_after=self.norm_after)
        heads = attn_kernels.paged_attention(qkv, inputs, g, cache, self.nq, self.nkv, self.d, self.scale, self.window,
                                             chunk=self.chunk, keep_first=self.keep_first, value_dim=self.dv,
                                             slopes32=self.slopes32, sink32=self.sink32, softcap=self.softcap)
        if self.head_gate or out_scale != 1.0 or out is not None:
            gate_rows = qkv if proj is None else proj
            return ops.head_gate(heads, gate_rows[:, self.gate_col:] if self.head_gate else None, self.nq, out_scale, out=out)
        return heads

    def forward(self, x, inputs, cache, epilogue=None, residual32=None):
        return ops.linear(self.inner(x, inputs, cache), self.w_o, out_dtype=self.ctx.dtype, epilogue=epilogue,
                          residual32=residual32 if epilogue is None else None)


_NO_FREQ: dict = {}


def _no_freq(device):
    if device not in _NO_FREQ:
        _NO_FREQ[device] = torch.zeros(0, dtype=torch.float32, device=device)
    return _NO_FREQ[device]
