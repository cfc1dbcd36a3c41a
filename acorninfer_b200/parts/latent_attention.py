"""Attention whose keys and values are up-projections of one cached latent per token, as a mixer.

Per token: ``q = W_q h`` laid out head by head as [dim unrotated | rot rotated]; ``W_dkv h`` gives
``kv_rank`` entries that are RMS-normed into the latent ``c`` and ``rot`` entries that are rotated into
one key part ``kr`` shared by all heads.  Head a's key is ``[U_a c | kr]``, its value ``V_a c``
(``U_a``: rows a*dim.. of ``uk``, ``V_a``: rows a*vdim.. of ``uv``).  Only ``[c | kr]`` is cached: one
row of ``kv_rank + rot`` per token, no separate values.  Since ``qu . U_a c = (U_a^T qu) . c``, every
head attends over those rows directly with the query ``[U_a^T qu_a | qr_a]`` and gets
``sum_j p_j c_j``, which ``V_a`` maps to the head's output: one kv head of size ``kv_rank + rot`` whose
value rows are the first ``kv_rank`` entries of its key rows.  A sliding window and a learned sink per
head (a term exp(sink_a) in the softmax denominator, with no key and no value) are the attention
kernel's (``sink`` false: no sink); ``scale`` multiplies the whole score.  With ``q_rank`` the queries come
through a latent of their own: ``q = W_uq RMSnorm(W_dq h)`` (tensors ``dq``, ``dq.norm``, ``uq`` instead of ``q``).

A run that reads another run's cache (``cache.write`` false) has no ``dkv`` matrices: it computes
queries only, against the rows the other run wrote, with its own up-projections, window and sinks.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, BuildContext, CacheNeeds, KVNeeds, Mixer, TensorSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, ctx: BuildContext, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int,
                 kv_rank: int, scale: float, norm_eps: float, position: str | None, window: int | None = None,
                 own_cache: bool = True, q_rank: int | None = None, sink: bool = True):
        if window is not None and window < 1:
            raise ValueError(f"window must be >= 1 or None, got {window}")
        self.ctx = ctx
        self.hidden_size = hidden_size
        self.H, self.dim, self.rot, self.vdim, self.rank = num_heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.window, self.own_cache = float(scale), float(norm_eps), window, own_cache
        self.q_rank, self.sink = q_rank, bool(sink)
        self.w_dq = self.w_uq = self.q_norm32 = None
        self.position = ctx.positions[position] if position is not None else None
        if self.position is not None and self.position.head_dim != rot_dim:
            raise ValueError("position encoding was built for another rotated size")
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_norm32 = self.sink32 = None

    def tensor_specs(self):
        H, qd = self.H, self.dim + self.rot
        specs = {
            "uk": TensorSpec((H * self.dim, self.rank)),
            "uv": TensorSpec((H * self.vdim, self.rank)),
            "o": TensorSpec((self.hidden_size, H * self.vdim)),
        }
        if self.q_rank is None:
            specs["q"] = TensorSpec((H * qd, self.hidden_size))
        else:
            specs["dq"] = TensorSpec((self.q_rank, self.hidden_size))
            specs["dq.norm"] = TensorSpec((self.q_rank,), "norm")
            specs["uq"] = TensorSpec((H * qd, self.q_rank))
        if self.sink:
            specs["sink"] = TensorSpec((H,), "sink")
        if self.own_cache:
            specs["dkv"] = TensorSpec((self.rank + self.rot, self.hidden_size))
            specs["dkv.norm"] = TensorSpec((self.rank,), "norm")
        return specs

    def bind(self, tensors):
        if self.q_rank is None:
            parts = [tensors["q"]] + ([tensors["dkv"]] if self.own_cache else [])
            dtype = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
            self.w_in = torch.cat([p.to(dtype) for p in parts], dim=0).contiguous()
        else:
            # the query latent is normed before its up-projection: its product stands alone (float32 out, so
            # that the norm reads the accumulator), the cache rows' product beside it
            self.w_dq, self.w_uq = tensors["dq"].contiguous(), tensors["uq"].contiguous()
            self.q_norm32 = tensors["dq.norm"].to(torch.float32).contiguous()
            self.w_in = tensors["dkv"].contiguous() if self.own_cache else None
        # U_a^T per head: [H, rank, dim], so that the query side is a per-head product like the value side
        self.w_uk_t = tensors["uk"].view(self.H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].view(self.H, self.vdim, self.rank).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.sink32 = tensors["sink"].to(torch.float32).contiguous() if self.sink else None
        if self.own_cache:
            self.c_norm32 = tensors["dkv.norm"].to(torch.float32).contiguous()

    def cache_needs(self):
        return CacheNeeds(kv=KVNeeds(1, self.rank + self.rot, self.window, values=False))

    def _tile_tokens(self):
        return max(1, ops.LATENT_TILE_ROWS // self.H)

    def step_arrays(self):
        # the tensor-core kernel's tiles: (row, first token within the row) of every group of 64 // H tokens
        import numpy as np
        n = self._tile_tokens()

        def tiles(plan):
            t = [(r, q0) for r, length in enumerate(plan.row_lens) for q0 in range(0, length, n)]
            return np.asarray(t, np.int32).reshape(-1, 2)

        return {f"latent.tiles{n}": tiles}

    def forward(self, x, inputs, cache):
        if cache.write != self.own_cache:
            raise ValueError("latent attention: the schedule and the layer disagree on who writes the cache")
        g = inputs.groups[cache.group]
        T, H, dt = x.shape[0], self.H, self.ctx.dtype
        pos = self.position
        kv_rows = None
        if self.q_rank is None:
            proj = ops.linear(x, self.w_in, out_dtype=dt)
        else:
            cq = ops.add_rmsnorm(ops.linear(x, self.w_dq, out_dtype=torch.float32), None, self.q_norm32, self.eps, dt)
            proj = ops.linear(cq, self.w_uq, out_dtype=dt)
            kv_rows = ops.linear(x, self.w_in, out_dtype=dt) if cache.write else None
        qcat = torch.empty((T, H, self.rank + self.rot), dtype=dt, device=x.device)
        ops.latent_prep(proj, qcat, self.c_norm32, pos.inv_freq if pos is not None else _no_freq(x.device),
                        pos.magnitude if pos is not None else 1.0, inputs.positions, inputs.token_row, g.block_table,
                        g.page_base, cache.k_pages if cache.write else None, H, self.dim, self.rot, self.rank,
                        pos.rotary_dim if pos is not None else 0, self.eps, kv_rows=kv_rows)
        qu = proj[:, :H * (self.dim + self.rot)].view(T, H, self.dim + self.rot)[:, :, :self.dim]
        ops.head_linear(qu, self.w_uk_t, qcat[:, :, :self.rank])
        if ops.latent_attention_tc_supported(dt, H, self.rank + self.rot, self.rank, cache.k_pages.shape[2]):
            o = ops.latent_attention_tc(qcat, cache.k_pages, g.block_table, g.page_base, inputs.row_start, inputs.row_pos,
                                        inputs.extra[f"latent.tiles{self._tile_tokens()}"], self.sink32, self.scale,
                                        self.window, self.rank)
        else:       # float32, or sizes the tensor-core kernel does not take
            o = ops.attention_plain(qcat, qcat.stride(0), cache.k_pages, cache.k_pages, g.block_table, g.page_base,
                                    inputs.token_row, inputs.positions, T, H, 1, self.rank + self.rot, self.scale,
                                    self.window, value_dim=self.rank, sink32=self.sink32)
        v = torch.empty((T, H, self.vdim), dtype=dt, device=x.device)
        ops.head_linear(o.view(T, H, self.rank), self.w_uv, v)
        return ops.linear(v.view(T, H * self.vdim), self.w_o, out_dtype=dt)


_NO_FREQ: dict = {}


def _no_freq(device):
    if device not in _NO_FREQ:
        _NO_FREQ[device] = torch.zeros(0, dtype=torch.float32, device=device)
    return _NO_FREQ[device]
