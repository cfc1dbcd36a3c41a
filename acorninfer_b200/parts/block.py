"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``x += mixer(norm_m(x)); x += feed_forward(norm_f(x))``
(``Qwen3Block`` in ``acorninfer/models/qwen3.py:399-410``).  The residual stream is float32;
each sum is fused into the norm that follows it, so a block takes ``(resid32, delta)``
where ``delta`` is what the previous block still has to add, and returns the same pair.  A layer may have
no feed-forward (the block is then its mixer's half alone).

``outnorm``: ``x += norm_m(mixer(x)); x += norm_f(feed_forward(x))``: the sublayers read the
stream itself and only their outputs are normed (Kogonex).  The sums are done here, in float32, by
the kernel that norms the output; it also hands on the stream rounded to the activation dtype, which
is what the next sublayer reads (``RoundedRows``).  A layer may have no feed-forward.

``parallel``: ``h = norm(x); x += mixer(h) + feed_forward(h)``: one norm, both sublayers read its
output.  Both results are added in float32: by the product that made them where it can add into the
stream itself, else by the norm kernel of the next block (``DeltaPair``).  A layer may have no feed-forward.

``sandwich``: ``x += norm_mo(mixer(norm_mi(x))); x += norm_fo(feed_forward(norm_fi(x)))``: a norm before and
after every sublayer (norms ``mixer_in``, ``mixer_out``, ``feed_forward_in``, ``feed_forward_out``), the sums in
float32 in the kernel that norms a sublayer's output, which where it can also applies the norm the next
sublayer reads the stream through.  A layer may have no feed-forward; an extra named ``side`` (a sublayer that
adds to the stream itself, such as a token's side rows) runs last.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BLOCKS, Block


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, ctx, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        missing = ({"mixer", "feed_forward"} if feed_forward is not None else {"mixer"}) - set(norms)
        if missing:
            raise ValueError(f"prenorm block needs norms named 'mixer' and 'feed_forward'; missing {sorted(missing)}")

    def _fuses(self, num_rows):
        return (self.feed_forward is not None and self.mixer.supports_epilogue and self.feed_forward.supports_epilogue
                and self.mixer.fusable(num_rows) and self.feed_forward.fusable(num_rows))

    def first_norm(self, num_rows):
        return self.norms["mixer"] if self._fuses(num_rows) else None

    def forward(self, resid32, delta, inputs, cache, next_norm=None):
        # With few rows on the tensor-core path, each residual sum and the norm after it are done
        # by the product before them (no kernel of their own); otherwise by the fused norm kernel.
        fuse = self._fuses(inputs.num_tokens)
        if isinstance(delta, ops.RoundedRows):          # the block before added its result itself
            delta = None
        h = delta if isinstance(delta, ops.NormedRows) else self.norms["mixer"].add_forward(resid32, delta)
        if self.feed_forward is None:
            if self.mixer.adds_residual:
                return resid32, self.mixer.forward(h, inputs, cache, residual32=resid32)
            return resid32, self.mixer.forward(h, inputs, cache)
        ep = self.norms["feed_forward"].as_epilogue(resid32) if fuse else None
        if ep is not None:
            h = self.mixer.forward(h, inputs, cache, epilogue=ep)
        else:
            # a part that can, adds its result to the residual stream itself (delta None)
            if self.mixer.adds_residual:
                delta = self.mixer.forward(h, inputs, cache, residual32=resid32)
            else:
                delta = self.mixer.forward(h, inputs, cache)
            h = self.norms["feed_forward"].add_forward(resid32, delta)
        ep = next_norm.as_epilogue(resid32) if (fuse and next_norm is not None) else None
        if ep is not None:
            return resid32, self.feed_forward.forward(h, inputs, epilogue=ep)
        if self.feed_forward.adds_residual:
            return resid32, self.feed_forward.forward(h, inputs, residual32=resid32)
        return resid32, self.feed_forward.forward(h, inputs)


@BLOCKS.register("outnorm")
class OutputNormBlock(Block):
    graph_safe = True

    def __init__(self, ctx, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        self.ctx = ctx
        want = {"mixer"} | ({"feed_forward"} if feed_forward is not None else set())
        if want - set(norms):
            raise ValueError(f"outnorm block needs norms named {sorted(want)}; missing {sorted(want - set(norms))}")

    def _rows(self, resid32, rounded):
        if self.ctx.dtype == torch.float32:
            return resid32
        return rounded if rounded is not None else ops.cast(resid32, self.ctx.dtype)

    def forward(self, resid32, delta, inputs, cache, next_norm=None):
        if isinstance(delta, ops.RoundedRows):
            h = self._rows(resid32, delta.x)
        else:
            if isinstance(delta, ops.NormedRows):
                raise ValueError("an outnorm block cannot follow a block that fused the next norm into its last product")
            if delta is not None:
                resid32.add_(delta)
            h = self._rows(resid32, None)
        h = self._rows(resid32, self.norms["mixer"].normed_add(resid32, self.mixer.forward(h, inputs, cache)))
        if self.feed_forward is not None:
            norm = self.norms["feed_forward"]
            if getattr(self.feed_forward, "adds_normed_residual", False) and hasattr(norm, "weight32"):
                # the feed-forward's last kernel norms its result and adds it to the stream itself
                h = self._rows(resid32, self.feed_forward.forward(h, inputs, add_normed=(resid32, norm)))
            else:
                h = self._rows(resid32, norm.normed_add(resid32, self.feed_forward.forward(h, inputs)))
        return resid32, ops.RoundedRows(h)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    graph_safe = True
    accepts_pair = True           # takes an ``ops.DeltaPair`` as the pending result of the block before

    def __init__(self, ctx, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        if "input" not in norms:
            raise ValueError("parallel block needs a norm named 'input'")
        if not getattr(norms["input"], "accepts_pair", False):
            raise ValueError("the norm of a parallel block must take two pending results (accepts_pair)")

    def forward(self, resid32, delta, inputs, cache, next_norm=None):
        if isinstance(delta, ops.RoundedRows):          # the block before added its result itself
            delta = None
        if isinstance(delta, ops.NormedRows):
            raise ValueError("a parallel block cannot follow a block that fused the next norm into its last product")
        h = self.norms["input"].add_forward(resid32, delta)
        # each sublayer adds its result to the stream itself where its last product can (None comes back)
        a = self.mixer.forward(h, inputs, cache, residual32=resid32) if self.mixer.adds_residual \
            else self.mixer.forward(h, inputs, cache)
        if self.feed_forward is None:
            return resid32, a
        b = self.feed_forward.forward(h, inputs, residual32=resid32) if self.feed_forward.adds_residual \
            else self.feed_forward.forward(h, inputs)
        if a is None or b is None:
            return resid32, (a if b is None else b)
        return resid32, ops.DeltaPair(a, b)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    graph_safe = True

    def __init__(self, ctx, mixer, feed_forward, norms, extras=None):
        super().__init__(mixer, feed_forward, norms)
        self.ctx = ctx
        want = {"mixer_in", "mixer_out"} | ({"feed_forward_in", "feed_forward_out"} if feed_forward is not None else set())
        if want - set(norms):
            raise ValueError(f"sandwich block needs norms named {sorted(want)}; missing {sorted(want - set(norms))}")
        extras = extras or {}
        if set(extras) - {"side"}:
            raise ValueError(f"sandwich block knows the extra 'side' only, got {sorted(extras)}")
        self.side = extras.get("side")

    @staticmethod
    def _pair_fuses(out_norm, in_norm, width):
        return (hasattr(out_norm, "normed_add_norm") and hasattr(in_norm, "weight32")
                and width <= ops.RMSNORM_ADD_NORM_MAX_WIDTH)

    accepts_normed_pending = True       # takes an ``ops.NormedPending`` as what the block before still has to add

    def forward(self, resid32, delta, inputs, cache, next_norm=None):
        if isinstance(delta, ops.NormedRows):
            raise ValueError("a sandwich block cannot follow a block that fused the next norm into its last product")
        if isinstance(delta, ops.RoundedRows):          # the block before added its result itself
            delta = None
        n = self.norms
        if isinstance(delta, ops.NormedPending):
            # the normed sum the block before left undone, and this block's first norm, in one kernel
            if hasattr(n["mixer_in"], "weight32") and resid32.shape[1] <= ops.RMSNORM_ADD_NORM_MAX_WIDTH:
                h = ops.rmsnorm_add_norm(resid32, delta.y, delta.weight32, delta.eps, n["mixer_in"].weight32, n["mixer_in"].eps)
            else:
                delta.settle(resid32)
                h = n["mixer_in"].forward(resid32)
        else:
            h = n["mixer_in"].add_forward(resid32, delta)
        y = self.mixer.forward(h, inputs, cache)
        last = self.feed_forward is None
        rounded = None
        if not last and self._pair_fuses(n["mixer_out"], n["feed_forward_in"], resid32.shape[1]):
            h = n["mixer_out"].normed_add_norm(resid32, y, n["feed_forward_in"])
        else:
            rounded = n["mixer_out"].normed_add(resid32, y, rounded=last and self.side is not None)
            if not last:
                h = n["feed_forward_in"].forward(resid32)
        if not last:
            y = self.feed_forward.forward(h, inputs)
            rounded = n["feed_forward_out"].normed_add(resid32, y, rounded=self.side is not None)
        if self.side is not None:
            return resid32, self.side.forward(resid32, rounded if rounded is not None else resid32, inputs, defer=True)
        return resid32, None
