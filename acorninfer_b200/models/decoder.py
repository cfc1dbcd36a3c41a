"""The generic decoder: parts built from a ModelSpec, run in the order its schedule says.

``forward`` is the whole model for one step: token table -> float32 residual stream ->
the scheduled layer runs -> final norm on the rows whose logits are wanted -> output
matrix -> float32 logits, with the spec's stages (if it names any) after the token table and
around the output matrix.  Reference for the order of operations:
``Qwen3ForCausalLM.forward`` in ``acorninfer/models/qwen3.py:491-518``.  The layer loop is a
loop over data: ``spec.schedule`` may name a layer twice, and a run may read the cache
of an earlier run instead of keeping its own.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in part kinds)
from ..kernels import ops
from ..parts.base import (BLOCKS, FEED_FORWARDS, LAYER_EXTRAS, MIXERS, NORMS, PASS_ENTRIES, POSITION_ENCODINGS, STAGES,
                          BuildContext, KVNeeds, ModelSpec, StateNeeds, TensorSpec, build_part)


@dataclass
class EntryCache:
    """What a schedule entry's mixer gets: the pages (its own or another run's), the cache
    group they belong to, whether this run writes them, and its state tensor if any."""

    entry: int
    group: int | None
    k_pages: torch.Tensor | None
    v_pages: torch.Tensor | None
    write: bool
    state: torch.Tensor | None


class Decoder:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, page_size: int = 16):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.ctx = BuildContext(dtype=dtype, device=self.device, page_size=page_size)
        for name, ps in spec.positions.items():
            self.ctx.positions[name] = build_part(POSITION_ENCODINGS, ps, self.ctx)
        self.blocks = []
        self._named_parts: list[tuple[str, object]] = []     # (prefix, part) for tensor collection
        for ls in spec.layers:
            mixer = build_part(MIXERS, ls.mixer, self.ctx)
            ff = build_part(FEED_FORWARDS, ls.feed_forward, self.ctx) if ls.feed_forward is not None else None
            norms = {k: build_part(NORMS, v, self.ctx) for k, v in ls.norms.items()}
            extras = {k: build_part(LAYER_EXTRAS, v, self.ctx) for k, v in ls.extras.items()}
            block = BLOCKS.get(ls.block.kind)(ctx=self.ctx, mixer=mixer, feed_forward=ff, norms=norms,
                                              **({"extras": extras} if extras else {}), **ls.block.params)
            self.blocks.append(block)
            self._named_parts.append((ls.mixer.prefix, mixer))
            if ff is not None:
                self._named_parts.append((ls.feed_forward.prefix, ff))
            for k, v in ls.norms.items():
                self._named_parts.append((v.prefix, norms[k]))
            for k, v in ls.extras.items():
                self._named_parts.append((v.prefix, extras[k]))
            self._named_parts.append((ls.block.prefix, block))
        self.final_norm = build_part(NORMS, spec.final_norm, self.ctx)
        self._named_parts.append((spec.final_norm.prefix, self.final_norm))
        self.stages = {}
        for where in ("after_embedding", "before_head", "after_head"):
            self.stages[where] = [build_part(STAGES, ps, self.ctx) for ps in getattr(spec, where)]
            self._named_parts.extend((ps.prefix, st) for ps, st in zip(getattr(spec, where), self.stages[where]))
        self.pass_entry = None
        if spec.pass_entry is not None:
            self.pass_entry = build_part(PASS_ENTRIES, spec.pass_entry, self.ctx)
            self._named_parts.append((spec.pass_entry.prefix, self.pass_entry))
        for i, e in enumerate(spec.schedule):
            if e.opens_pass is not None and self.pass_entry is None:
                raise ValueError(f"schedule entry {i} opens a pass, but the model names no pass_entry part")
            if not (0 <= e.layer < len(spec.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}; the model has {len(spec.layers)}")
            if e.reads_cache_of is not None and not (0 <= e.reads_cache_of < i):
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.reads_cache_of}, which is not earlier")
            if e.reads_cache_of is not None and spec.schedule[e.reads_cache_of].reads_cache_of is not None:
                raise ValueError(f"schedule entry {i} reads the cache of an entry that has none of its own")
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None

    # ------------------------------------------------------------------ tensors

    def expected_tensors(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        s = self.spec
        out[s.embedding] = TensorSpec((s.vocab_size, s.hidden_size))
        for prefix, part in self._named_parts:
            for rel, ts in part.tensor_specs().items():
                out[prefix + rel] = ts
        if s.head is not None:
            out[s.head] = TensorSpec((s.vocab_size, s.hidden_size))
        return out

    def ignorable_tensors(self) -> tuple[str, ...]:
        # A tied model's file may still carry a copy of the output matrix.
        return ("lm_head.weight",) if self.spec.head is None else ()

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding].contiguous()
        self.head = tensors[s.head].contiguous() if s.head is not None else self.embedding
        for prefix, part in self._named_parts:
            part.bind({rel: tensors[prefix + rel] for rel in part.tensor_specs() if prefix + rel in tensors})

    # ------------------------------------------------------------------ cache needs

    def cache_needs(self) -> tuple[dict[int, KVNeeds], dict[int, StateNeeds]]:
        """Per schedule entry that keeps something: its KV needs and its state needs.  An entry whose
        pages other runs read keeps them for the widest window among its readers and itself.  Stages
        that keep state per request appear under their own keys (``"<where>.<index>"``)."""
        from dataclasses import replace
        kv: dict[int, KVNeeds] = {}
        state: dict = {}
        for i, e in enumerate(self.spec.schedule):
            needs = self.blocks[e.layer].mixer.cache_needs()
            if e.reads_cache_of is not None:
                owner = kv.get(e.reads_cache_of)
                if needs.kv is None or owner is None or needs.kv.layout_key != owner.layout_key:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {e.reads_cache_of}: "
                                     "their mixers keep different things")
                if owner.window is not None and (needs.kv.window is None or needs.kv.window > owner.window):
                    kv[e.reads_cache_of] = replace(owner, window=needs.kv.window)
                continue
            if needs.kv is not None:
                kv[i] = needs.kv
            if needs.state is not None:
                state[i] = needs.state
        for where, stages in self.stages.items():
            for n, st in enumerate(stages):
                sn = st.state_needs()
                if sn is not None:
                    state[f"{where}.{n}"] = sn
        return kv, state

    def entry_caches(self, manager) -> list[EntryCache]:
        out = []
        for i, e in enumerate(self.spec.schedule):
            owner = i if e.reads_cache_of is None else e.reads_cache_of
            if owner in manager.entry_group:
                k, v = manager.kv_pages(owner)
                group = manager.group_of(owner)
            else:
                k = v = group = None
            out.append(EntryCache(i, group, k, v, e.reads_cache_of is None, manager.state.get(i)))
        for where, stages in self.stages.items():
            for n, st in enumerate(stages):
                if f"{where}.{n}" in manager.state:
                    st.state = manager.state[f"{where}.{n}"]
        return out

    def step_arrays(self) -> dict:
        """The per-step arrays all parts declare (``Part.step_arrays``), by name."""
        out: dict = {}
        for _, part in self._named_parts:
            for name, build in part.step_arrays().items():
                out.setdefault(name, build)
        return out

    @property
    def graph_safe(self) -> bool:
        """Every part allows a step to be captured and replayed (see ``Part.graph_safe``)."""
        return all(getattr(part, "graph_safe", False) for _, part in self._named_parts)

    # ------------------------------------------------------------------ forward

    def forward(self, inputs, caches: list[EntryCache]) -> torch.Tensor | None:
        """Runs the step's tokens; returns float32 logits [wanted, vocab] (None if none wanted)."""
        resid32 = ops.embed(inputs.token_ids, self.embedding, scale=self.spec.embedding_scale)
        for stage in self.stages["after_embedding"]:
            resid32 = stage.forward(resid32, inputs)
        delta = None
        sched = self.spec.schedule
        # a run that takes the tokens in again adds the stream as it was here
        def reenters(e):
            return e.add_embedding or e.opens_pass is not None

        entered32 = resid32.clone() if any(reenters(e) for e in sched) else None
        for i, e in enumerate(sched):
            if reenters(e):
                # whatever the run before still has to add is added first: the stream is read whole here
                if isinstance(delta, ops.NormedRows):
                    raise ValueError(f"schedule entry {i} takes the token rows in again, but the run before it already "
                                     "prepared this run's first norm")
                if isinstance(delta, ops.DeltaPair):
                    delta = ops.fold_pair(resid32, delta)
                if isinstance(delta, ops.NormedPending):
                    delta.settle(resid32)
                    delta = None
                if delta is not None and not isinstance(delta, ops.RoundedRows):
                    ops.add_into(resid32, delta)
                delta = None
                if e.add_embedding:
                    ops.add_into(resid32, entered32)
                if e.opens_pass is not None:
                    resid32 = self.pass_entry.forward(resid32, entered32, e.opens_pass, inputs)
            # the norm that consumes this run's output: the next run's first norm (the final norm
            # works on selected rows only and keeps its own kernel)
            nxt = self.blocks[sched[i + 1].layer].first_norm(inputs.num_tokens) \
                if i + 1 < len(sched) and not reenters(sched[i + 1]) else None
            resid32, delta = self.blocks[e.layer].forward(resid32, delta, inputs, caches[i], next_norm=nxt)
            # two pending results (a block whose sublayers run side by side): whoever comes next adds both, or
            # the first is added here
            taker = self.blocks[sched[i + 1].layer] if i + 1 < len(sched) else self.final_norm
            if isinstance(delta, ops.DeltaPair) and not getattr(taker, "accepts_pair", False):
                delta = ops.fold_pair(resid32, delta)
            # a normed sum left undone: the next block takes it into its first norm's kernel, or it is added here
            if isinstance(delta, ops.NormedPending) and not (i + 1 < len(sched) and not reenters(sched[i + 1])
                                                             and getattr(taker, "accepts_normed_pending", False)):
                delta.settle(resid32)
                delta = None
        if inputs.num_logits == 0:
            return None
        if isinstance(delta, ops.RoundedRows):          # the last block already added its result
            delta = None
        h = self.final_norm.add_forward(resid32, delta, rows=inputs.logit_tokens)
        for stage in self.stages["before_head"]:
            h = stage.forward(h, inputs)
        logits = ops.linear(h, self.head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0:
            ops.head_gate(logits, None, 1, self.spec.logit_scale)       # every entry times the factor, in place
        for stage in self.stages["after_head"]:
            logits = stage.forward(logits, inputs)
        return logits


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """The checkpoint tensors a model of this spec expects (no device needed)."""
    return Decoder(spec, torch.float32, "cpu").expected_tensors()
