"""Zigolix as data: which parts each layer has, with which sizes, in which order.

Layers in the ``prenorm`` arrangement with RMS norms.  A layer's mixer is ``attention`` with the options this
design uses (values that are the keys as projected, a part of each head rotated in neighbouring pairs with
stretched frequencies, q and k brought to unit root mean square after the rotation, a sliding window, a sink per
head) or ``differential_attention``; its feed-forward is ``gated`` with the tanh form of gelu, ``routed_experts``
with capped experts, normalised weights and a shared expert, or absent.  A loop over a span of layers becomes
schedule entries that name those layers again (every entry keeps a cache of its own); the first entry of every
pass, the first pass included, opens it through the ``mix_in`` pass entry.  The final norm is followed by an output
matrix of its own and a factor on the logits.

Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.model_config import CappedExpertsConfig, DiffAttentionConfig, SinkAttentionConfig, ZigolixConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

_ATTENTION_NAMES = {"q": "q", "k": "k", "o": "o", "sink": "sink"}
_FF_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _position(m: SinkAttentionConfig, positions: dict) -> str | None:
    """Name of the position encoding for this layer's rotated part (layers with equal settings share one)."""
    if m.rot_dims == 0:
        return None
    key = (m.dim, m.rot_dims, m.rot_base, m.scaling)
    for name, (k, _) in positions.items():
        if k == key:
            return name
    name = f"rot{len(positions)}"
    params = {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base, "pairing": "interleaved"}
    if m.scaling is None:
        positions[name] = (key, PartSpec("rope", params))
    else:
        sc = m.scaling
        positions[name] = (key, PartSpec("scaled_rope", {**params, "factor": sc.factor, "original": sc.original,
                                                         "fast": sc.fast, "slow": sc.slow}))
    return name


def schedule_of(cfg: ZigolixConfig) -> tuple[ScheduleEntry, ...]:
    n, lp = len(cfg.layers), cfg.loop
    if lp is None:
        return tuple(ScheduleEntry(i) for i in range(n))
    runs = [ScheduleEntry(i) for i in range(lp.start)]
    for p in range(lp.times):
        runs += [ScheduleEntry(i, opens_pass=p if i == lp.start else None) for i in range(lp.start, lp.stop)]
    return tuple(runs + [ScheduleEntry(i) for i in range(lp.stop, n)])


def zigolix_spec(cfg: ZigolixConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict = {}
    layers = []

    def norm(name):
        return PartSpec("rmsnorm", {"width": W, "eps": eps, "tensor": ""}, name)

    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, SinkAttentionConfig):
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "position": _position(m, positions), "scale": m.scale, "qk_norm_eps": eps, "window": m.mask_size,
                "values_from_keys": True, "norm_after_rotation": True, "qk_norm_weights": False, "sink": True,
                "names": _ATTENTION_NAMES}, p + "mix.")
        else:
            assert isinstance(m, DiffAttentionConfig)
            mixer = PartSpec("differential_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "dim": m.dim, "value_dim": m.vdim,
                "scale": m.scale, "diff": m.diff, "norm_eps": eps, "softcap": m.softcap, "window": m.mask_size}, p + "mix.")
        norms = {"mixer": norm(p + "norm1")}
        ff = None
        if isinstance(layer.ff, CappedExpertsConfig):
            f = layer.ff
            ff = PartSpec("routed_experts", {
                "hidden_size": W, "expert_size": f.ff, "num_experts": f.experts, "num_identity": 0, "top": f.top,
                "correction": False, "normalize": True, "activation": "capped_swish", "limit": f.limit,
                "shared_size": f.shared_ff, "shared_limit": f.shared_limit}, p + "mlp.")
        elif layer.ff is not None:
            ff = PartSpec("gated", {"hidden_size": W, "intermediate_size": layer.ff, "activation": "gelu_tanh",
                                    "names": _FF_NAMES}, p + "mlp.")
        if ff is not None:
            norms["feed_forward"] = norm(p + "norm2")
        layers.append(LayerSpec(PartSpec("prenorm", {}, p), mixer, ff, norms))
    entry = None
    if cfg.loop is not None:
        entry = PartSpec("mix_in", {"width": W, "passes": cfg.loop.times}, "loop.")
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=W, embedding="embed", layers=tuple(layers), schedule=schedule_of(cfg),
        final_norm=norm("final.norm"), head="head", positions={name: spec for name, (_, spec) in positions.items()},
        pass_entry=entry, logit_scale=cfg.logit_scale)


register_architecture(ZigolixConfig.architecture, ZigolixConfig, zigolix_spec)
