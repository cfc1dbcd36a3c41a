"""Tedenex as data: which parts each layer has, with which sizes, in which order.

Layers in the ``sandwich`` arrangement (a norm before and after every sublayer, weights stored as distances
from one), each with its own mixer (``attention`` with biases, a short convolution, a distance penalty and
blocks of positions; ``time_mix``; ``latent_attention`` with a query latent and no sink), a plain
feed-forward with the square of relu (or none), and a token's side rows as the layer's last sublayer.  A loop
over a span of layers becomes schedule entries that name those layers again: every entry keeps a cache or
state of its own, and the first entry of each pass but the first adds the token rows to the stream.  The
final norm is followed by the token table as output matrix.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b``, ``l<i>.mix.*``,
``l<i>.mlp.up`` / ``down``, ``l<i>.side.gate`` / ``proj`` / ``norm``, ``final.norm``.
"""

from __future__ import annotations

from ..config.model_config import ConvAttentionConfig, LatentAttentionConfig, TedenexConfig, TimeMixConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

SLOPE_EXPONENT = 8.0        # head h of H is penalised by 2^(-8 (h + 1) / H) per position of distance

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                    "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "q_conv": "q.conv", "k_conv": "k.conv",
                    "v_conv": "v.conv"}


def _position(m: LatentAttentionConfig, positions: dict) -> str | None:
    """Name of the position encoding for this layer's rotated part (layers with equal settings share one)."""
    if m.rot_dims == 0:
        return None
    key = (m.rot_dim, m.rot_dims, m.rot_base)
    for name, (k, _) in positions.items():
        if k == key:
            return name
    name = f"rot{len(positions)}"
    positions[name] = (key, PartSpec("rope", {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                              "pairing": "interleaved"}))
    return name


def schedule_of(cfg: TedenexConfig) -> tuple[ScheduleEntry, ...]:
    n, lp = len(cfg.layers), cfg.loop
    if lp is None:
        return tuple(ScheduleEntry(i) for i in range(n))
    runs = [ScheduleEntry(i) for i in range(lp.start)]
    for p in range(lp.times):
        runs += [ScheduleEntry(i, add_embedding=(p > 0 and i == lp.start)) for i in range(lp.start, lp.stop)]
    return tuple(runs + [ScheduleEntry(i) for i in range(lp.stop, n)])


def tedenex_spec(cfg: TedenexConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps
    positions: dict = {}
    layers = []

    def norm(name):
        return PartSpec("rmsnorm", {"width": W, "eps": eps, "tensor": "", "one_plus": True}, name)

    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, ConvAttentionConfig):
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "position": None, "scale": m.scale, "qk_norm_eps": eps, "chunk": m.mask_size, "bias": True,
                "conv_taps": m.conv, "slope_exponent": SLOPE_EXPONENT, "names": _ATTENTION_NAMES}, p + "mix.")
        elif isinstance(m, TimeMixConfig):
            mixer = PartSpec("time_mix", {"hidden_size": W, "num_heads": m.heads, "dim": m.dim, "norm_eps": eps,
                                          "decay_rank": m.decay_rank}, p + "mix.")
        else:
            assert isinstance(m, LatentAttentionConfig)
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "norm_eps": eps, "position": _position(m, positions),
                "q_rank": m.q_rank, "sink": False}, p + "mix.")
        norms = {"mixer_in": norm(p + "norm1"), "mixer_out": norm(p + "norm1b")}
        ff = None
        if layer.ff is not None:
            ff = PartSpec("dense", {"hidden_size": W, "intermediate_size": layer.ff, "activation": "relu_squared",
                                    "names": {"up": "up", "down": "down"}}, p + "mlp.")
            norms.update({"feed_forward_in": norm(p + "norm2"), "feed_forward_out": norm(p + "norm2b")})
        extras = {}
        if cfg.side_dim is not None:
            extras["side"] = PartSpec("token_side", {
                "hidden_size": W, "vocab_size": cfg.vocab_size, "dim": cfg.side_dim, "index": i,
                "table_width": len(cfg.layers) * cfg.side_dim, "eps": eps, "table": "side.embed",
                "names": {"gate": p + "side.gate", "proj": p + "side.proj", "norm": p + "side.norm"}}, "")
        layers.append(LayerSpec(PartSpec("sandwich", {}, p), mixer, ff, norms, extras))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=W, embedding="embed", layers=tuple(layers), schedule=schedule_of(cfg),
        final_norm=norm("final.norm"), head=None, positions={name: spec for name, (_, spec) in positions.items()})


register_architecture(TedenexConfig.architecture, TedenexConfig, tedenex_spec)
