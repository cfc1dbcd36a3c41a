"""Sizes of published Qwen3 dense models as ``config.json`` dictionaries, for runs with random
weights (benchmarks, the random-weights mode): no checkpoint is needed to measure at a model's
layer sizes.  Only the keys the architecture reads are given.  For Kogonex, of which no model is
published, two size sets with layers as wide as real models have them; the same for Vagulorn and Tedenex."""

from __future__ import annotations


def _qwen3(layers: int, hidden: int, heads: int, kv_heads: int, intermediate: int, tied: bool) -> dict:
    return {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": layers, "hidden_size": hidden,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128,
            "intermediate_size": intermediate, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "vocab_size": 151936,
            "tie_word_embeddings": tied, "eos_token_id": 151645}


PRESETS: dict[str, dict] = {
    "qwen3-0.6b": _qwen3(28, 1024, 16, 8, 3072, True),
    "qwen3-1.7b": _qwen3(28, 2048, 16, 8, 6144, True),
    "qwen3-4b": _qwen3(36, 2560, 32, 8, 9728, True),
    "qwen3-8b": _qwen3(36, 4096, 32, 8, 12288, False),
    "qwen3-14b": _qwen3(40, 5120, 40, 8, 17408, False),
    "qwen3-32b": _qwen3(64, 5120, 64, 8, 25600, False),
}


def _kogonex(width: int, vocab: int, heads: int, dim: int, rot: int, vdim: int, rank: int, window: int, d_heads: int,
             d_kv_heads: int, d_dim: int, d_vdim: int, taps: int, decay_rank: int, gate_rank: int, ff: int, experts: int,
             identity: int, top: int, groups: int, keep: int, repeats: int = 2) -> dict:
    """Layers in the pattern delta, latent, delta, delta, latent-reading-the-other's-cache, ``repeats`` times."""
    mlp = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    delta = {"heads": d_heads, "kv_heads": d_kv_heads, "dim": d_dim, "vdim": d_vdim, "conv": taps,
             "decay_rank": decay_rank, "gate_rank": gate_rank}
    latent = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": (dim + rot) ** -0.5,
              "mask": {"size": window},
              "rot": {"base": 1e6, "dims": rot, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    layers = []
    for _ in range(repeats):
        for kind in ("delta", "latent", "delta", "delta", "shared"):
            if kind == "delta":
                layers.append({"type": "channel_delta", "mixer": dict(delta), "mlp": mlp})
            else:
                mixer = dict(latent, kv_from=len(layers) - 3) if kind == "shared" else dict(latent)
                layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Kogonex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 100003, "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers}


PRESETS.update({
    "kogonex-w1024": _kogonex(1024, 32768, heads=8, dim=64, rot=32, vdim=64, rank=192, window=512, d_heads=8, d_kv_heads=4,
                              d_dim=64, d_vdim=128, taps=4, decay_rank=32, gate_rank=64, ff=512, experts=14, identity=2,
                              top=4, groups=4, keep=2),
    "kogonex-w2048": _kogonex(2048, 65536, heads=16, dim=128, rot=64, vdim=128, rank=384, window=1024, d_heads=16,
                              d_kv_heads=8, d_dim=128, d_vdim=128, taps=4, decay_rank=64, gate_rank=128, ff=1024, experts=30,
                              identity=2, top=6, groups=4, keep=2),
})


def _vagulorn(width: int, vocab: int, heads: int, kv_heads: int, ff: int, span: int, ssm_heads: int, ssm_groups: int,
              repeats: int = 2) -> dict:
    """Layers in the pattern state space, attention in blocks, attention beside linear attention, state space,
    ``repeats`` times; heads of 128, a state of 128 per state-space head of 64 inputs."""
    mlp = {"kind": "dense", "ff": ff}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
           "rot": {"base": 1e6, "dims": 64}}
    ssm = {"heads": ssm_heads, "vdim": 64, "state": 128, "groups": ssm_groups, "conv": 4, "norm_groups": ssm_groups}
    decay = [1.0 - 2.0 ** -(5 + 3 * h / max(1, heads - 1)) for h in range(heads)]
    layers = []
    for _ in range(repeats):
        layers.append({"type": "mamba2", "mixer": dict(ssm), "mlp": mlp})
        layers.append({"type": "attention", "mixer": dict(att, mask={"size": span}), "mlp": mlp})
        layers.append({"type": "parallel", "mlp": mlp, "mixer": {
            "left": dict(att, mask={"size": span, "keep_first": 4}), "left_scale": 0.8,
            "right": {"heads": heads, "dim": 128, "vdim": 128, "decay": decay}, "right_scale": 0.9}})
        layers.append({"type": "mamba2", "mixer": dict(ssm), "mlp": mlp})
    return {"architecture": "Vagulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 32.0},
            "layers": layers}


PRESETS.update({
    "vagulorn-w1024": _vagulorn(1024, 32768, heads=8, kv_heads=2, ff=3072, span=1024, ssm_heads=32, ssm_groups=4),
    "vagulorn-w2048": _vagulorn(2048, 65536, heads=16, kv_heads=4, ff=6144, span=1024, ssm_heads=64, ssm_groups=8),
})


def _tedenex(width: int, vocab: int, heads: int, kv_heads: int, ff: int, span: int, mix_heads: int, decay_rank: int,
             lat_heads: int, rank: int, rot: int, q_rank: int, side: int, times: int = 2) -> dict:
    """Layers in the pattern time mixing, convolved attention in blocks, latent attention, twice, the first three
    run ``times`` times in a row; attention heads of 128, time-mixing heads of 64."""
    mlp = {"kind": "dense", "ff": ff}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "conv": 4, "mask": {"size": span}}
    mix = {"heads": mix_heads, "dim": 64, "decay_rank": decay_rank}
    lat = {"heads": lat_heads, "dim": 128, "rot_dim": rot, "vdim": 128, "kv_rank": rank, "q_rank": q_rank,
           "scale": (128 + rot) ** -0.5, "rot": {"base": 1e6, "dims": rot}}
    layers = []
    for _ in range(2):
        layers.append({"type": "wkv", "mixer": dict(mix), "mlp": mlp})
        layers.append({"type": "attention", "mixer": dict(att), "mlp": mlp})
        layers.append({"type": "latent_attention", "mixer": dict(lat), "mlp": mlp})
    return {"architecture": "Tedenex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "token_side": {"dim": side},
            "loop": {"start": 0, "stop": 3, "times": times}, "layers": layers}


PRESETS.update({
    "tedenex-w1024": _tedenex(1024, 32768, heads=8, kv_heads=2, ff=3072, span=1024, mix_heads=16, decay_rank=64, lat_heads=8,
                              rank=192, rot=32, q_rank=384, side=128),
    "tedenex-w2048": _tedenex(2048, 65536, heads=16, kv_heads=4, ff=6144, span=1024, mix_heads=32, decay_rank=64, lat_heads=16,
                              rank=384, rot=64, q_rank=768, side=256),
})


def _zigolix(width: int, vocab: int, heads: int, kv_heads: int, ff: int, window: int, experts: int, top: int,
             times: int = 2) -> dict:
    """Layers in the pattern differential attention, differential attention with routed experts, attention with a sink,
    twice, layers 1 and 2 run ``times`` times in a row; key rows and value rows of 128 everywhere (a differential
    head holds two maps of 64); the routed layers' active width (the chosen experts and the shared one) is ``ff``."""
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // (2 * top), "limit": 7.0}, "router": {"experts": experts, "top": top},
           "shared": {"ff": ff // 2, "limit": 7.0}}
    dif = {"heads": heads, "kv_heads": kv_heads, "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "softcap": 30.0, "diff": 0.5,
           "mask": {"size": window}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 1.0, "mask": {"size": window},
           "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    layers = []
    for _ in range(2):
        layers.append({"type": "attention_2", "mixer": dict(dif), "mlp": dense})
        layers.append({"type": "attention_2", "mixer": dict(dif), "mlp": moe})
        layers.append({"type": "attention", "mixer": dict(att), "mlp": dense})
    return {"architecture": "Zigolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
            "loop": {"start": 1, "stop": 3, "times": times}, "layers": layers}


PRESETS.update({
    "zigolix-w1024": _zigolix(1024, 32768, heads=8, kv_heads=2, ff=3072, window=1024, experts=16, top=2),
    "zigolix-w2048": _zigolix(2048, 65536, heads=16, kv_heads=4, ff=6144, window=1024, experts=16, top=2),
})


def preset(name: str) -> dict:
    try:
        import copy
        return copy.deepcopy(PRESETS[name.lower()])
    except KeyError:
        raise ValueError(f"no preset {name!r}; there are {', '.join(sorted(PRESETS))}") from None
