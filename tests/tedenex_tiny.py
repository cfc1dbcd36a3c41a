"""Small Tedenex configurations for the tests, and helpers that make their model folders.

The configurations differ from one another in every size and option: the order and kinds of the layers, head
counts and groups (also one head, and as many key/value heads as query heads), key and value sizes (equal and
not), blocks of positions of several sizes (also 1, and none), convolutions of 1 to 4 taps (and none), rotated
parts (the whole rotated part, a part of it, none), query latents (and none), layers without feed-forward, a
span of layers that runs 2 or 3 times (starting at the first layer, ending at the last, a single layer; and no
span), side rows of several widths (and none), widths that are and are not multiples of 8.
"""

from __future__ import annotations

from pathlib import Path

import torch

from acorninfer_b200.config.model_config import (ConvAttentionConfig, LatentAttentionConfig, LayerLoop, TedenexConfig,
                                                 TedenexLayer, TimeMixConfig)
from acorninfer_b200.weights.random_init import write_random_model
from acorninfer_b200.weights.safetensors_io import SafetensorsFile


def att(heads, kv_heads, dim, vdim, scale, conv=None, mask=None):
    return ConvAttentionConfig(heads, kv_heads, dim, vdim, scale, conv, mask)


def wkv(heads, dim, rank):
    return TimeMixConfig(heads, dim, rank)


def lat(heads, dim, rot_dim, vdim, kv_rank, scale, rot_dims, rot_base=1e4, q_rank=None):
    return LatentAttentionConfig(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
                                 rot_dims=rot_dims, rot_base=rot_base, q_rank=q_rank)


def L(mixer, ff=None):
    kind = {ConvAttentionConfig: "attention", TimeMixConfig: "wkv", LatentAttentionConfig: "latent_attention"}[type(mixer)]
    return TedenexLayer(kind, mixer, ff)


TED_A = dict(page_size=8, seed=17, cfg=TedenexConfig(
    vocab_size=190, hidden_size=72, norm_eps=1e-6, side_dim=10, loop=LayerLoop(0, 2, 2), layers=(
        L(wkv(heads=3, dim=8, rank=5), ff=50),
        L(att(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.3, conv=3, mask=11), ff=None),
        L(lat(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=20, scale=0.25, rot_dims=6, rot_base=500.0, q_rank=12), ff=96),
    )))

TED_B = dict(page_size=4, seed=18, cfg=TedenexConfig(
    vocab_size=133, hidden_size=60, norm_eps=1e-5, side_dim=None, loop=LayerLoop(1, 4, 3), layers=(
        L(att(heads=5, kv_heads=1, dim=8, vdim=6, scale=0.35, conv=1, mask=None), ff=48),
        L(lat(heads=2, dim=16, rot_dim=8, vdim=8, kv_rank=16, scale=0.2, rot_dims=4, rot_base=1e5, q_rank=None), ff=None),
        L(wkv(heads=1, dim=20, rank=3), ff=30),
        L(att(heads=2, kv_heads=2, dim=24, vdim=24, scale=0.2, conv=4, mask=6), ff=20),
    )))

# sizes at which the bfloat16 engine takes its tensor-core paths (head sizes that are multiples of 16, also 128)
TED_C = dict(page_size=16, seed=19, cfg=TedenexConfig(
    vocab_size=320, hidden_size=128, norm_eps=1e-5, side_dim=16, loop=LayerLoop(1, 3, 2), layers=(
        L(att(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, conv=4, mask=40), ff=192),
        L(wkv(heads=2, dim=64, rank=8), ff=128),
        L(lat(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=48, scale=0.15, rot_dims=16, rot_base=1e6, q_rank=64), ff=None),
        L(att(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, conv=2, mask=100), ff=64),
    )))

# longer requests: blocks of 70 over pages of 16, a state and a convolution's memory carried far, latents of a
# row width (96) the tensor-core kernel takes
TED_LONG = dict(page_size=16, seed=20, cfg=TedenexConfig(
    vocab_size=600, hidden_size=96, norm_eps=1e-5, side_dim=8, loop=LayerLoop(0, 3, 2), layers=(
        L(att(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.18, conv=3, mask=70), ff=64),
        L(wkv(heads=3, dim=16, rank=6), ff=None),
        L(lat(heads=2, dim=24, rot_dim=16, vdim=40, kv_rank=80, scale=0.16, rot_dims=16, rot_base=1e4, q_rank=40), ff=48),
    )))

TEDS = {"ted_a": TED_A, "ted_b": TED_B, "ted_c": TED_C}


def read_weights(model_dir: Path) -> dict[str, torch.Tensor]:
    f = SafetensorsFile(Path(model_dir) / "model.safetensors")
    return {n: f.tensor(n).clone() for n in f.entries}


def make_model_dir(tmp: Path, tiny: dict, sigma: float = 0.12, sigma_norm: float = 0.2) -> Path:
    return write_random_model(tmp, tiny["cfg"], tiny["seed"], sigma, sigma_norm)


def random_config(seed: int) -> TedenexConfig:
    """A configuration drawn at random: 3 to 5 layers with each kind of mixer at least once, a span that runs 1 to 3
    times, sizes from lists that hold what real models have (heads of 32 to 128) beside odd ones."""
    import random
    rng = random.Random(seed)
    width = rng.choice([128, 192, 320])
    kinds = ["attention", "wkv", "latent_attention"]
    n = rng.randint(3, 5)
    order = [rng.choice(kinds) for _ in range(n)]
    for k in kinds:
        if k not in order:
            order[rng.randrange(n)] = k
    layers = []
    for k in order:
        ff = rng.choice([None, 200, 256, 384])
        if k == "attention":
            d, kv = rng.choice([32, 64, 96, 128]), rng.choice([1, 2, 4])
            dv = rng.choice([d, d, 48])
            layers.append(L(att(kv * rng.choice([1, 2, 3, 4]), kv, d, dv, d ** -0.5, conv=rng.choice([None, 2, 3, 4]),
                                mask=rng.choice([None, 32, 64, 100, 256])), ff))
        elif k == "wkv":
            layers.append(L(wkv(rng.choice([1, 2, 4]), rng.choice([16, 32, 64]), rng.choice([4, 16, 32])), ff))
        else:
            rot = rng.choice([16, 32])
            layers.append(L(lat(heads=rng.choice([2, 4, 8]), dim=rng.choice([32, 64]), rot_dim=rot, vdim=rng.choice([32, 48, 64]),
                                kv_rank=rng.choice([48, 96, 128]), scale=rng.choice([0.1, 0.125]), rot_dims=rng.choice([rot, rot // 2]),
                                rot_base=rng.choice([1e4, 1e6]), q_rank=rng.choice([None, 48, 96])), ff))
    start = rng.randrange(n)
    stop = rng.randint(start + 1, n)
    return TedenexConfig(vocab_size=rng.choice([300, 512, 1000]), hidden_size=width, norm_eps=rng.choice([1e-5, 1e-6]),
                         layers=tuple(layers), loop=rng.choice([None, LayerLoop(start, stop, rng.randint(1, 3))]),
                         side_dim=rng.choice([None, 8, 24, 20]))
