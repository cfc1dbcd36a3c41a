"""Small Zigolix configurations for the tests, and helpers that make their model folders.

The configurations differ from one another in every size and option: the order and kinds of the layers, head
counts and groups (also one head, and as many key/value heads as query heads), map and value sizes (values as
wide as a key row, wider, narrower), windows of several sizes (also 1, and none), rotated parts (the whole head,
a part of it, none; plain and stretched frequencies), score caps (also none), dense and routed feed-forwards (one
and several choices, with and without a shared expert, also none at all), a span of layers that runs 1 to 4 times
(starting at the first layer, ending at the last, a single layer; and no span), logit factors, widths that are
and are not multiples of 8.
"""

from __future__ import annotations

from pathlib import Path

import torch

from acorninfer_b200.config.model_config import (CappedExpertsConfig, DiffAttentionConfig, LayerLoop, RotaryScaling,
                                                 SinkAttentionConfig, ZigolixConfig, ZigolixLayer)
from acorninfer_b200.weights.random_init import write_random_model
from acorninfer_b200.weights.safetensors_io import SafetensorsFile


def sink(heads, kv_heads, dim, scale, mask=None, rot=0, base=1e4, scaling=None):
    return SinkAttentionConfig(heads, kv_heads, dim, dim, scale, mask, rot, base if rot else 1e4, scaling if rot else None)


def dif(heads, kv_heads, dim, vdim, scale, diff, softcap=None, mask=None):
    return DiffAttentionConfig(heads, kv_heads, dim, vdim, scale, diff, softcap, mask)


def moe(ff, limit, experts, top, shared=None, shared_limit=None):
    return CappedExpertsConfig(ff, limit, experts, top, shared, shared_limit if shared is not None else None)


def L(mixer, ff=None):
    return ZigolixLayer("attention" if isinstance(mixer, SinkAttentionConfig) else "attention_2", mixer, ff)


YARN = RotaryScaling(factor=4.0, original=64, fast=8.0, slow=0.5)

ZIG_A = dict(page_size=8, seed=31, cfg=ZigolixConfig(
    vocab_size=170, hidden_size=72, norm_eps=1e-6, logit_scale=0.7, loop=LayerLoop(0, 2, 2), layers=(
        L(dif(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.4, diff=0.3, softcap=3.0, mask=11), ff=50),
        L(sink(heads=3, kv_heads=1, dim=12, scale=0.5, mask=9, rot=8, base=300.0, scaling=YARN), ff=moe(20, 1.5, 5, 2, 14, 0.8)),
        L(dif(heads=2, kv_heads=2, dim=8, vdim=16, scale=0.3, diff=0.7, softcap=None, mask=None), ff=None),
    )))

ZIG_B = dict(page_size=4, seed=32, cfg=ZigolixConfig(
    vocab_size=141, hidden_size=60, norm_eps=1e-5, logit_scale=1.0, loop=LayerLoop(1, 4, 3), layers=(
        L(sink(heads=5, kv_heads=5, dim=6, scale=0.6, mask=None, rot=6, base=1e5), ff=moe(9, 3.0, 3, 1)),
        L(dif(heads=3, kv_heads=1, dim=10, vdim=4, scale=0.35, diff=0.5, softcap=8.0, mask=6), ff=48),
        L(sink(heads=2, kv_heads=2, dim=20, scale=0.3, mask=5, rot=0), ff=None),
        L(dif(heads=1, kv_heads=1, dim=12, vdim=30, scale=0.3, diff=0.2, softcap=1.0, mask=17), ff=moe(16, 0.7, 4, 4, 8, 2.0)),
    )))

# sizes at which the bfloat16 engine takes its tensor-core paths (key rows that are multiples of 16, values as wide)
ZIG_C = dict(page_size=16, seed=33, cfg=ZigolixConfig(
    vocab_size=330, hidden_size=128, norm_eps=1e-5, logit_scale=0.6, loop=LayerLoop(1, 3, 2), layers=(
        L(dif(heads=4, kv_heads=2, dim=32, vdim=64, scale=0.18, diff=0.55, softcap=20.0, mask=36), ff=192),
        L(sink(heads=4, kv_heads=2, dim=64, scale=0.3, mask=50, rot=32, base=2e4, scaling=RotaryScaling(2.5, 128, 16.0, 1.0)),
          ff=moe(64, 2.0, 8, 2, 64, 2.0)),
        L(dif(heads=2, kv_heads=1, dim=64, vdim=128, scale=0.12, diff=0.4, softcap=6.0, mask=100), ff=moe(32, 1.0, 6, 3)),
        L(sink(heads=8, kv_heads=1, dim=32, scale=0.4, mask=None, rot=32, base=1e4), ff=64),
    )))

# longer requests: windows of 70 and 45 over pages of 16, a looped span, routed experts over hundreds of tokens
ZIG_LONG = dict(page_size=16, seed=34, cfg=ZigolixConfig(
    vocab_size=600, hidden_size=96, norm_eps=1e-5, logit_scale=0.8, loop=LayerLoop(0, 2, 2), layers=(
        L(dif(heads=4, kv_heads=2, dim=16, vdim=32, scale=0.25, diff=0.5, softcap=10.0, mask=70), ff=moe(24, 2.0, 6, 2, 16, 2.0)),
        L(sink(heads=4, kv_heads=2, dim=32, scale=0.35, mask=45, rot=16, base=1e4, scaling=RotaryScaling(3.0, 96, 12.0, 1.0)), ff=64),
        L(dif(heads=3, kv_heads=3, dim=8, vdim=24, scale=0.3, diff=0.25, softcap=None, mask=130), ff=None),
    )))

ZIGS = {"zig_a": ZIG_A, "zig_b": ZIG_B, "zig_c": ZIG_C}


def read_weights(model_dir: Path) -> dict[str, torch.Tensor]:
    f = SafetensorsFile(Path(model_dir) / "model.safetensors")
    return {n: f.tensor(n).clone() for n in f.entries}


def make_model_dir(tmp: Path, tiny: dict, sigma: float = 0.12, sigma_norm: float = 0.2) -> Path:
    return write_random_model(tmp, tiny["cfg"], tiny["seed"], sigma, sigma_norm)


def random_config(seed: int) -> ZigolixConfig:
    """A configuration drawn at random: 3 to 5 layers with both kinds of mixer, a span that runs 1 to 3 times,
    sizes from lists that hold what real models have (key rows of 32 to 128) beside odd ones."""
    import random
    rng = random.Random(seed)
    width = rng.choice([128, 192, 320])
    n = rng.randint(3, 5)
    order = [rng.choice(["attention", "attention_2"]) for _ in range(n)]
    order[rng.randrange(n)] = "attention"
    order[(order.index("attention") + 1) % n] = "attention_2"
    layers = []
    for k in order:
        ff = rng.choice([None, 200, 256, moe(rng.choice([32, 48, 96]), rng.choice([1.0, 2.0, 7.0]), rng.choice([4, 8, 12]),
                                             rng.choice([1, 2, 4]), rng.choice([None, 32, 64]), 2.0)])
        kv = rng.choice([1, 2, 4])
        heads = kv * rng.choice([1, 2, 3, 4])
        if k == "attention":
            d = rng.choice([32, 64, 96, 128, 40])
            rot = rng.choice([0, d, d // 2, 16])
            sc = rng.choice([None, RotaryScaling(rng.choice([2.0, 8.0]), rng.choice([64, 256]), rng.choice([32.0, 8.0]), 1.0)])
            layers.append(L(sink(heads, kv, d, d ** -0.5 * 4, mask=rng.choice([None, 32, 64, 100, 256]), rot=rot,
                                 base=rng.choice([1e4, 2e5, 1e6]), scaling=sc if rot else None), ff))
        else:
            d = rng.choice([16, 32, 48, 64, 24])
            dv = rng.choice([2 * d, 2 * d, d, 48])
            layers.append(L(dif(heads, kv, d, dv, d ** -0.5, diff=rng.choice([0.2, 0.5, 0.8]),
                                softcap=rng.choice([None, 5.0, 30.0]), mask=rng.choice([None, 24, 36, 128])), ff))
    start = rng.randrange(n)
    stop = rng.randint(start + 1, n)
    return ZigolixConfig(vocab_size=rng.choice([300, 520, 1000]), hidden_size=width, norm_eps=rng.choice([1e-5, 1e-6]),
                         layers=tuple(layers), loop=rng.choice([None, LayerLoop(start, stop, rng.randint(1, 3))]),
                         logit_scale=rng.choice([1.0, 0.5, 0.3]))
