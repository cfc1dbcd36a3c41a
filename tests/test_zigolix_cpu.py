"""Zigolix without a GPU: its configuration, the model as data (a span of layers as schedule entries with caches
of their own, every pass opened by the pass entry), what its layers ask of the cache manager, and properties of
the plain implementation."""

import copy
import math

import pytest
import torch

from acorninfer_b200.config.model_config import ConfigError, ZigolixConfig
from acorninfer_b200.models.decoder import Decoder, expected_tensors
from acorninfer_b200.registry import config_from_dict, spec_for
from tests.plain import zigolix as plain
from tests.tiny import random_tokens
from tests.zigolix_tiny import ZIG_A, ZIG_B, ZIGS, make_model_dir, random_config, read_weights


@pytest.mark.parametrize("name", list(ZIGS))
def test_config_round_trip_and_registry(name):
    cfg = ZIGS[name]["cfg"]
    raw = cfg.to_dict()
    assert raw["architecture"] == "Zigolix" and len(raw["layers"]) == len(cfg.layers)
    again = config_from_dict(raw)
    assert isinstance(again, ZigolixConfig) and again == cfg
    for seed in range(6):
        drawn = random_config(seed)
        assert config_from_dict(drawn.to_dict()) == drawn


def test_config_errors_name_the_key():
    raw = ZIG_A["cfg"].to_dict()
    for path, value, word in ((("layers", 0, "type"), "mamba", "type"), (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "softcap"), 0.0, "softcap"),
                              (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"), (("layers", 0, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 1, "mixer", "vdim"), 7, "vdim"), (("layers", 1, "mlp", "router", "top"), 9, "top"),
                              (("layers", 1, "mlp", "expert", "limit"), 0.0, "limit"),
                              (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop"), (("norm", "eps"), 0.0, "eps")):
        bad = copy.deepcopy(raw)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["layers"][0]["mixer"]["diff"]
    with pytest.raises(ConfigError, match="diff"):
        config_from_dict(bad)
    # what a configuration leaves out does not exist: no window, no rotation, no cap, no span, no shared expert
    lean = copy.deepcopy(raw)
    del lean["loop"], lean["layers"][0]["mixer"]["mask"], lean["layers"][0]["mixer"]["softcap"]
    del lean["layers"][1]["mixer"]["rot"], lean["layers"][1]["mlp"]["shared"], lean["logit_scale"]
    cfg = config_from_dict(lean)
    assert cfg.loop is None and cfg.layers[0].mixer.mask_size is None and cfg.layers[0].mixer.softcap is None
    assert cfg.layers[1].mixer.rot_dims == 0 and cfg.layers[1].ff.shared_ff is None and cfg.logit_scale == 1.0
    spec = spec_for(cfg)
    assert spec.pass_entry is None and not spec.positions and "loop.in" not in expected_tensors(spec)


def test_model_as_data_schedule_and_cache_needs():
    cfg = ZIG_A["cfg"]
    spec = spec_for(cfg)
    assert [ls.mixer.kind for ls in spec.layers] == ["differential_attention", "attention", "differential_attention"]
    assert all(ls.block.kind == "prenorm" for ls in spec.layers)
    assert [ls.feed_forward.kind if ls.feed_forward else None for ls in spec.layers] == ["gated", "routed_experts", None]
    assert set(spec.layers[2].norms) == {"mixer"}
    # layers 0 and 1 run twice; each pass, the first too, is opened at its first layer
    assert [(e.layer, e.opens_pass) for e in spec.schedule] == [(0, 0), (1, None), (0, 1), (1, None), (2, None)]
    assert spec.pass_entry.kind == "mix_in" and spec.logit_scale == 0.7 and spec.head == "head"
    names = expected_tensors(spec)
    for n in ("embed", "head", "final.norm", "loop.in", "loop.step", "l0.norm1", "l0.norm2", "l0.mix.q.b", "l0.mix.lq1",
              "l0.mix.lk2", "l0.mix.g", "l0.mlp.gate", "l1.mix.sink", "l1.mlp.router", "l1.mlp.e4.down", "l1.mlp.shared.up"):
        assert n in names, n
    for n in ("l2.norm2", "l1.mix.v", "l1.mix.q.b", "l1.mlp.correction", "l1.mlp.e5.gate", "l1.mix.q.norm"):
        assert n not in names, n
    assert names["loop.in"].shape == (72, 144) and names["loop.step"].shape == (2, 72)
    assert names["l0.mix.q"].shape == (4 * 2 * 6, 72) and names["l0.mix.k"].shape == (2 * 2 * 6, 72)
    assert names["l0.mix.v"].shape == (2 * 10, 72) and names["l0.mix.g"].shape == (4 * 10, 72)
    assert names["l1.mix.sink"].shape == (3,) and names["l1.mlp.shared.gate"].shape == (14, 72)
    dec = Decoder(spec, torch.float32, "cpu", page_size=8)
    kv, state = dec.cache_needs()
    # every run keeps pages of its own: a key row of a differential layer holds both maps
    assert sorted(kv) == [0, 1, 2, 3, 4] and not state
    assert kv[0].head_dim == 12 and kv[0].value_dim == 10 and kv[0].window == 11 and kv[0].num_kv_heads == 2
    assert kv[1].head_dim == 12 and kv[1].value_dim is None and kv[1].window == 9
    assert kv[4].head_dim == 16 and kv[4].value_dim is None and kv[4].window is None
    pos = dec.ctx.positions["rot0"]
    assert pos.rotary_dim == 8 and pos.interleaved and pos.magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    b = spec_for(ZIG_B["cfg"])
    assert len(b.schedule) == 1 + 3 * 3 and [e.opens_pass for e in b.schedule if e.layer == 1] == [0, 1, 2]


def test_plain_implementation_properties(tmp_path):
    tiny = ZIG_A
    d = make_model_dir(tmp_path, tiny)
    w = read_weights(d)
    cfg = tiny["cfg"].to_dict()
    toks = random_tokens(40, tiny["cfg"].vocab_size, 5)
    full, layers = plain.forward(cfg, w, toks, return_layers=True)
    assert layers.shape == (5, 40, 72)
    # causal: a prefix gives the same logits
    assert (plain.forward(cfg, w, toks[:17]) - full[:17]).abs().max() < 1e-9
    # the factor on the logits
    other = dict(cfg, logit_scale=1.0)
    assert (plain.forward(other, w, toks) * 0.7 - full).abs().max() < 1e-9
    # the sink takes weight: with a very low sink the softmax is the ordinary one
    s = torch.randn(2, 5, 5, dtype=torch.float64)
    ok = plain.visible(5, 3)
    low = plain.sink_softmax(s, ok, torch.full((2,), -50.0, dtype=torch.float64))
    assert (low - plain.sink_softmax(s, ok)).abs().max() < 1e-12 and (low.sum(-1) - 1).abs().max() < 1e-12
    assert (plain.sink_softmax(s, ok, torch.zeros(2, dtype=torch.float64)).sum(-1) < 1).all()
    assert low[0, 4, 1] == 0 and low[0, 4, 2] > 0             # a window of 3: position 4 sees 2, 3, 4
    # stretched frequencies: fast pairs keep their rate, slow ones are divided by the factor
    rate, mag = plain.stretched_frequencies({"dims": 8, "base": 300.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}})
    base = torch.tensor([300.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float64)
    assert rate[0] == base[0] and abs(rate[3] - base[3] / 4.0) < 1e-15 and mag == pytest.approx(1.1386, abs=1e-4)
