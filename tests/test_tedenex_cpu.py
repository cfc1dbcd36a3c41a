"""Tedenex without a GPU: its configuration, the model as data (a span of layers as schedule entries with
caches of their own), what its layers ask of the cache manager, and properties of the plain implementation."""

import copy

import pytest
import torch

from acorninfer_b200.cache.manager import CacheManager
from acorninfer_b200.config.model_config import ConfigError, LayerLoop, TedenexConfig
from acorninfer_b200.models.decoder import Decoder, expected_tensors
from acorninfer_b200.registry import config_from_dict, spec_for
from tests.plain import tedenex as plain
from tests.tedenex_tiny import TED_A, TED_B, TEDS, L, att, make_model_dir, random_config, read_weights, wkv
from tests.tiny import random_tokens


@pytest.mark.parametrize("name", list(TEDS))
def test_config_round_trip_and_registry(name):
    cfg = TEDS[name]["cfg"]
    raw = cfg.to_dict()
    assert raw["architecture"] == "Tedenex" and len(raw["layers"]) == len(cfg.layers)
    again = config_from_dict(raw)
    assert isinstance(again, TedenexConfig) and again == cfg
    for seed in range(6):
        drawn = random_config(seed)
        assert config_from_dict(drawn.to_dict()) == drawn


def test_config_errors_name_the_key():
    raw = TED_A["cfg"].to_dict()
    for path, value, word in ((("layers", 0, "type"), "mamba", "type"), (("layers", 2, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mixer", "conv"), 0, "conv"),
                              (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"), (("layers", 0, "mlp", "kind"), "moe", "kind"),
                              (("loop", "stop"), 9, "loop"), (("loop", "times"), 0, "loop"), (("token_side", "dim"), 0, "dim"),
                              (("norm", "eps"), 0.0, "eps"), (("layers", 2, "mixer", "kv_from"), 0, "kv_from")):
        bad = copy.deepcopy(raw)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["layers"][0]["mixer"]["heads"]
    with pytest.raises(ConfigError, match="heads"):
        config_from_dict(bad)


def test_model_as_data_schedule_and_cache_needs():
    cfg = TED_A["cfg"]
    spec = spec_for(cfg)
    assert [ls.mixer.kind for ls in spec.layers] == ["time_mix", "attention", "latent_attention"]
    assert all(ls.block.kind == "sandwich" and set(ls.extras) == {"side"} for ls in spec.layers)
    assert set(spec.layers[0].norms) == {"mixer_in", "mixer_out", "feed_forward_in", "feed_forward_out"}
    assert set(spec.layers[1].norms) == {"mixer_in", "mixer_out"} and spec.layers[1].feed_forward is None
    # layers 0 and 1 run twice; the second pass takes the token rows in again at its first layer
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == [(0, False), (1, False), (0, True), (1, False), (2, False)]
    names = expected_tensors(spec)
    for n in ("embed", "side.embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2b", "l0.mix.mu.w", "l0.mix.w1", "l0.mix.u",
              "l0.side.gate", "l1.mix.q.b", "l1.mix.v.conv", "l1.mix.k.norm", "l2.mix.dq", "l2.mix.dq.norm", "l2.mix.uq",
              "l2.mix.dkv.norm", "l2.mlp.up", "l2.side.norm"):
        assert n in names, n
    assert "l1.norm2" not in names and "l2.mix.q" not in names and "l2.mix.sink" not in names and "head" not in names
    assert names["side.embed"].shape == (190, 30) and names["l1.mix.v.conv"].shape == (2 * 20, 3)
    assert names["l0.mix.u"].shape == (3, 8) and names["l0.mix.norm"].shape == (24,)
    dec = Decoder(spec, torch.float32, "cpu", page_size=8)
    kv, state = dec.cache_needs()
    # every run keeps its own: two runs of the time mixer (S and the row before), two of the attention (pages in
    # blocks of positions and the convolution's memory), one of the latent attention (one row a token, no values)
    assert sorted(kv) == [1, 3, 4] and sorted(state) == [0, 1, 2, 3]
    assert state[0].shape == (3 * 8 * 8 + 72,) and state[1].shape == (2 * (4 * 12 + 2 * 12 + 2 * 20),)
    assert kv[1].chunk == 11 and kv[1].value_dim == 20 and kv[4].values is False and kv[4].head_dim == 26
    # no span, no side rows, a convolution of one tap (no memory), no mask
    b = spec_for(TED_B["cfg"])
    assert len(b.schedule) == 1 + 3 * 3 and not any(ls.extras for ls in b.layers)
    assert sum(e.add_embedding for e in b.schedule) == 2 and [e.layer for e in b.schedule if e.add_embedding] == [1, 1]
    kvb, stb = Decoder(b, torch.float32, "cpu", page_size=4).cache_needs()
    assert 0 not in stb and kvb[0].chunk is None and 3 in stb and 3 in kvb


def test_pages_of_a_cache_in_blocks_are_given_back(tmp_path):
    spec = spec_for(TED_A["cfg"])
    dec = Decoder(spec, torch.float32, "cpu", page_size=8)
    kv, state = dec.cache_needs()
    m = CacheManager(kv, state, 40, 8, 2, allocate=False)
    rc = m.open("a")
    for length in (5, 11, 12, 40, 45):
        m.extend(rc, length)
        m.commit(rc, length)
        g_att, g_lat = m.group_of(1), m.group_of(4)
        # a later query at position >= length starts its block of 11 positions at length - length % 11
        assert rc.page_base[g_att] == (length - length % 11) // 8
        assert rc.page_base[g_lat] == 0 and len(rc.tables[g_lat]) == -(-length // 8)      # the latent rows all stay
    assert m.group_of(1) == m.group_of(3)           # both runs of the attention layer: pools of one group, pages of their own
    m.close(rc)
    m.assert_balanced()


def test_plain_implementation_is_causal_and_blocks_cut_attention():
    cfg = TedenexConfig(vocab_size=50, hidden_size=24, norm_eps=1e-5, side_dim=4, loop=LayerLoop(0, 1, 2), layers=(
        L(att(heads=2, kv_heads=1, dim=6, vdim=5, scale=0.4, conv=3, mask=7), ff=16), L(wkv(heads=2, dim=4, rank=3), ff=None)))
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        w = read_weights(make_model_dir(tmp, dict(cfg=cfg, seed=3), sigma=0.3))
    toks = random_tokens(30, 50, 1)
    full = plain.forward(cfg.to_dict(), w, toks)
    assert torch.allclose(plain.forward(cfg.to_dict(), w, toks[:19]), full[:19], atol=1e-12)      # causal
    # a convolution sees taps - 1 rows back and no further; before the start it sees zeros
    u = torch.randn(9, 3, dtype=torch.float64)
    taps = torch.randn(3, 4, dtype=torch.float64)
    y = plain.conv_over_time(u, taps)
    assert torch.allclose(y[0], taps[:, 3] * u[0]) and torch.allclose(y[5], (taps.T * u[2:6]).sum(0))
    # the schedule of a span: start 1, stop 3, three times, between a first and a last layer
    runs = plain.layer_runs({"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 3}})
    assert runs == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]


def test_plain_time_mix_state_form_equals_the_sum_over_the_past():
    """o_t = sum_{s<t} (r_t . (prod_{s<j<t} w_j) k_s) v_s + (r_t . u k_t) v_t."""
    g = torch.Generator().manual_seed(0)
    T, W, H, d = 7, 10, 2, 3
    names = {"mu." + s: torch.rand(W, generator=g, dtype=torch.float64) for s in "rkvgw"}
    for s in "rkvg":
        names[s] = torch.randn(H * d, W, generator=g, dtype=torch.float64)
    names.update(w1=torch.randn(4, W, generator=g, dtype=torch.float64), w2=torch.randn(H * d, 4, generator=g, dtype=torch.float64),
                 w0=torch.randn(H * d, generator=g, dtype=torch.float64) - 1, u=torch.randn(H, d, generator=g, dtype=torch.float64),
                 norm=torch.ones(H * d, dtype=torch.float64), o=torch.eye(H * d, dtype=torch.float64))
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    got = plain.wkv(h, {"heads": H, "dim": d}, lambda n: names[n], 1e-5)
    prev = torch.cat([torch.zeros(1, W, dtype=torch.float64), h[:-1]])
    mix = lambda s: h + (prev - h) * names["mu." + s]
    r, k, v = ((mix(s) @ names[s].T).view(T, H, d) for s in "rkv")
    gate = plain.silu(mix("g") @ names["g"].T)
    dec = torch.exp(-torch.exp(torch.tanh(mix("w") @ names["w1"].T) @ names["w2"].T + names["w0"])).view(T, H, d)
    o = torch.zeros(T, H, d, dtype=torch.float64)
    for t in range(T):
        for a in range(H):
            o[t, a] = (r[t, a] * names["u"][a] * k[t, a]).sum() * v[t, a]
            for s in range(t):
                carry = torch.ones(d, dtype=torch.float64)
                for j in range(s + 1, t):
                    carry = carry * dec[j, a]
                o[t, a] += (r[t, a] * carry * k[s, a]).sum() * v[s, a]
    want = plain.rms(o, 1e-5).reshape(T, H * d) * gate
    assert torch.allclose(got, want, atol=1e-10)
