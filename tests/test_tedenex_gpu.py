"""Tedenex on the GPU against the plain implementation (``tests/plain/tedenex.py``, float64).

Whole models of several small configurations, replayed whole, with a decoded tail, in portions down to
two tokens, and mixed with other requests in a pool so small that pages and state slots are used
again; every mechanism alone (a one-layer model, or its kernel with inputs made so that one key or a
block's edge decides the result); long decoding; greedy generation through the public entry point and
the scheduler.

Errors are relative: the root mean square over the vocabulary of the difference of the logits (mean
taken off) over the standard deviation of the plain model's logits.
"""

import math

import numpy as np
import pytest
import torch

from acorninfer_b200.config.model_config import LayerLoop, TedenexConfig
from tests import traces
from tests.paged import gather_from_pages, rows_layout, scatter_to_pages
from tests.plain import tedenex as plain
from tests.tedenex_tiny import TED_LONG, TEDS, L, att, lat, make_model_dir, random_config, read_weights, wkv
from tests.tiny import random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 4e-5, "bfloat16": 0.1}
LENGTHS = [45, 38, 61, 50, 33, 29]


def rel_err(got, ref):
    d = np.asarray(got, np.float64) - np.asarray(ref, np.float64)
    d = d - d.mean()
    return math.sqrt((d ** 2).mean()) / float(np.std(ref))


@pytest.fixture(scope="module", params=list(TEDS))
def case(request, tmp_path_factory):
    tiny = TEDS[request.param]
    d = make_model_dir(tmp_path_factory.mktemp(request.param), tiny)
    w = read_weights(d)
    reqs = {f"r{i}": random_tokens(n, tiny["cfg"].vocab_size, 4000 + i) for i, n in enumerate(LENGTHS)}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    return tiny, d, reqs, ref


def run_cut(tiny, model_dir, steps, dtype, max_requests=4, watch=None):
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession

    pool = traces.max_live_tokens(steps)
    runner = ModelRunner.from_model_dir(model_dir, dtype=dtype, num_blocks=-(-pool // tiny["page_size"]),
                                        page_size=tiny["page_size"], max_requests=max_requests, max_step_tokens=4096)
    session = TraceSession(runner)

    def step(msg):
        if watch is None:
            return session.step(msg)
        out = session.step(dict(msg, end=[]))
        watch(session, msg)
        session.step({"entries": [], "end": msg["end"]})
        return out

    got = traces.collect(step, steps)
    runner.manager.assert_balanced()
    return got, runner


def check(got, ref, dtype, what, tol=None):
    """Every position within the tolerance.  In bfloat16 a single position may come to twice the tolerance (a head
    whose output nearly cancels is divided by its own small size), as long as the mean over all positions stays
    below a third of it: a fault moves many positions, rounding few."""
    errs = {key: rel_err(row, ref[key[0]][key[1]]) for key, row in got.items()}
    worst = max(errs, key=errs.get)
    tol = tol or TOL[dtype]
    mean = float(np.mean(list(errs.values())))
    if dtype == "bfloat16":
        assert errs[worst] < 2 * tol and mean < tol / 3, f"{what}: {worst}: {errs[worst]:.3e}, mean {mean:.3e}"
    else:
        assert errs[worst] < tol, f"{what}: {worst}: {errs[worst]:.3e}, mean {mean:.3e}"


CUTS = {
    "whole": traces.whole,
    "decode_tail": lambda r: traces.decode_tail(r, tail=24),
    "portions": lambda r: traces.portions(r, sizes=(7, 2, 5, 3, 16, 2, 11, 4)),
    "mixed": lambda r: traces.mixed(r, max_live=4, seed=3, stagger=2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(case, cut, dtype):
    tiny, d, reqs, ref = case
    got, runner = run_cut(tiny, d, CUTS[cut](reqs), dtype)
    assert len(got) == sum(len(t) for t in reqs.values())
    check(got, ref, dtype, cut)
    if cut == "decode_tail":
        assert runner.graph_replays >= len(reqs) * 10        # single-token steps replay captured graphs


def test_cuts_agree_with_each_other_float32(case):
    """The logits at a position do not depend on how the tokens were cut into steps, on what else was
    in the batch or on which pages and slots held them, beyond rounding."""
    tiny, d, reqs, _ = case
    base, _ = run_cut(tiny, d, traces.whole(reqs), "float32")
    for cut in ("decode_tail", "portions", "mixed"):
        other, _ = run_cut(tiny, d, CUTS[cut](reqs), "float32")
        for key, row in base.items():
            assert rel_err(other[key], row) < 1e-5, f"{cut}: {key}"


def test_mixed_trace_uses_pages_and_slots_again(case):
    tiny, d, reqs, _ = case
    steps = CUTS["mixed"](reqs)
    pages: dict = {}
    slots: dict = {}

    def watch(session, msg):
        for rid, rc in session.live.items():
            slots.setdefault(rc.slot, set()).add(rid)
            for table in rc.tables:
                for page in table:
                    pages.setdefault(page, set()).add(rid)

    run_cut(tiny, d, steps, "float32", watch=watch)
    assert len(slots) <= 4 and sum(1 for users in slots.values() if len(users) >= 2) >= 1, slots
    assert sum(1 for users in pages.values() if len(users) >= 2) >= 2, pages


def test_first_step_of_one_token_and_requests_left_out(case):
    """A request whose first step is a single token (the convolution's and the blend's zeros before the
    start, a state that starts at zero, a block that holds one key), then portions beside another request
    that decodes and is left out of some steps."""
    tiny, d, reqs, ref = case
    a, b = reqs["r0"], reqs["r1"]
    steps = [{"entries": [{"id": "r0", "tokens": a[:1], "want": [0]}], "end": []},
             {"entries": [{"id": "r0", "tokens": a[1:3], "want": [0, 1]}, {"id": "r1", "tokens": b[:9], "want": list(range(9))}], "end": []},
             {"entries": [{"id": "r1", "tokens": b[9:10], "want": [0]}], "end": []},
             {"entries": [{"id": "r0", "tokens": a[3:20], "want": list(range(17))}, {"id": "r1", "tokens": b[10:11], "want": [0]}], "end": []},
             {"entries": [{"id": "r0", "tokens": a[20:], "want": list(range(len(a) - 20))}], "end": ["r0"]},
             {"entries": [{"id": "r1", "tokens": b[11:], "want": list(range(len(b) - 11))}], "end": ["r1"]}]
    for i, s in enumerate(steps):
        s["step"] = i
    for dtype in ("float32", "bfloat16"):
        got, _ = run_cut(tiny, d, steps, dtype)
        check(got, ref, dtype, "first token alone")


def test_long_decoding_float32(case):
    """A short prompt and 170 decoded tokens: blocks pass over decoded tokens many times, pages of a cache in
    blocks are given back and taken again, state and convolution memory are carried all the way."""
    tiny, d, _, _ = case
    toks = random_tokens(190, tiny["cfg"].vocab_size, 78)
    ref = {"long": plain.forward(tiny["cfg"].to_dict(), read_weights(d), toks).numpy()}
    steps = traces.decode_tail({"long": toks}, tail=170)
    got, _ = run_cut(tiny, d, steps, "float32")
    check(got, ref, "float32", "long decoding")


def test_long_requests_blocks_over_pages(tmp_path):
    """Requests of a few hundred tokens through blocks of 70 over pages of 16 and latent rows by the hundred:
    the tensor-core kernels walk several chunks of keys whose first and last are cut by the mask, the group in
    blocks gives pages back while a request is still fed, and the states are carried over hundreds of tokens."""
    tiny = TED_LONG
    reqs = {f"L{i}": random_tokens(n, tiny["cfg"].vocab_size, 700 + i) for i, n in enumerate([330, 260, 150])}
    cuts = {"whole": traces.whole, "decode_tail": lambda r: traces.decode_tail(r, tail=90),
            "portions": lambda r: traces.portions(r, sizes=(64, 3, 2, 128, 29, 16, 2, 70)),
            "mixed": lambda r: traces.mixed(r, max_live=3, seed=5, max_portion=80, stagger=1)}
    d = make_model_dir(tmp_path, tiny)
    w = read_weights(d)
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        for cut, build in cuts.items():
            got, runner = run_cut(tiny, d, build(reqs), dtype)
            assert len(got) == sum(len(t) for t in reqs.values())
            check(got, ref, dtype, f"long, {cut}")


@pytest.mark.parametrize("seed", [2, 5, 8, 11])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Models whose sizes are drawn from what real models have, requests of up to 400 tokens, whole, with a decoded
    tail and mixed in a small pool, float32 and bfloat16."""
    import random
    tiny = dict(cfg=random_config(seed), page_size=16, seed=seed)
    d = make_model_dir(tmp_path, tiny, sigma=0.06, sigma_norm=0.1)
    w = read_weights(d)
    rng = random.Random(seed)
    lengths = [rng.randint(250, 400), rng.randint(100, 250), rng.randint(2, 60), 1, rng.randint(60, 150)]
    reqs = {f"q{i}": random_tokens(n, tiny["cfg"].vocab_size, seed * 10 + i) for i, n in enumerate(lengths)}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for dtype, tol in (("float32", 6e-5), ("bfloat16", 0.15)):
        for cut, steps in (("whole", traces.whole(reqs)), ("decode_tail", traces.decode_tail(reqs, tail=40)),
                           ("mixed", traces.mixed(reqs, max_live=4, seed=seed, max_portion=90, stagger=1))):
            got, _ = run_cut(tiny, d, steps, dtype)
            check(got, ref, dtype, f"seed {seed}, {cut}", tol=tol)


def follows_plain(cfg, w, prompt, ids, slack):
    logits = plain.forward(cfg.to_dict(), w, ids[:-1])
    return all(float(logits[i - 1].max() - logits[i - 1][ids[i]]) <= slack for i in range(len(prompt), len(ids)))


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.15)])
def test_greedy_generation_through_the_engine(case, dtype, slack):
    """``generate``: the scheduler with a token budget (prompts cut into portions beside decoding
    requests), sampling on the device, a step ahead of the host."""
    from acorninfer_b200 import generate
    tiny, d, _, _ = case
    cfg = tiny["cfg"]
    w = read_weights(d)
    prompts = [random_tokens(n, cfg.vocab_size, 900 + n) for n in (1, 14, 23, 6, 31)]
    outs = generate(d, prompts, max_new_tokens=12, temperature=0.0, dtype=dtype, page_size=tiny["page_size"],
                    num_blocks=64, max_running=3, chunked_budget=10, watermark_blocks=0, eos_ids=())
    for p, ids in zip(prompts, outs):
        assert len(ids) == len(p) + 12 and follows_plain(cfg, w, p, ids, slack), (dtype, len(p))


def test_preemption_recomputes_state_float32(case):
    """So few pages that requests are preempted and recomputed from their first token: the recurrent
    states, the blend's row and the convolution's memory start over with the slot."""
    from acorninfer_b200.generation import build_engine, generate_with_engine
    tiny, d, _, _ = case
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 40 + n) for n in (20, 18, 13)]
    pages = -(-36 // tiny["page_size"]) * 2 + 1
    tight = build_engine(d, dtype="float32", page_size=tiny["page_size"], num_blocks=pages, watermark_blocks=0, max_running=3)
    got = generate_with_engine(tight, prompts, max_new_tokens=16, eos_ids=())
    w = read_weights(d)
    for p, a in zip(prompts, got):
        assert len(a) == len(p) + 16 and follows_plain(cfg, w, p, a, 1e-4)


# ------------------------------------------------------------------ one mechanism at a time


def _solo(mixer, ff=None, width=48, vocab=90, side=None, loop=None, more=()):
    return TedenexConfig(vocab_size=vocab, hidden_size=width, norm_eps=1e-5, side_dim=side, loop=loop, layers=(L(mixer, ff),) + tuple(more))


_SMALL = wkv(heads=1, dim=4, rank=2)
SOLOS = {
    "time mixing, 5 heads of 6": _solo(wkv(heads=5, dim=6, rank=7)),
    "time mixing, one head of 70, decay through one inner entry": _solo(wkv(heads=1, dim=70, rank=1)),
    "time mixing, heads of 130": _solo(wkv(heads=2, dim=130, rank=4)),
    "attention in blocks of 5, 4 taps, values wider than keys": _solo(att(heads=4, kv_heads=2, dim=6, vdim=22, scale=0.4, conv=4, mask=5)),
    "attention, no blocks, no convolution, values narrower": _solo(att(heads=3, kv_heads=3, dim=18, vdim=4, scale=0.3)),
    "attention in blocks of 1, 2 taps": _solo(att(heads=2, kv_heads=1, dim=8, vdim=8, scale=0.3, conv=2, mask=1)),
    "attention, 9 taps, one head": _solo(att(heads=1, kv_heads=1, dim=16, vdim=16, scale=0.25, conv=9, mask=13)),
    "latent attention, part of the rotated entries rotated": _solo(lat(heads=3, dim=5, rot_dim=8, vdim=7, kv_rank=9, scale=0.3, rot_dims=2, rot_base=50.0, q_rank=4)),
    "latent attention, nothing rotated, queries projected directly": _solo(lat(heads=2, dim=12, rot_dim=4, vdim=6, kv_rank=30, scale=0.2, rot_dims=0)),
    "latent attention, one head, no unshared part wider than the shared one": _solo(lat(heads=1, dim=2, rot_dim=10, vdim=3, kv_rank=6, scale=0.3, rot_dims=10, rot_base=1e6, q_rank=20)),
    "feed-forward, widths no multiple of 8": _solo(_SMALL, ff=37, width=44),
    "side rows of 3 entries, wide feed-forward": _solo(_SMALL, ff=200, side=3),
    "side rows without feed-forward": _solo(_SMALL, side=9),
    "one layer four times": _solo(att(heads=2, kv_heads=1, dim=8, vdim=8, scale=0.3, conv=3, mask=9), ff=20, side=5, loop=LayerLoop(0, 1, 4)),
    "the last two of three layers three times": _solo(_SMALL, ff=16, loop=LayerLoop(1, 3, 3), more=(
        L(lat(heads=2, dim=6, rot_dim=4, vdim=6, kv_rank=8, scale=0.3, rot_dims=4, q_rank=6)), L(wkv(heads=2, dim=5, rank=3), ff=24))),
}


@pytest.mark.parametrize("name", list(SOLOS))
def test_mechanism_alone(name, tmp_path):
    tiny = dict(cfg=SOLOS[name], page_size=4, seed=6)
    d = make_model_dir(tmp_path, tiny, sigma=0.3)
    w = read_weights(d)
    reqs = {f"s{i}": random_tokens(n, tiny["cfg"].vocab_size, 60 + i) for i, n in enumerate([26, 17, 9])}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for cut in ("whole", "portions", "mixed", "decode_tail"):
        steps = {"portions": traces.portions(reqs, sizes=(3, 2, 6, 2)), "decode_tail": traces.decode_tail(reqs, tail=8)}.get(cut) \
            or CUTS[cut](reqs)
        got, _ = run_cut(tiny, d, steps, "float32")
        check(got, ref, "float32", f"{name}, {cut}")
    got, _ = run_cut(tiny, d, CUTS["mixed"](reqs), "bfloat16")
    check(got, ref, "bfloat16", f"{name}, mixed, bfloat16", tol=0.2)


def ops():
    from acorninfer_b200.kernels import ops as o
    return o


def _sloped_attention(q, k, v, scale, slopes, chunk):
    """Plain float64 attention of one row: q [S, nq, d], k [S, nkv, d], v [S, nkv, dv]."""
    S, nq = q.shape[0], q.shape[1]
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    out = []
    for h in range(nq):
        g = h // (nq // k.shape[1])
        out.append(plain.softmax_rows(q[:, h] @ k[:, g].T * scale - slopes[h] * (i - j).double(), ok) @ v[:, g])
    return torch.stack(out, 1)


def _attention_case(befores, qlens, P, d, nq, nkv, chunk, spikes, dtype, kernel, slopes, seed=0):
    """Cache pages and queries for the attention kernels.  ``spikes``: (row, key position): that key and all
    queries of the row get a large component along one direction, so its score stands out wherever it is seen."""
    o = ops()
    g = torch.Generator().manual_seed(seed)
    NP = sum(-(-(b + q) // P) for b, q in zip(befores, qlens)) + 5
    lay = rows_layout(befores, qlens, P, NP, seed=seed)
    k_pages = torch.zeros(NP, nkv, P, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros(NP, nkv, P, d, dtype=dtype, device=DEV)
    full = []
    for r, (b, q) in enumerate(zip(befores, qlens)):
        S = b + q
        k = torch.randn(S, nkv, d, generator=g) * 0.3
        v = torch.randn(S, nkv, d, generator=g)
        qq = torch.randn(S, nq, d, generator=g) * 0.3
        for (rr, j) in spikes:
            if rr == r:
                k[j, :, d - 1] = 6.0
                qq[:, :, d - 1] = 4.0
        k, v, qq = k.to(dtype), v.to(dtype), qq.to(dtype)
        scatter_to_pages(k_pages, lay["tables"][r], k, P)
        scatter_to_pages(v_pages, lay["tables"][r], v, P)
        full.append((qq.double(), k.double(), v.double()))
    q_new = torch.cat([f[0][b:] for f, b in zip(full, befores)]).to(dtype).to(DEV).contiguous().view(-1, nq * d)
    scale = 0.5
    s32 = None if slopes is None else slopes.float().to(DEV)
    common = (k_pages, v_pages, lay["block_table"], lay["page_base"])
    if kernel == "plain":
        out = o.attention_plain(q_new, nq * d, *common, lay["token_row"], lay["positions"], lay["num_tokens"], nq, nkv,
                                d, scale, None, chunk=chunk, slopes32=s32)
    else:
        i32 = dict(dtype=torch.int32, device=DEV)
        starts = np.cumsum([0] + qlens)
        out = torch.zeros((lay["num_tokens"], nq * d), dtype=dtype, device=DEV)
        big = 32 if kernel.startswith("tc") else 10 ** 9          # rows from 32 tokens on go to the tcgen05 kernel
        tiles = torch.tensor([(r, q0) for r, n in enumerate(qlens) if n >= big for q0 in range(0, n, 128)], **i32).view(-1, 2)
        if tiles.shape[0]:
            o.attention_prefill_tc(q_new, nq * d, *common, torch.tensor(starts, **i32), torch.tensor(befores, **i32), tiles,
                                   lay["num_tokens"], nq, nkv, d, scale, None, out=out, chunk=chunk, slopes32=s32)
        tiles = torch.tensor([(r, q0) for r, n in enumerate(qlens) if 1 < n < big for q0 in range(0, n, 64)], **i32).view(-1, 2)
        if tiles.shape[0]:
            o.attention_prefill(q_new, nq * d, *common, torch.tensor(starts, **i32), torch.tensor(befores, **i32), tiles,
                                lay["num_tokens"], nq, nkv, d, scale, None, out=out, chunk=chunk, slopes32=s32)
        singles = torch.tensor([int(starts[r]) for r, n in enumerate(qlens) if n == 1], **i32)
        if singles.numel():
            o.attention_decode(q_new, nq * d, *common, lay["token_row"], lay["positions"], lay["num_tokens"], nq, nkv, d,
                               scale, None, int(kernel[-1]), token_list=singles, out=out, use_tma=False, chunk=chunk,
                               slopes32=s32)
    zero = torch.zeros(nq, dtype=torch.float64)
    want = [_sloped_attention(fq, fk, fv, scale, zero if slopes is None else slopes.double(), chunk)[b:]
            for (fq, fk, fv), b in zip(full, befores)]
    return out.float().cpu().view(-1, nq, d), torch.cat(want)


KERNELS = [(torch.float32, 2e-5, "plain", 24, 6, 3), (torch.bfloat16, 2e-2, "plain", 40, 3, 1),
           (torch.bfloat16, 2e-2, "mma1", 32, 4, 2), (torch.bfloat16, 2e-2, "mma3", 96, 6, 3),
           (torch.bfloat16, 2e-2, "mma2", 128, 8, 1), (torch.bfloat16, 2e-2, "tc2", 128, 8, 2)]


@pytest.mark.parametrize("dtype,tol,kernel,d,nq,nkv", KERNELS)
def test_attention_distance_penalty_in_blocks_of_positions(dtype, tol, kernel, d, nq, nkv):
    """A penalty per head on the distance to the key, in every attention kernel: with blocks of positions (a spiked
    key is seen by the later queries of its own block and by no other, wherever a portion starts, at page borders,
    in prompt rows and decoded tokens) and without (key 3 of 700 still decides the heads with small slopes, the
    near keys those with large ones)."""
    P, C = 16, 48
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nq) for h in range(nq)], dtype=torch.float64)
    befores = [0, 100, 2 * C - 1, 2 * C, 3 * C - 1, 3 * C - 1, C]
    qlens = [200, 70, 1, 1, 1, 1, 2]
    spikes = [(0, 0), (0, C - 1), (0, C), (0, 130), (1, 2 * C), (1, 2 * C + 5), (1, 3 * C - 1), (2, C), (3, 2 * C - 1),
              (4, 2 * C), (5, 2 * C - 1), (6, C - 1)]
    got, want = _attention_case(befores, qlens, P, d, nq, nkv, C, spikes, dtype, kernel, slopes)
    assert (got - want).abs().max() < tol
    at = np.cumsum([0] + qlens)
    assert (got[at[4]] - got[at[5]]).abs().max() > 0.05
    flat, _ = _attention_case(befores, qlens, P, d, nq, nkv, C, spikes, dtype, kernel, None)
    assert (flat - got).abs().max() > 0.05                       # the penalty changes the result, and is not optional
    for C2 in (1, 7, 64, 1000):
        got, want = _attention_case([0, 99, 40], [70, 1, 3], P, d, nq, nkv, C2, [(0, 20), (1, 98), (2, 41)],
                                    dtype, kernel, slopes, seed=C2)
        assert (got - want).abs().max() < tol, C2
    got, want = _attention_case([0, 699], [40, 1], P, d, nq, nkv, None, [(1, 3)], dtype, kernel, slopes)
    assert (got - want).abs().max() < tol
    # other slopes than powers of two, one of them zero
    odd = torch.linspace(0.0, 0.37, nq, dtype=torch.float64)
    got, want = _attention_case([0, 35, 200], [130, 40, 1], P, d, nq, nkv, 64, [(0, 64), (1, 63), (2, 199)], dtype, kernel, odd, seed=5)
    assert (got - want).abs().max() < tol


@pytest.mark.parametrize("long", [False, True])
@pytest.mark.parametrize("H,dim", [(3, 8), (1, 70), (2, 130), (4, 32), (2, 64)])
def test_recurrence_that_reads_the_state_first_across_steps_and_slots(H, dim, long):
    """``o = S^T r + (r . u k) v;  S = diag(w) S + k v^T`` over rows of unequal length from states in scattered
    slots, in three steps (each continues the one before), against the loop; what lies behind S in a slot and
    in other slots is left alone.  ``long``: rows of hundreds of tokens, which run in segments side by side (rows
    shorter than a segment, and of one token, beside them)."""
    o = ops()
    g = torch.Generator().manual_seed(dim)
    slots, cuts = [3, 0, 5], ([9, 1, 17], [1, 12, 2], [40, 1, 1])
    if long:
        cuts = ([700, 1, 130], [3, 400, 64], [1, 1, 300])
        assert o.delta_segments(700, 3, H, dim, dim)[1] >= 3
    tail = 13
    state = torch.full((7, H * dim * dim + tail), 123.0, device=DEV)
    state[slots, :H * dim * dim] = 0
    u = torch.randn(H, dim, generator=g).double()
    seqs = []
    for r in range(3):
        T = sum(c[r] for c in cuts)
        seqs.append(dict(r=torch.randn(T, H, dim, generator=g).double(), k=torch.randn(T, H, dim, generator=g).double() * 0.5,
                         v=torch.randn(T, H, dim, generator=g).double(),
                         w=torch.rand(T, H, dim, generator=g).double() * (0.1 if long else 0.6) + (0.9 if long else 0.4)))
    want = []
    for s in seqs:
        S = torch.zeros(H, dim, dim, dtype=torch.float64)
        out = []
        for t in range(s["r"].shape[0]):
            kv = s["k"][t][:, :, None] * s["v"][t][:, None, :]
            out.append(torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, s["r"][t]))
            S = s["w"][t][:, :, None] * S + kv
        want.append(torch.stack(out))
    i32 = dict(dtype=torch.int32, device=DEV)
    at = [0, 0, 0]
    for lens in cuts:
        cat = lambda key: torch.cat([s[key][a:a + n] for s, a, n in zip(seqs, at, lens)]).float().contiguous().to(DEV)
        y = o.delta_rule(cat("r"), cat("k"), cat("v"), None, cat("w"), state, torch.tensor(np.cumsum([0] + lens), **i32),
                         torch.tensor(slots, **i32), 3, bonus32=u.float().to(DEV), longest_row=max(lens)).cpu().double()
        t0 = 0
        for r, n in enumerate(lens):
            ref = want[r][at[r]:at[r] + n]
            assert (y[t0:t0 + n] - ref).abs().max() < (1e-3 if long else 2e-4) * max(1.0, float(ref.abs().max())), (r, lens)
            t0 += n
            at[r] += n
    assert float(state[1].min()) == 123.0 and float(state[3, H * dim * dim:].min()) == 123.0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("W,off,tail,single", [(20, 7, 3, False), (20, 8, 4, False), (20, 8, 4, True), (520, 4, 0, True),
                                               (22, 8, 2, True)])
def test_blends_with_the_row_before_carry_it_between_steps(dtype, tol, W, off, tail, single):
    """Widths, offsets and slot sizes that are and are not multiples of four (four channels a thread, or one);
    the kept row written by the follow-up kernel, or by the blend kernel itself for rows of one token."""
    o = ops()
    g = torch.Generator().manual_seed(4)
    n = 5
    slots, cuts = [2, 0], ([4, 1], [1, 3], [6, 2])
    rows = [torch.randn(sum(c[r] for c in cuts), W, generator=g).to(dtype) for r in range(2)]
    mu = torch.rand(n, W, generator=g)
    state = torch.zeros(4, off + W + tail, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    at = [0, 0]
    for lens in cuts:
        h = torch.cat([x[a:a + m] for x, a, m in zip(rows, at, lens)]).to(DEV)
        row_start = torch.tensor(np.cumsum([0] + lens), **i32)
        token_row = torch.tensor([r for r, m in enumerate(lens) for _ in range(m)], **i32)
        out = o.token_shift(h, mu.to(DEV), state, off, token_row, row_start, torch.tensor(slots, **i32),
                            update_single=single).float().cpu()
        o.conv_state_update(h, state, off, row_start, torch.tensor(slots, **i32), 2, W, 2, skip_single=single)
        t0 = 0
        for r, m in enumerate(lens):
            x = rows[r].double()
            prev = torch.cat([torch.zeros(1, W, dtype=torch.float64), x[:-1]])[at[r]:at[r] + m]
            cur = x[at[r]:at[r] + m]
            want = cur[None] + (prev - cur)[None] * mu.double()[:, None, :]
            assert (out[:, t0:t0 + m].double() - want).abs().max() < tol
            t0 += m
            at[r] += m
    assert float(state[:, :off].abs().max()) == 0.0
    assert tail == 0 or float(state[:, off + W:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("taps,nq,nkv,d,dv", [(4, 4, 2, 12, 20), (1, 2, 2, 16, 16), (2, 3, 1, 64, 64), (None, 2, 1, 8, 6),
                                              (3, 2, 1, 24, 40), (None, 2, 2, 32, 8), (5, 2, 1, 16, 16), (4, 3, 3, 128, 128)])
@pytest.mark.parametrize("pad,single,long", [(3, False, False), (8, False, False), (8, True, False), (8, True, True)])
def test_bias_convolution_norm_and_cache_write_across_steps(dtype, tol, taps, nq, nkv, d, dv, pad, single, long):
    """The projected rows of two requests in three steps: bias, convolution over time (its memory in the state
    slot between steps, zeros before a request's start), q/k norm; queries into their own buffer, keys and
    values into pages.  Rows and state slots whose sizes are and are not multiples of four (four channels a lane,
    or one); the memory moved on by the follow-up kernel, or for rows of one token by the convolving kernel; steps of
    hundreds of tokens (a lane then walks several tokens, also across the border of two rows)."""
    o = ops()
    g = torch.Generator().manual_seed(d)
    P, eps = 4, 1e-5
    C = (nq + nkv) * d + nkv * dv
    cuts, slots = ([5, 1], [1, 2], [7, 3]), [1, 3]
    if long:
        cuts = ([290, 1], [1, 331], [3, 1201], [1, 1])
    pages = 12 if not long else 800
    totals = [sum(c[r] for c in cuts) for r in range(2)]
    proj = [torch.randn(T, C + pad, generator=g).to(dtype) for T in totals]            # rows wider than the channels
    bias = torch.randn(C, generator=g)
    w = None if taps is None else torch.randn(C, taps, generator=g) * 0.5
    qw, kw = torch.rand(d, generator=g) + 0.5, torch.rand(d, generator=g) + 0.5
    lay = rows_layout([0, 0], totals, P, pages, seed=1)
    k_pages = torch.zeros(pages, nkv, P, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros(pages, nkv, P, dv, dtype=dtype, device=DEV)
    state = torch.zeros(5, max(((taps or 1) - 1) * C, 1) + (2 if pad == 3 else 4 - max(((taps or 1) - 1) * C, 1) % 4), device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    at = [0, 0]
    got_q = [[], []]
    for lens in cuts:
        rows = torch.cat([x[a:a + m] for x, a, m in zip(proj, at, lens)]).to(DEV)
        row_start = torch.tensor(np.cumsum([0] + lens), **i32)
        token_row = torch.tensor([r for r, m in enumerate(lens) for _ in range(m)], **i32)
        positions = torch.tensor([a + i for a, m in zip(at, lens) for i in range(m)], **i32)
        q_out = torch.zeros(sum(lens), nq * d + 8, dtype=dtype, device=DEV)
        conv = None if taps is None else o.ShortConv(w.to(DEV), state, 0, row_start, torch.tensor(slots, **i32),
                                                     update_single=single)
        o.qk_rope_kv(rows, qw.to(DEV), kw.to(DEV), torch.zeros(0, device=DEV), positions, token_row, lay["block_table"],
                     lay["page_base"], k_pages, v_pages, nq, nkv, d, 0, False, eps, value_dim=dv, bias32=bias.to(DEV),
                     conv=conv, q_out=q_out)
        if taps is not None and taps > 1:
            o.conv_state_update(rows, state, 0, row_start, torch.tensor(slots, **i32), 2, C, taps, skip_single=single,
                                bias32=bias.to(DEV))
        assert float(q_out[:, nq * d:].abs().max()) == 0.0
        t0 = 0
        for r, m in enumerate(lens):
            got_q[r].append(q_out[t0:t0 + m, :nq * d].float().cpu())
            t0 += m
            at[r] += m
    for r, T in enumerate(totals):
        u = proj[r][:, :C].double() + bias.double()
        x = u if taps is None else plain.conv_over_time(u, w.double())
        q = plain.norm_plain(x[:, :nq * d].view(T, nq, d), qw.double(), eps)
        k = plain.norm_plain(x[:, nq * d:(nq + nkv) * d].view(T, nkv, d), kw.double(), eps)
        v = x[:, (nq + nkv) * d:].view(T, nkv, dv)
        assert (torch.cat(got_q[r]).double().view(T, nq, d) - q).abs().max() < tol
        assert (gather_from_pages(k_pages, lay["tables"][r], T, P).double().cpu() - k).abs().max() < tol
        assert (gather_from_pages(v_pages, lay["tables"][r], T, P).double().cpu() - v).abs().max() < tol * max(1.0, float(v.abs().max()))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_activations_side_rows_norm_pairs_and_the_recurrence_inputs(dtype, tol):
    o = ops()
    g = torch.Generator().manual_seed(8)
    T, W = 13, 60
    # plain activations, on rows with a stride
    x = torch.randn(T, W + 4, generator=g).to(dtype)
    for kind, f in (("relu_squared", plain.relu_squared), ("tanh", torch.tanh), ("gelu_tanh", plain.gelu_tanh), ("silu", plain.silu)):
        for cols in (W, 37):
            got = o.activation(x.to(DEV)[:, 4:4 + cols], kind).double().cpu()
            want = f(x[:, 4:4 + cols].double())
            assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max())), kind
    # a token's columns of a side table, gated
    table = torch.randn(50, 23, generator=g).to(dtype)
    ids = torch.randint(0, 50, (T,), generator=g, dtype=torch.int32)
    z = torch.randn(T, 5, generator=g).to(dtype)
    got = o.side_gate(z.to(DEV), ids.to(DEV), table.to(DEV), 11).double().cpu()
    assert (got - plain.gelu_tanh(z.double()) * table[ids.long()][:, 11:16].double()).abs().max() < tol * 4
    # the same with the gate's product in front: as the epilogue of the tensor-core product (bfloat16, few rows), or as
    # product and gate kernel (float32; many rows; a width the tensor-core product does not take)
    for rows, K, n in ((T, 48, 5), (3, 64, 12), (300, 48, 5), (T, 44, 5)):
        xs = torch.randn(rows, K, generator=g).to(dtype)
        wg = (torch.randn(n, K, generator=g) / math.sqrt(K)).to(dtype)
        ids2 = torch.randint(0, 50, (rows,), generator=g, dtype=torch.int32)
        got = o.side_gate_linear(xs.to(DEV), wg.to(DEV), ids2.to(DEV), table.to(DEV).contiguous(), 17 - n).double().cpu()
        want = plain.gelu_tanh(xs.double() @ wg.double().T) * table[ids2.long()][:, 17 - n:17].double()
        assert (got - want).abs().max() < tol * 6, (rows, K, n)
    # a sublayer's output norm added to the stream, and the next sublayer's input norm of the sum
    # (widths that are no multiple of four: an entry a thread; the others four, with 1, 2 or 4 such parts a thread)
    for Wn in (W, 62, 4, 1000, 1028, 2048, 2052, 4100, 8192, 8196):
        resid = torch.randn(T, Wn, generator=g) * 3
        y = torch.randn(T, Wn, generator=g).to(dtype)
        w1, w2 = torch.rand(Wn, generator=g) + 0.5, torch.rand(Wn, generator=g) + 0.5
        stream = resid.clone().to(DEV)
        normed = o.rmsnorm_add_norm(stream, y.to(DEV), w1.to(DEV), 1e-5, w2.to(DEV), 1e-6).double().cpu()
        s = resid.double() + plain.norm_plain(y.double(), w1.double(), 1e-5)
        assert (stream.cpu().double() - s).abs().max() < 1e-5, Wn
        assert (normed - plain.norm_plain(s, w2.double(), 1e-6)).abs().max() < tol * 4, Wn
        stream = resid.clone().to(DEV)
        rounded = o.rmsnorm_add(stream, y.to(DEV), w1.to(DEV), 1e-5)
        assert (stream.cpu().double() - s).abs().max() < 1e-5, Wn
        assert rounded is None if dtype == torch.float32 else torch.equal(rounded.float().cpu(), stream.cpu().to(dtype).float()), Wn
    # the recurrence's inputs: float32 copies, decay = exp(-exp(z + w0)), gate = silu(g)
    H, d = 3, 10
    r, k, v, gg = (torch.randn(T, H * d, generator=g).to(dtype) for _ in range(4))
    zz, w0 = torch.randn(T, H * d, generator=g), torch.randn(H * d, generator=g) - 1
    r32, k32, v32, decay, gate = o.wkv_prep(r.to(DEV), k.to(DEV), v.to(DEV), gg.to(DEV), zz.to(DEV), w0.to(DEV), H)
    assert r32.shape == (T, H, d) and torch.equal(r32.cpu().view(T, -1), r.float()) and torch.equal(v32.cpu().view(T, -1), v.float())
    assert (decay.cpu().double().view(T, -1) - torch.exp(-torch.exp(zz.double() + w0.double()))).abs().max() < 1e-6
    assert (gate.cpu().double().view(T, -1) - plain.silu(gg.double())).abs().max() < 1e-5
    # the recurrence's output step with a weight per head
    o32, g32 = torch.randn(T, H, d, generator=g), torch.rand(T, H, d, generator=g)
    wn = torch.rand(H * d, generator=g) + 0.5
    got = o.delta_out(o32.to(DEV), g32.to(DEV), wn.to(DEV), 1e-5, dtype).double().cpu()
    want = plain.rms(o32.double(), 1e-5).reshape(T, H * d) * wn.double() * g32.double().reshape(T, H * d)
    assert (got - want).abs().max() < tol * 4


@pytest.mark.parametrize("M", [3, 32, 200])
def test_plain_activations_on_a_product(M):
    """The square of relu and tanh on a product: in the epilogue of the one-CTA tcgen05 kernel for few bfloat16 rows,
    by the activation kernel after the product otherwise (more rows, float32)."""
    o = ops()
    g = torch.Generator().manual_seed(M)
    K, N = 96, 136
    x, w = torch.randn(M, K, generator=g) * 0.5, torch.randn(N, K, generator=g) * 0.2
    for dtype, tol in ((torch.bfloat16, 3e-2), (torch.float32, 1e-5)):
        xd, wd = x.to(dtype), w.to(dtype)
        z = xd.double() @ wd.double().T
        for act, f in (("relu_squared", plain.relu_squared), ("tanh", torch.tanh)):
            got = o.linear(xd.to(DEV), wd.to(DEV), out_dtype=dtype, act=act).double().cpu()
            assert got.shape == (M, N) and (got - f(z)).abs().max() < tol * max(1.0, float(f(z).abs().max())), (dtype, act)
