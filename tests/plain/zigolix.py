"""Plain implementation of Zigolix: whole sequences, no cache, float64, one function per mechanism.

It shares no code with the package: it takes the ``config.json`` dictionary and the checkpoint's tensors
by name.  Notation: T tokens, W the width; a query/key head has ``dim`` entries, a value head ``vdim``; ``m``
is a mixer's part of the configuration and ``w(name)`` the tensor ``<layer>.mix.<name>``
(``<layer>.mlp.<name>`` in a feed-forward).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def stretched_frequencies(rot):
    """Turning rates of the rotated pairs and the factor on cos and sin, from ``rot`` (base, dims, scaling)."""
    n, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / n) for i in range(n // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0

    def pair_of(turns):
        return n * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo, hi = max(math.floor(pair_of(sc["fast"])), 0), min(math.ceil(pair_of(sc["slow"])), n - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_neighbours(x, rot):
    """x [T, heads, n]: entries (2i, 2i + 1), i < dims / 2, of every head turned by t * rate_i; the rest as it is."""
    if not rot or not rot.get("dims"):
        return x
    T, n = x.shape[0], rot["dims"]
    rate, mag = stretched_frequencies(rot)
    a = torch.arange(T, dtype=F64)[:, None] * rate[None, :]             # [T, n/2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    y = x.clone()
    y[..., 0:n:2] = u * c - v * s
    y[..., 1:n:2] = v * c + u * s
    return y


def visible(T, window):
    """[T, T] bool: query i reads key j when 0 <= i - j < window (no window: every earlier key)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j) < window
    return ok


def sink_softmax(scores, ok, sink=None):
    """Softmax over the visible keys of each row; ``sink`` [heads] adds exp(sink) to the denominator.
    scores [heads, T, T]."""
    s = scores.masked_fill(~ok[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def sink_attention(h, m, w, eps):
    """Grouped-query attention whose values are the keys as projected; part of each head rotated; q and k
    brought to unit root mean square after the rotation; sliding window; a sink per head."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    if m["vdim"] != d:
        raise ValueError("values are the keys: vdim must equal dim")
    q = (h @ w("q").T).view(T, H, d)
    k = (h @ w("k").T).view(T, G, d)
    v = k
    q = unit_rms(rotate_neighbours(q, m.get("rot")), eps)
    k = unit_rms(rotate_neighbours(k, m.get("rot")), eps)
    ok = visible(T, (m.get("mask") or {}).get("size"))
    group = torch.arange(H) // (H // G)
    scores = torch.einsum("thd,shd->hts", q, k[:, group]) * m["scale"]
    p = sink_softmax(scores, ok, w("sink"))
    o = torch.einsum("hts,shd->thd", p, v[:, group])
    return o.reshape(T, H * d) @ w("o").T


def differential_attention(h, m, w, eps):
    """Two score maps per head over the same values, combined as a1 - lambda a2; capped scores; biases;
    a unit-rms norm per head times (1 - diff); a gate on the heads' outputs."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w("q").T + w("q.b")).view(T, H, 2, d)
    k = (h @ w("k").T + w("k.b")).view(T, G, 2, d)
    v = (h @ w("v").T + w("v.b")).view(T, G, dv)
    ok = visible(T, (m.get("mask") or {}).get("size"))
    group = torch.arange(H) // (H // G)
    cap = m.get("softcap")
    outs = []
    for a in range(2):
        s = torch.einsum("thd,shd->hts", q[:, :, a], k[:, group, a]) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        p = sink_softmax(s, ok)
        outs.append(torch.einsum("hts,shd->thd", p, v[:, group]))
    lam = torch.exp((w("lq1") * w("lk1")).sum()) - torch.exp((w("lq2") * w("lk2")).sum()) + m["diff"]
    o = unit_rms(outs[0] - lam * outs[1], eps) * (1.0 - m["diff"])
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ w("g").T)
    return o @ w("o").T


MIXERS = {"attention": sink_attention, "attention_2": differential_attention}


def dense_ff(h, w):
    return (gelu_tanh(h @ w("gate").T) * (h @ w("up").T)) @ w("down").T


def capped_expert(h, w, prefix, limit):
    g = (h @ w(prefix + "gate").T).clamp(max=limit)
    u = (h @ w(prefix + "up").T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w(prefix + "down").T


def routed_ff(h, f, w, gaps=None):
    """The ``top`` experts of largest softmax score, weighted by their scores over the scores' sum, plus a
    shared expert that every token takes.  ``gaps`` (a list) receives, per token, how far the last chosen
    expert's router logit lies above the first one left out (infinity when all are chosen)."""
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w("router").T
    s = torch.softmax(z, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        ranked = sorted(range(E), key=lambda e: (-float(s[t, e]), e))
        order = ranked[:top]
        if gaps is not None:
            gaps.append(float(z[t, ranked[top - 1]] - z[t, ranked[top]]) if top < E else math.inf)
        total = sum(s[t, e] for e in order) + 1e-20
        for e in order:
            out[t] += (s[t, e] / total) * capped_expert(h[t:t + 1], w, f"e{e}.", f["expert"]["limit"])[0]
    if f.get("shared"):
        out = out + capped_expert(h, w, "shared.", f["shared"]["limit"])
    return out


def layer_runs(cfg):
    """(layer, pass number if the run opens a pass of the looped span else None), in running order."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for p in range(loop["times"]):
        runs += [(i, p if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, tensors, tokens, return_layers=False, router_gaps=None):
    """tokens: ids of one sequence.  float64 logits [T, vocab] (and the stream after every layer run).
    ``router_gaps`` (a list) receives one list per run of a routed feed-forward: see ``routed_ff``."""
    t64 = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x0 = t64["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    after = []
    for i, opens in layer_runs(cfg):
        L, name = cfg["layers"][i], f"l{i}"
        if opens is not None:
            x = torch.cat([x, x0], dim=-1) @ t64["loop.in"].T + t64["loop.step"][opens]
        wm = lambda n, p=name: t64[f"{p}.mix.{n}"]
        x = x + MIXERS[L["type"]](norm(x, t64[name + ".norm1"], eps), L["mixer"], wm, eps)
        f = L.get("mlp")
        if f is not None:
            wf = lambda n, p=name: t64[f"{p}.mlp.{n}"]
            hh = norm(x, t64[name + ".norm2"], eps)
            if f.get("kind", "dense") == "dense":
                x = x + dense_ff(hh, wf)
            else:
                gaps = [] if router_gaps is not None else None
                x = x + routed_ff(hh, f, wf, gaps)
                if router_gaps is not None:
                    router_gaps.append(gaps)
        after.append(x.clone())
    logits = (norm(x, t64["final.norm"], eps) @ t64["head"].T) * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(after)) if return_layers else logits
