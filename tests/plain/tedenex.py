"""Plain implementation of Tedenex: whole sequences, no cache, float64, one function per mechanism.

It shares no code with the package: it takes the ``config.json`` dictionary and the checkpoint's
tensors by name, and every recurrence is a loop over tokens.  Notation: T tokens, W the width; a head
has ``dim`` query/key entries and ``vdim`` value entries; ``m`` is a mixer's part of the configuration
and ``w(name)`` the tensor ``<layer>.mix.<name>`` (``<layer>.mlp.<name>`` in a feed-forward).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The model's norm: its weight is stored as the distance from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + torch.exp(-z))


def relu_squared(z):
    return z.clamp(min=0) ** 2


def conv_over_time(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotate_pairs(x, base, dims):
    """x [T, heads, n]: entries (2i, 2i+1), i < dims/2, of every head are turned by t * base^(-2i/dims)."""
    if dims == 0:
        return x
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def softmax_rows(score, ok):
    score = score.masked_fill(~ok, float("-inf"))
    score = score - score.max(-1, keepdim=True).values
    p = torch.exp(score)
    return p / p.sum(-1, keepdim=True)


def attention(h, m, w, eps):
    """Grouped-query attention with biased projections, a short convolution over time on q, k, v, a per-head
    norm of q and k, no rotation, a penalty slope_a * (i - j) on the score and blocks of ``mask.size``
    positions: query i reads key j <= i of its own block only."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    def project(name, heads, width):
        u = h @ w(name).T + w(name + ".b")
        return (conv_over_time(u, w(name + ".conv")) if m.get("conv") else u).view(T, heads, width)

    q, k, v = project("q", H, d), project("k", G, d), project("v", G, dv)
    q = norm_plain(q, w("q.norm"), eps)
    k = norm_plain(k, w("k.norm"), eps)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if m.get("mask") is not None:
        ok = ok & (i // m["mask"]["size"] == j // m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        score = (q[:, a] @ k[:, g].T) * m["scale"] - slope * (i - j).to(F64)
        out[:, a] = softmax_rows(score, ok) @ v[:, g]
    return out.reshape(T, H * dv) @ w("o").T


def wkv(h, m, w, eps):
    """Time mixing with a matrix state per head: every projection reads its own blend of the token's row and
    the row before it; the state decays per key channel by a factor computed from the token."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def blend(s):
        return h + (prev - h) * w("mu." + s)

    r = (blend("r") @ w("r").T).view(T, H, d)
    k = (blend("k") @ w("k").T).view(T, H, d)
    v = (blend("v") @ w("v").T).view(T, H, d)
    gate = silu(blend("g") @ w("g").T)
    decay = torch.exp(-torch.exp(torch.tanh(blend("w") @ w("w1").T) @ w("w2").T + w("w0"))).view(T, H, d)
    u = w("u")
    S = torch.zeros(H, d, d, dtype=F64)
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    y = rms(o, eps).reshape(T, H * d) * w("norm") * gate
    return y @ w("o").T


def latent_attention(h, m, w, eps):
    """Attention whose keys and values (and, with ``q_rank``, queries) come through low-rank latents; a head's key
    is an up-projection of the normed latent beside one rotated part that all heads share."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    if m.get("q_rank") is not None:
        q = (norm_plain(h @ w("dq").T, w("dq.norm"), eps) @ w("uq").T).view(T, H, d + r)
    else:
        q = (h @ w("q").T).view(T, H, d + r)
    qu, qr = q[..., :d], rotate_pairs(q[..., d:], m["rot"]["base"], m["rot"]["dims"])
    z = h @ w("dkv").T
    c = norm_plain(z[:, :rank], w("dkv.norm"), eps)
    kr = rotate_pairs(z[:, None, rank:], m["rot"]["base"], m["rot"]["dims"])[:, 0]
    ku = (c @ w("uk").T).view(T, H, d)
    v = (c @ w("uv").T).view(T, H, dv)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        score = (qu[:, a] @ ku[:, a].T + qr[:, a] @ kr.T) * m["scale"]
        out[:, a] = softmax_rows(score, ok) @ v[:, a]
    return out.reshape(T, H * dv) @ w("o").T


MIXERS = {"attention": attention, "wkv": wkv, "latent_attention": latent_attention}


def dense_ff(h, w):
    return relu_squared(h @ w("up").T) @ w("down").T


def token_side(x, tokens, tensors, layer, index, dim, eps):
    """What a layer adds from the token itself: its slice of the side table, gated by the stream."""
    e = tensors["side.embed"][tokens][:, index * dim:(index + 1) * dim]
    g = gelu_tanh(x @ tensors[f"{layer}.side.gate"].T) * e
    y = g @ tensors[f"{layer}.side.proj"].T
    return rms(y, eps) * tensors[f"{layer}.side.norm"]


def layer_runs(cfg):
    """The order in which layers run: the looped span repeated in place."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for p in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, p > 0 and i == loop["start"]))      # True: the token rows are added before this run
    runs += [(i, False) for i in range(loop["stop"], n)]
    return runs


def forward(cfg, tensors, tokens, return_layers=False):
    """tokens: list of ids of one sequence.  Returns float64 logits [T, vocab] (and the stream after every run)."""
    t64 = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = t64["embed"][ids]
    x = x0.clone()
    after = []
    for i, add_rows in layer_runs(cfg):
        L, name = cfg["layers"][i], f"l{i}"
        if add_rows:
            x = x + x0
        w = lambda n, p=name: t64[f"{p}.mix.{n}"]
        y = MIXERS[L["type"]](norm_one_plus(x, t64[name + ".norm1"], eps), L["mixer"], w, eps)
        x = x + norm_one_plus(y, t64[name + ".norm1b"], eps)
        if L.get("mlp") is not None:
            wf = lambda n, p=name: t64[f"{p}.mlp.{n}"]
            y = dense_ff(norm_one_plus(x, t64[name + ".norm2"], eps), wf)
            x = x + norm_one_plus(y, t64[name + ".norm2b"], eps)
        if cfg.get("token_side") is not None:
            x = x + token_side(x, ids, t64, name, i, cfg["token_side"]["dim"], eps)
        after.append(x.clone())
    logits = norm_one_plus(x, t64["final.norm"], eps) @ t64["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
