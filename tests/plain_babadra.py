"""A plain, slow Babadra in float64 on the CPU: one function per mechanism, whole sequences only
(no cache, no state carried between calls, no batches).  It shares no code with the package;
the GPU tests hold the engine to it.

Notation: x [T, width] is the stream, h the normalised input of a sub-layer, W[name] the
checkpoint tensor of that name (linear weights [out, in], applied as h @ W.T)."""
from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import load_file


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    weights = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    return cfg, weights


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The block norms and the final norm: their weight is stored as its distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    """The norms inside the mixers: their weight is the factor itself."""
    return unit_rms(x, eps) * w


def frequencies(rot):
    """(f_i for i < dims/2, the factor on cos and sin).  Without "scaling": base^(-2i/dims) and 1.
    With it, the waves that fit the original context less than ``slow`` times are divided by
    ``factor``, those that fit more than ``fast`` times stay, a linear ramp over the pair index
    between the two, and cos and sin grow by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], float(rot["base"])
    sc = rot.get("scaling")
    out = []

    def index_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    if sc:
        lo = max(math.floor(index_of(sc["fast"])), 0)
        hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        out.append(f)
    grow = 0.1 * math.log(sc["factor"]) + 1.0 if sc else 1.0
    return torch.tensor(out, dtype=torch.float64), grow


def rotate(x, positions, rot, pairing):
    """x [T, heads, n]: the first rot.dims elements turn in pairs by p * f_i, the rest pass.
    ``pairing`` "half": element i with i + dims/2; "neighbours": element 2i with 2i + 1."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    f, grow = frequencies(rot)
    ang = positions.double()[:, None] * f[None, :]
    c, s = (ang.cos() * grow)[:, None, :], (ang.sin() * grow)[:, None, :]
    if pairing == "half":
        a, b = x[..., : dims // 2], x[..., dims // 2: dims]
        return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], dim=-1)


def causal_softmax(scores):
    """scores [T, T] (query, key): softmax over the keys j <= i."""
    T = scores.shape[0]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    return torch.softmax(scores.masked_fill(hidden, -math.inf), dim=-1)


# ----------------------------------------------------------------------------- mixers
def latent_attention(h, W, p, m, eps):
    """Queries through a normed latent; per token one normed key/value latent c and one rotated key
    part shared by all heads; per head the plain key W_uk c and the value W_uv c."""
    T = h.shape[0]
    H, n, nr, nv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = norm_plain(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(T, H, n + nr)
    q_rot = rotate(q[..., n:], pos, m.get("rot"), "neighbours")
    down = h @ W[p + "dkv"].T
    c = norm_plain(down[:, :r], W[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, r:], pos, m.get("rot"), "neighbours")[:, 0]
    k_plain = (c @ W[p + "uk"].T).view(T, H, n)
    v = (c @ W[p + "uv"].T).view(T, H, nv)
    out = torch.zeros(T, H, nv, dtype=torch.float64)
    for a in range(H):
        s = (q[:, a, :n] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = causal_softmax(s) @ v[:, a]
    return out.reshape(T, H * nv) @ W[p + "o"].T


def differential_lambda(W, p, m):
    """The one number of a layer by which the second map is taken off the first."""
    return float(torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum())
                 + m["diff"])


def differential_attention(h, W, p, m, eps):
    """Grouped-query attention with two score maps per head over the same values: each map has its
    own normed and rotated q and k and its own capped scores and softmax; the maps' outputs are
    subtracted, the difference divided by its root mean square per head and scaled."""
    T = h.shape[0]
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = norm_plain((h @ W[p + "q"].T).view(T, H * 2, n), W[p + "q.norm"], eps)
    k = norm_plain((h @ W[p + "k"].T).view(T, G * 2, n), W[p + "k.norm"], eps)
    q = rotate(q, pos, m.get("rot"), "half").view(T, H, 2, n)
    k = rotate(k, pos, m.get("rot"), "half").view(T, G, 2, n)
    v = (h @ W[p + "v"].T).view(T, G, nv)
    lam = differential_lambda(W, p, m)
    cap = m.get("softcap")
    out = torch.zeros(T, H, nv, dtype=torch.float64)
    for a in range(H):
        g = a // (H // G)
        maps = []
        for which in (0, 1):
            s = (q[:, a, which] @ k[:, g, which].T) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            maps.append(causal_softmax(s) @ v[:, g])
        out[:, a] = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return out.reshape(T, H * nv) @ W[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def bounded_gate(g, u, limit):
    """min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    g = g.clamp(max=limit)
    u = u.clamp(-limit, limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def gated_ff(h, W, p, limit):
    return bounded_gate(h @ W[p + "gate"].T, h @ W[p + "up"].T, limit) @ W[p + "down"].T


def route(h, W, p, r):
    """(expert numbers [T, top], their weights [T, top]): the experts with the largest logits,
    weighted by the softmax over those logits alone."""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    best, idx = torch.topk(z, r["top"], dim=-1)
    return idx, torch.softmax(best, dim=-1)


def experts(h, W, p, mlp):
    idx, w = route(h, W, p, mlp["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=torch.float64)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t].tolist(), w[t]):
            out[t] += g * gated_ff(h[t][None], W, p + f"e{e}.", mlp["expert"]["limit"])[0]
    return out


def feed_forward(h, W, p, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, W, p, mlp["limit"])
    return experts(h, W, p, mlp)


# ----------------------------------------------------------------------------- the model
def run_order(cfg):
    """The layers in the order they run: (layer, first of a repeated pass?) pairs."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for t in range(times):
        order += [(i, t > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def layer(x, cfg, W, i):
    eps = cfg["norm"]["eps"]
    spec = cfg["layers"][i]
    p = f"l{i}."
    h = norm_around_zero(x, W[p + "norm1"], eps)
    if spec["type"] == "latent_attention":
        y = latent_attention(h, W, p + "mix.", spec["mixer"], eps)
    elif spec["type"] == "attention":
        y = differential_attention(h, W, p + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = x + y * W[p + "ls1"]
    if spec.get("mlp") is not None:
        h = norm_around_zero(x, W[p + "norm2"], eps)
        x = x + feed_forward(h, W, p + "mlp.", spec["mlp"]) * W[p + "ls2"]
    return x


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and, on request, the stream after every layer run)."""
    T = len(tokens)
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"] + W["pos"][:T]
    first = x
    streams = []
    for i, again in run_order(cfg):
        if again:
            x = x + first
        x = layer(x, cfg, W, i)
        streams.append(x)
    y = norm_around_zero(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        y = cap * torch.tanh(y / cap)
    return (y, torch.stack(streams)) if return_layers else y


def logits(cfg, W, tokens):
    return forward(cfg, W, tokens)


def greedy(cfg, W, prompt, n):
    """n greedy tokens after ``prompt``; with each, the gap between the best and the second logit."""
    ids, out, gaps = list(prompt), [], []
    for _ in range(n):
        row = forward(cfg, W, ids)[-1]
        best = torch.topk(row, 2)
        out.append(int(best.indices[0]))
        gaps.append(float(best.values[0] - best.values[1]))
        ids.append(out[-1])
    return out, gaps
