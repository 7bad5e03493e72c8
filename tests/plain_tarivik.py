"""A plain, slow implementation of the Tarivik design: one function per mechanism, whole
sequences at a time, float64 on the CPU.  It shares no code with the package; the tests hold
the package's step function, cache, states and kernels to it.

Notation: x [T, W] is the residual stream of one sequence, h the input of a sub-layer,
``w`` a dict of the layer's tensors by checkpoint name without the layer prefix."""
from __future__ import annotations

import json
import math
import os

import torch

F64 = torch.float64


def load_folder(folder):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    return cfg, {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, weight, groups, eps):
    """RMS norm of every one of ``groups`` equal consecutive parts of the last axis, then the weight."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rms(parts, eps).reshape(shape) * weight


def input_conv(x, taps_weight):
    """x + causal convolution over time per channel; taps_weight [W, taps], its last column is the
    current token's, zeros before the sequence's start."""
    T, W = x.shape
    taps = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, W, dtype=x.dtype), x])
    out = x.clone()
    for j in range(taps):
        out = out + padded[j:j + T] * taps_weight[:, j]
    return out


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def hgrn2(h, w, cfg, eps):
    H, K, V = cfg["heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = silu(h @ w["q"].T).view(T, H, K)
    v = (h @ w["v"].T).view(T, H, V)
    low = w["lower"]
    f = (low + (1 - low) * torch.sigmoid(h @ w["f"].T + w["f.b"])).view(T, H, K)
    S = torch.zeros(H, K, V, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    out = rms(out, eps) * w["norm"]
    return out.reshape(T, H * V) @ w["o"].T


def mlstm(h, w, cfg, eps):
    H, K, V, cap = cfg["heads"], cfg["dim"], cfg["vdim"], float(cfg["gate_cap"])
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, K) * K ** -0.5
    k = (h @ w["k"].T).view(T, H, K)
    v = (h @ w["v"].T).view(T, H, V)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)                       # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    S = torch.zeros(H, K, V, dtype=h.dtype)
    n = torch.zeros(H, K, dtype=h.dtype)
    m = torch.zeros(H, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        keep, write = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    out = rms(out, eps).reshape(T, H * V) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def alibi_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)], dtype=F64)


def chunked_attention(h, w, cfg, eps):
    H, G, K, V = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    size, scale = (cfg.get("mask") or {}).get("size", 1 << 40), float(cfg["scale"])
    T = h.shape[0]
    q = rms(h @ w["q"].T + w["q.b"], eps) * w["q.norm"]
    k = rms(h @ w["k"].T + w["k.b"], eps) * w["k.norm"]
    v = h @ w["v"].T + w["v.b"]
    q, k, v = q.view(T, H, K), k.view(T, G, K), v.view(T, G, V)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) & (i // size == j // size)
    slopes = alibi_slopes(H).to(h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        score = (q[:, a] @ k[:, g].T) * scale - slopes[a] * (i - j)
        score = score.masked_fill(~seen, -math.inf)
        top = torch.maximum(score.max(-1, keepdim=True).values, w["sink"][a])
        e = torch.exp(score - top)
        out[:, a] = (e / (e.sum(-1, keepdim=True) + torch.exp(w["sink"][a] - top))) @ v[:, g]
    out = out.reshape(T, H * V) * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def mamba2(h, w, cfg, eps):
    H, V, N, G, parts = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"], cfg["norm_groups"]
    inner = H * V
    T = h.shape[0]
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    taps = w["conv"].shape[1]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc])
    conv = w["conv.b"].expand(T, -1).clone()
    for j in range(taps):
        conv = conv + padded[j:j + T] * w["conv"][:, j]
    xbc = silu(conv)
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"])                                         # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)
    S = torch.zeros(H, N, V, dtype=h.dtype)
    y = torch.zeros(T, H, V, dtype=h.dtype)
    group_of = torch.arange(H) // (H // G)
    for t in range(T):
        Bt, Ct = B[t][group_of], C[t][group_of]                             # [H, N]
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, Ct) + w["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = group_norm(y, w["norm"], parts, eps)
    return y @ w["o"].T


def side_by_side(h, w, cfg, eps):
    left = chunked_attention(h, {k[5:]: t for k, t in w.items() if k.startswith("left.")}, cfg["left"], eps)
    right = mamba2(h, {k[6:]: t for k, t in w.items() if k.startswith("right.")}, cfg["right"], eps)
    return float(cfg["left_scale"]) * left + float(cfg["right_scale"]) * right


def route(h, router, correction, top, groups, keep):
    """(chosen experts [T, top], their weights [T, top])."""
    s = torch.sigmoid(h @ router.T)
    choice = s + correction
    T, E = choice.shape
    per = E // groups
    grouped = choice.view(T, groups, per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = grouped.masked_fill(~allowed[:, :, None], -math.inf).reshape(T, E)
    chosen = masked.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def experts(h, w, cfg):
    r = cfg["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(h, w["router"], w["correction"], r["top"], groups["count"], groups["keep"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            a = silu(w[f"e{e}.gate"] @ h[t]) * (w[f"e{e}.up"] @ h[t])
            out[t] += g * (w[f"e{e}.down"] @ a)
    return out


MIXERS = {"hgrn2": hgrn2, "mlstm": mlstm, "parallel": side_by_side}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (float64).  ``tensors``: name -> tensor."""
    t64 = {k: v.to(F64) for k, v in tensors.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"]["groups"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = t64["embed"][ids] + t64["pos"][:len(ids)]
    layers = []
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        h = input_conv(x, t64[pre + "canon1"])
        mix = {k[len(pre) + 4:]: v for k, v in t64.items() if k.startswith(pre + "mix.")}
        x = x + group_norm(MIXERS[layer["type"]](h, mix, layer["mixer"], eps), t64[pre + "norm1"], groups, eps)
        if layer.get("mlp") is not None:
            h = input_conv(x, t64[pre + "canon2"])
            mlp = {k[len(pre) + 4:]: v for k, v in t64.items() if k.startswith(pre + "mlp.")}
            x = x + group_norm(experts(h, mlp, layer["mlp"]), t64[pre + "norm2"], groups, eps)
        layers.append(x.clone())
    logits = group_norm(x, t64["final.norm"], groups, eps) @ t64["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


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
