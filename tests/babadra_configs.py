"""Tiny Babadra configurations for the tests; they differ from one another in every size, in the
order of the layers, in where the repeated group lies and in which options are there at all."""
from __future__ import annotations


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
        if scaling:
            m["rot"]["scaling"] = scaling
    return m


def _attention(heads, kv_heads, dim, vdim, scale, diff, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = rot
    return m


BABADRA_TINY = {
    # attention first; the repeated group is the two middle layers, twice; experts of which a token takes
    # one, and all; a latent layer whose rotated part is smaller than its plain part, stretched waves
    "P": {
        "vocab": 180, "width": 64, "max_positions": 160, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
        "logit_softcap": 7.0, "loop": {"start": 1, "stop": 3, "times": 2},
        "layers": [
            {"type": "attention", "mlp": _moe(40, 4, 1, 0.8),
             "mixer": _attention(4, 2, 16, 32, 0.5, 0.2, softcap=4.0, rot={"base": 1e4, "dims": 8})},
            {"type": "latent_attention", "mlp": _dense(72, 0.6),
             "mixer": _latent(3, 16, 8, 24, 40, 24, 0.25, 1e4, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0})},
            {"type": "attention", "mlp": None,
             "mixer": _attention(2, 2, 24, 16, 0.35, 0.0, softcap=30.0, rot={"base": 100.0, "dims": 24})},
            {"type": "latent_attention", "mlp": _moe(24, 3, 3, 2.0), "mixer": _latent(2, 8, 12, 16, 16, 20, 0.4, 5e5)},
        ]},
    # no repeated group, no cap on the logits, an embedding scale of one; attention without rotation and
    # without a cap on its scores, a latent layer without a rotated part, sizes that are no power of two
    "Q": {
        "vocab": 301, "width": 96, "max_positions": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
        "layers": [
            {"type": "latent_attention", "mlp": _moe(56, 5, 2, 1.0), "mixer": _latent(5, 20, 0, 12, 24, 40, 0.3, 1e4)},
            {"type": "attention", "mlp": _dense(104, 1.2), "mixer": _attention(3, 1, 48, 16, 0.2, 0.7)},
            {"type": "attention", "mlp": _moe(48, 1, 1, 0.5),
             "mixer": _attention(6, 3, 20, 40, 0.45, 0.35, softcap=2.5, rot={"base": 5e5, "dims": 20})},
            {"type": "latent_attention", "mlp": None,
             "mixer": _latent(1, 32, 16, 48, 56, 16, 0.2, 7e5, {"factor": 16.0, "original": 16, "fast": 4.0, "slow": 2.0})},
        ]},
    # the whole model is the repeated group, three times; head sizes the tensor-core kernels take
    "R": {
        "vocab": 384, "width": 128, "max_positions": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
        "logit_softcap": 20.0, "loop": {"start": 0, "stop": 3, "times": 3},
        "layers": [
            {"type": "latent_attention", "mlp": _dense(192, 1.0),
             "mixer": _latent(4, 32, 16, 32, 64, 48, 0.15, 1e6, {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 1.0})},
            {"type": "attention", "mlp": _moe(64, 8, 2, 1.5),
             "mixer": _attention(8, 2, 64, 64, 0.125, 0.5, softcap=10.0, rot={"base": 1e4, "dims": 32})},
            {"type": "attention", "mlp": _moe(32, 16, 5, 0.9),
             "mixer": _attention(2, 1, 32, 64, 0.2, 0.1, rot={"base": 2.5e5, "dims": 16})},
        ]},
}


def babadra_config_dict(name: str) -> dict:
    import copy
    return dict(copy.deepcopy(BABADRA_TINY[name]), architecture="Babadra")


def babadra_config(name: str):
    from tinyserve_b200.config import config_from_dict
    return config_from_dict(babadra_config_dict(name))


def decisive(folder: str, seed: int = 0) -> str:
    """A random model made to show its parts.  With weights of 0.02 every router scores all experts
    alike (which of them a token takes would hang on the last bit of a sum), every latent attention
    looks at all keys alike and every layer's lambda is its constant; here the routers are ten times
    as large, the latent queries and keys eight times, the four lambda vectors are drawn so that
    their products are of order one, and the factors on the sub-layers' outputs spread over [0.3, 1.7]."""
    import os
    import torch
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    g = torch.Generator().manual_seed(1000 + seed)
    with open(os.path.join(folder, "config.json")) as fh:
        import json
        cfg = json.load(fh)
    for name in list(weights):
        w = weights[name]
        if name.endswith(".router"):
            w = w.float() * 10.0
        elif name.endswith((".mix.uq", ".mix.uk")):
            w = w.float() * 8.0
        elif name.endswith(".mix.dkv"):
            rank = cfg["layers"][int(name[1:name.index(".")])]["mixer"]["kv_rank"]
            w = w.float().clone()
            w[rank:] *= 8.0
        elif name.rsplit(".", 1)[-1] in ("lq1", "lk1", "lq2", "lk2"):
            w = (torch.rand(w.shape, generator=g) - 0.3) * (1.6 / w.numel() ** 0.5)
        elif name.rsplit(".", 1)[-1] in ("ls1", "ls2"):
            w = 0.3 + 1.4 * torch.rand(w.shape, generator=g)
        else:
            continue
        weights[name] = w.to(weights[name].dtype)
    save_file(weights, path)
    return folder


def make_babadra_dir(folder, name: str, seed: int = 0) -> str:
    from tinyserve_b200.weights import write_random_model
    return decisive(write_random_model(babadra_config(name), str(folder), seed=seed), seed)


def random_babadra_config_dict(seed: int) -> dict:
    """A configuration drawn from a seed: sizes that are no power of two and no multiple of 16 among
    them, any order of layer kinds, a repeated group anywhere (or none), layers without feed-forward,
    rotation over all, a part or none of a head, with and without stretched waves and caps."""
    import random
    r = random.Random(seed)
    even = lambda lo, hi: 2 * r.randint(lo // 2, hi // 2)
    width = 8 * r.randint(4, 14)
    layers = []
    for _ in range(r.randint(1, 5)):
        limit = r.choice([0.4, 1.0, 1.5, 3.0])
        experts = r.randint(1, 9)
        pick = r.random()
        mlp = None if pick < 0.2 else (_dense(8 * r.randint(2, 12), limit) if pick < 0.55 else
                                       _moe(8 * r.randint(2, 10), experts, r.randint(1, experts), limit))
        if r.random() < 0.5:
            rot_dim = r.choice([0, even(2, 24), even(2, 24)])
            scaling = None
            if rot_dim and r.random() < 0.6:
                scaling = {"factor": r.choice([2.0, 4.0, 8.0, 32.0]), "original": r.choice([16, 64, 256]),
                           "fast": r.choice([4.0, 8.0, 32.0]), "slow": r.choice([0.5, 1.0, 2.0])}
            mixer = _latent(r.randint(1, 5), even(4, 40), rot_dim, r.choice([6, 10, 16, 24, 40]), 8 * r.randint(1, 6),
                            r.choice([8, 12, 20, 40, 56]), r.choice([0.1, 0.3]), r.choice([100.0, 1e4, 7e5]), scaling)
            layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
        else:
            kv = r.randint(1, 3)
            dim = even(8, 72)
            dims = r.choice([dim, even(2, dim), 0])
            mixer = _attention(kv * r.randint(1, 3), kv, dim, r.choice([8, 16, 24, 40, 64, 80]), r.choice([0.1, dim ** -0.5, 0.4]),
                               r.choice([0.0, 0.2, 0.5, 0.8]), r.choice([None, 1.5, 8.0, 50.0]),
                               {"base": r.choice([100.0, 1e4, 7e5]), "dims": dims} if dims else None)
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    raw = {"architecture": "Babadra", "vocab": r.randint(50, 400), "width": width, "max_positions": r.randint(70, 300),
           "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4])}, "embedding": {"scale": r.choice([1.0, 2.0, 5.5, 12.0])},
           "layers": layers}
    if r.random() < 0.7:
        raw["logit_softcap"] = r.choice([5.0, 15.0, 30.0])
    if r.random() < 0.7:
        start = r.randint(0, len(layers) - 1)
        raw["loop"] = {"start": start, "stop": r.randint(start, len(layers)), "times": r.randint(1, 3)}
    return raw
