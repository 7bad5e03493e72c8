"""Tiny Tarivik configurations for the tests; they differ from one another in every size, in the
order of the layers and in which options are there at all."""
from __future__ import annotations


def _moe(ff, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _parallel(heads, kv_heads, dim, vdim, scale, chunk, s_heads, s_vdim, state, groups, conv, norm_groups, left_scale,
              right_scale):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        left["mask"] = {"size": chunk}
    return {"left": left, "left_scale": left_scale, "right_scale": right_scale,
            "right": {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv,
                      "norm_groups": norm_groups}}


TARIVIK_TINY = {
    # one layer of every kind; chunks of 24, three taps, experts in two groups of which one is kept
    "P": {
        "vocab": 180, "width": 64, "max_positions": 256, "norm": {"eps": 1e-5, "groups": 2}, "canon": {"taps": 3},
        "layers": [
            {"type": "parallel", "mlp": _moe(40, 6, 2, (2, 1)),
             "mixer": _parallel(4, 2, 16, 32, 0.3, 24, 4, 16, 16, 2, 4, 2, 1.25, 0.75)},
            {"type": "hgrn2", "mlp": _moe(24, 4, 1), "mixer": {"heads": 2, "dim": 16, "vdim": 32}},
            {"type": "mlstm", "mlp": None, "mixer": {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 8.0}},
        ]},
    # sizes that are no power of two; a chunk of 7 (shorter than a page), one of 33 (longer than two), one group in
    # the norms, a convolution of two taps in the blocks and of one and of five in the state spaces, one key/value
    # head, one state-space group, groups of one expert, every expert chosen
    "Q": {
        "vocab": 301, "width": 96, "max_positions": 200, "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 2},
        "layers": [
            {"type": "mlstm", "mlp": _moe(56, 5, 2), "mixer": {"heads": 3, "dim": 20, "vdim": 30, "gate_cap": 15.0}},
            {"type": "parallel", "mlp": _moe(48, 3, 3, (3, 3)),
             "mixer": _parallel(3, 1, 48, 16, 0.2, 7, 3, 24, 20, 1, 1, 1, 0.5, 2.0)},
            {"type": "hgrn2", "mlp": None, "mixer": {"heads": 3, "dim": 12, "vdim": 24}},
            {"type": "parallel", "mlp": _moe(72, 8, 2, (4, 2)),
             "mixer": _parallel(2, 2, 24, 40, 0.4, 33, 6, 8, 36, 3, 5, 3, 1.0, 1.0)},
            {"type": "hgrn2", "mlp": _moe(56, 2, 1, (2, 1)), "mixer": {"heads": 1, "dim": 32, "vdim": 64}},
        ]},
    # head sizes the tensor-core kernels take, a chunk of a whole page multiple, no chunk at all, a block
    # convolution of one tap (the current token's alone: no state), four norm groups
    "R": {
        "vocab": 384, "width": 128, "max_positions": 320, "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 1},
        "layers": [
            {"type": "parallel", "mlp": _moe(64, 8, 2, (2, 1)),
             "mixer": _parallel(8, 2, 64, 64, 0.125, 64, 4, 32, 64, 4, 4, 4, 1.1, 0.9)},
            {"type": "mlstm", "mlp": _moe(32, 16, 5, (4, 3)), "mixer": {"heads": 4, "dim": 64, "vdim": 32, "gate_cap": 10.0}},
            {"type": "parallel", "mlp": None,
             "mixer": _parallel(4, 4, 32, 32, 0.2, 0, 2, 64, 32, 2, 3, 1, 0.7, 1.3)},
            {"type": "hgrn2", "mlp": _moe(64, 2, 2), "mixer": {"heads": 4, "dim": 64, "vdim": 32}},
        ]},
}


def tarivik_config_dict(name: str) -> dict:
    import copy
    return dict(copy.deepcopy(TARIVIK_TINY[name]), architecture="Tarivik")


def tarivik_config(name: str):
    from tinyserve_b200.config import config_from_dict
    return config_from_dict(tarivik_config_dict(name))


def decisive_routers(folder: str, factor: float = 25.0) -> str:
    """The routers of a random model multiplied by ``factor`` and their corrections spread out: with
    weights of 0.02 all experts score alike, and which of them a token takes would hang on the last bit
    of a sum."""
    import os
    import torch
    from safetensors.torch import load_file, save_file
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    g = torch.Generator().manual_seed(11)
    for name in weights:
        if name.endswith(".router"):
            weights[name] = (weights[name].float() * factor).to(weights[name].dtype)
        if name.endswith(".correction"):
            weights[name] = (torch.rand(weights[name].shape, generator=g) * 0.6 - 0.3).to(weights[name].dtype)
    save_file(weights, path)
    return folder


def make_tarivik_dir(folder, name: str, seed: int = 0) -> str:
    from tinyserve_b200.weights import write_random_model
    return decisive_routers(write_random_model(tarivik_config(name), str(folder), seed=seed))


def random_tarivik_config_dict(seed: int) -> dict:
    """A configuration drawn from a seed: sizes that are no power of two and no multiple of 16 among
    them, any order of layer kinds, chunks shorter and longer than a page, layers without
    feed-forward, experts with and without groups."""
    import random
    r = random.Random(seed)
    norm_groups = r.choice([1, 2, 4])
    width = 8 * norm_groups * r.randint(2, 6)
    layers = []
    for _ in range(r.randint(1, 4)):
        per, count = r.randint(1, 4), r.randint(1, 4)
        keep = r.randint(1, count)
        experts = per * count
        mlp = None if r.random() < 0.25 else _moe(8 * r.randint(2, 8), experts, r.randint(1, keep * per),
                                                  (count, keep) if r.random() < 0.8 else None)
        if mlp is not None and "groups" not in mlp["router"]:
            mlp["router"]["top"] = r.randint(1, experts)
        kind = r.choice(["hgrn2", "mlstm", "parallel"])
        if kind == "parallel":
            kv, s_groups = r.randint(1, 3), r.randint(1, 3)
            dim = 2 * r.randint(4, 30)
            s_heads, s_vdim = s_groups * r.randint(1, 3), r.choice([6, 8, 12, 20, 32])
            parts = r.choice([d for d in (1, 2, 3, 4) if (s_heads * s_vdim) % d == 0])
            mixer = _parallel(kv * r.randint(1, 3), kv, dim, r.choice([8, 16, 24, 40, 64]), r.choice([0.1, dim ** -0.5, 0.4]),
                              r.choice([0, 1, 5, 16, 23, 40]), s_heads, s_vdim, r.choice([4, 8, 12, 20, 24, 36]), s_groups,
                              r.randint(1, 6), parts, r.choice([0.5, 1.0, 1.3]), r.choice([0.6, 1.0, 1.7]))
        else:
            mixer = {"heads": r.randint(1, 4), "dim": r.choice([4, 8, 12, 20, 24, 36, 40, 64]),
                     "vdim": r.choice([6, 10, 16, 24, 30, 48, 72])}
            if kind == "mlstm":
                mixer["gate_cap"] = r.choice([5.0, 12.0, 30.0])
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Tarivik", "vocab": r.randint(50, 400), "width": width, "max_positions": 160,
            "norm": {"eps": r.choice([1e-6, 1e-5, 1e-4]), "groups": norm_groups}, "canon": {"taps": r.randint(1, 5)},
            "layers": layers}
