"""Babadra off the device: the configuration reader, the run order, cache entries and stream
operations it makes, the checkpoint's tensor names, the ramp rule of the rotary frequencies, and the
plain implementation against closed forms of its own mechanisms."""
import math

import pytest
import torch

import plain_babadra as plain
from babadra_configs import (BABADRA_TINY, babadra_config, babadra_config_dict, make_babadra_dir,
                             random_babadra_config_dict)


def test_registry_reads_the_architecture_key_and_round_trips():
    from tinyserve_b200.config import BabadraConfig, architecture_of, config_from_dict
    raw = babadra_config_dict("P")
    assert architecture_of(raw) == "Babadra"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, BabadraConfig) and cfg.vocab == 180 and cfg.width == 64 and cfg.embedding_scale == 3.5
    assert config_from_dict(cfg.to_dict()) == cfg
    for seed in range(30):
        drawn = config_from_dict(random_babadra_config_dict(seed))
        assert config_from_dict(drawn.to_dict()) == drawn


@pytest.mark.parametrize("damage,text", [
    (lambda r: r.pop("width"), "width"),
    (lambda r: r.pop("max_positions"), "max_positions"),
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda r: r["layers"][0]["mixer"].update(diff=1.0), "diff"),
    (lambda r: r["layers"][0]["mixer"].update(softcap=-2.0), "softcap"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=18), "rot"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=4), "rot"),
    (lambda r: r["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0), "scaling"),
    (lambda r: r["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda r: r["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda r: r["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda r: r["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["layers"][0]["mlp"]["expert"].update(limit=0), "limit"),
    (lambda r: r["loop"].update(stop=9), "loop"),
    (lambda r: r["loop"].update(times=0), "loop"),
    (lambda r: r["norm"].update(eps=0), "eps"),
])
def test_a_damaged_configuration_is_refused(damage, text):
    from tinyserve_b200.config import ConfigError, config_from_dict
    raw = babadra_config_dict("P")
    damage(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_run_order_caches_and_stream_operations():
    from tinyserve_b200.parts import build_model
    p = build_model(babadra_config("P"))
    # layer 0, then layers 1 and 2 twice, then layer 3: every run with a cache entry of its own, and the
    # embedding output joins the stream again before the second pass only
    assert [c.layer for c in p.calls] == [0, 1, 2, 1, 2, 3]
    assert [c.cache for c in p.calls] == [0, 1, 2, 3, 4, 5] and all(c.writes_cache for c in p.calls)
    assert [len(c.before) for c in p.calls] == [0, 0, 0, 1, 0, 0]
    assert p.blocks[2].ffn is None and p.blocks[0].layer_scale and p.lm_head is not None and p.embed_position is not None
    # two score maps: a key head per map and one value head for both, rows as wide as the wider of key and value
    kinds = [(g.kind, [(t.name, t.heads, t.width) for t in g.tensors]) for g in p.cache_groups]
    assert sorted(kinds) == [("full", [("k", 4, 32), ("v", 2, 32)]), ("full", [("latent", 1, 32)])]      # 24 + 8, and 20 + 12
    assert p.group_sizes == [3, 3]
    q = build_model(babadra_config("Q"))
    assert [c.layer for c in q.calls] == [0, 1, 2, 3] and not q.stream_ops and q.spec.logit_softcap == 0.0
    assert q.spec.embedding_scale == 1.0
    r = build_model(babadra_config("R"))
    assert [c.layer for c in r.calls] == [0, 1, 2] * 3
    assert [len(c.before) for c in r.calls] == [0, 0, 0, 1, 0, 0, 1, 0, 0]
    assert p.capturable and q.capturable and r.capturable
    for seed in range(30):
        raw = random_babadra_config_dict(seed)
        model = build_model(babadra_config_from(raw))
        assert [(c.layer, bool(c.before)) for c in model.calls] == plain.run_order(raw)


def babadra_config_from(raw):
    from tinyserve_b200.config import config_from_dict
    return config_from_dict(raw)


def test_a_loop_of_one_pass_or_of_no_layers_changes_nothing():
    from tinyserve_b200.parts import build_model
    for loop in ({"start": 1, "stop": 3, "times": 1}, {"start": 2, "stop": 2, "times": 3}):
        raw = babadra_config_dict("P")
        raw["loop"] = loop
        model = build_model(babadra_config_from(raw))
        assert [c.layer for c in model.calls] == [0, 1, 2, 3] and not model.stream_ops
        assert plain.run_order(raw) == [(i, False) for i in range(4)]


def test_checkpoint_names(tmp_path):
    from safetensors import safe_open
    folder = make_babadra_dir(tmp_path, "P", seed=3)
    with safe_open(f"{folder}/model.safetensors", "pt") as fh:
        names = set(fh.keys())
        shapes = {k: tuple(fh.get_slice(k).get_shape()) for k in names}
    for name in ("embed", "pos", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.ls1", "l0.ls2", "l0.mix.q", "l0.mix.k",
                 "l0.mix.v", "l0.mix.o", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.lq1", "l0.mix.lk1", "l0.mix.lq2",
                 "l0.mix.lk2", "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e3.gate", "l0.mlp.e3.up", "l0.mlp.e3.down",
                 "l1.mix.dq", "l1.mix.dq.norm", "l1.mix.uq", "l1.mix.dkv", "l1.mix.dkv.norm", "l1.mix.uk", "l1.mix.uv",
                 "l1.mix.o", "l1.mlp.gate", "l1.mlp.up", "l1.mlp.down", "l2.ls1"):
        assert name in names, name
    assert "l2.norm2" not in names and "l2.ls2" not in names and not any(n.endswith(".weight") for n in names)
    assert shapes["l0.mix.q"] == (4 * 2 * 16, 64) and shapes["l0.mix.k"] == (2 * 2 * 16, 64) and shapes["l0.mix.v"] == (2 * 32, 64)
    assert shapes["l0.mix.q.norm"] == (16,) and shapes["l0.mix.lq1"] == (16,) and shapes["l0.mlp.router.b"] == (4,)
    assert shapes["l1.mix.dkv"] == (24 + 8, 64) and shapes["l1.mix.uq"] == (3 * (16 + 8), 40) and shapes["pos"] == (160, 64)
    assert shapes["l0.ls1"] == (64,)
    # a checkpoint may hold the norm and the factors of a feed-forward that a layer does not have
    from tinyserve_b200.parts import build_model
    from tinyserve_b200.weights.loader import check_checkpoint
    index = {k: ("f", v, "BF16") for k, v in shapes.items()}
    index["l2.norm2"], index["l2.ls2"] = ("f", (64,), "BF16"), ("f", (64,), "BF16")
    check_checkpoint(build_model(babadra_config("P")), index)


def test_ramp_rule_of_the_rotary_tables():
    from tinyserve_b200.parts.rotary import Rotary
    for rot in ({"base": 1e4, "dims": 8, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}},
                {"base": 7e5, "dims": 16, "scaling": {"factor": 16.0, "original": 16, "fast": 4.0, "slow": 2.0}},
                {"base": 5e5, "dims": 32, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                {"base": 100.0, "dims": 12}):
        part = Rotary(rot["dims"], rot["base"], "interleaved", rot.get("scaling"))
        cos, sin = Rotary.tables(part.rotary_dim, part.theta, 300, part.scaling)
        f, grow = plain.frequencies(rot)
        ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
        assert (cos.double() - ang.cos() * grow).abs().max() < 1e-6 and (sin.double() - ang.sin() * grow).abs().max() < 1e-6
        if "scaling" in rot:
            sc = rot["scaling"]
            plainf = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
            assert grow == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
            assert ((f <= plainf * (1 + 1e-12)) & (f >= plainf / sc["factor"] * (1 - 1e-12))).all()
            assert f[-1] == pytest.approx(float(plainf[-1]) / sc["factor"]) or sc["original"] > 1000, "the longest wave is stretched in full"


# ----------------------------------------------------------------------------- the plain implementation itself
def _weights(name, seed=1, tmp=None):
    folder = make_babadra_dir(tmp, name, seed=seed)
    return plain.load_folder(folder)


@pytest.mark.parametrize("name", sorted(BABADRA_TINY))
def test_plain_model_is_causal_and_sees_far_tokens(name, tmp_path):
    cfg, W = _weights(name, tmp=tmp_path)
    ids = torch.randint(0, cfg["vocab"], (50,), generator=torch.Generator().manual_seed(5)).tolist()
    full, layers = plain.forward(cfg, W, ids, return_layers=True)
    assert layers.shape == (len(plain.run_order(cfg)), 50, cfg["width"])
    assert (plain.logits(cfg, W, ids[:31]) - full[:31]).abs().max() < 1e-9, "a position does not see what follows"
    other = list(ids)
    other[0] = (ids[0] + 1) % cfg["vocab"]
    assert (plain.logits(cfg, W, other)[-1] - full[-1]).abs().max() > 1e-6, "the last position sees the first token"
    if cfg.get("logit_softcap"):
        assert full.abs().max() < cfg["logit_softcap"]


def test_plain_mechanisms_against_closed_forms():
    g = torch.Generator().manual_seed(0)
    # the bounded gate: beyond the bound nothing changes; at u = 0 it is g sigmoid(1.702 g)
    a = plain.bounded_gate(torch.tensor([0.5, 3.0, 9.0, -4.0], dtype=torch.float64), torch.tensor([0.0, 5.0, 2.0, -7.0], dtype=torch.float64), 2.0)
    s = lambda z: z / (1.0 + math.exp(-1.702 * z))
    assert a.tolist() == pytest.approx([s(0.5), s(2.0) * 3.0, s(2.0) * 3.0, s(-4.0) * -1.0])
    # the router: weights of the chosen experts sum to one and follow their logits
    h = torch.randn(7, 12, generator=g, dtype=torch.float64)
    W = {"router": torch.randn(5, 12, generator=g, dtype=torch.float64), "router.b": torch.tensor([0.0, 0.0, 50.0, 0.0, 0.0], dtype=torch.float64)}
    idx, w = plain.route(h, W, "", {"experts": 5, "top": 2})
    assert (idx[:, 0] == 2).all() and (w.sum(-1) - 1).abs().max() < 1e-12 and (w[:, 0] > 0.999).all()
    # neighbouring pairs against the half pairing: the same rotation on permuted elements
    x = torch.randn(6, 2, 12, generator=g, dtype=torch.float64)
    rot = {"base": 50.0, "dims": 8}
    pos = torch.arange(6) + 3
    perm = [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]
    back = [perm.index(i) for i in range(12)]
    assert (plain.rotate(x, pos, rot, "neighbours") - plain.rotate(x[..., perm], pos, rot, "half")[..., back]).abs().max() < 1e-12
    # a rotation keeps the length of every pair, times the factor that stretched waves bring
    sc = dict(rot, scaling={"factor": 4.0, "original": 8, "fast": 4.0, "slow": 1.0})
    y = plain.rotate(x, pos, sc, "half")
    grow = 0.1 * math.log(4.0) + 1.0
    assert (y[..., :8].pow(2).sum(-1) - grow ** 2 * x[..., :8].pow(2).sum(-1)).abs().max() < 1e-9 and (y[..., 8:] == x[..., 8:]).all()
    # two score maps with lambda = 0 and diff = 0 are the first map alone, normed per head
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.7, "diff": 0.0}
    Wd = {k: torch.randn(*s, generator=g, dtype=torch.float64) for k, s in
          {"q": (16, 10), "k": (8, 10), "v": (6, 10), "o": (10, 12)}.items()}
    Wd.update({"q.norm": torch.ones(4, dtype=torch.float64), "k.norm": torch.ones(4, dtype=torch.float64),
               "lq1": torch.zeros(4, dtype=torch.float64), "lk1": torch.zeros(4, dtype=torch.float64),
               "lq2": torch.zeros(4, dtype=torch.float64), "lk2": torch.zeros(4, dtype=torch.float64)})
    assert plain.differential_lambda(Wd, "", m) == 0.0
    hh = torch.randn(9, 10, generator=g, dtype=torch.float64)
    got = plain.differential_attention(hh, Wd, "", m, 1e-6)
    q = plain.unit_rms((hh @ Wd["q"].T).view(9, 4, 4), 1e-6)[:, 0::2]
    k = plain.unit_rms((hh @ Wd["k"].T).view(9, 2, 4), 1e-6)[:, 0]
    v = hh @ Wd["v"].T
    heads = [plain.unit_rms(plain.causal_softmax(q[:, a] @ k.T * 0.7) @ v, 1e-6) for a in range(2)]
    assert (got - torch.cat(heads, -1) @ Wd["o"].T).abs().max() < 1e-9
