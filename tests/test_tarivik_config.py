"""Tarivik off the device: the configuration reader, the run order, cache and state entries it makes,
the checkpoint's tensor names, and the plain implementation against closed forms of its own
mechanisms."""
import math

import pytest
import torch

import plain_tarivik as plain
from tarivik_configs import TARIVIK_TINY, random_tarivik_config_dict, tarivik_config, tarivik_config_dict


def test_registry_reads_the_architecture_key_and_round_trips():
    from tinyserve_b200.config import TarivikConfig, architecture_of, config_from_dict
    raw = tarivik_config_dict("P")
    assert architecture_of(raw) == "Tarivik"
    cfg = config_from_dict(raw)
    assert isinstance(cfg, TarivikConfig) and cfg.vocab == 180 and cfg.width == 64 and cfg.canon_taps == 3
    assert config_from_dict(cfg.to_dict()) == cfg
    for seed in range(20):
        drawn = config_from_dict(random_tarivik_config_dict(seed))
        assert config_from_dict(drawn.to_dict()) == drawn


@pytest.mark.parametrize("damage,text", [
    (lambda r: r.pop("width"), "width"),
    (lambda r: r.pop("max_positions"), "max_positions"),
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["left"]["mask"].update(size=0), "size"),
    (lambda r: r["layers"][0]["mixer"]["right"].update(groups=3), "groups"),
    (lambda r: r["layers"][0]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda r: r["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda r: r["layers"][2]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda r: r["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda r: r["layers"][1]["mlp"].update(kind="dense"), "kind"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda r: r["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=4), "groups"),
    (lambda r: r["norm"].update(eps=0), "eps"),
    (lambda r: r["norm"].update(groups=5), "groups"),
    (lambda r: r["canon"].update(taps=0), "taps"),
])
def test_a_damaged_configuration_is_refused(damage, text):
    from tinyserve_b200.config import ConfigError, config_from_dict
    raw = tarivik_config_dict("P")
    damage(raw)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(raw)


def test_run_order_caches_and_states():
    from tinyserve_b200.parts import build_model
    model = build_model(tarivik_config("Q"))
    # two parallel layers keep pages, of two head geometries; every layer keeps states
    assert len(model.cache_entries) == 2 and len(model.cache_groups) == 2
    calls = model.calls
    assert [c.cache >= 0 for c in calls] == [False, True, False, True, False]
    names = [tuple(k for k, _ in c.states) for c in calls]
    assert names[0] == ("", "max", "block.mixer_in", "block.ffn_in")
    assert names[1] == ("right", "block.mixer_in", "block.ffn_in")          # one tap in that state space: no conv state
    assert names[2] == ("", "block.mixer_in")                                # no feed-forward, no second convolution
    assert names[3] == ("right", "right.conv", "block.mixer_in", "block.ffn_in")
    shapes = [model.state_entries[i].shape for _, i in calls[3].states]
    assert shapes == [(6, 36, 8), (4, 6 * 8 + 2 * 3 * 36), (1, 96), (1, 96)]
    assert len({i for c in calls for _, i in c.states}) == len(model.state_entries), "no two calls share a state"
    # a block convolution of one tap keeps nothing
    assert all(not k.startswith("block.") for c in build_model(tarivik_config("R")).calls for k, _ in c.states)
    scoped = calls[3].scoped("right")
    assert [k for k, _ in scoped.states] == ["", "conv"] and scoped.state == calls[3].state_of("right")


def test_checkpoint_names(tmp_path):
    from tinyserve_b200.parts import build_model
    from tinyserve_b200.weights.loader import expected_tensors
    names = {e.name: e.shape for e in expected_tensors(build_model(tarivik_config("P")))}
    for name, shape in {
            "embed": (180, 64), "pos": (256, 64), "head": (180, 64), "final.norm": (64,),
            "l0.norm1": (64,), "l0.canon1": (64, 3), "l0.canon2": (64, 3), "l0.mix.left.q": (64, 64),
            "l0.mix.left.q.b": (64,), "l0.mix.left.k.norm": (32,), "l0.mix.left.v.b": (64,), "l0.mix.left.sink": (4,),
            "l0.mix.left.g": (128, 64), "l0.mix.left.o": (64, 128), "l0.mix.right.in": (2 * 64 + 2 * 2 * 16 + 4, 64),
            "l0.mix.right.conv": (64 + 64, 4), "l0.mix.right.conv.b": (128,), "l0.mix.right.dt_bias": (4,),
            "l0.mix.right.A_log": (4,), "l0.mix.right.D": (4,), "l0.mix.right.norm": (64,), "l0.mlp.router": (6, 64),
            "l0.mlp.correction": (6,), "l0.mlp.e5.gate": (40, 64), "l0.mlp.e0.down": (64, 40), "l1.mix.f.b": (32,),
            "l1.mix.lower": (32,), "l1.mix.norm": (32,), "l2.mix.i": (2, 64), "l2.mix.i.b": (2,), "l2.mix.norm": (48,),
            "l2.mix.g": (48, 64)}.items():
        assert names.get(name) == shape, (name, names.get(name))
    assert "l2.norm2" not in names and "l2.canon2" not in names and "l0.mix.left.g.b" not in names


# ----------------------------------------------------------------------------- the plain implementation itself
def test_plain_input_convolution_and_group_norm():
    x = torch.arange(12, dtype=torch.float64).reshape(4, 3) + 1
    w = torch.tensor([[0.5, 2.0], [0.0, 1.0], [1.0, 0.0]], dtype=torch.float64)
    got = plain.input_conv(x, w)
    assert torch.equal(got[0], x[0] + x[0] * w[:, 1])                  # zeros before the start
    assert torch.equal(got[2], x[2] + x[1] * w[:, 0] + x[2] * w[:, 1])
    y = plain.group_norm(torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64), torch.tensor([1.0, 2.0, 3.0, 4.0]).double(), 2, 0.0)
    want = torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5), 0.0, 4 * 2 / math.sqrt(2.0)]], dtype=torch.float64)
    assert torch.allclose(y, want)


def test_plain_router_against_a_search():
    """Groups by the sum of their two largest choice scores, experts of the kept groups only, weights
    without the correction."""
    g = torch.Generator().manual_seed(3)
    h = torch.randn(40, 8, generator=g).double()
    router, corr = torch.randn(12, 8, generator=g).double(), torch.randn(12, generator=g).double() - 0.5
    chosen, weights = plain.route(h, router, corr, 3, 4, 2)
    s = torch.sigmoid(h @ router.T)
    for t in range(40):
        c = (s[t] + corr).tolist()
        groups = sorted(range(4), key=lambda a: -sum(sorted(c[3 * a:3 * a + 3])[-2:]))[:2]
        allowed = sorted((e for a in groups for e in range(3 * a, 3 * a + 3)), key=lambda e: -c[e])[:3]
        assert sorted(chosen[t].tolist()) == sorted(allowed)
        assert torch.equal(weights[t], s[t][chosen[t]])
    assert (s + corr).min() < 0, "negative choice scores are among the cases"


def test_plain_hgrn2_state_is_a_mixture_of_the_values():
    """With one constant value every state row ends at (1 - prod f) times it: what the gate forgets is what it writes."""
    cfg = {"heads": 1, "dim": 2, "vdim": 3}
    T, W = 5, 4
    g = torch.Generator().manual_seed(1)
    h = torch.randn(T, W, generator=g).double()
    w = {"q": torch.randn(2, W, generator=g).double(), "v": torch.zeros(3, W).double(), "f": torch.randn(2, W, generator=g).double(),
         "f.b": torch.zeros(2).double(), "lower": torch.tensor([0.2, 0.9]).double(), "norm": torch.ones(3).double(),
         "o": torch.eye(3).double()}
    h[:, 0] = 1.0
    w["v"][:, 0] = torch.tensor([1.0, -2.0, 0.5])
    out = plain.hgrn2(h, w, cfg, 0.0)
    # every row of S is a multiple of v, so is o, and the unit norm leaves v / rms(v) up to the sign
    v = torch.tensor([1.0, -2.0, 0.5]).double()
    assert torch.allclose(out.abs(), (v / v.pow(2).mean().sqrt()).abs().expand(T, 3))


def test_plain_mlstm_first_token():
    """At the first token m_1 = max(f_1, i_1) (the maximum starts at zero, not at minus infinity)."""
    cfg = {"heads": 1, "dim": 2, "vdim": 2, "gate_cap": 50.0}
    W = 3
    g = torch.Generator().manual_seed(2)
    h = torch.randn(1, W, generator=g).double()
    w = {n: torch.randn(2, W, generator=g).double() for n in ("q", "k", "v", "g")}
    w.update({"i": torch.randn(1, W, generator=g).double(), "f": torch.randn(1, W, generator=g).double(),
              "i.b": torch.tensor([-4.0]).double(), "f.b": torch.tensor([1.0]).double(), "norm": torch.ones(2).double(),
              "o": torch.eye(2).double()})
    out = plain.mlstm(h, w, cfg, 0.0)
    gi = 50 * math.tanh(float(h @ w["i"].T - 4.0) / 50)
    gf = math.log(1 / (1 + math.exp(-50 * math.tanh(float(h @ w["f"].T + 1.0) / 50))))
    m = max(gf, gi)
    q, k, v = (h @ w["q"].T)[0] * 2 ** -0.5, (h @ w["k"].T)[0], (h @ w["v"].T)[0]
    o = math.exp(gi - m) * float(k @ q) * v / (max(abs(math.exp(gi - m) * float(k @ q)), math.exp(-m)) + 1e-6)
    want = o / o.pow(2).mean().sqrt() * torch.sigmoid(h @ w["g"].T)[0]
    assert torch.allclose(out[0], want)


def test_plain_models_run_and_depend_on_far_tokens(tmp_path):
    from tarivik_configs import make_tarivik_dir
    for name in sorted(TARIVIK_TINY):
        raw, tensors = plain.load_folder(make_tarivik_dir(tmp_path / name, name, seed=5))
        vocab = raw["vocab"]
        ids = [(7 * i + 3) % vocab for i in range(60)]
        a = plain.logits(raw, tensors, ids)
        assert a.shape == (60, vocab) and torch.isfinite(a).all()
        b = plain.logits(raw, tensors, [ids[0] + 1] + ids[1:])
        assert (a[-1] - b[-1]).abs().max() > 0, "the first token reaches the last position through the states"
