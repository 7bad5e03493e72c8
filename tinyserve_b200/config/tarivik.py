"""Tarivik: a decoder with the norm on every sub-layer's output only (r <- r + norm1(mixer(in(r))),
r <- r + norm2(ffn(in(r))), RMS norms in groups), whose sub-layers read the stream through a short
causal convolution over time, with learned positions added to the embeddings, three kinds of mixer
in any order and a mixture of experts as feed-forward.

Mixers: *hgrn2* (a matrix state whose forget gate, bounded from below, also decides what is
written), *mlstm* (a matrix memory with an exponential input gate, a running maximum and a
normaliser), *parallel* (chunked softmax attention with a distance bias, a sink and an output gate,
beside a selective state space, their outputs added with two constants).

config.json: ``architecture`` "Tarivik"; ``vocab``, ``width``, ``max_positions``; ``norm``
{eps, groups}; ``canon`` {taps}; ``layers``: a list of {"type": "hgrn2" | "mlstm" | "parallel",
"mixer": {...}, "mlp": {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups"
{count, keep}}} | null}.  Mixers: hgrn2 gives heads, dim, vdim; mlstm heads, dim, vdim, gate_cap;
parallel left {heads, kv_heads, dim, vdim, scale, mask {size}}, right {heads, vdim, state, groups,
conv, norm_groups}, left_scale, right_scale.

Tensor names: ``embed``, ``pos``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``, ``norm2``,
``canon1``, ``canon2``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``correction``, ``e<k>.{gate,up,down}``:
the tensor itself carries the name (no ".weight"), a bias is the name with ".b"."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import ClassVar

from .dudatar import _need, _number, _positive_int
from .model_config import ConfigError, LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec

LAYER_TYPES = ("hgrn2", "mlstm", "parallel")


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    if _need(mlp, "kind", where) != "moe":
        raise ConfigError(f"config.json: {where}.kind {mlp['kind']!r} is not 'moe'")
    _positive_int(_need(mlp, "expert", where), "ff", where + ".expert")
    router = _need(mlp, "router", where)
    experts = _positive_int(router, "experts", where + ".router")
    top = _positive_int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: top exceeds experts")
    groups = router.get("groups")
    if groups is not None:
        count = _positive_int(groups, "count", where + ".router.groups")
        keep = _positive_int(groups, "keep", where + ".router.groups")
        if experts % count or keep > count or top > keep * (experts // count):
            raise ConfigError(f"config.json: {where}.router.groups: {experts} experts in {count} groups, {keep} kept, "
                              f"{top} chosen do not fit")


@dataclass(frozen=True)
class TarivikConfig(ModelConfig):
    architecture: ClassVar[str] = "Tarivik"

    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    norm_eps: float = 0.0
    norm_groups: int = 1
    canon_taps: int = 1
    layers: tuple = ()               # the config's layer entries, checked

    @classmethod
    def from_dict(cls, raw: dict) -> "TarivikConfig":
        layers = copy.deepcopy(_need(raw, "layers", "the model"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        width = _positive_int(raw, "width", "the model")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {LAYER_TYPES}")
            mixer = _need(layer, "mixer", where)
            at = where + ".mixer"
            if kind == "parallel":
                left, right = _need(mixer, "left", at), _need(mixer, "right", at)
                for key in ("heads", "dim", "vdim"):
                    _positive_int(left, key, at + ".left")
                left.setdefault("kv_heads", left["heads"])
                if left["heads"] % _positive_int(left, "kv_heads", at + ".left"):
                    raise ConfigError(f"config.json: {at}.left: heads is no multiple of kv_heads")
                _number(left, "scale", at + ".left")
                mask = left.get("mask")
                if mask is not None:
                    _positive_int(mask, "size", at + ".left.mask")
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    _positive_int(right, key, at + ".right")
                if right["heads"] % right["groups"]:
                    raise ConfigError(f"config.json: {at}.right: heads is no multiple of groups")
                if (right["heads"] * right["vdim"]) % right["norm_groups"]:
                    raise ConfigError(f"config.json: {at}.right: heads * vdim is no multiple of norm_groups")
                _number(mixer, "left_scale", at)
                _number(mixer, "right_scale", at)
            else:
                for key in ("heads", "dim", "vdim"):
                    _positive_int(mixer, key, at)
                if kind == "mlstm" and not _number(mixer, "gate_cap", at) > 0:
                    raise ConfigError(f"config.json: {at}.gate_cap must be positive")
            _check_mlp(layer.get("mlp"), where + ".mlp")
        norm = _need(raw, "norm", "the model")
        eps = _number(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        groups = norm.get("groups", 1)
        if isinstance(groups, bool) or not isinstance(groups, int) or groups < 1 or width % groups:
            raise ConfigError(f"config.json: norm.groups {groups!r} must divide the width {width}")
        canon = raw.get("canon") or {"taps": 1}
        return cls(vocab=_positive_int(raw, "vocab", "the model"), width=width,
                   max_positions=_positive_int(raw, "max_positions", "the model"), norm_eps=eps, norm_groups=groups,
                   canon_taps=_positive_int(canon, "taps", "canon"), layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "canon": {"taps": self.canon_taps}, "layers": copy.deepcopy(list(self.layers))}

    # ------------------------------------------------------------------ parts
    def _mixer(self, layer: dict) -> PartSpec:
        m, w, eps = layer["mixer"], self.width, self.norm_eps
        if layer["type"] == "hgrn2":
            return PartSpec("hgrn2", {"hidden_size": w, "num_heads": m["heads"], "key_dim": m["dim"],
                                      "value_dim": m["vdim"], "eps": eps})
        if layer["type"] == "mlstm":
            return PartSpec("mlstm", {"hidden_size": w, "num_heads": m["heads"], "key_dim": m["dim"],
                                      "value_dim": m["vdim"], "gate_cap": float(m["gate_cap"]), "eps": eps})
        left, right = m["left"], m["right"]
        heads = left["heads"]
        attention = PartSpec("attention", {
            "hidden_size": w, "num_heads": heads, "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "value_dim": left["vdim"], "scale": float(left["scale"]), "bias": True, "joint_norm": True, "norm_eps": eps,
            "chunk": (left.get("mask") or {}).get("size", 0),
            # the design's slopes: 2^(-8 (h + 1) / H)
            "distance_slopes": tuple(2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)),
            "sinks": True, "out_gate": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_norm": "q.norm", "k_norm": "k.norm",
                      "sinks": "sink"}})
        ssm = PartSpec("mamba2", {
            "hidden_size": w, "num_heads": right["heads"], "value_dim": right["vdim"], "state_dim": right["state"],
            "groups": right["groups"], "conv_taps": right["conv"], "norm_groups": right["norm_groups"], "eps": eps})
        return PartSpec("side_by_side", {
            "hidden_size": w, "branches": (("left", attention), ("right", ssm)), "combine": "weighted_sum",
            "scales": (float(m["left_scale"]), float(m["right_scale"]))})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("group_rmsnorm", {"eps": self.norm_eps, "groups": self.norm_groups})
        names = {"mixer": "mix", "ffn": "mlp", "mixer_out_norm": "norm1", "ffn_out_norm": "norm2",
                 "mixer_in_conv": "canon1", "ffn_in_conv": "canon2"}
        layers, order = [], []
        for i, layer in enumerate(self.layers):
            ffn = None
            mlp = layer.get("mlp")
            if mlp is not None:
                router = mlp["router"]
                groups = router.get("groups") or {"count": 1, "keep": 1}
                ffn = PartSpec("moe", {"hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"],
                                       "num_experts": router["experts"], "top": router["top"], "activation": "silu_gated",
                                       "router": "sigmoid_corrected", "groups": groups["count"],
                                       "keep_groups": groups["keep"]})
            layers.append(LayerSpec(self._mixer(layer), ffn, norm, arrangement="post_norm", names=names,
                                    options={"input_conv_taps": self.canon_taps}))
            order.append(LayerCall(i, i))
        unread = tuple(rf"l{i}\.(norm2|canon2)" for i, layer in enumerate(self.layers) if layer.get("mlp") is None)
        return ModelSpec(
            self.vocab, self.width, tuple(layers), tuple(order), norm, tie_word_embeddings=False, weight_prefix="",
            names={"embed": "embed", "layers": "l{i}", "final_norm": "final.norm", "lm_head": "head", "embed_position": "pos"},
            embedding_position=PartSpec("learned_positions", {"max_positions": self.max_positions, "hidden_size": self.width}),
            name_rules=((r"\.weight$", ""), (r"\.bias$", ".b")), unread_names=unread)
