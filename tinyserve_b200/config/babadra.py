"""Babadra: a pre-norm decoder (RMS norms whose weights are stored around zero) whose sub-layers
join the stream through a learned factor per column, with scaled embeddings plus learned position
vectors, two kinds of mixer in any order, a dense or a mixture-of-experts feed-forward per layer,
a group of layers that may run several times with the same weights (the embedding output added to
the stream again before every pass but the first; every pass with a cache of its own), and
soft-capped logits.

Mixers: *latent_attention* (queries through a normed latent; per token one normed key/value latent
and one rotated key part shared by all heads are all that is cached; the rotated parts turn in
neighbouring pairs, with frequencies that may be stretched by the ramp rule) and *attention*
(grouped-query attention with two score maps per head over the same values: per-head RMS norm of q
and k with shared weights, rotation of the first rot.dims columns in the (i, i + dims/2) pairing,
soft-capped scores, the maps' outputs subtracted with a learned factor and normed per head).

Feed-forward: y = g sigmoid(1.702 g) (u + 1) with g = min(W_gate h, limit) and
u = clamp(W_up h, -limit, limit), W_down y; dense, or as experts chosen by the largest router
logits (W_router h + b) and weighted by the softmax over the chosen logits.

config.json: ``architecture`` "Babadra"; ``vocab``, ``width``, ``max_positions``; ``norm.eps``;
``embedding.scale``; ``logit_softcap``; ``loop`` {start, stop, times} or none; ``layers``: a list of
{"type": "latent_attention" | "attention", "mixer": {...}, "mlp": {...} | null}.  latent_attention
gives heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {base, dims, scaling {factor, original,
fast, slow} or none}; attention gives heads, kv_heads, dim, vdim, scale, softcap, diff, rot {base,
dims}; mlp is {"kind": "dense", "ff", "limit"} or {"kind": "moe", "expert": {"ff", "limit"},
"router": {"experts", "top"}}.

Tensor names: ``embed``, ``pos``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``, ``norm2``,
``ls1``, ``ls2``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router``, ``router.b``,
``e<k>.{gate,up,down}``: the tensor itself carries the name (no ".weight")."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import ClassVar

from .dudatar import _need, _number, _positive_int
from .model_config import ConfigError, LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec

LAYER_TYPES = ("latent_attention", "attention")


def _rot(mixer: dict, where: str, most: int, exact: bool):
    """The checked ``rot`` entry of a mixer, or None where it has none (nothing is rotated)."""
    rot = mixer.get("rot")
    if rot is None:
        return None
    dims = _need(rot, "dims", where + ".rot")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > most or (exact and dims != most):
        raise ConfigError(f"config.json: {where}.rot.dims {dims!r} must be even and "
                          f"{'equal to' if exact else 'at most'} {most}")
    if not _number(rot, "base", where + ".rot") > 1:
        raise ConfigError(f"config.json: {where}.rot.base must be above one")
    scaling = rot.get("scaling")
    if scaling is not None:
        for key in ("factor", "original", "fast", "slow"):
            if not _number(scaling, key, where + ".rot.scaling") > 0:
                raise ConfigError(f"config.json: {where}.rot.scaling.{key} must be positive")
    return rot


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        _positive_int(mlp, "ff", where)
        if not _number(mlp, "limit", where) > 0:
            raise ConfigError(f"config.json: {where}.limit must be positive")
    elif kind == "moe":
        expert = _need(mlp, "expert", where)
        _positive_int(expert, "ff", where + ".expert")
        if not _number(expert, "limit", where + ".expert") > 0:
            raise ConfigError(f"config.json: {where}.expert.limit must be positive")
        router = _need(mlp, "router", where)
        experts = _positive_int(router, "experts", where + ".router")
        if _positive_int(router, "top", where + ".router") > experts:
            raise ConfigError(f"config.json: {where}.router: top exceeds experts")
    else:
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not 'dense' or 'moe'")


@dataclass(frozen=True)
class BabadraConfig(ModelConfig):
    architecture: ClassVar[str] = "Babadra"

    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    layers: tuple = ()               # the config's layer entries, checked
    loop: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, raw: dict) -> "BabadraConfig":
        layers = copy.deepcopy(_need(raw, "layers", "the model"))
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {LAYER_TYPES}")
            mixer = _need(layer, "mixer", where)
            at = where + ".mixer"
            for key in ("heads", "dim", "vdim"):
                _positive_int(mixer, key, at)
            _number(mixer, "scale", at)
            if kind == "latent_attention":
                for key in ("q_rank", "kv_rank"):
                    _positive_int(mixer, key, at)
                rot_dim = mixer.get("rot_dim", 0)
                if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0 or rot_dim % 2:
                    raise ConfigError(f"config.json: {at}.rot_dim {rot_dim!r} must be even and not negative")
                mixer["rot_dim"] = rot_dim
                rot = _rot(mixer, at, rot_dim, exact=True)
                if rot_dim and rot is None:
                    raise ConfigError(f"config.json: {at}: a rotated part of {rot_dim} needs 'rot'")
            else:
                mixer.setdefault("kv_heads", mixer["heads"])        # (left out: every query head has its own)
                if mixer["heads"] % _positive_int(mixer, "kv_heads", at):
                    raise ConfigError(f"config.json: {at}: heads is no multiple of kv_heads")
                _rot(mixer, at, mixer["dim"], exact=False)
                diff = _number(mixer, "diff", at)
                if not 0.0 <= diff < 1.0:
                    raise ConfigError(f"config.json: {at}.diff {diff!r} must lie in [0, 1)")
                cap = mixer.get("softcap")
                if cap is not None and not _number(mixer, "softcap", at) > 0:
                    raise ConfigError(f"config.json: {at}.softcap must be positive")
            _check_mlp(layer.get("mlp"), where + ".mlp")
        loop = dict(raw.get("loop") or {})
        if loop:
            start, stop, times = (_need(loop, k, "loop") for k in ("start", "stop", "times"))
            if any(isinstance(v, bool) or not isinstance(v, int) for v in (start, stop, times)) \
                    or not (0 <= start <= stop <= len(layers) and times >= 1):
                raise ConfigError(f"config.json: loop {loop!r} does not fit {len(layers)} layers")
            loop = {"start": start, "stop": stop, "times": times}
        norm = _need(raw, "norm", "the model")
        eps = _number(norm, "eps", "norm")
        if not eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        cap = raw.get("logit_softcap")
        if cap is not None and not _number(raw, "logit_softcap", "the model") >= 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        embedding = raw.get("embedding") or {}
        scale = _number(embedding, "scale", "embedding") if "scale" in embedding else 1.0
        return cls(vocab=_positive_int(raw, "vocab", "the model"), width=_positive_int(raw, "width", "the model"),
                   max_positions=_positive_int(raw, "max_positions", "the model"), norm_eps=eps, embedding_scale=scale,
                   logit_softcap=float(cap) if cap else 0.0, layers=tuple(layers), loop=loop)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(list(self.layers))}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop:
            out["loop"] = dict(self.loop)
        return out

    # ------------------------------------------------------------------ parts
    @staticmethod
    def _rotary(rot, pairing):
        if not rot or not rot["dims"]:
            return None
        return PartSpec("rotary", {"rotary_dim": rot["dims"], "theta": float(rot["base"]), "pairing": pairing,
                                   "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})

    def _mixer(self, layer: dict) -> PartSpec:
        m, w, eps = layer["mixer"], self.width, self.norm_eps
        if layer["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": w, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                "value_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]),
                "eps": eps, "position": self._rotary(m.get("rot"), "interleaved"), "sink": False, "gate": False})
        return PartSpec("attention", {
            "hidden_size": w, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "position": self._rotary(m.get("rot"), "half"), "scale": float(m["scale"]),
            "qk_norm": PartSpec("rmsnorm", {"eps": eps}), "softcap": float(m.get("softcap") or 0.0),
            "differential": {"diff": float(m["diff"]), "eps": eps},
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})

    def _ffn(self, mlp):
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                          "activation": "bounded_swish", "limit": float(mlp["limit"]),
                                          "names": {"gate": "gate", "up": "up", "down": "down"}})
        return PartSpec("moe", {"hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"],
                                "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                                "activation": "bounded_swish_gated", "limit": float(mlp["expert"]["limit"]),
                                "router": "softmax_chosen", "router_bias": True})

    def run_order(self):
        """(layer, first of a repeated pass?) in the order the layers run."""
        n = len(self.layers)
        start, stop, times = (self.loop["start"], self.loop["stop"], self.loop["times"]) if self.loop else (0, 0, 1)
        runs = [(i, False) for i in range(start)]
        for t in range(times):
            runs += [(i, t > 0 and i == start) for i in range(start, stop)]
        return runs + [(i, False) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"eps": self.norm_eps, "offset": 1.0})
        names = {"mixer": "mix", "ffn": "mlp", "input_norm": "norm1", "post_mixer_norm": "norm2",
                 "mixer_scale": "ls1", "ffn_scale": "ls2"}
        layers = [LayerSpec(self._mixer(layer), self._ffn(layer.get("mlp")), norm, arrangement="pre_norm", names=names,
                            options={"layer_scale": True}) for layer in self.layers]
        # every run of a layer has a cache entry of its own; the embedding output joins the stream
        # again right before the first layer of every pass but the first
        runs = self.run_order()
        order = tuple(LayerCall(i, entry, True, before=(("again", 0),) if again else ())
                      for entry, (i, again) in enumerate(runs))
        stream_ops = ()
        if any(again for _, again in runs):
            stream_ops = (("again", PartSpec("input_add", {"hidden_size": self.width})),)
        # a layer without a feed-forward has no use for its norm and its factors, should a checkpoint hold them
        unread = tuple(rf"l{i}\.(norm2|ls2)" for i, layer in enumerate(self.layers) if layer.get("mlp") is None)
        return ModelSpec(
            self.vocab, self.width, tuple(layers), order, norm, tie_word_embeddings=False, weight_prefix="",
            names={"embed": "embed", "layers": "l{i}", "final_norm": "final.norm", "lm_head": "head", "embed_position": "pos"},
            embedding_position=PartSpec("learned_positions", {"max_positions": self.max_positions, "hidden_size": self.width}),
            logit_softcap=self.logit_softcap, embedding_scale=self.embedding_scale, stream_ops=stream_ops,
            name_rules=((r"\.weight$", ""), (r"\.bias$", ".b")), unread_names=unread)
