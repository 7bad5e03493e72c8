"""Mixture of experts: ``num_experts`` small feed-forward layers, of which every token uses ``top``.

Router: z = W_r h in 32-bit, s = softmax(z) over all experts; the ``top`` largest s are the token's
experts and their weights, as they are (not divided by their sum).  Expert e:
W_down,e act(W_up,e h), no biases; the token's output is the weighted sum over its experts.

The experts' up-projections are stacked into one matrix [E ff, hidden] and their down-projections
side by side into one [hidden, E ff]: act(.) of an expert that a token did not choose is multiplied
by zero, the others by their weight, and one product over K = E ff adds the chosen experts'
outputs in 32-bit inside the product.  That is how a few tokens run (decoding: they touch most
experts' weights anyway) and how the 32-bit engine runs; a bfloat16 step of many tokens sorts its
rows by expert instead, so that an expert multiplies its own rows only (``ops.moe_grouped``).

Further forms, each a parameter.  ``activation`` "silu_gated": expert e is
W_down,e (silu(W_gate,e h) * (W_up,e h)); its gate and up rows are stacked expert by expert
[E 2 ff, hidden].  ``router`` "sigmoid_corrected": s = sigmoid(z); the choice is made on s + correction (a
learned vector, ``correction``), the weights are s itself; with ``groups`` > 1 the experts form that
many equal groups of neighbours, a group's score is the sum of its two largest choice scores, and
only the experts of the ``keep_groups`` best groups can be chosen.  ``activation``
"bounded_swish_gated" with ``limit`` L: expert e is W_down,e (g sigmoid(1.702 g) (u + 1)) with
g = min(W_gate,e h, L), u = clamp(W_up,e h, -L, L), laid out like "silu_gated".  ``router``
"softmax_chosen": the ``top`` largest logits choose, and the weights are the softmax over those
logits alone.  ``router_bias``: z = W_r h + b, the bias added in 32-bit."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, Source, register_feed_forward

DEFAULT_NAMES = {"router": "router", "expert": "e{e}", "up": "up", "down": "down", "gate": "gate", "correction": "correction"}
#: expert activation -> (gated?, the gated activation's name for the kernels)
EXPERT_ACTIVATIONS = {"relu_squared": (False, ""), "silu_gated": (True, "silu"), "bounded_swish_gated": (True, "bounded_swish")}
ROUTERS = ("softmax", "softmax_chosen", "sigmoid_corrected")


class MixtureOfExperts(FeedForward):
    tree_name = "mlp"
    capturable = True
    accepts_scaled_rows = False

    def __init__(self, hidden_size, intermediate_size, num_experts, top, activation="relu_squared", names=None,
                 router="softmax", groups=1, keep_groups=1, limit=0.0, router_bias=False):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        if activation not in EXPERT_ACTIVATIONS:
            raise ValueError(f"mixture of experts: unknown activation {activation!r}; known: {sorted(EXPERT_ACTIVATIONS)}")
        if router not in ROUTERS:
            raise ValueError(f"mixture of experts: unknown router {router!r}; known: {ROUTERS}")
        if not 0 < top <= num_experts:
            raise ValueError(f"mixture of experts: {top} of {num_experts} experts")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top = int(num_experts), int(top)
        self.gated, self.gate_activation = EXPERT_ACTIVATIONS[activation]
        self.limit = ops.activation_code(self.gate_activation, limit)[1] if self.gated else 0.0
        self.router, self.router_bias = router, bool(router_bias)
        self.groups, self.keep_groups = int(groups), int(keep_groups)
        if self.groups < 1 or self.num_experts % self.groups or not 1 <= self.keep_groups <= self.groups:
            raise ValueError(f"mixture of experts: {num_experts} experts in {groups} groups of which {keep_groups} are kept")
        if (self.groups > 1 or self.keep_groups > 1) and router != "sigmoid_corrected":
            raise ValueError("mixture of experts: groups of experts come with the sigmoid_corrected router")
        if self.top > self.keep_groups * (self.num_experts // self.groups):
            raise ValueError(f"mixture of experts: {top} experts cannot come from {keep_groups} groups of "
                             f"{self.num_experts // self.groups}")

    def param_specs(self):
        nm, E, ff, n = self.names, self.num_experts, self.intermediate_size, self.hidden_size
        expert = lambda e: nm["expert"].format(e=e)
        if self.gated:
            up_sources = tuple(src for e in range(E) for src in (
                Source(f"{expert(e)}.{nm['gate']}.weight", 2 * e * ff, (2 * e + 1) * ff),
                Source(f"{expert(e)}.{nm['up']}.weight", (2 * e + 1) * ff, (2 * e + 2) * ff)))
        else:
            up_sources = tuple(Source(f"{expert(e)}.{nm['up']}.weight", e * ff, (e + 1) * ff) for e in range(E))
        specs = {}
        if self.router == "sigmoid_corrected":
            specs["correction"] = ParamSpec((E,), role="vector", init="around_zero", sources=(Source(nm["correction"], 0, E),))
        if self.router_bias:
            # (drawn like a matrix in the random-weights mode: a bias of zeros would hide its loss)
            specs["router.bias"] = ParamSpec((E,), role="vector", init="wide", sources=(Source(f"{nm['router']}.bias", 0, E),))
        return {
            **specs,
            "router.weight": ParamSpec((E, n), sources=(Source(f"{nm['router']}.weight", 0, E),)),
            "up.weight": ParamSpec((len(up_sources) * ff, n), sources=up_sources),
            # stored expert by expert [E hidden, ff]; ``bind`` lays them side by side
            "down.weight": ParamSpec((E * n, ff), sources=tuple(
                Source(f"{expert(e)}.{nm['down']}.weight", e * n, (e + 1) * n) for e in range(E))),
        }

    def bind(self, tensors):
        E, ff, n = self.num_experts, self.intermediate_size, self.hidden_size
        tensors = dict(tensors)
        for name in ("correction", "router.bias"):
            if name in tensors:
                tensors[name] = tensors[name].float().contiguous()       # it joins 32-bit scores
        if "down.weight" in tensors:
            down = tensors["down.weight"]
            tensors["down.weight"] = down.view(E, n, ff).permute(1, 0, 2).reshape(n, E * ff).contiguous()
        super().bind(tensors)

    def _route(self, logits):
        if self.router == "sigmoid_corrected":
            return ops.moe_route_scored(logits, self.w["correction"], self.top, self.groups, self.keep_groups)
        return ops.moe_route(logits, self.top, renormalize=self.router == "softmax_chosen", bias=self.w.get("router.bias"))

    def forward(self, h, ctx):
        logits = ops.linear(h, self.w["router.weight"], out_float32=True)
        if self.router_bias and self.router == "sigmoid_corrected":
            ops.add_row_vector_(logits, self.w["router.bias"])
        if (h.dtype == torch.bfloat16 and self.top < self.num_experts and h.shape[0] >= ops.MOE_GROUPED_MIN_TOKENS
                and self.hidden_size % 8 == 0 and self.intermediate_size % 8 == 0):
            return ops.moe_grouped(h, self._route(logits), self.w["up.weight"], self.w["down.weight"], self.top,
                                   gated=self.gated, activation=self.gate_activation, limit=self.limit)
        a = ops.materialize(ops.linear(h, self.w["up.weight"]))
        if self.gated and self.router != "sigmoid_corrected":
            # (routes in the same kernel)
            a = ops.moe_gated_activate(a, None, self.num_experts, self.gate_activation, self.limit, logits=logits, top=self.top,
                                       renormalize=self.router == "softmax_chosen", bias=self.w.get("router.bias"))
        elif self.gated:
            a = ops.moe_gated_activate(a, self._route(logits), self.num_experts, self.gate_activation, self.limit)
        elif self.router == "softmax" and not self.router_bias:
            ops.moe_activate_(a, None, self.num_experts, logits=logits, top=self.top)      # (routes in the same kernel)
        else:
            ops.moe_activate_(a, self._route(logits), self.num_experts)
        return ops.linear(a, self.w["down.weight"], allow_pending=True)


register_feed_forward("moe", MixtureOfExperts)
