"""Several mixers side by side on the same input.  ``combine`` "mean_of_normed" (the default):
out = mean_i rmsnorm_i(mixer_i(h)), every branch normalised over the model width with a weight of
its own before the mean.  ``combine`` "weighted_sum": out = sum_i scales[i] * mixer_i(h), no norm and
no tensors of its own.  The branches are any registered mixers; at most one of them may keep a paged
cache (a run-order entry names one cache entry); each may keep states, which the run-order entry
holds under the branch's name."""
from __future__ import annotations

from ..kernels import ops
from .base import Mixer, ParamSpec, build_mixer, register_mixer


class SideBySide(Mixer):
    tree_name = "mixer"

    def __init__(self, hidden_size, branches, eps=0.0, combine="mean_of_normed", scales=None):
        """``branches``: ((name, PartSpec), ...); branch ``name`` lives under that name in the
        checkpoint and, with "mean_of_normed", its output weight is ``name``.out.weight."""
        super().__init__()
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.branches = [(name, build_mixer(spec)) for name, spec in branches]
        if not 1 <= len(self.branches) <= 4:
            raise ValueError("side by side: one to four branches")
        if combine not in ("mean_of_normed", "weighted_sum"):
            raise ValueError(f"side by side: unknown combination {combine!r}")
        self.combine = combine
        self.scales = tuple(float(x) for x in scales) if scales is not None else (1.0,) * len(self.branches)
        if len(self.scales) != len(self.branches) or (combine == "weighted_sum" and len(self.branches) != 2):
            raise ValueError("side by side: a scale per branch; the weighted sum takes two branches")
        if sum(m.cache_spec() is not None for _, m in self.branches) > 1:
            raise ValueError("side by side: at most one branch with a cache")
        self.capturable = all(m.capturable for _, m in self.branches)

    def children(self):
        return dict(self.branches)

    def param_specs(self):
        if self.combine != "mean_of_normed":
            return {}
        return {f"{name}.out.weight": ParamSpec((self.hidden_size,), role="vector", init="norm_weight")
                for name, _ in self.branches}

    def cache_spec(self):
        return next((m.cache_spec() for _, m in self.branches if m.cache_spec() is not None), None)

    def state_specs(self):
        return {(f"{name}.{key}" if key else name): spec
                for name, m in self.branches for key, spec in m.state_specs().items()}

    def work_tile_queries(self, dtype, page_size):
        return max(m.work_tile_queries(dtype, page_size) for _, m in self.branches)

    def forward(self, h, ctx, call):
        outs = [m.forward(h, ctx, call.scoped(name)) for name, m in self.branches]
        if self.combine == "weighted_sum":
            return ops.axpby(self.scales[0], outs[0], self.scales[1], outs[1])
        return ops.mean_of_normed(outs, [self.w[f"{name}.out.weight"] for name, _ in self.branches], self.eps)


register_mixer("side_by_side", SideBySide)
