"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in 32-bit, output in the compute
dtype (serve.py:799-809).  ``add_forward`` is the fused residual form of
serve.py:1183-1193 / tinykernels.py:26-61; here the residual stream itself stays in
32-bit between layers, so the residual sum is never rounded."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    capturable = True

    def __init__(self, dim: int, eps: float, offset: float = 0.0):
        """``offset``: the checkpoint stores the weight as its distance from ``offset`` (a weight kept
        around zero has offset 1); the sum is made once, in 32-bit, when the tensor is bound."""
        super().__init__()
        self.dim = dim
        self.eps = float(eps)
        self.offset = float(offset)
        self.compute_dtype = None

    def bind(self, tensors):
        if self.offset and "weight" in tensors:
            tensors = dict(tensors, weight=(tensors["weight"].float() + self.offset).contiguous())
        super().bind(tensors)

    def prepare(self, runtime):
        self.compute_dtype = runtime.dtype

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), role="vector", init="around_zero" if self.offset else "norm_weight")}

    def forward(self, x, out=None):
        return ops.rmsnorm(x, self.w["weight"], self.eps, out=out)

    def add_forward(self, x, residual, rows=None):
        return ops.add_rmsnorm(x, residual, self.w["weight"], self.eps, self.compute_dtype, rows=rows)

    def rms_parameters(self):
        return self.w["weight"], self.eps


register_norm("rmsnorm", RMSNorm)


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w (+ b), var the mean of the squared deviations, all in
    32-bit, output in the compute dtype.  ``add_forward`` adds what the block before left (one or
    two tensors) to the 32-bit residual in the same kernel."""
    capturable = True
    takes_pending = True

    def __init__(self, dim: int, eps: float, bias: bool = False):
        super().__init__()
        self.dim, self.eps, self.bias = dim, float(eps), bool(bias)
        self.compute_dtype = None

    def prepare(self, runtime):
        self.compute_dtype = runtime.dtype

    def param_specs(self):
        specs = {"weight": ParamSpec((self.dim,), role="vector", init="norm_weight")}
        if self.bias:
            specs["bias"] = ParamSpec((self.dim,), role="vector", init="normal")
        return specs

    def forward(self, x, out=None):
        residual = x.float().contiguous()
        return ops.add_layernorm(None, residual, self.w["weight"], self.eps, x.dtype, bias=self.w.get("bias"))

    def add_forward(self, x, residual, rows=None):
        return ops.add_layernorm(x, residual, self.w["weight"], self.eps, self.compute_dtype,
                                 bias=self.w.get("bias"), rows=rows)


register_norm("layernorm", LayerNorm)


class GroupRMSNorm(Norm):
    """RMS norm in groups: the row is cut into ``groups`` equal consecutive parts, each divided by
    its own sqrt(mean(part^2) + eps), and the whole multiplied by the weight.  32-bit arithmetic;
    one group is the plain RMS norm."""
    capturable = True

    def __init__(self, dim: int, eps: float, groups: int = 1):
        super().__init__()
        self.dim, self.eps, self.groups = dim, float(eps), int(groups)
        if self.groups < 1 or dim % self.groups:
            raise ValueError(f"group norm: {dim} columns do not split into {groups} equal groups")
        self.compute_dtype = None

    def prepare(self, runtime):
        self.compute_dtype = runtime.dtype

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), role="vector", init="norm_weight")}

    def forward(self, x, out=None):
        return ops.group_norm(x, self.w["weight"], self.groups, self.eps, x.dtype)

    def add_forward(self, x, residual, rows=None):
        if x is not None:
            raise ValueError("group norm: the stream it reads is complete (the block before adds its own outputs)")
        return ops.group_norm(residual, self.w["weight"], self.groups, self.eps, self.compute_dtype, rows=rows)

    def add_normed(self, y, residual):
        """residual (float32, in place) += this norm of y."""
        return ops.group_norm_add_(y, self.w["weight"], self.groups, self.eps, residual)


register_norm("group_rmsnorm", GroupRMSNorm)
