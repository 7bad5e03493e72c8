"""Mixers with a matrix state instead of a cache: per request and head

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,

S of key size x value size in 32-bit, kept in the request's state slot between steps and zero
for a request that starts.  What the two kinds share (fused projection, state, output norm over
the value size, silu gate, output projection) is ``MatrixStateMixer``; they differ in a_t:

* ``Retention``: one constant decay per head (a list), rotary positions on q and k, k times
  key_dim^(-1/2), no weight on the output norm.
* ``GatedLinearAttention``: one decay per key channel and token, a = sigmoid(z)^(1 / tau) with
  z = W2 (W1 h) + b a low-rank projection of the mixer's input, q times key_dim^(-1/2), a weight
  of value size on the output norm (one for all heads).

* ``Lightning``: one constant decay per head (a list), silu on q, k and v, no positions and no
  factor; the heads of a token are normed together with one weight over all of them and multiplied
  by sigmoid (not silu) of the gate.

* ``HGRN2``: the forget gate also decides what is written: per key channel and token
  f = l + (1 - l) sigmoid(W_f h + b) with a learned lower bound l, S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T
  (no key), q = silu(W_q h), a weight of value size on the output norm, no gate.
* ``MLSTM``: the matrix memory of xLSTM.  Per head and token a log input gate i and a log forget gate f,
  both capped by cap tanh(. / cap), f through log-sigmoid; with the running maximum m_t = max(f_t + m_(t-1), i_t),
  S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T and n_t the same with k alone;
  o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6), q times key_dim^(-1/2).  n rides in the state as a value
  column of its own (the values get a column of ones); m is a second, small state.
* ``Mamba2``: a selective state space in its state-space-duality form.  One input projection gives a gate z, values
  x, per group B and C, and a step size per head; x, B, C pass a short causal convolution and silu;
  dt = softplus(dt + bias), S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D x_t;
  y silu(z) is RMS-normed in groups over all heads.  B plays k, C plays q, shared by the heads of a group.

Everything behind the projections is 32-bit (angles, decays, gates, step sizes, state, output norm):
csrc/linear_attention.cu.  The decay logits z leave their product in 32-bit."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, ParamSpec, Source, StateSpec, build_position_encoding, register_mixer

DEFAULT_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "g": "g_proj", "o": "o_proj",
                 "decay_down": "a1", "decay_up": "a2", "norm": "norm"}


class MatrixStateMixer(Mixer):
    tree_name = "mixer"
    capturable = True
    accepts_scaled_rows = True

    def __init__(self, hidden_size, num_heads, key_dim, value_dim, eps, names=None):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim, self.eps = key_dim, value_dim, float(eps)
        if not ops.linear_attention_supports(key_dim) or not 0 < value_dim <= ops.LINEAR_ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"linear attention: key size {key_dim} or value size {value_dim} is not supported")
        self.qk_size, self.v_size = num_heads * key_dim, num_heads * value_dim

    def _projection_rows(self):
        qk, v, nm = self.qk_size, self.v_size, self.names
        return [(nm["q"], qk), (nm["k"], qk), (nm["v"], v), (nm["g"], v)]

    def param_specs(self):
        sources, at = [], 0
        for name, rows in self._projection_rows():
            sources.append(Source(f"{name}.weight", at, at + rows))
            at += rows
        return {
            "in_proj.weight": ParamSpec((at, self.hidden_size), sources=tuple(sources)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.v_size),
                                       sources=(Source(f"{self.names['o']}.weight", 0, self.hidden_size),)),
        }

    def state_spec(self):
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), "float32")

    def _split(self, h):
        proj = ops.materialize(ops.linear(h, self.w["in_proj.weight"]))
        qk, v = self.qk_size, self.v_size
        return proj, proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + v], proj[:, 2 * qk + v:2 * qk + 2 * v]


class Retention(MatrixStateMixer):
    def __init__(self, hidden_size, num_heads, key_dim, value_dim, decay, eps, position=None, names=None):
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, names)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != num_heads:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {num_heads} heads")
        self.position = build_position_encoding(position) if position is not None else None
        self.decay = None

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    def prepare(self, runtime):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def forward(self, h, ctx, call):
        _, q, k, v, g = self._split(h)
        out = ops.linear_attention(q, k, v, g, ctx.state(call.state), ctx, self.num_heads, self.key_dim,
                                   self.value_dim, ctx.dtype, decay=self.decay, rotary=self.position,
                                   k_scale=self.key_dim ** -0.5, eps=self.eps)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class GatedLinearAttention(MatrixStateMixer):
    def __init__(self, hidden_size, num_heads, key_dim, value_dim, tau, decay_rank, eps, names=None):
        self.decay_rank = int(decay_rank)
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, names)
        self.tau = float(tau)
        if not self.tau > 0 or self.decay_rank <= 0:
            raise ValueError("gated linear attention: tau and the rank of the decay projection must be positive")

    def _projection_rows(self):
        # the first factor of the decay projection reads the same input: it rides with q, k, v and the gate
        return super()._projection_rows() + [(self.names["decay_down"], self.decay_rank)]

    def param_specs(self):
        specs = super().param_specs()
        nm = self.names
        specs["decay_up.weight"] = ParamSpec((self.qk_size, self.decay_rank),
                                             sources=(Source(f"{nm['decay_up']}.weight", 0, self.qk_size),))
        # drawn like a matrix in the random-weights mode: a bias of zeros would hide a fault
        specs["decay_up.bias"] = ParamSpec((self.qk_size,), role="vector", init="normal",
                                           sources=(Source(f"{nm['decay_up']}.bias", 0, self.qk_size),))
        specs["norm.weight"] = ParamSpec((self.value_dim,), role="vector", init="norm_weight",
                                         sources=(Source(f"{nm['norm']}.weight", 0, self.value_dim),))
        return specs

    def forward(self, h, ctx, call):
        proj, q, k, v, g = self._split(h)
        low = proj[:, 2 * self.qk_size + 2 * self.v_size:]
        z = ops.linear(low, self.w["decay_up.weight"], self.w["decay_up.bias"], out_float32=True)
        out = ops.linear_attention(q, k, v, g, ctx.state(call.state), ctx, self.num_heads, self.key_dim,
                                   self.value_dim, ctx.dtype, decay_logits=z, tau=self.tau,
                                   q_scale=self.key_dim ** -0.5, norm_weight=self.w["norm.weight"], eps=self.eps)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class Lightning(MatrixStateMixer):
    def __init__(self, hidden_size, num_heads, key_dim, value_dim, decay, eps, names=None):
        super().__init__(hidden_size, num_heads, key_dim, value_dim, eps, names)
        self.decay_values = tuple(float(d) for d in decay)
        if len(self.decay_values) != num_heads:
            raise ValueError(f"lightning: {len(self.decay_values)} decays for {num_heads} heads")
        self.decay = None

    def param_specs(self):
        specs = super().param_specs()
        specs["norm.weight"] = ParamSpec((self.v_size,), role="vector", init="norm_weight",
                                         sources=(Source(f"{self.names['norm']}.weight", 0, self.v_size),))
        return specs

    def prepare(self, runtime):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def forward(self, h, ctx, call):
        _, q, k, v, g = self._split(h)
        out = ops.linear_attention(q, k, v, g, ctx.state(call.state), ctx, self.num_heads, self.key_dim,
                                   self.value_dim, ctx.dtype, decay=self.decay, norm_weight=self.w["norm.weight"],
                                   eps=self.eps, input_activation="silu", gate_activation="sigmoid", joint_norm=True)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class HGRN2(Mixer):
    tree_name = "mixer"
    capturable = True

    def __init__(self, hidden_size, num_heads, key_dim, value_dim, eps, names=None):
        super().__init__()
        self.names = dict({"q": "q", "f": "f", "v": "v", "o": "o", "lower": "lower", "norm": "norm"}, **(names or {}))
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim, self.eps = key_dim, value_dim, float(eps)
        if not ops.linear_attention_supports(key_dim) or not 0 < value_dim <= ops.LINEAR_ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"hgrn2: key size {key_dim} or value size {value_dim} is not supported")
        self.qk_size, self.v_size = num_heads * key_dim, num_heads * value_dim

    def param_specs(self):
        nm, qk, v, n = self.names, self.qk_size, self.v_size, self.hidden_size
        return {
            "in_proj.weight": ParamSpec((qk + v, n), sources=(Source(f"{nm['q']}.weight", 0, qk),
                                                              Source(f"{nm['v']}.weight", qk, qk + v))),
            "f_proj.weight": ParamSpec((qk, n), sources=(Source(f"{nm['f']}.weight", 0, qk),)),
            "f_proj.bias": ParamSpec((qk,), role="vector", init="wide", sources=(Source(f"{nm['f']}.bias", 0, qk),)),
            "lower": ParamSpec((qk,), role="vector", init="unit_interval", sources=(Source(nm["lower"], 0, qk),)),
            "norm.weight": ParamSpec((self.value_dim,), role="vector", init="norm_weight",
                                     sources=(Source(f"{nm['norm']}.weight", 0, self.value_dim),)),
            "o_proj.weight": ParamSpec((n, v), sources=(Source(f"{nm['o']}.weight", 0, n),)),
        }

    def bind(self, tensors):
        if "lower" in tensors:
            tensors = dict(tensors, lower=tensors["lower"].float().contiguous())      # the bound enters a 32-bit gate
        super().bind(tensors)

    def state_spec(self):
        return StateSpec((self.num_heads, self.key_dim, self.value_dim), "float32")

    def forward(self, h, ctx, call):
        proj = ops.materialize(ops.linear(h, self.w["in_proj.weight"]))
        z = ops.linear(h, self.w["f_proj.weight"], self.w["f_proj.bias"], out_float32=True)
        out = ops.linear_attention(proj[:, :self.qk_size], None, proj[:, self.qk_size:], None, ctx.state(call.state), ctx,
                                   self.num_heads, self.key_dim, self.value_dim, ctx.dtype, decay_logits=z,
                                   lower=self.w["lower"], tied_key=True, input_activation="q",
                                   norm_weight=self.w["norm.weight"], eps=self.eps)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class MLSTM(Mixer):
    tree_name = "mixer"
    capturable = True

    def __init__(self, hidden_size, num_heads, key_dim, value_dim, gate_cap, eps, names=None):
        super().__init__()
        self.names = dict({"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "i": "i", "f": "f", "norm": "norm"},
                          **(names or {}))
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim, self.eps, self.gate_cap = key_dim, value_dim, float(eps), float(gate_cap)
        if not self.gate_cap > 0:
            raise ValueError("mlstm: the gate cap must be positive")
        # the state's value columns: the values, the normaliser's column of ones, zeros up to a multiple of four
        self.state_cols = (value_dim // 4 + 1) * 4
        if not ops.linear_attention_supports(key_dim) or not 0 < self.state_cols <= ops.LINEAR_ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"mlstm: key size {key_dim} or value size {value_dim} is not supported")
        self.qk_size, self.v_size = num_heads * key_dim, num_heads * value_dim

    def param_specs(self):
        nm, qk, v, n, H = self.names, self.qk_size, self.v_size, self.hidden_size, self.num_heads
        rows, at = [], 0
        for name, count in ((nm["q"], qk), (nm["k"], qk), (nm["v"], v), (nm["g"], v)):
            rows.append(Source(f"{name}.weight", at, at + count))
            at += count
        return {
            "in_proj.weight": ParamSpec((at, n), sources=tuple(rows)),
            "gates.weight": ParamSpec((2 * H, n), sources=(Source(f"{nm['i']}.weight", 0, H), Source(f"{nm['f']}.weight", H, 2 * H))),
            "gates.bias": ParamSpec((2 * H,), role="vector", init="wide",
                                    sources=(Source(f"{nm['i']}.bias", 0, H), Source(f"{nm['f']}.bias", H, 2 * H))),
            "norm.weight": ParamSpec((v,), role="vector", init="norm_weight", sources=(Source(f"{nm['norm']}.weight", 0, v),)),
            "o_proj.weight": ParamSpec((n, v), sources=(Source(f"{nm['o']}.weight", 0, n),)),
        }

    def state_specs(self):
        return {"": StateSpec((self.num_heads, self.key_dim, self.state_cols), "float32"),
                "max": StateSpec((self.num_heads,), "float32")}

    def forward(self, h, ctx, call):
        proj = ops.materialize(ops.linear(h, self.w["in_proj.weight"]))
        qk, v = self.qk_size, self.v_size
        raw_gates = ops.linear(h, self.w["gates.weight"], self.w["gates.bias"], out_float32=True)
        keep, write, floor = ops.mlstm_gates(raw_gates, self.gate_cap, ctx.state(call.state_of("max")), ctx, self.num_heads)
        raw = ops.linear_attention(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + v], None, ctx.state(call.state),
                                   ctx, self.num_heads, self.key_dim, self.state_cols, ctx.dtype, token_keep=keep,
                                   token_write=write, q_scale=self.key_dim ** -0.5, value_width=self.value_dim, raw=True)
        out = ops.mlstm_finish(raw, floor, self.w["norm.weight"], proj[:, 2 * qk + v:], self.eps, self.num_heads,
                               self.value_dim, ctx.dtype)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


class Mamba2(Mixer):
    tree_name = "mixer"
    capturable = True

    def __init__(self, hidden_size, num_heads, value_dim, state_dim, groups, conv_taps, norm_groups, eps, names=None):
        super().__init__()
        self.names = dict({"in": "in", "conv": "conv", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D", "norm": "norm",
                           "o": "o"}, **(names or {}))
        self.hidden_size, self.num_heads, self.value_dim = hidden_size, int(num_heads), int(value_dim)
        self.state_dim, self.groups, self.taps = int(state_dim), int(groups), int(conv_taps)
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        self.inner = self.num_heads * self.value_dim
        if self.groups < 1 or self.num_heads % self.groups:
            raise ValueError(f"mamba2: {num_heads} heads do not split into {groups} groups")
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} channels do not split into {norm_groups} norm groups")
        if not 1 <= self.taps <= ops.CAUSAL_CONV_MAX_TAPS:
            raise ValueError(f"mamba2: a convolution of 1 to {ops.CAUSAL_CONV_MAX_TAPS} taps, got {conv_taps}")
        if not ops.linear_attention_supports(self.state_dim) or not 0 < self.value_dim <= ops.LINEAR_ATTENTION_MAX_VALUE_DIM:
            raise ValueError(f"mamba2: state size {state_dim} or value size {value_dim} is not supported")
        self.conv_channels = self.inner + 2 * self.groups * self.state_dim

    def param_specs(self):
        nm, n, H, C = self.names, self.hidden_size, self.num_heads, self.conv_channels
        rows = self.inner + C + H
        return {
            "in_proj.weight": ParamSpec((rows, n), sources=(Source(f"{nm['in']}.weight", 0, rows),)),
            "conv.weight": ParamSpec((C, self.taps), init="around_zero", sources=(Source(f"{nm['conv']}.weight", 0, C),)),
            "conv.bias": ParamSpec((C,), role="matrix", init="normal", sources=(Source(f"{nm['conv']}.bias", 0, C),)),
            "dt_bias": ParamSpec((H,), role="vector", init="wide", sources=(Source(nm["dt_bias"], 0, H),)),
            "a_log": ParamSpec((H,), role="vector", init="wide", sources=(Source(nm["a_log"], 0, H),)),
            "skip": ParamSpec((H,), role="vector", init="norm_weight", sources=(Source(nm["skip"], 0, H),)),
            "norm.weight": ParamSpec((self.inner,), role="vector", init="norm_weight",
                                     sources=(Source(f"{nm['norm']}.weight", 0, self.inner),)),
            "o_proj.weight": ParamSpec((n, self.inner), sources=(Source(f"{nm['o']}.weight", 0, n),)),
        }

    def state_specs(self):
        specs = {"": StateSpec((self.num_heads, self.state_dim, self.value_dim), "float32")}
        if self.taps > 1:
            specs["conv"] = StateSpec((self.taps - 1, self.conv_channels), "float32")
        return specs

    def forward(self, h, ctx, call):
        inner, C, H, GN = self.inner, self.conv_channels, self.num_heads, self.groups * self.state_dim
        weight = self.w["in_proj.weight"]
        proj = ops.materialize(ops.linear(h, weight[:inner + C]))
        # the step sizes enter the recurrence: their product leaves in 32-bit
        dt_raw = ops.linear(h, weight[inner + C:], out_float32=True)
        conv_state = ctx.state(call.state_of("conv")) if self.taps > 1 else None
        xbc = ops.causal_conv(proj[:, inner:], self.w["conv.weight"], conv_state, ctx, ctx.dtype, bias=self.w["conv.bias"],
                              activation="silu")
        x = xbc[:, :inner]
        # (the scan makes the step sizes, the decays and the factors on B from the logits while it stages a token)
        raw = ops.linear_attention(xbc[:, inner + GN:], xbc[:, inner:inner + GN], x, None, ctx.state(call.state), ctx, H,
                                   self.state_dim, self.value_dim, ctx.dtype,
                                   step_sizes=(dt_raw, self.w["dt_bias"], self.w["a_log"]), qk_group=H // self.groups, raw=True)
        out = ops.ssm_finish(raw, x, self.w["skip"], proj[:, :inner], self.w["norm.weight"], self.norm_groups, self.eps, H,
                             self.value_dim, ctx.dtype)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)


register_mixer("hgrn2", HGRN2)
register_mixer("mlstm", MLSTM)
register_mixer("mamba2", Mamba2)
register_mixer("retention", Retention)
register_mixer("lightning", Lightning)
register_mixer("gated_linear_attention", GatedLinearAttention)
