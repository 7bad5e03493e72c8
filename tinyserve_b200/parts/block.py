"""A block arranges a mixer, a feed-forward and their norms.

"pre_norm" is tinyserve's decoder layer (serve.py:1177-1181): the stream travels as
(x, residual); each norm first adds x to the residual, then normalises it; the
sub-layer's output becomes the next x, so that r1 = r0 + mixer(norm1(r0)),
r2 = r1 + ffn(norm2(r1)).  Another arrangement is another class in ARRANGEMENTS ("parallel": mixer
and feed-forward side by side on one norm; "sandwich": a norm before and after each sub-layer).

The block also owns what lies below the parts' interfaces: a product may hand its result on
unfinished (split-K partial tiles, a product that has not run yet, rows without their norm
factor: ``kernels.ops``), and the kernel of the next norm or product finishes it.  That is
decided here, between built-in parts that say they can take part in it; every other part gets
and returns plain tensors."""
from __future__ import annotations

from ..config.model_config import LayerSpec
from ..kernels import ops
from .base import ParamSpec, Part, StateSpec, build_feed_forward, build_mixer, build_norm


def add_and_norm(norm, x, residual, reader=None, rows=None, compute_dtype=None):
    """residual += x; returns norm(residual) for ``reader`` (a part, or None).  ``x`` is what a
    mixer or feed-forward returned: a tensor or one of ops' unfinished products.  A plain RMSNorm
    goes to the fused kernels, and a reader that only multiplies its input by a matrix
    (``accepts_scaled_rows``) may get rows without their norm factor; any other norm gets a
    finished tensor."""
    rms = norm.rms_parameters()
    if isinstance(x, ops.NormedAddend) and rms is not None:
        # the norm on the sub-layer's output, the add and this norm are one kernel
        return ops.normed_add_rmsnorm(x, residual, rms[0], rms[1], compute_dtype or x.dtype, rows=rows)
    if rms is None:
        return norm.add_forward(x if norm.takes_pending else ops.materialize(x), residual, rows=rows)
    weight, eps = rms
    scaled_ok = rows is None and reader is not None and getattr(reader, "accepts_scaled_rows", False)
    return ops.add_rmsnorm(x, residual, weight, eps, compute_dtype or residual_compute_dtype(norm, x),
                           rows=rows, scaled_ok=scaled_ok)


def residual_compute_dtype(norm, x):
    dtype = getattr(norm, "compute_dtype", None)
    if dtype is None and x is not None:
        dtype = x.dtype
    return dtype


class PreNormBlock(Part):
    """r <- r + mixer(norm1(r)), then r <- r + ffn(norm2(r)).  A layer without a feed-forward
    (``LayerSpec.ffn`` None) has the first line only.  With ``LayerSpec.options["layer_scale"]``
    each sub-layer's output is multiplied, column by column, by a learned vector before it joins the
    stream (r <- r + s1 * mixer(..), r <- r + s2 * ffn(..)); the product is made in 32-bit by the
    kernel that adds it to the residual (``ops.ColumnScaled``)."""
    capturable = True

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn) if spec.ffn is not None else None
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.post_mixer_norm = build_norm(spec.norm, hidden_size) if self.ffn is not None else None
        self.layer_scale = bool(spec.options.get("layer_scale", False))
        self._names = {
            "mixer": spec.name_of("mixer", self.mixer.tree_name),
            "ffn": spec.name_of("ffn", self.ffn.tree_name if self.ffn is not None else ""),
            "input_norm": spec.name_of("input_norm"),
            "post_mixer_norm": spec.name_of("post_mixer_norm"),
            "mixer_scale": spec.name_of("mixer_scale", "mixer_scale"),
            "ffn_scale": spec.name_of("ffn_scale", "ffn_scale"),
        }

    def children(self):
        n = self._names
        out = {n["mixer"]: self.mixer, n["input_norm"]: self.input_norm}
        if self.ffn is not None:
            out.update({n["ffn"]: self.ffn, n["post_mixer_norm"]: self.post_mixer_norm})
        return out

    def param_specs(self):
        if not self.layer_scale:
            return {}
        specs = {self._names["mixer_scale"]: ParamSpec((self.hidden_size,), role="vector", init="norm_weight")}
        if self.ffn is not None:
            specs[self._names["ffn_scale"]] = ParamSpec((self.hidden_size,), role="vector", init="norm_weight")
        return specs

    def _scaled(self, x, which):
        return ops.ColumnScaled(x, self.w[self._names[which]]) if self.layer_scale else x

    def forward(self, x, residual, ctx, call):
        """(x, residual) -> x of the next block; ``residual`` (32-bit) is updated in place.
        x is None for the first block: the residual then already holds the embeddings."""
        h = add_and_norm(self.input_norm, x, residual, self.mixer, compute_dtype=ctx.dtype)
        if not getattr(self.mixer, "accepts_scaled_rows", False):
            h = ops.materialize(h)
        x = self._scaled(self.mixer.forward(h, ctx, call), "mixer_scale")
        if self.ffn is None:
            return x
        h = add_and_norm(self.post_mixer_norm, x, residual, self.ffn, compute_dtype=ctx.dtype)
        if not getattr(self.ffn, "accepts_scaled_rows", False):
            h = ops.materialize(h)
        return self._scaled(self.ffn.forward(h, ctx), "ffn_scale")


class ParallelBlock(Part):
    """One norm, and the mixer and the feed-forward side by side on its output:
    h = norm(r), r <- r + (mixer(h) + ffn(h)).  The block hands both outputs on as they are
    (``ops.PairSum``); the kernel of the next norm adds them to the 32-bit residual, so their sum
    is never rounded.  A layer without a feed-forward (``LayerSpec.ffn`` None) is r + mixer(h)."""
    capturable = True

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__()
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn) if spec.ffn is not None else None
        self.input_norm = build_norm(spec.norm, hidden_size)
        self._names = {"mixer": spec.name_of("mixer", self.mixer.tree_name),
                       "ffn": spec.name_of("ffn", self.ffn.tree_name if self.ffn is not None else ""),
                       "input_norm": spec.name_of("input_norm")}

    def children(self):
        n = self._names
        out = {n["mixer"]: self.mixer, n["input_norm"]: self.input_norm}
        if self.ffn is not None:
            out[n["ffn"]] = self.ffn
        return out

    def forward(self, x, residual, ctx, call):
        h = ops.materialize(add_and_norm(self.input_norm, x, residual, None, compute_dtype=ctx.dtype))
        mixed = self.mixer.forward(h, ctx, call)
        return ops.PairSum(mixed, self.ffn.forward(h, ctx) if self.ffn is not None else None)


class SandwichBlock(Part):
    """A norm before and after each sub-layer: r <- r + post1(mixer(pre1(r))), then
    r <- r + post2(ffn(pre2(r))).  What a sub-layer returns travels on with its post-norm
    (``ops.NormedAddend``); the kernel of the next pre-norm (the next block's, or the model's final
    norm) norms it, adds it to the 32-bit residual and norms the sum.  A layer without a
    feed-forward (``LayerSpec.ffn`` None) has the first line only."""
    capturable = True

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__()
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn) if spec.ffn is not None else None
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.mixer_out_norm = build_norm(spec.norm, hidden_size)
        self.post_mixer_norm = build_norm(spec.norm, hidden_size) if self.ffn is not None else None
        self.ffn_out_norm = build_norm(spec.norm, hidden_size) if self.ffn is not None else None
        for norm in (self.input_norm, self.mixer_out_norm, self.post_mixer_norm, self.ffn_out_norm):
            if norm is not None and not hasattr(norm, "eps"):
                raise ValueError("sandwich block: its norms are RMS norms")
        self._names = {"mixer": spec.name_of("mixer", self.mixer.tree_name),
                       "ffn": spec.name_of("ffn", self.ffn.tree_name if self.ffn is not None else ""),
                       "input_norm": spec.name_of("input_norm"),
                       "mixer_out_norm": spec.name_of("mixer_out_norm", "post_mixer_out_layernorm"),
                       "post_mixer_norm": spec.name_of("post_mixer_norm"),
                       "ffn_out_norm": spec.name_of("ffn_out_norm", "post_feedforward_layernorm")}

    def children(self):
        n = self._names
        out = {n["mixer"]: self.mixer, n["input_norm"]: self.input_norm, n["mixer_out_norm"]: self.mixer_out_norm}
        if self.ffn is not None:
            out.update({n["ffn"]: self.ffn, n["post_mixer_norm"]: self.post_mixer_norm,
                        n["ffn_out_norm"]: self.ffn_out_norm})
        return out

    def forward(self, x, residual, ctx, call):
        h = ops.materialize(add_and_norm(self.input_norm, x, residual, None, compute_dtype=ctx.dtype))
        mixed = ops.NormedAddend(self.mixer.forward(h, ctx, call), *self.mixer_out_norm.rms_parameters())
        if self.ffn is None:
            return mixed
        h = ops.materialize(add_and_norm(self.post_mixer_norm, mixed, residual, None, compute_dtype=ctx.dtype))
        return ops.NormedAddend(self.ffn.forward(h, ctx), *self.ffn_out_norm.rms_parameters())


class PostNormBlock(Part):
    """The norm on the sub-layer's output only: r <- r + norm1(mixer(in1(r))), then
    r <- r + norm2(ffn(in2(r))).  The sub-layers read the stream itself, through an input
    convolution: in(r)_t = r_t + sum_j w[:, j] r_(t - taps + 1 + j), causal over time on every
    channel (``LayerSpec.options["input_conv_taps"]``; the last taps - 1 rows of the stream are part
    of a request's state, for each sub-layer of each block run).  The stream is 32-bit and every
    output is added to it in 32-bit by the kernel that norms it; the block hands nothing on
    unfinished.  A layer without a feed-forward (``LayerSpec.ffn`` None) has the first line only."""
    capturable = True

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.taps = int(spec.options.get("input_conv_taps", 0))
        if not 1 <= self.taps <= ops.CAUSAL_CONV_MAX_TAPS:
            raise ValueError(f"post-norm block: an input convolution of 1 to {ops.CAUSAL_CONV_MAX_TAPS} taps, got {self.taps}")
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn) if spec.ffn is not None else None
        self.mixer_out_norm = build_norm(spec.norm, hidden_size)
        self.ffn_out_norm = build_norm(spec.norm, hidden_size) if self.ffn is not None else None
        for norm in (self.mixer_out_norm, self.ffn_out_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("post-norm block: its norms add their output to the stream themselves (group_rmsnorm)")
        self._names = {"mixer": spec.name_of("mixer", self.mixer.tree_name),
                       "ffn": spec.name_of("ffn", self.ffn.tree_name if self.ffn is not None else ""),
                       "mixer_out_norm": spec.name_of("mixer_out_norm", "mixer_out_norm"),
                       "ffn_out_norm": spec.name_of("ffn_out_norm", "ffn_out_norm"),
                       "mixer_in_conv": spec.name_of("mixer_in_conv", "mixer_in_conv"),
                       "ffn_in_conv": spec.name_of("ffn_in_conv", "ffn_in_conv")}

    def children(self):
        n = self._names
        out = {n["mixer"]: self.mixer, n["mixer_out_norm"]: self.mixer_out_norm}
        if self.ffn is not None:
            out.update({n["ffn"]: self.ffn, n["ffn_out_norm"]: self.ffn_out_norm})
        return out

    def param_specs(self):
        n = self._names
        specs = {f"{n['mixer_in_conv']}.weight": ParamSpec((self.hidden_size, self.taps), init="around_zero")}
        if self.ffn is not None:
            specs[f"{n['ffn_in_conv']}.weight"] = ParamSpec((self.hidden_size, self.taps), init="around_zero")
        return specs

    def state_specs(self):
        if self.taps < 2:
            return {}
        specs = {"mixer_in": StateSpec((self.taps - 1, self.hidden_size), "float32")}
        if self.ffn is not None:
            specs["ffn_in"] = StateSpec((self.taps - 1, self.hidden_size), "float32")
        return specs

    def _read(self, residual, which, ctx, call):
        weight = self.w[f"{self._names[which + '_conv']}.weight"]
        state = ctx.state(call.state_of(f"block.{which}")) if self.taps > 1 else None
        return ops.causal_conv(residual, weight, state, ctx, ctx.dtype, add_input=True)

    def forward(self, x, residual, ctx, call):
        if x is not None:
            raise ValueError("post-norm block: the block before it must leave the stream complete")
        self.mixer_out_norm.add_normed(self.mixer.forward(self._read(residual, "mixer_in", ctx, call), ctx, call), residual)
        if self.ffn is not None:
            self.ffn_out_norm.add_normed(self.ffn.forward(self._read(residual, "ffn_in", ctx, call), ctx), residual)
        return None


ARRANGEMENTS = {"pre_norm": PreNormBlock, "parallel": ParallelBlock, "sandwich": SandwichBlock,
                "post_norm": PostNormBlock}


def build_block(spec: LayerSpec, hidden_size: int):
    if spec.arrangement not in ARRANGEMENTS:
        raise KeyError(f"block arrangement {spec.arrangement!r} is not registered")
    return ARRANGEMENTS[spec.arrangement](spec, hidden_size)
