"""Grouped-query attention over a paged cache (serve.py:816-906).

One fused projection for q, k and v (rows q heads, k heads, v heads: serve.py:827-828),
optional per-head norm of q and k before the position encoding (serve.py:873-876),
keys and values written to the cache pages of this step's tokens (serve.py:897-904),
attention of every query over its request's cached keys with j <= position and,
with ``window`` > 0, j > position - window (serve.py:668-680), output projection
(serve.py:883).  All sizes are parameters, and so are the checkpoint's names of the four
projections and the two norms (``names``).

Beyond that model: values may have a head size of their own (``value_dim``); q and k may be
divided by their root mean square per head, without a weight, after the position encoding
(``unit_norm_eps``); every head's output may be multiplied by sigmoid of one number per head, a
projection of the same input (``head_gate``, rows of the fused projection after v).  With any
of these the heads are stored ``stored_dim`` wide (the larger of the two head sizes, rounded up
to what the attention kernels take), padded with zeros: zero key columns add nothing to a score
and the padded output columns are dropped.

With a window, ``keep_first`` > 0 keeps the first tokens of every sequence visible to all later
queries (they keep their own positions, and their pages are never released).

Further forms, each a parameter: ``joint_norm`` (q and k each divided by the root mean square over
all their heads at once, before they are split into heads, with one weight per column, plain);
``chunk`` > 0 (position i sees j <= i only if i // chunk == j // chunk, chunks counted from
position 0 of the sequence); ``distance_slopes`` (one slope per head: slope * (i - j) is taken off
the scaled score); ``sinks`` (a learned number per head whose exponential joins the softmax sum,
without key or value); ``out_gate`` (the concatenated heads times sigmoid(W_g h), element by
element, before the output projection).  Biases on q, k and v go with all of them.

``softcap`` c > 0: the scaled score s becomes c tanh(s / c) before the softmax.

``differential`` = {"diff": d, "eps": e}: every head has two score maps over the same values.  q
holds 2 dim columns per head and k 2 dim per key/value head, [map 1 | map 2]; each map is normed
(``qk_norm``), rotated, capped and softmaxed on its own and gives an output a_1, a_2 over the
head's values; with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + d (four learned vectors of dim
elements, one number per layer, made once in 32-bit) the head's output is
o = a_1 - lambda a_2, divided by sqrt(mean(o^2) + e) over its value columns and multiplied by 1 - d.
The attention kernels run it as 2 H query heads on 2 G key heads that read G value heads (key
head i reads value head i / 2); ``ops.map_difference`` then combines the pairs."""
from __future__ import annotations

from ..kernels import ops
from .base import (CacheSpec, Mixer, ParamSpec, Source, build_norm, build_position_encoding,
                   register_mixer)


DEFAULT_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm",
                 "gate": "g_proj", "sinks": "sinks", "lambda_q1": "lq1", "lambda_k1": "lk1", "lambda_q2": "lq2",
                 "lambda_k2": "lk2"}


class Attention(Mixer):
    tree_name = "self_attn"
    capturable = True

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, bias=False, qk_norm=None,
                 position=None, window=0, scale=None, names=None, value_dim=None, unit_norm_eps=None,
                 head_gate=False, keep_first=0, joint_norm=False, norm_eps=0.0, chunk=0, distance_slopes=None,
                 sinks=False, out_gate=False, softcap=0.0, differential=None):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.bias, self.window = head_dim, bool(bias), int(window or 0)
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.q_norm = build_norm(qk_norm, head_dim) if qk_norm is not None else None
        self.k_norm = build_norm(qk_norm, head_dim) if qk_norm is not None else None
        self.position = build_position_encoding(position) if position is not None else None
        self.value_dim = int(value_dim) if value_dim else head_dim
        self.unit_norm_eps = None if unit_norm_eps is None else float(unit_norm_eps)
        self.head_gate = bool(head_gate)
        self.keep_first = int(keep_first or 0) if self.window > 0 else 0
        if self.keep_first < 0:
            raise ValueError("attention: keep_first must not be negative")
        #: the plain form runs the kernels that fuse per-head norm, rotary and cache write (and, for
        #: a few decoded tokens, the attention itself); the general form has kernels of its own
        self.joint_norm, self.norm_eps, self.chunk = bool(joint_norm), float(norm_eps), int(chunk or 0)
        self.slope_values = tuple(float(x) for x in distance_slopes) if distance_slopes is not None else None
        self.has_sinks, self.out_gate = bool(sinks), bool(out_gate)
        if self.chunk < 0 or (self.chunk and self.window):
            raise ValueError("attention: a chunk is positive and comes without a window")
        if self.slope_values is not None and len(self.slope_values) != num_heads:
            raise ValueError(f"attention: {len(self.slope_values)} slopes for {num_heads} heads")
        if self.out_gate and self.head_gate:
            raise ValueError("attention: one gate, per head or per element")
        extended = self.joint_norm or self.chunk > 0 or self.slope_values is not None or self.has_sinks or self.out_gate
        self.softcap = float(softcap or 0.0)
        if self.softcap < 0:
            raise ValueError("attention: a soft cap is positive (0: none)")
        self.differential = dict(differential) if differential else None
        self.maps = 2 if self.differential else 1
        if self.differential and (extended or self.head_gate or self.unit_norm_eps is not None or bias):
            raise ValueError("attention: two score maps come with a per-head q/k norm, rotation, a window and a soft cap only")
        self.general = (self.value_dim != head_dim or self.unit_norm_eps is not None or self.head_gate
                        or self.keep_first > 0 or extended or self.softcap > 0 or self.maps > 1)
        if self.general and ((qk_norm is not None and (extended or self.unit_norm_eps is not None))
                             or (bias and not extended)):
            raise ValueError("attention: the unit norm and the forms with a joint norm, chunks, slopes, sinks or an output "
                             "gate come without a weighted per-head q/k norm; a value size of its own, the unit norm and "
                             "the head gate come without biases")
        if self.joint_norm and (self.unit_norm_eps is not None or position is not None):
            raise ValueError("attention: the norm over all heads comes without rotation and without the unit norm")
        self.slopes = self.sinks = None
        widest = max(head_dim, self.value_dim)
        self.stored_dim = -(-widest // 16) * 16 if self.general else head_dim
        self.q_size = num_heads * self.maps * head_dim
        self.kv_size = num_kv_heads * self.maps * head_dim
        self.v_size = num_kv_heads * self.value_dim
        self.map_factor = None       # lambda of the two maps, made when the tensors are bound
        self.gate_size = num_heads if self.head_gate else (num_heads * self.value_dim if self.out_gate else 0)

    def children(self):
        out = {}
        if self.q_norm is not None:
            out[self.names["q_norm"]], out[self.names["k_norm"]] = self.q_norm, self.k_norm
        if self.position is not None:
            out["position"] = self.position
        return out

    def param_specs(self):
        q, kv, vs = self.q_size, self.kv_size, self.v_size
        nm = self.names
        rows = ((nm["q"], 0, q), (nm["k"], q, q + kv), (nm["v"], q + kv, q + kv + vs))
        if self.gate_size:
            rows += ((nm["gate"], q + kv + vs, q + kv + vs + self.gate_size),)
        specs = {
            "qkv_proj.weight": ParamSpec((q + kv + vs + self.gate_size, self.hidden_size), sources=tuple(
                Source(f"{n}.weight", a, b) for n, a, b in rows)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.num_heads * self.value_dim),
                                       sources=(Source(f"{nm['o']}.weight", 0, self.hidden_size),)),
        }
        if self.bias:
            # drawn like a matrix in the random-weights mode: a bias of zeros would hide a fault
            # (the gate's rows, where there are any, have no bias: ``bind`` zeroes theirs)
            specs["qkv_proj.bias"] = ParamSpec((q + kv + vs + self.gate_size,), role="matrix", init="normal", sources=tuple(
                Source(f"{n}.bias", a, b) for n, a, b in rows[:3]))
        if self.joint_norm:
            specs["q_norm.weight"] = ParamSpec((q,), role="vector", init="norm_weight",
                                               sources=(Source(f"{nm['q_norm']}.weight", 0, q),))
            specs["k_norm.weight"] = ParamSpec((kv,), role="vector", init="norm_weight",
                                               sources=(Source(f"{nm['k_norm']}.weight", 0, kv),))
        if self.has_sinks:
            specs["sinks"] = ParamSpec((self.num_heads,), role="vector", init="wide", sources=(Source(nm["sinks"], 0, self.num_heads),))
        if self.differential:
            for key in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"):
                # (drawn wide in the random-weights mode, so that lambda is far from the constant it starts from)
                specs[key] = ParamSpec((self.head_dim,), role="vector", init="normal", sources=(Source(nm[key], 0, self.head_dim),))
        return specs

    def bind(self, tensors):
        tensors = dict(tensors)
        if self.bias and self.gate_size and "qkv_proj.bias" in tensors:
            tensors["qkv_proj.bias"][self.q_size + self.kv_size + self.v_size:] = 0
        if "sinks" in tensors:
            tensors["sinks"] = tensors["sinks"].float().contiguous()       # they join a 32-bit sum
        if self.differential and "lambda_q1" in tensors:
            import math
            dot = lambda a, b: float((tensors[a].float() * tensors[b].float()).sum())
            self.map_factor = (math.exp(dot("lambda_q1", "lambda_k1")) - math.exp(dot("lambda_q2", "lambda_k2"))
                               + float(self.differential["diff"]))
        super().bind(tensors)

    def prepare(self, runtime):
        super().prepare(runtime)
        if self.slope_values is not None:
            import torch
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float32, device=runtime.device)

    def cache_spec(self):
        kind = "window" if self.window > 0 else "full"
        if self.maps > 1:
            # a key head per map, one value head for both
            from .base import CacheTensor
            tensors = (CacheTensor("k", self.num_kv_heads * self.maps, self.stored_dim), CacheTensor("v", self.num_kv_heads, self.stored_dim))
            return CacheSpec(kind, self.num_kv_heads * self.maps, self.stored_dim, self.window, tensors=tensors,
                             keep_first=self.keep_first)
        return CacheSpec(kind, self.num_kv_heads, self.stored_dim, self.window, keep_first=self.keep_first)

    def _biased(self):
        return self.chunk > 0 or self.slope_values is not None

    accepts_scaled_rows = True

    def work_tile_queries(self, dtype, page_size):
        return ops.prefill_tile_queries(dtype, self.num_heads * self.maps, self.num_kv_heads * self.maps, self.stored_dim,
                                        page_size)

    def _forward_general(self, h, ctx, call):
        qkv = ops.materialize(ops.linear(h, self.w["qkv_proj.weight"], self.w.get("qkv_proj.bias")))
        q_end, k_end = self.q_size, self.q_size + self.kv_size
        v_end = k_end + self.v_size
        cache = ctx.cache(call.cache)
        view = ctx.group(cache.group)
        if self.joint_norm or self._biased() or self.has_sinks or self.out_gate:
            q = ops.joint_norm_kvwrite(
                qkv[:, :q_end], qkv[:, q_end:k_end], qkv[:, k_end:v_end], self.num_heads, self.num_kv_heads, self.head_dim,
                self.value_dim, self.stored_dim, self.w.get("q_norm.weight"), self.w.get("k_norm.weight"), self.norm_eps,
                k_cache=cache.k, v_cache=cache.v, slot_mapping=view.slot_mapping if call.writes_cache else None,
                page_size=view.page_size)
            out = ops.paged_attention(q, cache.k, cache.v, view, ctx, self.scale, self.window, keep_first=self.keep_first,
                                      sinks=self.w.get("sinks"), chunk=self.chunk, slopes=self.slopes)
            if self.out_gate:
                out = ops.gate_columns(out, qkv[:, v_end:], self.value_dim)
            elif self.head_gate or self.stored_dim != self.value_dim:
                out = ops.head_gate(out, qkv[:, v_end:] if self.head_gate else None, self.value_dim)
            else:
                out = out.view(out.shape[0], self.num_heads * self.value_dim)
            return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)
        M = self.maps
        q = ops.rope_unit_kvwrite(
            qkv[:, :q_end], qkv[:, q_end:k_end], qkv[:, k_end:v_end], ctx.positions, self.num_heads * M,
            self.num_kv_heads * M, self.head_dim, self.value_dim, self.stored_dim, rotary=self.position,
            unit_norm=self.unit_norm_eps is not None, eps=self.unit_norm_eps or 0.0, k_cache=cache.k, v_cache=cache.v,
            slot_mapping=view.slot_mapping if call.writes_cache else None, page_size=view.page_size,
            q_weight=self.q_norm.w["weight"] if self.q_norm is not None else None,
            k_weight=self.k_norm.w["weight"] if self.k_norm is not None else None,
            pre_eps=self.q_norm.eps if self.q_norm is not None else 0.0, maps=M)
        out = ops.paged_attention(q, cache.k, cache.v, view, ctx, self.scale, self.window, keep_first=self.keep_first,
                                  softcap=self.softcap)
        if M > 1:
            d = self.differential
            out = ops.map_difference(out, self.num_heads, self.num_kv_heads, self.value_dim, self.map_factor,
                                     float(d["eps"]), 1.0 - float(d["diff"]))
        elif self.head_gate or self.stored_dim != self.value_dim:
            out = ops.head_gate(out, qkv[:, v_end:] if self.head_gate else None, self.value_dim)
        else:
            out = out.view(out.shape[0], self.num_heads * self.value_dim)
        return ops.linear(out, self.w["o_proj.weight"], allow_pending=True)

    def forward(self, h, ctx, call):
        if self.general:
            return self._forward_general(h, ctx, call)
        qkv = ops.linear(h, self.w["qkv_proj.weight"], self.w.get("qkv_proj.bias"), allow_partials=True)
        cache = ctx.cache(call.cache)
        view = ctx.group(cache.group)
        out = ops.attention_from_qkv(
            qkv, ctx.positions, self.num_heads, self.num_kv_heads, self.head_dim, self.position,
            self.q_norm.w["weight"] if self.q_norm is not None else None,
            self.k_norm.w["weight"] if self.k_norm is not None else None,
            self.q_norm.eps if self.q_norm is not None else 0.0,
            cache.k, cache.v, view, ctx, self.scale, self.window, write_cache=call.writes_cache)
        return ops.linear(out.view(out.shape[0], self.q_size), self.w["o_proj.weight"], allow_pending=True)


register_mixer("attention", Attention)
