"""Attention whose keys and values are expanded from one small latent per token.

Per token the mixer keeps c = rmsnorm(W_dkv h)[:kv_rank] (a weight of its own) and one rotated key
part r = rotate(W_dkv h)[kv_rank:] that all heads share; nothing else is cached.  Head a has the
query [q_a | q'_a] (``dim`` plain and ``rot_dim`` rotated columns of W_uq rmsnorm(W_dq h)), the key
[W_uk,a c | r] and the value W_uv,a c.  The products with W_uk and W_uv move to the query's side:

    q_a . (W_uk,a c_j) = (W_uk,a^T q_a) . c_j,        sum_j p_j W_uv,a c_j = W_uv,a (sum_j p_j c_j),

so the attention kernel sees one key/value head whose rows are [c_j | r_j] (the cache rows as they
are, keys and values alike), H query heads of ``kv_rank + rot_dim`` columns, and returns per head
the weighted sum of the latents, which W_uv,a then expands.  The softmax sum of head a holds one
more term exp(sink_a) (a learned number per head, no key, no value, not scaled; ``sink`` False:
the ordinary softmax); the concatenated heads are multiplied by sigmoid(W_g h) before the output
projection (``gate`` False: they are not).  The rotated parts of q and k turn as the position
encoding says: pairs (i, i + rot_dim/2) or neighbours (2i, 2i + 1), frequencies stretched or not.

A layer built with ``own_kv`` False has no W_dkv: it reads the cache entry that another layer of
the same geometry writes (``LayerCall.cache`` / ``writes_cache``) with its own W_uk, W_uv and
queries."""
from __future__ import annotations

from ..kernels import ops
from .base import CacheSpec, CacheTensor, Mixer, ParamSpec, Source, build_position_encoding, register_mixer

DEFAULT_NAMES = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm",
                 "k_up": "uk", "v_up": "uv", "sink": "sink", "gate": "g", "o": "o"}


class LatentAttention(Mixer):
    tree_name = "self_attn"
    capturable = True

    def __init__(self, hidden_size, num_heads, head_dim, rot_dim, value_dim, q_rank, kv_rank, scale, eps,
                 position=None, own_kv=True, sink=True, names=None, gate=True):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.head_dim, self.rot_dim, self.value_dim = head_dim, int(rot_dim), value_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale, self.eps = float(scale), float(eps)
        self.own_kv, self.sink, self.gate = bool(own_kv), bool(sink), bool(gate)
        self.position = build_position_encoding(position) if position is not None and self.rot_dim else None
        if self.position is not None and self.position.rotary_dim != self.rot_dim:
            raise ValueError("latent attention: the rotated part is rotated as a whole")
        if self.rot_dim % 2:
            raise ValueError("latent attention: the rotated part has an even size")
        #: width of a cache row and of a query row: what the attention kernels take
        self.stored_dim = -(-(kv_rank + self.rot_dim) // 16) * 16
        if self.stored_dim > ops.SUPPORTED_HEAD_DIMS[-1]:
            raise ValueError(f"latent attention: latent {kv_rank} + rotated part {self.rot_dim} exceeds rows of "
                             f"{ops.SUPPORTED_HEAD_DIMS[-1]} that the attention kernels take")
        self.q_size = num_heads * (head_dim + self.rot_dim)
        self.v_size = num_heads * value_dim
        self.kv_size = kv_rank + self.rot_dim if self.own_kv else 0
        self._sinks = None

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    def param_specs(self):
        nm, H = self.names, self.num_heads
        # the three products that read the mixer's input are one: query latent | kv latent + shared key part | gate
        rows, at = [], 0
        for name, n in ((nm["q_down"], self.q_rank), (nm["kv_down"], self.kv_size), (nm["gate"], self.v_size if self.gate else 0)):
            if n:
                rows.append(Source(f"{name}.weight", at, at + n))
                at += n
        specs = {
            "in_proj.weight": ParamSpec((at, self.hidden_size), sources=tuple(rows)),
            "q_norm.weight": ParamSpec((self.q_rank,), role="vector", init="norm_weight",
                                       sources=(Source(f"{nm['q_norm']}.weight", 0, self.q_rank),)),
            "q_up.weight": ParamSpec((self.q_size, self.q_rank), sources=(Source(f"{nm['q_up']}.weight", 0, self.q_size),)),
            "k_up.weight": ParamSpec((H * self.head_dim, self.kv_rank),
                                     sources=(Source(f"{nm['k_up']}.weight", 0, H * self.head_dim),)),
            "v_up.weight": ParamSpec((self.v_size, self.kv_rank), sources=(Source(f"{nm['v_up']}.weight", 0, self.v_size),)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.v_size),
                                       sources=(Source(f"{nm['o']}.weight", 0, self.hidden_size),)),
        }
        if self.own_kv:
            specs["kv_norm.weight"] = ParamSpec((self.kv_rank,), role="vector", init="norm_weight",
                                                sources=(Source(f"{nm['kv_norm']}.weight", 0, self.kv_rank),))
        if self.sink:
            # drawn like a matrix in the random-weights mode: sinks of zero would hide little, equal ones a mix-up of heads
            specs["sink"] = ParamSpec((H,), role="vector", init="normal", sources=(Source(nm["sink"], 0, H),))
        return specs

    def cache_spec(self):
        return CacheSpec("full", tensors=(CacheTensor("latent", 1, self.stored_dim),))

    def prepare(self, runtime):
        # sinks enter the softmax sum in 32-bit, whatever the checkpoint stores them as
        self._sinks = self.w["sink"].float().contiguous() if self.sink else None

    accepts_scaled_rows = True

    def work_tile_queries(self, dtype, page_size):
        return ops.prefill_tile_queries(dtype, self.num_heads, 1, self.stored_dim, page_size)

    def forward(self, h, ctx, call):
        H, n, nr, nv, r = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        proj = ops.materialize(ops.linear(h, self.w["in_proj.weight"]))
        cache = ctx.cache(call.cache)
        view = ctx.group(cache.group)
        rows = cache.tensors["latent"]
        writes = self.own_kv and call.writes_cache
        q_latent = ops.latent_prepare(
            proj, self.q_rank, self.w["q_norm.weight"], self.eps, kv_rank=r, rot_dim=nr,
            kv_weight=self.w["kv_norm.weight"] if writes else None, rotary=self.position, positions=ctx.positions,
            cache=rows if writes else None, slot_mapping=view.slot_mapping if writes else None)
        q = ops.materialize(ops.linear(q_latent, self.w["q_up.weight"]))
        T = q.shape[0]
        # the plain part of every head's query, carried into the latent space: [H, T, dim] x [H, dim, kv_rank]
        q_plain = q.view(T, H, n + nr)[:, :, :n].transpose(0, 1)
        carried = ops.batched_matmul(q_plain, self.w["k_up.weight"].view(H, n, r))
        q_rows = ops.latent_query(carried, q, H, n, nr, self.stored_dim, self.position, ctx.positions)
        mixed = ops.paged_attention(q_rows, rows, rows, view, ctx, self.scale, sinks=self._sinks)
        # [H, T, kv_rank] x [H, kv_rank, vdim]: every head's weighted latent expanded to its values
        wide, w_uv = mixed[:, :, :r].transpose(0, 1), self.w["v_up.weight"].view(H, nv, r).transpose(1, 2)
        if not self.gate:
            return ops.linear(ops.batched_matmul(wide, w_uv, side_by_side=True), self.w["o_proj.weight"], allow_pending=True)
        gate = proj[:, self.q_rank + self.kv_size:]
        return ops.linear(ops.gate_heads(ops.batched_matmul(wide, w_uv), gate), self.w["o_proj.weight"], allow_pending=True)


register_mixer("latent_attention", LatentAttention)
