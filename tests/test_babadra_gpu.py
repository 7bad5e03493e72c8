"""Babadra on the device against the plain implementation (tests/plain_babadra.py): each
mechanism alone through its kernel, then whole models through the step function: whole prompts,
prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages and
slots that are used again, far keys and keys at page borders that the weights are made to show,
long decoding, other sizes, and greedy generation through the entry point."""
import json
import math
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_babadra as plain
from babadra_configs import BABADRA_TINY, _attention, _dense, _latent, _moe, decisive, make_babadra_dir, random_babadra_config_dict
from helpers import (collect_logits, lines_of, max_live_tokens, random_ids, schedule_mixed, schedule_portions,
                     schedule_tail_decode, schedule_whole)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# Largest |logit difference|, and largest root-mean-square difference over the vocabulary at one
# position, over the largest plain |logit|.  float32: 32-bit sums against float64, the sharp test of
# every schedule.  bfloat16: products and activations rounded to 8 bits through tiny random layers;
# it catches a kernel that is wrong, not one that rounds elsewhere.
TOLERANCE = {"float32": 5e-5, "bfloat16": 2e-1}
RMS_TOLERANCE = {"float32": 1.7e-5, "bfloat16": 6e-2}
MEASURED = {}


def draws(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).bfloat16().double()


def on_device(x, dtype):
    return x.to(dtype).to(DEV).contiguous()


class Tables:
    def __init__(self, rot, n, pairing):
        from tinyserve_b200.parts.rotary import Rotary
        part = Rotary(rot["dims"], rot["base"], pairing, rot.get("scaling"))
        self.rotary_dim, self.interleaved = rot["dims"], part.interleaved
        cos, sin = Rotary.tables(part.rotary_dim, part.theta, n, part.scaling)
        self.cos, self.sin = cos.to(DEV), sin.to(DEV)


# ----------------------------------------------------------------------------- the stream
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("T,n", [(23, 41), (23, 40), (7, 200), (600, 1000), (4, 2048), (3, 5000), (40, 2048)])
def test_sub_layer_output_times_its_factors_joins_the_stream_in_32_bit(dtype, tol, T, n):
    """The kernels that add and norm (rows of any length, many rows, few rows over a cluster), with
    one factor per column on what is added; on chosen rows; and the add alone, with the kept
    embedding output beside it."""
    from tinyserve_b200.kernels import ops
    r, y = draws(T, n, seed=1, scale=3.0), draws(T, n, seed=2, scale=0.5)
    s, w = (draws(n, seed=3, scale=0.7) + 0.2).bfloat16().double(), draws(n, seed=4, scale=0.1)
    residual = on_device(r, torch.float32)
    scaled = ops.ColumnScaled(on_device(y, dtype), on_device(s, dtype))
    out = ops.add_rmsnorm(scaled, residual, on_device(1 + w, torch.float32), 1e-6, dtype)
    stream = r + y * s
    want = plain.norm_around_zero(stream, w, 1e-6)
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()
    assert (residual.double().cpu() - stream).abs().max() <= 1e-6 * stream.abs().max(), "the product and the sum are 32-bit"
    assert (scaled.materialize().double().cpu() - y * s).abs().max() <= tol * (y * s).abs().max()
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device=DEV)
    before = residual.clone()
    some = ops.add_rmsnorm(scaled, residual, on_device(1 + w, torch.float32), 1e-6, dtype, rows=rows)
    assert torch.equal(before, residual), "with rows the residual is left as it is"
    want = plain.norm_around_zero(before.double().cpu() + y * s, w, 1e-6)[[T - 1, 0, T // 2]]
    assert (some.double().cpu() - want).abs().max() <= tol * want.abs().max()
    # the add alone: pending output times its factors, and the stream as it left the embedding
    first = draws(T, n, seed=5, scale=2.0)
    residual = on_device(r, torch.float32)
    ops.stream_add_(residual, scaled, on_device(first, torch.float32))
    assert (residual.double().cpu() - (r + y * s + first)).abs().max() <= 1e-6 * stream.abs().max()
    ops.stream_add_(residual, None, on_device(first, torch.float32))
    ops.stream_add_(residual, on_device(y, dtype))
    assert (residual.double().cpu() - (r + y * s + 2 * first + y)).abs().max() <= 2e-6 * stream.abs().max()


@pytest.mark.parametrize("M,K,N", [(3, 2048, 1024), (16, 4096, 512), (1, 1024, 2048)])
def test_factors_on_a_product_that_is_still_partial_tiles(M, K, N):
    """A few bfloat16 rows: the product before the add stops at its split-K partial tiles, and the
    kernel that adds them to the stream multiplies their sum by the factors."""
    from tinyserve_b200.kernels import ops
    x, W = draws(M, K, seed=1), draws(N, K, seed=2, scale=0.05)
    s, w, r = (draws(N, seed=3) + 0.1).bfloat16().double(), draws(N, seed=4, scale=0.1), draws(M, N, seed=5, scale=2.0)
    for first in (None, draws(M, N, seed=6)):
        pending = ops.linear(on_device(x, torch.bfloat16), on_device(W, torch.bfloat16), allow_pending=True)
        scaled = ops.ColumnScaled(pending, on_device(s, torch.bfloat16))
        residual = on_device(r, torch.float32)
        stream = r + (x @ W.T) * s
        if first is not None:
            ops.stream_add_(residual, scaled, on_device(first, torch.float32))
            assert (residual.double().cpu() - (stream + first)).abs().max() <= 1e-5 * stream.abs().max()
            continue
        want = plain.norm_around_zero(stream, w, 1e-6)
        for scaled_ok in (False, True):
            # (a reader that only multiplies takes rows without their norm factor: the product then adds to the
            # residual itself, factors included)
            residual = on_device(r, torch.float32)
            out = ops.add_rmsnorm(scaled, residual, on_device(1 + w, torch.float32), 1e-6, torch.bfloat16, scaled_ok=scaled_ok)
            assert isinstance(out, ops.ScaledRows if scaled_ok else torch.Tensor)
            assert (residual.double().cpu() - stream).abs().max() <= 1e-5 * stream.abs().max()
            assert (ops.materialize(out).double().cpu() - want).abs().max() <= 1e-2 * want.abs().max()


def test_embedding_rows_are_scaled_in_32_bit():
    from tinyserve_b200.kernels import ops
    table = draws(50, 24, seed=1)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device=DEV)
    for dtype in (torch.float32, torch.bfloat16):
        out = ops.embed_lookup(on_device(table, dtype), ids, scale=5.5)
        assert out.dtype == torch.float32 and (out.double().cpu() - table[[3, 49, 0, 3]] * 5.5).abs().max() < 1e-6 * 5.5 * table.abs().max()
        assert torch.equal(ops.embed_lookup(on_device(table, dtype), ids).cpu(), table[[3, 49, 0, 3]].float())


# ----------------------------------------------------------------------------- feed-forward
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("limit", [0.5, 1.5, 20.0])
def test_bounded_gate(dtype, tol, limit):
    """gate | up in halves and in alternating blocks of 64 columns; values on both sides of the bound."""
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts.base import interleave_halves
    T, ff = 19, 192
    g, u = draws(T, ff, seed=1, scale=2.0), draws(T, ff, seed=2, scale=2.0)
    want = plain.bounded_gate(g, u, limit)
    halves = torch.cat([g, u], 1)
    got = ops.gated_activation(on_device(halves, dtype), "bounded_swish", 0, limit)
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    blocks = interleave_halves(halves.T.contiguous(), 64).T.contiguous()
    got = ops.gated_activation(on_device(blocks, dtype), "bounded_swish", 64, limit)
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()
    odd = ops.gated_activation(on_device(halves[:, list(range(5)) + list(range(ff, ff + 5))], dtype), "bounded_swish", 0, limit)
    assert (odd.double().cpu() - want[:, :5]).abs().max() <= tol * want.abs().max()
    with pytest.raises(ValueError):
        ops.gated_activation(on_device(halves, dtype), "bounded_swish")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T,width,ff", [(1, 64, 72), (9, 128, 192), (70, 256, 384), (300, 96, 104)])
def test_dense_feed_forward_against_the_plain_one(dtype, tol, T, width, ff):
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts.base import interleave_halves
    from tinyserve_b200.parts.mlp import GatedMLP
    h = draws(T, width, seed=1)
    W = {"gate": draws(ff, width, seed=2, scale=0.2), "up": draws(ff, width, seed=3, scale=0.2), "down": draws(width, ff, seed=4, scale=0.2)}
    part = GatedMLP(width, ff, "bounded_swish", limit=0.9)
    fused = interleave_halves(torch.cat([W["gate"], W["up"]]), part.block)
    part.bind({"gate_up_proj.weight": on_device(fused, dtype), "down_proj.weight": on_device(W["down"], dtype)})
    got = ops.materialize(part.forward(on_device(h, dtype), None))
    want = plain.gated_ff(h, W, "", 0.9)
    assert (got.double().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("M,K,N", [(7, 256, 384), (16, 512, 2048), (2048, 4096, 512)])
def test_bounded_gate_in_the_epilogue_of_the_products(M, K, N):
    """A few bfloat16 rows and a long prompt portion: the product applies the gate itself; the same
    numbers, to a rounding, as the product followed by the activation kernel."""
    from tinyserve_b200.kernels import ops
    x, W = on_device(draws(M, K, seed=1), torch.bfloat16), on_device(draws(N, K, seed=2, scale=0.05), torch.bfloat16)
    launches = ops.launch_count()
    fused = ops.gated_linear(x, W, "bounded_swish", ops.GATED_BLOCK, 0.7)
    assert ops.launch_count() - launches == 1 or ops.gemm_splits(M, N, K) > 1, "one kernel where the product is not cut along K"
    apart = ops.gated_activation(ops.materialize(ops.linear(x, W)), "bounded_swish", ops.GATED_BLOCK, 0.7)
    assert fused.shape == (M, N // 2)
    assert (fused.double() - apart.double()).abs().max() <= 1e-2 * apart.double().abs().max()
    assert apart.double().abs().max() > 0.5


@pytest.mark.parametrize("E,top", [(8, 2), (5, 5), (1, 1), (40, 7), (3, 1)])
def test_router_weights_are_the_softmax_over_the_chosen_logits(E, top):
    from tinyserve_b200.kernels import ops
    z = torch.randn(33, E, generator=torch.Generator().manual_seed(E), dtype=torch.float64) * 3.0
    z[5] -= 60.0                                  # a shift of all logits changes nothing
    gates = ops.moe_route(on_device(z, torch.float32), top, renormalize=True).double().cpu()
    best, idx = torch.topk(z, top, -1)
    want = torch.zeros_like(z).scatter(1, idx, torch.softmax(best, -1))
    assert (gates - want).abs().max() < 1e-6
    assert ((gates.sum(-1) - 1).abs() < 1e-6).all() and ((gates > 0).sum(-1) <= top).all()
    b = draws(E, seed=9, scale=2.0)
    biased = ops.moe_route(on_device(z, torch.float32), top, renormalize=True, bias=on_device(b, torch.float32)).double().cpu()
    best, at = torch.topk(z + b, top, -1)
    assert (biased - torch.zeros_like(z).scatter(1, at, torch.softmax(best, -1))).abs().max() < 1e-6
    kept = ops.moe_route(on_device(z, torch.float32), top).double().cpu()
    assert (kept - torch.zeros_like(z).scatter(1, idx, torch.softmax(z, -1).gather(1, idx))).abs().max() < 1e-6, "the other form stays"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("E,top,ff,width", [(4, 1, 40, 64), (6, 2, 24, 64), (1, 1, 48, 96), (7, 7, 72, 96), (16, 5, 32, 128), (12, 4, 64, 192)])
@pytest.mark.parametrize("T", [29, 300])
def test_experts_against_the_plain_ones(dtype, tol, E, top, ff, width, T):
    """A few tokens (all experts on all tokens, the unchosen ones times zero) and a step of 300 tokens
    (in bfloat16: rows sorted by expert); a router bias that decides who is chosen."""
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts.moe import MixtureOfExperts
    h = draws(T, width, seed=1)
    W = {"router": draws(E, width, seed=2, scale=0.5), "router.b": draws(E, seed=3, scale=3.0)}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"] = draws(ff, width, seed=10 + e, scale=0.2), draws(ff, width, seed=70 + e, scale=0.2)
        W[f"e{e}.down"] = draws(width, ff, seed=40 + e, scale=0.2)
    mlp = {"expert": {"ff": ff, "limit": 0.8}, "router": {"experts": E, "top": top}}
    without = plain.route(h, {**W, "router.b": torch.zeros(E, dtype=torch.float64)}, "", mlp["router"])[0]
    assert E == 1 or top == E or not torch.equal(without, plain.route(h, W, "", mlp["router"])[0]), "the bias matters here"
    part = MixtureOfExperts(width, ff, E, top, activation="bounded_swish_gated", router="softmax_chosen", limit=0.8, router_bias=True)
    part.bind({"router.weight": on_device(W["router"], dtype), "router.bias": on_device(W["router.b"], dtype),
               "up.weight": on_device(torch.cat([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(E)]), dtype),
               "down.weight": on_device(torch.cat([W[f"e{e}.down"] for e in range(E)]), dtype)})
    got = ops.materialize(part.forward(on_device(h, dtype), None))
    want = plain.experts(h, W, "", mlp)
    # (in bfloat16 a token whose router logits are a rounding apart may take another expert: one row in fifty may differ)
    err = (got.double().cpu() - want).abs().max(-1).values
    allowed = T // 50 if dtype == torch.bfloat16 else 0
    assert int((err > tol * want.abs().max()).sum()) <= allowed
    if dtype == torch.bfloat16 and T >= ops.MOE_GROUPED_MIN_TOKENS and top < E:
        keep, ops.MOE_GROUPED_MIN_TOKENS = ops.MOE_GROUPED_MIN_TOKENS, 10 ** 9
        try:
            dense = ops.materialize(part.forward(on_device(h, dtype), None))
        finally:
            ops.MOE_GROUPED_MIN_TOKENS = keep
        assert (got.double() - dense.double()).abs().max() <= tol * want.abs().max(), "both forms route alike and agree to a rounding"


# ----------------------------------------------------------------------------- latent attention
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,n,nr,nv,qr,r", [(3, 16, 8, 24, 40, 24), (2, 8, 12, 16, 16, 20), (4, 32, 16, 32, 64, 48), (1, 20, 0, 6, 8, 12)])
def test_latent_rows_turn_in_neighbouring_pairs_with_stretched_waves(dtype, tol, H, n, nr, nv, qr, r):
    from tinyserve_b200.kernels import ops
    T, page, eps = 9, 4, 1e-5
    stored = -(-(r + nr) // 16) * 16
    rot = {"base": 100.0, "dims": nr, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    tables = Tables(rot, 64, "interleaved") if nr else None
    pos = torch.tensor([40, 41, 42, 43, 44, 0, 1, 2, 3], dtype=torch.int32)
    proj = draws(T, qr + r + nr, seed=1, scale=2.0)
    wq, wk = draws(qr, seed=2) + 1, draws(r, seed=3) + 1
    slots = torch.tensor([37, 2, 19, -1, 8, 11, 30, 4, 25], dtype=torch.int32)
    cache = torch.full((10, 1, page, stored), 7.0).to(dtype).to(DEV)
    ql = ops.latent_prepare(on_device(proj, dtype), qr, on_device(wq, dtype), eps, kv_rank=r, rot_dim=nr,
                            kv_weight=on_device(wk, dtype), rotary=tables, positions=pos.to(DEV), cache=cache,
                            slot_mapping=slots.to(DEV))
    want_q = plain.norm_plain(proj[:, :qr], wq, eps)
    assert (ql.double().cpu() - want_q).abs().max() <= tol * want_q.abs().max()
    c = plain.norm_plain(proj[:, qr:qr + r], wk, eps)
    kr = plain.rotate(proj[:, None, qr + r:], pos, rot, "neighbours")[:, 0] if nr else proj[:, :0]
    flat = cache.view(-1, stored).double().cpu()
    for t in range(T):
        if slots[t] < 0:
            continue
        row = flat[slots[t]]
        assert (row[:r] - c[t]).abs().max() <= tol * c.abs().max()
        assert nr == 0 or (row[r:r + nr] - kr[t]).abs().max() <= tol * kr.abs().max()
        assert (row[r + nr:] == 0).all()
    q = draws(T, H * (n + nr), seed=4)
    w_uk = draws(H * n, r, seed=5)
    carried = ops.batched_matmul(on_device(q, dtype).view(T, H, n + nr)[:, :, :n].transpose(0, 1), on_device(w_uk, dtype).view(H, n, r))
    rows = ops.latent_query(carried, on_device(q, dtype), H, n, nr, stored, tables, pos.to(DEV))
    qv = q.view(T, H, n + nr)
    if nr:
        assert (rows[..., r:r + nr].double().cpu() - plain.rotate(qv[..., n:], pos, rot, "neighbours")).abs().max() <= tol * 2 * q.abs().max()
    assert (rows[..., r + nr:] == 0).all()
    # the values' side without a gate: every head's weighted latent expanded, heads side by side
    mixed = draws(T, H, stored, seed=6)
    w_uv = draws(H * nv, r, seed=7)
    values = ops.batched_matmul(on_device(mixed, dtype)[:, :, :r].transpose(0, 1), on_device(w_uv, dtype).view(H, nv, r).transpose(1, 2))
    got = ops.gate_heads(values, None)
    want = torch.einsum("thr,hvr->thv", mixed[..., :r], w_uv.view(H, nv, r)).reshape(T, H * nv)
    assert (got.double().cpu() - want).abs().max() <= 2 * tol * want.abs().max()
    straight = ops.batched_matmul(on_device(mixed, dtype)[:, :, :r].transpose(0, 1), on_device(w_uv, dtype).view(H, nv, r).transpose(1, 2),
                                  side_by_side=True)
    assert straight.shape == got.shape and straight.is_contiguous()
    assert (straight.double() - got.double()).abs().max() <= tol * want.abs().max(), "the product writes the heads side by side itself"


# ----------------------------------------------------------------------------- two score maps
def _pages(lengths, page, seed):
    """A block table over shuffled pages for requests of these lengths, and every token's slot."""
    g = torch.Generator().manual_seed(seed)
    need = sum(-(-n // page) for n in lengths)
    order = (torch.randperm(need + 2, generator=g) + 1).tolist()
    table = torch.zeros(len(lengths), max(-(-n // page) for n in lengths) + 2, dtype=torch.int32)
    slots = []
    for b, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
        slots += [int(table[b, j // page]) * page + j % page for j in range(n)]
    return table.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV), need + 3


def _two_map_case(H, G, n, nv, rot, scale, cap, diff, kv_lens, seed):
    """Projections of whole sequences (bfloat16 numbers), the plain result per request, and the weights."""
    T = sum(kv_lens)
    width = (2 * H + 2 * G) * n + G * nv
    h = draws(T, width, seed=seed, scale=1.5)
    eye = torch.eye(width, dtype=torch.float64)
    W = {"q": eye[:2 * H * n], "k": eye[2 * H * n:2 * (H + G) * n], "v": eye[2 * (H + G) * n:], "o": torch.eye(H * nv, dtype=torch.float64),
         "q.norm": (draws(n, seed=seed + 1, scale=0.3) + 1).bfloat16().double(),
         "k.norm": (draws(n, seed=seed + 2, scale=0.3) + 1).bfloat16().double()}
    for i, key in enumerate(("lq1", "lk1", "lq2", "lk2")):
        W[key] = draws(n, seed=seed + 3 + i, scale=0.6 / math.sqrt(n)) + 0.3 / math.sqrt(n)
    m = {"heads": H, "kv_heads": G, "dim": n, "vdim": nv, "scale": scale, "diff": diff, "rot": rot}
    if cap:
        m["softcap"] = cap
    want, at = [], 0
    for kv in kv_lens:
        want.append(plain.differential_attention(h[at:at + kv], W, "", m, 1e-5))
        at += kv
    return h, W, m, want


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("H,G,n,nv,page", [(4, 2, 16, 32, 8), (3, 1, 48, 16, 16), (2, 2, 24, 16, 4), (6, 3, 20, 40, 16),
                                           (4, 1, 64, 64, 32), (2, 1, 128, 128, 64), (2, 2, 32, 128, 16)])
@pytest.mark.parametrize("cap", [None, 3.0, 40.0])
def test_two_score_maps_over_the_same_values(dtype, tol, H, G, n, nv, page, cap):
    """q/k norm with shared weights, rotation of a part of every map, the maps' rows as the
    attention kernels want them, one value head for both maps, capped scores, the maps' difference normed per head:
    a whole prompt, single tokens, a portion after a prefix, two tokens and a request of one token, on
    every attention kernel that takes the head size, with and without key ranges."""
    from tinyserve_b200.kernels import ops
    kv_lens, q_lens = [70, 24, 97, 9, 150, 1], [70, 1, 29, 2, 1, 1]
    rot = {"base": 100.0, "dims": n // 2 if n % 4 == 0 else n}
    scale, diff = 2.0 / math.sqrt(n), 0.3
    h, W, m, want = _two_map_case(H, G, n, nv, rot, scale, cap, diff, kv_lens, seed=11)
    lam = plain.differential_lambda(W, "", m)
    assert abs(lam - diff) > 0.05, "lambda is not its constant here"
    D = -(-max(n, nv) // 16) * 16
    table, slots, pages = _pages(kv_lens, page, seed=2)
    kc = torch.full((pages, 2 * G, page, D), 30.0).to(dtype).to(DEV)
    vc = torch.full((pages, G, page, D), 30.0).to(dtype).to(DEV)            # one value head for both maps of a key/value head
    pos = torch.cat([torch.arange(kv) for kv in kv_lens]).to(torch.int32).to(DEV)
    x = on_device(h, dtype)
    q_end, k_end = 2 * H * n, 2 * (H + G) * n
    tables = Tables(rot, 256, "half")
    q_all = ops.rope_unit_kvwrite(x[:, :q_end], x[:, q_end:k_end], x[:, k_end:], pos, 2 * H, 2 * G, n, nv, D, rotary=tables,
                                  k_cache=kc, v_cache=vc, slot_mapping=slots, page_size=page,
                                  q_weight=on_device(W["q.norm"], dtype), k_weight=on_device(W["k.norm"], dtype), pre_eps=1e-5, maps=2)
    # what the step reads of q: the last q_len tokens of every request
    starts = np.concatenate([[0], np.cumsum(kv_lens)])
    take = torch.cat([torch.arange(starts[b] + kv - ql, starts[b] + kv) for b, (kv, ql) in enumerate(zip(kv_lens, q_lens))])
    q = q_all[take.to(DEV)].contiguous()
    expect = torch.cat([w[kv - ql:] for w, kv, ql in zip(want, kv_lens, q_lens)])
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(cu_q=cu, kv_lens=torch.tensor(kv_lens, dtype=torch.int32, device=DEV), num_requests=len(q_lens),
                          max_q_len=max(q_lens), max_kv_len=max(kv_lens), host={}, tile_cache={})
    view = SimpleNamespace(block_table=table, page_size=page)
    chosen = ops.attention_backend(dtype, D, page)
    for backend in {"tcgen05": ["tcgen05", "mma", "simt"], "mma": ["mma", "simt"], "simt": ["simt"]}[chosen]:
        for splits in (None, 3):
            if splits and backend == "tcgen05":
                continue
            out = ops.paged_attention(q, kc, vc, view, ctx, scale, num_splits=splits, backend=backend, softcap=cap or 0.0)
            got = ops.map_difference(out, H, G, nv, lam, 1e-5, 1.0 - diff)
            assert (got.double().cpu() - expect).abs().max() <= tol * expect.abs().max(), (backend, splits)
    # decoding alone (every request one token): the split-KV kernels
    one = torch.tensor([starts[b] + kv - 1 for b, kv in enumerate(kv_lens)])
    ctx1 = SimpleNamespace(cu_q=torch.arange(len(kv_lens) + 1, dtype=torch.int32, device=DEV), kv_lens=ctx.kv_lens,
                           num_requests=len(kv_lens), max_q_len=1, max_kv_len=max(kv_lens), host={}, tile_cache={})
    out = ops.paged_attention(q_all[one.to(DEV)].contiguous(), kc, vc, view, ctx1, scale, softcap=cap or 0.0)
    got = ops.map_difference(out, H, G, nv, lam, 1e-5, 1.0 - diff)
    expect1 = torch.stack([w[-1] for w in want])
    assert (got.double().cpu() - expect1).abs().max() <= tol * expect1.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,page", [(32, 16), (64, 16), (128, 64)])
def test_capped_scores_flatten_a_key_that_stands_out(dtype, D, page):
    """One key's score is far above all others: without a cap the output is its value; with a cap of c
    no score exceeds c, and the key weighs exp(c - s) against a key of score s.  The key stands far
    back, at a page's border, and last; prompts and single tokens."""
    from tinyserve_b200.kernels import ops
    H, G, n = 2, 1, 300
    direction = torch.ones(D) / math.sqrt(D)
    for marked in (0, page - 1, page, n - 140, n - 1):
        k = draws(n, G, D, seed=1, scale=0.02)
        v = draws(n, G, D, seed=2)
        k[marked] = (direction * 40).bfloat16().double()
        qrow = (direction * 40).bfloat16().double()
        table, slots, pages = _pages([n], page, seed=3)
        flat_k, flat_v = torch.zeros(pages * page, G, D, dtype=dtype, device=DEV), torch.zeros(pages * page, G, D, dtype=dtype, device=DEV)
        flat_k[slots.long()], flat_v[slots.long()] = on_device(k, dtype), on_device(v, dtype)
        kc = flat_k.view(pages, page, G, D).permute(0, 2, 1, 3).contiguous()
        vc = flat_v.view(pages, page, G, D).permute(0, 2, 1, 3).contiguous()
        view = SimpleNamespace(block_table=table, page_size=page)
        for q_len in (1, 40):
            q = on_device(qrow.repeat(q_len, H, 1), dtype)
            ctx = SimpleNamespace(cu_q=torch.tensor([0, q_len], dtype=torch.int32, device=DEV),
                                  kv_lens=torch.tensor([n], dtype=torch.int32, device=DEV), num_requests=1, max_q_len=q_len,
                                  max_kv_len=n, host={}, tile_cache={})
            for cap in (0.0, 2.0):
                out = ops.paged_attention(q, kc, vc, view, ctx, 1.0, softcap=cap)[-1, 0].double().cpu()
                s = k[:, 0] @ qrow
                if cap:
                    s = cap * torch.tanh(s / cap)
                want = torch.softmax(s, 0) @ v[:, 0]
                assert (out - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * v.abs().max(), (marked, q_len, cap)
                miss = (out - v[marked, 0]).abs().max().item()
                assert (miss < 2e-2) == (cap == 0.0), (marked, q_len, cap, miss)


# ----------------------------------------------------------------------------- whole models
LENGTHS = {"P": [5, 37, 40, 70, 2, 1, 33], "Q": [1, 9, 64, 100, 31, 48], "R": [150, 130, 57, 3, 129]}


@pytest.fixture(scope="module", params=sorted(BABADRA_TINY))
def model(request, tmp_path_factory):
    name = request.param
    folder = make_babadra_dir(tmp_path_factory.mktemp(f"babadra{name}"), name, seed=41)
    cfg, weights = plain.load_folder(folder)
    reqs = {f"r{i}": random_ids(cfg["vocab"], n, seed=300 + i) for i, n in enumerate(LENGTHS[name])}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs, "ref": ref}


def run_replay(folder, dtype, steps, out_dir, page=16, max_live=4, graphs=False):
    from tinyserve_b200.engine import replay
    runner = replay.make_runner(folder, dtype, max_live_tokens(steps, max(64, page)), block_size=page,
                                max_live=max_live, use_cuda_graphs=graphs)
    done = []
    replay.replay(runner, lines_of(steps), str(out_dir), done.append)
    assert done == [f"done {s['step']}" for s in steps]
    runner.manager.check_invariants()
    assert not runner.manager.requests and all(p.num_free == p.num_usable for p in runner.manager.pools)
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            data = np.fromfile(os.path.join(str(out_dir), f"{s['step']}.f32"), dtype="<f4")
            outputs[s["step"]] = torch.from_numpy(data.reshape(wanted, runner.model.vocab_size))
    return outputs, runner


def check(model, dtype, steps, out_dir, slack=1.0, **kw):
    outputs, runner = run_replay(model["folder"], dtype, steps, out_dir, **kw)
    got = collect_logits(steps, outputs, model["cfg"]["vocab"])
    # In bfloat16 a token whose router logits lie within a rounding of one another may take another
    # expert than the plain model does; one position in twenty may differ for that reason; none in
    # 32-bit, where every schedule is held to the plain model at every position.
    positions = sum(out.shape[0] for out in got.values())
    allowed = positions // 20 if dtype == "bfloat16" else 0
    over = []
    for rid, out in got.items():
        ref = model["ref"][rid.rstrip("x")]
        assert out.shape == ref.shape
        scale = ref.abs().max().item()
        err = (out.double() - ref).abs().max(-1).values / scale
        rms = (out.double() - ref).pow(2).mean(-1).sqrt() / scale
        bad = ((err > slack * TOLERANCE[dtype]) | (rms > slack * RMS_TOLERANCE[dtype]))
        seen = MEASURED.setdefault((model["name"], dtype), [0.0, 0.0])
        if (~bad).any():
            seen[0], seen[1] = max(seen[0], err[~bad].max().item()), max(seen[1], rms[~bad].max().item())
        over += [(rid, int(i), err[int(i)].item(), rms[int(i)].item()) for i in bad.nonzero()]
    assert len(over) <= allowed, (f"{model['name']} {dtype}: {len(over)} of {positions} positions differ; the first is place "
                                  f"{over[0][1]} of request {over[0][0]} (error {over[0][2]:.3e}, rms {over[0][3]:.3e})")
    return runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(model, dtype, tmp_path):
    check(model, dtype, schedule_whole(model["requests"]), tmp_path)


def test_stream_after_every_layer_run(model):
    """The 32-bit stream behind every run of a layer (a repeated layer counts each time), read off the
    model's own forward pass, against the plain one's."""
    from tinyserve_b200.engine import replay
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.kernels import ops
    ids = model["requests"]["r1"]
    _, want = plain.forward(model["cfg"], model["weights"], ids, return_layers=True)
    runner = replay.make_runner(model["folder"], "float32", 256)
    seen = []
    blocks = runner.model.blocks
    originals = [b.forward for b in blocks]

    def watched(block, original):
        def forward(x, residual, ctx, call):
            out = original(x, residual, ctx, call)
            stream = residual.clone()
            ops.stream_add_(stream, out)
            seen.append(stream.double().cpu())
            return out
        return forward

    for b, original in zip(blocks, originals):
        b.forward = watched(b, original)
    runner.manager.begin("a")
    runner.step([StepEntry("a", ids, [len(ids) - 1])])
    runner.manager.free("a")
    assert len(seen) == want.shape[0]
    for i, got in enumerate(seen):
        assert (got - want[i]).abs().max() <= 2e-5 * want[i].abs().max(), f"layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_against_token_by_token(model, dtype, tmp_path):
    """The last 32 tokens one by one; and everything but the first token one by one (the first
    tokens of a sequence, a long run of decoding)."""
    check(model, dtype, schedule_tail_decode(model["requests"], 32), tmp_path / "tail")
    longest = max(model["requests"], key=lambda r: len(model["requests"][r]))
    one = {longest: model["requests"][longest]}
    check(model, dtype, schedule_tail_decode(one, len(one[longest]) - 1), tmp_path / "all", graphs=dtype == "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(model, dtype, tmp_path):
    check(model, dtype, schedule_portions(model["requests"]), tmp_path / "a")
    check(model, dtype, schedule_portions(model["requests"], sizes=(2,)), tmp_path / "twos")
    check(model, dtype, schedule_portions(model["requests"], sizes=(16, 1, 15, 17, 32, 3)), tmp_path / "edges", page=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_reuse_pages_and_slots(model, dtype, seed, tmp_path):
    reqs = dict(model["requests"])
    more = {f"{rid}x": ids for rid, ids in reqs.items()}
    steps = schedule_mixed({**reqs, **more}, max_live=4, seed=seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), "portions beside single tokens"
    runner = check(model, dtype, steps, tmp_path, max_live=4)
    assert len(reqs) + len(more) > runner.manager.slots.num_slots == 4, "slots are used again"
    total = sum(-(-len(i) // 16) for i in {**reqs, **more}.values())
    assert total > runner.manager.pools[0].num_usable, "the pool is too small to avoid reuse"


def test_batch_of_unequal_requests_equals_each_alone(model, tmp_path):
    reqs = model["requests"]
    together = [{"step": 0, "entries": [{"id": r, "tokens": ids, "want": list(range(len(ids)))} for r, ids in reqs.items()],
                 "end": list(reqs)}]
    out_a, _ = run_replay(model["folder"], "float32", together, tmp_path / "a", max_live=len(reqs))
    out_b, _ = run_replay(model["folder"], "float32", schedule_whole(reqs), tmp_path / "b")
    a = collect_logits(together, out_a, model["cfg"]["vocab"])
    b = collect_logits(schedule_whole(reqs), out_b, model["cfg"]["vocab"])
    for rid in reqs:
        # (the attention kernel cuts a request's keys into ranges by how full the batch is: the
        # order of its sums, not what is summed, depends on the batch)
        assert (a[rid] - b[rid]).abs().max() <= 1e-5 * b[rid].abs().max()


@pytest.mark.parametrize("seed", range(12))
def test_drawn_configurations(seed, tmp_path):
    """Configurations drawn from a seed (odd head sizes, head counts, ranks, orders, repeated groups,
    layers without feed-forward, rotation over all, a part or none of a head): whole prompts,
    portions and a mixed batch against the plain implementation."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model
    raw = random_babadra_config_dict(seed)
    folder = decisive(write_random_model(config_from_dict(raw), str(tmp_path / "model"), seed=seed), seed)
    cfg, weights = plain.load_folder(folder)
    reqs = {f"r{i}": random_ids(cfg["vocab"], n, seed=700 + 10 * seed + i) for i, n in enumerate((37, 5, 66, 1))}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    model = {"name": f"drawn{seed}", "folder": folder, "cfg": cfg, "requests": reqs, "ref": ref}
    check(model, "float32", schedule_whole(reqs), tmp_path / "whole", slack=2.0)
    check(model, "float32", schedule_portions(reqs, sizes=(17, 2, 16, 1, 3)), tmp_path / "portions", slack=2.0)
    check(model, "float32", schedule_mixed(reqs, max_live=3, seed=seed), tmp_path / "mixed", slack=2.0, max_live=3)
    check(model, "bfloat16", schedule_mixed(reqs, max_live=3, seed=seed), tmp_path / "mixed16", slack=2.0, max_live=3)


# ----------------------------------------------------------------------------- weights that show a fault
def sharpened(folder, out, cfg):
    """The same model with its attention sharp (large scales, so that a far key, a key at a page's
    border or a wrong position moves the logits) and small caps on the scores (so that a cap that is
    left out shows)."""
    weights = load_file(os.path.join(folder, "model.safetensors"))
    cfg = {**cfg, "layers": [dict(layer) for layer in cfg["layers"]]}
    for layer in cfg["layers"]:
        m = dict(layer["mixer"])
        m["scale"] = 3.0 if layer["type"] == "attention" else 1.5
        if layer["type"] == "attention":
            m["softcap"] = 6.0
        layer["mixer"] = m
    os.makedirs(out, exist_ok=True)
    save_file(weights, os.path.join(out, "model.safetensors"))
    with open(os.path.join(out, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "R"])
def test_far_keys_caps_and_the_first_tokens(dtype, name, tmp_path):
    folder = make_babadra_dir(tmp_path / "base", name, seed=43)
    cfg, _ = plain.load_folder(folder)
    sharp = sharpened(folder, str(tmp_path / "sharp"), cfg)
    cfg, weights = plain.load_folder(sharp)
    most = cfg["max_positions"]
    ids = random_ids(cfg["vocab"], min(200, most), seed=7)
    ids[130] = ids[-1] = ids[3]               # a token that comes back far behind
    reqs = {"far": ids, "near": ids[:70]}
    ref = {rid: plain.logits(cfg, weights, t) for rid, t in reqs.items()}
    other = list(ids)
    other[3] = (ids[3] + 1) % cfg["vocab"]
    assert (plain.logits(cfg, weights, other)[-1] - ref["far"][-1]).abs().max() > 0.01 * ref["far"].abs().max(), "a far token matters here"
    uncapped = {**cfg, "layers": [{**l, "mixer": {k: v for k, v in l["mixer"].items() if k != "softcap"}} for l in cfg["layers"]]}
    assert (plain.logits(uncapped, weights, ids) - ref["far"]).abs().max() > 1e-2 * ref["far"].abs().max(), "the caps matter"
    unscaled = {k: (torch.ones_like(v) if k.endswith((".ls1", ".ls2")) else v) for k, v in weights.items()}
    assert (plain.logits(cfg, unscaled, ids) - ref["far"]).abs().max() > 1e-2 * ref["far"].abs().max(), "the factors matter"
    model = {"name": name + "sharp", "folder": sharp, "cfg": cfg, "requests": reqs, "ref": ref}
    slack = 2.0 if dtype == "float32" else 3.0
    check(model, dtype, schedule_whole(reqs), tmp_path / "whole", slack=slack)
    check(model, dtype, schedule_tail_decode(reqs, 90), tmp_path / "tail", slack=slack)
    check(model, dtype, schedule_portions(reqs, sizes=(63, 2, 1, 64, 5, 16, 15)), tmp_path / "portions", slack=slack)
    check(model, dtype, schedule_mixed({**reqs, "farx": ids, "nearx": ids[:70]}, max_live=3, seed=5), tmp_path / "mixed",
          slack=slack, max_live=3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_sizes_of_real_models(dtype, tmp_path):
    """Cache rows of 256 and of 128, two maps of heads of 128 and of 64, a width whose few rows are
    normed over a cluster, pages of 64: the kernels that real layer sizes reach (tcgen05 prefill,
    mma.sync with wide heads, decode by whole pages, products cut along K), prompts longer than two
    key tiles of any kernel."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model
    raw = {"architecture": "Babadra", "vocab": 1000, "width": 1024, "max_positions": 512, "norm": {"eps": 1e-6},
           "embedding": {"scale": 4.0}, "logit_softcap": 25.0, "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
        {"type": "latent_attention", "mlp": _dense(512, 1.5),
         "mixer": _latent(4, 128, 64, 128, 256, 192, 0.08, 1e4, {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0})},
        {"type": "attention", "mlp": _moe(256, 8, 2, 1.5),
         "mixer": _attention(4, 1, 128, 128, 0.09, 0.5, softcap=20.0, rot={"base": 1e6, "dims": 64})},
        {"type": "latent_attention", "mlp": _moe(256, 8, 2, 1.0), "mixer": _latent(4, 128, 32, 128, 256, 96, 0.08, 1e4)},
        {"type": "attention", "mlp": None,
         "mixer": _attention(8, 2, 64, 64, 0.125, 0.25, softcap=50.0, rot={"base": 1e4, "dims": 64})},
    ]}
    folder = decisive(write_random_model(config_from_dict(raw), str(tmp_path / "model"), seed=5), 5)
    cfg, weights = plain.load_folder(folder)
    reqs = {"a": random_ids(1000, 420, seed=1), "b": random_ids(1000, 130, seed=2)}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    model = {"name": "real", "folder": folder, "cfg": cfg, "requests": reqs, "ref": ref}
    check(model, dtype, schedule_tail_decode(reqs, 40), tmp_path / "tail", page=64)
    check(model, dtype, schedule_mixed(reqs, max_live=2, seed=1, chunk_sizes=(200, 2, 129, 64, 1)), tmp_path / "mixed", max_live=2)


# ----------------------------------------------------------------------------- the entry point
def test_greedy_generation_through_the_scheduler(tmp_path):
    """Five prompts of unequal length through LLM.generate with three slots and at most 48 tokens a
    step (prompts in portions beside decoding requests, slots and pages used again)."""
    from tinyserve_b200 import LLM, SamplingParams
    folder = make_babadra_dir(tmp_path, "P", seed=44)
    cfg, weights = plain.load_folder(folder)
    prompts = [random_ids(cfg["vocab"], n, seed=500 + n) for n in (3, 60, 17, 1, 90)]
    params = SamplingParams(temperature=0.0, max_tokens=12, repetition_penalty=1.0, ignore_eos=True)
    llm = LLM(folder, dtype="float32", max_model_len=128, block_size=16, max_num_seqs=3, max_num_batched_tokens=48,
              num_blocks=20, use_cuda_graphs=False)
    outs = llm.generate(prompts, params)
    for prompt, out in zip(prompts, outs):
        want, gaps = plain.greedy(cfg, weights, prompt, 12)
        assert out.finished and len(out.token_ids) == 12
        for j, (a, b, gap) in enumerate(zip(out.token_ids, want, gaps)):
            if gap < 1e-3:
                break                        # a near tie: either side is a right answer, the rest differs
            assert a == b, (len(prompt), j)
    outs16 = LLM(folder, dtype="bfloat16", max_model_len=128, block_size=16, max_num_seqs=3,
                 max_num_batched_tokens=48, num_blocks=20, use_cuda_graphs=True).generate(prompts, params)
    for prompt, out in zip(prompts, outs16):
        ids = list(prompt)
        for tok in out.token_ids:
            row = plain.logits(cfg, weights, ids)[-1]
            assert row[tok] >= row.max() - 0.05 * row.abs().max()
            ids.append(tok)


def test_programs_replay_and_generate(tmp_path):
    """bin/trace_run and ``python -m tinyserve_b200 generate`` as programs on a Babadra folder: the
    architecture is chosen by config.json; stdin to files, 'done' lines, exit code 0; greedy tokens."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = make_babadra_dir(tmp_path / "m", "Q", seed=2)
    cfg, weights = plain.load_folder(folder)
    reqs = {"p": random_ids(cfg["vocab"], 45, seed=1), "q": random_ids(cfg["vocab"], 30, seed=2)}
    steps = schedule_mixed(reqs, max_live=2, seed=0)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(max_live_tokens(steps))],
        input="\n".join(lines_of(steps)) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        outputs[s["step"]] = torch.from_numpy(np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(wanted, cfg["vocab"]))
    got = collect_logits(steps, outputs, cfg["vocab"])
    for rid, ids in reqs.items():
        ref = plain.logits(cfg, weights, ids)
        assert (got[rid].double() - ref).abs().max().item() < TOLERANCE["float32"] * ref.abs().max().item()
    prompt = reqs["q"][:9]
    proc = subprocess.run(
        [sys.executable, "-m", "tinyserve_b200", "generate", "--model", folder, "--dtype", "float32", "--prompt-ids",
         ",".join(map(str, prompt)), "--max-tokens", "5", "--repetition-penalty", "1.0", "--ignore-eos", "--max-model-len", "64",
         "--max-num-seqs", "2", "--max-num-batched-tokens", "32", "--num-blocks", "16", "--block-size", "16"],
        capture_output=True, text=True, timeout=600, cwd=root)
    assert proc.returncode == 0, proc.stderr[-2000:]
    tokens = [int(t) for t in proc.stdout.strip().split("\n")[-1].split()]
    want, gaps = plain.greedy(cfg, weights, prompt, 5)
    for a, b, gap in zip(tokens, want, gaps):
        if gap < 1e-3:
            break
        assert a == b, (tokens, want)
    assert len(tokens) == 5


def test_measured_differences_are_reported():
    print({k: (f"{v[0]:.2e}", f"{v[1]:.2e}") for k, v in sorted(MEASURED.items())})
