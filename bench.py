#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on Qwen3-8B shapes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A step is one decode step of the whole batch.  Prints ONE JSON line:
  value     decoded tokens per second over K steps, timed on the device with CUDA events;
            each step uploads the batch, runs the model and samples greedily on the device;
            tokens are fed back on the device and the host packs one step ahead
  e2e       the same through the Python entry point (LLM.add_request / LLM.step): host
            token ids in, sampled tokens out, scheduler and cache manager included
  prefill   one 2,048-token prompt in one step
  roofline  bytes the decode step must read (every weight once + the live cache) / time
  points    decode tokens per second at batch 1 and 64
The engine runs on one GPU; with --gpus > 1 it says so and exits with 2.

    python bench.py --arch dudatar [--sizes 2048,4096]

measures another design beside Qwen3 at equal size instead (random weights, same width, block
runs, feed-forward width, heads and vocabulary): prefill of one 2,048-token prompt, decode at
batch 8, and the design's own kernels beside the like kernels of Qwen3, each against its roofline.

    python bench.py --arch delilorn [--sizes 2048,4096]

does the same for Delilorn (latent attention, lightning attention, attention over a window beside
kept first tokens, a mixture of experts whose active weights equal Qwen3's feed-forward).

    python bench.py --arch babadra [--sizes 2048,4096]

measures Babadra (latent attention, attention with two capped score maps per head, bounded gated
feed-forwards, dense and as experts, a repeated group of layers) beside Delilorn, the closest design.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6,
                tie_word_embeddings=False, max_position_embeddings=40960)
CONTEXT = 4096
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
# the other two configurations of the baseline: a burst of short requests on a small model (it
# measures the host path and mixed batches) and a large model at long context
QWEN3_0P6B = dict(QWEN3_8B, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16,
                  num_key_value_heads=8, intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
                 num_key_value_heads=8, intermediate_size=25600)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  It runs from ``start()`` on (the
    tool needs a moment to come up, and the timed region may be shorter than that); ``window()``
    marks the timed region, and ``stop()`` reports the samples that fall into it (or, if the
    region was shorter than a sampling period, the samples nearest to it)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.t0, self.t1 = [], None, None, None

    def start(self):
        if self.proc is not None:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.monotonic(), parts))

    def window(self, begin: bool):
        if begin:
            self.t0 = time.monotonic()
        else:
            self.t1 = time.monotonic()

    def stop(self):
        if self.proc is not None:
            time.sleep(0.12)                      # one more sample after the region
            self.proc.terminate()
        t0, t1 = self.t0 or 0.0, self.t1 or float("inf")
        inside = [s for t, s in self.samples if t0 <= t <= t1]
        if not inside and self.samples:
            mid = (t0 + min(t1, t0 + 3600)) / 2
            inside = [s for _, s in sorted(self.samples, key=lambda ts: abs(ts[0] - mid))[:3]]
        mhz = [int(s[0]) for s in inside if s[0].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in inside)]
        mx = [int(s[1]) for s in inside if s[1].isdigit()]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(inside)}


def decode_bytes(cfg, layers, batch, ctx):
    h, H, Hkv, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                          cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = ((H + 2 * Hkv) * D * h + h * H * D + 2 * I * h + h * I + 2 * h + 2 * D) * 2
    weights = layers * per_layer + V * h * 2 + h * 2
    kv = batch * ctx * layers * 2 * Hkv * D * 2
    return weights + kv


def prefill_flops(cfg, layers, T):
    h, H, Hkv, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                          cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    linear = 2 * T * layers * ((H + 2 * Hkv) * D * h + h * H * D + 3 * I * h) + 2 * V * h
    attention = layers * 4 * H * D * T * (T + 1) // 2
    return linear + attention


def run_decode(llm, batch, steps, warmup, seed, clock=None, prompt_len=PROMPT_LEN):
    """Prefill `batch` prompts of `prompt_len` tokens, then time `steps` decode steps."""
    import torch
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.kernels import ops
    runner, vocab = llm.runner, llm.runner.model.vocab_size
    gen = torch.Generator().manual_seed(seed)
    rids = [f"bench{batch}_{i}" for i in range(batch)]
    temps = torch.zeros(batch, dtype=torch.float32, device=runner.device)
    streams = torch.zeros(batch, dtype=torch.int64, device=runner.device)
    counters = torch.zeros(batch, dtype=torch.int32, device=runner.device)
    host = torch.empty(batch, dtype=torch.int32).pin_memory()
    last = []
    for rid in rids:
        runner.manager.begin(rid)
    budget = runner.cfg.max_num_batched_tokens
    if prompt_len <= budget:
        per_step = max(1, budget // prompt_len)
        for i in range(0, batch, per_step):
            group = rids[i:i + per_step]
            prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in group]
            logits = runner.step([StepEntry(r, p, [prompt_len - 1]) for r, p in zip(group, prompts)])
            last += logits.argmax(-1).tolist()
    else:
        for rid in rids:                      # a long prompt goes in portions of the budget
            ids = torch.randint(0, vocab, (prompt_len,), generator=gen).tolist()
            for at in range(0, prompt_len, budget):
                part = ids[at:at + budget]
                logits = runner.step([StepEntry(rid, part, [len(part) - 1] if at + budget >= prompt_len else [])])
            last += logits.argmax(-1).tolist()

    # Tokens stay on the device: the sampler leaves each request's token at its state slot and the
    # next step's embedding lookup reads it there.  The host packs step n+1 while step n runs and
    # never lags more than one step (it waits for the event of step n-1 before it reuses a buffer).
    from tinyserve_b200.engine.runner import PENDING
    slots = torch.tensor([runner.manager.slot(r) for r in rids], dtype=torch.int64, device=runner.device)
    runner.slot_tokens[slots] = torch.tensor(last, dtype=torch.int32, device=runner.device)
    entries = [StepEntry(r, [PENDING], [0]) for r in rids]
    events = []

    def one_step():
        if len(events) >= 2:
            events[-2].synchronize()
        logits = runner.step(entries)
        out = ops.sample(logits, temps, streams, counters, 0, slot_tokens=runner.slot_tokens,
                         slots=runner.state_slots_on_device(batch))
        host.copy_(out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        events.append(ev)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    if clock:
        clock.window(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count()
    start.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    if clock:
        clock.window(False)
    clocks = clock.stop() if clock else None
    ms = start.elapsed_time(end) / steps
    ctx = prompt_len + warmup + steps / 2
    for rid in rids:
        runner.manager.free(rid)
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "ctx": ctx,
            "launches": ops.launch_count() - launches0, "clocks": clocks}


def run_e2e(llm, batch, steps, warmup, seed):
    """The same decode through LLM.add_request / LLM.step, wall clock, host ids in and out."""
    import torch
    from tinyserve_b200 import SamplingParams
    vocab = llm.runner.model.vocab_size
    gen = torch.Generator().manual_seed(seed + 1)
    params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, repetition_penalty=1.0,
                            ignore_eos=True)
    for i in range(batch):
        llm.add_request(torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist(), params,
                        request_id=f"e2e{i}")
    while any(r.num_computed_tokens < r.prompt_len for r in llm.requests.values()) or llm.scheduler.waiting:
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(llm.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for rid in list(llm.requests):
        llm.abort(rid)
    h2d = llm.runner.last_upload_bytes
    return {"value": produced / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": batch * 4}


def run_prefill(llm, seed, repeats=3):
    import torch
    from tinyserve_b200.engine.batch import StepEntry
    runner, vocab = llm.runner, llm.runner.model.vocab_size
    gen = torch.Generator().manual_seed(seed + 2)
    times = []
    for i in range(repeats + 1):
        rid = f"prefill{i}"
        runner.manager.begin(rid)
        ids = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(rid, ids, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
        runner.manager.free(rid)
    return min(times[1:])


def _release(llm):
    import gc
    import torch
    del llm
    gc.collect()
    torch.cuda.empty_cache()


def run_burst_0p6b(seed, block_size=16):
    """Qwen3-0.6B shapes: 256 requests arrive at once, prompts of 1 to 2,048 tokens, 128 greedy
    tokens each, 2,048 tokens a step, through LLM.generate.  Returns tokens per second (prompt +
    generated, and generated alone) over the whole run, wall clock."""
    import torch
    from tinyserve_b200 import LLM, Qwen3Config, SamplingParams
    llm = LLM(model_config=Qwen3Config.from_dict(QWEN3_0P6B), random_weights=True, dtype="bfloat16",
              max_model_len=4096, block_size=block_size, max_num_seqs=256, max_num_batched_tokens=2048, seed=seed)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, 2049, (256,), generator=g).tolist()
    prompts = [torch.randint(0, QWEN3_0P6B["vocab_size"], (n,), generator=g).tolist() for n in lens]
    params = SamplingParams(temperature=0.0, max_tokens=128, repetition_penalty=1.0, ignore_eos=True)
    llm.generate(prompts[:8], SamplingParams(temperature=0.0, max_tokens=4, repetition_penalty=1.0, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    generated = sum(len(o.token_ids) for o in outs)
    steps = llm.num_steps
    _release(llm)
    return {"burst_0p6b_total_tok_s": round((generated + sum(lens)) / dt, 1),
            "burst_0p6b_gen_tok_s": round(generated / dt, 1), "burst_0p6b_seconds": round(dt, 3),
            "burst_0p6b_steps": steps}


def run_large_32b(seed, block_size=16):
    """Qwen3-32B shapes at 8,192 context: 16 requests with prompts of 4,096 tokens and 256 greedy
    tokens each.  Returns prompt tokens per second while the prompts run and decoded tokens per
    second afterwards (CUDA events around the two phases, through LLM.step)."""
    import torch
    from tinyserve_b200 import LLM, Qwen3Config, SamplingParams
    llm = LLM(model_config=Qwen3Config.from_dict(QWEN3_32B), random_weights=True, dtype="bfloat16",
              max_model_len=8192, block_size=block_size, max_num_seqs=16, max_num_batched_tokens=4096,
              gpu_memory_utilization=0.9, seed=seed)        # the rest of the memory goes to the cache
    g = torch.Generator().manual_seed(seed)
    params = SamplingParams(temperature=0.0, max_tokens=256, repetition_penalty=1.0, ignore_eos=True)
    for i in range(16):
        llm.add_request(torch.randint(0, QWEN3_32B["vocab_size"], (4096,), generator=g).tolist(), params, request_id=f"big{i}")
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    torch.cuda.synchronize()
    marks[0].record()
    while any(r.num_computed_tokens < r.prompt_len for r in llm.requests.values()) or llm.scheduler.waiting:
        llm.step()
    marks[1].record()
    decoded = 0
    while llm.has_work():
        decoded += len(llm.step())
    marks[2].record()
    torch.cuda.synchronize()
    prefill_ms, decode_ms = marks[0].elapsed_time(marks[1]), marks[1].elapsed_time(marks[2])
    _release(llm)
    return {"large_32b_prefill_tok_s": round(16 * 4096 * 1000.0 / prefill_ms, 1),
            "large_32b_decode_b16_tok_s": round(decoded * 1000.0 / decode_ms, 1)}


def run_long_context(seed, steps, warmup, block_size=16):
    """Qwen3-8B shapes, batch 8, decode at 4,096 and at 16,384 tokens of context."""
    import torch
    from tinyserve_b200 import LLM, Qwen3Config
    from tinyserve_b200.engine.batch import StepEntry
    out = {}
    llm = LLM(model_config=Qwen3Config.from_dict(QWEN3_8B), random_weights=True, dtype="bfloat16",
              max_model_len=16384 + 256, block_size=block_size, max_num_seqs=8, max_num_batched_tokens=4096,
              num_blocks=8 * (16384 + 256) // block_size + 16, use_cuda_graphs=False, seed=seed)
    llm.runner.capture_decode_graphs([8])
    for name, ctx in (("decode_b8_ctx4k_tok_s", 4096), ("decode_b8_ctx16k_tok_s", 16384)):
        r = run_decode(llm, 8, steps, warmup, seed + ctx, prompt_len=ctx - warmup - steps)
        out[name] = round(r["tok_s"], 1)
    _release(llm)
    return out


# ----------------------------------------------------------------------------- another design beside Qwen3
def dudatar_shapes(width):
    """A Dudatar of real layer sizes at ``width``: a gated layer, two layers of attention beside
    retention (this pair runs twice), a gated layer: six block runs; and the Qwen3 of the same
    width, block runs, feed-forward width, attention heads and vocabulary."""
    heads, ff, vocab = width // 128, width * 11 // 4, 32768
    rot = lambda dims: {"dims": dims, "base": 1e6}
    gla = {"type": "gla", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": heads // 2, "dim": 128, "vdim": 256, "tau": 8.0, "rank": 32}}
    par = {"type": "parallel", "mlp": {"kind": "dense", "ff": ff}, "mixer": {
        "left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": rot(64)},
        "right": {"heads": heads // 2, "dim": 128, "vdim": 256, "rot": rot(128),
                  "decay": [1.0 - 2.0 ** -(5 + 5 * i / max(1, heads // 2 - 1)) for i in range(heads // 2)]}}}
    dudatar = {"architecture": "Dudatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
               "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [gla, par, par, gla]}
    qwen3 = dict(QWEN3_8B, hidden_size=width, num_hidden_layers=6, num_attention_heads=heads,
                 num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=ff, vocab_size=vocab)
    return dudatar, qwen3


def delilorn_shapes(width):
    """A Delilorn of real layer sizes at ``width``: latent attention, lightning, latent attention on
    the first layer's cache, attention over a window of 1,024 beside 4 kept tokens, lightning,
    window attention: six blocks, each with 8 experts of which a token takes 2, sized so that a
    token's active expert weights equal the feed-forward of the Qwen3 beside it (same width, block
    count, attention heads and vocabulary)."""
    heads, ff, vocab = width // 128, width * 11 // 4, 32768
    ffe = (3 * ff // 4 + 63) // 64 * 64             # 2 experts x 2 matrices = 3 matrices of the gated feed-forward
    moe = {"kind": "moe", "expert": {"ff": ffe}, "router": {"experts": 8, "top": 2}}
    rank, rot = (96, 32) if width < 4096 else (192, 64)          # cache rows of 128 and of 256
    latent = {"heads": heads, "dim": 128, "rot_dim": rot, "vdim": 128, "q_rank": width // 2, "kv_rank": rank,
              "scale": (128 + rot) ** -0.5, "rot": {"base": 1e4, "dims": rot}}
    lightning = {"heads": heads // 2, "dim": 128, "vdim": 256,
                 "decay": [1.0 - 2.0 ** -(5 + 5 * i / max(1, heads // 2 - 1)) for i in range(heads // 2)]}
    window = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
              "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
              "mask": {"size": 1024, "keep_first": 4}}
    layer = lambda kind, mixer: {"type": kind, "mixer": mixer, "mlp": moe}
    delilorn = {"architecture": "Delilorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [
        layer("latent_attention", latent), layer("lightning", lightning), layer("latent_attention", dict(latent, kv_from=0)),
        layer("attention", window), layer("lightning", lightning), layer("attention", window)]}
    qwen3 = dict(QWEN3_8B, hidden_size=width, num_hidden_layers=6, num_attention_heads=heads,
                 num_key_value_heads=max(1, heads // 4), head_dim=128, intermediate_size=ff, vocab_size=vocab)
    return delilorn, qwen3


def tarivik_shapes(width):
    """A Tarivik of real layer sizes at ``width``: attention in chunks of 1,024 beside a selective state
    space, an HGRN2 layer, an mLSTM layer, and the three again: six blocks, each with 8 gated experts in
    4 groups of which a token takes 2 from the best 2 groups, sized so that a token's active expert weights
    equal those of the Delilorn beside it (same width, block count, attention heads, vocabulary)."""
    delilorn, _ = delilorn_shapes(width)
    heads, vocab = width // 128, 32768
    ffe = (delilorn["layers"][0]["mlp"]["expert"]["ff"] * 2 // 3 + 63) // 64 * 64      # three matrices where Delilorn has two
    moe = {"kind": "moe", "expert": {"ff": ffe}, "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}}
    parallel = {"left": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                         "mask": {"size": 1024}},
                "right": {"heads": width // 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1},
                "left_scale": 1.0, "right_scale": 1.0}
    hgrn2 = {"heads": heads // 2, "dim": 128, "vdim": 256}
    mlstm = {"heads": heads, "dim": 128, "vdim": 128, "gate_cap": 15.0}
    layer = lambda kind, mixer: {"type": kind, "mixer": mixer, "mlp": moe}
    order = [layer("parallel", parallel), layer("hgrn2", hgrn2), layer("mlstm", mlstm)]
    tarivik = {"architecture": "Tarivik", "vocab": vocab, "width": width, "max_positions": CONTEXT, "norm": {"eps": 1e-6, "groups": 2},
               "canon": {"taps": 4}, "layers": order + order}
    return tarivik, delilorn


def babadra_shapes(width):
    """A Babadra of real layer sizes at ``width``: latent attention with a dense feed-forward, attention
    with two score maps per head and experts, twice; the two middle layers run twice, which makes six
    block runs.  The attention kernels see as many query heads of 128 on as many key/value heads as the
    Delilorn beside it has (half as many heads, two maps each); 8 gated experts of which a token takes
    2, sized so that a token's active expert weights equal the dense feed-forward's."""
    delilorn, _ = delilorn_shapes(width)
    heads, ff, vocab = width // 128, width * 11 // 4, 32768
    rank, rot = (96, 32) if width < 4096 else (192, 64)          # cache rows of 128 and of 256
    latent = {"heads": heads, "dim": 128, "rot_dim": rot, "vdim": 128, "q_rank": width // 2, "kv_rank": rank,
              "scale": (128 + rot) ** -0.5,
              "rot": {"base": 5e5, "dims": rot, "scaling": {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}
    two_maps = {"heads": heads // 2, "kv_heads": max(1, heads // 8), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "diff": 0.5,
                "softcap": 50.0, "rot": {"base": 2.5e5, "dims": 64}}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": (ff // 2 + 63) // 64 * 64, "limit": 7.0}, "router": {"experts": 8, "top": 2}}
    order = [{"type": "latent_attention", "mixer": latent, "mlp": dense}, {"type": "attention", "mixer": two_maps, "mlp": moe}]
    babadra = {"architecture": "Babadra", "vocab": vocab, "width": width, "max_positions": CONTEXT, "norm": {"eps": 1e-6},
               "embedding": {"scale": float(width) ** 0.5}, "logit_softcap": 30.0, "loop": {"start": 1, "stop": 3, "times": 2},
               "layers": order + order}
    return babadra, delilorn


def _time_us(fn, iters=20):
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / iters


def _time_graph_us(fn, iters=20):
    """Device time of ``fn`` per call, its launches replayed from a CUDA graph as the engine replays a decode
    step: the host's time between launches is not in it."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    return _time_us(graph.replay, iters=5) / iters


def kernel_table(width, peaks):
    """The design's own kernels beside the like kernels of Qwen3 at this width, one launch each
    (operands larger than L2 where the size allows: 2,048 tokens of prefill; at decode the state
    and the cache of 8 requests), time over roofline time.  Roofline of the matrix-state scan: the
    slower of its bytes over the copy bandwidth and its 32-bit multiply-adds over the FMA rate of
    the CUDA cores (SMs x 128 lanes x 2 x the maximum clock): its arithmetic is 32-bit by design."""
    import torch
    from types import SimpleNamespace
    from tinyserve_b200.kernels import ops
    dev, bf = "cuda:0", torch.bfloat16
    heads = width // 128
    H, n, nv = heads // 2, 128, 256
    fma_tflops = ops.num_sms() * 128 * 2 * 1.965e9 / 1e12
    out = {}
    for name, lengths, starts in (("prefill_2048", [2048], [0]), ("decode_b8", [1] * 8, [512] * 8)):
        T, B = sum(lengths), len(lengths)
        cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=dev)
        ctx = SimpleNamespace(num_requests=B, cu_q=cu, max_q_len=max(lengths),
                              state_slots=torch.arange(B, dtype=torch.int32, device=dev),
                              fresh=torch.zeros(B, dtype=torch.int32, device=dev),
                              positions=torch.cat([torch.arange(s, s + m) for s, m in zip(starts, lengths)]).int().to(dev))
        proj = torch.randn(T, 2 * H * n + 2 * H * nv, device=dev).to(bf)
        q, k, v, g = proj[:, :H * n], proj[:, H * n:2 * H * n], proj[:, 2 * H * n:2 * H * n + H * nv], proj[:, 2 * H * n + H * nv:]
        z = torch.randn(T, H * n, device=dev) + 3
        state = torch.zeros(B, H, n, nv, device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        w = torch.ones(nv, device=dev, dtype=bf)
        flops = 4.0 * T * H * n * nv
        nbytes = T * (2 * H * n + 3 * H * nv) * 2 + 2 * B * H * n * nv * 4
        for kind, kw in (("retention", dict(decay=decay, k_scale=n ** -0.5)),
                         ("gla", dict(decay_logits=z, tau=8.0, q_scale=n ** -0.5, norm_weight=w))):
            us = _time_us(lambda: ops.linear_attention(q, k, v, g, state, ctx, H, n, nv, bf, eps=1e-5, **kw))
            extra = T * H * n * 4 if kind == "gla" else 0
            roof = max((nbytes + extra) / (peaks["hbm_gbs"] * 1e3), flops / (fma_tflops * 1e6))
            out[f"{kind}_scan_{name}"] = {"us": round(us, 1), "roofline_us": round(roof, 1), "frac": round(roof / us, 3)}
        # the attention kernel both designs run, at the left mixer's (= Qwen3's) sizes
        Ha, G, D, page = heads, max(1, heads // 4), 128, 64
        kv_len = starts[0] + lengths[0]
        pages_per = -(-kv_len // page)
        kc = torch.randn(B * pages_per + 1, G, page, D, device=dev).to(bf)
        vc = torch.randn_like(kc)
        table = (torch.arange(B * pages_per, dtype=torch.int32, device=dev) + 1).view(B, pages_per)
        from tinyserve_b200.engine.batch import GroupView, StepContext
        sc = StepContext()
        sc.num_tokens, sc.num_requests, sc.max_q_len, sc.max_kv_len = T, B, max(lengths), kv_len
        sc.cu_q, sc.kv_lens = cu, torch.full((B,), kv_len, dtype=torch.int32, device=dev)
        sc.host = {"cu_q": cu.tolist(), "kv_lens": [kv_len] * B}
        view = GroupView(page, pages_per, None, table, kc.shape[0])
        qa = torch.randn(T, Ha, D, device=dev).to(bf)
        us = _time_us(lambda: ops.paged_attention(qa, kc, vc, view, sc, D ** -0.5))
        if T > B:
            roof = 4.0 * Ha * D * T * (T + 1) / 2 / (peaks["bf16_tflops"] * 1e6)
        else:
            roof = B * kv_len * 2 * G * D * 2 / (peaks["hbm_gbs"] * 1e3)
        out[f"attention_{name}"] = {"us": round(us, 1), "roofline_us": round(roof, 1), "frac": round(roof / us, 3)}
        # the norms: layer norm with two addends beside residual add + RMSNorm
        res = torch.randn(T, width, device=dev)
        a1, a2 = torch.randn(T, width, device=dev).to(bf), torch.randn(T, width, device=dev).to(bf)
        wn = torch.ones(width, device=dev, dtype=bf)
        us_ln = _time_us(lambda: ops.add_layernorm(ops.PairSum(a1, a2), res, wn, 1e-5, bf))
        us_rms = _time_us(lambda: ops.add_rmsnorm(a1, res, wn, 1e-5, bf))
        for key, us, addends in (("add_layernorm", us_ln, 2), ("add_rmsnorm", us_rms, 1)):
            roof = T * width * (8 + 2 * addends + 2) / (peaks["hbm_gbs"] * 1e3)
            out[f"{key}_{name}"] = {"us": round(us, 1), "roofline_us": round(roof, 2), "frac": round(roof / us, 3)}
    return out


def delilorn_kernel_table(width, peaks):
    """Delilorn's kernels beside the like kernels of Qwen3 at this width, one launch each, time over
    roofline time: attention over one latent head with a sink (prefill FLOPs over the library's GEMM
    rate; decode bytes of the cache rows, read once for keys and values alike), attention over a window
    beside kept tokens (the FLOPs and bytes of the visible keys only), the lightning form of the
    matrix-state scan, the experts (the FLOPs of the chosen experts; at decode the bytes of all experts'
    weights), and the norm that norms a sub-layer's output, adds it and norms the sum."""
    import torch
    from types import SimpleNamespace
    from tinyserve_b200.engine.batch import GroupView, StepContext
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts.moe import MixtureOfExperts
    dev, bf = "cuda:0", torch.bfloat16
    raw, _ = delilorn_shapes(width)
    lat, lig, win = (raw["layers"][i]["mixer"] for i in (0, 1, 3))
    moe = raw["layers"][0]["mlp"]
    heads = lat["heads"]
    fma_tflops = ops.num_sms() * 128 * 2 * 1.965e9 / 1e12
    out = {}

    def frac(key, us, roof):
        out[key] = {"us": round(us, 1), "roofline_us": round(roof, 2), "frac": round(roof / us, 3)}

    for name, lengths, starts in (("prefill_2048", [2048], [0]), ("decode_b8", [1] * 8, [2048] * 8)):
        T, B = sum(lengths), len(lengths)
        kv_len, page = starts[0] + lengths[0], 64
        pages_per = -(-kv_len // page)
        cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=dev)
        table = (torch.arange(B * pages_per, dtype=torch.int32, device=dev) + 1).view(B, pages_per)

        def context():
            sc = StepContext()
            sc.num_tokens, sc.num_requests, sc.max_q_len, sc.max_kv_len = T, B, max(lengths), kv_len
            sc.cu_q, sc.kv_lens = cu, torch.full((B,), kv_len, dtype=torch.int32, device=dev)
            sc.host = {"cu_q": cu.tolist(), "kv_lens": [kv_len] * B}
            return sc

        def attention(H, G, D, window=0, keep=0, sinks=None, shared=False):
            kc = torch.randn(B * pages_per + 1, G, page, D, device=dev).to(bf)
            vc = kc if shared else torch.randn_like(kc)
            view = GroupView(page, pages_per, None, table, kc.shape[0])
            q = torch.randn(T, H, D, device=dev).to(bf)
            sc = context()
            return _time_us(lambda: ops.paged_attention(q, kc, vc, view, sc, D ** -0.5, window, keep_first=keep, sinks=sinks))

        def visible(window, keep):
            pos = torch.arange(kv_len - lengths[0], kv_len)
            seen = pos + 1 if not window else torch.minimum(pos + 1, torch.full_like(pos, window)) + torch.clamp(
                torch.minimum(pos + 1 - window, torch.full_like(pos, keep)), min=0)
            return float(seen.sum())

        def attention_roof(H, G, D, window=0, keep=0, tensors=2):
            if T > B:
                return 4.0 * H * D * visible(window, keep) / (peaks["bf16_tflops"] * 1e6)
            return B * visible(window, keep) * tensors * G * D * 2 / (peaks["hbm_gbs"] * 1e3)

        D = -(-(lat["kv_rank"] + lat["rot_dim"]) // 16) * 16
        sinks = torch.randn(heads, device=dev)
        frac(f"latent_attention_{name}", attention(heads, 1, D, sinks=sinks, shared=True), attention_roof(heads, 1, D, tensors=1))
        G = win["kv_heads"]
        frac(f"window_attention_{name}", attention(heads, G, 128, win["mask"]["size"], win["mask"]["keep_first"]),
             attention_roof(heads, G, 128, win["mask"]["size"], win["mask"]["keep_first"]))
        frac(f"qwen3_attention_{name}", attention(heads, G, 128), attention_roof(heads, G, 128))
        # the scan: lightning form beside the retention form (the same kernel)
        H, n, nv = lig["heads"], lig["dim"], lig["vdim"]
        ctx = SimpleNamespace(num_requests=B, cu_q=cu, max_q_len=max(lengths),
                              state_slots=torch.arange(B, dtype=torch.int32, device=dev),
                              fresh=torch.zeros(B, dtype=torch.int32, device=dev),
                              positions=torch.cat([torch.arange(s, s + m) for s, m in zip(starts, lengths)]).int().to(dev))
        proj = torch.randn(T, 2 * H * n + 2 * H * nv, device=dev).to(bf)
        q, k, v, g = proj[:, :H * n], proj[:, H * n:2 * H * n], proj[:, 2 * H * n:2 * H * n + H * nv], proj[:, 2 * H * n + H * nv:]
        state = torch.zeros(B, H, n, nv, device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        wj = torch.ones(H * nv, device=dev)
        roof = max((T * (2 * H * n + 3 * H * nv) * 2 + 2 * B * H * n * nv * 4) / (peaks["hbm_gbs"] * 1e3),
                   4.0 * T * H * n * nv / (fma_tflops * 1e6))
        frac(f"lightning_scan_{name}", _time_us(lambda: ops.linear_attention(
            q, k, v, g, state, ctx, H, n, nv, bf, decay=decay, norm_weight=wj, eps=1e-6, input_activation="silu",
            gate_activation="sigmoid", joint_norm=True)), roof)
        frac(f"retention_scan_{name}", _time_us(lambda: ops.linear_attention(
            q, k, v, g, state, ctx, H, n, nv, bf, decay=decay, k_scale=n ** -0.5, eps=1e-6)), roof)
        # the experts beside the gated feed-forward of equal active weights
        E, top, ffe, ff = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"], width * 11 // 4
        part = MixtureOfExperts(width, ffe, E, top)
        part.bind({"router.weight": (torch.randn(E, width, device=dev) * 0.1).to(bf),
                   "up.weight": (torch.randn(E * ffe, width, device=dev) * 0.02).to(bf),
                   "down.weight": (torch.randn(E * width, ffe, device=dev) * 0.02).to(bf)})
        h = torch.randn(T, width, device=dev).to(bf)
        gate_up = (torch.randn(2 * ff, width, device=dev) * 0.02).to(bf)
        down = (torch.randn(width, ff, device=dev) * 0.02).to(bf)
        block = ops.GATED_BLOCK if ff % ops.GATED_BLOCK == 0 else 0
        us_moe = _time_us(lambda: ops.materialize(part.forward(h, None)))
        us_mlp = _time_us(lambda: ops.materialize(ops.linear(ops.gated_linear(h, gate_up, "silu", block), down)))
        if T > B:
            frac(f"experts_{name}", us_moe, 4.0 * T * top * width * ffe / (peaks["bf16_tflops"] * 1e6))
            frac(f"qwen3_feed_forward_{name}", us_mlp, 6.0 * T * width * ff / (peaks["bf16_tflops"] * 1e6))
        else:
            frac(f"experts_{name}", us_moe, 2.0 * E * width * ffe * 2 / (peaks["hbm_gbs"] * 1e3))
            frac(f"qwen3_feed_forward_{name}", us_mlp, 3.0 * width * ff * 2 / (peaks["hbm_gbs"] * 1e3))
        # the norms
        res = torch.randn(T, width, device=dev)
        y = torch.randn(T, width, device=dev).to(bf)
        wn = torch.ones(width, device=dev)
        frac(f"normed_add_rmsnorm_{name}", _time_us(lambda: ops.normed_add_rmsnorm(ops.NormedAddend(y, wn, 1e-6), res, wn, 1e-6, bf)),
             T * width * (8 + 2 + 2) / (peaks["hbm_gbs"] * 1e3))
        frac(f"add_rmsnorm_{name}", _time_us(lambda: ops.add_rmsnorm(y, res, wn, 1e-6, bf)),
             T * width * (8 + 2 + 2) / (peaks["hbm_gbs"] * 1e3))
    return out


def tarivik_kernel_table(width, peaks):
    """Tarivik's kernels beside the like kernels of Delilorn at this width, time over roofline time:
    attention in chunks with a distance bias and a sink beside attention over a window with kept tokens (the
    FLOPs and bytes of the visible keys only); the HGRN2, mLSTM (gates, scan, finish) and state-space
    (convolution, step sizes, scan, finish) forms of the matrix-state scan beside the lightning form; the
    gated experts beside Delilorn's; the output norm added to the stream plus the next input convolution
    beside the norm that norms a sub-layer's output, adds it and norms the sum."""
    import torch
    from types import SimpleNamespace
    from tinyserve_b200.engine.batch import GroupView, StepContext
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts.moe import MixtureOfExperts
    dev, bf = "cuda:0", torch.bfloat16
    raw, other = tarivik_shapes(width)
    par, hg, ml = (raw["layers"][i]["mixer"] for i in (0, 1, 2))
    left, right = par["left"], par["right"]
    lig, win = other["layers"][1]["mixer"], other["layers"][3]["mixer"]
    fma_tflops = ops.num_sms() * 128 * 2 * 1.965e9 / 1e12
    out = {}

    def frac(key, us, roof):
        out[key] = {"us": round(us, 1), "roofline_us": round(roof, 2), "frac": round(roof / us, 3)}

    for name, lengths, starts in (("prefill_2048", [2048], [0]), ("decode_b8", [1] * 8, [2047] * 8)):
        T, B = sum(lengths), len(lengths)
        timer = _time_us if T > B else _time_graph_us          # a decode step's launches are replayed from a graph
        kv_len, page = starts[0] + lengths[0], 64
        pages_per = -(-kv_len // page)
        cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=dev)
        table = (torch.arange(B * pages_per, dtype=torch.int32, device=dev) + 1).view(B, pages_per)
        pos = torch.arange(kv_len - lengths[0], kv_len)

        def attention(H, G, D, seen, **kw):
            kc = torch.randn(B * pages_per + 1, G, page, D, device=dev).to(bf)
            vc = torch.randn_like(kc)
            view = GroupView(page, pages_per, None, table, kc.shape[0])
            q = torch.randn(T, H, D, device=dev).to(bf)
            sc = StepContext()
            sc.num_tokens, sc.num_requests, sc.max_q_len, sc.max_kv_len = T, B, max(lengths), kv_len
            sc.cu_q, sc.kv_lens = cu, torch.full((B,), kv_len, dtype=torch.int32, device=dev)
            sc.host = {"cu_q": cu.tolist(), "kv_lens": [kv_len] * B}
            us = timer(lambda: ops.paged_attention(q, kc, vc, view, sc, D ** -0.5, **kw))
            roof = (4.0 * H * D * seen / (peaks["bf16_tflops"] * 1e6) if T > B
                    else B * seen * 2 * G * D * 2 / (peaks["hbm_gbs"] * 1e3))
            return us, roof

        H, G, chunk = left["heads"], left["kv_heads"], left["mask"]["size"]
        slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device=dev)
        frac(f"chunked_attention_{name}", *attention(H, G, 128, float((pos % chunk + 1).sum()), chunk=chunk, slopes=slopes,
                                                     sinks=torch.randn(H, device=dev)))
        window, keep = win["mask"]["size"], win["mask"]["keep_first"]
        seen = torch.minimum(pos + 1, torch.full_like(pos, window)) + torch.clamp(
            torch.minimum(pos + 1 - window, torch.full_like(pos, keep)), min=0)
        frac(f"delilorn_window_attention_{name}", *attention(H, G, 128, float(seen.sum()), window=window, keep_first=keep))
        # the scans
        ctx = SimpleNamespace(num_requests=B, cu_q=cu, max_q_len=max(lengths),
                              state_slots=torch.arange(B, dtype=torch.int32, device=dev),
                              fresh=torch.zeros(B, dtype=torch.int32, device=dev),
                              positions=torch.cat([torch.arange(s, s + m) for s, m in zip(starts, lengths)]).int().to(dev))

        def scan_roof(heads, n, nv, row_bytes):
            return max((T * row_bytes + 2 * B * heads * n * nv * 4) / (peaks["hbm_gbs"] * 1e3),
                       4.0 * T * heads * n * nv / (fma_tflops * 1e6))

        Hh, n, nv = hg["heads"], hg["dim"], hg["vdim"]
        proj = torch.randn(T, Hh * n + Hh * nv, device=dev).to(bf)
        z, low = torch.randn(T, Hh * n, device=dev) + 3, torch.rand(Hh * n, device=dev)
        state, wv = torch.zeros(B, Hh, n, nv, device=dev), torch.ones(nv, device=dev, dtype=bf)
        frac(f"hgrn2_scan_{name}", timer(lambda: ops.linear_attention(
            proj[:, :Hh * n], None, proj[:, Hh * n:], None, state, ctx, Hh, n, nv, bf, decay_logits=z, lower=low, tied_key=True,
            input_activation="q", norm_weight=wv, eps=1e-6)), scan_roof(Hh, n, nv, (Hh * n + 2 * Hh * nv) * 2 + Hh * n * 4))
        Hm, n, nv = ml["heads"], ml["dim"], ml["vdim"]
        cols = (nv // 4 + 1) * 4
        proj = torch.randn(T, 2 * Hm * n + 2 * Hm * nv, device=dev).to(bf)
        gates_raw, m_state = torch.randn(T, 2 * Hm, device=dev), torch.zeros(B, Hm, device=dev)
        state, wn = torch.zeros(B, Hm, n, cols, device=dev), torch.ones(Hm * nv, device=dev, dtype=bf)

        def mlstm():
            keep_, write, floor = ops.mlstm_gates(gates_raw, 15.0, m_state, ctx, Hm)
            o = ops.linear_attention(proj[:, :Hm * n], proj[:, Hm * n:2 * Hm * n], proj[:, 2 * Hm * n:2 * Hm * n + Hm * nv], None,
                                     state, ctx, Hm, n, cols, bf, token_keep=keep_, token_write=write, q_scale=n ** -0.5,
                                     value_width=nv, raw=True)
            return ops.mlstm_finish(o, floor, wn, proj[:, 2 * Hm * n + Hm * nv:], 1e-6, Hm, nv, bf)
        frac(f"mlstm_gates_scan_finish_{name}", timer(mlstm), scan_roof(Hm, n, nv, (2 * Hm * n + 3 * Hm * nv) * 2))
        Hs, nv, n, taps = right["heads"], right["vdim"], right["state"], right["conv"]
        inner, C = Hs * nv, Hs * nv + 2 * right["groups"] * n
        proj = torch.randn(T, inner + C, device=dev).to(bf)
        dt_raw, conv_state = torch.randn(T, Hs, device=dev), torch.zeros(B, taps - 1, C, device=dev)
        cw, cb = (torch.randn(C, taps, device=dev) * 0.3).to(bf), torch.zeros(C, device=dev, dtype=bf)
        dtb, alog, skip = (torch.zeros(Hs, device=dev, dtype=bf) for _ in range(3))
        state, wn = torch.zeros(B, Hs, n, nv, device=dev), torch.ones(inner, device=dev, dtype=bf)

        def ssm():
            xbc = ops.causal_conv(proj[:, inner:], cw, conv_state, ctx, bf, bias=cb, activation="silu")
            o = ops.linear_attention(xbc[:, inner + n * right["groups"]:], xbc[:, inner:inner + n * right["groups"]], xbc[:, :inner],
                                     None, state, ctx, Hs, n, nv, bf, step_sizes=(dt_raw, dtb, alog),
                                     qk_group=Hs // right["groups"], raw=True)
            return ops.ssm_finish(o, xbc[:, :inner], skip, proj[:, :inner], wn, right["norm_groups"], 1e-6, Hs, nv, bf)
        frac(f"state_space_conv_scan_finish_{name}", timer(ssm), scan_roof(Hs, n, nv, (2 * inner + C) * 2))
        Hl, n, nv = lig["heads"], lig["dim"], lig["vdim"]
        proj = torch.randn(T, 2 * Hl * n + 2 * Hl * nv, device=dev).to(bf)
        state, wj = torch.zeros(B, Hl, n, nv, device=dev), torch.ones(Hl * nv, device=dev)
        decay = torch.full((Hl,), 0.99, device=dev)
        frac(f"delilorn_lightning_scan_{name}", timer(lambda: ops.linear_attention(
            proj[:, :Hl * n], proj[:, Hl * n:2 * Hl * n], proj[:, 2 * Hl * n:2 * Hl * n + Hl * nv], proj[:, 2 * Hl * n + Hl * nv:],
            state, ctx, Hl, n, nv, bf, decay=decay, norm_weight=wj, eps=1e-6, input_activation="silu", gate_activation="sigmoid",
            joint_norm=True)), scan_roof(Hl, n, nv, (2 * Hl * n + 3 * Hl * nv) * 2))
        # the experts of both designs (equal active weights)
        h = torch.randn(T, width, device=dev).to(bf)
        for key, cfg, kw in (("gated_experts", raw["layers"][0]["mlp"], dict(activation="silu_gated", router="sigmoid_corrected",
                                                                           groups=4, keep_groups=2)),
                             ("delilorn_experts", other["layers"][0]["mlp"], {})):
            E, top, ffe = cfg["router"]["experts"], cfg["router"]["top"], cfg["expert"]["ff"]
            mats = 3 if kw else 2
            part = MixtureOfExperts(width, ffe, E, top, **kw)
            tensors = {"router.weight": (torch.randn(E, width, device=dev) * 0.1).to(bf),
                       "up.weight": (torch.randn(E * ffe * (mats - 1), width, device=dev) * 0.02).to(bf),
                       "down.weight": (torch.randn(E * width, ffe, device=dev) * 0.02).to(bf)}
            if kw:
                tensors["correction"] = torch.zeros(E, device=dev)
            part.bind(tensors)
            us = timer(lambda: ops.materialize(part.forward(h, None)))
            frac(f"{key}_{name}", us, 2.0 * mats * T * top * width * ffe / (peaks["bf16_tflops"] * 1e6) if T > B
                 else mats * E * width * ffe * 2 / (peaks["hbm_gbs"] * 1e3))
        # what stands between two sub-layers
        res = torch.randn(T, width, device=dev)
        y = torch.randn(T, width, device=dev).to(bf)
        wn, wf = torch.ones(width, device=dev, dtype=bf), torch.ones(width, device=dev)
        cw, cstate = (torch.randn(width, 4, device=dev) * 0.1).to(bf), torch.zeros(B, 3, width, device=dev)

        def between():
            ops.group_norm_add_(y, wn, 2, 1e-6, res)
            return ops.causal_conv(res, cw, cstate, ctx, bf, add_input=True)
        frac(f"group_norm_add_and_input_conv_{name}", timer(between), T * width * (8 + 2 + 4 + 2) / (peaks["hbm_gbs"] * 1e3))
        frac(f"delilorn_normed_add_rmsnorm_{name}", timer(lambda: ops.normed_add_rmsnorm(ops.NormedAddend(y, wf, 1e-6), res, wf, 1e-6, bf)),
             T * width * (8 + 2 + 2) / (peaks["hbm_gbs"] * 1e3))
    return out


def babadra_kernel_table(width, peaks):
    """Babadra's kernels beside the like kernels of Delilorn at this width, time over roofline time.  Attention
    over one latent head (both designs: the same kernel, here without a sink); attention with two capped score
    maps per head (the attention kernel on twice the heads with the cap, then the maps' difference) beside
    Delilorn's window attention and plain attention of as many heads (prefill: FLOPs of the visible keys over the
    library's GEMM rate; decode: bytes of the cached keys and values, the values once per key/value head); the experts with the bounded gate beside Delilorn's (prefill: FLOPs of the chosen
    experts; decode: bytes of all experts' weights); the dense bounded feed-forward beside the gated one of
    Qwen3; the add of a sub-layer's output times its factors with the next norm beside Delilorn's norm + add +
    norm.  Decode launches are replayed from a graph, as the engine replays a decode step."""
    import torch
    from tinyserve_b200.engine.batch import GroupView, StepContext
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts.moe import MixtureOfExperts
    dev, bf = "cuda:0", torch.bfloat16
    raw, beside = babadra_shapes(width)
    lat, two = raw["layers"][0]["mixer"], raw["layers"][1]["mixer"]
    dense, moe, moe_d = raw["layers"][0]["mlp"], raw["layers"][1]["mlp"], beside["layers"][0]["mlp"]
    win = beside["layers"][3]["mixer"]
    out = {}

    def frac(key, us, roof):
        out[key] = {"us": round(us, 1), "roofline_us": round(roof, 2), "frac": round(roof / us, 3)}

    for name, lengths, starts in (("prefill_2048", [2048], [0]), ("decode_b8", [1] * 8, [2048] * 8)):
        T, B = sum(lengths), len(lengths)
        timed = _time_us if T > B else _time_graph_us
        kv_len, page = starts[0] + lengths[0], 64
        pages_per = -(-kv_len // page)
        cu = torch.tensor([0] + list(torch.tensor(lengths).cumsum(0)), dtype=torch.int32, device=dev)
        table = (torch.arange(B * pages_per, dtype=torch.int32, device=dev) + 1).view(B, pages_per)

        def context():
            sc = StepContext()
            sc.num_tokens, sc.num_requests, sc.max_q_len, sc.max_kv_len = T, B, max(lengths), kv_len
            sc.cu_q, sc.kv_lens = cu, torch.full((B,), kv_len, dtype=torch.int32, device=dev)
            sc.host = {"cu_q": cu.tolist(), "kv_lens": [kv_len] * B}
            return sc

        def attention(H, G, D, window=0, keep=0, sinks=None, shared=False, softcap=0.0, after=None, value_heads=0):
            kc = torch.randn(B * pages_per + 1, G, page, D, device=dev).to(bf)
            vc = kc if shared else torch.randn(B * pages_per + 1, value_heads or G, page, D, device=dev).to(bf)
            view = GroupView(page, pages_per, None, table, kc.shape[0])
            q = torch.randn(T, H, D, device=dev).to(bf)
            sc = context()
            ops.paged_attention(q, kc, vc, view, sc, D ** -0.5, window, keep_first=keep, sinks=sinks, softcap=softcap)   # (work lists)
            run = lambda: ops.paged_attention(q, kc, vc, view, sc, D ** -0.5, window, keep_first=keep, sinks=sinks, softcap=softcap)
            return timed((lambda: after(run())) if after else run)

        def seen(window=0, keep=0):
            pos = torch.arange(kv_len - lengths[0], kv_len)
            n = pos + 1 if not window else torch.minimum(pos + 1, torch.full_like(pos, window)) + torch.clamp(
                torch.minimum(pos + 1 - window, torch.full_like(pos, keep)), min=0)
            return float(n.sum())

        def attention_roof(H, D, key_heads, value_heads, window=0, keep=0):
            if T > B:
                return 4.0 * H * D * seen(window, keep) / (peaks["bf16_tflops"] * 1e6)
            return B * seen(window, keep) * (key_heads + value_heads) * D * 2 / (peaks["hbm_gbs"] * 1e3)

        heads = lat["heads"]
        D = -(-(lat["kv_rank"] + lat["rot_dim"]) // 16) * 16
        frac(f"latent_attention_{name}", attention(heads, 1, D, shared=True), attention_roof(heads, D, 1, 0))
        frac(f"delilorn_latent_attention_{name}", attention(heads, 1, D, sinks=torch.randn(heads, device=dev), shared=True),
             attention_roof(heads, D, 1, 0))
        H2, G2 = two["heads"], two["kv_heads"]
        combine = lambda o: ops.map_difference(o, H2, G2, 128, 0.8, 1e-6, 0.5)
        frac(f"two_map_attention_{name}", attention(2 * H2, 2 * G2, 128, softcap=two["softcap"], after=combine, value_heads=G2),
             attention_roof(2 * H2, 128, 2 * G2, G2))
        frac(f"two_map_attention_kernel_alone_{name}", attention(2 * H2, 2 * G2, 128, softcap=two["softcap"], value_heads=G2),
             attention_roof(2 * H2, 128, 2 * G2, G2))
        frac(f"attention_as_many_heads_{name}", attention(2 * H2, 2 * G2, 128), attention_roof(2 * H2, 128, 2 * G2, 2 * G2))
        Gw = win["kv_heads"]
        frac(f"delilorn_window_attention_{name}", attention(heads, Gw, 128, win["mask"]["size"], win["mask"]["keep_first"]),
             attention_roof(heads, 128, Gw, Gw, win["mask"]["size"], win["mask"]["keep_first"]))
        # what stands before the attention kernel: norm of q and k per map, rotation, the maps' rows, keys and values
        qkv = torch.randn(T, (2 * H2 + 2 * G2) * 128 + G2 * 128, device=dev).to(bf)
        kc = torch.zeros(B * pages_per + 1, 2 * G2, page, 128, device=dev, dtype=bf)
        vc = torch.zeros(B * pages_per + 1, G2, page, 128, device=dev, dtype=bf)
        slots = torch.cat([table[b, (s + torch.arange(m, device=dev)) // page] * page + (s + torch.arange(m, device=dev)) % page
                           for b, (s, m) in enumerate(zip(starts, lengths))]).int()
        positions = torch.cat([torch.arange(s, s + m) for s, m in zip(starts, lengths)]).int().to(dev)
        from tinyserve_b200.parts.rotary import Rotary
        cos, sin = Rotary.tables(64, 2.5e5, CONTEXT)
        rotary = type("R", (), {"cos": cos.to(dev), "sin": sin.to(dev), "rotary_dim": 64, "interleaved": False})()
        wq = torch.ones(128, device=dev)
        q_end, k_end = 2 * H2 * 128, (2 * H2 + 2 * G2) * 128
        frac(f"two_map_norm_rotary_cache_write_{name}", timed(lambda: ops.rope_unit_kvwrite(
            qkv[:, :q_end], qkv[:, q_end:k_end], qkv[:, k_end:], positions, 2 * H2, 2 * G2, 128, 128, 128, rotary=rotary,
            k_cache=kc, v_cache=vc, slot_mapping=slots, page_size=page, q_weight=wq, k_weight=wq, pre_eps=1e-6, maps=2)),
            T * (2 * H2 + 2 * G2 + G2) * 128 * 2 * 2 / (peaks["hbm_gbs"] * 1e3))
        # (the like kernel of Delilorn's window attention: as many heads, rotation and cache write alone)
        qkv1 = torch.randn(T, (heads + 2 * Gw) * 128, device=dev).to(bf)
        kc1 = torch.zeros(B * pages_per + 1, Gw, page, 128, device=dev, dtype=bf)
        vc1 = torch.zeros_like(kc1)
        frac(f"delilorn_rotary_cache_write_{name}", timed(lambda: ops.rope_unit_kvwrite(
            qkv1[:, :heads * 128], qkv1[:, heads * 128:(heads + Gw) * 128], qkv1[:, (heads + Gw) * 128:], positions, heads, Gw,
            128, 128, 128, rotary=rotary, k_cache=kc1, v_cache=vc1, slot_mapping=slots, page_size=page)),
            T * (heads + 2 * Gw) * 128 * 2 * 2 / (peaks["hbm_gbs"] * 1e3))
        # the experts, and the dense feed-forward
        E, top = moe["router"]["experts"], moe["router"]["top"]
        ffe, ffd, ff = moe["expert"]["ff"], moe_d["expert"]["ff"], dense["ff"]
        mine = MixtureOfExperts(width, ffe, E, top, activation="bounded_swish_gated", router="softmax_chosen", limit=7.0, router_bias=True)
        mine.bind({"router.weight": (torch.randn(E, width, device=dev) * 0.1).to(bf), "router.bias": torch.randn(E, device=dev),
                   "up.weight": (torch.randn(E * 2 * ffe, width, device=dev) * 0.02).to(bf),
                   "down.weight": (torch.randn(E * width, ffe, device=dev) * 0.02).to(bf)})
        theirs = MixtureOfExperts(width, ffd, E, top)
        theirs.bind({"router.weight": (torch.randn(E, width, device=dev) * 0.1).to(bf),
                     "up.weight": (torch.randn(E * ffd, width, device=dev) * 0.02).to(bf),
                     "down.weight": (torch.randn(E * width, ffd, device=dev) * 0.02).to(bf)})
        h = torch.randn(T, width, device=dev).to(bf)
        gate_up = (torch.randn(2 * ff, width, device=dev) * 0.02).to(bf)
        down = (torch.randn(width, ff, device=dev) * 0.02).to(bf)
        block = ops.GATED_BLOCK if ff % ops.GATED_BLOCK == 0 else 0
        us_mine = timed(lambda: ops.materialize(mine.forward(h, None)))
        us_theirs = timed(lambda: ops.materialize(theirs.forward(h, None)))
        us_dense = timed(lambda: ops.materialize(ops.linear(ops.gated_linear(h, gate_up, "bounded_swish", block, 7.0), down)))
        us_silu = timed(lambda: ops.materialize(ops.linear(ops.gated_linear(h, gate_up, "silu", block), down)))
        if T > B:
            frac(f"experts_{name}", us_mine, 6.0 * T * top * width * ffe / (peaks["bf16_tflops"] * 1e6))
            frac(f"delilorn_experts_{name}", us_theirs, 4.0 * T * top * width * ffd / (peaks["bf16_tflops"] * 1e6))
            frac(f"dense_feed_forward_{name}", us_dense, 6.0 * T * width * ff / (peaks["bf16_tflops"] * 1e6))
            frac(f"qwen3_feed_forward_{name}", us_silu, 6.0 * T * width * ff / (peaks["bf16_tflops"] * 1e6))
        else:
            frac(f"experts_{name}", us_mine, 3.0 * E * width * ffe * 2 / (peaks["hbm_gbs"] * 1e3))
            frac(f"delilorn_experts_{name}", us_theirs, 2.0 * E * width * ffd * 2 / (peaks["hbm_gbs"] * 1e3))
            frac(f"dense_feed_forward_{name}", us_dense, 3.0 * width * ff * 2 / (peaks["hbm_gbs"] * 1e3))
            frac(f"qwen3_feed_forward_{name}", us_silu, 3.0 * width * ff * 2 / (peaks["hbm_gbs"] * 1e3))
        # the stream: output times its factors, added and normed; Delilorn: output normed, added and normed
        res = torch.randn(T, width, device=dev)
        y = torch.randn(T, width, device=dev).to(bf)
        wn, ls = torch.ones(width, device=dev), torch.ones(width, device=dev).to(bf)
        roof = T * width * (8 + 2 + 2) / (peaks["hbm_gbs"] * 1e3)
        frac(f"scaled_add_rmsnorm_{name}", timed(lambda: ops.add_rmsnorm(ops.ColumnScaled(y, ls), res, wn, 1e-6, bf)), roof)
        frac(f"delilorn_normed_add_rmsnorm_{name}", timed(lambda: ops.normed_add_rmsnorm(ops.NormedAddend(y, wn, 1e-6), res, wn, 1e-6, bf)), roof)
        first = torch.randn(T, width, device=dev)
        frac(f"stream_add_{name}", timed(lambda: ops.stream_add_(res, ops.ColumnScaled(y, ls), first)),
             T * width * (8 + 2 + 4) / (peaks["hbm_gbs"] * 1e3))
    return out


# design -> (its shapes and those of the model beside it, its kernel table, the name of the model beside it)
ARCH_BENCHES = {"dudatar": (dudatar_shapes, kernel_table, "qwen3"), "delilorn": (delilorn_shapes, delilorn_kernel_table, "qwen3"),
                "tarivik": (tarivik_shapes, tarivik_kernel_table, "delilorn"),
                "babadra": (babadra_shapes, babadra_kernel_table, "delilorn")}


def arch_main(a) -> int:
    """``--arch dudatar`` / ``--arch delilorn``: the design beside Qwen3 at equal size; ``--arch tarivik`` and
    ``--arch babadra``: beside Delilorn, the closest design (experts, latent attention, matrix-state mixers).  One
    JSON line."""
    import torch
    from tinyserve_b200 import LLM
    from tinyserve_b200.config import config_from_dict
    peaks = load_peaks()
    warmup, steps = max(a.warmup, 3), min(a.steps, 64)
    sizes = {}
    for width in [int(w) for w in a.sizes.split(",")]:
        entry = {}
        shapes, table, beside = ARCH_BENCHES[a.arch]
        for name, raw in zip((a.arch, beside), shapes(width)):
            llm = LLM(model_config=config_from_dict(raw), random_weights=True, dtype="bfloat16", max_model_len=CONTEXT,
                      block_size=a.block_size, max_num_seqs=8, max_num_batched_tokens=PREFILL_TOKENS,
                      num_blocks=8 * (CONTEXT // a.block_size) // 2 + 4096 // a.block_size, use_cuda_graphs=False, seed=a.seed)
            llm.runner.capture_decode_graphs([8])
            dec = run_decode(llm, 8, steps, warmup, a.seed)
            ms = run_prefill(llm, a.seed)
            entry[name] = {"decode_b8_tok_s": round(dec["tok_s"], 1), "decode_ms": round(dec["ms"], 4),
                           "decode_launches_per_step": dec["launches"] // steps,
                           "prefill_2048_tok_s": round(PREFILL_TOKENS * 1000.0 / ms, 1), "prefill_ms": round(ms, 3),
                           "weight_gib": round(llm.runner.weight_bytes / 2 ** 30, 3)}
            _release(llm)
            llm = None
        entry["kernels"] = table(width, peaks)
        sizes[str(width)] = entry
    beside = ARCH_BENCHES[a.arch][2].capitalize()
    print(json.dumps({"metric": f"prefill and decode tok/s, {a.arch.capitalize()} beside {beside} at equal size (random weights)",
                      "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "steps": steps,
                      "warmup": warmup, "block_runs": 6, "sizes": sizes, "peaks": peaks}))
    return 0


def reference_main(a) -> int:
    """``--impl reference``: priyammaz/tinyserve, unmodified, from baseline/_ref, through its own
    Engine (see baseline/reference_arm.py).  If it cannot start here, the line says why."""
    if a.gpus != 1:
        print(f"bench.py: the reference arm runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
        raw = dict(QWEN3_8B, num_hidden_layers=a.layers)
        line = reference_arm.run(raw, a.batch, a.steps, max(a.warmup, 3), a.seed, CONTEXT, PROMPT_LEN,
                                 PREFILL_TOKENS, not a.no_points, load_peaks(), ClockSampler(),
                                 burst_raw=None if a.no_workloads else QWEN3_0P6B)
    except BaseException as exc:                      # noqa: BLE001 - the reason goes into the line
        if isinstance(exc, KeyboardInterrupt):
            raise
        import traceback
        traceback.print_exc()
        why = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:400]
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="tinyserve_b200")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and prefill")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the 0.6B burst, the 32B run and the long-context decode")
    ap.add_argument("--arch", choices=["qwen3", "dudatar", "delilorn", "tarivik", "babadra"], default="qwen3",
                    help="dudatar, delilorn: measure that design beside Qwen3 at equal size instead of the default workload; "
                         "tarivik, babadra: beside Delilorn")
    ap.add_argument("--sizes", default="2048,4096", help="--arch dudatar / delilorn / tarivik / babadra: model widths to measure")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_main(a)
    if a.arch in ARCH_BENCHES:
        if a.gpus != 1:
            print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
            return 2
        return arch_main(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    sampler = ClockSampler()
    sampler.start()                   # early: nvidia-smi takes longer to come up than a short timed region lasts
    import torch
    from tinyserve_b200 import LLM, Qwen3Config
    from tinyserve_b200.kernels import ops
    warmup = max(a.warmup, 3)
    raw = dict(QWEN3_8B, num_hidden_layers=a.layers)
    config = Qwen3Config.from_dict(raw)
    peaks = load_peaks()
    sizes = sorted({1, a.batch, 64}) if not a.no_points else [a.batch]
    llm = LLM(model_config=config, random_weights=True, dtype="bfloat16", max_model_len=CONTEXT,
              block_size=a.block_size, max_num_seqs=max(sizes), max_num_batched_tokens=PREFILL_TOKENS,
              num_blocks=max(sizes) * (CONTEXT // a.block_size) // 2 + 4096 // a.block_size, use_cuda_graphs=False,
              seed=a.seed)
    llm.runner.capture_decode_graphs(sizes)

    main_run = run_decode(llm, a.batch, a.steps, warmup, a.seed, sampler)
    e2e = run_e2e(llm, a.batch, a.steps, warmup, a.seed)
    points, prefill = {}, None
    if not a.no_points:
        for b in (1, 64):
            r = run_decode(llm, b, min(a.steps, 64), warmup, a.seed + b)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        ms = run_prefill(llm, a.seed)
        flops = prefill_flops(raw, a.layers, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS * 1000.0 / ms, 1), "tokens": PREFILL_TOKENS,
                   "ms": round(ms, 3), "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
    if not a.no_points and not a.no_workloads and a.layers == QWEN3_8B["num_hidden_layers"]:
        _release(llm)
        llm = None
        for fn, args in ((run_burst_0p6b, (a.seed, a.block_size)), (run_large_32b, (a.seed, 16)),
                         (run_long_context, (a.seed, min(a.steps, 32), warmup, a.block_size))):
            try:
                points.update(fn(*args))
            except Exception as exc:                  # noqa: BLE001 - a workload that fails is named, the line still prints
                points[fn.__name__ + "_error"] = f"{type(exc).__name__}: {exc}"[:200]
    nbytes = decode_bytes(raw, a.layers, a.batch, main_run["ctx"])
    achieved = nbytes / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s (Qwen3-8B shapes, random weights)", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(main_run["tok_s"] / (42.2 * a.batch), 3) if a.batch == 1 else None,
        "dtype": "bf16", "data": "synthetic", "impl": "tinyserve_b200",
        "config": {"model": "Qwen3-8B shapes", "global_batch": a.batch, "seq_len": CONTEXT,
                   "parallelism": "none", "layers": a.layers,
                   "layers_of_model": QWEN3_8B["num_hidden_layers"], "hidden": raw["hidden_size"],
                   "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"],
                   "vocab": raw["vocab_size"], "prompt_len": PROMPT_LEN, "block_size": a.block_size,
                   "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": peaks["source"], "peak_hbm_gbs": peaks["hbm_gbs"],
                   "peak_bf16_tflops": peaks["bf16_tflops"]},
        "clocks": main_run["clocks"], "e2e": {k: (round(v, 1) if isinstance(v, float) else v)
                                               for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
    }
    if prefill:
        line["prefill"] = prefill
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
