#!/usr/bin/env python3
"""Benchmark: decode tokens per second of the Llama-3.1-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on standard output.  A "step" is one decode step of a batch of 8 requests,
each holding a 2,048-token prompt in the cache (context 4,096), random weights, random
token ids.  ``value`` is decoded tokens per second timed on the device with CUDA events
around K steps of the engine's step function and its sampling kernel; ``e2e`` is the same
through the Python entry point (``Engine.generate``: host token lists in, host token lists
out, every step copies its inputs from pinned memory and reads the sampled tokens back).
``prefill`` is one 2,048-token prompt in one step; ``points`` adds decode at batch 1 and
64; ``roofline`` is the bytes a decode step has to read (every weight once and the cache
of the live requests, at their mean length over the timed steps) over its time, against the
measured copy bandwidth, and ``roofline_points`` the same fraction for every batch size.

``--shape llama32_3b`` runs that shape's own workload (32 prompts of 128 to 4,096 tokens in
portions of 512 beside decodes, 512 new tokens each) through ``Engine.generate``;
``--shape llama2_13b`` decodes at batch 16 after 3,584-token prompts; ``--cpu-baseline``
times the plain CPU implementation at the tiny configurations.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 14336, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": False, "mlp_bias": False,
    "max_position_embeddings": 4096, "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# Two further shapes for --shape (the default run and its record are the first one's): their
# batch, prompt length and context follow the workloads they are quoted with.
LLAMA32_3B = {**LLAMA31_8B, "num_hidden_layers": 28, "hidden_size": 3072, "num_attention_heads": 24, "intermediate_size": 8192,
              "tie_word_embeddings": True, "rope_scaling": {**LLAMA31_8B["rope_scaling"], "factor": 32.0}}
LLAMA2_13B = {**LLAMA31_8B, "num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 40,
              "intermediate_size": 13824, "vocab_size": 32000, "rope_theta": 10000.0, "rope_scaling": None}
SHAPES = {"llama31_8b": ("Llama-3.1-8B shape", LLAMA31_8B, 8, 2048, 4096),
          "llama32_3b": ("Llama-3.2-3B shape", LLAMA32_3B, 32, 2048, 4096),
          "llama2_13b": ("Llama-2-13B shape", LLAMA2_13B, 16, 3584, 4096)}
PROMPT_LEN = 2048
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(cfg) -> int:
    """Bytes of every weight a decode step reads once (bfloat16): the layers and the head."""
    E, F, H, G, D, V, L = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                           cfg.head_dim, cfg.vocab_size, cfg.num_hidden_layers)
    per_layer = (H + 2 * G) * D * E + E * H * D + 3 * F * E
    return 2 * (L * per_layer + V * E) + 4 * (2 * L + 1) * E


def step_flops(cfg, n_tokens: int, kv_lens) -> float:
    """Matrix products (2 flops per weight per token) plus causal attention."""
    E, F, H, G, D, V, L = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                           cfg.head_dim, cfg.vocab_size, cfg.num_hidden_layers)
    per_layer = (H + 2 * G) * D * E + E * H * D + 3 * F * E
    mm = 2.0 * n_tokens * L * per_layer + 2.0 * V * E          # the head runs on one row
    att = sum(4.0 * H * D * L * (k * (k + 1) / 2) for k in kv_lens)   # q.k and p.v over the causal triangle
    return mm + att


def run_decode(runner, cfg, batch: int, steps: int, warmup: int, seed: int = 0):
    """Prefill ``batch`` prompts, then time ``steps`` decode steps on the device."""
    import torch

    from lgml_b200 import ops

    g = torch.Generator().manual_seed(seed)
    reqs = [runner.open(("bench", batch, i)) for i in range(batch)]
    try:
        for r in reqs:
            ids = torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=g).tolist()
            for p in range(0, PROMPT_LEN, 512):
                runner.step([(r, ids[p:p + 512], [])])
        tok = torch.randint(0, cfg.vocab_size, (batch,), generator=g).to(torch.int32).to(runner.rt.device)
        scratch = torch.empty(64 * batch, dtype=torch.int32, device=runner.rt.device)

        def one():
            # the sampled ids stay on the device and feed the next step
            logits = runner.decode_step(reqs, tok)
            ops.argmax_rows(logits, tok, scratch)

        for _ in range(warmup):
            one()
        launches0 = ops.launch_count()
        replays0 = runner.graph_replays
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        # keys a timed step reads, on average: what the requests held half-way through the timed steps
        kv_tokens = sum(r.n_tokens for r in reqs) - batch * (steps - 1) / 2.0
        launches = ops.launch_count() - launches0 + (runner.graph_replays - replays0) * runner.graph_kernels(batch)
        runner.rt.check_status()
        return ms / steps, kv_tokens, launches
    finally:
        for r in reqs:
            runner.close(r)


def run_prefill(runner, cfg, reps: int = 3, seed: int = 1):
    import torch

    g = torch.Generator().manual_seed(seed)
    best = None
    for i in range(reps + 1):
        ids = torch.randint(0, cfg.vocab_size, (PREFILL_TOKENS,), generator=g).tolist()
        r = runner.open(("prefill", i))
        try:
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for p0 in range(0, PREFILL_TOKENS, 2048):
                part = ids[p0:p0 + 2048]
                runner.step([(r, part, [len(part) - 1] if p0 + 2048 >= PREFILL_TOKENS else [])])
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
            if i > 0:                      # the first run loads kernels
                best = ms if best is None else min(best, ms)
        finally:
            runner.close(r)
    return best


def run_mixed_workload(shape_name, shape, args, warmup: int) -> dict:
    """The workload the 3B shape is quoted with: 32 prompts of 128 to 4,096 uniform-random tokens,
    read in portions of 512 beside the decoding of the requests that are further on, 512 new
    tokens each, through ``Engine.generate`` (host token lists in and out).  Rates as the
    reference reports them per request (``prompt_per_second`` / ``predicted_per_second``,
    ``lua/lgml/engine.lua:3225-3239``), here over the whole job, with the share of turns that
    held portions of prompts beside decoded tokens."""
    import torch

    import lgml_b200
    from lgml_b200.config import config_from_dict

    n_req, new_tokens, ubatch, budget = 32, 512, 512, 2048
    n_ctx = 4096 + new_tokens + 64
    d = dict(shape)
    full_layers = d["num_hidden_layers"]
    if args.layers:
        d["num_hidden_layers"] = args.layers
    d["max_position_embeddings"] = 8192
    cfg = config_from_dict(d)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(128, 4097, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    eng = lgml_b200.Engine(config=cfg, random_weights=0, dtype="bfloat16", n_ctx=n_ctx, kv_tokens=n_req * n_ctx, slots=n_req, ubatch=ubatch,
                           max_batch_tokens=budget)
    eng.generate([p[:600] for p in prompts[:n_req]], max_tokens=max(warmup, 3) + 2, temperature=0.0, stop=[])    # kernels loaded, decode graph captured
    # measured twice, the faster run kept: the host shares its machine with other jobs, and a few stalled
    # turns (tens of milliseconds each) otherwise decide the figure
    clocks = ClockSampler()
    clocks.start()
    best = None
    for _ in range(2):
        out = eng.generate(prompts, max_tokens=new_tokens, temperature=0.0, stop=[])
        if best is None or eng.timings["total"] < best[0]:
            best = (eng.timings["total"], list(eng.turn_log), out)
    clock_rec = clocks.stop()
    wall, log, out = best
    kinds = {"prompt": [t for t in log if t["decode"] == 0], "mixed": [t for t in log if t["decode"] > 0 and not t["pure_decode"]],
             "decode": [t for t in log if t["pure_decode"]]}
    n_prompt, n_new = sum(lens), sum(len(o) for o in out)
    secs = {k: sum(t["s"] for t in v) for k, v in kinds.items()}
    prompt_in_mixed = sum(t["tokens"] - t["decode"] for t in kinds["mixed"])
    decode_in_mixed = sum(t["decode"] for t in kinds["mixed"])
    mixed = {
        "requests": n_req, "prompt_tokens": n_prompt, "new_tokens": n_new, "ubatch": ubatch, "max_batch_tokens": budget,
        "turns": len(log), "mixed_turn_share": round(len(kinds["mixed"]) / max(len(log), 1), 4),
        "mixed_time_share": round(secs["mixed"] / max(wall, 1e-9), 4),
        "prompt_tok_s": round(n_prompt / max(secs["prompt"] + secs["mixed"], 1e-9), 1),
        "decode_tok_s": round(sum(t["decode"] for t in kinds["decode"]) / max(secs["decode"], 1e-9), 1),
        "mixed_turn_ms": round(1e3 * secs["mixed"] / max(len(kinds["mixed"]), 1), 3),
        "mixed_turn_tokens": round((prompt_in_mixed + decode_in_mixed) / max(len(kinds["mixed"]), 1), 1),
        "decode_turn_ms": round(1e3 * secs["decode"] / max(len(kinds["decode"]), 1), 3),
        "preemptions": eng.scheduler.stats["preemptions"],
    }
    total = (n_prompt + n_new) / wall
    h2d = sum(t["h2d"] for t in log) // max(len(log), 1)
    d2h = sum(t["d2h"] for t in log) // max(len(log), 1)
    return {
        "metric": f"total tok/s (prompt + new) of the mixed workload ({shape_name}: {n_req} prompts of 128-4,096 tokens, portions of {ubatch} beside decodes, {new_tokens} new tokens each)",
        "value": round(total, 1), "unit": "tok/s", "n_gpus": 1, "steps": len(log), "warmup": max(warmup, 3),
        "ms_per_step": round(1e3 * wall / max(len(log), 1), 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids and prompt lengths",
        "config": {"model": shape_name, "layers": cfg.num_hidden_layers, "layers_of_model": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": n_req, "seq_len": n_ctx, "page": 64,
                   "parallelism": "single GPU", "l2": "inputs exceed L2 (the weights alone are %.1f GB)" % (weight_bytes(cfg) / 1e9),
                   "peaks": peak_src, "timing": "host clock around Engine.generate (a step is a scheduler turn), best of 2"},
        "clocks": clock_rec,
        "e2e": {"value": round(total, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": len(log)},
        "gpu_launches": int(lgml_b200.ops.launch_count()),
        "mixed": mixed,
        "kernel_libraries": lgml_b200.csrc.loaded_libraries(),
    }


def run_cpu_baseline() -> dict:
    """The stated CPU baseline: the plain float64 implementation under ``tests/plain`` (whole
    sequences, no cache) on the host, at the two tiny configurations: tokens per second of a
    prompt of 130 tokens in one pass, and of 16 greedy tokens after it (each a pass over the
    whole sequence so far, as that implementation works)."""
    import tempfile

    from tests import helpers as H
    from tests.plain import llama_plain as P

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name in ("A", "B"):
            cfg_d, seed = H.TINY[name]
            folder = H.make_folder(Path(tmp) / name, cfg_d, seed)
            cfg, w = P.load_folder(folder)
            n = min(130, cfg_d["max_position_embeddings"] - 17)
            ids = H.random_ids(n, cfg_d["vocab_size"], 1)
            P.forward(cfg, w, ids[:8])
            t0 = time.perf_counter()
            P.forward(cfg, w, ids)
            t1 = time.perf_counter()
            P.greedy(cfg, w, ids, 16)
            t2 = time.perf_counter()
            out[f"tiny_{name}"] = {"prompt_tokens": n, "prompt_tok_s": round(n / (t1 - t0), 1), "decode_tok_s": round(16 / (t2 - t1), 1)}
    return {"impl": "plain-cpu", "what": "tests/plain/llama_plain.py, float64, whole sequences, host threads", "points": out}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in the record)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--shape", default="llama31_8b", choices=list(SHAPES), help="layer sizes and workload (the default is the headline's)")
    ap.add_argument("--decode-only", action="store_true", help="with --shape llama32_3b: plain decode steps at batch 32 instead of its mixed workload")
    ap.add_argument("--batch", type=int, default=0, help="batch of the decode run instead of the shape's own")
    ap.add_argument("--prompt-len", type=int, default=0, help="prompt length of the decode runs instead of the shape's own (for other context lengths)")
    ap.add_argument("--context", type=int, default=0, help="context (tokens a request may hold) instead of the shape's own")
    ap.add_argument("--prefill-tokens", type=int, default=0, help="tokens of the timed prompt instead of 2,048 (read in portions of 2,048)")
    ap.add_argument("--no-kernel-times", action="store_true", help="leave out the per-kernel-class times of a decode step")
    ap.add_argument("--cpu-baseline", action="store_true", help="time the plain CPU implementation at the tiny configurations and stop")
    args = ap.parse_args()
    if args.cpu_baseline:
        print(json.dumps(run_cpu_baseline()))
        return 0

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "mischief/lgml is Lua on a ggml fork fetched over the network with a "
                          "Vulkan GPU path; it has no pip-installable package and cannot be built or run offline on this box"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    import torch

    import lgml_b200
    from lgml_b200 import ops
    from lgml_b200.config import config_from_dict
    from lgml_b200.engine.runner import ModelRunner

    global BATCH, PROMPT_LEN, CONTEXT
    shape_name, shape, BATCH, PROMPT_LEN, CONTEXT = SHAPES[args.shape]
    global PREFILL_TOKENS
    if args.batch:
        BATCH = args.batch
    if args.prompt_len:
        PROMPT_LEN = args.prompt_len
    if args.context:
        CONTEXT = args.context
    if args.prefill_tokens:
        PREFILL_TOKENS = args.prefill_tokens
    # turns in which the engine still reads prompts: a request that is done with its prompt decodes beside
    # the others' portions, so every request gets this many new tokens more than the turns that are timed
    prompt_turns = -(-BATCH * PROMPT_LEN // 2048)
    CONTEXT = -(-max(CONTEXT, PROMPT_LEN + args.steps + 64 + prompt_turns, PREFILL_TOKENS) // 64) * 64
    if args.shape == "llama32_3b" and not args.decode_only:
        print(json.dumps(run_mixed_workload(shape_name, shape, args, warmup)))
        return 0
    d = dict(shape)
    full_layers = d["num_hidden_layers"]
    if args.layers:
        d["num_hidden_layers"] = args.layers
    d["max_position_embeddings"] = max(d["max_position_embeddings"], CONTEXT)
    cfg = config_from_dict(d)
    hbm_gbs, bf16_tflops, peak_src = peaks()
    points_too = args.shape == "llama31_8b" and not args.skip_points
    n_pages = (64 if points_too else BATCH) * (CONTEXT // 64) + 8     # room for 64 requests of the benchmark context
    runner = ModelRunner.from_config(cfg, seed=0, dtype=torch.bfloat16, n_pages=n_pages, max_slots=max(64, BATCH), max_step_tokens=2048)

    prefill_ms = run_prefill(runner, cfg)
    clocks = ClockSampler()
    clocks.start()
    ms_step, kv_tokens, launches = run_decode(runner, cfg, BATCH, args.steps, warmup)
    clock_rec = clocks.stop()
    kv_token_bytes = 2 * cfg.num_key_value_heads * cfg.head_dim * 2 * cfg.num_hidden_layers

    def hbm_frac(ms, kv):
        """bytes a decode step has to read (every weight once, the live requests' cache) / time / the copy peak"""
        return (weight_bytes(cfg) + kv * kv_token_bytes) / (ms * 1e-3) / 1e9 / hbm_gbs

    points = {}
    roofline_points = {f"decode_b{BATCH}": round(hbm_frac(ms_step, kv_tokens), 4)}
    if points_too:
        for b, k in ((1, min(args.steps, 64)), (64, min(args.steps, 32))):
            ms_b, kv_b, _ = run_decode(runner, cfg, b, k, warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / ms_b, 1)
            roofline_points[f"decode_b{b}"] = round(hbm_frac(ms_b, kv_b), 4)

    # device time by kernel class, from events around every launch of a few eager steps (they run one after
    # the other then: shares of a step, not its time, which the captured graph's kernels overlap)
    kernel_us = {}
    if not args.no_kernel_times:
        g = torch.Generator().manual_seed(9)
        reqs = [runner.open(("classes", i)) for i in range(BATCH)]
        try:
            for r in reqs:
                ids = torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=g).tolist()
                for p0 in range(0, PROMPT_LEN, 512):
                    runner.step([(r, ids[p0:p0 + 512], [])])
            toks = [[int(t)] for t in torch.randint(0, cfg.vocab_size, (BATCH,), generator=g)]
            runner.step([(r, t, [0]) for r, t in zip(reqs, toks)])
            with ops.KernelTimes() as kt:
                for _ in range(3):
                    runner.step([(r, t, [0]) for r, t in zip(reqs, toks)])
            tot = kt.totals()
            kernel_us = {k: round(v / 3.0, 1) for k, v in tot.items() if not k.endswith(" calls")}
        finally:
            for r in reqs:
                runner.close(r)

    value = BATCH * 1000.0 / ms_step
    step_bytes = weight_bytes(cfg) + kv_tokens * kv_token_bytes
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    pf_flops = step_flops(cfg, PREFILL_TOKENS, [PREFILL_TOKENS])      # (read in portions: the same products and the same causal triangle)
    prefill = {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(pf_flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12), 4)}

    # end to end through the Python entry point, on the same weights
    del runner
    torch.cuda.empty_cache()
    eng = lgml_b200.Engine(config=cfg, random_weights=0, dtype="bfloat16", n_ctx=CONTEXT, kv_tokens=BATCH * CONTEXT, slots=BATCH, ubatch=512,
                           max_batch_tokens=2048)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (PROMPT_LEN,), generator=g).tolist() for _ in range(BATCH)]
    eng.generate(prompts, max_tokens=warmup + 2 + prompt_turns, temperature=0.0, stop=[])      # warm-up: kernels loaded, graph captured
    # measured three times, the best run kept: the host shares its machine with other jobs, and a
    # single stalled turn (hundreds of milliseconds) otherwise decides the figure
    e2e = None
    for _ in range(3):
        eng.generate(prompts, max_tokens=min(args.steps, 64) + 1 + prompt_turns, temperature=0.0, stop=[])
        r = eng.decode_rate(skip=1, rows=BATCH)      # the turns in which all requests decode
        if r["steps"] == 0:
            r = eng.decode_rate(skip=0)              # too few steps asked for: every decode turn
        if e2e is None or r["tok_s"] > e2e["tok_s"]:
            e2e = r

    rec = {
        "metric": f"decode tok/s at batch {BATCH} ({shape_name}, {PROMPT_LEN:,}-token prompts, context {CONTEXT:,})",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform-random token ids",
        "config": {"model": shape_name, "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": BATCH, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page": 64, "parallelism": "single GPU",
                   "l2": "inputs exceed L2 (a step reads %.1f GB)" % (step_bytes / 1e9), "peaks": peak_src, "e2e_runs": "best of 3"},
        "clocks": clock_rec,
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                "d2h_bytes_per_step": e2e["d2h_bytes_per_step"], "steps": e2e["steps"]},
        "gpu_launches": int(launches),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4)},
        "points": points,
        "roofline_points": roofline_points,
        "kernel_us_per_decode_step": kernel_us,
        "kernel_libraries": lgml_b200.csrc.loaded_libraries(),
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
