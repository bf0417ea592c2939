"""The Python entry point: load a model, generate.

Option names and meanings follow mischief/lgml's ``engine.new``
(``lua/lgml/engine.lua:376-467``): ``model`` (a folder with config.json and
safetensors here), ``n_ctx`` (the size of the cache pool all slots share, and the
most tokens of one request; ``kv_tokens``, which the reference does not have, makes
the pool larger than one request's context), ``slots`` (the most requests kept at once, default 4:
``lua/lgml/kvpool.lua:28``), ``ubatch`` (prompt tokens per request per step,
default 512), ``max_tokens`` (default reply length: the free context),
``sampling`` (sampler defaults, a request's values replace them),
``repeat_stop_tokens``.  ``run_ahead`` (not in the reference): launch a decode step before
the host has seen the ids of the one before, when those are chosen on the device.
``prefix_cache`` (always on in the reference, ``E:reuse`` ``lua/lgml/engine.lua:1775-1819``; off by default
here): the full pages of ended and preempted requests stay findable by a key of their tokens, and a
prompt that begins like one of them computes only the rest.  ``generate.greedy`` of the reference
(``lua/lgml/generate.lua:19-34``) is ``Engine.greedy``.
"""
from __future__ import annotations

import math
import time
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .. import ops
from ..cache import PAGE_SIZE
from ..sampling import Sampler, SamplingParams, log_min_p
from .runner import ModelRunner
from .runtime import MAX_RESULT
from .scheduler import REPEAT_STOP, UBATCH, GenRequest, Scheduler

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not '{name}'") from None


class Engine:
    def __init__(self, model=None, *, config=None, random_weights: Optional[int] = None, dtype="bfloat16", n_ctx: Optional[int] = None,
                 kv_tokens: Optional[int] = None, slots: int = 4, ubatch: int = UBATCH, max_batch_tokens: Optional[int] = None, max_tokens: Optional[int] = None,
                 sampling: Optional[dict] = None, repeat_stop_tokens: int = REPEAT_STOP, device="cuda:0",
                 run_ahead: bool = True, prefix_cache: bool = False):
        dt = parse_dtype(dtype)
        if model is None and config is None:
            raise ValueError("give a model folder, or a config with random_weights=seed")
        if model is not None:
            from ..config import load_config
            cfg = load_config(model)
        else:
            cfg = config
        self.config = cfg
        # a configuration that names no limit of positions is bounded by n_ctx alone
        max_pos = getattr(cfg, "max_position_embeddings", None) or None
        if n_ctx is None and max_pos is None:
            raise ValueError("this configuration names no max_position_embeddings: give n_ctx")
        n_ctx = min(n_ctx or max_pos, max_pos or n_ctx)
        max_pos = max_pos or n_ctx
        self.n_ctx = n_ctx
        # the pool all slots share: n_ctx tokens as in the reference, or kv_tokens when given
        n_pages = -(-(kv_tokens or n_ctx) // PAGE_SIZE)
        max_batch_tokens = max_batch_tokens or max(ubatch, 2048)
        kw = dict(n_pages=n_pages, max_slots=slots, max_step_tokens=max_batch_tokens, prefix_cache=prefix_cache)
        if model is not None:
            self.runner = ModelRunner.from_folder(model, dt, device, **kw)
        else:
            self.runner = ModelRunner.from_config(cfg, int(random_weights or 0), dt, device, **kw)
        self.rt = self.runner.rt
        self.default_max_tokens = max_tokens
        self.sampling_defaults = dict(sampling or {})
        self.scheduler = Scheduler(self.runner.cache, max_position=min(max_pos, n_ctx), ubatch=ubatch,
                                   max_batch_tokens=max_batch_tokens, repeat_stop_tokens=repeat_stop_tokens)
        self.eos_ids = list(getattr(cfg, "eos_token_ids", []) or [])
        # What exists now (modules, the model's objects) lives as long as the engine: keep the
        # collector from walking it again and again.  A full collection over it takes tens of
        # milliseconds, several decode steps, whenever it happens to trigger.
        import gc
        gc.collect()
        gc.freeze()
        self._next_id = 0
        self._on_token = None
        self.run_ahead = run_ahead
        self._ahead: Optional[dict] = None          # the step whose ids the host has not seen yet
        self._host_ring = [torch.empty(MAX_RESULT + 1, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._host_turn = 0
        self._t_mark = time.perf_counter()
        self.timings: Dict[str, float] = {}
        # one record per scheduler turn: wall seconds, prompt tokens, decoded tokens, bytes copied each way
        self.turn_log: List[dict] = []

    # ---- one scheduler turn -------------------------------------------------------------
    # A step whose tokens are chosen on the device is not waited for: its ids travel to the
    # host in the background, and the next decode step, planned ahead of them, is launched
    # with the ids still on the device.  The host's work of a turn then runs beside the GPU's.
    def _launch(self, plan, device_tokens: Optional[torch.Tensor]) -> dict:
        """Run the planned step and choose its tokens.  Returns the record that ``_resolve``
        finishes: ``toks`` when the host already has the ids, else a pinned buffer and the
        event after which it holds them, followed by the status word."""
        if device_tokens is None:
            entries = [(e.request.cache_req, e.tokens, [len(e.tokens) - 1] if e.sample else []) for e in plan]
            logits = self.runner.step(entries)
        else:
            logits = self.runner.decode_step([e.request.cache_req for e in plan], device_tokens)
        rows = [e for e in plan if e.sample]
        rec = {"plan": plan, "rows": rows, "toks": None, "out": None, "h2d": self.runner.last_batch.h2d_bytes + 12 * len(rows)}
        if not rows:
            rec["toks"] = []
            return rec
        n = len(rows)
        neutral = n <= MAX_RESULT and all(e.request.params.on_device for e in rows)
        if neutral:
            res = self.rt.result
            out = res[MAX_RESULT - n:MAX_RESULT]
            if all(e.request.params.greedy for e in rows):
                ops.argmax_rows(logits, out)
            else:
                temps = torch.tensor([e.request.params.temperature for e in rows], dtype=torch.float32).pin_memory()
                us = torch.tensor([0.0 if e.request.params.greedy else e.request.sampler.uniform() for e in rows],
                                  dtype=torch.float64).pin_memory()
                ops.sample_rows(logits, temps.to(logits.device, non_blocking=True), us.to(logits.device, non_blocking=True), out)
            self._ids_to_host(rec, out)
        elif n <= MAX_RESULT and self._candidates_on_device(rows, logits.shape[1]):
            # top_k, then the rest of the chain on its candidates, all on the device: the ids stay
            # there for the next step, as with the argmax
            k = next(e.request.params.top_k for e in rows if not e.request.params.greedy)
            vals, ids = ops.topk_rows(logits, k)
            params = torch.tensor([[p.top_p, log_min_p(p.min_p) if p.min_p > 0.0 else -math.inf, p.temperature]
                                   for p in (e.request.params for e in rows)], dtype=torch.float32).pin_memory()
            us = torch.tensor([0.0 if e.request.params.greedy else e.request.sampler.uniform() for e in rows], dtype=torch.float64).pin_memory()
            res = self.rt.result
            out = res[MAX_RESULT - n:MAX_RESULT]
            ops.sample_candidates(vals, ids, params.to(logits.device, non_blocking=True), us.to(logits.device, non_blocking=True), out)
            self._ids_to_host(rec, out)
        elif all(e.request.params.top_k_on_device and e.request.params.top_k == rows[0].request.params.top_k for e in rows) \
                and rows[0].request.params.top_k < logits.shape[1]:
            # bias, penalties and top_k on the device; the host runs the rest of the chain on k
            # candidates per row, not on the row (the penalties need the ids the host has seen)
            if any(e.request.params.edits_logits for e in rows):
                logits = self._apply_edits(logits, rows)
            vals, ids = ops.topk_rows(logits, rows[0].request.params.top_k)
            vals, ids = vals.cpu().numpy(), ids.cpu().numpy()
            rec["toks"] = [int(e.request.sampler.sample_candidates(ids[i], vals[i])) for i, e in enumerate(rows)]
        else:
            host_logits = logits.cpu().numpy()
            rec["toks"] = [int(e.request.sampler.sample(host_logits[i])) for i, e in enumerate(rows)]
        return rec

    def _ids_to_host(self, rec: dict, out: torch.Tensor) -> None:
        """Start the copy of the chosen ids and the status word after them to pinned memory."""
        n = out.shape[0]
        host = self._host_ring[self._host_turn % len(self._host_ring)]
        self._host_turn += 1
        host[:n + 1].copy_(self.rt.result[MAX_RESULT - n:], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        rec.update(out=out, host=host, event=ev)

    @staticmethod
    def _candidates_on_device(rows, vocab: int) -> bool:
        """Every row's chain is top_k and what follows it (or the argmax), with one k for all and
        nothing that alters the logits first."""
        ks = set()
        for e in rows:
            p = e.request.params
            if p.edits_logits:
                return False
            if p.greedy:
                continue
            if not p.top_k_on_device:
                return False
            ks.add(p.top_k)
        return len(ks) == 1 and next(iter(ks)) < vocab

    def _apply_edits(self, logits: torch.Tensor, rows) -> torch.Tensor:
        """The requests' logit biases and history penalties, applied to their rows on the device."""
        import struct

        per_row = [e.request.sampler.device_edits() for e in rows]
        stride = 2 + 2 * max(len(b) + len(h) for b, h, _ in per_row)
        edits = torch.zeros((len(rows), stride), dtype=torch.int32)
        params = torch.empty((len(rows), 3), dtype=torch.float32)
        for i, (bias, hist, pen) in enumerate(per_row):
            flat = [len(bias), len(hist)]
            for t, b in bias:
                flat += [t, struct.unpack("<i", struct.pack("<f", b))[0]]
            for t, c in hist:
                flat += [t, c]
            edits[i, :len(flat)] = torch.tensor(flat, dtype=torch.int32)
            params[i] = torch.tensor(pen, dtype=torch.float32)
        # in place: a row of logits belongs to one request and is not read again after its token is chosen
        return ops.sampler_edits(logits, edits.to(logits.device), params.to(logits.device))

    def _resolve(self, rec: dict) -> List[GenRequest]:
        """Wait for the step's ids, check the status word, and tell the scheduler."""
        rows, plan = rec["rows"], rec["plan"]
        if rec["toks"] is None:
            rec["event"].synchronize()
            got = rec["host"][:len(rows) + 1].tolist()
            toks, code = got[:-1], got[-1]
            if code:
                self.rt.status.zero_()
            self.rt.check_status(code)
        else:
            toks = rec["toks"]
            self.rt.check_status()
        # a request that an earlier step ended has a token too many in this one: not counted
        n_decode = sum(1 for e in plan if len(e.tokens) == 1 and e.sample and e.request.finish_reason is None)
        done = self.scheduler.complete(plan, {e.request.id: int(t) for e, t in zip(rows, toks)})
        if self._on_token is not None:
            # (a token too many, run ahead of the end token that finished its request, was dropped by ``complete``)
            for e, t in zip(rows, toks):
                r = e.request
                if r.generated and r.generated[-1] == int(t) and r._told < len(r.generated):
                    r._told = len(r.generated)
                    self._on_token(r.index, int(t))
        now = time.perf_counter()
        self.turn_log.append({"s": now - self._t_mark, "tokens": sum(len(e.tokens) for e in plan),
                              "decode": n_decode, "pure_decode": all(len(e.tokens) == 1 for e in plan),
                              "h2d": rec["h2d"], "d2h": 4 * len(rows) + 4})
        self._t_mark = now
        return done

    def _turn(self) -> List[GenRequest]:
        sch = self.scheduler
        prev, self._ahead = self._ahead, None
        if prev is not None:
            plan = sch.plan_ahead(prev["plan"]) if self.run_ahead else None
            if plan is not None:
                self._ahead = self._launch(plan, prev["out"])
            return self._resolve(prev)
        plan = sch.plan()
        if not plan:
            return []
        rec = self._launch(plan, None)
        if rec["out"] is not None:
            self._ahead = rec          # its ids are on their way; the next turn takes them up
            return []
        return self._resolve(rec)

    def decode_rate(self, skip: int = 0, rows: Optional[int] = None) -> dict:
        """Decoded tokens per second over the turns that held only decode tokens (the
        reference reports the same as ``predicted_per_second``, ``lua/lgml/engine.lua:3225-3239``),
        leaving out the first ``skip`` of them; with ``rows``, over the turns that decoded
        exactly that many requests (the rate at one batch size, without the turns in which
        requests that started later are still going on alone)."""
        turns = [t for t in self.turn_log if t["pure_decode"] and (rows is None or t["decode"] == rows)][skip:]
        secs = sum(t["s"] for t in turns)
        toks = sum(t["decode"] for t in turns)
        n = max(len(turns), 1)
        return {"tok_s": toks / secs if secs > 0 else 0.0, "steps": len(turns),
                "h2d_bytes_per_step": sum(t["h2d"] for t in turns) // n, "d2h_bytes_per_step": sum(t["d2h"] for t in turns) // n}

    def write_turn_csv(self, path) -> None:
        """The turns of the last ``generate`` as CSV: wall seconds of the turn, tokens run, decoded tokens,
        whether it held decoded tokens only, bytes copied each way (the reference logs the same per pass,
        ``lua/lgml/engine.lua:1488-1492``)."""
        import csv

        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["turn", "seconds", "tokens", "decoded", "pure_decode", "h2d_bytes", "d2h_bytes"])
            for i, t in enumerate(self.turn_log):
                w.writerow([i, f"{t['s']:.6f}", t["tokens"], t["decode"], int(t["pure_decode"]), t["h2d"], t["d2h"]])

    # ---- public --------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: Optional[int] = None, stop: Optional[Sequence[int]] = None,
                 seed: Optional[int] = None, return_details: bool = False, per_prompt: Optional[Sequence[dict]] = None,
                 on_token=None, **sampling):
        """Token ids in, token ids out.  ``prompts``: lists of token ids.  Sampler options
        (``temperature``, ``top_k``, ``top_p``, ``min_p``, ``repeat_penalty``,
        ``frequency_penalty``, ``presence_penalty``, ``repeat_last_n``, ``logit_bias``) and
        ``seed`` as in the sampler; request i draws from the stream of ``seed + i``.
        ``per_prompt``: one dict of sampler options per prompt that override the common ones.
        ``on_token(i, id)`` is called for every new token of prompt i as soon as the host knows it
        (the reference streams its replies the same way).
        Returns one list of new ids per prompt (with the stop id when one ends it)."""
        opts = {**self.sampling_defaults, **sampling}
        stop_ids = list(stop) if stop is not None else self.eos_ids
        reqs = []
        self._on_token = on_token
        self.turn_log = []
        t0 = self._t_mark = time.perf_counter()
        for i, p in enumerate(prompts):
            p = [int(t) for t in p]
            room = self.scheduler.max_position - len(p)
            limit = max_tokens if max_tokens is not None else (self.default_max_tokens or room)
            params = SamplingParams(seed=None if seed is None else seed + i, **({**opts, **per_prompt[i]} if per_prompt else opts))
            req = GenRequest(id=("gen", self._next_id), prompt=p, max_new_tokens=max(min(limit, room), 0), params=params,
                             stop_ids=stop_ids)
            req.index, req._told = i, 0
            self._next_id += 1
            if req.max_new_tokens == 0:
                req.finish_reason = "length"
            else:
                self.scheduler.add(req)
            reqs.append(req)
        while not self.scheduler.idle or self._ahead is not None:
            self._turn()
        torch.cuda.synchronize(self.rt.device)
        self.timings = {"total": time.perf_counter() - t0}
        if return_details:
            return reqs
        return [r.generated for r in reqs]

    def greedy(self, prompt: Sequence[int], n_predict: int, stop: Optional[Sequence[int]] = None):
        """Greedy decode of one prompt: (new ids, timings {prefill, decode, n_decode}), as
        ``generate.greedy`` (``lua/lgml/generate.lua:19-34``)."""
        runner = self.runner
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("greedy: empty prompt")
        if n_predict <= 0:
            return [], {"prefill": 0.0, "decode": 0.0, "n_decode": 0}
        req = runner.open(("greedy", self._next_id))
        self._next_id += 1
        out: List[int] = []
        tok = torch.empty(1, dtype=torch.int32, device=self.rt.device)
        stop = set(stop or ())
        try:
            t0 = time.perf_counter()
            ids = prompt
            pos = 0
            while pos < len(ids):          # the prompt in portions of ubatch
                part = ids[pos:pos + self.scheduler.ubatch]
                pos += len(part)
                logits = runner.step([(req, part, [len(part) - 1] if pos == len(ids) else [])])
            cur = int(ops.argmax_rows(logits, tok).item())
            t1 = time.perf_counter()
            out.append(cur)
            while len(out) < n_predict and cur not in stop:
                logits = runner.step([(req, [cur], [0])])
                cur = int(ops.argmax_rows(logits, tok).item())
                out.append(cur)
            t2 = time.perf_counter()
            self.rt.check_status()
        finally:
            runner.close(req)
        return out, {"prefill": t1 - t0, "decode": t2 - t1, "n_decode": len(out) - 1}
