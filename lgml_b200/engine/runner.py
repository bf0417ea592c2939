"""The step function: run one batch of (request, its next tokens) from the cache.

``ModelRunner.step`` is the only way tokens go through the model; generation, the
scheduler and trace replay all call it.  It runs exactly the tokens it is given, as
one batch, on the cache that earlier steps left, writes their keys and values,
advances the requests, and returns float32 logits at the wanted places
(mischief/lgml: ``M:run_batch``, ``lua/lgml/transformer.lua:2585-2624``: several
sequences, "one id for a decode step, or a chunk of a prompt", ``:2493-2494``;
positions advance after the pass, ``:2620-2622``).
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import CacheManager, PoolFull, Request
from ..models import build_model
from ..weights import load_tensors, random_tensors
from .batch import StepBatch
from .runtime import Runtime


MAX_GRAPH_BATCH = 256
PROMPT_GRAPH_TOKENS = 256      # portions of one request up to this length are replayed from captured graphs
# Batch sizes that decode steps are captured at.  A step of another size runs the next larger
# graph with its last request repeated in the spare rows: those rows compute the same token at
# the same position again (the same key and value into the same cell) and their logits are
# dropped.  Requests that end one after the other would otherwise cost a capture per size.
GRAPH_SIZES = [1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16, 20, 24, 28, 32, 40, 48, 56, 64, 80, 96, 112, 128, 160, 192, 224, 256]


def graph_size(n: int) -> int:
    for s in GRAPH_SIZES:
        if s >= n:
            return s
    return n


def prompt_graph_length(n: int, page: int) -> int:
    """The number of tokens a short portion of n tokens is padded to for its captured step: 16 or
    32 inside the first page (the products' narrower tiles), else the next page's edge."""
    for small in (16, 32):
        if n <= small < page:
            return small
    return -(-n // page) * page


class StepError(ValueError):
    """A step the runner refuses before anything is launched."""


class ModelRunner:
    def __init__(self, model, rt: Runtime, n_pages: int, max_slots: int = 4, max_step_tokens: int = 0, use_graphs: bool = True,
                 prefix_cache: bool = False):
        self.model = model
        self.rt = rt
        self.cache = CacheManager(model.cache_layout(), n_pages=n_pages, max_slots=max_slots, dtype=rt.dtype,
                                  device=rt.device, max_step_tokens=max_step_tokens, prefix_cache=prefix_cache)
        # a ring of pinned staging buffers: a buffer is reused only after its copy has run
        self._pinned = [[torch.empty(1 << 16, dtype=torch.int32).pin_memory(), None] for _ in range(4)]
        self.steps = 0
        self.tokens_run = 0
        # decode steps (one token per request) replay a CUDA graph captured per batch size
        self.use_graphs = use_graphs and getattr(model, "graph_safe", False)
        self._graphs = {}
        self._prompt_graphs = {}
        self._graph_seen = set()
        max_pos = model.max_position or (n_pages * self.cache.page_size)
        self._graph_widths = [min(g.pool.n_pages, -(-max_pos // self.cache.page_size)) for g in self.cache.groups]
        self.graph_replays = 0

    # ---- construction ------------------------------------------------------------------
    @classmethod
    def from_folder(cls, folder, dtype: torch.dtype, device="cuda:0", **kw) -> "ModelRunner":
        from ..config import load_config

        cfg = load_config(folder)
        rt = Runtime(device, dtype)
        model = build_model(cfg)
        tensors = load_tensors(folder, model.tensor_specs(), dtype, rt.device, ignore=getattr(model, "ignored_tensors", ()))
        model.bind(tensors, rt)
        return cls(model, rt, **kw)

    @classmethod
    def from_config(cls, cfg, seed: int, dtype: torch.dtype, device="cuda:0", std: float = 0.02, on_device: bool = True,
                    **kw) -> "ModelRunner":
        """Random weights without a folder: drawn on the device, or on the host; either way
        the values of ``write_random_model(folder, cfg, seed)``, bit for bit (one generator)."""
        from .. import ops
        from ..weights.loader import target_dtype
        from ..weights.random_init import tensor_key

        rt = Runtime(device, dtype)
        model = build_model(cfg)
        specs = [s for s in model.tensor_specs() if not s.optional]
        if on_device:
            tensors = {}
            for s in specs:
                t = torch.empty(s.shape, dtype=target_dtype(s.kind, dtype), device=rt.device)
                ops.fill_normal(t, s.init[0], s.init[1] * std, tensor_key(seed, s.name))
                tensors[s.name] = t
        else:
            host = random_tensors(specs, seed, std)
            tensors = {s.name: host[s.name].to(device=rt.device, dtype=target_dtype(s.kind, dtype)) for s in specs}
        model.bind(tensors, rt)
        return cls(model, rt, **kw)

    @staticmethod
    def _mark_busy(stage) -> None:
        """The copies out of this staging buffer queued so far must run before it is written again."""
        stage[1] = torch.cuda.Event()
        stage[1].record()

    # ---- requests ----------------------------------------------------------------------
    def open(self, rid: Hashable, tokens: Optional[Sequence[int]] = None) -> Request:
        """A slot for a new request; with the prefix cache on and its tokens given, it starts
        behind what the cache already holds of them (``Request.n_tokens``)."""
        return self.cache.open(rid, tokens)

    def close(self, req: Request) -> None:
        self.cache.close(req)

    # ---- the step ----------------------------------------------------------------------
    def validate(self, entries: Sequence[Tuple[Request, Sequence[int], Sequence[int]]]) -> None:
        seen = set()
        vocab = self.model.vocab_size
        max_pos = self.model.max_position
        if not entries:
            raise StepError("a step needs at least one entry")
        for req, tokens, want in entries:
            if req.closed:
                raise StepError(f"request {req.id!r} is closed")
            if id(req) in seen:
                raise StepError(f"request {req.id!r} appears twice in one step")
            seen.add(id(req))
            if len(tokens) == 0:
                raise StepError(f"request {req.id!r} brings no tokens")
            if len(tokens) > 16:
                arr = np.asarray(tokens, dtype=np.int64)
                bad = np.nonzero((arr < 0) | (arr >= vocab))[0]
                if bad.size:
                    raise StepError(f"request {req.id!r}: token id {int(arr[bad[0]])} is outside the vocabulary of {vocab}")
            else:
                for t in tokens:
                    if not 0 <= int(t) < vocab:
                        raise StepError(f"request {req.id!r}: token id {t} is outside the vocabulary of {vocab}")
            for i in want:
                if not 0 <= int(i) < len(tokens):
                    raise StepError(f"request {req.id!r}: wanted place {i} is outside the {len(tokens)} tokens it brings")
            if max_pos is not None and req.n_tokens + len(tokens) > max_pos:
                raise StepError(f"request {req.id!r}: context full ({req.n_tokens} + {len(tokens)} tokens > {max_pos} positions)")

    def _reserve_all(self, wanted: Sequence[Tuple[Request, int]]) -> None:
        """Pages for every entry of a step, or for none: when one entry finds no page, the
        entries before it give back what they took in this call, so that a step that fails
        leaves the pool and every block table as they were (the reference fails such a step
        alone, ``lua/lgml/engine.lua:1436-1448``)."""
        failed = self.cache.reserve_all(wanted)
        if failed is not None:
            req, n = wanted[failed]
            raise PoolFull(f"kv pool full: request {req.id!r} needs pages for {n} more tokens, "
                           f"{self.cache.n_free_pages} of {self.cache.n_pages} pages are free")

    def step(self, entries: Sequence[Tuple[Request, Sequence[int], Sequence[int]]]) -> torch.Tensor:
        """entries: (request, its next tokens, the places among them whose logits are
        wanted).  Returns float32 [wanted, vocab] in the order of entries and places."""
        self.validate(entries)
        self._reserve_all([(req, len(tokens)) for req, tokens, _ in entries])
        stage = self._pinned[self.steps % len(self._pinned)]
        if stage[1] is not None:
            stage[1].synchronize()
        S = len(entries)
        if self._graphs_now() and all(len(e[1]) == 1 for e in entries) and S <= MAX_GRAPH_BATCH:
            logits = self._graph_step(entries, stage)
        elif self._graphs_now() and self._prompt_graph_fits(entries):
            logits = self._prompt_graph_step(entries[0], stage)
        else:
            batch = StepBatch(self.cache, [e[0] for e in entries], [e[1] for e in entries], [e[2] for e in entries],
                              self.rt.device, stage[0])
            self._mark_busy(stage)
            batch.after_staged_copy = lambda: self._mark_busy(stage)
            self.last_batch = batch
            logits = self.model.forward(self.rt, batch)
        for req, tokens, _ in entries:
            self.cache.commit(req, len(tokens))
        self.steps += 1
        self.tokens_run += sum(len(e[1]) for e in entries)
        return logits

    def _graphs_now(self) -> bool:
        """Captured graphs, unless the kernels are being timed one by one (a replay would hide them)."""
        from .. import ops
        return self.use_graphs and ops.KernelTimes.active is None

    def graph_kernels(self, batch_size: int) -> int:
        """Launches of this package's kernels that one replay of the graph for ``batch_size`` requests holds."""
        size = graph_size(batch_size)
        return max((g.kernels for (s, _), g in self._graphs.items() if s == size), default=0)

    def _prompt_graph_fits(self, entries) -> bool:
        """A short portion of one request that starts on a page's edge and wants no logits or
        those of its last token: such a step is replayed from a captured graph (a prompt of a few
        dozen tokens is bound by the host otherwise).  Models with windows or per-request state
        are left out: a padded token would move their window or their state."""
        if len(entries) != 1:
            return False
        req, tokens, want = entries[0]
        n, page = len(tokens), self.cache.page_size
        if not 2 <= n <= PROMPT_GRAPH_TOKENS or req.n_tokens % page or list(want) not in ([], [n - 1]):
            return False
        if self.cache.state_groups or any(g.spec.window is not None for g in self.cache.groups):
            return False
        padded = prompt_graph_length(n, page)
        limit = self.model.max_position or (self.cache.n_pages * page)
        return req.n_tokens + padded <= min(limit, self._graph_widths[0] * page if self._graph_widths else limit)

    def _prompt_graph_step(self, entry, stage) -> torch.Tensor:
        from .graph import PromptGraph

        req, tokens, want = entry
        page = self.cache.page_size
        key = (prompt_graph_length(len(tokens), page), len(want))
        g = self._prompt_graphs.get(key)
        if g is None:
            g = self._prompt_graphs[key] = PromptGraph(self, key[0], key[1])
        else:
            self.graph_replays += 1
        self.last_batch = g.run(req, tokens, want, stage[0])
        self._mark_busy(stage)
        return g.logits

    def _graph_step(self, entries, stage, device_tokens=None) -> torch.Tensor:
        """A decode step through a captured graph.  The first step of a kind (batch size, reach of
        the context) runs eagerly (it also loads the kernels); the second captures; later ones
        replay.  The graph computes the logits of every token; the wanted rows are picked after it."""
        from .graph import DecodeGraph

        n = len(entries)
        # (a mixer with state of its own would count a repeated row twice: such a model gets a graph per size)
        size = graph_size(n) if not self.cache.state_groups else n
        reqs = [e[0] for e in entries]
        # A graph fixes into how many key ranges attention cuts a request's context, and that number is
        # chosen for a context length: so a graph per power of two of the longest context in the step
        # (from 1,024 tokens up), or a pool of 128k tokens would cut a 2k context into ranges of a page.
        longest = max(r.n_tokens for r in reqs) + 1
        reach = 1024
        while reach < longest:
            reach *= 2
        key = (size, reach)
        if key not in self._graph_seen:
            self._graph_seen.add(key)
            toks = [e[1] for e in entries]
            if device_tokens is not None:
                toks = [[int(t)] for t in device_tokens.cpu().tolist()]
            batch = StepBatch(self.cache, reqs, toks, [e[2] for e in entries], self.rt.device, stage[0])
            stage[1] = torch.cuda.Event()
            stage[1].record()
            self.last_batch = batch
            return self.model.forward(self.rt, batch)
        g = self._graphs.get(key)
        if g is None:
            g = self._graphs[key] = DecodeGraph(self, size, reach=reach)
        logits = g.run(reqs, None if device_tokens is not None else [e[1][0] for e in entries], device_tokens)[:n]
        self.last_batch = g.batch
        self.graph_replays += 1
        if all(len(e[2]) == 1 for e in entries):
            return logits
        want_rows = [i for i, e in enumerate(entries) for _ in e[2]]
        if not want_rows:
            return logits[:0]
        return logits[torch.tensor(want_rows, dtype=torch.long, device=logits.device)]

    def decode_step(self, requests: Sequence[Request], device_tokens: torch.Tensor) -> torch.Tensor:
        """One decode step whose token ids are already on the device (int32, one per request),
        for example the output of the sampling kernel of the step before: the host need not
        see the tokens before the next step is launched.  Ids out of the vocabulary are
        caught by the embedding kernel (status 1) instead of the host.  Returns the logits of
        every request's token."""
        if device_tokens.dtype != torch.int32 or device_tokens.numel() != len(requests) or not device_tokens.is_cuda:
            raise StepError("decode_step takes one int32 token id per request, on the device")
        entries = [(r, [0], [0]) for r in requests]
        self.validate(entries)
        self._reserve_all([(r, 1) for r in requests])
        stage = self._pinned[self.steps % len(self._pinned)]
        if stage[1] is not None:
            stage[1].synchronize()
        if self._graphs_now() and len(requests) <= MAX_GRAPH_BATCH:
            logits = self._graph_step(entries, stage, device_tokens=device_tokens)
        else:
            toks = [[int(t)] for t in device_tokens.cpu().tolist()]
            batch = StepBatch(self.cache, list(requests), toks, [[0]] * len(requests), self.rt.device, stage[0])
            stage[1] = torch.cuda.Event()
            stage[1].record()
            self.last_batch = batch
            logits = self.model.forward(self.rt, batch)
        for r in requests:
            self.cache.commit(r, 1)
        self.steps += 1
        self.tokens_run += len(requests)
        return logits
