"""Decode steps (one token per request), and one request's short portions, as replays of a captured CUDA graph.

A graph is captured per batch size.  Its kernels were recorded with fixed addresses, so the
step's description lives in one device buffer per batch size, laid out as ``StepBatch`` lays
it out, with block tables of a fixed width; a step refreshes that buffer with one copy from
pinned memory and replays.  The host side keeps a NumPy image of the buffer and rewrites only
what changes from step to step (tokens, positions, and the table rows of requests that took a
page), because at batch 1 the host's work per step is comparable to the GPU's.

The reference keeps its last graph per cache and refills the input leaves when the pass has
the same shape (``lua/lgml/replay.lua:152-216``, key ``M:batch_key``
``lua/lgml/transformer.lua:2560-2572``); this is the same idea with CUDA graphs.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from .batch import CacheView, StepBatch
from .runtime import AHEAD_MAX_BATCH


class DecodeBatch:
    """The batch description of a captured decode step: the same attributes as ``StepBatch``,
    as views of a device buffer that stays put."""

    def __init__(self, cache_manager, S: int, widths: Sequence[int], device, reach: Optional[int] = None):
        cm = self.cache_manager = cache_manager
        self.n_tokens = self.n_seqs = self.n_rows = S
        self.widths = list(widths)
        self.seq_lens = [1] * S
        self.max_q_len = 1
        # the longest context the captured step describes: every mixer cuts its keys into ranges
        # for this length and its own heads, so a replay launches what the capture recorded
        self.max_kv_len = max(self.widths, default=1) * cm.page_size
        if reach:
            self.max_kv_len = min(self.max_kv_len, reach)       # the longest context of the steps this graph replays
        self.decode_splits = None
        total = 3 * S + (S + 1) + 4 * S + S * sum(self.widths)
        self.total = total
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.host = np.zeros(total, dtype=np.int32)
        off = 0

        def take(n):
            nonlocal off
            sl = slice(off, off + n)
            off += n
            return sl

        self.sl_tokens, self.sl_pos, self.sl_seq_of = take(S), take(S), take(S)
        self.sl_start, self.sl_pos0, self.sl_slots, self.sl_kv, self.sl_rows = take(S + 1), take(S), take(S), take(S), take(S)
        self.sl_tables = [take(S * w) for w in self.widths]
        self.host[self.sl_seq_of] = np.arange(S)
        self.host[self.sl_start] = np.arange(S + 1)
        self.host[self.sl_rows] = np.arange(S)
        for sl in self.sl_tables:
            self.host[sl] = -1
        d = self.dev
        self.token_ids, self.positions, self.seq_of_token = d[self.sl_tokens], d[self.sl_pos], d[self.sl_seq_of]
        self.seq_start, self.seq_pos0, self.slots, self.seq_kv_len = d[self.sl_start], d[self.sl_pos0], d[self.sl_slots], d[self.sl_kv]
        self.logit_rows = d[self.sl_rows]
        self.block_tables = [d[sl].view(S, w) for sl, w in zip(self.sl_tables, self.widths)]
        self._seen: List[Optional[tuple]] = [None] * S      # per row: (request, pages per group) last written
        self.requests: List = []
        self.h2d_bytes = total * 4

    def fill(self, requests, tokens: Optional[Sequence[int]]) -> None:
        """Write this step into the host image.  ``tokens`` None leaves the token ids alone
        (they are then copied on the device)."""
        h, S = self.host, self.n_seqs
        self.requests = list(requests)
        pos = [r.n_tokens for r in requests]
        h[self.sl_pos] = pos
        h[self.sl_pos0] = pos
        h[self.sl_kv] = [p + 1 for p in pos]
        if tokens is not None:
            h[self.sl_tokens] = tokens
        for s, r in enumerate(requests):
            key = (id(r), tuple(len(t) for t in r.tables))
            if self._seen[s] == key:
                continue
            self._seen[s] = key
            h[self.sl_slots.start + s] = r.slot
            for g, (sl, w) in enumerate(zip(self.sl_tables, self.widths)):
                row = r.tables[g]
                if len(row) > w:
                    raise ValueError(f"request {r.id!r} holds {len(row)} pages, the captured step describes at most {w}")
                base = sl.start + s * w
                h[base:base + len(row)] = row
                h[base + len(row):base + w] = -1
        self.pos0 = pos
        self.kv_lens = [p + 1 for p in pos]

    def invalidate(self) -> None:
        """Forget what the rows held (a window group rewrites old table entries in place)."""
        self._seen = [None] * self.n_seqs

    def cache_view(self, owner: int, writable: bool = True) -> CacheView:
        cm = self.cache_manager
        g = cm.group_of_layer.get(owner)
        if g is not None:
            grp = cm.groups[g]
            return CacheView(k=grp.k[owner], v=grp.v[owner], block_table=self.block_tables[g], writable=writable,
                             page_size=cm.page_size)
        sg = cm.state_group_of_layer.get(owner)
        if sg is not None:
            return CacheView(state=cm.state_groups[sg].state[owner], writable=writable)
        return CacheView(writable=False)


class DecodeGraph:
    """One captured decode step of a fixed batch size."""

    RING = 4

    def __init__(self, runner, S: int, reach: Optional[int] = None):
        self.runner = runner
        self.S = S
        self.batch = DecodeBatch(runner.cache, S, runner._graph_widths, runner.rt.device, reach=reach)
        self.pinned = [torch.empty(self.batch.total, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.pinned_np = [p.numpy() for p in self.pinned]
        self.events: List[Optional[torch.cuda.Event]] = [None] * self.RING
        self.turn = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels = 0
        self.has_window = any(g.spec.window is not None for g in runner.cache.groups)

    def run(self, requests, tokens: Optional[Sequence[int]], device_tokens: Optional[torch.Tensor]) -> torch.Tensor:
        """Replay for ``requests`` (at most S of them; the spare rows repeat the last one).  Returns
        the logits of all S rows: the caller keeps the first ``len(requests)``."""
        b = self.batch
        n, spare = len(requests), self.S - len(requests)
        if spare:
            requests = list(requests) + [requests[-1]] * spare
            if tokens is not None:
                tokens = list(tokens) + [tokens[-1]] * spare
        if self.has_window:
            b.invalidate()
        b.fill(requests, tokens)
        i = self.turn % self.RING
        self.turn += 1
        if self.events[i] is not None:
            self.events[i].synchronize()          # the copy that last used this staging buffer has run
        self.pinned_np[i][:] = b.host
        b.dev.copy_(self.pinned[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        if device_tokens is not None:
            b.token_ids[:n].copy_(device_tokens)
            if spare:
                b.token_ids[n:].copy_(device_tokens[n - 1:].expand(spare))
        if self.graph is None:
            # Nothing but the step's own launches may touch CUDA while the stream is capturing:
            # a finaliser that frees device or pinned memory in the middle (Python's collector
            # can run at any allocation) would invalidate the capture.  So collect first, keep
            # the collector off during the capture, and let the capture tolerate such calls.
            import gc

            gc.collect()
            was_on = gc.isenabled()
            gc.disable()
            try:
                g = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                rt = self.runner.rt
                ahead = rt.dtype == torch.bfloat16 and self.S <= AHEAD_MAX_BATCH
                rt.side = torch.cuda.Stream() if ahead else None
                try:
                    with torch.cuda.graph(g, capture_error_mode="relaxed"):
                        self.logits = self.runner.model.forward(rt, b)
                        rt.join()
                finally:
                    rt.side = None
                self.kernels = ops.launch_count() - before
                self.graph = g
            finally:
                if was_on:
                    gc.enable()
        self.graph.replay()
        return self.logits


class PromptGraph:
    """One captured step for a portion of one request: ``n_tokens`` tokens (16, 32 or a whole
    number of pages) that start on a page's edge, ``n_rows`` wanted logits rows (0 or 1).

    A short prompt's step is bound by the host (hundreds of launches for a few milliseconds of
    GPU work), so it is replayed like a decode step.  A portion is padded with token 0 to that
    length: the padded tokens come after the real ones, no real token looks at them (they
    lie in the future), and the cells they write in the portion's last page, which the request
    holds anyway, are written again by the tokens that really come there before anything reads
    them.  The step's description lives in one device buffer as ``StepBatch`` lays it out, with
    block tables of a fixed width; a replay refreshes it with one copy from pinned memory."""

    def __init__(self, runner, n_tokens: int, n_rows: int):
        self.runner, self.n_tokens, self.n_rows = runner, n_tokens, n_rows
        self.widths = list(runner._graph_widths)
        total = StepBatch.buffer_ints(n_tokens, 1, n_rows, self.widths)
        self.dev = torch.zeros(total, dtype=torch.int32, device=runner.rt.device)
        self.tiles = {}                 # the attention kernels' tile lists: they depend on the shape only
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels = 0

    def run(self, req, tokens: Sequence[int], want: Sequence[int], pinned: torch.Tensor) -> StepBatch:
        """Launch the step; returns the batch (``.logits`` of this object holds the result)."""
        pad = self.n_tokens - len(tokens)
        batch = StepBatch(self.runner.cache, [req], [list(tokens) + [0] * pad], [list(want)], self.runner.rt.device, pinned,
                          table_widths=self.widths, device_buffer=self.dev)
        batch._tiles = self.tiles
        batch.after_staged_copy = None
        if self.graph is None:
            import gc

            rt = self.runner.rt
            self.runner.model.forward(rt, batch)            # eagerly once: kernels loaded, tile lists made (no copy inside the capture)
            gc.collect()
            was_on = gc.isenabled()
            gc.disable()
            try:
                g = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                with torch.cuda.graph(g, capture_error_mode="relaxed"):
                    self.logits = self.runner.model.forward(rt, batch)
                self.kernels = ops.launch_count() - before
                self.graph = g
            finally:
                if was_on:
                    gc.enable()
        self.graph.replay()
        return batch
