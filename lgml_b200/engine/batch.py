"""The description of one step's batch, as the kernels read it.

A step holds, for each request in it, that request's next tokens: a prompt, a
portion of one, or a single decoded token.  All tokens of the step form one
ragged batch (mischief/lgml: ``M:batch_inputs``, ``lua/lgml/transformer.lua:2502-2551``):

* ``token_ids[N]``, ``positions[N]`` (= tokens already cached + index in the portion,
  ``:2441-2447``), ``seq_of_token[N]`` (the row of the request in this batch),
* ``seq_start[S+1]`` (first token of each request), ``seq_pos0[S]``, ``slots[S]``,
* one block table ``[S, width]`` per cache group, -1 where a request has no page,
* ``logit_rows[R]``: the token rows whose logits are wanted (``:2540-2545``).

Everything goes to the device in one copy from pinned memory; no dense mask is
built (the reference fills an (n, window) mask on the host each pass,
``src/lgml.c:2993-3010``; here the attention kernel walks the block table).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class CacheView:
    """What one layer call sees of the cache."""

    k: Optional[torch.Tensor] = None            # [pages, Hkv, page, D]
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None  # int32 [S, width]
    writable: bool = True
    state: Optional[torch.Tensor] = None        # [max_slots, ...] for a fixed-state layer
    page_size: int = 0


class StepBatch:
    """Host lists -> one int32 buffer -> one copy -> device views.

    ``table_widths`` forces the width of each group's block table and ``device_buffer``
    makes the views live in a buffer the caller keeps: both are what a captured CUDA graph
    needs, since its kernels were recorded with fixed addresses and strides."""

    def __init__(self, cache_manager, requests: Sequence, tokens: Sequence[Sequence[int]], want: Sequence[Sequence[int]],
                 device, pinned: Optional[torch.Tensor] = None, table_widths: Optional[Sequence[int]] = None,
                 device_buffer: Optional[torch.Tensor] = None):
        cm = cache_manager
        self.cache_manager = cm
        self.requests = list(requests)
        S = len(self.requests)
        lens = [len(t) for t in tokens]
        N = sum(lens)
        self.n_tokens, self.n_seqs = N, S
        self.seq_lens = lens
        self.pos0 = [r.n_tokens for r in self.requests]
        self.kv_lens = [p + n for p, n in zip(self.pos0, lens)]
        self.max_q_len = max(lens) if lens else 0
        self.max_kv_len = max(self.kv_lens) if lens else 0
        self.decode_splits = None       # a fixed split count (set by a captured graph)
        self._tiles = {}
        self.after_staged_copy = None   # called after a later copy out of the pinned buffer (its owner marks the buffer busy again)

        # Everything below is array arithmetic: a prompt portion brings thousands of tokens, and a
        # Python loop over them would cost as much as the step's first layers.
        tok_arrays = [np.asarray(t, dtype=np.int64).reshape(-1) for t in tokens]
        lens_a = np.asarray(lens, dtype=np.int64)
        starts = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(lens_a, out=starts[1:])
        rows: List[int] = []
        self.rows_of_seq: List[List[int]] = []
        for s, w in enumerate(want):
            mine = []
            for i in w:
                if not 0 <= i < lens[s]:
                    raise IndexError(f"wanted place {i} is outside the {lens[s]} tokens request {self.requests[s].id!r} brings")
                mine.append(len(rows))
                rows.append(int(starts[s]) + int(i))
            self.rows_of_seq.append(mine)
        self.n_rows = len(rows)

        tables = []
        for g in range(len(cm.groups)):
            tables.append(cm.block_table_rows(self.requests, g, table_widths[g] if table_widths else None))
        self.table_width = [len(t[0]) if t else 1 for t in tables]
        n_rows_field = max(len(rows), 1)
        total = 3 * N + (S + 1) + 3 * S + n_rows_field + S * sum(self.table_width)
        if pinned is not None and pinned.numel() >= total:
            host = pinned[:total]
            self._pinned, self._pinned_used = pinned, total
        else:
            host = torch.empty(total, dtype=torch.int32)
            self._pinned, self._pinned_used = None, 0
        h = host.numpy()
        seq_of = np.repeat(np.arange(S, dtype=np.int64), lens_a)
        off = 0
        h[off:off + N] = np.concatenate(tok_arrays) if S else 0
        off += N
        # position of token j of request s: its first position + j
        h[off:off + N] = np.asarray(self.pos0, dtype=np.int64)[seq_of] + (np.arange(N, dtype=np.int64) - starts[seq_of]) if N else 0
        off += N
        h[off:off + N] = seq_of
        off += N
        h[off:off + S + 1] = starts
        off += S + 1
        h[off:off + S] = self.pos0
        off += S
        h[off:off + S] = [r.slot for r in self.requests]
        off += S
        h[off:off + S] = self.kv_lens
        off += S
        h[off:off + n_rows_field] = rows or [0]
        off += n_rows_field
        for t, w in zip(tables, self.table_width):
            if S:
                h[off:off + S * w] = np.asarray(t, dtype=np.int64).reshape(-1)
            off += S * w
        if device_buffer is not None:
            if device_buffer.numel() < total:
                raise ValueError("the step's description does not fit the buffer kept for it")
            dev = device_buffer[:total]
        else:
            dev = torch.empty(total, dtype=torch.int32, device=device)
        dev.copy_(host, non_blocking=True)
        self.h2d_bytes = total * 4
        self._dev = dev
        off = 0

        def take(n):
            nonlocal off
            v = dev[off:off + n]
            off += n
            return v

        self.token_ids = take(N)
        self.positions = take(N)
        self.seq_of_token = take(N)
        self.seq_start = take(S + 1)
        self.seq_pos0 = take(S)
        self.slots = take(S)
        self.seq_kv_len = take(S)
        r = take(max(len(rows), 1))
        self.logit_rows = r[: len(rows)]
        self.block_tables = [take(S * w).view(S, w) for w in self.table_width]

    def attention_tiles(self, tile_tokens: int) -> torch.Tensor:
        """The new tokens cut into tiles of at most ``tile_tokens`` consecutive tokens of one
        request, for the prefill attention kernel: int32 [n_tiles, 4] on the device, rows
        (request row, first token row, tokens, 0), the tile with the most keys to visit first:
        the kernel starts its CTAs in this order, and a long tile that starts last would run on
        alone at the end.  Made once per tile size."""
        cached = self._tiles.get(tile_tokens)
        if cached is None:
            rows = []
            start = 0
            for s, n in enumerate(self.seq_lens):
                for t0 in range(0, n, tile_tokens):
                    rows.append((s, start + t0, min(tile_tokens, n - t0), self.pos0[s] + min(t0 + tile_tokens, n)))
                start += n
            rows.sort(key=lambda r: -r[3])
            arr = np.asarray(rows, dtype=np.int32).reshape(-1, 4)
            arr[:, 3] = 0
            n_ints = arr.size
            dev = self.token_ids.device
            if self._pinned is not None and self._pinned.numel() >= self._pinned_used + n_ints:
                # the rest of the step's staging buffer: no copy has to wait for pageable memory
                stage = self._pinned[self._pinned_used:self._pinned_used + n_ints]
                self._pinned_used += n_ints
                stage.numpy()[:] = arr.reshape(-1)
                cached = torch.empty(n_ints, dtype=torch.int32, device=dev)
                cached.copy_(stage, non_blocking=True)
                cached = cached.view(-1, 4)
                if self.after_staged_copy is not None:
                    self.after_staged_copy()
            else:
                cached = torch.from_numpy(arr).to(dev)
            self._tiles[tile_tokens] = cached
        return cached

    @staticmethod
    def buffer_ints(n_tokens: int, n_seqs: int, n_rows: int, table_widths: Sequence[int]) -> int:
        return 3 * n_tokens + (n_seqs + 1) + 3 * n_seqs + max(n_rows, 1) + n_seqs * sum(table_widths)

    def cache_view(self, owner: int, writable: bool = True) -> CacheView:
        """The cache of schedule entry ``owner`` as this batch's requests see it."""
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
