"""The cache manager: paged keys and values, block tables, per-request state slots.

What a layer's mixer needs from the cache is a ``CacheSpec``.  Layers with equal
paged needs form a *group*; a group has its own pool of pages (one page id is
valid in every layer of the group, as a cell index is in mischief/lgml's pool,
``lua/lgml/transformer.lua:690-698``), and a request has one block table per
group: table[b] is the page that holds positions [b * page, (b + 1) * page)
(``:1126-1133``).  A group that keeps only a window of keys gives a page back
once every position in it is out of reach of all later queries.  Beside the
pages there are slots of fixed size for per-request state (recurrent state and
the like; ``:583-600``): one slot per live request, zeroed when the request
starts (``:1549-1559``).  Llama registers one paged group and no state.

Pages are taken before a step for the positions it will write
(``check_pass`` -> ``grow`` -> ``reserve``, ``:1543``, ``:963-981``) and given
back when the request ends (``free_seq``, ``:784-803``) or a window has passed
them.  All of the pool exists from the start (``kv_initial = 0``,
``lua/lgml/engine.lua:397-399``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from .pages import PagePool, PoolFull

PAGE_SIZE = 64  # tokens per page: BLOCK of lua/lgml/transformer.lua:30


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every position (window None) or of the last ``window``."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request: one tensor of ``shape`` and ``dtype`` per layer."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class NoSlot(RuntimeError):
    """Every request slot is taken."""


@dataclass
class PagedGroup:
    spec: PagedKV
    layers: List[int]
    pool: PagePool
    k: Dict[int, torch.Tensor] = field(default_factory=dict)  # layer -> [n_pages, Hkv, page, D]
    v: Dict[int, torch.Tensor] = field(default_factory=dict)


@dataclass
class StateGroup:
    spec: FixedState
    layers: List[int]
    state: Dict[int, torch.Tensor] = field(default_factory=dict)  # layer -> [max_slots, *shape]


class Request:
    """What one live request holds in the cache."""

    def __init__(self, rid: Hashable, slot: int, n_groups: int):
        self.id = rid
        self.slot = slot
        self.n_tokens = 0                                  # positions written so far
        self.tables: List[List[int]] = [[] for _ in range(n_groups)]  # page per block, -1 once given back
        self.closed = False


class CacheManager:
    """Owns the pages, the block tables and the state slots of all live requests.

    ``layout`` maps a layer index to its ``CacheSpec`` (layers without a cache of their
    own are absent).  ``n_pages`` is the size of each full-attention group's pool;
    a window group gets what ``max_slots`` requests can hold at once.
    """

    def __init__(self, layout: Dict[int, object], n_pages: int, max_slots: int, dtype: torch.dtype, device,
                 page_size: int = PAGE_SIZE, max_step_tokens: int = 0):
        if max_slots <= 0:
            raise ValueError("max_slots must be positive")
        self.page_size = page_size
        self.max_slots = max_slots
        self.device = torch.device(device)
        self.dtype = dtype
        self.groups: List[PagedGroup] = []
        self.state_groups: List[StateGroup] = []
        self.group_of_layer: Dict[int, int] = {}
        self.state_group_of_layer: Dict[int, int] = {}
        by_spec: Dict[object, int] = {}
        for layer in sorted(layout):
            spec = layout[layer]
            if isinstance(spec, PagedKV):
                if spec not in by_spec:
                    pages = n_pages
                    if spec.window is not None:
                        # a request holds at most the window plus one step's tokens, rounded out to pages
                        span = spec.window + (max_step_tokens or page_size)
                        pages = min(n_pages, max_slots * (-(-span // page_size) + 1))
                    by_spec[spec] = len(self.groups)
                    self.groups.append(PagedGroup(spec, [], PagePool(pages)))
                g = by_spec[spec]
                self.groups[g].layers.append(layer)
                self.group_of_layer[layer] = g
            elif isinstance(spec, FixedState):
                key = ("state", spec)
                if key not in by_spec:
                    by_spec[key] = len(self.state_groups)
                    self.state_groups.append(StateGroup(spec, []))
                g = by_spec[key]
                self.state_groups[g].layers.append(layer)
                self.state_group_of_layer[layer] = g
            elif spec is not None:
                raise TypeError(f"layer {layer}: unknown cache spec {spec!r}")
        for grp in self.groups:
            shape = (grp.pool.n_pages, grp.spec.n_kv_heads, page_size, grp.spec.head_dim)
            for layer in grp.layers:
                grp.k[layer] = torch.zeros(shape, dtype=dtype, device=self.device)
                grp.v[layer] = torch.zeros(shape, dtype=dtype, device=self.device)
        for sg in self.state_groups:
            for layer in sg.layers:
                sg.state[layer] = torch.zeros((max_slots,) + tuple(sg.spec.shape), dtype=sg.spec.dtype, device=self.device)
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self.live: Dict[Hashable, Request] = {}

    # ---- sizes -------------------------------------------------------------------------
    def pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    @property
    def n_free_pages(self) -> int:
        """Free pages of the tightest full-attention group (the scheduler's budget)."""
        full = [g.pool.n_free for g in self.groups if g.spec.window is None]
        return min(full) if full else min((g.pool.n_free for g in self.groups), default=1 << 30)

    @property
    def n_pages(self) -> int:
        full = [g.pool.n_pages for g in self.groups if g.spec.window is None]
        return min(full) if full else min((g.pool.n_pages for g in self.groups), default=1 << 30)

    def bytes_held(self) -> int:
        n = 0
        for g in self.groups:
            n += sum(t.numel() * t.element_size() for t in g.k.values()) * 2
        for sg in self.state_groups:
            n += sum(t.numel() * t.element_size() for t in sg.state.values())
        return n

    # ---- requests ----------------------------------------------------------------------
    def open(self, rid: Hashable) -> Request:
        if rid in self.live:
            raise ValueError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise NoSlot(f"all {self.max_slots} request slots are taken")
        slot = self._free_slots.pop()
        req = Request(rid, slot, len(self.groups))
        for sg in self.state_groups:
            for t in sg.state.values():
                t[slot].zero_()
        self.live[rid] = req
        return req

    def _first_needed_block(self, grp: PagedGroup, n_tokens: int) -> int:
        """Lowest block that a query at position >= n_tokens can still reach."""
        if grp.spec.window is None:
            return 0
        lowest_pos = max(0, n_tokens - grp.spec.window + 1)
        return lowest_pos // self.page_size

    def pages_missing(self, req: Request, n_new: int) -> int:
        """Pages of the tightest full-attention group that ``reserve(req, n_new)`` would take."""
        need = self.pages_for(req.n_tokens + n_new)
        worst = 0
        for gi, grp in enumerate(self.groups):
            if grp.spec.window is None:
                worst = max(worst, need - len(req.tables[gi]))
        return max(worst, 0)

    def reserve(self, req: Request, n_new: int) -> bool:
        """Take the pages that positions [n_tokens, n_tokens + n_new) need, in every group,
        or none at all.  False when a pool cannot give them."""
        if req.closed:
            raise ValueError(f"request {req.id!r} is closed")
        if n_new < 0:
            raise ValueError("n_new must not be negative")
        need_blocks = self.pages_for(req.n_tokens + n_new)
        taken: List[Tuple[int, int]] = []
        try:
            for gi, grp in enumerate(self.groups):
                table = req.tables[gi]
                first = self._first_needed_block(grp, req.n_tokens)
                while len(table) < need_blocks:
                    b = len(table)
                    if b < first:
                        table.append(-1)       # the window never reaches this block
                        taken.append((gi, -1))
                    else:
                        table.append(grp.pool.take())
                        taken.append((gi, table[-1]))
        except PoolFull:
            for gi, page in reversed(taken):
                req.tables[gi].pop()
                if page >= 0:
                    self.groups[gi].pool.release(page)
            return False
        return True

    def commit(self, req: Request, n_new: int) -> None:
        """The step wrote ``n_new`` positions: advance, and give back what a window passed."""
        req.n_tokens += n_new
        if self.groups and req.n_tokens > len(req.tables[0]) * self.page_size:
            raise AssertionError("a request advanced past its reserved pages")
        for gi, grp in enumerate(self.groups):
            if grp.spec.window is None:
                continue
            first = self._first_needed_block(grp, req.n_tokens)
            table = req.tables[gi]
            for b in range(min(first, len(table))):
                if table[b] >= 0:
                    grp.pool.release(table[b])
                    table[b] = -1

    def close(self, req: Request) -> None:
        """The request ended (or is preempted): give back its pages and its slot."""
        if req.closed:
            raise ValueError(f"request {req.id!r} closed twice")
        for gi, grp in enumerate(self.groups):
            for page in req.tables[gi]:
                if page >= 0:
                    grp.pool.release(page)
            req.tables[gi] = []
        req.closed = True
        req.n_tokens = 0
        self._free_slots.append(req.slot)
        del self.live[req.id]

    # ---- views for a step --------------------------------------------------------------
    def block_table_rows(self, reqs: Sequence[Request], group: int, width: Optional[int] = None) -> List[List[int]]:
        width = width or max([len(r.tables[group]) for r in reqs] + [1])
        return [r.tables[group] + [-1] * (width - len(r.tables[group])) for r in reqs]

    def check(self) -> None:
        """Bookkeeping invariants: every held page belongs to exactly one live request."""
        for gi, grp in enumerate(self.groups):
            grp.pool.check()
            held = [p for r in self.live.values() for p in r.tables[gi] if p >= 0]
            if len(set(held)) != len(held):
                raise AssertionError(f"group {gi}: a page is in two block tables")
            if len(held) != grp.pool.n_held:
                raise AssertionError(f"group {gi}: {grp.pool.n_held} pages held but {len(held)} in block tables (a page was lost)")
        slots = [r.slot for r in self.live.values()]
        if len(set(slots)) != len(slots) or len(slots) + len(self._free_slots) != self.max_slots:
            raise AssertionError("slots lost or held twice")
