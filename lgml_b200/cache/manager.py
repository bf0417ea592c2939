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

With ``prefix_cache`` the full pages of a request get keys when it ends or is preempted
(a chain of hashes over the tokens, ``M.key``, ``lua/lgml/kvpool.lua:51-59``), and a new
request whose tokens begin the same way shares those pages instead of computing them
(``E:reuse`` ``lua/lgml/engine.lua:1775-1819``, ``E:attach_blocks`` ``:2038``); at least its
last token is always computed, since its logits are wanted.  Shared pages are only read:
a request writes behind its prefix, into pages of its own.  This needs every layer to keep
all its keys (no window, no state of fixed size: those cannot be taken up in the middle,
``check_pass`` ``lua/lgml/transformer.lua:1548-1563``).
"""
from __future__ import annotations

import hashlib
import struct
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
                 page_size: int = PAGE_SIZE, max_step_tokens: int = 0, prefix_cache: bool = False):
        if max_slots <= 0:
            raise ValueError("max_slots must be positive")
        self.prefix_cache = bool(prefix_cache)
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
        if self.prefix_cache and (self.state_groups or any(g.spec.window is not None for g in self.groups)):
            raise ValueError("prefix_cache needs layers that keep all their keys: a window or a state of fixed size cannot be taken up in the middle")
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
    def open(self, rid: Hashable, tokens: Optional[Sequence[int]] = None) -> Request:
        """A slot for a new request.  With ``prefix_cache`` and the request's ``tokens`` it
        starts with the pages that already hold its first tokens: ``n_tokens`` says how many."""
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
        if self.prefix_cache and tokens:
            for pages in self._cached_prefix(tokens):
                for gi, page in enumerate(pages):
                    self.groups[gi].pool.share(page)
                    req.tables[gi].append(page)
                req.n_tokens += self.page_size
        return req

    # ---- prefix cache ------------------------------------------------------------------
    def _keys(self, tokens: Sequence[int], n_blocks: int):
        """The keys of the first ``n_blocks`` full pages of ``tokens``: each hashes the key
        before it and its own tokens, so a key stands for the whole prefix."""
        key = b"lgml_b200 page %d" % self.page_size
        for b in range(n_blocks):
            block = tokens[b * self.page_size:(b + 1) * self.page_size]
            key = hashlib.sha256(key + struct.pack(f"<{self.page_size}q", *block)).digest()
            yield key

    def _cached_prefix(self, tokens: Sequence[int]) -> List[List[int]]:
        """Per leading full page of ``tokens`` that every group still holds under its key: the
        group's pages.  The last token is never part of it."""
        out: List[List[int]] = []
        for key in self._keys(tokens, (len(tokens) - 1) // self.page_size):
            pages = [g.pool.lookup(key) for g in self.groups]
            if any(p is None for p in pages):
                break
            out.append(pages)
        return out

    def cached_prefix_tokens(self, tokens: Sequence[int]) -> int:
        """How many leading tokens ``open(rid, tokens)`` would find in the cache."""
        return len(self._cached_prefix(tokens)) * self.page_size if self.prefix_cache and tokens else 0

    def cached_pages_in_prefix(self, tokens: Sequence[int]) -> int:
        """Of the pages ``open(rid, tokens)`` would share, those that nobody holds now: they
        count among the free pages until they are shared (the tightest group's number)."""
        if not self.prefix_cache or not tokens:
            return 0
        pref = self._cached_prefix(tokens)
        return max((sum(1 for pages in pref if g.pool.refcount(pages[gi]) == 0) for gi, g in enumerate(self.groups)), default=0)

    def publish(self, req: Request, tokens: Sequence[int]) -> int:
        """Give the request's full pages their keys (``tokens[p]`` is the token at position p; only
        positions the cache holds count).  Returns the pages that are findable afterwards."""
        if not self.prefix_cache or req.closed:
            return 0
        n_blocks = min(req.n_tokens, len(tokens)) // self.page_size
        found = 0
        for b, key in enumerate(self._keys(tokens, n_blocks)):
            ok = [g.pool.publish(req.tables[gi][b], key) for gi, g in enumerate(self.groups)]
            found += all(ok)
        return found

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

    def reserve_all(self, wanted: Sequence[Tuple[Request, int]]) -> Optional[int]:
        """``reserve`` for every (request, new tokens) of a step, or for none: when one finds
        no page, those before it give back what this call took for them.  Returns the index
        of the entry that found no page, or None when all have theirs."""
        before = [[len(t) for t in req.tables] for req, _ in wanted]
        for i, (req, n) in enumerate(wanted):
            if not self.reserve(req, n):
                for (r, _), lens in zip(wanted[:i], before[:i]):
                    self.unreserve(r, lens)
                return i
        return None

    def unreserve(self, req: Request, table_lens: Sequence[int]) -> None:
        """Give back the pages a ``reserve`` took: cut every group's table back to the length
        it had before (``table_lens``, one per group).  Only pages behind what the request has
        written can go, so nothing that holds keys is lost."""
        written = self.pages_for(req.n_tokens)
        for gi, grp in enumerate(self.groups):
            table = req.tables[gi]
            if table_lens[gi] < written or table_lens[gi] > len(table):
                raise ValueError(f"request {req.id!r}: cannot cut a table of {len(table)} pages, {written} of them written, back to {table_lens[gi]}")
            while len(table) > table_lens[gi]:
                page = table.pop()
                if page >= 0:
                    grp.pool.release(page)

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
            # the deepest page first: of a chain of cached pages the pool then takes the end
            # before the beginning, and what is left is still a prefix (the reference evicts by
            # depth too, ``lua/lgml/kvpool.lua:139-160``)
            for page in reversed(req.tables[gi]):
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
            for p in set(held):
                if held.count(p) != grp.pool.refcount(p):
                    raise AssertionError(f"group {gi}: page {p} is in {held.count(p)} block tables but held {grp.pool.refcount(p)} times")
                if held.count(p) > 1 and not self.prefix_cache:
                    raise AssertionError(f"group {gi}: a page is in two block tables")
            if len(set(held)) != grp.pool.n_held:
                raise AssertionError(f"group {gi}: {grp.pool.n_held} pages held but {len(set(held))} in block tables (a page was lost)")
        slots = [r.slot for r in self.live.values()]
        if len(set(slots)) != len(slots) or len(slots) + len(self._free_slots) != self.max_slots:
            raise AssertionError("slots lost or held twice")
