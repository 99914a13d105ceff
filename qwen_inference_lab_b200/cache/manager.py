"""Per-request memory of a model's layers: paged keys/values and fixed-size state.

Every call of the model's order may own a cache: paged keys and values
(:class:`KVCacheSpec`) or a state of fixed size (:class:`StateSpec`).  Calls with
the same spec form a *group*.  A key/value group has its own page pool, its own
free list and one block table per request; a page id addresses the same slot range
in every member layer's plane, as in the reference's pool (qil/cache.py:47-49).
A group with a window gives pages back as soon as the window has passed them; the
others keep theirs until the request ends.  A state group is an array with one
slot per request row, zeroed at admission.  Whoever runs requests may keep state of
its own in such slots too (``request_state``: the engine keeps each request's sampling
settings and draw count there), beside the slots that layers own.

Admission can reserve capacity for the whole request (credits only: no page is
taken until tokens arrive), so that several partial prefills can never exhaust
the pool between them (qil/cache.py:1-6,58-77).  A request admitted without a
limit reserves nothing and grows until the free list is empty (trace replay).

Layout of a group's storage: ``[member, page, 2 (K,V), kv_head, slot, head_dim]``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass

import torch

from ..parts.base import KVCacheSpec, StateSpec
from ..utils.staging import PinnedRing


class CacheError(ValueError):
    """A call that breaks the cache's rules (unknown owner, write beyond the reservation...)."""


class OutOfPages(RuntimeError):
    """The free list cannot cover a request's next tokens."""


@dataclass
class KVCacheView:
    """What an attention-like mixer gets: its layer's pages and the request block tables."""
    pages: torch.Tensor          # [num_pages, 2, kv_heads, page_size, head_dim]
    block_table: torch.Tensor    # int32 [max_requests, table_width]; -1 where no page is held
    page_size: int
    window: int


@dataclass
class StateView:
    """What a stateful mixer gets: one slot per request row."""
    slots: torch.Tensor          # [max_requests, *shape]


class _KVGroup:
    def __init__(self, spec, members, num_pages, page_size, max_requests, table_width, dtype, device):
        self.spec, self.members = spec, list(members)
        self.capacity, self.page_size = int(num_pages), int(page_size)
        self.storage = torch.empty((len(self.members), num_pages, 2, spec.kv_heads, page_size, spec.head_dim),
                                   dtype=dtype, device=device)
        self.free = deque(range(num_pages))
        self.tables: dict = {}       # request -> list of page ids by logical page index (-1: given back)
        self.first_live: dict = {}   # request -> first logical page index still needed
        self.reserved: dict = {}     # request -> pages of credit
        self.host_table = torch.full((max_requests, table_width), -1, dtype=torch.int32)
        self.dev_table = torch.full((max_requests, table_width), -1, dtype=torch.int32, device=device)
        self.dirty: set = set()

    def pages_for(self, tokens):
        return (tokens + self.page_size - 1) // self.page_size

    def credit(self, limit, max_step_tokens):
        pages = self.pages_for(limit)
        if self.spec.window > 0:
            pages = min(pages, self.pages_for(self.spec.window + max_step_tokens) + 1)
        return pages

    @property
    def unreserved(self):
        """Pages neither promised to a reserved request nor held by an unreserved one."""
        held_without_credit = sum(sum(1 for p in table if p >= 0)
                                  for rid, table in self.tables.items() if rid not in self.reserved)
        return self.capacity - sum(self.reserved.values()) - held_without_credit


class CacheManager:
    def __init__(self, specs, *, num_pages, page_size, max_requests, max_context, dtype, device,
                 max_step_tokens=None, request_state=None):
        if any(type(v) is not int or v < 1 for v in (num_pages, page_size, max_requests, max_context)):
            raise CacheError("cache dimensions must be positive integers")
        self.page_size, self.num_pages = page_size, num_pages
        self.max_requests, self.max_context = max_requests, max_context
        self.max_step_tokens = int(max_step_tokens or max_context)
        self.device, self.dtype = torch.device(device), dtype
        self.specs = list(specs)
        windowed = any(isinstance(s, KVCacheSpec) and s.window > 0 for s in self.specs)
        span = max_context if windowed else min(max_context, num_pages * page_size)
        self.table_width = (span + page_size - 1) // page_size
        self.kv_groups: list = []
        self.state_groups: list = []   # (spec, members, tensor)
        self._owner: dict = {}         # call index -> ("kv", group, member) | ("state", group, member)
        by_spec: dict = {}
        for call, spec in enumerate(self.specs):
            if spec is not None:
                by_spec.setdefault(spec, []).append(call)
        for spec, members in by_spec.items():
            if isinstance(spec, KVCacheSpec):
                group = _KVGroup(spec, members, num_pages, page_size, max_requests, self.table_width, dtype, device)
                for m, call in enumerate(members):
                    self._owner[call] = ("kv", len(self.kv_groups), m)
                self.kv_groups.append(group)
            elif isinstance(spec, StateSpec):
                tensor = torch.zeros((len(members), max_requests, *spec.shape), dtype=spec.dtype, device=device)
                for m, call in enumerate(members):
                    self._owner[call] = ("state", len(self.state_groups), m)
                self.state_groups.append((spec, members, tensor))
            else:
                raise CacheError(f"unknown cache spec {spec!r}")
        # state that belongs to a request, not to a layer: name -> tensor [max_requests, *shape]
        self._request_state = {name: torch.zeros((max_requests, *spec.shape), dtype=spec.dtype, device=device)
                               for name, spec in (request_state or {}).items()}
        self._ring = PinnedRing(depth=8) if self.device.type == "cuda" else None
        self.free_rows = deque(range(max_requests))
        self.rows: dict = {}       # request -> row
        self.limits: dict = {}     # request -> reserved tokens or None
        self.progress: dict = {}   # request -> tokens written (all layers; a step is atomic)

    # ------------------------------------------------------------------ sizes
    def pages_for(self, tokens):
        return (tokens + self.page_size - 1) // self.page_size

    @property
    def capacity(self):
        return self.num_pages

    def free_pages(self, group=0):
        return len(self.kv_groups[group].free) if self.kv_groups else 0

    @property
    def unreserved(self):
        return min((g.unreserved for g in self.kv_groups), default=self.num_pages)

    def fits(self, limit) -> bool:
        """Could a request of ``limit`` cached tokens ever be admitted into an empty cache?"""
        return limit <= self.table_width * self.page_size and all(
            g.credit(limit, self.max_step_tokens) <= g.capacity for g in self.kv_groups)

    # ------------------------------------------------------------------ life of a request
    def admit(self, request_id, limit=None) -> bool:
        """Give the request a row (block-table row and state slot) and, with ``limit``, reserve
        pages for that many cached tokens.  False when rows or credits do not suffice now."""
        if request_id in self.rows:
            raise CacheError("duplicate cache owner")
        if limit is not None and (type(limit) is not int or limit < 1):
            raise CacheError("cache reservation must be positive")
        if not self.free_rows:
            return False
        if limit is not None:
            if limit > self.table_width * self.page_size:
                return False
            for g in self.kv_groups:
                if g.credit(limit, self.max_step_tokens) > g.unreserved:
                    return False
        row = self.free_rows.popleft()
        self.rows[request_id] = row
        self.limits[request_id] = limit
        self.progress[request_id] = 0
        for g in self.kv_groups:
            g.tables[request_id] = []
            g.first_live[request_id] = 0
            if limit is not None:
                g.reserved[request_id] = g.credit(limit, self.max_step_tokens)
        for _, _, tensor in self.state_groups:
            tensor[:, row].zero_()
        for tensor in self._request_state.values():
            tensor[row].zero_()
        return True

    def request_state(self, name) -> torch.Tensor:
        """The slots of the per-request state ``name`` given at construction: [max_requests, *shape],
        indexed by ``row(request_id)``, zeroed when a request is admitted."""
        return self._request_state[name]

    def row(self, request_id) -> int:
        return self.rows[request_id]

    def written(self, request_id) -> int:
        return self.progress[request_id]

    def ensure(self, request_id, end) -> None:
        """Hold pages for positions [written, end) in every key/value group."""
        if request_id not in self.rows:
            raise CacheError("unknown cache owner")
        limit = self.limits[request_id]
        if end <= 0 or (limit is not None and end > limit) or end > self.table_width * self.page_size:
            raise CacheError("write exceeds reserved context")
        row = self.rows[request_id]
        for g in self.kv_groups:
            table = g.tables[request_id]
            needed = g.pages_for(end) - len(table)
            if needed <= 0:
                continue
            if limit is None:
                # pages promised to reserved requests but not taken yet are not for the taking
                promised = sum(credit - sum(1 for p in g.tables[rid] if p >= 0) for rid, credit in g.reserved.items())
                if needed > len(g.free) - promised:
                    raise OutOfPages(f"request {request_id!r} needs {needed} more pages, "
                                     f"{len(g.free) - promised} are free and unpromised")
            elif needed > len(g.free):
                raise RuntimeError("cache reservation invariant violated")
            for _ in range(needed):
                page = g.free.popleft()
                g.host_table[row, len(table)] = page
                table.append(page)
            g.dirty.add(row)

    def advance(self, request_id, end) -> None:
        """Record that positions below ``end`` are written; give back pages a window has passed."""
        if end < self.progress[request_id]:
            raise CacheError("cache progress cannot move backwards")
        self.progress[request_id] = end
        row = self.rows[request_id]
        for g in self.kv_groups:
            if g.spec.window <= 0:
                continue
            first_needed = max(0, end - g.spec.window + 1) // g.page_size
            table = g.tables[request_id]
            for index in range(g.first_live[request_id], min(first_needed, len(table))):
                if table[index] >= 0:
                    g.free.append(table[index])
                    table[index] = -1
                    g.host_table[row, index] = -1
                    g.dirty.add(row)
            g.first_live[request_id] = max(g.first_live[request_id], min(first_needed, len(table)))

    def release(self, request_id) -> None:
        if request_id not in self.rows:
            raise CacheError("unknown cache owner")
        row = self.rows.pop(request_id)
        for g in self.kv_groups:
            table = g.tables.pop(request_id)
            g.free.extend(page for page in table if page >= 0)
            if table:
                g.host_table[row, :len(table)] = -1
                g.dirty.add(row)
            g.first_live.pop(request_id)
            g.reserved.pop(request_id, None)
        del self.limits[request_id]
        del self.progress[request_id]
        self.free_rows.append(row)

    def owners(self):
        return list(self.rows)

    # ------------------------------------------------------------------ device side
    def flush_tables(self) -> None:
        """Copy block-table rows that changed since the last flush to the device.

        The rows are snapshotted into a pinned staging buffer first: the host table
        may change again (pages given back, a row reused) before the copy runs.
        """
        for g in self.kv_groups:
            if not g.dirty:
                continue
            rows = sorted(g.dirty)
            g.dirty.clear()
            if self.device.type != "cuda":
                for row in rows:
                    g.dev_table[row].copy_(g.host_table[row])
                continue
            width = self.table_width
            stage = self._ring.acquire(len(rows) * width * 4).view(torch.int32)[:len(rows) * width]
            stage = stage.view(len(rows), width)
            stage.copy_(g.host_table[rows])
            if len(rows) == self.max_requests:
                g.dev_table.copy_(stage, non_blocking=True)
            else:
                for i, row in enumerate(rows):
                    g.dev_table[row].copy_(stage[i], non_blocking=True)
            self._ring.commit()

    def views(self, order=None) -> list:
        """One view per call of the order (``order[i].reads_cache_of`` redirects to the owner)."""
        result = []
        for call in range(len(self.specs)):
            source = call
            if order is not None and order[call].reads_cache_of is not None:
                source = order[call].reads_cache_of
            owner = self._owner.get(source)
            if owner is None:
                result.append(None)
            elif owner[0] == "kv":
                g = self.kv_groups[owner[1]]
                result.append(KVCacheView(g.storage[owner[2]], g.dev_table, g.page_size, g.spec.window))
            else:
                result.append(StateView(self.state_groups[owner[1]][2][owner[2]]))
        return result

    def poison(self, value=float("nan")) -> None:
        """Fill every page with ``value`` (tests: reads of unwritten memory then show)."""
        for g in self.kv_groups:
            g.storage.fill_(value)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, held twice or freed twice; tables and mirrors agree."""
        if sorted(list(self.free_rows) + list(self.rows.values())) != list(range(self.max_requests)):
            raise AssertionError("request rows lost or duplicated")
        for index, g in enumerate(self.kv_groups):
            held = [p for table in g.tables.values() for p in table if p >= 0]
            everything = sorted(held + list(g.free))
            if everything != list(range(g.capacity)):
                raise AssertionError(f"group {index}: pages lost, held twice or freed twice")
            if set(g.tables) != set(self.rows):
                raise AssertionError(f"group {index}: tables and owners disagree")
            for request_id, table in g.tables.items():
                row = self.rows[request_id]
                mirror = g.host_table[row, :len(table)].tolist()
                if mirror != table or (g.host_table[row, len(table):] != -1).any():
                    raise AssertionError(f"group {index}: host block table differs from the page list")
                live = sum(1 for p in table if p >= 0)
                if request_id in g.reserved and live > g.reserved[request_id]:
                    raise AssertionError(f"group {index}: request holds more pages than it reserved")
            if sum(g.reserved.values()) > g.capacity:
                raise AssertionError(f"group {index}: reservations exceed capacity")
