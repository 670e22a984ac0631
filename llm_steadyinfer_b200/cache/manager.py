"""Cache manager: which pages and which state slot each live request holds.

Layers whose mixers need the same kind of cache (same heads, head size and window) form a
*group*; a group has its own page pool and one block table per request, shared by the
group's layers (the reference has one uniform pool, src/source/scheduler/kv_manager.cpp:41-53).
Pages are taken when a request grows, given back when it ends, when it is cut back for
preemption, and, in a windowed group, as soon as the window has passed them. Every request
also holds one state slot, the index at which mixers with fixed-size state keep theirs.

Prefix reuse (single group without window, no fixed-size state): whole pages are keyed by a
hash chained over all tokens before and in them, so equal content at another place or after
another prefix never matches; the reference hashes a block's own 16 tokens only
(src/source/scheduler/prefix_cache.cpp:8-18).

This module is host bookkeeping only; the tensors live in ``CacheStorage``.
"""
from __future__ import annotations

import itertools

import hashlib
import struct
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..parts.base import CacheNeed, StateNeed
from .pages import PageError, PagePool, SlotPool


class OutOfPages(RuntimeError):
    """A request cannot grow: some group has too few free pages (nothing was taken)."""


class OutOfSlots(RuntimeError):
    """No state slot is free: too many live requests."""


@dataclass
class CacheGroup:
    need: CacheNeed
    layers: List[int]                      # layers that own cache in this group, in storage order
    pool: PagePool
    tables: Dict[Hashable, List[int]] = field(default_factory=dict)   # request -> page per block, -1 = given back

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclass
class RequestCache:
    slot: int
    length: int = 0                        # tokens whose keys/values are stored
    shared_pages: int = 0                  # leading pages mounted from the prefix index


class CacheLayout:
    """Groups the places of the run order ("layers" below) by their cache need.
    ``cache_from[i]`` names the place whose cache place i reads instead of owning one."""

    def __init__(self, needs: Sequence[Optional[CacheNeed]], states: Sequence[Optional[StateNeed]],
                 cache_from: Optional[Sequence[Optional[int]]] = None):
        n = len(needs)
        cache_from = list(cache_from) if cache_from is not None else [None] * n
        self.needs = list(needs)
        self.states = list(states)
        self.cache_from = cache_from
        self.group_keys: List[Tuple] = []
        self.group_layers: List[List[int]] = []
        self.layer_group: List[Optional[int]] = [None] * n
        self.layer_index_in_group: List[Optional[int]] = [None] * n
        for i, need in enumerate(needs):
            if cache_from[i] is not None or need is None:
                continue
            key = need.group_key()
            if key not in self.group_keys:
                self.group_keys.append(key)
                self.group_layers.append([])
            g = self.group_keys.index(key)
            self.layer_group[i] = g
            self.layer_index_in_group[i] = len(self.group_layers[g])
            self.group_layers[g].append(i)
        for i, src in enumerate(cache_from):
            if src is None:
                continue
            if not 0 <= src < n or cache_from[src] is not None or needs[src] is None:
                raise ValueError(f"layer {i} reads the cache of layer {src}, which owns none")
            if needs[i] is None or needs[i].group_key()[:3] != needs[src].group_key()[:3]:
                raise ValueError(f"layer {i} cannot read layer {src}'s cache: their head layouts differ")
            sw, rw = needs[src].window, needs[i].window
            if sw is not None and (rw is None or rw > sw):
                raise ValueError(f"layer {i} would read further back than layer {src}'s window of {sw} keeps")
            self.layer_group[i] = self.layer_group[src]
            self.layer_index_in_group[i] = self.layer_index_in_group[src]

    @property
    def num_groups(self) -> int:
        return len(self.group_keys)

    def group_need(self, g: int) -> CacheNeed:
        return self.needs[self.group_layers[g][0]]


class CacheManager:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages: int, max_requests: int,
                 prefix_reuse: bool = False):
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.layout = layout
        self.page_size = int(page_size)
        self.groups = [CacheGroup(layout.group_need(g), layout.group_layers[g], PagePool(num_pages))
                       for g in range(layout.num_groups)]
        self.slots = SlotPool(max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}
        has_state = any(s is not None for s in layout.states)
        self.prefix_reuse = bool(prefix_reuse) and len(self.groups) == 1 \
            and self.groups[0].window is None and not has_state
        self._hash_to_page: Dict[bytes, int] = {}
        self._page_to_hash: Dict[int, bytes] = {}
        if self.prefix_reuse:
            self.groups[0].pool.on_evict = self._forget_page
        self.new_slots: List[int] = []     # slots admitted since the storage last zeroed state
        # A number per live request that changes whenever its tables change. The numbers are never used
        # twice, also not by a later request under the same name, so that whoever caches something
        # derived from a table under (name, number) cannot mistake one request's table for another's.
        self.versions: Dict[Hashable, int] = {}
        self._version = itertools.count(1)

    # ---- queries -------------------------------------------------------------------
    def has(self, req) -> bool:
        return req in self.requests

    def length(self, req) -> int:
        return self.requests[req].length

    def slot(self, req) -> int:
        return self.requests[req].slot

    def blocks_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    def table(self, group: int, req) -> List[int]:
        return self.groups[group].tables[req]

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def pages_missing(self, req, new_length: int) -> List[int]:
        """Per group, how many pages must still be taken for the request to hold ``new_length`` tokens."""
        return [max(0, self.blocks_for(new_length) - len(g.tables[req])) for g in self.groups]

    def can_grow(self, req, new_length: int) -> bool:
        return all(m <= g.pool.num_free for m, g in zip(self.pages_missing(req, new_length), self.groups))

    # ---- life of a request -----------------------------------------------------------
    def admit(self, req, tokens: Optional[Sequence[int]] = None, chain: Optional[List[bytes]] = None) -> int:
        """Give the request a state slot and empty tables. With prefix reuse and its prompt
        ``tokens``, mount the longest stored chain of whole pages that leaves at least one
        token to compute (``chain``: ``chain_hashes(tokens)`` if the caller has them already).
        Returns the number of tokens already held."""
        if req in self.requests:
            raise ValueError(f"request {req!r} is already live")
        slot = self.slots.take()
        if slot is None:
            raise OutOfSlots(f"all {self.slots.num_slots} state slots are in use")
        rc = RequestCache(slot=slot)
        self.requests[req] = rc
        self.versions[req] = next(self._version)
        self.new_slots.append(slot)
        for g in self.groups:
            g.tables[req] = []
        if self.prefix_reuse and tokens is not None:
            pages = self.match_prefix(tokens, chain)
            pool = self.groups[0].pool
            for p in pages:
                pool.retain(p)
            self.groups[0].tables[req] = list(pages)
            rc.shared_pages = len(pages)
            rc.length = len(pages) * self.page_size
        return rc.length

    def grow(self, req, new_length: int) -> None:
        """Take pages so that tokens [0, new_length) have a place, in every group or in none."""
        need = -(-new_length // self.page_size)
        if all(len(g.tables[req]) >= need for g in self.groups):
            return                                  # the usual decode step: the last page still has room
        missing = self.pages_missing(req, new_length)
        for m, g in zip(missing, self.groups):
            if m > g.pool.num_free:
                raise OutOfPages(f"request {req!r} needs {m} more pages, {g.pool.num_free} are free")
        for m, g in zip(missing, self.groups):
            got = g.pool.allocate(m)
            assert got is not None
            if got:
                g.tables[req].extend(got)
                self.versions[req] = next(self._version)

    def commit(self, req, new_length: int) -> None:
        """The request now holds ``new_length`` tokens; windowed groups give back the pages
        that no later position can read."""
        rc = self.requests[req]
        rc.length = new_length
        for g in self.groups:
            if g.window is None:
                continue
            first_needed = new_length - g.window + 1      # the next token reads keys from here on
            dead = max(0, first_needed) // self.page_size
            t = g.tables[req]
            for b in range(min(dead, len(t))):
                if t[b] >= 0:
                    g.pool.release(t[b])
                    t[b] = -1
                    self.versions[req] = next(self._version)

    def can_truncate_to(self, keep_length: int) -> int:
        """Preemption keeps a whole number of pages; with windows or fixed-size state nothing
        can be kept, since what the kept part would need is gone or cannot be cut."""
        if any(g.window is not None for g in self.groups) or any(s is not None for s in self.layout.states):
            return 0
        return (keep_length // self.page_size) * self.page_size

    def truncate(self, req, keep_length: int) -> int:
        """Cut the request back to ``keep_length`` tokens (rounded down as
        ``can_truncate_to`` says) and give the pages behind it back. Returns the new length."""
        rc = self.requests[req]
        keep = min(self.can_truncate_to(keep_length), rc.length // self.page_size * self.page_size)
        nb = keep // self.page_size
        for g in self.groups:
            t = g.tables[req]
            for p in t[nb:]:
                if p >= 0:
                    self._release(g, p)
            del t[nb:]
        rc.length = keep
        self.versions[req] = next(self._version)
        rc.shared_pages = min(rc.shared_pages, nb)
        if keep == 0:
            self.new_slots.append(rc.slot)           # state starts over
        return keep

    def release(self, req) -> None:
        """The request has ended: all its pages and its slot go back."""
        rc = self.requests.pop(req)
        self.versions.pop(req, None)
        for g in self.groups:
            for p in g.tables.pop(req):
                if p >= 0:
                    self._release(g, p)
        self.slots.give_back(rc.slot)

    def _release(self, g: CacheGroup, page: int) -> None:
        g.pool.release(page, park=self.prefix_reuse and page in self._page_to_hash)

    # ---- prefix reuse ---------------------------------------------------------------
    def chain_hashes(self, tokens: Sequence[int]) -> List[bytes]:
        """One hash per whole page of ``tokens``, each chained over every token up to the page's end. A
        caller that asks about the same tokens again and again keeps the list and hands it back."""
        if not self.prefix_reuse:
            return []
        out, h, ps = [], b"", self.page_size
        for b in range(len(tokens) // ps):
            h = hashlib.blake2b(h + struct.pack(f"<{ps}i", *tokens[b * ps:(b + 1) * ps]), digest_size=16).digest()
            out.append(h)
        return out

    def match_prefix(self, tokens: Sequence[int], chain: Optional[List[bytes]] = None) -> List[int]:
        if not self.prefix_reuse:
            return []
        chain = self.chain_hashes(tokens) if chain is None else chain
        pages = []
        for h in chain[:(len(tokens) - 1) // self.page_size]:      # at least one token is left to compute
            p = self._hash_to_page.get(h)
            if p is None:
                break
            pages.append(p)
        return pages

    def remember_prefix(self, req, tokens: Sequence[int], chain: Optional[List[bytes]] = None) -> None:
        """Key the request's whole, fully written pages by their chained hashes."""
        if not self.prefix_reuse:
            return
        rc = self.requests[req]
        t = self.groups[0].tables[req]
        n = min(rc.length, len(tokens)) // self.page_size
        chain = self.chain_hashes(tokens) if chain is None else chain
        for b, h in enumerate(chain[:n]):
            if h in self._hash_to_page or t[b] in self._page_to_hash:
                continue
            self._hash_to_page[h] = t[b]
            self._page_to_hash[t[b]] = h

    def _forget_page(self, page: int) -> None:
        h = self._page_to_hash.pop(page, None)
        if h is not None:
            self._hash_to_page.pop(h, None)

    # ---- self check -----------------------------------------------------------------
    def check_invariant(self) -> None:
        """No page lost, held twice without a count for it, or free while held; no slot shared."""
        for g in self.groups:
            held = [p for t in g.tables.values() for p in t if p >= 0]
            g.pool.check_invariant(held)
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots):
            raise PageError("two live requests share a state slot")
        if len(slots) + self.slots.num_free != self.slots.num_slots:
            raise PageError("a state slot was lost")
        for h, p in self._hash_to_page.items():
            if self._page_to_hash.get(p) != h:
                raise PageError(f"prefix index is inconsistent at page {p}")
