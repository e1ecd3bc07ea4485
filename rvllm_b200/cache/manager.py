"""The cache manager: paged keys and values with a block table per request and cache group,
and slots of fixed-size per-request state.

Layers whose mixers need the same thing (same kv heads, head size and window) form a group; a
group has its own pages, its own block table per request and one device tensor
[cache slots of the group, num_pages, 2 (k, v), kv_heads, page_size, head_dim].  A page id
addresses the same page in every slot of its group.  Pages are handed out when tokens are about
to be written into them and come back when the request ends, is pre-empted, or - for a window
group - when every later query is past them.  The block table keeps -1 where a page was
given back.  Every request also holds one state slot; mixers with `StateNeed` get a tensor
[max_seqs, *shape] that is zeroed when the slot is handed to a new request.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Tuple

import torch

from ..errors import KvExhausted, SchedulerError
from ..parts.base import KvCacheNeed, StateNeed
from .pools import PagePool, SlotPool


@dataclass
class CacheView:
    """What a mixer sees of its cache slot."""
    group: Optional[int]                 # index of the page group (None: no pages)
    kv: Optional[torch.Tensor]           # [num_pages, 2, kv_heads, page_size, head_dim]
    state: Optional[torch.Tensor] = None  # [max_seqs, *shape]


@dataclass
class _Group:
    need: KvCacheNeed
    cache_slots: List[int]
    pool: PagePool
    tensor: Optional[torch.Tensor] = None


@dataclass
class _Request:
    state_slot: int
    num_tokens: int = 0
    tables: List[List[int]] = field(default_factory=list)   # per group: page of each logical block, -1 if freed
    first_live: List[int] = field(default_factory=list)     # per group: first logical block still held


class CacheManager:
    def __init__(self, needs: Dict[int, object], num_pages: int, page_size: int, max_seqs: int,
                 dtype: torch.dtype = torch.float32, device="cpu", allocate: bool = True):
        self.page_size, self.num_pages, self.max_seqs = page_size, num_pages, max_seqs
        self.dtype, self.device = dtype, device
        self.groups: List[_Group] = []
        self._slot_group: Dict[int, int] = {}
        self._slot_index: Dict[int, int] = {}
        self._state: Dict[int, torch.Tensor] = {}
        self._state_needs: Dict[int, StateNeed] = {}
        for slot in sorted(needs):
            need = needs[slot]
            if isinstance(need, KvCacheNeed):
                for gi, g in enumerate(self.groups):
                    if g.need == need:
                        break
                else:
                    gi = len(self.groups)
                    self.groups.append(_Group(need, [], PagePool(num_pages)))
                self._slot_group[slot] = gi
                self._slot_index[slot] = len(self.groups[gi].cache_slots)
                self.groups[gi].cache_slots.append(slot)
            elif isinstance(need, StateNeed):
                self._state_needs[slot] = need
            elif need is not None:
                raise SchedulerError(f"cache slot {slot}: unknown kind of need {need!r}")
        self.slots = SlotPool(max_seqs)
        self._has_window = any(g.need.window is not None for g in self.groups)
        self.requests: Dict[Hashable, _Request] = {}
        if allocate:
            for g in self.groups:
                g.tensor = torch.zeros((len(g.cache_slots), num_pages, 2, g.need.num_kv_heads, page_size,
                                        g.need.head_dim), dtype=dtype, device=device)
            for slot, need in self._state_needs.items():
                self._state[slot] = torch.zeros((max_seqs, *need.shape), dtype=getattr(torch, need.dtype), device=device)

    # ---- sizes ------------------------------------------------------------------------------
    @staticmethod
    def bytes_per_page(needs: Dict[int, object], page_size: int, dtype: torch.dtype) -> int:
        """Bytes that one more page per group costs over all cache slots."""
        el = torch.empty((), dtype=dtype).element_size()
        return sum(2 * n.num_kv_heads * page_size * n.head_dim * el for n in needs.values() if isinstance(n, KvCacheNeed))

    def view(self, cache_slot: int) -> CacheView:
        gi = self._slot_group.get(cache_slot)
        kv = None
        if gi is not None and self.groups[gi].tensor is not None:
            kv = self.groups[gi].tensor[self._slot_index[cache_slot]]
        return CacheView(gi, kv, self._state.get(cache_slot))

    def blocks_for(self, num_tokens: int) -> int:
        return (num_tokens + self.page_size - 1) // self.page_size

    def peak_pages(self, num_tokens: int, largest_portion: int) -> List[int]:
        """Per group, the most pages a request of `num_tokens` tokens holds at any one time when no
        step brings it more than `largest_portion` tokens.  A group that keeps every key needs the
        pages of all its tokens; a window group holds the window behind the first token of a step
        plus the step's own tokens (what lies below is given back after each step)."""
        out = []
        for g in self.groups:
            full = self.blocks_for(num_tokens)
            w = g.need.window
            if w is None:
                out.append(full)
            else:
                # keys [first - w + 1, first + portion) straddle at most one page more than their count fills
                out.append(min(full, self.blocks_for(w - 1 + max(1, largest_portion)) + 1))
        return out

    # ---- requests ---------------------------------------------------------------------------
    def has(self, req: Hashable) -> bool:
        return req in self.requests

    def admit(self, req: Hashable) -> int:
        if req in self.requests:
            raise SchedulerError(f"request {req!r} is already in the cache")
        slot = self.slots.allocate(req)
        self.requests[req] = _Request(slot, 0, [[] for _ in self.groups], [0 for _ in self.groups])
        for t in self._state.values():
            t[slot].zero_()
        return slot

    def num_tokens(self, req: Hashable) -> int:
        return self.requests[req].num_tokens

    def state_slot(self, req: Hashable) -> int:
        return self.requests[req].state_slot

    def pages_needed(self, req: Optional[Hashable], n_new: int, have_tokens: Optional[int] = None) -> List[int]:
        """New pages per group that appending `n_new` tokens would take."""
        if req is not None and req in self.requests:
            r = self.requests[req]
            return [self.blocks_for(r.num_tokens + n_new) - len(t) for t in r.tables]
        have = have_tokens or 0
        return [self.blocks_for(have + n_new) - self.blocks_for(have) for _ in self.groups]

    def can_append(self, req: Optional[Hashable], n_new: int, reserved: Optional[List[int]] = None) -> bool:
        need = self.pages_needed(req, n_new)
        res = reserved or [0] * len(self.groups)
        return all(n + r <= g.pool.num_free for n, r, g in zip(need, res, self.groups))

    def append(self, req: Hashable, n_new: int) -> int:
        """Reserve room for `n_new` more tokens; returns the position of the first.  Takes every
        page it needs or none (`KvExhausted`)."""
        r = self.requests[req]
        blocks = (r.num_tokens + n_new + self.page_size - 1) // self.page_size
        need = [blocks - len(t) for t in r.tables]
        if any(need):
            for n, g in zip(need, self.groups):
                if n > g.pool.num_free:
                    raise KvExhausted(n, g.pool.num_free, f"request {req!r}")
            for n, g, table in zip(need, self.groups, r.tables):
                if n > 0:
                    table.extend(g.pool.allocate(n, req))
        start = r.num_tokens
        r.num_tokens += n_new
        return start

    def block_table(self, req: Hashable, group: int) -> List[int]:
        return self.requests[req].tables[group]

    def slot_mapping(self, req: Hashable, group: int, start: int, n: int) -> List[int]:
        table = self.requests[req].tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + n):
            page = table[pos // ps]
            if page < 0:
                raise SchedulerError(f"request {req!r}: position {pos} lies in a page that was given back")
            out.append(page * ps + pos % ps)
        return out

    def release_passed(self, req: Hashable) -> int:
        """Give back the pages of window groups that no later query can see.  The next query
        sits at position >= num_tokens and sees keys > position - window."""
        r = self.requests[req]
        freed = 0
        if not self._has_window:
            return 0
        for gi, g in enumerate(self.groups):
            w = g.need.window
            if w is None:
                continue
            first_needed = max(0, r.num_tokens - w + 1)          # lowest key position still visible
            first_block = first_needed // self.page_size
            table = r.tables[gi]
            give = []
            for b in range(r.first_live[gi], min(first_block, len(table))):
                if table[b] >= 0:
                    give.append(table[b])
                    table[b] = -1
            if give:
                g.pool.release(give, req)
                freed += len(give)
            r.first_live[gi] = max(r.first_live[gi], min(first_block, len(table)))
        return freed

    def free(self, req: Hashable) -> None:
        r = self.requests.pop(req)
        for g, table in zip(self.groups, r.tables):
            g.pool.release([p for p in table if p >= 0], req)
        self.slots.release(r.state_slot, req)

    def num_free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or free while held; tables agree with the pools."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held = {}
            for req, r in self.requests.items():
                for p in r.tables[gi]:
                    if p < 0:
                        continue
                    if p in held:
                        raise SchedulerError(f"page {p} of group {gi} is in the tables of {held[p]!r} and {req!r}")
                    held[p] = req
                    if g.pool.owner(p) != req:
                        raise SchedulerError(f"page {p} of group {gi}: table of {req!r}, pool says {g.pool.owner(p)!r}")
            if len(held) + g.pool.num_free != g.pool.num_pages:
                raise SchedulerError(f"group {gi}: {len(held)} held + {g.pool.num_free} free != {g.pool.num_pages}")
        self.slots.check()
