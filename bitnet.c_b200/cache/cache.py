"""The cache of a model instance: paged keys and values per group of runs, and fixed-size state.

Every schedule entry whose mixer asks for cached keys and values gets a plane of its own in
the *group* of all entries with the same request (heads, head size, window).  A group has its
own storage, page pool and page table, so runs with different needs never share memory:

    k             [entries, pages, kv_heads, 64, head_dim]   compute type
    v             [entries, pages, kv_heads, 64, v_head_dim] (a value head may be narrower or wider than a key head)
    page_table    [slots, pages_per_sequence]  int32, on the device and mirrored on the host

A sequence lives in a *slot* from its first token to its end and holds, in each group, the
pages its length needs; a group with a window gives pages back as soon as they lie wholly
before the window.  A run that reads another run's cache (``cache_of``) gets a view of that
run's plane and writes nothing.  Runs that ask for fixed-size state get one tensor
``[slots, ...]`` each, zeroed when a slot is opened (the reference keeps recurrent state of
this kind in its run state, include/model_run_state.h:21-23, zeroed on reset,
src/session.c:145-167).  The reference's own key/value arrays are per session and
[layers, seq_len, kv_dim] (src/transformer/kv.c:123-131).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KvRequest, StateRequest
from .pages import PAGE, CacheError, CacheFull, PagePool, SlotTable, pages_for


@dataclass
class KvView:
    """What a mixer sees of the cache for one run."""

    k: torch.Tensor  # [pages, kv_heads, PAGE, head_dim]
    v: torch.Tensor  # [pages, kv_heads, PAGE, v_head_dim]
    page_table: torch.Tensor  # [slots, pages_per_sequence] int32
    n_kv_heads: int
    head_dim: int
    window: int
    owner: bool  # False: this run reads another run's plane and must not write
    v_head_dim: int = 0  # 0: as head_dim

    @property
    def v_dim(self) -> int:
        return self.v_head_dim or self.head_dim

    def append(self, x: torch.Tensor, k_off: int, v_off: int, ctx) -> None:
        """Write the key heads at ``k_off`` and value heads at ``v_off`` of each row of x."""
        from ..csrc import ops
        if not self.owner:
            raise CacheError("a run that reads another run's cache must not write it")
        if self.v_dim != self.head_dim:
            # values of another width than keys: the append kernel takes one width, so the rows are
            # placed by index (page and row of every token from the device arrays of the step)
            n = ctx.n_tokens
            page = self.page_table[ctx.slots[ctx.tok_seq.long()].long(), (ctx.tok_pos // PAGE).long()].long()
            row = (ctx.tok_pos % PAGE).long()
            self.k[page, :, row] = x[:n, k_off:k_off + self.n_kv_heads * self.head_dim].reshape(n, self.n_kv_heads, self.head_dim)
            self.v[page, :, row] = x[:n, v_off:v_off + self.n_kv_heads * self.v_dim].reshape(n, self.n_kv_heads, self.v_dim)
            return
        ops.rope_append(x, 0, self.head_dim, 0, 1.0, ctx.tok_pos, k_off=k_off, v_off=v_off,
                        n_kv_heads=self.n_kv_heads, tok_seq=ctx.tok_seq, slots=ctx.slots,
                        page_table=self.page_table, k_cache=self.k, v_cache=self.v)


class KvGroup:
    """Storage of all runs with one request."""

    def __init__(self, request: KvRequest, entries: List[int], n_pages: int, n_slots: int,
                 pages_per_seq: int, dtype: torch.dtype, device, allocate: bool = True):
        self.request = request
        self.entries = entries
        self.pool = PagePool(n_pages)
        self.pages_per_seq = pages_per_seq
        self.host_table = np.zeros((n_slots, pages_per_seq), dtype=np.int32)
        self.held: Dict[int, Dict[int, int]] = {}  # slot -> {page index in sequence -> page id}
        self.dirty: set = set()
        shape = (len(entries), n_pages, request.n_kv_heads, PAGE, request.head_dim)
        if allocate:
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape[:-1] + (request.v_dim,), dtype=dtype, device=device)
            self.page_table = torch.zeros((n_slots, pages_per_seq), dtype=torch.int32, device=device)
        else:  # bookkeeping only (tests without a device)
            self.k = self.v = self.page_table = None

    def bytes_per_token(self, itemsize: int) -> int:
        return len(self.entries) * self.request.n_kv_heads * (self.request.head_dim + self.request.v_dim) * itemsize

    def reserve(self, slot: int, old_len: int, new_len: int) -> None:
        """Hold pages for positions [first needed, new_len)."""
        held = self.held.setdefault(slot, {})
        last = (new_len - 1) // PAGE
        if old_len > 0 and (old_len - 1) // PAGE == last and last in held:
            return  # the new tokens lie in the page that holds the sequence's last token
        first = 0
        if self.request.window > 0:
            # the oldest key any new token needs: position old_len - window + 1
            first = max(0, old_len - self.request.window + 1) // PAGE
        need = [i for i in range(first, pages_for(new_len)) if i not in held]
        if need and need[-1] >= self.pages_per_seq:
            raise CacheFull(f"a sequence of {new_len} tokens needs page {need[-1]}, "
                            f"the table holds {self.pages_per_seq} per sequence")
        ids = self.pool.alloc(len(need))
        for i, p in zip(need, ids):
            held[i] = p
            self.host_table[slot, i] = p
        if need:
            self.dirty.add(slot)

    def trim(self, slot: int, length: int) -> None:
        """Give back pages that lie wholly before the window of a sequence of ``length`` tokens."""
        if self.request.window <= 0:
            return
        held = self.held.get(slot, {})
        first_needed = max(0, length - self.request.window + 1) // PAGE
        gone = [i for i in held if i < first_needed]
        self.pool.free([held.pop(i) for i in gone])

    def release(self, slot: int) -> None:
        held = self.held.pop(slot, {})
        self.pool.free(list(held.values()))
        self.dirty.discard(slot)

    def tokens_held(self) -> int:
        return sum(len(h) for h in self.held.values()) * PAGE


class Cache:
    """Slots, page groups and state for one model instance.

    ``kv_requests[i]`` / ``state_requests[i]`` are what schedule entry ``i`` asks for (None for
    nothing); ``cache_of[i]`` names the entry whose plane entry ``i`` reads instead.
    ``max_tokens`` is the number of tokens all live sequences may hold together, each
    sequence's length rounded up to whole pages of 64.
    """

    def __init__(self, kv_requests: Sequence[Optional[KvRequest]], cache_of: Sequence[Optional[int]],
                 state_requests: Sequence[Optional[StateRequest]], max_tokens: int, max_positions: int,
                 dtype: torch.dtype, device, max_seqs: Optional[int] = None, allocate: bool = True):
        if max_tokens <= 0 or max_positions <= 0:
            raise CacheError("max_tokens and max_positions must be positive")
        n_pages = pages_for(max_tokens)
        self.max_tokens = n_pages * PAGE
        self.max_positions = max_positions
        self.dtype, self.device = dtype, device
        n_slots = min(n_pages, max_seqs) if max_seqs else min(n_pages, 4096)
        self.slots = SlotTable(n_slots)
        pages_per_seq = min(pages_for(max_positions), n_pages)
        self.groups: List[KvGroup] = []
        self._plane: Dict[int, Tuple[int, int]] = {}  # schedule entry -> (group, plane)
        by_request: Dict[KvRequest, List[int]] = {}
        for i, req in enumerate(kv_requests):
            if req is not None and cache_of[i] is None:
                by_request.setdefault(req, []).append(i)
        for req, entries in by_request.items():
            g = KvGroup(req, entries, n_pages, n_slots, pages_per_seq, dtype, device, allocate)
            for plane, e in enumerate(entries):
                self._plane[e] = (len(self.groups), plane)
            self.groups.append(g)
        self._reader: Dict[int, int] = {}
        for i, src in enumerate(cache_of):
            if src is None:
                continue
            if src not in self._plane:
                raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which has none")
            a, b = kv_requests[i], kv_requests[src]
            if a is not None and (a.n_kv_heads, a.head_dim, a.v_dim) != (b.n_kv_heads, b.head_dim, b.v_dim):
                raise CacheError(f"schedule entry {i} cannot read entry {src}'s cache: "
                                 f"{a.n_kv_heads}x{a.head_dim}/{a.v_dim} against {b.n_kv_heads}x{b.head_dim}/{b.v_dim}")
            self._reader[i] = src
        self.states: Dict[int, torch.Tensor] = {}
        self.state_requests = {i: r for i, r in enumerate(state_requests) if r is not None}
        if allocate:
            for i, r in self.state_requests.items():
                self.states[i] = torch.zeros((n_slots,) + tuple(r.shape), dtype=r.dtype, device=device)

    # ---- slots ----------------------------------------------------------------------------
    def open(self) -> int:
        """A free slot for a new sequence: length 0, no pages, state zero."""
        slot = self.slots.open()
        for t in self.states.values():
            t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        """The sequence has ended: its pages and its slot are free for the next one."""
        self.slots.length(slot)  # raises if not open
        for g in self.groups:
            g.release(slot)
        self.slots.close(slot)

    def length(self, slot: int) -> int:
        return self.slots.length(slot)

    def reserve(self, slot: int, n_new: int) -> None:
        """Make room for ``n_new`` more tokens of the sequence in ``slot`` (nothing is held on failure)."""
        old = self.slots.length(slot)
        new = old + n_new
        if n_new <= 0:
            raise CacheError(f"a step must bring at least one token per sequence, got {n_new}")
        if new > self.max_positions:
            raise CacheFull(f"slot {slot}: {new} tokens exceed the context of {self.max_positions}")
        try:
            for g in self.groups:
                g.reserve(slot, old, new)
        except CacheFull:
            self.unreserve(slot)
            raise

    def unreserve(self, slot: int) -> None:
        """Give back pages held beyond what the sequence's present length needs."""
        keep = pages_for(self.slots.length(slot))
        for g in self.groups:
            held = g.held.get(slot, {})
            extra = [i for i in held if i >= keep]
            g.pool.free([held.pop(i) for i in extra])

    def advance(self, slot: int, n_new: int) -> None:
        """The step has run: the sequence is ``n_new`` tokens longer."""
        new = self.slots.length(slot) + n_new
        self.slots.set_length(slot, new)
        for g in self.groups:
            g.trim(slot, new)

    def sync(self) -> None:
        """Bring the device page tables up to date with the host's."""
        for g in self.groups:
            if not g.dirty or g.page_table is None:
                g.dirty.clear()
                continue
            rows = sorted(g.dirty)
            idx = torch.tensor(rows, dtype=torch.int64)
            staged = torch.from_numpy(g.host_table[rows]).pin_memory()
            g.page_table.index_copy_(0, idx.to(self.device, non_blocking=True),
                                     staged.to(self.device, non_blocking=True))
            g.dirty.clear()

    # ---- views ----------------------------------------------------------------------------
    def view(self, entry: int) -> Optional[KvView]:
        owner = entry in self._plane
        src = entry if owner else self._reader.get(entry)
        if src is None:
            return None
        gi, plane = self._plane[src]
        g = self.groups[gi]
        return KvView(k=g.k[plane], v=g.v[plane], page_table=g.page_table, n_kv_heads=g.request.n_kv_heads,
                      head_dim=g.request.head_dim, window=g.request.window, owner=owner,
                      v_head_dim=g.request.v_head_dim)

    def state(self, entry: int) -> Optional[torch.Tensor]:
        return self.states.get(entry)

    # ---- accounting -----------------------------------------------------------------------
    def tokens_free(self) -> int:
        return min((g.pool.n_free for g in self.groups), default=self.max_tokens // PAGE) * PAGE

    def bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(item) for g in self.groups)

    def check(self) -> None:
        """Invariants: no slot or page lost, held twice or freed twice; tables agree."""
        self.slots.check()
        active = set(self.slots.active())
        for g in self.groups:
            g.pool.check()
            seen: Dict[int, int] = {}
            for slot, held in g.held.items():
                if slot not in active and held:
                    raise CacheError(f"closed slot {slot} still holds pages")
                for i, p in held.items():
                    if p in seen:
                        raise CacheError(f"page {p} is held by slots {seen[p]} and {slot}")
                    seen[p] = slot
                    if g.host_table[slot, i] != p:
                        raise CacheError(f"page table of slot {slot} disagrees at index {i}")
            if len(seen) + g.pool.n_free != g.pool.n_pages:
                raise CacheError("pages are lost: held + free != total")
