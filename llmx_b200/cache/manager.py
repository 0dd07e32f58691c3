"""The cache manager: paged keys and values by group, and slots of fixed-size state.

What a mixer needs of the cache is declared, not assumed: `KVSpec` (keys and
values of `kv_heads x head_dim` per token, all of them or a window of them) or
`StateSpec` (a tensor of fixed shape per request), or nothing.  Cache entries
with the same KVSpec form a *group*: one page pool, one block table per
request, and page id p naming the same page in every member's storage (as the
reference's page id does across the layers of one storage,
src/backends/backend.hpp:238-242).  Groups with different needs have pools of
their own, so a windowed group can give pages back while a full group keeps
them.  The reference keeps one KV geometry per model and refuses a mix
(src/model/runtime.hpp:531-533); here the mix is the point.

Storage of one member: `[num_pages, 2, kv_heads, page_size, head_dim]`, plane 0
keys and plane 1 values, so one (page, head) run of keys is contiguous
(`page_size * head_dim` elements), which is what a bulk copy wants.

State: `StateSlots` hands out slot ids; each state entry owns
`[num_slots, *shape]`.  A request takes one slot for its life.  A mixer must
treat the state as zero at a request's first token whatever the slot holds
(the reference's rule, src/backends/backend.hpp:386-393), so recycled slots
are not cleared.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple, Union

from .pages import BlockTable, CacheExhausted, PagePool


@dataclass(frozen=True)
class KVSpec:
    kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every key is kept


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]
    dtype: str = "float32"            # a torch dtype name


CacheSpec = Union[KVSpec, StateSpec, None]


class StateSlots:
    """Slot ids for fixed-size per-request state.

    A live request holds two: the one its state lies in and a spare.  A step reads the first and writes the
    second (`RequestCache.state_slot` / `state_slot_out`), and commit swaps them, so a step that fails leaves
    the state as it was without anything being copied (the reference keeps checkpoints of its state slots for
    the same end, src/model/kv_cache.hpp:183-278)."""

    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._held = [False] * self.num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheExhausted(f"state slots: all {self.num_slots} are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise RuntimeError(f"state slot {slot} given back twice")
        self._held[slot] = False
        self._free.append(slot)

    def check(self) -> None:
        if len(set(self._free)) != len(self._free):
            raise AssertionError("a state slot is free twice")
        for s in range(self.num_slots):
            if self._held[s] == (s in self._free):
                raise AssertionError(f"state slot {s} is both held and free, or neither")


class CacheGroup:
    """Cache entries that share page geometry, a pool and the requests' block tables."""

    def __init__(self, spec: KVSpec, members: List[int], page_size: int, num_pages: int):
        self.spec = spec
        self.members = members            # cache entry indices, in storage order
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.storage = None               # torch tensor [len(members), num_pages, 2, G, page, D] once allocated

    def bytes_per_page(self, element_size: int) -> int:
        return len(self.members) * 2 * self.spec.kv_heads * self.page_size * self.spec.head_dim * element_size


class RequestCache:
    """Everything one live request holds: a block table per group and a state slot."""

    def __init__(self, manager: "CacheManager", request_id: Hashable):
        self.manager = manager
        self.request_id = request_id
        self.tables: List[BlockTable] = [BlockTable(g.pool, g.page_size, g.spec.window) for g in manager.groups]
        self.state_slot: int = -1          # where the request's state lies (read by a step)
        self.state_slot_out: int = -1      # where a step writes the state it leaves; the two swap at commit
        if manager.has_state:
            self.state_slot = manager.state_slots.take()
            try:
                self.state_slot_out = manager.state_slots.take()
            except CacheExhausted:
                manager.state_slots.give_back(self.state_slot)
                raise
        self.length = 0
        self.pending = 0
        self.freed = False

    def prepare(self, n: int) -> None:
        """Reserve room for n more tokens in every group, or in none."""
        done: List[BlockTable] = []
        try:
            for t in self.tables:
                t.prepare(n)
                done.append(t)
        except CacheExhausted:
            for t in done:
                t.abort()
            raise
        self.pending = n

    def commit(self) -> None:
        for t in self.tables:
            t.commit()
        if self.pending:
            self.state_slot, self.state_slot_out = self.state_slot_out, self.state_slot
        self.length += self.pending
        self.pending = 0

    def abort(self) -> None:
        """Undo a prepare: pages taken for the step go back; the state the step may have written went to the
        spare slot, so the request's state is what it was."""
        for t in self.tables:
            t.abort()
        self.pending = 0

    def truncate(self, length: int) -> None:
        """Roll the request back to `length` tokens (the reference's KVSequence::truncate,
        src/model/kv_cache.hpp:126-130).  Keys beyond are forgotten and their pages given back.  A request with
        fixed-size state cannot be rolled back (the state has no history), nor can a windowed group below what
        its window has given back."""
        if self.pending:
            raise RuntimeError("KV cache: a step is in progress for this request")
        if not 0 <= length <= self.length:
            raise ValueError(f"cannot truncate a request of {self.length} tokens to {length}")
        if length == self.length:
            return
        if self.state_slot >= 0:
            raise RuntimeError("a request whose layers keep fixed-size state cannot be rolled back")
        for t in self.tables:
            if t.window is not None and length < t._first_live * t.page_size:
                raise RuntimeError("KV cache: cannot roll back into pages the window has given back")
        for t in self.tables:
            t.truncate(length)
        self.length = length

    def held_pages(self) -> List[int]:
        return [t.held_pages for t in self.tables]

    def free(self) -> None:
        if self.freed:
            raise RuntimeError(f"request {self.request_id!r}: cache freed twice")
        for t in self.tables:
            t.free()
        for slot in (self.state_slot, self.state_slot_out):
            if slot >= 0:
                self.manager.state_slots.give_back(slot)
        self.state_slot = self.state_slot_out = -1
        self.freed = True
        self.length = self.pending = 0


class CacheManager:
    """Builds the groups from the model's cache entries and owns the device storage.

    `entry_specs[i]` is what cache entry i needs (the model's layer order names
    entries by index; two steps of the order may name the same entry, so that a
    layer reads another layer's keys).
    """

    def __init__(self, entry_specs: Sequence[CacheSpec], page_size: int, kv_tokens: int,
                 max_requests: int, kv_dtype=None, device=None, window_kv_tokens: Optional[int] = None):
        """`kv_tokens`: tokens the pool of every group that keeps all keys is made for; `window_kv_tokens`: the
        same for groups that keep a window (default: as many; a windowed group holds at most its window, two
        pages and the step's portion per request, so it can be made much smaller)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = int(page_size)
        self.entry_specs = list(entry_specs)
        self.kv_tokens = int(kv_tokens)
        self.window_kv_tokens = self.kv_tokens if window_kv_tokens is None else int(window_kv_tokens)
        self.max_requests = int(max_requests)
        by_spec: Dict[KVSpec, List[int]] = {}
        for i, s in enumerate(self.entry_specs):
            if isinstance(s, KVSpec):
                by_spec.setdefault(s, []).append(i)
        self.groups: List[CacheGroup] = [
            CacheGroup(s, m, self.page_size, (self.kv_tokens if s.window is None else self.window_kv_tokens) // self.page_size)
            for s, m in by_spec.items()]
        self.group_of_entry: Dict[int, Tuple[int, int]] = {}
        for gi, g in enumerate(self.groups):
            for mi, e in enumerate(g.members):
                self.group_of_entry[e] = (gi, mi)
        self.state_entries = [i for i, s in enumerate(self.entry_specs) if isinstance(s, StateSpec)]
        self.has_state = bool(self.state_entries)
        self.state_slots = StateSlots(2 * self.max_requests if self.has_state else 0)
        self.state_storage: Dict[int, object] = {}
        self.live: Dict[Hashable, RequestCache] = {}
        self.kv_dtype = kv_dtype
        self.device = device
        self.views = None                 # the entries as the native runtime sees them (runtime.CacheViews)
        if device is not None:
            self._allocate()

    def _allocate(self) -> None:
        import torch
        for g in self.groups:
            s = g.spec
            # Zero-filled: a kernel may load (and mask) slots of a page that were never written.
            g.storage = torch.zeros((len(g.members), g.pool.num_pages, 2, s.kv_heads, g.page_size, s.head_dim),
                                    dtype=self.kv_dtype, device=self.device)
        for e in self.state_entries:
            s = self.entry_specs[e]
            self.state_storage[e] = torch.zeros((self.state_slots.num_slots,) + tuple(s.shape),
                                                dtype=getattr(torch, s.dtype), device=self.device)
        if torch.device(self.device).type == "cuda":
            from .. import runtime
            # The runtime's view of the entries owns the kernels' descriptors of the storage, so that they go when
            # the cache goes.
            self.views = runtime.CacheViews(len(self.entry_specs))
            for e in range(len(self.entry_specs)):
                gi, storage = self.entry_storage(e) if (e in self.group_of_entry or e in self.state_storage) else (None, None)
                if storage is None:
                    continue
                if gi >= 0:
                    self.views.set_kv(e, gi, storage)
                else:
                    self.views.set_state(e, storage)

    # -- requests -------------------------------------------------------------
    def new_request(self, request_id: Hashable) -> RequestCache:
        if request_id in self.live:
            raise RuntimeError(f"request {request_id!r} is already live")
        rc = RequestCache(self, request_id)
        self.live[request_id] = rc
        return rc

    def free_request(self, request_id: Hashable) -> None:
        self.live.pop(request_id).free()

    # -- accounting -----------------------------------------------------------
    def pages_needed(self, tokens: int, step_tokens: int = 1) -> List[int]:
        """Pages a request of `tokens` positions holds at most, per group.

        A windowed group holds its window, the page the window starts in, and the
        portion being written (`step_tokens`), never more than the whole history.
        """
        out = []
        for g in self.groups:
            if g.spec.window is None:
                held = tokens
            else:
                held = min(tokens, g.spec.window + g.page_size + max(step_tokens, 1) + g.page_size)
            out.append(-(-held // g.page_size))
        return out

    def free_pages(self) -> List[int]:
        return [g.pool.free_pages for g in self.groups]

    def used_pages(self) -> List[int]:
        return [g.pool.used_pages for g in self.groups]

    def total_pages(self) -> List[int]:
        return [g.pool.num_pages for g in self.groups]

    def storage_bytes(self) -> int:
        total = 0
        for g in self.groups:
            if g.storage is not None:
                total += g.storage.numel() * g.storage.element_size()
        return total

    def entry_storage(self, entry: int):
        """(group index, this entry's [num_pages, 2, G, page, D] storage) or the state tensor."""
        if entry in self.group_of_entry:
            gi, mi = self.group_of_entry[entry]
            return gi, self.groups[gi].storage[mi]
        return -1, self.state_storage[entry]

    def check(self) -> None:
        """No page lost, held twice or freed twice: the pools' counts equal what live requests hold."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            held: Dict[int, int] = {}
            for rc in self.live.values():
                t = rc.tables[gi]
                for p in t.pages[t._first_live:]:
                    held[p] = held.get(p, 0) + 1
            for p in range(g.pool.num_pages):
                if g.pool.refs(p) != held.get(p, 0):
                    raise AssertionError(f"group {gi} page {p}: pool counts {g.pool.refs(p)} holders, requests hold {held.get(p, 0)}")
        self.state_slots.check()
