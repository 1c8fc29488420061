"""The cache: a slot per sequence, keys and values per cache entry in pages of 64
positions, and per-sequence state of fixed size beside it.

The reference keeps, per layer, two persistent regions K and V of ``n_ctx`` positions
addressed by position (src/graph/alloc.rs:260-268, src/cache.rs:1-85), one whole set per
server slot (src/server/slot.rs:15-32), and has one kind of layer only.  Here:

* Storage is sized by the number of tokens that live sequences may hold together
  (``max_tokens``), in pages of 64 positions; a sequence takes pages as it grows and gives
  them all back when its slot is released, so later batches use them again.
* Cache entries with the same needs form a *group* with storage, pages and page tables of
  its own.  A group is either linear (every position is kept) or a ring of
  ``ceil((window + step_tokens - 1) / 64) * 64`` positions: a windowed mixer never reads
  further back than ``window`` positions, and a step writes its new positions before it
  attends, so a sequence may add up to ``ring - window + 1`` positions in one step without
  overwriting a position that the step's first new token still sees
  (``CacheGroup.max_new_positions``).  Whole prompts attend over the step's own keys and are
  not bound by this.
* Validity is a sequence's length, never a memset: a reused page still holds the last
  owner's values and nothing reads them.
* ``StatePool`` holds fixed-size state per slot (zeroed when the slot is handed out) for
  parts that ask for it, and for the sampler.

Layout of a group's storage: ``[entry][page][kv_head][64][head_dim]`` for K and for V (V with
its own last dimension where a mixer asks for values of another width).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

PAGE = 64


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


def pages_for(n_positions: int) -> int:
    return (n_positions + PAGE - 1) // PAGE


def ring_positions(window: int, step_tokens: int = 1) -> int:
    """Positions a ring keeps for a window of ``window`` when a sequence may add
    ``step_tokens`` positions in a step that reads the ring (0 for no window)."""
    if window <= 0:
        return 0
    return pages_for(window + max(1, int(step_tokens)) - 1) * PAGE


GUARD_BYTES = 256
GUARD_VALUE = 0xA5


class Guarded:
    """Device storage with a guard of 256 bytes before and after it.  The host writes a fixed
    value into the guards when the storage is made and reads them back on request: a kernel
    that wrote past either end of the tensor has changed them.  Costs nothing in a step."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, device: torch.device | str,
                 what: str):
        n_bytes = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.what = what
        self.raw = torch.empty(n_bytes + 2 * GUARD_BYTES, dtype=torch.uint8, device=device)
        self.raw[:GUARD_BYTES] = GUARD_VALUE
        self.raw[GUARD_BYTES + n_bytes:] = GUARD_VALUE
        body = self.raw[GUARD_BYTES:GUARD_BYTES + n_bytes]
        body.zero_()
        self.tensor = body.view(dtype).view(*shape)

    def intact(self) -> bool:
        n = self.raw.numel()
        ends = torch.cat([self.raw[:GUARD_BYTES], self.raw[n - GUARD_BYTES:]])
        return bool((ends == GUARD_VALUE).all().item())


class SlotTable:
    """Hands out slot numbers; a slot is held by at most one sequence at a time."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise CacheError("the cache needs at least one slot")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._held = [False] * n_slots
        self.length = [0] * n_slots

    def acquire(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.n_slots} sequence slots are in use")
        s = self._free.pop()
        self._held[s] = True
        self.length[s] = 0
        return s

    def release(self, slot: int) -> None:
        self.check(slot)
        self._held[slot] = False
        self.length[slot] = 0
        self._free.append(slot)

    def check(self, slot: int) -> None:
        if not isinstance(slot, int) or not 0 <= slot < self.n_slots:
            raise CacheError(f"slot {slot!r} is out of range (0..{self.n_slots - 1})")
        if not self._held[slot]:
            raise CacheError(f"slot {slot} is not held by any sequence (released twice?)")

    def held(self) -> List[int]:
        return [s for s in range(self.n_slots) if self._held[s]]

    def n_free(self) -> int:
        return len(self._free)


class PagePool:
    """Free list of a group's pages."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._owner: List[int] = [-1] * n_pages       # slot that holds the page, or -1

    def take(self, slot: int) -> int:
        if not self._free:
            raise OutOfPages(
                f"the cache has no free page left ({self.n_pages} pages of {PAGE} positions); "
                f"it was sized for fewer tokens than the live sequences now hold")
        p = self._free.pop()
        self._owner[p] = slot
        return p

    def give_back(self, page: int, slot: int) -> None:
        if not 0 <= page < self.n_pages:
            raise CacheError(f"page {page} is out of range")
        if self._owner[page] != slot:
            raise CacheError(
                f"page {page} is returned by slot {slot} but is held by {self._owner[page]}")
        self._owner[page] = -1
        self._free.append(page)

    def n_free(self) -> int:
        return len(self._free)

    def owner(self, page: int) -> int:
        return self._owner[page]


@dataclass(frozen=True)
class GroupKey:
    n_kv_heads: int
    head_dim: int
    window: int          # 0: linear
    value_dim: int = 0   # width of a value vector if it differs from head_dim (0: the same)


class CacheGroup:
    """Storage, pages and page tables of the cache entries that share one ``GroupKey``."""

    def __init__(self, key: GroupKey, entries: Sequence[int], n_pages: int, n_slots: int,
                 dtype: torch.dtype, device: torch.device | str, step_tokens: int = 1):
        self.key = key
        self.entries = list(entries)
        self.ring = ring_positions(key.window, step_tokens)
        self.n_pages = n_pages
        self.pool = PagePool(n_pages)
        self.pages: List[List[int]] = [[] for _ in range(n_slots)]
        # one page more than the pool hands out: the spare page, for rows that only fill a batch
        # up to a size the engine has a captured graph for
        self.spare_page = n_pages
        # the page lists once more as one integer table (a row per slot, -1 where a sequence
        # has no page, the spare slot's row last): a step's page tables are one slice of it
        self._table = np.full((n_slots + 1, 8), -1, dtype=np.int32)
        self._table[n_slots, 0] = self.spare_page
        shape = (len(self.entries), n_pages + 1, key.n_kv_heads, PAGE, key.head_dim)
        v_shape = shape[:-1] + (key.value_dim or key.head_dim,)
        # zeros, once: a page's unwritten positions are masked by length but still multiplied
        # by a zero weight in the tensor-core kernels, so they must never hold NaN or Inf
        self._guarded = [Guarded(shape, dtype, device, f"keys of cache group {key}"),
                         Guarded(v_shape, dtype, device, f"values of cache group {key}")]
        self.k = self._guarded[0].tensor
        self.v = self._guarded[1].tensor
        self._index = {e: i for i, e in enumerate(self.entries)}

    def max_new_positions(self) -> Optional[int]:
        """Most positions a sequence may add in one step whose tokens attend over this group's
        storage (None: no bound).  Position ``p`` lies at ``p % ring``; the first new token at
        ``s`` sees back to ``s - window + 1``, which the write of ``s + n - 1`` must not reach:
        ``n <= ring - window + 1``."""
        if not self.ring:
            return None
        return self.ring - self.key.window + 1

    def pages_needed(self, length: int) -> int:
        need = pages_for(length)
        if self.ring:
            need = min(need, self.ring // PAGE)
        return need

    def ensure(self, slot: int, length: int) -> None:
        """Pages so that a sequence of ``length`` positions can be written."""
        have = self.pages[slot]
        need = self.pages_needed(length)
        while len(have) < need:
            have.append(self.pool.take(slot))
            if len(have) > self._table.shape[1]:
                wider = np.full((self._table.shape[0], 2 * self._table.shape[1]), -1, dtype=np.int32)
                wider[:, :self._table.shape[1]] = self._table
                self._table = wider
            self._table[slot, len(have) - 1] = have[-1]

    def release(self, slot: int) -> None:
        for p in self.pages[slot]:
            self.pool.give_back(p, slot)
        self.pages[slot] = []
        self._table[slot, :] = -1

    def entry_tensors(self, entry: int) -> Tuple[torch.Tensor, torch.Tensor]:
        i = self._index[entry]
        return self.k[i], self.v[i]

    def table_rows(self, slots: Sequence[int], width: int) -> List[List[int]]:
        rows = []
        for s in slots:
            pg = [self.spare_page] if s == len(self.pages) else self.pages[s]   # the spare slot
            if len(pg) > width:
                raise CacheError("the page table is narrower than a sequence's pages")
            rows.append(pg + [-1] * (width - len(pg)))
        return rows

    def table_flat(self, slots: Sequence[int], width: int) -> List[int]:
        """``table_rows`` row after row in one list, from the integer table."""
        if self.max_pages_of(slots) > width:
            raise CacheError("the page table is narrower than a sequence's pages")
        have = self._table.shape[1]
        if width <= have:
            return self._table[list(slots), :width].ravel().tolist()
        out = np.full((len(slots), width), -1, dtype=np.int32)
        out[:, :have] = self._table[list(slots)]
        return out.ravel().tolist()

    def max_pages_of(self, slots: Sequence[int]) -> int:
        return max((len(self.pages[s]) for s in slots if s < len(self.pages)), default=0)


class StatePool:
    """Fixed-size state per slot: one tensor ``[n_slots, *shape]`` per name."""

    def __init__(self, n_slots: int, device: torch.device | str):
        self.n_slots = n_slots
        self.device = device
        self.tensors: Dict[str, torch.Tensor] = {}
        self._guarded: List[Guarded] = []

    def add(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        if name in self.tensors:
            raise CacheError(f"state '{name}' is already defined")
        g = Guarded((self.n_slots, *shape), dtype, self.device, f"state '{name}'")
        self._guarded.append(g)
        self.tensors[name] = g.tensor
        return g.tensor

    def reset(self, slot: int) -> None:
        for t in self.tensors.values():
            t[slot].zero_()

    def bytes_per_slot(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.tensors.values())


class Cache:
    """Slots, groups and state together.  ``requests`` maps a cache entry to the
    ``GroupKey`` of the mixer that writes it."""

    def __init__(self, requests: Dict[int, GroupKey], max_tokens: int, max_seqs: int,
                 dtype: torch.dtype, device: torch.device | str, step_tokens: int = 1):
        if max_tokens <= 0 or max_tokens % PAGE != 0:
            raise CacheError(f"max_tokens must be a positive multiple of {PAGE}, got {max_tokens}")
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.dtype = dtype
        self.device = device
        self.slots = SlotTable(max_seqs)
        # one state row more than there are slots: the spare slot (index max_seqs), never handed
        # out; rows that only pad a batch point at it and at each group's spare page
        self.spare_slot = max_seqs
        self.state = StatePool(max_seqs + 1, device)
        by_key: Dict[GroupKey, List[int]] = {}
        for entry in sorted(requests):
            by_key.setdefault(requests[entry], []).append(entry)
        self.groups: List[CacheGroup] = []
        self.group_of: Dict[int, CacheGroup] = {}
        total_pages = max_tokens // PAGE
        for key, entries in by_key.items():
            n_pages = total_pages
            if key.window > 0:
                n_pages = min(total_pages, max_seqs * (ring_positions(key.window, step_tokens) // PAGE))
            g = CacheGroup(key, entries, n_pages, max_seqs, dtype, device, step_tokens)
            self.groups.append(g)
            for e in entries:
                self.group_of[e] = g

    # ---- slots --------------------------------------------------------------------------
    def acquire(self) -> int:
        s = self.slots.acquire()
        self.state.reset(s)
        return s

    def release(self, slot: int) -> None:
        self.slots.check(slot)
        for g in self.groups:
            g.release(slot)
        self.slots.release(slot)

    def length(self, slot: int) -> int:
        self.slots.check(slot)
        return self.slots.length[slot]

    def reserve(self, slot: int, new_length: int) -> None:
        """Pages in every group for a sequence that grows to ``new_length``."""
        self.slots.check(slot)
        for g in self.groups:
            g.ensure(slot, new_length)

    def set_length(self, slot: int, length: int) -> None:
        self.slots.check(slot)
        self.slots.length[slot] = length

    def max_new_positions(self) -> Optional[int]:
        """Most tokens a sequence may bring in one step that attends over the cache (None: no
        bound): the smallest bound of the groups."""
        bounds = [b for b in (g.max_new_positions() for g in self.groups) if b is not None]
        return min(bounds) if bounds else None

    def check_canaries(self) -> None:
        """Raises if a guard before or after a group's keys or values or a state tensor no longer
        holds the value the host wrote there (reads the device: a sync; for tests and audits)."""
        broken = [g.what for group in self.groups for g in group._guarded if not g.intact()]
        broken += [g.what for g in self.state._guarded if not g.intact()]
        if broken:
            raise CacheError("something wrote outside " + "; ".join(broken))

    def bytes(self) -> int:
        """Bytes of key/value storage that sequences can hold (the spare pages not counted)."""
        return sum(2 * g.k[:, :g.n_pages].numel() * g.k.element_size() for g in self.groups)

    def free_pages(self) -> List[int]:
        return [g.pool.n_free() for g in self.groups]
