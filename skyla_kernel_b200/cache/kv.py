"""The cache: a slot per sequence, paged keys and values per group of layers,
and a fixed-size state area per slot.

The reference keeps one flat f16 buffer indexed ``slot(layer) * max_ctx * kv_dim``
for the one sequence it serves, gives a cache index only to layers that cache
(skyla-engine/src/kv.rs:34-49,68-75) and keeps the fixed-size state of recurrent
layers in regions that are zeroed together on reset
(skyla-engine/src/arena.rs:114-142, engine.rs:82-89).  Here many sequences share
the memory, so positions live in pages:

* layers whose mixers have the same need (key/value heads, head size, window, precision)
  form a *group* with one pool ``[layer, page, kv_head, position_in_page, head_dim]``
  for keys and one for values, and a page list per slot;
* a group with a window gives back the pages that no later token can see;
* every slot also owns ``state`` tensors, one per layer that asks for fixed-size
  state, zeroed when the slot is handed out.

Kernels never see slots: each step uploads, for the sequences it runs, their
page lists (see engine/batch.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .slots import CacheError, CacheFull, FreeList

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVNeed:
    """What an attention-like mixer asks of the cache."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: every earlier position stays visible
    #: precision of the stored keys and values; None: the runtime's (bfloat16, or float32 in the 32-bit
    #: path).  Mixers with different precisions fall into different groups, like any other difference.
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence: a tensor of ``shape`` per slot, zero at the start."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class KVGroup:
    """Storage of the layers that share one :class:`KVNeed`."""

    def __init__(self, need: KVNeed, n_layers: int, n_pages: int, max_slots: int,
                 dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        self.need = need
        self.n_layers = n_layers
        self.page_size = page_size
        self.n_pages = n_pages
        self.pages = FreeList(n_pages, "cache page")
        self.dtype = dtype = need.dtype or dtype
        shape = (n_layers, n_pages, need.num_kv_heads, page_size, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device) if device is not None else None
        self.v = torch.zeros(shape, dtype=dtype, device=device) if device is not None else None
        # per slot: page number for each page index, -1 where none is held
        self.slot_pages: List[List[int]] = [[] for _ in range(max_slots)]

    def bytes_per_token(self) -> int:
        esize = torch.empty((), dtype=self.dtype).element_size()
        return 2 * self.n_layers * self.need.num_kv_heads * self.need.head_dim * esize

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.slot_pages[slot])
        return max(0, -(-new_len // self.page_size) - have)

    def grow(self, slot: int, new_len: int) -> None:
        for _ in range(self.pages_needed(slot, new_len)):
            self.slot_pages[slot].append(self.pages.take())

    def trim(self, slot: int, length: int) -> None:
        """Give back the pages that lie wholly before the window of the next token."""
        w = self.need.window
        if not w:
            return
        first_visible = max(0, length - w + 1)  # the next token sits at `length`
        lst = self.slot_pages[slot]
        for j in range(min(first_visible // self.page_size, len(lst))):
            if lst[j] >= 0:
                self.pages.give_back(lst[j])
                lst[j] = -1

    def release(self, slot: int) -> None:
        for p in self.slot_pages[slot]:
            if p >= 0:
                self.pages.give_back(p)
        self.slot_pages[slot] = []


class SequenceCache:
    """All groups, the state area and the slots, sized once.

    ``max_tokens`` bounds, per group, the positions held by live sequences, each
    sequence's count rounded up to a whole page.
    """

    def __init__(self, kv_needs: List[Optional[KVNeed]], state_needs: List[Optional[StateNeed]],
                 max_tokens: int, max_slots: Optional[int], dtype: torch.dtype, device,
                 page_size: int = PAGE_SIZE):
        """``kv_needs[i]`` / ``state_needs[i]``: what cache entry ``i`` asks for (``None``: nothing)."""
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        self.page_size = page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_slots = max_slots or self.n_pages
        self.slots = FreeList(self.max_slots, "sequence slot")
        self.lengths = [0] * self.max_slots
        self.device = device
        self.dtype = dtype
        # group the entries by need
        self.groups: List[KVGroup] = []
        self.entry_group: List[Optional[Tuple[int, int]]] = []  # entry -> (group, layer in group)
        by_need: Dict[KVNeed, List[int]] = {}
        for i, need in enumerate(kv_needs):
            if need is not None:
                by_need.setdefault(need, []).append(i)
        self.entry_group = [None] * len(kv_needs)
        for need, entries in by_need.items():
            g = len(self.groups)
            self.groups.append(KVGroup(need, len(entries), self.n_pages, self.max_slots, dtype,
                                       device, page_size))
            for j, e in enumerate(entries):
                self.entry_group[e] = (g, j)
        self.state: List[Optional[torch.Tensor]] = []
        for need in state_needs:
            if need is None or device is None:
                self.state.append(None)
            else:
                self.state.append(torch.zeros((self.max_slots,) + tuple(need.shape),
                                              dtype=need.dtype, device=device))
        self.state_needs = state_needs

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        s = self.slots.take()
        self.lengths[s] = 0
        for st in self.state:
            if st is not None:
                st[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.give_back(slot)  # raises on a slot that is not held
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        self._held(slot)
        return self.lengths[slot]

    def _held(self, slot: int) -> None:
        if not self.slots.held(slot):
            raise CacheError(f"slot {slot} is not in use")

    # ------------------------------------------------------------------ pages
    def reserve(self, growth: List[Tuple[int, int]]) -> None:
        """Make room for ``n`` more positions in each ``(slot, n)``, all or nothing."""
        seen = set()
        for slot, n in growth:
            self._held(slot)
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n <= 0:
                raise CacheError(f"slot {slot}: a step must bring at least one token")
        for g in self.groups:
            need = sum(g.pages_needed(s, self.lengths[s] + n) for s, n in growth)
            if need > g.pages.n_free:
                raise CacheFull(
                    f"cache full: the step needs {need} more pages of {g.page_size} positions, "
                    f"{g.pages.n_free} of {g.n_pages} are free")
        for g in self.groups:
            for s, n in growth:
                g.grow(s, self.lengths[s] + n)

    def advance(self, growth: List[Tuple[int, int]]) -> None:
        """The step ran: lengths move on and windowed groups give back dead pages."""
        for slot, n in growth:
            self.lengths[slot] += n
            for g in self.groups:
                g.trim(slot, self.lengths[slot])

    def pages_of(self, group: int, slot: int) -> List[int]:
        return self.groups[group].slot_pages[slot]

    def kv_of_entry(self, entry: int):
        """(group index, key pool, value pool) of one cache entry's layer."""
        gi = self.entry_group[entry]
        if gi is None:
            raise CacheError(f"cache entry {entry} holds no keys and values")
        g = self.groups[gi[0]]
        return gi[0], g.k[gi[1]], g.v[gi[1]]

    def state_of_entry(self, entry: int) -> Optional[torch.Tensor]:
        return self.state[entry]

    def tokens_held(self) -> int:
        return max((g.pages.n_held for g in self.groups), default=0) * self.page_size

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

    def check(self) -> None:
        """Invariants for tests: nothing lost, nothing held twice."""
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            owned = [p for lst in g.slot_pages for p in lst if p >= 0]
            assert len(owned) == len(set(owned)), "a page is held by two sequences"
            assert len(owned) == g.pages.n_held, "a page is held by no sequence"
            for s, lst in enumerate(g.slot_pages):
                assert not lst or self.slots.held(s), "a free slot still holds pages"
