"""The cache of a model: a slot per live sequence, paged keys and values per
cache line, and fixed-size state per sequence.

* A *slot* is the handle of one sequence: its length and what it holds.  Slots
  are given back when a sequence ends and are used again.
* A *cache line* is what one entry of the layer schedule reads and writes; the
  mixer of the layer that writes it says what it needs: `KVNeed` (keys and values
  of every position, or of a window of them) and/or `StateNeed` (a tensor of
  fixed shape per sequence).
* Lines with the same need form a *group* with storage of its own.  A KV group
  is a pool of pages of PAGE tokens, `[lines, pages, kv heads, PAGE, head size]`
  for keys and the same for values, and a page table `[slots, pages per sequence]`
  shared by the group's lines (a sequence has the same length in all of them).
  A windowed group is a ring: position p lives at p mod ring, ring = the window
  rounded up to whole pages, so a sequence never holds more than ring / PAGE
  pages there.  A state group is `[lines, slots, *shape]`, zeroed when a slot
  is handed out.

The host owns all bookkeeping (free lists, tables, lengths); the device copy of
a page table is refreshed when it changed.  Everything here is checked: a page
or slot is never handed out twice, never freed twice, and `audit()` proves that
none is lost.

The reference keeps one growing `[1, n_kv, T, hd]` pair per layer for its single
sequence (`qwen/cache.go:30-39`, `:90-111`) and chooses the kind of cache per
layer (`qwen/session.go:49-51`, `:157-162`); its fixed-size state is the linear
attention cache (`qwen35/deltanet.go:16-29`).  Slots over persistent tensors with
host-side maps and a free-first policy follow `qwen/slotcache.go:35-46`, `:242-257`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Sequence

import numpy as np
import torch

PAGE = 64


class CacheError(RuntimeError):
    """Misuse of the cache: unknown slot, double free, and the like."""


class CacheFull(CacheError):
    """No free slot or page is left."""


@dataclass(frozen=True)
class KVNeed:
    n_kv_heads: int
    head_dim: int
    window: int | None = None      # None: every position is kept


@dataclass(frozen=True)
class StateNeed:
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class PagePool:
    """Free list of page numbers 0 .. n-1."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))   # pop() hands out low numbers first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise CacheFull(f"cache is full: {n} pages wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise CacheError(f"page {p} handed out twice")
            self._held[p] = True
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not (0 <= p < self.n_pages) or not self._held[p]:
                raise CacheError(f"page {p} freed but not held")
            self._held[p] = False
            self._free.append(p)

    def audit(self, held_pages: Sequence[int]) -> None:
        held = sorted(held_pages)
        if len(set(held)) != len(held):
            raise CacheError("a page is held by two sequences")
        if sorted(self._free) != sorted(set(range(self.n_pages)) - set(held)):
            raise CacheError("free list and held pages do not add up to the pool")


class KVGroup:
    """Storage of the cache lines that share one KVNeed."""

    def __init__(self, need: KVNeed, lines: list[int], n_pages: int, n_slots: int, max_ctx: int,
                 dtype: torch.dtype, device):
        self.need = need
        self.lines = list(lines)
        self.ring_len = round_up(need.window, PAGE) if need.window else 0
        span = self.ring_len if self.ring_len else round_up(max_ctx, PAGE)
        self.pages_per_seq = max(1, min(n_pages, span // PAGE))
        self.pool = PagePool(n_pages)
        self.table_host = np.zeros((n_slots, self.pages_per_seq), dtype=np.int32)
        self.table = torch.zeros((n_slots, self.pages_per_seq), dtype=torch.int32, device=device)
        shape = (len(lines), n_pages, need.n_kv_heads, PAGE, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.held: dict[int, list[int]] = {}
        self.dirty = False

    def pages_for(self, length: int) -> int:
        span = min(length, self.ring_len) if self.ring_len else length
        return (span + PAGE - 1) // PAGE

    def ensure(self, slot: int, length: int) -> None:
        """Make room for positions < length of the sequence in `slot`."""
        have = self.held.setdefault(slot, [])
        want = self.pages_for(length)
        if want > self.pages_per_seq:
            raise CacheFull(f"sequence of {length} tokens needs {want} pages, a sequence may hold "
                            f"{self.pages_per_seq}")
        if want > len(have):
            new = self.pool.alloc(want - len(have))
            self.table_host[slot, len(have):len(have) + len(new)] = new
            have.extend(new)
            self.dirty = True

    def release(self, slot: int) -> None:
        pages = self.held.pop(slot, [])
        self.pool.free(pages)
        if pages:
            self.table_host[slot, :] = 0
            self.dirty = True

    def sync(self) -> None:
        if self.dirty:
            self.table.copy_(torch.from_numpy(self.table_host))
            self.dirty = False

    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


class StateGroup:
    """Fixed-size state: [lines, slots, *shape]."""

    def __init__(self, need: StateNeed, lines: list[int], n_slots: int, device):
        self.need = need
        self.lines = list(lines)
        self.data = torch.zeros((len(lines), n_slots) + tuple(need.shape), dtype=need.dtype, device=device)

    def reset(self, slot: int) -> None:
        self.data[:, slot].zero_()


@dataclass
class KVLine:
    """What a mixer sees of its key/value cache line."""
    group: KVGroup
    k: torch.Tensor            # [pages, kv heads, PAGE, head size]
    v: torch.Tensor
    write: bool

    @property
    def table(self) -> torch.Tensor:
        return self.group.table

    @property
    def ring_len(self) -> int:
        return self.group.ring_len

    @property
    def window(self) -> int:
        return self.group.need.window or 0


@dataclass
class StateLine:
    group: StateGroup
    data: torch.Tensor         # [slots, *shape]
    write: bool


@dataclass
class CacheLine:
    """One schedule entry's view of the cache: its parts by the names the mixer gave them."""
    index: int
    write: bool
    parts: dict = field(default_factory=dict)
    has_readers: bool = False      # another schedule entry reads what this one writes

    def __getitem__(self, name: str):
        return self.parts[name]


class ModelCache:
    def __init__(self, line_needs: Sequence[Mapping[str, object]], max_tokens: int, max_ctx: int,
                 dtype: torch.dtype, device, max_seqs: int | None = None):
        if max_tokens < 1:
            raise CacheError("max_tokens must be positive")
        self.max_ctx = max_ctx
        self.n_pages = round_up(max_tokens, PAGE) // PAGE
        self.n_slots = max(1, min(max_seqs if max_seqs else self.n_pages, self.n_pages))
        self.device = device
        self.kv_groups: dict[KVNeed, KVGroup] = {}
        self.state_groups: dict[StateNeed, StateGroup] = {}
        self._line_parts: list[dict[str, tuple[object, int]]] = []
        kv_lines: dict[KVNeed, list[int]] = {}
        st_lines: dict[StateNeed, list[int]] = {}
        for i, needs in enumerate(line_needs):
            for name, need in (needs or {}).items():
                if isinstance(need, KVNeed):
                    kv_lines.setdefault(need, []).append(i)
                elif isinstance(need, StateNeed):
                    st_lines.setdefault(need, []).append(i)
                else:
                    raise CacheError(f"cache line {i}: unknown need {need!r} for {name!r}")
        group_pages = {}
        for need, lines in kv_lines.items():
            n_pages = self.n_pages
            if need.window:
                n_pages = min(n_pages, self.n_slots * (round_up(need.window, PAGE) // PAGE))
            group_pages[need] = n_pages
        self._check_room(kv_lines, st_lines, group_pages, max_tokens, dtype, device)
        for need, lines in kv_lines.items():
            self.kv_groups[need] = KVGroup(need, lines, group_pages[need], self.n_slots, max_ctx, dtype, device)
        for need, lines in st_lines.items():
            self.state_groups[need] = StateGroup(need, lines, self.n_slots, device)
        for i, needs in enumerate(line_needs):
            parts = {}
            for name, need in (needs or {}).items():
                g = self.kv_groups[need] if isinstance(need, KVNeed) else self.state_groups[need]
                parts[name] = (g, g.lines.index(i))
            self._line_parts.append(parts)
        self._free_slots = list(range(self.n_slots - 1, -1, -1))
        self._live: dict[int, int] = {}            # slot -> length

    def _check_room(self, kv_lines, st_lines, group_pages, max_tokens, dtype, device) -> None:
        """Refuse, with the sizes, a cache that the device has no room for (before anything is allocated)."""
        item = torch.empty((), dtype=dtype).element_size()
        sizes = []
        for need, lines in kv_lines.items():
            b = 2 * len(lines) * group_pages[need] * need.n_kv_heads * PAGE * need.head_dim * item
            kind = f"window {need.window}" if need.window else "all positions"
            sizes.append((f"{len(lines)} lines of {need.n_kv_heads} x {need.head_dim} keys and values, {kind}", b))
        for need, lines in st_lines.items():
            n = 1
            for d in need.shape:
                n *= int(d)
            b = len(lines) * self.n_slots * n * torch.empty((), dtype=need.dtype).element_size()
            sizes.append((f"{len(lines)} lines of state {tuple(need.shape)}", b))
        self.planned_bytes = sum(b for _, b in sizes)
        dev = torch.device(device)
        if dev.type != "cuda":
            return
        free, total = torch.cuda.mem_get_info(dev)
        free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)     # what the allocator holds unused
        if self.planned_bytes > free:
            gib = lambda b: f"{b / 2 ** 30:.2f} GiB"
            parts = "; ".join(f"{what}: {gib(b)}" for what, b in sizes)
            raise CacheFull(f"a cache of {max_tokens} tokens ({self.n_pages} pages, {self.n_slots} sequences) needs "
                            f"{gib(self.planned_bytes)} ({parts}); the device has {gib(free)} free of {gib(total)} "
                            "(the rest holds the weights and other allocations): ask for fewer tokens")

    # -- slots ------------------------------------------------------------
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def alloc_slot(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"no free slot: all {self.n_slots} are in use")
        slot = self._free_slots.pop()
        if slot in self._live:
            raise CacheError(f"slot {slot} handed out twice")
        self._live[slot] = 0
        for g in self.state_groups.values():
            g.reset(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        if slot not in self._live:
            raise CacheError(f"slot {slot} freed but not in use")
        for g in self.kv_groups.values():
            g.release(slot)
        del self._live[slot]
        self._free_slots.append(slot)

    def is_live(self, slot: int) -> bool:
        return slot in self._live

    def length(self, slot: int) -> int:
        try:
            return self._live[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not in use") from None

    def live_slots(self) -> list[int]:
        return sorted(self._live)

    # -- room -------------------------------------------------------------
    def can_hold(self, lengths: Sequence[int]) -> bool:
        """Whether sequences of these final lengths fit beside what is held now."""
        if len(lengths) > len(self._free_slots):
            return False
        for g in self.kv_groups.values():
            if sum(g.pages_for(n) for n in lengths) > g.pool.n_free:
                return False
            if any(g.pages_for(n) > g.pages_per_seq for n in lengths):
                return False
        return all(n <= self.max_ctx for n in lengths)

    def reserve(self, slot: int, new_length: int) -> None:
        """Room for positions < new_length in every KV group (the length itself moves in `advance`)."""
        if slot not in self._live:
            raise CacheError(f"slot {slot} is not in use")
        if new_length > self.max_ctx:
            raise CacheFull(f"sequence would reach {new_length} tokens, the context holds {self.max_ctx}")
        for g in self.kv_groups.values():
            g.ensure(slot, new_length)

    def advance(self, slot: int, new_length: int) -> None:
        if new_length < self._live[slot]:
            raise CacheError("a sequence cannot shrink")
        self._live[slot] = new_length

    def sync(self) -> None:
        for g in self.kv_groups.values():
            g.sync()

    # -- views ------------------------------------------------------------
    def line(self, index: int, write: bool = True, has_readers: bool = False) -> CacheLine:
        parts = {}
        for name, (g, j) in self._line_parts[index].items():
            if isinstance(g, KVGroup):
                parts[name] = KVLine(g, g.k[j], g.v[j], write)
            else:
                parts[name] = StateLine(g, g.data[j], write)
        return CacheLine(index, write, parts, has_readers)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.kv_groups.values()) + \
            sum(g.data.numel() * g.data.element_size() for g in self.state_groups.values())

    def audit(self) -> None:
        """Raise unless every slot and page is either free or held exactly once."""
        if sorted(self._free_slots + list(self._live)) != list(range(self.n_slots)):
            raise CacheError("slots lost or held twice")
        for g in self.kv_groups.values():
            for slot in g.held:
                if slot not in self._live:
                    raise CacheError(f"pages held for slot {slot}, which is free")
            g.pool.audit([p for pages in g.held.values() for p in pages])
