"""The cache manager: paged keys and values, block tables, and state slots.

What the reference does with one free set of block ids shared by all layers,
one row of a ``[max_batch, nblocks]`` device table per lane and per-lane device
rows for everything else (fastgen/generate.py:258-294, 477-518, 898-932;
fastgen/cache.py:37-140) is generalised here:

* runs of layers whose mixers need the same thing per token (head count, head
  size, window) form a *group*; each group has a page pool of its own, storage
  of its own and a block table of its own per request;
* a group with a window gives pages back as soon as the window has passed them;
* every live request holds one *slot*: the row of its block tables on the
  device and the index of its fixed-size state (zeroed on admission), for
  mixers that keep state of fixed size instead of per-token entries.

All bookkeeping is host-side and runs without a GPU; device tensors are created
only when a device is given.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheSpec, StateSpec


class OutOfPages(RuntimeError):
    """Not enough free pages (or slots) for what was asked; nothing was taken."""


class CacheError(RuntimeError):
    """A bookkeeping invariant was violated (double free, unknown request...)."""


class PagePool:
    """Free list of page ids ``0 .. n_pages-1`` with ownership checks.

    Pages are handed out lowest id first, like the reference's ordered set
    (fastgen/utils/iset.py:312-319); results never depend on which ids are used.
    """

    def __init__(self, n_pages: int) -> None:
        if n_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))  # pop() gives the lowest id
        self._held = np.zeros(n_pages, dtype=bool)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages asked, {len(self._free)} free of {self.n_pages}")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            if self._held[p]:
                raise CacheError(f"page {p} was handed out twice")
            self._held[p] = True
        return pages

    def give(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise CacheError(f"page {p} is given back but is not held")
            self._held[p] = False
        self._free.extend(sorted(pages, reverse=True))
        # keep "lowest id first" cheap: the list is a stack, order it lazily
        self._free.sort(reverse=True)

    def held(self) -> int:
        return int(self._held.sum())


@dataclass
class CacheGroup:
    """One group of runs with the same per-token need."""

    spec: CacheSpec
    entries: List[int]  # schedule entries that own storage in this group
    page_size: int
    pool: PagePool
    table_width: int
    host_table: np.ndarray  # [n_slots, table_width] int32, -1 = no page
    k_pages: Optional[torch.Tensor] = None  # [len(entries), n_pages, Hkv, page, hd]
    v_pages: Optional[torch.Tensor] = None  # the second pool; None when the spec asks for one
    device_table: Optional[torch.Tensor] = None  # [n_slots, table_width] int32
    tensor_maps: Optional[tuple] = None  # made by the kernels' side for pools it can tile
    dirty: List[Tuple[int, int, int]] = field(default_factory=list)  # (slot, col, page)

    def first_needed_page(self, length: int) -> int:
        """Lowest logical page that a query at position >= ``length`` may read."""
        if self.spec.window is None:
            return 0
        return max(0, length - self.spec.window + 1) // self.page_size

    def bytes_per_token(self, elt_size: int) -> int:
        return self.spec.n_pools * len(self.entries) * self.spec.n_kv_heads * self.spec.head_dim * elt_size


@dataclass
class LayerMemory:
    """What one run of a layer is handed: its pages (or another run's) and the
    state tensor of its mixer, both indexed by the request's slot."""

    k_pages: Optional[torch.Tensor] = None  # [n_pages, Hkv, page, hd]
    v_pages: Optional[torch.Tensor] = None  # None for a one-pool group
    block_table: Optional[torch.Tensor] = None  # [n_slots, width] int32
    page_size: int = 0
    writes: bool = True  # False: the run reads the cache another run writes
    state: Optional[torch.Tensor] = None  # [n_slots, *state_shape] float32
    tensor_maps: Optional[tuple] = None  # TMA descriptors of the group's (key, value) pools
    layer_index: int = 0  # this run's index within the group's pools


class RequestCache:
    """A live request's holdings: its slot, its length and its pages per group."""

    def __init__(self, request_id, slot: int, n_groups: int) -> None:
        self.request_id = request_id
        self.slot = slot
        self.length = 0  # tokens whose keys/values (or state) are in the cache
        self.pages: List[Dict[int, int]] = [dict() for _ in range(n_groups)]  # logical -> page
        # Positions below this have a page in every group.  A request's pages in a group are
        # a contiguous run of logical pages (taken upward, given back from below), so the
        # bound answers most reservations of a decoding request without a look at the maps.
        self.reserved = 0

    def n_pages(self) -> int:
        return sum(len(p) for p in self.pages)


class CacheManager:
    """Pages, block tables and state slots for up to ``max_requests`` requests.

    ``cache_specs[e]`` / ``state_specs[e]`` give, for schedule entry ``e``, what
    its mixer needs (``None`` if nothing, or if the entry reads another entry's
    cache -- then ``kv_from[e]`` names it).  ``page_size`` is the page of every group
    whose spec does not ask for its own.  ``n_pages`` is the pool size of each group: a
    list with one number per group, or one number, which then counts pages of
    ``page_size`` tokens and is converted for a group with other pages so that every
    group holds the same number of tokens.
    """

    def __init__(
        self,
        cache_specs: Sequence[Optional[CacheSpec]],
        state_specs: Sequence[Optional[StateSpec]],
        kv_from: Sequence[Optional[int]],
        page_size: int,
        n_pages,
        max_requests: int,
        max_length: int,
        dtype: torch.dtype = torch.float32,
        device=None,
        tensor_map_factory=None,
    ) -> None:
        if page_size <= 0:
            raise ValueError(f"page size must be positive, got {page_size}")
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_length = max_length
        self.dtype = dtype
        self.device = device
        self.kv_from = list(kv_from)
        n_entries = len(cache_specs)

        # group the entries that own storage by their per-token need
        self.groups: List[CacheGroup] = []
        self.entry_group: List[Optional[int]] = [None] * n_entries
        self.entry_index: List[Optional[int]] = [None] * n_entries  # index within the group
        by_spec: Dict[CacheSpec, int] = {}
        for e, spec in enumerate(cache_specs):
            if spec is None or self.kv_from[e] is not None:
                continue
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                group_page = spec.page_size or page_size
                if isinstance(n_pages, int):
                    pages = max(1, n_pages * page_size // group_page)
                else:
                    pages = n_pages[len(self.groups)]
                width = -(-max_length // group_page)
                self.groups.append(
                    CacheGroup(
                        spec=spec,
                        entries=[],
                        page_size=group_page,
                        pool=PagePool(pages),
                        table_width=width,
                        host_table=np.full((max_requests, width), -1, dtype=np.int32),
                    )
                )
            g = by_spec[spec]
            self.entry_group[e] = g
            self.entry_index[e] = len(self.groups[g].entries)
            self.groups[g].entries.append(e)
        for e, src in enumerate(self.kv_from):
            if src is not None:
                if cache_specs[e] != cache_specs[src]:
                    raise ValueError(
                        f"schedule entry {e} reads the cache of entry {src}, whose "
                        f"layout {cache_specs[src]} differs from its own {cache_specs[e]}"
                    )
                self.entry_group[e] = self.entry_group[src]
                self.entry_index[e] = self.entry_index[src]

        self.state_specs = list(state_specs)
        self.states: List[Optional[torch.Tensor]] = [None] * n_entries
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[object, RequestCache] = {}

        if device is not None:
            for grp in self.groups:
                shape = (
                    len(grp.entries),
                    grp.pool.n_pages,
                    grp.spec.n_kv_heads,
                    grp.page_size,
                    grp.spec.head_dim,
                )
                grp.k_pages = torch.zeros(shape, dtype=dtype, device=device)
                if grp.spec.n_pools == 2:
                    grp.v_pages = torch.zeros(shape, dtype=dtype, device=device)
                grp.device_table = torch.full(
                    (max_requests, grp.table_width), -1, dtype=torch.int32, device=device
                )
                if tensor_map_factory is not None and grp.v_pages is not None:
                    grp.tensor_maps = tensor_map_factory(grp.k_pages, grp.v_pages, grp.page_size)
            for e, st in enumerate(self.state_specs):
                if st is not None:
                    self.states[e] = torch.zeros(
                        (max_requests, *st.shape), dtype=torch.float32, device=device
                    )

    # -- queries -------------------------------------------------------------------
    @property
    def n_live(self) -> int:
        return len(self._requests)

    def free_pages(self) -> List[int]:
        return [g.pool.n_free for g in self.groups]

    def free_slots(self) -> int:
        return len(self._free_slots)

    def get(self, request_id) -> RequestCache:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def pages_needed(self, req: RequestCache, new_length: int) -> List[int]:
        """New pages per group that ``req`` needs to hold ``new_length`` tokens."""
        if new_length <= req.reserved:
            return [0] * len(self.groups)
        out = []
        for gi, grp in enumerate(self.groups):
            have = req.pages[gi]
            first = grp.first_needed_page(req.length)
            last = (new_length - 1) // grp.page_size if new_length > 0 else -1
            out.append(sum(1 for lp in range(first, last + 1) if lp not in have))
        return out

    def pages_for(self, length: int) -> List[int]:
        """Pages per group that a fresh request of ``length`` tokens needs at most
        at one time if it is fed in one portion."""
        return [-(-length // g.page_size) for g in self.groups]

    def can_ever_hold(self, length: int) -> bool:
        """Whether a request of ``length`` tokens fits an empty cache at all."""
        if length > self.max_length:
            return False
        return all(n <= g.pool.n_pages for n, g in zip(self.pages_for(length), self.groups))

    # -- life cycle ----------------------------------------------------------------
    def admit(self, request_id) -> RequestCache:
        """Give a new request its slot.  No pages are taken yet."""
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        req = RequestCache(request_id, slot, len(self.groups))
        self._requests[request_id] = req
        for st in self.states:
            if st is not None:
                st[slot].zero_()
        return req

    def reserve(self, req: RequestCache, new_length: int) -> None:
        """Make sure ``req`` has pages for positions ``< new_length`` in every
        group.  Either every group succeeds or nothing changes."""
        if new_length > self.max_length:
            raise OutOfPages(
                f"request {req.request_id!r} would hold {new_length} tokens; the cache "
                f"was built for at most {self.max_length} per request"
            )
        if new_length <= req.reserved:
            return
        need = self.pages_needed(req, new_length)
        for n, grp in zip(need, self.groups):
            if n > grp.pool.n_free:
                raise OutOfPages(
                    f"request {req.request_id!r} needs {need} new pages per group, "
                    f"free: {self.free_pages()}"
                )
        for gi, grp in enumerate(self.groups):
            first = grp.first_needed_page(req.length)
            last = (new_length - 1) // grp.page_size if new_length > 0 else -1
            missing = [lp for lp in range(first, last + 1) if lp not in req.pages[gi]]
            for lp, page in zip(missing, grp.pool.take(len(missing))):
                req.pages[gi][lp] = page
                grp.host_table[req.slot, lp] = page
                grp.dirty.append((req.slot, lp, page))
        if self.groups:
            req.reserved = min((max(req.pages[gi]) + 1) * grp.page_size if req.pages[gi] else 0
                               for gi, grp in enumerate(self.groups))

    def advance(self, req: RequestCache, new_length: int) -> None:
        """Record that ``req`` now holds ``new_length`` tokens and give back the
        pages a window has passed."""
        if new_length < req.length:
            raise CacheError("a request's length cannot shrink")
        req.length = new_length
        for gi, grp in enumerate(self.groups):
            first = grp.first_needed_page(new_length)
            gone = [lp for lp in req.pages[gi] if lp < first]
            if gone:
                grp.pool.give([req.pages[gi].pop(lp) for lp in gone])
                for lp in gone:
                    grp.host_table[req.slot, lp] = -1
                    grp.dirty.append((req.slot, lp, -1))

    def release(self, request_id) -> None:
        """The request ended (or is preempted): give everything back."""
        req = self._requests.pop(request_id, None)
        if req is None:
            raise CacheError(f"request {request_id!r} is released but is not live")
        for gi, grp in enumerate(self.groups):
            if req.pages[gi]:
                grp.pool.give(list(req.pages[gi].values()))
                for lp in req.pages[gi]:
                    grp.host_table[req.slot, lp] = -1
                    grp.dirty.append((req.slot, lp, -1))
                req.pages[gi] = {}
        self._free_slots.append(req.slot)
        self._free_slots.sort(reverse=True)

    # -- device side ---------------------------------------------------------------
    def flush_tables(self) -> None:
        """Bring the device block tables up to date with the host's."""
        if self.device is None:
            for grp in self.groups:
                grp.dirty.clear()
            return
        for grp in self.groups:
            if not grp.dirty:
                continue
            flat = np.array([s * grp.table_width + c for s, c, _ in grp.dirty], dtype=np.int64)
            vals = np.array([p for _, _, p in grp.dirty], dtype=np.int32)
            # later writes to the same entry must win: keep the last of each index
            _, last = np.unique(flat[::-1], return_index=True)
            keep = len(flat) - 1 - last
            idx = torch.from_numpy(flat[keep]).to(self.device, non_blocking=False)
            val = torch.from_numpy(vals[keep]).to(self.device, non_blocking=False)
            grp.device_table.view(-1).index_copy_(0, idx, val)
            grp.dirty.clear()

    def memory(self, entry: int) -> LayerMemory:
        """The :class:`LayerMemory` of schedule entry ``entry``."""
        g = self.entry_group[entry]
        mem = LayerMemory(state=self.states[entry])
        if g is not None:
            grp = self.groups[g]
            i = self.entry_index[entry]
            mem.page_size = grp.page_size
            mem.writes = self.kv_from[entry] is None
            if grp.k_pages is not None:
                mem.k_pages = grp.k_pages[i]
                mem.v_pages = grp.v_pages[i] if grp.v_pages is not None else None
                mem.block_table = grp.device_table
                mem.tensor_maps = grp.tensor_maps
                mem.layer_index = i
        return mem

    # -- invariants (used by tests) --------------------------------------------------
    def check(self) -> None:
        """No page lost, none held twice; tables agree with the holdings."""
        for gi, grp in enumerate(self.groups):
            seen: Dict[int, object] = {}
            for req in self._requests.values():
                for lp, page in req.pages[gi].items():
                    if page in seen:
                        raise CacheError(
                            f"page {page} of group {gi} is held by {seen[page]!r} and {req.request_id!r}"
                        )
                    seen[page] = req.request_id
                    if grp.host_table[req.slot, lp] != page:
                        raise CacheError("block table disagrees with a request's pages")
                held = req.pages[gi]
                if held and sorted(held) != list(range(min(held), max(held) + 1)):
                    raise CacheError(f"request {req.request_id!r} holds a broken run of pages in group {gi}")
                if req.reserved > ((max(held) + 1) * grp.page_size if held else 0):
                    raise CacheError(f"request {req.request_id!r}: reserved bound beyond its pages in group {gi}")
            if len(seen) + grp.pool.n_free != grp.pool.n_pages:
                raise CacheError(
                    f"group {gi}: {len(seen)} held + {grp.pool.n_free} free != {grp.pool.n_pages}"
                )
            if grp.pool.held() != len(seen):
                raise CacheError(f"group {gi}: pool and requests disagree on held pages")
            live_rows = {r.slot for r in self._requests.values()}
            for slot in range(self.max_requests):
                if slot not in live_rows and (grp.host_table[slot] != -1).any():
                    raise CacheError(f"group {gi}: slot {slot} is free but its table is not empty")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a slot is held twice or is both held and free")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a slot was lost")
