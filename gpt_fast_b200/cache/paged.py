"""The cache of a model: a slot per live sequence, paged keys and values per
cache entry, and fixed-size per-sequence state.

gpt-fast keeps, per layer, two dense buffers [max_batch, n_kv, max_seq, d] that
every row of the batch writes at the same positions (model.py:84-100).  Here
each sequence has a slot with its own length; keys and values live in pages of
`page_size` tokens that a slot collects as it grows, so memory is sized by
the number of tokens that are live at once, not by slots times the longest
sequence.  Cache entries whose mixers ask for the same thing (same heads, head
size and window) form a group with storage, page table and page allocator of
its own.  A mixer that asks for fixed-size state gets a [n_slots, *shape] tensor
per entry, zeroed when a slot is handed out.  Slots and pages go back to their
free lists when a sequence ends and are used again without clearing: nothing
reads beyond a slot's length.
"""
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from ..ops.types import PagedKV
from .needs import CacheNeeds, KVNeed, StateNeed
from .slots import CacheFull, FreeList

DEFAULT_PAGE_SIZE = 64


@dataclass
class EntryView:
    """What one run of a layer sees of the cache."""
    kv: Optional[PagedKV] = None
    state: Optional[torch.Tensor] = None        # [n_slots, *shape]


class _KVGroup:
    def __init__(self, need: KVNeed, entries: List[int], n_pages, n_slots, max_pages, page_size, dtype, device):
        self.need, self.entries = need, entries
        self.index = {e: i for i, e in enumerate(entries)}
        shape = (len(entries), n_pages, need.n_kv, page_size, need.head_dim)
        self.k_pool = torch.zeros(shape, dtype=dtype, device=device)
        self.v_pool = torch.zeros(shape, dtype=dtype, device=device)
        self.pages = FreeList(n_pages, "page")
        self.table_host = torch.full((n_slots, max_pages), -1, dtype=torch.int32)
        self.table = self.table_host.to(device)
        self.slot_pages: Dict[int, List[int]] = {}
        self.dirty = set()


class _StateGroup:
    def __init__(self, need: StateNeed, entries: List[int], n_slots, device):
        self.need, self.entries = need, entries
        self.index = {e: i for i, e in enumerate(entries)}
        self.data = torch.zeros((len(entries), n_slots) + tuple(need.shape), dtype=need.dtype, device=device)


class Cache:
    def __init__(self, needs: Dict[int, CacheNeeds], dtype: torch.dtype, device, *, max_tokens: int,
                 max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None,
                 page_size: int = DEFAULT_PAGE_SIZE):
        """needs: cache entry id -> what its mixer asks for.
        max_tokens: the most tokens live sequences hold at once, each sequence
          rounded up to whole pages.
        max_seqs: the most live sequences (default: one per page).
        max_seq_len: the longest one sequence may get (default: all pages)."""
        if page_size <= 0 or max_tokens <= 0:
            raise ValueError("page_size and max_tokens must be positive")
        self.page_size = page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_seq_len = min(max_seq_len or self.n_pages * page_size, self.n_pages * page_size)
        self.max_pages = -(-self.max_seq_len // page_size)
        self.n_slots = min(max_seqs or self.n_pages, self.n_pages)
        self.dtype, self.device = dtype, torch.device(device)
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths_host = [0] * self.n_slots
        self.reserved_host = [0] * self.n_slots
        self.lengths = torch.zeros(self.n_slots, dtype=torch.int32, device=device)

        by_kv: Dict[KVNeed, List[int]] = {}
        by_state: Dict[StateNeed, List[int]] = {}
        for entry in sorted(needs):
            n = needs[entry]
            if n is None:
                continue
            if n.kv is not None:
                by_kv.setdefault(n.kv, []).append(entry)
            if n.state is not None:
                by_state.setdefault(n.state, []).append(entry)
        self.kv_groups = [_KVGroup(need, entries, self.n_pages, self.n_slots, self.max_pages, page_size, dtype, device)
                          for need, entries in by_kv.items()]
        self.state_groups = [_StateGroup(need, entries, self.n_slots, device) for need, entries in by_state.items()]
        self._views: Dict[int, EntryView] = {}
        for entry in needs:
            v = EntryView()
            for g in self.kv_groups:
                if entry in g.index:
                    i = g.index[entry]
                    v.kv = PagedKV(g.k_pool[i], g.v_pool[i], g.table, page_size)
            for g in self.state_groups:
                if entry in g.index:
                    v.state = g.data[g.index[entry]]
            self._views[entry] = v

    # ---- what a step reads ------------------------------------------------------
    def view(self, entry: int) -> EntryView:
        return self._views[entry]

    # ---- life of a sequence -----------------------------------------------------------
    def begin(self, n: int) -> List[int]:
        """Hand out n slots with length 0 and zeroed state."""
        slots = self.slots.alloc(n)
        for s in slots:
            self.lengths_host[s] = 0
            self.reserved_host[s] = 0
        if slots:
            idx = torch.tensor(slots, dtype=torch.long).to(self.device)
            self.lengths.index_fill_(0, idx, 0)
            for g in self.state_groups:
                g.data.index_fill_(1, idx, 0)
        return slots

    def reserve(self, slot: int, n_tokens: int) -> None:
        """Make sure `slot` has pages for positions 0 .. n_tokens-1 in every group."""
        if slot not in self.slots.in_use:
            raise ValueError(f"slot {slot} is not in use")
        if n_tokens > self.max_seq_len:
            raise CacheFull(f"a sequence of {n_tokens} tokens exceeds the cache's longest sequence {self.max_seq_len}")
        need_pages = -(-n_tokens // self.page_size)
        for g in self.kv_groups:
            have = g.slot_pages.setdefault(slot, [])
            if need_pages > len(have):
                new = g.pages.alloc(need_pages - len(have))
                g.table_host[slot, len(have):len(have) + len(new)] = torch.tensor(new, dtype=torch.int32)
                have.extend(new)
                g.dirty.add(slot)
        self.reserved_host[slot] = max(self.reserved_host[slot], need_pages * self.page_size)

    def can_reserve(self, totals: Sequence[int]) -> bool:
        """Whether fresh sequences of these final lengths fit right now."""
        pages = sum(-(-t // self.page_size) for t in totals)
        return (len(totals) <= self.slots.n_free and max(totals, default=0) <= self.max_seq_len
                and all(pages <= g.pages.n_free for g in self.kv_groups))

    def sync_tables(self) -> None:
        """Copy page-table rows that changed on the host to the device."""
        for g in self.kv_groups:
            if not g.dirty:
                continue
            rows = sorted(g.dirty)
            idx = torch.tensor(rows, dtype=torch.long)
            g.table.index_copy_(0, idx.to(self.device), g.table_host[idx].to(self.device))
            g.dirty.clear()

    def note_advance(self, slots: Iterable[int], q_lens: Iterable[int]) -> None:
        """Host mirror of the device-side `advance_lengths`."""
        for s, q in zip(slots, q_lens):
            self.lengths_host[s] += q

    def end(self, slots: Iterable[int]) -> None:
        """Give slots and their pages back."""
        slots = list(slots)
        self.slots.free(slots)
        for g in self.kv_groups:
            for s in slots:
                pages = g.slot_pages.pop(s, [])
                if pages:
                    g.pages.free(pages)
                    g.table_host[s, :len(pages)] = -1
                    g.dirty.add(s)

    # ---- accounting ---------------------------------------------------------------------
    @property
    def pages_free(self) -> int:
        return min((g.pages.n_free for g in self.kv_groups), default=self.n_pages)

    def bytes(self) -> int:
        n = sum(g.k_pool.numel() * g.k_pool.element_size() * 2 for g in self.kv_groups)
        return n + sum(g.data.numel() * g.data.element_size() for g in self.state_groups)

    def kv_bytes_per_token(self) -> int:
        return sum(2 * len(g.entries) * g.need.n_kv * g.need.head_dim * g.k_pool.element_size() for g in self.kv_groups)
