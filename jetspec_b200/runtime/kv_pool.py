"""Slot-addressed paged KV pool.

One pool serves every layer and every sequence::

    k_pool, v_pool : (L, Hkv, S, D)       S = num_pages * page_size slots
    slot_map       : (max_seqs, max_len)  int32, on the device

A *page* (``page_size`` consecutive slots) is the unit of allocation and is shared
by all layers (one page id addresses the same slots in each layer's slice), so a
sequence of ``n`` tokens owns ``ceil(n / page_size)`` ids, not ``L`` times that.
A *slot map row* translates a sequence's logical position to a slot.  Attention
reads K/V through the slot map, so committing an accepted tree path never moves
KV bytes: it only permutes the ``N`` slot-map entries of the tree window so that
the accepted nodes' slots come first (positions ``past .. past+k``) and the
rejected nodes' slots are recycled for the next round's tree.  Memory in use is
therefore exactly ``committed tokens + tree window``, with nothing leaked between
rounds.

Compared with the reference cache (``jetspec/inference_engine/paged_kv_cache.py``):
same responsibilities (admission, allocation, eviction with LRU, refcounts, status,
``EvictionRequired`` / ``EvictionFailed``), but layer-shared page ids from the start
(the reference allocates distinct ids per layer, ``:189-203``), O(1) free-list
operations, and no per-step host-side block-table rebuild (``:867-883``).
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

import torch


class EvictionRequired(RuntimeError):
    """The pool cannot serve the request without evicting another sequence."""


class EvictionFailed(RuntimeError):
    """No sequence can be evicted (nothing else is resident)."""


@dataclass
class SeqState:
    seq_id: int
    row: int
    pages: list = field(default_factory=list)
    length: int = 0          # committed KV length (logical positions with valid KV)
    capacity: int = 0        # slots granted (positions that have a slot id in the map)
    last_used: int = 0


class PagedKVPool:
    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, num_pages: int,
                 page_size: int = 16, max_seqs: int = 64, max_seq_len: int = 4096,
                 device="cpu", dtype=torch.float32):
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.page_size, self.num_pages = int(page_size), int(num_pages)
        self.max_seqs, self.max_seq_len = int(max_seqs), int(max_seq_len)
        self.device, self.dtype = torch.device(device), dtype
        S = self.num_pages * self.page_size
        self.k_pool = torch.zeros(num_layers, num_kv_heads, S, head_dim, dtype=dtype, device=device)
        self.v_pool = torch.zeros(num_layers, num_kv_heads, S, head_dim, dtype=dtype, device=device)
        self.slot_map = torch.zeros(self.max_seqs, self.max_seq_len, dtype=torch.int32, device=device)
        self._free_pages: deque = deque(range(self.num_pages))
        self._refcount = [0] * self.num_pages
        self._free_rows: deque = deque(range(self.max_seqs))
        self._seqs: dict = {}
        self._clock = itertools.count(1)
        self.frozen = False   # set while CUDA graphs hold pointers into the pool

    # -- sizing ---------------------------------------------------------------
    @classmethod
    def for_model(cls, cfg, num_pages: int, **kw) -> "PagedKVPool":
        return cls(cfg.num_hidden_layers, cfg.num_key_value_heads, cfg.head_dim, num_pages, **kw)

    @property
    def num_slots(self) -> int:
        return self.num_pages * self.page_size

    def pages_for(self, tokens: int) -> int:
        return (int(tokens) + self.page_size - 1) // self.page_size

    @property
    def free_page_count(self) -> int:
        return len(self._free_pages)

    def utilization(self) -> float:
        return 1.0 - len(self._free_pages) / max(1, self.num_pages)

    def layer(self, li: int):
        return self.k_pool[li], self.v_pool[li]

    # -- sequences ------------------------------------------------------------
    def has(self, seq_id: int) -> bool:
        return seq_id in self._seqs

    def state(self, seq_id: int) -> SeqState:
        return self._seqs[seq_id]

    def touch(self, seq_id: int) -> None:
        self._seqs[seq_id].last_used = next(self._clock)

    def reclaimable_pages(self, exclude: Optional[int] = None) -> int:
        return sum(len(s.pages) for sid, s in self._seqs.items() if sid != exclude)

    def admit_sequence(self, seq_id: int, num_tokens: int) -> bool:
        """True when ``num_tokens`` positions could be granted, counting pages that
        evicting *other* sequences would free."""
        if num_tokens > self.max_seq_len:
            return False
        have = len(self._seqs[seq_id].pages) if seq_id in self._seqs else 0
        need = self.pages_for(num_tokens) - have
        if seq_id not in self._seqs and not self._free_rows and not self._seqs:
            return False
        return need <= len(self._free_pages) + self.reclaimable_pages(exclude=seq_id)

    def allocate_slots(self, seq_id: int, num_tokens: int, allow_evict: bool = True) -> bool:
        """Grant slots so that positions ``[0, num_tokens)`` are mapped; evicts least-recently
        used *other* sequences if the free list is short.  False when it cannot fit."""
        if num_tokens > self.max_seq_len:
            return False
        st = self._seqs.get(seq_id)
        if st is None:
            if not self._free_rows:
                if not allow_evict:
                    return False
                try:
                    self.evict_sequence(exclude=seq_id)
                except EvictionFailed:
                    return False
            st = SeqState(seq_id, self._free_rows.popleft(), last_used=next(self._clock))
            self._seqs[seq_id] = st
        need = self.pages_for(num_tokens) - len(st.pages)
        while need > len(self._free_pages):
            if not allow_evict:
                return False
            try:
                self.evict_sequence(exclude=seq_id)
            except EvictionFailed:
                return False
        if need > 0:
            new_pages = [self._free_pages.popleft() for _ in range(need)]
            for p in new_pages:
                assert self._refcount[p] == 0, f"page {p} handed out twice"
                self._refcount[p] = 1
            base = len(st.pages) * self.page_size
            st.pages.extend(new_pages)
            ids = (torch.tensor(new_pages, dtype=torch.int32).repeat_interleave(self.page_size) * self.page_size
                   + torch.arange(self.page_size, dtype=torch.int32).repeat(len(new_pages)))
            end = min(base + ids.numel(), self.max_seq_len)
            self.slot_map[st.row, base:end] = ids[: end - base].to(self.device, non_blocking=True)
        st.capacity = min(len(st.pages) * self.page_size, self.max_seq_len)
        st.last_used = next(self._clock)
        return True

    def reserve(self, seq_id: int, num_tokens: int) -> None:
        """Like :meth:`allocate_slots` but never evicts and raises when it does not fit."""
        if not self.allocate_slots(seq_id, num_tokens, allow_evict=False):
            raise EvictionRequired(f"sequence {seq_id} needs {self.pages_for(num_tokens)} pages; "
                                   f"{len(self._free_pages)} free")

    def free(self, seq_id: int) -> None:
        st = self._seqs.pop(seq_id, None)
        if st is None:
            return
        for p in st.pages:
            self._refcount[p] -= 1
            assert self._refcount[p] >= 0, f"page {p} refcount went negative"
            if self._refcount[p] == 0:
                self._free_pages.append(p)
        self._free_rows.append(st.row)

    def evict_sequence(self, seq_id: Optional[int] = None, exclude: Optional[int] = None) -> int:
        """Drop a resident sequence (named, or the least recently used one) and return its id."""
        if seq_id is None:
            cands = [s for sid, s in self._seqs.items() if sid != exclude]
            if not cands:
                raise EvictionFailed("no evictable sequence resident")
            seq_id = min(cands, key=lambda s: s.last_used).seq_id
        elif seq_id not in self._seqs:
            raise EvictionFailed(f"sequence {seq_id} is not resident")
        self.free(seq_id)
        return seq_id

    def crop(self, seq_id: int, length: int) -> None:
        st = self._seqs[seq_id]
        st.length = min(st.length, int(length))

    def reset(self) -> None:
        for sid in list(self._seqs):
            self.free(sid)

    def resident(self) -> list:
        return list(self._seqs)

    def get_seq_status(self, seq_id: int) -> dict:
        st = self._seqs[seq_id]
        return {"seq_id": seq_id, "row": st.row, "length": st.length, "capacity": st.capacity,
                "pages": len(st.pages), "last_used": st.last_used}

    # -- tree window ------------------------------------------------------------
    def commit_path(self, seq_id: int, past: int, num_nodes: int, path) -> None:
        """Make the accepted nodes' slots the next committed positions.

        ``path`` lists accepted node indices (root first).  The window
        ``slot_map[row, past:past+num_nodes]`` is permuted to ``path`` followed by the
        remaining nodes in index order, and the committed length becomes
        ``past + len(path)``.  No KV bytes move.
        """
        st = self._seqs[seq_id]
        if isinstance(path, (list, tuple)):      # host path: the permutation is built without a device read
            taken = set(path)
            order = torch.tensor(list(path) + [i for i in range(num_nodes) if i not in taken], dtype=torch.long,
                                 device=self.device)
            n_path = len(path)
        else:
            p = torch.as_tensor(path, dtype=torch.long, device=self.device)
            keep = torch.ones(num_nodes, dtype=torch.bool, device=self.device)
            keep[p] = False
            order = torch.cat((p, torch.nonzero(keep, as_tuple=True)[0]))
            n_path = int(p.numel())
        win = self.slot_map[st.row, past:past + num_nodes]
        self.slot_map[st.row, past:past + num_nodes] = win[order]
        st.length = past + n_path
        st.last_used = next(self._clock)
