"""The cache manager: device pools for every group of layers with the same
need, and (through the native runtime) the pages and the state slot each live
request holds.

Paged groups: keys and values of all order items with the same
(kv heads, head size, window), pool [items, pages, kv heads, page size, head
size] each for K and V; one page id of a group means that page in every item
of the group. The reference sizes one pool for all layers, convolution layers
included (tools/infer/src/main.rs:386-392); here only items that keep keys
have pages. State groups: [items, slots, *shape] for order items with
fixed-size state; a request's slot is zeroed when it is admitted.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np
import torch

from ..parts.base import CacheBinding, FixedState, PagedKV
from .native import CacheError, checked, int_array, last_error, lib


class OutOfPages(CacheError):
    pass


class CacheManager:
    def __init__(self, needs: Sequence, cache_of: Sequence[Optional[int]], page_size: int, total_blocks,
                 num_slots: int, dtype: torch.dtype, device):
        """needs[i]: PagedKV | FixedState | None for order item i (None: no cache of
        its own); cache_of[i]: the item whose cache item i reads, or None.
        total_blocks: pages of every paged group (an int) or one count per group."""
        self.page_size, self.num_slots, self.dtype, self.device = int(page_size), int(num_slots), dtype, torch.device(device)
        self.paged_keys: list[PagedKV] = []
        self.state_keys: list[FixedState] = []
        self._item_group: list[Optional[tuple[str, int, int]]] = []   # (family, group, index in group)
        members: dict[tuple[str, int], int] = {}
        for need in needs:
            if need is None:
                self._item_group.append(None)
                continue
            if isinstance(need, PagedKV):
                fam, keys = "paged", self.paged_keys
            elif isinstance(need, FixedState):
                fam, keys = "state", self.state_keys
            else:
                raise CacheError(f"unknown cache need {need!r}")
            if need not in keys:
                keys.append(need)
            g = keys.index(need)
            idx = members.get((fam, g), 0)
            members[(fam, g)] = idx + 1
            self._item_group.append((fam, g, idx))
        for i, src in enumerate(cache_of):
            if src is not None:
                self._item_group[i] = self._item_group[src]
        self._borrowed = [c is not None for c in cache_of]
        n_paged = len(self.paged_keys)
        if isinstance(total_blocks, int):
            total_blocks = [total_blocks] * n_paged
        if len(total_blocks) != n_paged:
            raise CacheError(f"{len(total_blocks)} page counts for {n_paged} paged groups")
        self.group_pages = [int(p) for p in total_blocks]
        self.k_pools, self.v_pools, self.states = [], [], []
        for g, need in enumerate(self.paged_keys):
            shape = (members[("paged", g)], self.group_pages[g], need.num_kv_heads, self.page_size, need.head_dim)
            self.k_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
            self.v_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
        for g, need in enumerate(self.state_keys):
            self.states.append(torch.zeros((members[("state", g)], self.num_slots) + tuple(need.shape),
                                           dtype=need.dtype, device=self.device))
        # A model without paged items (no attention at all) has no page group: its requests hold a slot only.
        windows = [k.window for k in self.paged_keys]
        self._h = lib().cellm_cache_create(self.page_size, n_paged, int_array(self.group_pages), int_array(windows),
                                           self.num_slots)
        if not self._h:
            raise CacheError(last_error())

    def __del__(self):
        if getattr(self, "_h", None):
            lib().cellm_cache_destroy(self._h)
            self._h = None

    # ------------------------------------------------------------ requests
    @property
    def handle(self):
        return self._h

    def add(self, request_id: int) -> int:
        """Takes a state slot for a new request and zeroes its state; returns the slot."""
        slot = lib().cellm_cache_add(self._h, int(request_id))
        if slot == -2:
            raise OutOfPages("no free state slot")
        checked(slot)
        self.zero_slot(slot)
        return slot

    def zero_slot(self, slot: int) -> None:
        for s in self.states:
            s[:, slot].zero_()

    def has(self, request_id: int) -> bool:
        return bool(lib().cellm_cache_has(self._h, int(request_id)))

    def reserve(self, request_id: int, new_total: int) -> bool:
        return bool(checked(lib().cellm_cache_reserve(self._h, int(request_id), int(new_total))))

    def commit(self, request_id: int, new_total: int) -> None:
        checked(lib().cellm_cache_commit(self._h, int(request_id), int(new_total)))

    def release(self, request_id: int) -> None:
        checked(lib().cellm_cache_release(self._h, int(request_id)))

    def tokens(self, request_id: int) -> int:
        return checked(lib().cellm_cache_tokens(self._h, int(request_id)))

    def slot(self, request_id: int) -> int:
        return checked(lib().cellm_cache_slot(self._h, int(request_id)))

    def block_table(self, request_id: int, group: int, out: Optional[np.ndarray] = None) -> np.ndarray:
        """The request's pages of a paged group, in order; -1 where a page was given back."""
        if out is None:
            out = np.full((self.max_blocks(group),), -1, dtype=np.int32)
        n = checked(lib().cellm_cache_block_table(self._h, int(request_id), int(group),
                                                  out.ctypes.data_as(ctypes.c_void_p), out.shape[0]))
        return out[:n]

    def free_pages(self, group: int = 0) -> int:
        return checked(lib().cellm_cache_free_pages(self._h, group))

    @property
    def free_slots(self) -> int:
        return lib().cellm_cache_free_slots(self._h)

    @property
    def live(self) -> int:
        return lib().cellm_cache_live(self._h)

    def max_blocks(self, group: int) -> int:
        return self.group_pages[group]

    def pages_for(self, group: int, tokens: int, portion: int) -> int:
        return checked(lib().cellm_cache_pages_for(self._h, group, tokens, portion))

    # ------------------------------------------------------------ bindings
    def bindings(self, block_tables: Sequence[torch.Tensor]) -> list[CacheBinding]:
        """One CacheBinding per order item for a step whose block tables
        (one [B, blocks] int32 tensor per paged group) are given."""
        out = []
        for i, ig in enumerate(self._item_group):
            if ig is None:
                out.append(CacheBinding())
                continue
            fam, g, idx = ig
            if fam == "paged":
                out.append(CacheBinding(need=self.paged_keys[g], writes=not self._borrowed[i],
                                        k=self.k_pools[g][idx], v=self.v_pools[g][idx],
                                        block_table=block_tables[g], page_size=self.page_size,
                                        num_pages=self.group_pages[g]))
            else:
                out.append(CacheBinding(need=self.state_keys[g], writes=not self._borrowed[i],
                                        state=self.states[g][idx], num_slots=self.num_slots))
        return out

    def bytes_per_token(self) -> int:
        """Bytes of keys and values one token occupies over all paged groups."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * p.shape[0] * p.shape[2] * p.shape[4] * el for p in self.k_pools)
