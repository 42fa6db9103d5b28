"""Host-side bookkeeping of what a sequence slot owns on the device: pages of the token cache, and (for models with
recurrent layers) the slot's row in the state pools."""
from __future__ import annotations

import numpy as np

PAGE = 32          # tokens per cache page (ops.kernels.PAGE_SIZE)


class PageAllocator:
    """Host-side KV page allocator: per-slot page lists over one shared pool (per-user KV caches;
    the reference has a single cache shared by all users, src/llm.cpp:197-198)."""

    def __init__(self, n_pages: int, n_slots: int, max_pages_per_seq: int):
        self.free_pages = list(range(n_pages - 1, -1, -1))
        self.free_slots = list(range(n_slots - 1, -1, -1))
        self.max_pages = max_pages_per_seq
        self.table = np.zeros((n_slots, max_pages_per_seq), dtype=np.int32)
        self.n_used = np.zeros(n_slots, dtype=np.int32)
        self.dirty = True

    def alloc_slot(self) -> int:
        if not self.free_slots:
            raise RuntimeError("no free sequence slot")
        return self.free_slots.pop()

    def free_slot(self, slot: int):
        for i in range(int(self.n_used[slot])):
            self.free_pages.append(int(self.table[slot, i]))
        self.n_used[slot] = 0
        self.free_slots.append(slot)

    def release_pages(self, slot: int):
        """Return a slot's pages to the pool; the slot id itself stays with its owner (the scheduler)."""
        for i in range(int(self.n_used[slot])):
            self.free_pages.append(int(self.table[slot, i]))
        self.n_used[slot] = 0

    def ensure(self, slot: int, n_tokens: int):
        need = (n_tokens + PAGE - 1) // PAGE
        if need > self.max_pages:
            raise RuntimeError(f"sequence of {n_tokens} tokens exceeds max_seq_len")
        while self.n_used[slot] < need:
            if not self.free_pages:
                raise RuntimeError("KV cache exhausted")
            self.table[slot, self.n_used[slot]] = self.free_pages.pop()
            self.n_used[slot] += 1
            self.dirty = True
