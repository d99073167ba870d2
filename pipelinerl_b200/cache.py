"""What a sampler engine keeps per live sequence, independent of the model it serves.

`PagePool` hands out fixed-size KV pages with reference counts (a page may belong to a request and to the prefix cache
at once); `SlotStates` owns every per-slot tensor a model registers for state that is NOT addressed by position — the
matrix state of a linear-attention or state-space layer, the tail of inputs of a short convolution — and clears a slot
when a new sequence takes it.  The engines in engine.py (softmax-attention decoders) and hybrid.py (attention +
recurrent mixers) both allocate through these two classes, so a page or slot that one request gave back is what the
next request gets, whatever the model.
"""
from __future__ import annotations

import torch

PAGE_SIZE = 64


class PagePool:
    """Free list + reference counts of the pages 1 .. n_pages-1 (page 0 is the scratch page idle slots point at)."""

    def __init__(self, n_pages: int):
        if n_pages < 2:
            raise ValueError("a page pool needs at least one page besides the scratch page")
        self.n_pages = n_pages
        self.free: list[int] = list(range(n_pages - 1, 0, -1))
        self.ref: list[int] = [0] * n_pages

    def available(self) -> int:
        return len(self.free)

    def alloc(self, n: int) -> list[int]:
        if len(self.free) < n:
            raise RuntimeError("engine out of KV pages")
        pages = [self.free.pop() for _ in range(n)]
        for pg in pages:
            self.ref[pg] = 1
        return pages

    def retain(self, pg: int) -> None:
        self.ref[pg] += 1

    def release(self, pages) -> None:
        for pg in pages:
            self.ref[pg] -= 1
            if self.ref[pg] == 0:
                self.free.append(pg)
            elif self.ref[pg] < 0:
                raise RuntimeError(f"page {pg} released more often than it was taken")


class SlotStates:
    """Per-slot state tensors `[n_slots, *shape]`, zeroed for a slot when a sequence is admitted into it."""

    def __init__(self, n_slots: int, device):
        self.n_slots, self.device = n_slots, device
        self.tensors: dict[str, torch.Tensor] = {}

    def add(self, name: str, shape, dtype=torch.float32) -> torch.Tensor:
        if name in self.tensors:
            raise KeyError(f"state {name!r} registered twice")
        t = torch.zeros((self.n_slots, *shape), dtype=dtype, device=self.device)
        self.tensors[name] = t
        return t

    def reset(self, slot: int) -> None:
        for t in self.tensors.values():
            t[slot].zero_()

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())
