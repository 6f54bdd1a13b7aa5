"""Paged KV-cache allocator (host side).

llama.cpp keeps one contiguous f16 K and V buffer per layer sized n_ctx and a slot finder
(`llama_kv_cache`, un-vendored upstream behind /root/reference/api.py:24-28).
This engine pages it: the device holds one pool of fixed-size pages shared by all sequences,
and each sequence owns a page table. This class hands out page ids; the engine only ever sees
`b2_seq_set_blocks(slot, pages)`.

Invariants (property-tested in tests/test_kv_pages.py): a page is owned by at most one sequence,
pages are never leaked, `free + owned == num_blocks`.
"""
from __future__ import annotations

import threading
from typing import Dict, List


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_blocks: int, block_tokens: int):
        if num_blocks <= 0 or block_tokens <= 0:
            raise ValueError("num_blocks and block_tokens must be positive")
        self.num_blocks = num_blocks
        self.block_tokens = block_tokens
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))   # pop() hands out low ids first
        self._owned: Dict[int, List[int]] = {}
        self._lock = threading.Lock()

    def pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block_tokens - 1) // self.block_tokens

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def table(self, seq_id: int) -> List[int]:
        return list(self._owned.get(seq_id, ()))

    def ensure(self, seq_id: int, n_tokens: int) -> bool:
        """Grow seq_id's page table to cover n_tokens. Returns True if the table changed."""
        with self._lock:
            pages = self._owned.setdefault(seq_id, [])
            need = self.pages_for(n_tokens) - len(pages)
            if need <= 0:
                return False
            if need > len(self._free):
                raise OutOfPages(f"need {need} KV pages, {len(self._free)} free")
            for _ in range(need):
                pages.append(self._free.pop())
            return True

    def release(self, seq_id: int) -> None:
        with self._lock:
            pages = self._owned.pop(seq_id, [])
            self._free.extend(reversed(pages))

    def truncate(self, seq_id: int, n_tokens: int) -> None:
        """Keep only the pages covering the first n_tokens (prefix reuse)."""
        with self._lock:
            pages = self._owned.get(seq_id, [])
            keep = self.pages_for(n_tokens)
            while len(pages) > keep:
                self._free.append(pages.pop())


class SequenceSlots:
    """Sequence slots of one engine: a slot is a page table plus, for models with recurrent layers, one state slot on
    the device. `open` binds a caller's key to a free slot and starts the sequence from nothing (the engine zeroes the
    slot's recurrent state; pages are taken as the sequence grows), `close` gives the pages and the slot back for the
    next sequence. Used by the trace runner and by anything else that steps an engine without the request scheduler."""

    def __init__(self, engine):
        self.engine = engine
        self._free: List[int] = list(range(engine.max_seqs - 1, -1, -1))
        self._slot: Dict[object, int] = {}
        self._len: Dict[object, int] = {}

    def __contains__(self, key) -> bool:
        return key in self._slot

    def slot(self, key) -> int:
        return self._slot[key]

    def length(self, key) -> int:
        return self._len[key]

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def open(self, key, sampling=None, uniforms=None) -> int:
        if key in self._slot:
            raise ValueError(f"sequence {key!r} is already open")
        if not self._free:
            raise RuntimeError(f"all {self.engine.max_seqs} sequence slots are in use")
        slot = self._free.pop()
        if sampling is None:
            from .engine import SamplingSettings
            sampling = SamplingSettings(temperature=0.0, repeat_penalty=1.0)
        self.engine.release(slot)
        self.engine.seq_begin(slot, 0, [], sampling, uniforms)
        self._slot[key], self._len[key] = slot, 0
        return slot

    def extend(self, key, n_tokens: int) -> int:
        """Reserve pages for n_tokens more tokens of the sequence; returns its slot."""
        slot = self._slot[key]
        self._len[key] += int(n_tokens)
        self.engine.ensure_pages(slot, self._len[key])
        return slot

    def close(self, key) -> None:
        slot = self._slot.pop(key)
        self._len.pop(key)
        self.engine.release(slot)
        self._free.append(slot)
