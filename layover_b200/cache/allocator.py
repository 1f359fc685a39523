"""Free lists for pages and for per-request state slots.

Pages are handed out all-or-nothing and the most recently freed page is reused first
(layover/kv/allocator.py:15-60). There is no sharing between requests in this engine, so a page
is either free or held by exactly one table; freeing a page twice or freeing one that was never
handed out is an error, not a no-op.
"""

from __future__ import annotations


class OutOfBlocks(RuntimeError):
    """The pool cannot satisfy an allocation. No state changed."""


OutOfPages = OutOfBlocks


class BlockAllocator:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        self.num_blocks = num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))  # pop() hands out 0 first
        self._held = [False] * num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_blocks - len(self._free)

    def alloc(self, count: int = 1) -> list[int]:
        if count < 0:
            raise ValueError("count must not be negative")
        if count > len(self._free):
            raise OutOfBlocks(f"need {count} blocks, {len(self._free)} free")
        blocks = [self._free.pop() for _ in range(count)]
        for block in blocks:
            self._held[block] = True
        return blocks

    def is_held(self, block: int) -> bool:
        return 0 <= block < self.num_blocks and self._held[block]

    def free(self, block: int) -> None:
        if not 0 <= block < self.num_blocks:
            raise ValueError(f"block {block} is outside a pool of {self.num_blocks}")
        if not self._held[block]:
            raise ValueError(f"block {block} is not allocated (freed twice?)")
        self._held[block] = False
        self._free.append(block)

    def check(self) -> None:
        """No block lost, none both free and held, none free twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a block is on the free list twice")
        for block in range(self.num_blocks):
            if self._held[block] == (block in free):
                raise AssertionError(f"block {block} is {'held and free' if self._held[block] else 'lost'}")
