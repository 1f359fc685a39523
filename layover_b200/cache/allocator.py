"""A pool of numbered pages (or state slots): which are out, which may be handed out next.

What the reference's allocator does and this one keeps (layover/kv/allocator.py:15-60): a request
for several pages is served whole or not at all, and the page given back last is handed out
first. What it drops: reference counts. No two requests share a page in this engine, so a page
is either free or out to exactly one table, and giving back a page that is not out (a second
time, or one that never left) is an error rather than a no-op.
"""

from __future__ import annotations


class OutOfBlocks(RuntimeError):
    """The pool is too empty for what was asked. Nothing was taken."""


OutOfPages = OutOfBlocks


class BlockAllocator:
    """Pages 0 .. num_blocks - 1. `_stack` holds the free ones, the next to go out at its end;
    `_out[page]` says whether a page is with a caller."""

    def __init__(self, num_blocks: int):
        if num_blocks < 1:
            raise ValueError(f"a pool needs at least one block, got {num_blocks}")
        self.num_blocks = int(num_blocks)
        self._stack = list(reversed(range(self.num_blocks)))    # page 0 leaves first
        self._out = bytearray(self.num_blocks)

    @property
    def num_free(self) -> int:
        return len(self._stack)

    @property
    def num_used(self) -> int:
        return self.num_blocks - self.num_free

    def alloc(self, count: int = 1) -> list[int]:
        """`count` pages, most recently freed first; OutOfBlocks (and no change) if fewer are free."""
        if count < 0:
            raise ValueError(f"cannot hand out {count} blocks")
        if count > self.num_free:
            raise OutOfBlocks(f"{count} blocks wanted, {self.num_free} of {self.num_blocks} free")
        if count == 0:
            return []
        taken = self._stack[-count:]
        del self._stack[-count:]
        taken.reverse()
        for page in taken:
            self._out[page] = 1
        return taken

    def is_held(self, block: int) -> bool:
        return 0 <= block < self.num_blocks and bool(self._out[block])

    def free(self, block: int) -> None:
        if not 0 <= block < self.num_blocks:
            raise ValueError(f"block {block} is outside a pool of {self.num_blocks}")
        if not self._out[block]:
            raise ValueError(f"block {block} is not allocated (freed twice?)")
        self._out[block] = 0
        self._stack.append(block)

    def check(self) -> None:
        """No block lost, none both free and held, none free twice."""
        free = set(self._stack)
        if len(free) != len(self._stack):
            raise AssertionError("a block is on the free list twice")
        for block in range(self.num_blocks):
            if bool(self._out[block]) == (block in free):
                raise AssertionError(f"block {block} is {'held and free' if self._out[block] else 'lost'}")
