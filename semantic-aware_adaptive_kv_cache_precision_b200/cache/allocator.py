"""Who holds what: sequence slots and cache blocks. Host-side bookkeeping only.

A slot stands for one live sequence; a block holds 64 consecutive positions of
one sequence (for every cache entry of its group). Both come from a pool of
fixed size and go back to it when the sequence ends, to be used again by a later
batch. Taking is all-or-nothing, and every misuse (freeing twice, freeing what
was never taken) is an error, so that a slot or block can neither leak nor be
held by two sequences. The reference's counterpart is the all-or-nothing
`reserve` of its page allocator (`src/core_kernels/kv_pages.cu:219-263`).
"""

from __future__ import annotations


class CacheFull(RuntimeError):
    """The cache has no room for what was asked; nothing was taken."""


class Pool:
    """Identifiers 0..size-1, handed out lowest-free-first and taken back."""

    def __init__(self, size: int, what: str):
        if size < 0:
            raise ValueError(f"a pool of {what}s cannot have size {size}")
        self.size, self.what = size, what
        self._free = list(range(size - 1, -1, -1))      # pop() gives the lowest id
        self._held = set()

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self, count: int = 1) -> list[int]:
        if count < 0:
            raise ValueError(f"cannot take {count} {self.what}s")
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) asked for, {len(self._free)} of "
                            f"{self.size} free; nothing was taken")
        got = [self._free.pop() for _ in range(count)]
        self._held.update(got)
        return got

    def give_back(self, ids) -> None:
        ids = list(ids)
        bad = [i for i in ids if i not in self._held]
        if bad or len(set(ids)) != len(ids):
            raise RuntimeError(f"{self.what}(s) {sorted(set(bad)) or ids} given back but not "
                               "held (freed twice, or never taken)")
        for i in ids:
            self._held.remove(i)
        self._free.extend(ids)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every id is either free or held, exactly once."""
        free = list(self._free)
        if len(set(free)) != len(free) or set(free) & self._held \
                or set(free) | self._held != set(range(self.size)):
            raise RuntimeError(f"the {self.what} pool is inconsistent: free {sorted(free)}, "
                               f"held {sorted(self._held)}")
