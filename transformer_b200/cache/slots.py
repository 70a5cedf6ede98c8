"""Host-side bookkeeping of the cache: slots (one per live sequence) and pages (64 tokens each).

Pure Python, no device: the rules that must never break are checked here and tested on the CPU --
no slot or page is lost, held twice or freed twice, and what a finished batch held is used again.
"""
from __future__ import annotations

from typing import Dict, List

PAGE = 64  # tokens per page; equals TB_PAGE of the kernels


class CacheError(RuntimeError):
    pass


class FreeList:
    """Integers 0..n-1, handed out lowest first and taken back."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))   # pop() gives the lowest
        self._held = set()

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what}: all {self.n} are in use")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is not held (freed twice, or never taken)")
        self._held.remove(i)
        self._free.append(i)
        if len(self._free) > 1 and self._free[-1] > self._free[-2]:
            self._free.sort(reverse=True)

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def check(self) -> None:
        assert len(self._free) + len(self._held) == self.n, f"{self.what} lost"
        assert not (set(self._free) & self._held), f"{self.what} both free and held"
        assert len(set(self._free)) == len(self._free), f"{self.what} twice in the free list"


class SequenceTable:
    """Slots with their lengths and page lists."""

    def __init__(self, max_slots: int, n_pages: int, max_context: int):
        self.max_slots = max_slots
        self.n_pages = n_pages
        self.max_context = max_context
        self.max_pages_per_seq = (max_context + PAGE - 1) // PAGE
        self.slots = FreeList(max_slots, "slot")
        self.pages = FreeList(n_pages, "page")
        self.length: Dict[int, int] = {}
        self.page_list: Dict[int, List[int]] = {}

    def open(self) -> int:
        s = self.slots.take()
        self.length[s] = 0
        self.page_list[s] = []
        return s

    def close(self, slot: int) -> None:
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open (closed twice, or never opened)")
        for p in self.page_list.pop(slot):
            self.pages.give_back(p)
        del self.length[slot]
        self.slots.give_back(slot)

    def pages_needed(self, slot: int, new_tokens: int) -> int:
        total = self.length[slot] + new_tokens
        return max(0, (total + PAGE - 1) // PAGE - len(self.page_list[slot]))

    def extend(self, slot: int, new_tokens: int) -> int:
        """Make room for new_tokens more tokens; returns the position of the first of them."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open")
        start = self.length[slot]
        total = start + new_tokens
        if total > self.max_context:
            raise CacheError(f"sequence in slot {slot} would reach {total} tokens; the context holds {self.max_context}")
        need = self.pages_needed(slot, new_tokens)
        if need > self.pages.free:
            raise CacheError(f"cache full: {need} more pages of {PAGE} tokens needed, {self.pages.free} free "
                             f"of {self.n_pages}")
        for _ in range(need):
            self.page_list[slot].append(self.pages.take())
        self.length[slot] = total
        return start

    def truncate(self, slot: int, length: int) -> None:
        """Forget the sequence's tokens from position ``length`` on and give back the pages that then hold
        nothing (a step that failed after :meth:`extend` puts the sequence back to where it was)."""
        if slot not in self.length:
            raise CacheError(f"slot {slot} is not open")
        if not (0 <= length <= self.length[slot]):
            raise CacheError(f"slot {slot} holds {self.length[slot]} tokens; cannot truncate to {length}")
        keep = (length + PAGE - 1) // PAGE
        pl = self.page_list[slot]
        while len(pl) > keep:
            self.pages.give_back(pl.pop())
        self.length[slot] = length

    def check(self) -> None:
        self.slots.check()
        self.pages.check()
        held = [p for pl in self.page_list.values() for p in pl]
        assert len(held) == len(set(held)), "a page is held by two sequences"
        assert len(held) == self.pages.held, "pages held do not match the sequences' lists"
        assert set(self.length) == set(self.page_list)
        assert len(self.length) == self.slots.held
        for s, n in self.length.items():
            assert len(self.page_list[s]) == (n + PAGE - 1) // PAGE
