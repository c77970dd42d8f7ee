"""Slots for per-request state of fixed size.

A request takes a slot when it is admitted and keeps it until it ends (also across a preemption
that gives its pages back).  The slot indexes everything that is one fixed-size record per live
request: the rows of the block tables, the sampling record (temperature, seed, output count) and
any mixer state tensor ``[num_slots, ...]``.  The reference keeps such facts scattered in its host
``Sequence`` (``ginfer/engine/sequence.h:22-37``) and has nothing per request on the device.
"""
from __future__ import annotations


class NoFreeSlot(RuntimeError):
    pass


class SlotPool:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("at least one slot is needed")
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._holder: dict[int, object] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, holder) -> int:
        if not self._free:
            raise NoFreeSlot(f"all {self.num_slots} request slots are taken")
        s = self._free.pop()
        self._holder[s] = holder
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._holder:
            raise RuntimeError(f"slot {slot} is returned twice or was never taken")
        del self._holder[slot]
        self._free.append(slot)

    def holder_of(self, slot: int):
        return self._holder.get(slot)
