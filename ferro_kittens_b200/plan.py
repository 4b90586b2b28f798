"""The shared-memory plan cursor and the launch envelope.

``SharedPlan`` mirrors the reference's cursor (src/plan.rs:73-304): each
reservation aligns to its own rule and the running total is what the launch
declares. ``admit_shared_plan`` mirrors src/launch.rs:110-132.
"""
from __future__ import annotations

import ctypes
from ctypes import c_uint32

from ._lib import FK_BF16, Plan, check, library


class SharedPlan:
    TILE_ALIGN = 128
    BARRIER_BYTES = 8
    BARRIER_ALIGN = 8
    TMEM_SLOT_BYTES = 4

    def __init__(self):
        self._raw = Plan()
        library().fk_plan_sizing(ctypes.byref(self._raw))

    @classmethod
    def sizing(cls) -> "SharedPlan":
        return cls()

    def bytes(self) -> int:
        return self._raw.bytes

    def reserve(self, size: int, align: int) -> int:
        if align & (align - 1):
            raise ValueError("an alignment is a power of two")
        return library().fk_plan_reserve(ctypes.byref(self._raw), size, align)

    def tile(self, rows: int, columns: int, element: int = FK_BF16) -> int:
        return library().fk_plan_tile(ctypes.byref(self._raw), element, rows, columns)

    def tile_ring(self, rows: int, columns: int, count: int, element: int = FK_BF16) -> int:
        return library().fk_plan_tile_ring(ctypes.byref(self._raw), element, rows, columns, count)

    def semaphores(self, count: int) -> int:
        return library().fk_plan_semaphores(ctypes.byref(self._raw), count)

    def semaphore(self) -> int:
        return self.semaphores(1)

    def tmem_slot(self) -> int:
        return library().fk_plan_tmem_slot(ctypes.byref(self._raw))


def admit_shared_plan(kernel: int, size: int) -> int:
    """Opt a kernel into ``size`` bytes of dynamic shared memory; returns the device limit."""
    limit = c_uint32(0)
    check(library().fk_admit_shared_plan(kernel, size, ctypes.byref(limit)))
    return limit.value
