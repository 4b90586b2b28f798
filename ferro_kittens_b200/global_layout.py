"""Global layouts and their TMA tensor maps.

Python spelling of the host half of the reference's ``global`` module
(src/global.rs:1649-2076): ``GlobalLayout::packed`` / ``strided``,
``descriptor_shape``, ``check_driver_requirements``, ``tensor_map`` and
``encode_bf16_panels``. Dimension 0 is the contiguous one, so a row-major
``[rows, columns]`` matrix has ``extents = [columns, rows]``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_uint32, c_uint64

from . import _lib
from ._lib import FK_BF16, FK_SWIZZLE_128B, Layout, check, library

#: One SWIZZLE_128B atom of bf16: the only box width a swizzled tile takes.
ATOM_COLUMNS = 64


class TensorMap:
    """A 128-byte, 64-byte-aligned ``CUtensorMap`` owned by this object."""

    def __init__(self):
        self._raw = ctypes.create_string_buffer(128 + 64)
        address = ctypes.addressof(self._raw)
        self._address = (address + 63) & ~63

    def as_ptr(self) -> int:
        """The address kernels' launchers take as their tensor-map parameter."""
        return self._address

    def bytes(self) -> bytes:
        return ctypes.string_at(self._address, 128)


class GlobalLayout:
    """A rank-1..5 global buffer, dimension 0 contiguous (src/global.rs:1767-1889).

    Does not own or borrow the buffer: the caller keeps the allocation alive for
    every launch consuming a map built from the layout.
    """

    def __init__(self, raw: Layout):
        self._raw = raw

    @classmethod
    def packed(cls, base: int, extents, element: int = FK_BF16) -> "GlobalLayout":
        raw = Layout()
        array = (c_uint64 * len(extents))(*extents)
        check(library().fk_layout_packed(ctypes.byref(raw), base, element, len(extents), array))
        return cls(raw)

    @classmethod
    def strided(cls, base: int, extents, element_strides, element: int = FK_BF16) -> "GlobalLayout":
        raw = Layout()
        array = (c_uint64 * len(extents))(*extents)
        strides = (c_uint64 * len(element_strides))(*element_strides)
        check(library().fk_layout_strided(ctypes.byref(raw), base, element, len(extents), array, strides))
        return cls(raw)

    @property
    def rank(self) -> int:
        return self._raw.rank

    @property
    def extents(self) -> list[int]:
        return list(self._raw.extents[: self.rank])

    @property
    def strides(self) -> list[int]:
        return list(self._raw.strides_bytes[: self.rank])

    def descriptor_shape(self, box_columns: int, box_rows: int) -> tuple[list[int], list[int]]:
        extents = (c_uint64 * 5)()
        box = (c_uint32 * 5)()
        check(library().fk_layout_descriptor_shape(ctypes.byref(self._raw), box_columns, box_rows, extents, box))
        return list(extents[: self.rank]), list(box[: self.rank])

    def check_driver_requirements(self, extents, box) -> None:
        extents_array = (c_uint64 * 5)(*extents)
        box_array = (c_uint32 * 5)(*box)
        check(library().fk_layout_check(ctypes.byref(self._raw), extents_array, box_array))

    def tensor_map(self, box_rows: int, box_columns: int = ATOM_COLUMNS,
                   swizzle: int = FK_SWIZZLE_128B) -> TensorMap:
        """Encode the map that moves ``[box_rows, box_columns]`` boxes of this buffer."""
        out = TensorMap()
        check(library().fk_tensor_map(out.as_ptr(), ctypes.byref(self._raw), box_columns, box_rows, swizzle))
        return out


def encode_bf16_panels(base: int, box_rows: int, columns: int, rows: int, planes: int) -> TensorMap:
    """Rank-3 SWIZZLE_128B map over packed ``[planes, rows, columns]`` bf16 (src/global.rs:2067-2076)."""
    out = TensorMap()
    check(library().fk_encode_bf16_panels(out.as_ptr(), base, box_rows, columns, rows, planes))
    return out
