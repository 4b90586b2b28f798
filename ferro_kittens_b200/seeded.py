"""Counter-based seeded operands: every value is a function of (seed, tensor id, flat index) alone.

A rank that holds rows ``[r0, r1)`` of a matrix derives exactly the words any other rank, the host
or a test would derive for those rows: nothing is generated whole and sliced, and no generator
state is shared. Only integer arithmetic and single IEEE operations are used, so a CUDA device
and the host produce the same bits.

* the hash is splitmix64's finaliser over ``seed``, ``tensor`` and ``index``;
* ``uniform``: the top 24 bits ``u`` of one hash -> ``2 u / 2^24 - 1`` in [-1, 1);
* ``normal``: the sum of the twelve 16-bit lanes of three hashes, centred and scaled by
  ``1 / 65536`` -- the Irwin-Hall(12) stand-in for N(0, 1) (mean 0, variance 1 + O(2^-32), support
  +-6): Box-Muller's logarithm and cosine differ in the last place between libm and CUDA, which
  would break the bit-for-bit agreement this module exists for.

Values are rounded to bf16 (round to nearest even) once, here; everything downstream consumes the
rounded words.
"""
from __future__ import annotations

import torch

_GOLDEN = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB


def _signed(value: int) -> int:
    value &= (1 << 64) - 1
    return value - (1 << 64) if value >= (1 << 63) else value


def _lsr(x: torch.Tensor, bits: int) -> torch.Tensor:
    """Logical shift right of int64 words (torch's ``>>`` is arithmetic)."""
    return (x >> bits) & ((1 << (64 - bits)) - 1)


def mix64(x: torch.Tensor) -> torch.Tensor:
    """splitmix64's output function on int64 words (two's-complement wrap-around)."""
    z = x + _signed(_GOLDEN)
    z = (z ^ _lsr(z, 30)) * _signed(_M1)
    z = (z ^ _lsr(z, 27)) * _signed(_M2)
    return z ^ _lsr(z, 31)


def _key(seed: int, tensor: int, draw: int) -> int:
    return _signed((seed * 0xD1342543DE82EF95 + tensor * 0xA0761D6478BD642F + draw * 0xE7037ED1A0B428DB) & ((1 << 64) - 1))


def _hashed_index(first: int, count: int, device) -> torch.Tensor:
    return mix64(torch.arange(first, first + count, dtype=torch.int64, device=device))


def _stream(seed: int, tensor: int, first: int, count: int, draw: int, device) -> torch.Tensor:
    """Hash words of flat indices ``[first, first + count)``, draw number ``draw``:
    ``mix64(mix64(index) ^ key(seed, tensor, draw))``."""
    return mix64(_hashed_index(first, count, device) ^ _key(seed, tensor, draw))


def uniform(seed: int, tensor: int, first: int, count: int, device="cpu") -> torch.Tensor:
    """fp32 values in [-1, 1) for flat indices ``[first, first + count)``."""
    top = _lsr(_stream(seed, tensor, first, count, 0, device), 40)  # 24 bits
    return (top.to(torch.float32) * (2.0 / (1 << 24))) - 1.0


def normal(seed: int, tensor: int, first: int, count: int, device="cpu") -> torch.Tensor:
    """fp64 Irwin-Hall(12) values (mean 0, variance 1) for flat indices ``[first, first + count)``:
    the twelve 16-bit lanes of draws 1, 2 and 3, summed."""
    hashed = _hashed_index(first, count, device)
    pairs = torch.zeros(count, dtype=torch.int64, device=device)
    for draw in range(3):
        word = mix64(hashed ^ _key(seed, tensor, 1 + draw))
        # lanes 0 and 2 in one add, lanes 1 and 3 in another: two 32-bit fields each holding a sum of lanes
        pairs += (word & 0x0000FFFF0000FFFF) + (_lsr(word, 16) & 0x0000FFFF0000FFFF)
    total = (pairs & 0xFFFFFFFF) + _lsr(pairs, 32)
    # twelve lanes of mean 32767.5 and variance (2^32 - 1) / 12 each
    return (total.to(torch.float64) - 12 * 32767.5) * (1.0 / 65536.0)


def bf16_rows(kind: str, seed: int, tensor: int, row0: int, rows: int, columns: int, scale: float = 1.0,
              device="cpu", chunk_rows: int | None = None) -> torch.Tensor:
    """Rows ``[row0, row0 + rows)`` of a row-major ``[*, columns]`` matrix as bf16.

    ``kind`` is ``"normal"`` (value x ``scale`` in fp64, narrowed to fp32 and then to bf16, each a
    single IEEE rounding, so host and device agree) or ``"uniform"``.
    Generated in blocks of ``chunk_rows`` rows to bound the temporaries: by default about a million
    elements on the host (the element-wise passes then stay in cache) and sixteen million on a device
    (few launches).
    """
    if chunk_rows is None:
        on_host = torch.device(device).type == "cpu"
        chunk_rows = max(1, ((1 << 20) if on_host else (1 << 24)) // max(1, columns))
    out = torch.empty((rows, columns), dtype=torch.bfloat16, device=device)
    for start in range(0, rows, chunk_rows):
        stop = min(rows, start + chunk_rows)
        first, count = (row0 + start) * columns, (stop - start) * columns
        if kind == "normal":
            values = (normal(seed, tensor, first, count, device) * scale).to(torch.float32)
        elif kind == "uniform":
            values = uniform(seed, tensor, first, count, device) * scale
        else:
            raise ValueError(f"unknown distribution {kind!r}")
        out[start:stop] = values.view(stop - start, columns).to(torch.bfloat16)
    return out
