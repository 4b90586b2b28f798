"""B200-native (sm_100a) implementation of ferro-kittens' two dense-contraction
hot paths -- the two-CTA-cluster bf16 GEMM and flash-attention forward -- behind
a C ABI, with this package as the thin host-side mirror of the crate's surface.
"""
from . import _lib, flash_backward, flash_forward, gemm, global_layout, plan, rows, shard, watchdog  # noqa: F401
from ._lib import FerroKittensError  # noqa: F401
