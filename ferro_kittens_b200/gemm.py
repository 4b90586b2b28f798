"""bf16 GEMM ``C = A . B^T`` through the C ABI.

Host-side mirror of ``examples/src/gemm.rs``: ``tile_grid`` (:466-468), ``grid``
(:472-475) and ``run`` (:477-538) with torch tensors standing in for the
reference's device buffers. torch supplies memory and streams only.
"""
from __future__ import annotations

import torch

from ._lib import FK_SWIZZLE_NONE, check, library
from .global_layout import GlobalLayout

BLOCK_M = 128
BLOCK_N = 256
BLOCK_K = 64
#: The traversal width: the reference ships 8 for its kernel (examples/src/gemm.rs:138); this one measures
#: best at 6 on 148 SMs (its 74 items in flight then cover 6 x 12.3 tiles: the fewest operand bytes per wave).
GROUP = 6
#: fp16 A and B (C stays bf16): the operand types of examples/src/gemm_sol.rs.
F16_OPERANDS = 1
#: C += A . B^T through the copy engine's reduce-add (src/shared.rs:974-1009).
ACCUMULATE = 2
#: max(x, 0) before the rounding (the `Relu` unary map, src/reg.rs:261).
RELU = 4
#: Pick the kernel instead of letting the launch choose: one CTA per [128, 128] tile (the reference's
#: narrow entry for launches at or below half a wave, examples/src/gemm_sol.rs:1063), or the wide
#: persistent two-CTA clusters.
TILE_NARROW = 8
TILE_WIDE = 16
#: Pick how the wide kernel's clusters get their items: handed out through cluster launch control as
#: clusters fall free, or a static round-robin.
ORDER_FEED = 32
ORDER_STATIC = 64


def tile_grid(m: int, n: int) -> tuple[int, int]:
    return m // (2 * BLOCK_M), n // BLOCK_N


def grid(m: int, n: int, sm_count: int = 148) -> int:
    return library().fk_gemm_grid(m, n, sm_count)


def _require_cuda_bf16(name: str, tensor: torch.Tensor) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
    if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
        raise ValueError(f"{name} must be a contiguous bfloat16 tensor")


def new_status(device) -> torch.Tensor:
    """Zeroed device words for a launch; it writes the first four only if one of its waits gives up."""
    return torch.zeros(8, dtype=torch.int32, device=device)


def maps(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor):
    """The three tensor maps of a launch: A and B as loads, C as a store."""
    m, k = a.shape
    n = b.shape[0]
    a_map = GlobalLayout.packed(a.data_ptr(), [k, m]).tensor_map(BLOCK_M)
    b_map = GlobalLayout.packed(b.data_ptr(), [k, n]).tensor_map(BLOCK_N // 2)
    c_map = GlobalLayout.strided(c.data_ptr(), [n, m], [1, c.stride(0)]).tensor_map(32)
    return a_map, b_map, c_map


def launch(a_map, b_map, c_map, m: int, n: int, k: int, group: int = GROUP, status=None,
           stream=None) -> None:
    """Enqueue the kernel on ``stream`` (torch's current stream by default)."""
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    check(library().fk_gemm_bf16_launch(a_map.as_ptr(), b_map.as_ptr(), c_map.as_ptr(), m, n, k,
                                        group, handle, status.data_ptr() if status is not None else None))


def group_for(m: int, n: int, device) -> int:
    """The traversal width this library would pick for an [m, n] product on ``device`` (:data:`GROUP` for
    matrices at least as wide as the items in flight span, shorter bands for narrower ones)."""
    sm_count = torch.cuda.get_device_properties(device).multi_processor_count
    return library().fk_gemm_group(m, n, sm_count)


def item_columns(m: int, n: int, k: int, device, flags: int = 0) -> int:
    """Columns of C per item the wide kernel would take for this shape on ``device``: 256, or 224 / 192
    where a launch's tiles sit just past a whole number of waves and narrower items fill them better."""
    sm_count = torch.cuda.get_device_properties(device).multi_processor_count
    return library().fk_gemm_item_columns(m, n, k, flags, sm_count)


class TiledMaps:
    """The maps of a launch whose item width was chosen for the shape (:func:`item_columns`): B's box is
    ``columns / 2`` rows, and items of 224 columns store their last 32 through ``c_tail``."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, columns: int | None = None):
        m, k = a.shape
        n = b.shape[0]
        self.columns = item_columns(m, n, k, a.device) if columns is None else columns
        self.a = GlobalLayout.packed(a.data_ptr(), [k, m]).tensor_map(BLOCK_M)
        self.b = GlobalLayout.packed(b.data_ptr(), [k, n]).tensor_map(self.columns // 2)
        c_layout = GlobalLayout.strided(c.data_ptr(), [n, m], [1, c.stride(0)])
        self.c = c_layout.tensor_map(32)
        self.c_tail = c_layout.tensor_map(32, 32, FK_SWIZZLE_NONE) if self.columns % 64 else None


def launch_tiled(maps: TiledMaps, m: int, n: int, k: int, group: int = GROUP, status=None, stream=None,
                 flags: int = 0, bias: torch.Tensor | None = None) -> None:
    """:func:`launch` for maps built to the chosen item width."""
    handle = (stream or torch.cuda.current_stream()).cuda_stream
    check(library().fk_gemm_launch_tiled(maps.a.as_ptr(), maps.b.as_ptr(), maps.c.as_ptr(),
                                         maps.c_tail.as_ptr() if maps.c_tail is not None else None, maps.columns,
                                         bias.data_ptr() if bias is not None else None,
                                         m, n, k, group, flags, handle,
                                         status.data_ptr() if status is not None else None))


def workspace(m: int, n: int, k: int, device, sm_count: int | None = None) -> torch.Tensor | None:
    """A zeroed workspace for a launch that would split K (fewer items than half a wave), or None.

    Pass it to :func:`run`; every launch leaves it zeroed, so one tensor serves any number of
    launches of shapes up to this one, as long as they do not overlap on the device."""
    if sm_count is None:
        sm_count = torch.cuda.get_device_properties(device).multi_processor_count
    size = library().fk_gemm_workspace_bytes(m, n, k, sm_count)
    return torch.zeros(size, dtype=torch.uint8, device=device) if size else None


def run(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None = None, group: int = GROUP,
        status: torch.Tensor | None = None, accumulate: bool = False, bias: torch.Tensor | None = None,
        relu: bool = False, workspace: torch.Tensor | None = None, tile: str | None = None,
        order: str | None = None) -> torch.Tensor:
    """``C[m, n] (+)= map(sum_k A[m, k] * B[n, k] + bias[n])``; A is [m, k], B is [n, k], both bf16 or both fp16 on
    one GPU, C bf16. With ``accumulate`` the rounded product is added into ``c`` (in bf16, by the
    copy engine), which must then be given and hold values. With a ``workspace`` (see :func:`workspace`) a
    launch under one wave splits K across the idle SMs."""
    for name, tensor in (("a", a), ("b", b)):
        if not tensor.is_cuda:
            raise RuntimeError(f"{name} must live on a CUDA device: there is no CPU path")
        if tensor.dtype not in (torch.bfloat16, torch.float16) or not tensor.is_contiguous():
            raise ValueError(f"{name} must be a contiguous bfloat16 or float16 tensor")
    if a.dtype != b.dtype:
        raise ValueError("a and b must share one element type")
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] != k:
        raise ValueError("a and b disagree on K")
    if c is None:
        if accumulate:
            raise ValueError("accumulating needs the C to add into")
        c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if not c.is_cuda:
        raise RuntimeError("c must live on a CUDA device: there is no CPU path")
    if c.dtype != torch.bfloat16 or c.dim() != 2 or c.stride(1) != 1 or c.shape != (m, n):
        raise ValueError("c must be an [m, n] bfloat16 tensor with unit column stride (rows may be padded)")
    if bias is not None and (not bias.is_cuda or bias.dtype != torch.bfloat16 or bias.shape != (n,)
                             or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous bfloat16 [n] tensor on the device")
    if tile not in (None, "narrow", "wide"):
        raise ValueError("tile is None (the launch chooses), 'narrow' or 'wide'")
    if order not in (None, "feed", "static"):
        raise ValueError("order is None (the launch chooses), 'feed' or 'static'")
    flags = ((F16_OPERANDS if a.dtype == torch.float16 else 0) | (ACCUMULATE if accumulate else 0)
             | (RELU if relu else 0) | {None: 0, "narrow": TILE_NARROW, "wide": TILE_WIDE}[tile]
             | {None: 0, "feed": ORDER_FEED, "static": ORDER_STATIC}[order])
    if workspace is not None and (not workspace.is_cuda or not workspace.is_contiguous()):
        raise ValueError("the workspace must be a contiguous tensor on the device")
    with torch.cuda.device(a.device):
        handle = torch.cuda.current_stream().cuda_stream
        check(library().fk_gemm_fused_workspace(
            a.data_ptr(), b.data_ptr(), c.data_ptr(), bias.data_ptr() if bias is not None else None, m, n, k,
            c.stride(0), group, flags, workspace.data_ptr() if workspace is not None else None,
            workspace.numel() * workspace.element_size() if workspace is not None else 0, handle,
            status.data_ptr() if status is not None else None))
    return c


def check_status(status: torch.Tensor) -> None:
    """Raise if the kernel recorded a stalled wait."""
    with torch.cuda.device(status.device):
        check(library().fk_status_check(status.data_ptr(), torch.cuda.current_stream().cuda_stream))


def run_host(a, b, c, m: int, n: int, k: int, group: int = GROUP) -> None:
    """The whole path from host buffers (numpy uint16 / pinned torch tensors): stage, launch, read back."""
    def address(x):
        return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
    check(library().fk_gemm_bf16_host(address(a), address(b), address(c), m, n, k, group))


def run_host_noalloc(a, b, c, m: int, n: int, k: int, group: int = GROUP) -> None:
    """``run_host`` for callers that must not reach the CUDA allocator: the staging lives in an
    array built into the library, so each of A, B and C is limited to 8 MiB."""
    def address(x):
        return x.data_ptr() if hasattr(x, "data_ptr") else x.ctypes.data
    check(library().fk_gemm_bf16_host_noalloc(address(a), address(b), address(c), m, n, k, group))


class ShardedHostGemm:
    """``C[:, n0:n1] = A . B[n0:n1]^T`` from HOST buffers on every rank of a node, A replicated.

    The call a multi-GPU user of the host-buffer path makes. Each rank passes only ITS share of
    A's rows (``shard.a_rows``), its block of B's rows (``shard.gemm_columns``) and receives its
    column block of C: A crosses PCIe once in total instead of once per rank. Per block of rows
    (``shard.gather_blocks``) the pipeline is upload -> all-gather into this GPU's own memory
    (``torch.distributed``, NCCL over NVLink) -> GEMM over the gathered block -> read-back, on four
    streams, so the copies, the gather and the kernels of different blocks overlap. The kernels read
    local memory only; the gather is staging. With one rank it is ``run_host``'s pipeline without
    the gather. Buffers and streams are made once, here; ``run`` allocates nothing.
    """

    def __init__(self, m: int, n_local: int, k: int, world: int, rank: int, device, group: int = GROUP,
                 blocks: int = 4, process_group=None):
        from . import shard

        self.m, self.n, self.k, self.world, self.rank, self.group = m, n_local, k, world, rank, group
        self.device = torch.device(device)
        self.process_group = process_group
        self.row0, self.row1 = shard.a_rows(m, world, rank)
        self.share = self.row1 - self.row0
        self.blocks = shard.gather_blocks(m, world, blocks)
        bf16 = dict(dtype=torch.bfloat16, device=self.device)
        self.b = torch.empty((n_local, k), **bf16)
        self.own = [torch.empty((rows, k), **bf16) for _, rows in self.blocks]
        self.gathered = ([torch.empty((world, rows, k), **bf16) for _, rows in self.blocks] if world > 1
                         else [own.unsqueeze(0) for own in self.own])
        self.c = [torch.empty((world * rows, n_local), **bf16) for _, rows in self.blocks]
        self.status = new_status(self.device)
        with torch.cuda.device(self.device):
            self.upload, self.comm, self.compute, self.download = (torch.cuda.Stream() for _ in range(4))

    def run(self, a_share: torch.Tensor, b_block: torch.Tensor, c_out: torch.Tensor) -> None:
        """``a_share`` [share, k], ``b_block`` [n_local, k], ``c_out`` [m, n_local]: pinned host bf16
        tensors. Returns once ``c_out`` is complete on the host."""
        import torch.distributed as dist

        if a_share.shape != (self.share, self.k) or b_block.shape != (self.n, self.k) or c_out.shape != (self.m, self.n):
            raise ValueError("host operands do not have this plan's shapes")
        with torch.cuda.device(self.device):
            start = torch.cuda.Event()
            start.record(torch.cuda.current_stream())
            for stream in (self.upload, self.comm, self.compute, self.download):
                stream.wait_event(start)
            with torch.cuda.stream(self.compute):
                self.status.zero_()
            with torch.cuda.stream(self.upload):
                self.b.copy_(b_block, non_blocking=True)
                b_ready = torch.cuda.Event()
                b_ready.record(self.upload)
            self.compute.wait_event(b_ready)
            for index, (offset, rows) in enumerate(self.blocks):
                with torch.cuda.stream(self.upload):
                    self.own[index].copy_(a_share[offset:offset + rows], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(self.upload)
                whole = landed
                if self.world > 1:
                    with torch.cuda.stream(self.comm):
                        self.comm.wait_event(landed)
                        dist.all_gather_into_tensor(self.gathered[index], self.own[index], group=self.process_group)
                        whole = torch.cuda.Event()
                        whole.record(self.comm)
                with torch.cuda.stream(self.compute):
                    self.compute.wait_event(whole)
                    a_block = self.gathered[index].view(self.world * rows, self.k)
                    check(library().fk_gemm_bf16(a_block.data_ptr(), self.b.data_ptr(), self.c[index].data_ptr(),
                                                 self.world * rows, self.n, self.k, self.n, self.group,
                                                 self.compute.cuda_stream, self.status.data_ptr()))
                    computed = torch.cuda.Event()
                    computed.record(self.compute)
                with torch.cuda.stream(self.download):
                    self.download.wait_event(computed)
                    for slab in range(self.world):
                        first = slab * self.share + offset
                        c_out[first:first + rows].copy_(self.c[index][slab * rows:(slab + 1) * rows], non_blocking=True)
            # Every wait carries the launch deadline (FK_ERR_TIMEOUT instead of a hang).
            for stream in (self.upload, self.comm, self.compute, self.download):
                check(library().fk_wait_stream(stream.cuda_stream, library().fk_launch_budget_ms()))
            check(library().fk_status_check(self.status.data_ptr(), self.compute.cuda_stream))

    def bytes_per_step(self) -> tuple[int, int]:
        """(host-to-device, device-to-host) bytes one ``run`` copies on this rank."""
        return (self.share * self.k + self.n * self.k) * 2, self.m * self.n * 2
