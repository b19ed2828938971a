"""Tensor-parallel wrappers for the compressed linears (one process per GPU, ``torch.distributed``).

The reference has no distributed code; the sharding follows the usual Megatron split of a
decoder block, which the compressed format supports without re-quantising:

* column-parallel (q, k, v, gate, up): each rank holds a contiguous block of OUTPUT rows
  (whole rows of the tile image), the input is replicated, the output stays sharded;
* row-parallel (o, down): each rank holds a contiguous block of INPUT columns, cut on
  128-column group boundaries so that no scale/zero group straddles ranks; the partial
  outputs are summed with ONE all-reduce per layer (fp32 on the wire, rounded to bf16 once).

Shards are packed per rank from RAW slices (``format.slice_rows`` / ``format.slice_cols``).

The all-reduce is NCCL by default.  For decode-sized outputs ``PeerReducer`` replaces it with one small
kernel per rank that reads the peers' fp32 partials over NVLink (plain peer loads from a symmetric buffer,
no multicast) and adds them in rank order: the GEMV writes its partial into the buffer, the kernel
publishes/awaits a flag per peer and sums.  NCCL's latency for a 16 KB message is several times that.
"""
from __future__ import annotations

from typing import Callable, Optional

import ctypes

import torch
import torch.distributed as dist
import torch.nn as nn

from .format import GROUP, slice_cols, slice_rows

COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
ROW_PARALLEL = ("o_proj", "down_proj")


def shard_bounds(total: int, rank: int, world: int, align: int = 1):
    """[begin, end) of rank's share of `total`, which must split evenly into `align`-sized units."""
    if total % (world * align):
        raise ValueError(f"{total} does not split into {world} shards of a multiple of {align}")
    per = total // world
    return rank * per, (rank + 1) * per


def shard_raw(kind: str, keep, q, scale, zero, rank: int, world: int):
    """RAW tensors of rank's shard.  ``kind`` is 'column' (split output rows) or 'row' (split input columns)."""
    K, N = keep.shape
    if kind == "column":
        r0, r1 = shard_bounds(K, rank, world, 1)
        return slice_rows(keep, q, scale, zero, r0, r1)
    if kind == "row":
        c0, c1 = shard_bounds(N, rank, world, GROUP)
        return slice_cols(keep, q, scale, zero, c0, c1)
    raise ValueError(f"unknown shard kind {kind!r}")


def kind_of(proj_name: str) -> str:
    leaf = proj_name.split(".")[-1]
    if leaf in COLUMN_PARALLEL:
        return "column"
    if leaf in ROW_PARALLEL:
        return "row"
    raise ValueError(f"no tensor-parallel rule for {proj_name!r}")


class ColumnParallelLinear(nn.Module):
    """y_local = local(x): output rows of this rank only.  ``gather_output`` concatenates over ranks."""

    def __init__(self, local: Callable, group: Optional[dist.ProcessGroup] = None, gather_output: bool = False):
        super().__init__()
        self.local, self.group, self.gather_output = local, group, gather_output

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        if not self.gather_output:
            return y
        world = dist.get_world_size(self.group)
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


class PeerReducer:
    """Sum of fp32 partials over peer memory (``cobalt_allreduce_peer``).  One symmetric buffer per rank: a
    staging area the local GEMV writes to, two data slots of ``world`` rows of ``max_floats`` fp32 (every rank pushes
    its partial into its row of every rank's slot; the kernel alternates the slots by a device-side epoch counter,
    so captured graphs and eager calls can be mixed), and a flag block.  All ranks
    must make the same sequence of calls.  Needs ``torch.distributed._symmetric_memory`` (NVLink peer
    mappings); construction raises if that is unavailable, and the caller keeps using NCCL."""

    FLAG_BYTES = 256

    def __init__(self, max_floats: int, device, group: Optional[dist.ProcessGroup] = None):
        import ctypes
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        self._lib = _lib.load()
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.stride = (int(max_floats) * 4 + 255) // 256 * 256
        self.flags_off = (1 + 2 * self.world) * self.stride      # staging + two slots of `world` rows
        total = self.flags_off + self.FLAG_BYTES
        self.buf = symm.empty(total // 4, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._ptrs = (ctypes.c_uint64 * self.world)(*ptrs)
        self.slots = _lib.CobaltPeerSlots(ctypes.cast(self._ptrs, ctypes.c_void_p), self.rank, self.world, self.stride, self.flags_off)
        self.status = torch.zeros(64, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)                     # every buffer is zeroed before anyone publishes a flag

    def slot_view(self, n: int) -> torch.Tensor:
        """fp32 view of the staging area: the local GEMV writes its partial here before ``reduce``."""
        if n * 4 > self.stride:
            raise ValueError("partial larger than the slot")
        return self.buf[:n]

    def reduce(self, n: int, out: torch.Tensor) -> torch.Tensor:
        """Sum the ranks' partials into ``out`` (bf16 or fp32, ``n`` elements)."""
        from . import _lib
        if out.numel() != n or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("`out` must be a contiguous bf16 or fp32 tensor of n elements")
        rc = self._lib.cobalt_allreduce_peer(self._ptrs, self.rank, self.world, n, self.stride, self.flags_off,
                                             out.data_ptr(), 1 if out.dtype == torch.float32 else 0, self.status.data_ptr(),
                                             torch.cuda.current_stream(out.device).cuda_stream)
        _lib.check("cobalt_allreduce_peer", rc)
        return out

    def sum_pushed(self, n: int, out: torch.Tensor) -> torch.Tensor:
        """Sum over ranks of the partials that a pushing GEMV (``FusedProjections.staged(..., push=self)``) left in this
        rank's buffer, into ``out`` (bf16 or fp32, ``n`` elements): the summing half of ``reduce`` as its own kernel."""
        from . import _lib
        if out.numel() != n or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("`out` must be a contiguous bf16 or fp32 tensor of n elements")
        rc = self._lib.cobalt_peer_sum(ctypes.byref(self.slots), n, out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                                       self.status.data_ptr(), torch.cuda.current_stream(out.device).cuda_stream)
        _lib.check("cobalt_peer_sum", rc)
        return out

    def device_status(self) -> int:
        return int(self.status[0].item())


class RowParallelLinear(nn.Module):
    """y = sum over ranks of local(x_local): one all-reduce of the [M, out_features] partial output (NCCL, or the
    peer-memory kernel when a ``PeerReducer`` is given and the output fits its slot)."""

    def __init__(self, local: Callable, group: Optional[dist.ProcessGroup] = None, reducer: Optional["PeerReducer"] = None):
        super().__init__()
        self.local, self.group, self.reducer = local, group, reducer

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        # fp32 partial sums (no rounding yet): summing bf16-rounded partials would add one rounding error
        # per rank and miss the 1e-3 rel-L2 bar already at two ranks
        if self.reducer is not None:
            lead = x_local.shape[:-1]
            M = x_local.numel() // x_local.shape[-1]
            K = getattr(self.local, "out_features", None)
            if K is not None and M * K * 4 <= self.reducer.stride:
                self.local(x_local, out_fp32=True, out=self.reducer.slot_view(M * K))
                y = torch.empty(M * K, dtype=x_local.dtype, device=x_local.device)
                return self.reducer.reduce(M * K, y).view(*lead, K)
        acc = self.local(x_local, out_fp32=True)
        if acc.dtype != torch.float32:
            raise TypeError("the local layer of a row-parallel linear must return fp32 partial sums")
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        return acc.to(x_local.dtype)
