"""Tensor-parallel wrappers for the compressed linears (one process per GPU, ``torch.distributed``).

The reference has no distributed code; the sharding follows the usual Megatron split of a
decoder block, which the compressed format supports without re-quantising:

* column-parallel (q, k, v, gate, up): each rank holds a contiguous block of OUTPUT rows
  (whole rows of the tile image), the input is replicated, the output stays sharded;
* row-parallel (o, down): each rank holds a contiguous block of INPUT columns, cut on
  128-column group boundaries so that no scale/zero group straddles ranks; the partial
  outputs are summed with ONE all-reduce per layer (fp32 on the wire, rounded to bf16 once).

Shards are packed per rank from RAW slices (``format.slice_rows`` / ``format.slice_cols``).
No kernel reads another GPU's memory: NCCL leaves the reduced tensor in local HBM.
"""
from __future__ import annotations

from typing import Callable, Optional

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


class RowParallelLinear(nn.Module):
    """y = sum over ranks of local(x_local): one all-reduce of the [M, out_features] partial output."""

    def __init__(self, local: Callable, group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.local, self.group = local, group

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        # fp32 partial sums (no rounding yet): summing bf16-rounded partials would add one rounding error
        # per rank and miss the 1e-3 rel-L2 bar already at two ranks
        acc = self.local(x_local, out_fp32=True)
        if acc.dtype != torch.float32:
            raise TypeError("the local layer of a row-parallel linear must return fp32 partial sums")
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        return acc.to(x_local.dtype)
