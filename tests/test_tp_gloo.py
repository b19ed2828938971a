"""Tensor-parallel plumbing on the CPU: two gloo ranks, the oracle standing in for the CUDA
forward of each shard.  Checks the shard algebra end to end (column-parallel concatenation,
row-parallel all-reduce) against the unsharded oracle, and the host-side error paths."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cobalt_b200 import tp
from oracle import cobalt_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_linear(keep, q, sc, zr):
    W = O.dequantize(q, sc, zr, keep).to(torch.bfloat16)

    def f(x, out_fp32=False):
        if out_fp32:                                   # what cobalt_linear_f32 returns: unrounded fp32 sums
            return torch.matmul(x.float(), W.float().t())
        return torch.matmul(x, W.t())
    return f


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        raw = O.synth_raw(64, 1024, 0.5, 4, seed=5)
        keep, q, sc, zr = raw["keep"], raw["q"], raw["scale"], raw["zero"]
        x = O.seeded_activation(4, 1024, 6)
        full = _oracle_linear(keep, q, sc, zr)(x)
        # column-parallel: shards of the output rows, gathered
        col = tp.ColumnParallelLinear(_oracle_linear(*tp.shard_raw("column", keep, q, sc, zr, rank, world)), gather_output=True)
        y_col = col(x)
        # row-parallel: shards of the input columns, all-reduced
        c0, c1 = tp.shard_bounds(1024, rank, world, 128)
        row = tp.RowParallelLinear(_oracle_linear(*tp.shard_raw("row", keep, q, sc, zr, rank, world)))
        y_row = row(x[:, c0:c1].contiguous())
        rel = float((y_row.double() - full.double()).norm() / full.double().norm())
        out[rank] = (bool(torch.equal(y_col, full)), rel)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_matches_unsharded():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for rank in range(world):
        col_equal, rel = out[rank]
        assert col_equal, "column-parallel concatenation differs from the unsharded result"
        assert rel <= 1e-3, f"row-parallel all-reduce rel-L2 {rel}"


def test_shard_rules_and_errors():
    assert tp.kind_of("model.layers.3.self_attn.k_proj") == "column"
    assert tp.kind_of("mlp.down_proj") == "row"
    with pytest.raises(ValueError):
        tp.kind_of("lm_head")
    assert tp.shard_bounds(4096, 3, 8, 128) == (1536, 2048)
    with pytest.raises(ValueError):
        tp.shard_bounds(5376, 0, 8, 128)          # 5376 / 8 = 672 is not a multiple of 128
    raw = O.synth_raw(32, 256, 0.5, 4, seed=1)
    with pytest.raises(ValueError):
        tp.shard_raw("row", raw["keep"], raw["q"], raw["scale"], raw["zero"], 0, 4)   # 64-column shards
    with pytest.raises(ValueError):
        tp.shard_raw("diagonal", raw["keep"], raw["q"], raw["scale"], raw["zero"], 0, 2)
