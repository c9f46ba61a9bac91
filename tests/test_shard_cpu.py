"""CPU (gloo, world size 2 and 3) tests of the multi-GPU host logic: nnz-balanced row blocks,
per-rank generation of a block, and the ragged assembly of y on every rank. The per-block SpMV is
done by the CPU oracle here; on GPUs the same host code drives the CUDA kernels."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mcsparse_b200 import sharding, workloads
from oracle import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, factor, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = workloads.scaled(name, factor)
        lengths = workloads.row_lengths(cfg, "cpu")
        bounds, nnz = sharding.shard_bounds(lengths, world)
        row_ptr = np.concatenate([[0], np.cumsum(lengths.numpy())]).astype(np.int32)
        assert bounds == oracle.shard_row_bounds(row_ptr, nnz, world).tolist()
        r0, r1 = bounds[rank], bounds[rank + 1]
        w = workloads.generate(cfg, "cpu", row_range=(r0, r1))
        np.testing.assert_array_equal(w.row_ptr.numpy(), oracle.shard_local_row_offsets(row_ptr, r0, r1 - r0))
        y_full = torch.zeros(cfg.rows, dtype=torch.float64)
        y_local, _ = oracle.spmv(w.row_ptr, w.col, w.val, w.x, cfg.alpha, cfg.beta, w.y0)
        parts = [y_full[bounds[g]:bounds[g + 1]] for g in range(world)]
        sharding.all_gather_ragged(parts, torch.from_numpy(y_local))
        whole = workloads.generate(cfg, "cpu")
        ref, _ = oracle.spmv(whole.row_ptr, whole.col, whole.val, whole.x, cfg.alpha, cfg.beta, whole.y0)
        np.testing.assert_array_equal(y_full.numpy(), ref)  # same oracle arithmetic row by row: bit-identical
        # nnz balance: no block is more than one row's worth above the ideal share
        share = [int(row_ptr[bounds[g + 1]] - row_ptr[bounds[g]]) for g in range(world)]
        assert sum(share) == nnz and max(share) <= nnz // world + int(lengths.max()) + 1
        out[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,name,factor", [(2, "C3", 2048), (2, "C5", 4096), (3, "C2", 4096)])
def test_sharded_assembly_matches_single_process(world, name, factor):
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, name, factor, out), nprocs=world, join=True)
        assert sorted(out.keys()) == list(range(world))


def test_shard_bounds_edge_cases():
    lengths = torch.tensor([0, 0, 5, 0, 0], dtype=torch.int64)
    b, nnz = sharding.shard_bounds(lengths, 4)
    assert nnz == 5 and b[0] == 0 and b[-1] == 5 and b == sorted(b)
    rp = np.array([0, 0, 0, 5, 5, 5], np.int32)
    assert b == oracle.shard_row_bounds(rp, 5, 4).tolist()
    b, nnz = sharding.shard_bounds(torch.zeros(7, dtype=torch.int64), 2)
    assert nnz == 0 and b == [0, 0, 7]
    assert b == oracle.shard_row_bounds(np.zeros(8, np.int32), 0, 2).tolist()


def test_destination_order(monkeypatch):
    """Push destinations of a rank: every other rank once; rank order by default, rotated on request."""
    from mcsparse_b200 import sharding

    monkeypatch.delenv("MCSPARSE_B200_PEER_ORDER", raising=False)
    assert sharding.destination_order(2, 4) == [0, 1, 3]
    assert sharding.destination_order(0, 1) == []
    monkeypatch.setenv("MCSPARSE_B200_PEER_ORDER", "rotated")
    assert sharding.destination_order(2, 4) == [3, 0, 1]
    assert sharding.destination_order(7, 8) == [0, 1, 2, 3, 4, 5, 6]
    for world in (2, 3, 8):
        for rank in range(world):
            for mode in ("ascending", "rotated"):
                assert sorted(sharding.destination_order(rank, world, mode)) == [g for g in range(world) if g != rank]
