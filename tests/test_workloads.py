"""CPU tests of the synthetic workload generators."""

import numpy as np
import pytest
import torch

from mcsparse_b200 import workloads
from oracle import oracle

SMALL = [("C1", 1024), ("C2", 2048), ("C3", 8192), ("C4", 512), ("C5", 2048)]


@pytest.mark.parametrize("name,factor", SMALL)
def test_structure_is_valid_sorted_distinct(name, factor):
    cfg = workloads.scaled(name, factor)
    for base in (0, 1):
        w = workloads.generate(cfg, "cpu", base=base)
        assert oracle.csr_validate(w.rows, w.cols, w.row_ptr, w.col, base) == 0
        rp, col = w.row_ptr.numpy().astype(np.int64) - base, w.col.numpy()
        inner = np.ones(col.size, bool)
        inner[rp[:-1][rp[:-1] < col.size]] = False
        assert (np.diff(col)[inner[1:]] > 0).all(), "columns must ascend strictly inside a row"
        assert w.val.dtype == cfg.dtype and w.nnz == col.size


@pytest.mark.parametrize("name,factor", SMALL)
def test_row_block_equals_slice_of_whole(name, factor):
    cfg = workloads.scaled(name, factor)
    w = workloads.generate(cfg, "cpu")
    r0, r1 = w.rows // 3, (2 * w.rows) // 3 + 1
    b = workloads.generate(cfg, "cpu", row_range=(r0, r1))
    a0, a1 = int(w.row_ptr[r0]), int(w.row_ptr[r1])
    assert torch.equal(w.col[a0:a1], b.col) and torch.equal(w.val[a0:a1], b.val)
    assert torch.equal(w.row_ptr[r0:r1 + 1] - w.row_ptr[r0], b.row_ptr)
    assert torch.equal(workloads.row_lengths(cfg, "cpu", r0, r1), torch.diff(b.row_ptr.long()))
    if cfg.op == "spmv":
        assert torch.equal(w.y0[r0:r1], b.y0) and torch.equal(w.x, b.x)


def test_deterministic_and_seeded():
    cfg = workloads.scaled("C2", 4096)
    a, b = workloads.generate(cfg, "cpu"), workloads.generate(cfg, "cpu")
    assert torch.equal(a.col, b.col) and torch.equal(a.val, b.val) and torch.equal(a.x, b.x)
    cfg2 = workloads.scaled("C2", 4096)
    cfg2.seed += 1
    c = workloads.generate(cfg2, "cpu")
    assert not torch.equal(a.val[:100], c.val[:100])


def test_row_length_laws():
    c2 = workloads.scaled("C2", 64)
    L = workloads.row_lengths(c2, "cpu").double()
    assert L.min() >= 1 and abs(L.mean() - 16.0) < 0.2 and abs(L.var() - 16.0) < 1.0
    c4 = workloads.scaled("C4", 16)
    L = workloads.row_lengths(c4, "cpu").double()
    assert abs(L.mean() - 32.0) < 0.3
    c3 = workloads.scaled("C3", 64)
    L = workloads.row_lengths(c3, "cpu")
    assert L.min() >= 1 and L.max() <= c3.max_len
    assert abs(L.sum().item() / c3.nnz_target - 1.0) < 0.2  # rounding and clamping move the total a little
    assert (L == 1).float().mean() < 0.9 and L.max() > 100  # heavy tail present


def test_full_size_shapes_without_generating():
    assert workloads.CONFIGS["C1"].rows == 1048576
    assert workloads.CONFIGS["C5"].rows == 16777216
    L = workloads.row_lengths(workloads.CONFIGS["C1"], "cpu")
    assert int(L.sum()) == 5238784
    c5 = workloads.scaled("C5", 512)  # 32^3
    assert int(workloads.row_lengths(c5, "cpu").sum()) == (3 * c5.grid - 2) ** 3


def test_algorithmic_bytes_formula():
    # C1: nnz * 8 + (m + 1) * 4 + x + y
    assert workloads.algorithmic_bytes(1048576, 1048576, 5238784, 4, 0.0) == 54493188
    b = workloads.algorithmic_bytes(10, 10, 100, 8, 0.5)
    assert b == 100 * 12 + 11 * 4 + 10 * 8 + 2 * 10 * 8
    assert workloads.algorithmic_bytes(10, 20, 100, 4, 0.0, dense_cols=64) == 100 * 8 + 11 * 4 + 20 * 64 * 4 + 10 * 64 * 4
