"""CPU tests of the oracle: golden fixtures, scipy cross-check, analytic answers, partition rules."""

import os

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from mcsparse_b200 import workloads
from oracle import oracle
from tests.util import ADVERSARIAL_LENGTHS, TOL, assert_close, csr_from_lengths

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "csr_cases.npz"))
CASES = sorted({k.split(".")[0] for k in GOLDEN.files})


def g(case, key):
    return GOLDEN[f"{case}.{key}"]


@pytest.mark.parametrize("case", CASES)
def test_oracle_spmv_matches_golden(case):
    base, _, alpha, beta = g(case, "meta")
    y, d = oracle.spmv(g(case, "row_ptr"), g(case, "col"), g(case, "val"), g(case, "x"), alpha, beta, g(case, "y0"),
                       base=int(base))
    # The oracle accumulates wider than scipy's float64, so they agree to float64 rounding.
    assert_close(y, g(case, "y"), g(case, "d"), 1e-14, case)
    np.testing.assert_allclose(d, g(case, "d"), rtol=1e-13)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("order", [1, 2])
def test_oracle_spmm_matches_golden(case, order):
    base, ncols, alpha, beta = g(case, "meta")
    B, C0 = g(case, "B"), g(case, "C0")
    n = B.shape[1]
    if order == 2:
        Bf, ldb, Cf, ldc = B, n, C0, n
    else:
        Bf, ldb, Cf, ldc = np.asfortranarray(B).T, B.shape[0], np.asfortranarray(C0).T, C0.shape[0]
    out, d = oracle.spmm(g(case, "row_ptr"), g(case, "col"), g(case, "val"), np.ascontiguousarray(Bf), ldb, order, n,
                         alpha, beta, np.ascontiguousarray(Cf), ldc, order, base=int(base))
    assert_close(out, g(case, "C"), g(case, "dC"), 1e-14, case)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_oracle_vs_scipy(name, dtype):
    lengths = ADVERSARIAL_LENGTHS[name]
    ncols = max(max(lengths), 1) + 13
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=3)
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, ncols).astype(dtype)
    y0 = rng.uniform(-1, 1, len(lengths)).astype(dtype)
    y, d = oracle.spmv(rp, col, val, x, 0.75, -1.5, y0)
    A = sp.csr_matrix((val.astype(np.float64), col, rp), shape=(len(lengths), ncols))
    ref = 0.75 * (A @ x.astype(np.float64)) - 1.5 * y0.astype(np.float64)
    assert_close(y, ref, d, 1e-14, name)


def test_oracle_beta_zero_ignores_y():
    rp, col, val = csr_from_lengths([2, 0, 3], 5, np.float64)
    x = np.ones(5)
    y_nan = np.full(3, np.nan)
    y, _ = oracle.spmv(rp, col, val, x, 1.0, 0.0, y_nan)
    assert np.isfinite(y).all()


@pytest.mark.parametrize("name,factor", [("C1", 256), ("C5", 4096)])
def test_stencil_times_ones_is_row_sum(name, factor):
    """Interior rows of a Laplacian-type stencil sum to zero; boundary rows to the number of
    missing neighbours."""
    cfg = workloads.scaled(name, factor)
    w = workloads.generate(cfg, "cpu")
    ones = np.ones(w.cols, dtype=w.val.numpy().dtype)
    y, _ = oracle.spmv(w.row_ptr, w.col, w.val, ones, 1.0, 0.0)
    full = 5 if name == "C1" else 27
    lengths = np.diff(w.row_ptr.numpy())
    np.testing.assert_array_equal(y, (full - lengths).astype(np.float64))
    assert lengths.max() == full and lengths.min() == (3 if name == "C1" else 8)


def test_alpha_zero_and_identity():
    m = 50
    rp = np.arange(m + 1, dtype=np.int32)
    col = np.arange(m, dtype=np.int32)
    val = np.full(m, 3.0)
    x = np.linspace(-1, 1, m)
    y0 = np.linspace(2, 3, m)
    y, _ = oracle.spmv(rp, col, val, x, 0.0, 1.0, y0)
    np.testing.assert_array_equal(y, y0)
    y, _ = oracle.spmv(rp, col, val, x, 1.0, 0.0, y0)
    np.testing.assert_array_equal(y, 3.0 * x)


def _partition_reference(row_ptr, nnz, T, base):
    """Slow restatement: walk the merge list item by item."""
    m = len(row_ptr) - 1
    ends = [int(row_ptr[r + 1]) - base for r in range(m)]
    starts, r, k = [], 0, 0
    items = m + nnz
    for d in range(items + 1):
        if d % T == 0:
            starts.append((r, k))
        if d == items:
            break
        if r < m and ends[r] <= k:
            r += 1
        else:
            k += 1
    if items % T != 0:
        starts.append((m, nnz))
    return np.asarray(starts, np.int32)


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_merge_path_partition_rules(name, base):
    lengths = ADVERSARIAL_LENGTHS[name]
    rp = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32) + base
    nnz, m = int(rp[-1] - base), len(lengths)
    for T in (7, 64, 2048, 4096):
        part = oracle.merge_path_partition(rp, nnz, T, base)
        ntiles = (m + nnz + T - 1) // T
        assert part.shape == (ntiles + 1, 2)
        assert (part[0] == 0).all() and part[-1, 0] == m and part[-1, 1] == nnz
        assert (np.diff(part[:, 0]) >= 0).all() and (np.diff(part[:, 1]) >= 0).all()
        per_tile = np.diff(part.sum(axis=1))
        assert (per_tile[:-1] == T).all() and (0 < per_tile[-1] <= T if ntiles else True)
        if m + nnz <= 30000:
            np.testing.assert_array_equal(part, _partition_reference(rp, nnz, T, base))


def test_shard_bounds_and_local_offsets():
    lengths = ADVERSARIAL_LENGTHS["long_then_short"] + ADVERSARIAL_LENGTHS["lengths_1_to_33"]
    for base in (0, 1):
        rp = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32) + base
        nnz = int(rp[-1] - base)
        for G in (1, 2, 3, 8):
            b = oracle.shard_row_bounds(rp, nnz, G, base)
            assert b[0] == 0 and b[-1] == len(lengths) and (np.diff(b) >= 0).all()
            for g_ in range(1, G):
                target = (g_ * nnz) // G
                assert rp[b[g_]] - base >= target and (b[g_] == 0 or rp[b[g_] - 1] - base < target)
            for g_ in range(G):
                loc = oracle.shard_local_row_offsets(rp, int(b[g_]), int(b[g_ + 1] - b[g_]), base)
                assert loc[0] == base and loc[-1] - base == rp[b[g_ + 1]] - rp[b[g_]]


def test_baseline_matches_oracle():
    for dtype in (np.float32, np.float64):
        rp, col, val = csr_from_lengths(ADVERSARIAL_LENGTHS["many_short"], 700, dtype, seed=9)
        rng = np.random.default_rng(1)
        x = rng.uniform(-1, 1, 700).astype(dtype)
        y = rng.uniform(-1, 1, rp.size - 1).astype(dtype)
        ref, d = oracle.spmv(rp, col, val, x, 1.5, 0.25, y)
        oracle.baseline_spmv(rp, col, val, x, 1.5, 0.25, y)
        assert_close(y, ref, d, TOL[np.dtype(dtype)], "baseline spmv")
        n = 8
        B = rng.uniform(-1, 1, (700, n)).astype(dtype)
        Cm = rng.uniform(-1, 1, (rp.size - 1, n)).astype(dtype)
        refC, dC = oracle.spmm(rp, col, val, B, n, 2, n, 1.5, 0.25, Cm.copy(), n, 2)
        oracle.baseline_spmm(rp, col, val, B, n, 1.5, 0.25, Cm)
        assert_close(Cm, refC, dC, TOL[np.dtype(dtype)], "baseline spmm")


def test_csr_validate():
    rp, col, val = csr_from_lengths([2, 0, 3], 5, np.float32)
    assert oracle.csr_validate(3, 5, rp, col) == 0
    bad = rp.copy(); bad[0] = 1
    assert oracle.csr_validate(3, 5, bad, col) == 1
    bad = rp.copy(); bad[1], bad[2] = 3, 2
    assert oracle.csr_validate(3, 5, bad, col) == 2
    badc = col.copy(); badc[0] = 5
    assert oracle.csr_validate(3, 5, rp, badc) == 4


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("name", sorted(ADVERSARIAL_LENGTHS))
def test_coo_row_offsets(name, base):
    lengths = np.asarray(ADVERSARIAL_LENGTHS[name])
    rp = (np.concatenate([[0], np.cumsum(lengths)]) + base).astype(np.int32)
    coo_rows = (np.repeat(np.arange(lengths.size), lengths) + base).astype(np.int32)
    np.testing.assert_array_equal(oracle.coo_row_offsets(coo_rows, lengths.size, base), rp)


def test_csr_transpose_matches_scipy():
    sp = pytest.importorskip("scipy.sparse")
    from tests.util import ADVERSARIAL_LENGTHS, csr_from_lengths

    for name in ("lengths_1_to_33", "empty_start_mid_end", "long_then_short", "all_empty", "one_row"):
        for base in (0, 1):
            lengths = ADVERSARIAL_LENGTHS[name]
            n = max(max(lengths), 1) + 3
            rp, col, val = csr_from_lengths(lengths, n, np.float64, seed=5, base=base)
            t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, n, base)
            ref = sp.csr_matrix((val, col - base, rp - base), shape=(len(lengths), n)).T.tocsr()
            ref.sort_indices()
            np.testing.assert_array_equal(t_ptr, ref.indptr)
            np.testing.assert_array_equal(t_idx, ref.indices)
            np.testing.assert_array_equal(val[perm], ref.data)
            assert sorted(perm.tolist()) == list(range(col.size))


GOLDEN_C = np.load(os.path.join(os.path.dirname(__file__), "golden", "csr_cases_complex.npz"))
CASES_C = sorted({k.split(".")[0] for k in GOLDEN_C.files})


@pytest.mark.parametrize("case", CASES_C)
def test_complex_oracle_matches_golden(case):
    gc = lambda key: GOLDEN_C[f"{case}.{key}"]
    base, _, alpha, beta = gc("meta")
    base = int(base.real)
    y, d = oracle.spmv(gc("row_ptr"), gc("col"), gc("val"), gc("x"), alpha, beta, gc("y0"), base=base)
    assert_close(y, gc("y"), gc("d"), 1e-14, case)
    np.testing.assert_allclose(d, gc("d"), rtol=1e-13)
    # conjugate-transposed product: transpose on the CPU, then multiply with conj(values)
    n = gc("x").size
    t_ptr, t_idx, perm = oracle.csr_transpose(gc("row_ptr"), gc("col"), n, base)
    yh, dh = oracle.spmv(t_ptr, t_idx, gc("val")[perm], gc("xh"), alpha, beta, gc("yh0"), conj=True)
    assert_close(yh, gc("yh"), gc("dh"), 1e-14, case + " A^H")
    B, C0 = gc("B"), gc("C0")
    out, dC = oracle.spmm(gc("row_ptr"), gc("col"), gc("val"), B, B.shape[1], 2, B.shape[1], alpha, beta, C0,
                          B.shape[1], 2, base=base)
    assert_close(out, gc("C"), gc("dC"), 1e-14, case + " SpMM")


def _random_lengths(rng, rows):
    kind = rng.integers(0, 4)
    if kind == 0:
        return rng.integers(0, 4, rows)
    if kind == 1:
        return rng.poisson(6.0, rows)
    if kind == 2:
        L = rng.integers(0, 3, rows)
        L[rng.integers(0, rows, max(1, rows // 50))] = rng.integers(100, 700)
        return L
    return np.where(rng.random(rows) < 0.9, 0, rng.integers(1, 40, rows))


@pytest.mark.parametrize("seed", range(12))
def test_partition_and_transposition_invariants(seed):
    """Properties that hold for any matrix: the merge-path partition tiles the (rows + nnz) merge list without
    gaps, every tile start is a valid merge point; transposing twice gives the matrix back; the permutation of a
    transposition is a permutation."""
    rng = np.random.default_rng(1000 + seed)
    rows, base = int(rng.integers(1, 900)), int(rng.integers(0, 2))
    lengths = _random_lengths(rng, rows)
    ncols = int(max(lengths.max(), 1) + rng.integers(0, 50))
    rp, col, val = csr_from_lengths(lengths, ncols, np.float64, seed=seed, base=base)
    nnz = col.size
    for items in (64, 1024, 2048):
        part = oracle.merge_path_partition(rp, nnz, items, base)
        assert (part[0] == (0, 0)).all() and (part[-1] == (rows, nnz)).all()
        assert (np.diff(part[:, 0]) >= 0).all() and (np.diff(part[:, 1]) >= 0).all()
        covered = np.diff(part.sum(axis=1))
        assert (covered[:-1] == items).all() and 0 < covered[-1] <= items if covered.size else True
        r, k = part[:, 0], part[:, 1]
        ends = rp[1:].astype(np.int64) - base
        # at a tile start (r, k): every earlier row has ended by nonzero k, and row r has not ended before it
        assert all(r[i] == 0 or ends[r[i] - 1] <= k[i] for i in range(len(r)))
        assert all(r[i] == rows or ends[r[i]] > k[i] - 1 or k[i] == 0 for i in range(len(r)))
    t_ptr, t_idx, perm = oracle.csr_transpose(rp, col, ncols, base)
    assert sorted(perm.tolist()) == list(range(nnz))
    b_ptr, b_idx, perm2 = oracle.csr_transpose(t_ptr, t_idx, rows, 0)
    np.testing.assert_array_equal(b_ptr, rp.astype(np.int64) - base)
    np.testing.assert_array_equal(b_idx, col.astype(np.int64) - base)
    np.testing.assert_array_equal(val[perm][perm2], val)
