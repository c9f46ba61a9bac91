"""Helpers shared by the tests: small CSR builders and the tolerance check."""

import numpy as np
import torch

TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12,
       np.dtype(np.complex64): 1e-5, np.dtype(np.complex128): 1e-12,
       torch.float32: 1e-5, torch.float64: 1e-12, torch.complex64: 1e-5, torch.complex128: 1e-12}


def csr_from_lengths(lengths, ncols, dtype, seed=0, base=0):
    """Random CSR with the given row lengths: sorted distinct columns, values in [-1, 1)."""
    rng = np.random.default_rng(seed)
    lengths = np.asarray(lengths, dtype=np.int64)
    row_ptr = np.zeros(lengths.size + 1, np.int64)
    np.cumsum(lengths, out=row_ptr[1:])
    col = np.empty(row_ptr[-1], np.int32)
    for r, L in enumerate(lengths):
        if L:
            col[row_ptr[r]:row_ptr[r + 1]] = np.sort(rng.choice(ncols, size=L, replace=False))
    val = rng.uniform(-1, 1, size=row_ptr[-1]).astype(dtype)
    if np.iscomplexobj(val):
        val = (val + 1j * rng.uniform(-1, 1, size=row_ptr[-1])).astype(dtype)
    return (row_ptr + base).astype(np.int32), col + np.int32(base), val


def assert_close(got, ref, d, tol, what=""):
    """|got - ref| <= tol * d elementwise (d = |alpha| sum |a||x| + |beta||y0|)."""
    got = np.asarray(got, dtype=np.complex128 if np.iscomplexobj(ref) or np.iscomplexobj(got) else np.float64)
    err = np.abs(got - ref)
    bad = ~(err <= tol * d + 1e-300)
    if bad.any():
        i = np.flatnonzero(bad.ravel())[0]
        ratio = (err.ravel() / np.maximum(d.ravel(), 1e-300))
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements outside {tol:g}*d; first at {i}: "
                             f"got {got.ravel()[i]!r} ref {ref.ravel()[i]!r} d {d.ravel()[i]!r}; max err/d {ratio.max():g}")


ADVERSARIAL_LENGTHS = {
    "one_row": [7],
    "single_empty_row": [0],
    "all_empty": [0] * 37,
    "empty_start_mid_end": [0, 0, 5, 0, 0, 0, 3, 9, 0, 0],
    "lengths_1_to_33": list(range(1, 34)),
    "lengths_63_65": [63, 64, 65] * 5,
    "lengths_255_257": [255, 256, 257, 1, 0, 256],
    "one_row_all_nnz": [0, 0, 20000, 0],
    "long_then_short": [9000] + [1] * 3000,
    "tile_straddle": [2047, 2049, 4095, 4097, 1, 2048, 4096],
    "many_short": [1, 2, 0, 3] * 4000,
    "uniform_27": [27] * 3000,
    "mostly_empty": [0] * 5000 + [3] + [0] * 3000 + [1] * 10,  # whole tiles of row ends only
    "mixed_medium_long": ([2] * 150 + [300] + [5] * 100 + [1500] + [9] * 50 + [40]) * 6 + [7000],
}
