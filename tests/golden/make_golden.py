"""Writes tests/golden/csr_cases.npz: small CSR SpMV / SpMM cases with expected outputs.

The reference publishes no golden vectors for this path and cannot run here, so the expected
outputs come from an implementation independent of both the oracle and the CUDA code:
scipy.sparse (float64 products accumulated in float64; for the float32 cases the inputs are
widened to float64 first). Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys

import numpy as np
import scipy.sparse as sp

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from tests.util import csr_from_lengths  # noqa: E402


def main():
    out = {}
    rng = np.random.default_rng(20240607)
    cases = [
        ("f32_b0", np.float32, 0, [3, 0, 5, 1, 0, 8, 2, 33, 0, 4], 40, 1.0, 0.0),
        ("f32_b1", np.float32, 1, [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 0, 0, 64], 70, -0.5, 2.0),
        ("f64_b0", np.float64, 0, [16] * 50 + [0, 0, 100], 128, 1.0, 0.5),
        ("f64_b1", np.float64, 1, [0, 0, 0, 7, 300, 1], 301, 2.25, -1.0),
    ]
    for name, dt, base, lengths, ncols, alpha, beta in cases:
        rp, col, val = csr_from_lengths(lengths, ncols, dt, seed=len(name) + base, base=base)
        x = rng.uniform(-1, 1, ncols).astype(dt)
        y0 = rng.uniform(-1, 1, len(lengths)).astype(dt)
        A = sp.csr_matrix((val.astype(np.float64), col.astype(np.int64) - base, rp.astype(np.int64) - base),
                          shape=(len(lengths), ncols))
        y = alpha * (A @ x.astype(np.float64)) + (beta * y0.astype(np.float64) if beta != 0 else 0.0)
        absA = abs(A)
        d = abs(alpha) * (absA @ np.abs(x.astype(np.float64))) + abs(beta) * np.abs(y0.astype(np.float64))
        n = 6
        B = rng.uniform(-1, 1, (ncols, n)).astype(dt)
        C0 = rng.uniform(-1, 1, (len(lengths), n)).astype(dt)
        Cx = alpha * (A @ B.astype(np.float64)) + (beta * C0.astype(np.float64) if beta != 0 else 0.0)
        dC = abs(alpha) * (absA @ np.abs(B.astype(np.float64))) + abs(beta) * np.abs(C0.astype(np.float64))
        for k, v in dict(row_ptr=rp, col=col, val=val, x=x, y0=y0, y=y, d=d, B=B, C0=C0, C=Cx, dC=dC,
                         meta=np.array([base, ncols, alpha, beta], np.float64)).items():
            out[f"{name}.{k}"] = v
    path = os.path.join(os.path.dirname(__file__), "csr_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_complex():
    """tests/golden/csr_cases_complex.npz: the same kind of cases with complex values and complex alpha, beta,
    plus the product with the conjugate-transposed matrix (what op(A) = A^H computes)."""
    out = {}
    rng = np.random.default_rng(20240608)

    def cplx(shape, dt):
        return (rng.uniform(-1, 1, shape) + 1j * rng.uniform(-1, 1, shape)).astype(dt)

    cases = [
        ("c32_b0", np.complex64, 0, [3, 0, 5, 1, 0, 8, 2, 33, 0, 4], 40, 1.0 - 0.5j, 0.0),
        ("c32_b1", np.complex64, 1, [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 0, 0, 64], 70, -0.5 + 2.0j, 2.0 - 1.0j),
        ("c64_b0", np.complex128, 0, [16] * 50 + [0, 0, 100], 128, 1.0, 0.5j),
        ("c64_b1", np.complex128, 1, [0, 0, 0, 7, 300, 1], 301, 2.25 + 0.75j, -1.0),
    ]
    for name, dt, base, lengths, ncols, alpha, beta in cases:
        rp, col, val = csr_from_lengths(lengths, ncols, dt, seed=len(name) + base, base=base)
        m = len(lengths)
        x, y0 = cplx(ncols, dt), cplx(m, dt)
        wide = np.complex128
        A = sp.csr_matrix((val.astype(wide), col.astype(np.int64) - base, rp.astype(np.int64) - base), shape=(m, ncols))
        y = alpha * (A @ x.astype(wide)) + beta * y0.astype(wide)
        absA = abs(A)
        d = abs(alpha) * (absA @ np.abs(x.astype(wide))) + abs(beta) * np.abs(y0.astype(wide))
        xh, yh0 = cplx(m, dt), cplx(ncols, dt)
        AH = A.conj().T.tocsr()
        yh = alpha * (AH @ xh.astype(wide)) + beta * yh0.astype(wide)
        dh = abs(alpha) * (abs(AH) @ np.abs(xh.astype(wide))) + abs(beta) * np.abs(yh0.astype(wide))
        n = 6
        B, C0 = cplx((ncols, n), dt), cplx((m, n), dt)
        Cx = alpha * (A @ B.astype(wide)) + beta * C0.astype(wide)
        dC = abs(alpha) * (absA @ np.abs(B.astype(wide))) + abs(beta) * np.abs(C0.astype(wide))
        for k, v in dict(row_ptr=rp, col=col, val=val, x=x, y0=y0, y=y, d=d, xh=xh, yh0=yh0, yh=yh, dh=dh, B=B, C0=C0,
                         C=Cx, dC=dC, meta=np.array([base, ncols, alpha, beta], np.complex128)).items():
            out[f"{name}.{k}"] = v
    path = os.path.join(os.path.dirname(__file__), "csr_cases_complex.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
    main_complex()
