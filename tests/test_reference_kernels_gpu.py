"""Pins the CPU oracle against the mcSparse reference's own CSR device kernels.

oracle/_ref/libmcsp_refkernels.so holds mcspSpmvCsrVectorKernel and mcspBatchedSpmmCsrNnKernel
compiled from the reference source tree (oracle/Makefile, target `ref`) and launched with the
reference's launch shapes. It is built where that tree is mounted and travels as a built file;
where it is absent these tests skip. The reference sums in a different order than the oracle,
so the comparison uses the path's stated tolerance.
"""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import ADVERSARIAL_LENGTHS, TOL, assert_close, csr_from_lengths

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(os.path.dirname(oracle.__file__), "_ref", "libmcsp_refkernels.so")


@pytest.fixture(scope="module")
def ref(device):
    if not os.path.exists(REF_LIB):
        pytest.skip("reference kernels not built (needs the mcSparse source tree at build time)")
    return C.CDLL(REF_LIB)


def P(t):
    return C.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("name", ["lengths_1_to_33", "empty_start_mid_end", "lengths_255_257", "long_then_short",
                                  "uniform_27"])
def test_oracle_spmv_matches_reference_kernel(ref, device, name, dtype, base):
    lengths = ADVERSARIAL_LENGTHS[name]
    ncols = max(max(lengths), 1) + 9
    rp, col, val = csr_from_lengths(lengths, ncols, dtype, seed=21, base=base)
    rng = np.random.default_rng(12)
    x, y0 = rng.uniform(-1, 1, ncols).astype(dtype), rng.uniform(-1, 1, len(lengths)).astype(dtype)
    alpha, beta = 1.5, -0.5
    want, d = oracle.spmv(rp, col, val, x, alpha, beta, y0, base=base)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, x, y0.copy())]
    ct = C.c_float if dtype == np.float32 else C.c_double
    fn = ref.ref_csr_spmv_f32 if dtype == np.float32 else ref.ref_csr_spmv_f64
    rc = fn(len(lengths), ct(alpha), ct(beta), P(t[0]), P(t[1]), P(t[2]), P(t[3]), P(t[4]), base)
    assert rc == 0
    assert_close(t[4].cpu().numpy(), want, d, TOL[np.dtype(dtype)], f"reference kernel vs oracle, {name}")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("order_c", [1, 2])
def test_oracle_spmm_matches_reference_kernel(ref, device, dtype, order_c):
    lengths = ADVERSARIAL_LENGTHS["lengths_1_to_33"] + [0, 0, 70]
    k, n, base = 80, 10, 1
    rp, col, val = csr_from_lengths(lengths, k, dtype, seed=22, base=base)
    m = len(lengths)
    rng = np.random.default_rng(13)
    ldb = k + 1  # the reference kernel reads B column-major
    B = rng.uniform(-1, 1, n * ldb).astype(dtype)
    ldc = (m if order_c == 1 else n) + 2
    C0 = rng.uniform(-1, 1, (n if order_c == 1 else m) * ldc).astype(dtype)
    alpha, beta = -2.0, 0.75
    want, d = oracle.spmm(rp, col, val, B, ldb, 1, n, alpha, beta, C0, ldc, order_c, base=base)
    t = [torch.from_numpy(a).to(device) for a in (rp, col, val, B, C0.copy())]
    ct = C.c_float if dtype == np.float32 else C.c_double
    fn = ref.ref_csr_spmm_f32 if dtype == np.float32 else ref.ref_csr_spmm_f64
    rc = fn(m, n, ct(alpha), ct(beta), P(t[0]), P(t[1]), P(t[2]), P(t[3]), ldb, P(t[4]), ldc, base, order_c)
    assert rc == 0
    raw = t[4].cpu().numpy()
    got = raw.reshape(n, ldc)[:, :m].T if order_c == 1 else raw.reshape(m, ldc)[:, :n]
    assert_close(got, want, d, TOL[np.dtype(dtype)], "reference SpMM kernel vs oracle")
