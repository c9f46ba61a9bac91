"""GPU parity tests of mcsparseSpMV with fp16 / bf16 / int8 operands and fp32 / int32 sums.

The oracle runs on the operands converted to float32 (exact for all three types); what is left to allow
for is the fp32 summation (1e-5 * d, as for the fp32 kernels) and, where y is fp16 or bf16, the one
rounding of the result to y's type (half a unit in the last place of an 11-bit / 8-bit significand, and
fp16's smallest subnormal step). int8 -> int32 is integer arithmetic: bit-exact.
"""

import ctypes as C

import numpy as np
import pytest
import torch

import mcsparse_b200 as mc
from mcsparse_b200 import capi
from mcsparse_b200.capi import lib
from oracle import oracle
from tests.util import ADVERSARIAL_LENGTHS, csr_from_lengths

pytestmark = pytest.mark.gpu

# operand type, type of y, compute type, relative rounding of the stored result, absolute floor of that rounding
KINDS = {
    "f16_f32": (torch.float16, torch.float32, torch.float32, 0.0, 0.0),
    "bf16_f32": (torch.bfloat16, torch.float32, torch.float32, 0.0, 0.0),
    "i8_f32": (torch.int8, torch.float32, torch.float32, 0.0, 0.0),
    "f16_f16": (torch.float16, torch.float16, torch.float32, 2.0 ** -11, 2.0 ** -25),
    "bf16_bf16": (torch.bfloat16, torch.bfloat16, torch.float32, 2.0 ** -8, 0.0),
    "i8_i32": (torch.int8, torch.int32, torch.int32, 0.0, 0.0),
}
SHAPES = sorted(ADVERSARIAL_LENGTHS)


def operands(kind, lengths, ncols, base, device, seed=5):
    """(rp, col, val, x, y0) as torch tensors on the device plus float32 / float64 numpy copies for the oracle."""
    vt, yt, _, _, _ = KINDS[kind]
    rp, col, val32 = csr_from_lengths(lengths, ncols, np.float32, seed=seed, base=base)
    rng = np.random.default_rng(seed + 1)
    x32 = rng.uniform(-1, 1, ncols).astype(np.float32)
    y32 = rng.uniform(-1, 1, len(lengths)).astype(np.float32)
    if vt == torch.int8:
        val32, x32 = np.round(val32 * 127), np.round(x32 * 127)
    if yt == torch.int32:
        y32 = np.round(y32 * 1000)
    val, x = torch.from_numpy(val32).to(vt), torch.from_numpy(x32).to(vt)
    y0 = torch.from_numpy(y32).to(yt)
    host = (rp, col, val.to(torch.float32).numpy(), x.to(torch.float32).numpy(), y0.to(torch.float64).numpy())

    def up(t):  # one spare element, so that an empty array still has an address
        buf = torch.empty(t.numel() + 1, dtype=t.dtype, device=device)
        buf[:t.numel()] = t.to(device)
        return buf[:t.numel()]

    return tuple(up(t) for t in (torch.from_numpy(rp), torch.from_numpy(col), val, x, y0)), host


def check(kind, y, host, alpha, beta, base, what):
    rp, col, val, x, y0 = host
    _, yt, _, rel, floor = KINDS[kind]
    # the oracle takes y0 in the values' type (float32): exact for fp16 / bf16 / small integers
    ref, d = oracle.spmv(rp, col, val, x, float(alpha), float(beta), y0.astype(np.float32), base=base)
    got = y.to(torch.float64).cpu().numpy()
    if yt == torch.int32:
        assert np.array_equal(got, ref), what
        return
    err = np.abs(got - ref)
    allowed = 1e-5 * d + rel * (np.abs(ref) + 1e-5 * d) + floor + 1e-300
    assert (err <= allowed).all(), f"{what}: max err/allowed {(err / allowed).max():g}"


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("beta", [0, -0.75])
@pytest.mark.parametrize("kind", sorted(KINDS))
@pytest.mark.parametrize("name", SHAPES)
def test_low_precision_operands(handle, device, name, kind, beta, base):
    lengths = ADVERSARIAL_LENGTHS[name]
    if kind == "i8_i32" and max(lengths) > 1000:
        pytest.skip("127 * 127 * row length would leave 31 bits")
    ncols = max(max(lengths), 1) + 17
    (rp, col, val, x, y), host = operands(kind, lengths, ncols, base, device)
    integer = KINDS[kind][2] == torch.int32
    alpha, beta = (3, -2 if beta else 0) if integer else (1.25, beta)
    A = mc.CsrMatrix(len(lengths), ncols, rp, col, val, base=base)
    X, Y = mc.DnVec(x), mc.DnVec(y)
    compute = KINDS[kind][2]
    size = mc.spmv_buffer_size(handle, A, X, Y, compute=compute)
    buf = torch.empty(max(size, 1), dtype=torch.uint8, device=device)
    mc.spmv_preprocess(handle, A, X, Y, buf, compute=compute)
    if beta == 0:
        y.fill_(float("nan") if y.dtype.is_floating_point else 12345)  # beta = 0 does not read y
    mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta, compute=compute)
    torch.cuda.synchronize()
    check(kind, y, host, alpha, beta, base, f"{kind} {name}")


@pytest.mark.parametrize("kind", sorted(KINDS))
def test_low_precision_device_scalars_and_row_length_classes(handle, device, kind):
    """alpha / beta read from device memory, without the preprocess call, over several mean row lengths."""
    integer = KINDS[kind][2] == torch.int32
    sdt = torch.int32 if integer else torch.float32
    alpha = torch.tensor([2 if integer else 0.5], dtype=sdt, device=device)
    beta = torch.tensor([-1 if integer else 1.5], dtype=sdt, device=device)
    handle.set_pointer_mode(capi.MCSPARSE_POINTER_MODE_DEVICE)
    try:
        for mean in (3, 9, 20, 70):
            lengths = [mean] * 1500 + [0, 2 * mean]
            ncols = 4096
            (rp, col, val, x, y), host = operands(kind, lengths, ncols, 0, device, seed=mean)
            A = mc.CsrMatrix(len(lengths), ncols, rp, col, val)
            X, Y = mc.DnVec(x), mc.DnVec(y)
            size = mc.spmv_buffer_size(handle, A, X, Y, alpha, beta, compute=KINDS[kind][2])
            buf = torch.empty(size, dtype=torch.uint8, device=device)
            mc.spmv(handle, A, X, Y, buf, alpha=alpha, beta=beta, compute=KINDS[kind][2])
            torch.cuda.synchronize()
            check(kind, y, host, alpha.item(), beta.item(), 0, f"{kind} mean {mean}")
    finally:
        handle.set_pointer_mode(capi.MCSPARSE_POINTER_MODE_HOST)


def test_low_precision_limits(handle, device):
    """What the low-precision path does not take answers NOT_SUPPORTED, as the reference's table does for
    pairs of types it does not list (mcsp_spmv_gpu.cpp:563-564)."""
    lengths = [3] * 64
    (rp, col, val, x, y), _ = operands("f16_f32", lengths, 64, 0, device)
    A = mc.CsrMatrix(64, 64, rp, col, val)
    X, Y = mc.DnVec(x), mc.DnVec(y)
    buf = torch.empty(4096, dtype=torch.uint8, device=device)
    one, zero = C.c_float(1.0), C.c_float(0.0)
    pa, pb = C.cast(C.byref(one), C.c_void_p), C.cast(C.byref(zero), C.c_void_p)
    N, T = capi.MCSPARSE_OPERATION_NON_TRANSPOSE, capi.MCSPARSE_OPERATION_TRANSPOSE
    bp = C.c_void_p(buf.data_ptr())
    call = lambda op, xd, yd, ct: lib.mcsparseSpMV(handle.h, op, pa, A.d, xd, pb, yd, ct, capi.MCSPARSE_SPMV_ALG_DEFAULT, bp)
    assert call(N, X.d, Y.d, capi.MACA_R_32F) == capi.MCSPARSE_STATUS_SUCCESS
    assert call(T, X.d, Y.d, capi.MACA_R_32F) == capi.MCSPARSE_STATUS_NOT_SUPPORTED  # A^T x needs square: sizes match here
    assert call(N, X.d, Y.d, capi.MACA_R_16F) == capi.MCSPARSE_STATUS_NOT_SUPPORTED  # fp16 sums
    Y64 = mc.DnVec(torch.zeros(64, dtype=torch.float64, device=device))
    assert call(N, X.d, Y64.d, capi.MACA_R_32F) == capi.MCSPARSE_STATUS_NOT_SUPPORTED
    Xb = mc.DnVec(x.to(torch.bfloat16))
    assert call(N, Xb.d, Y.d, capi.MACA_R_32F) == capi.MCSPARSE_STATUS_NOT_SUPPORTED  # A and x of different types
    assert lib.mcsparseSpMV(handle.h, N, pa, A.d, X.d, pb, Y.d, capi.MACA_R_32F, capi.MCSPARSE_SPMV_ALG_DEFAULT,
                            None) == capi.MCSPARSE_STATUS_INVALID_VALUE  # the buffer is still required
    torch.cuda.synchronize()
