"""Seeded synthetic CSR workloads: the five benchmark configurations and scaled-down copies.

No public dataset is involved; every matrix is defined by this code. Each random draw is a
counter-based hash of (seed, global row or index, draw number), so a row block generated on
one rank equals the same rows of the whole matrix, on the CPU or on a GPU, whatever the
batching. The code is plain torch integer/float tensor arithmetic and runs on either device.

  C1  2-D 5-point Laplacian, 1024 x 1024 grid, fp32, y = A x
  C2  rows of max(1, Poisson(16)) nonzeros, n = 4,194,304, fp64, y = A x + 0.5 y
  C3  power-law rows (Zipf 2.1 on [1, 131072], rescaled to ~2e8 nonzeros), n = 16,777,216, fp32
  C4  rows of Poisson(32) nonzeros, n = 1,048,576, fp32, SpMM with row-major B of 64 / 128 columns
  C5  3-D 27-point stencil on 256^3, fp64

Random columns of a row of length L are one uniform draw from each of L equal strata of
[0, n): sorted, distinct, uniform marginal density (stands in for "uniform without
replacement, sorted", which has no data-parallel form).
"""

import math
from dataclasses import dataclass, field

import numpy as np
import torch

_M64 = (1 << 64) - 1


def _s64(v):
    """Python int (mod 2^64) as a signed 64-bit value torch accepts."""
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


_GOLD = _s64(0x9E3779B97F4A7C15)
_MUL1 = _s64(0xBF58476D1CE4E5B9)
_MUL2 = _s64(0x94D049BB133111EB)
_KEY_A = _s64(0xD6E8FEB86659FD93)
_KEY_B = _s64(0xA0761D6478BD642F)


def _lsr(z, k):
    return (z >> k) & ((1 << (64 - k)) - 1)


def _mix64(z):
    """splitmix64 finaliser on int64 tensors (wrapping arithmetic)."""
    z = z + _GOLD
    z = (z ^ _lsr(z, 30)) * _MUL1
    z = (z ^ _lsr(z, 27)) * _MUL2
    return z ^ _lsr(z, 31)


def _hash(seed, a, b, stream):
    """64 random bits per element of the broadcast of int64 tensors a, b."""
    h = _mix64(a * _KEY_A + _s64(seed))
    h = _mix64(h ^ (b * _KEY_B + stream))
    return h


def _u01(h):
    """[0, 1) doubles from the top 53 bits: exact on CPU and GPU."""
    return _lsr(h, 11).to(torch.float64) * (1.0 / (1 << 53))


def _uniform_pm1(seed, a, b, stream):
    return 2.0 * _u01(_hash(seed, a, b, stream)) - 1.0


def _normal(seed, a, b, stream):
    u1 = _u01(_hash(seed, a, b, stream))
    u2 = _u01(_hash(seed, a, b, stream + 1))
    return torch.sqrt(-2.0 * torch.log1p(-u1)) * torch.cos((2.0 * math.pi) * u2)


# --------------------------------------------------------------------------- configurations

@dataclass
class Config:
    name: str
    kind: str  # "stencil2d" | "stencil3d" | "poisson" | "powerlaw"
    op: str  # "spmv" | "spmm"
    dtype: torch.dtype
    alpha: float
    beta: float
    grid: int = 0  # stencils: points per dimension
    n: int = 0  # random kinds: rows = cols
    mean: float = 0.0  # poisson mean row length
    min_len: int = 0
    nnz_target: float = 0.0  # powerlaw
    max_len: int = 131072
    zipf: float = 2.1
    values: str = "uniform"  # "uniform" | "normal"
    dense_cols: tuple = ()  # SpMM: columns of B
    seed: int = 0

    @property
    def rows(self):
        if self.kind == "stencil2d":
            return self.grid ** 2
        if self.kind == "stencil3d":
            return self.grid ** 3
        return self.n


CONFIGS = {
    "C1": Config("C1", "stencil2d", "spmv", torch.float32, 1.0, 0.0, grid=1024, seed=0x5EED0001),
    "C2": Config("C2", "poisson", "spmv", torch.float64, 1.0, 0.5, n=4194304, mean=16.0, min_len=1,
                 seed=0x5EED0002),
    "C3": Config("C3", "powerlaw", "spmv", torch.float32, 1.0, 0.0, n=16777216, nnz_target=2.0e8,
                 values="normal", seed=0x5EED0003),
    "C4": Config("C4", "poisson", "spmm", torch.float32, 1.0, 0.0, n=1048576, mean=32.0, min_len=0,
                 dense_cols=(64, 128), seed=0x5EED0004),
    "C5": Config("C5", "stencil3d", "spmv", torch.float64, 1.0, 0.0, grid=256, seed=0x5EED0005),
}


def scaled(name, factor):
    """A copy of a configuration shrunk by about `factor` in rows (same row-length law)."""
    c = CONFIGS[name]
    out = Config(**{**c.__dict__})
    if c.kind == "stencil2d":
        out.grid = max(2, int(round(c.grid / math.sqrt(factor))))
    elif c.kind == "stencil3d":
        out.grid = max(2, int(round(c.grid / factor ** (1.0 / 3.0))))
    else:
        out.n = max(16, int(c.n // factor))
        out.nnz_target = c.nnz_target / factor
        out.max_len = min(c.max_len, out.n)
    return out


# --------------------------------------------------------------------------- row lengths

def _poisson_cdf(mean, kmax=256):
    p = math.exp(-mean)
    acc, cdf = 0.0, []
    for k in range(kmax):
        acc += p
        cdf.append(min(acc, 1.0))
        p *= mean / (k + 1)
    return np.asarray(cdf, dtype=np.float64)


def _zipf_cdf(s, kmax):
    w = np.arange(1, kmax + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    return c / c[-1]


def _stencil_axis_counts(grid, idx):
    """Neighbours (self included) of coordinate idx along one axis: 2 at the ends, else 3."""
    return 3 - (idx == 0).to(torch.int64) - (idx == grid - 1).to(torch.int64)


def row_lengths(cfg, device, r0=0, r1=None):
    """int64 nonzeros per row for global rows [r0, r1)."""
    r1 = cfg.rows if r1 is None else r1
    rows = torch.arange(r0, r1, dtype=torch.int64, device=device)
    g = cfg.grid
    if cfg.kind == "stencil2d":
        i, j = rows // g, rows % g
        ci, cj = _stencil_axis_counts(g, i), _stencil_axis_counts(g, j)
        return ci + cj - 1  # 5-point: the two axis neighbourhoods share the centre
    if cfg.kind == "stencil3d":
        i, j, k = rows // (g * g), (rows // g) % g, rows % g
        return _stencil_axis_counts(g, i) * _stencil_axis_counts(g, j) * _stencil_axis_counts(g, k)
    if cfg.kind == "poisson":
        u = _u01(_hash(cfg.seed, rows, torch.zeros_like(rows), 11))
        cdf = torch.from_numpy(_poisson_cdf(cfg.mean)).to(device)
        k = torch.searchsorted(cdf, u, right=True)
        return torch.clamp(k, min=cfg.min_len, max=cfg.n)
    if cfg.kind == "powerlaw":
        return _powerlaw_lengths(cfg, device, r0, r1)
    raise ValueError(cfg.kind)


def _zipf_draws(cfg, device, r0, r1):
    rows = torch.arange(r0, r1, dtype=torch.int64, device=device)
    u = _u01(_hash(cfg.seed, rows, torch.zeros_like(rows), 11))
    cdf = torch.from_numpy(_zipf_cdf(cfg.zipf, cfg.max_len)).to(device)
    return torch.clamp(torch.searchsorted(cdf, u, right=True) + 1, max=cfg.max_len)


_SCALE_CACHE = {}


def _powerlaw_scale(cfg, device):
    """nnz_target / sum of all Zipf draws: a property of the whole matrix (integer sum, so
    the same on every device and rank)."""
    key = (cfg.seed, cfg.n, cfg.max_len, cfg.zipf, cfg.nnz_target)
    if key not in _SCALE_CACHE:
        total, step = 0, 1 << 24
        for a in range(0, cfg.n, step):
            total += int(_zipf_draws(cfg, device, a, min(cfg.n, a + step)).sum().item())
        _SCALE_CACHE[key] = cfg.nnz_target / total
    return _SCALE_CACHE[key]


def _powerlaw_lengths(cfg, device, r0, r1):
    c = _powerlaw_scale(cfg, device)
    z = _zipf_draws(cfg, device, r0, r1).to(torch.float64)
    return torch.clamp(torch.round(z * c).to(torch.int64), min=1, max=cfg.max_len)


# --------------------------------------------------------------------------- matrices

@dataclass
class Workload:
    cfg: Config
    base: int
    row_begin: int  # global index of local row 0
    rows: int  # local rows
    cols: int  # global columns
    nnz: int
    row_ptr: torch.Tensor  # int32, rows + 1, local offsets + base
    col: torch.Tensor  # int32, global columns + base
    val: torch.Tensor
    x: torch.Tensor = None  # SpMV: dense vector of `cols`
    y0: torch.Tensor = None  # initial y of the local rows (read when beta != 0)
    B: dict = field(default_factory=dict)  # SpMM: n -> (cols x n) row-major
    alpha: float = 1.0
    beta: float = 0.0


def _stencil_block(cfg, device, r0, r1):
    g = cfg.grid
    rows = torch.arange(r0, r1, dtype=torch.int32, device=device)
    if cfg.kind == "stencil2d":
        coords = [rows // g, rows % g]
        offs = [(-1, 0), (0, -1), (0, 0), (0, 1), (1, 0)]
        diag = 4.0
    else:
        coords = [rows // (g * g), (rows // g) % g, rows % g]
        offs = [(a, b, c) for a in (-1, 0, 1) for b in (-1, 0, 1) for c in (-1, 0, 1)]
        diag = 26.0
    cand = torch.empty((rows.numel(), len(offs)), dtype=torch.int32, device=device)
    valid = torch.empty((rows.numel(), len(offs)), dtype=torch.bool, device=device)
    centre = offs.index(tuple([0] * len(coords)))
    for s, off in enumerate(offs):
        ok = torch.ones_like(rows, dtype=torch.bool)
        lin = torch.zeros_like(rows)
        for cdim, o in zip(coords, off):
            q = cdim + o
            ok &= (q >= 0) & (q < g)
            lin = lin * g + q
        cand[:, s] = lin
        valid[:, s] = ok
    lengths = valid.sum(dim=1, dtype=torch.int64)
    col = cand[valid]
    vals = torch.full((len(offs),), -1.0, dtype=cfg.dtype, device=device)
    vals[centre] = diag
    val = vals.expand(rows.numel(), len(offs))[valid]
    return lengths, col, val


def _random_block(cfg, device, r0, r1, lengths):
    n = cfg.n
    m = r1 - r0
    local_ptr = torch.zeros(m + 1, dtype=torch.int64, device=device)
    torch.cumsum(lengths, 0, out=local_ptr[1:])
    nnz = int(local_ptr[-1].item())
    lrow = torch.repeat_interleave(torch.arange(m, dtype=torch.int64, device=device), lengths, output_size=nnz)
    slot = torch.arange(nnz, dtype=torch.int64, device=device) - local_ptr[lrow]
    L = lengths[lrow]
    grow = lrow + r0
    del lrow
    lo = (slot * n) // L
    width = ((slot + 1) * n) // L - lo
    del L
    u = _u01(_hash(cfg.seed, grow, slot, 21))
    col = (lo + torch.floor(u * width.to(torch.float64)).to(torch.int64)).to(torch.int32)
    del lo, width, u
    if cfg.values == "normal":
        val = _normal(cfg.seed, grow, slot, 31).to(cfg.dtype)
    else:
        val = _uniform_pm1(cfg.seed, grow, slot, 31).to(cfg.dtype)
    return col, val


def dense_values(cfg, device, count, stream, first=0, normal=False):
    """`count` values of a dense operand (x, y0, B, C0), starting at flat index `first`."""
    idx = torch.arange(first, first + count, dtype=torch.int64, device=device)
    zero = torch.zeros_like(idx)
    v = _normal(cfg.seed, idx, zero, stream) if normal else _uniform_pm1(cfg.seed, idx, zero, stream)
    return v.to(cfg.dtype)


def generate(cfg, device, base=0, row_range=None, with_dense=True):
    """Builds global rows [r0, r1) of the configuration (default: all) on `device`."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    r0, r1 = (0, cfg.rows) if row_range is None else row_range
    device = torch.device(device)
    if cfg.kind in ("stencil2d", "stencil3d"):
        lengths, col, val = _stencil_block(cfg, device, r0, r1)
    else:
        lengths = row_lengths(cfg, device, r0, r1)
        col, val = _random_block(cfg, device, r0, r1, lengths)
    row_ptr = torch.zeros(r1 - r0 + 1, dtype=torch.int64, device=device)
    torch.cumsum(lengths, 0, out=row_ptr[1:])
    nnz = int(row_ptr[-1].item())
    assert nnz < 2 ** 31
    w = Workload(cfg=cfg, base=base, row_begin=r0, rows=r1 - r0, cols=cfg.rows, nnz=nnz,
                 row_ptr=(row_ptr + base).to(torch.int32), col=(col + base) if base else col, val=val,
                 alpha=cfg.alpha, beta=cfg.beta)
    if with_dense:
        normal = cfg.values == "normal"
        if cfg.op == "spmv":
            w.x = dense_values(cfg, device, cfg.rows, 41, normal=normal)
            w.y0 = dense_values(cfg, device, r1 - r0, 51, first=r0)
        else:
            for n in cfg.dense_cols:
                w.B[n] = dense_values(cfg, device, cfg.rows * n, 61 + n).view(cfg.rows, n)
    return w


def algorithmic_bytes(rows, cols, nnz, value_size, beta, dense_cols=None, index_size=4):
    """Bytes one call must move: A once, row offsets, x (or B) once, y (or C) written, and read iff beta != 0."""
    a = nnz * (value_size + index_size) + (rows + 1) * index_size
    n = 1 if dense_cols is None else dense_cols
    dense_in = cols * n * value_size
    out = rows * n * value_size
    return a + dense_in + out * (2 if beta != 0 else 1)
