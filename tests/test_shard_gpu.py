"""GPU tests of the sharding entry points. The bounds / local-offset kernels need one GPU; the
fused row push (mcsparseB200SpMVPush over peer-mapped y) and the NCCL ragged all-gather need two
and are skipped on a single-GPU box."""

import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import mcsparse_b200 as mc
from mcsparse_b200 import capi, sharding, workloads
from mcsparse_b200.capi import lib
from oracle import oracle
from tests.util import ADVERSARIAL_LENGTHS, TOL, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("base", [0, 1])
@pytest.mark.parametrize("name", ["long_then_short", "empty_start_mid_end", "many_short", "all_empty"])
def test_shard_bounds_and_local_offsets_bit_exact(handle, device, name, base):
    lengths = ADVERSARIAL_LENGTHS[name]
    rp = (np.concatenate([[0], np.cumsum(lengths)]) + base).astype(np.int32)
    nnz, m = int(rp[-1] - base), len(lengths)
    d_rp = torch.from_numpy(rp).to(device)
    for G in (1, 2, 3, 8):
        out = (C.c_int64 * (G + 1))()
        capi.check(lib.mcsparseB200ShardRowBounds(handle.h, m, nnz, base, C.c_void_p(d_rp.data_ptr()), G, out))
        want = oracle.shard_row_bounds(rp, nnz, G, base)
        assert list(out) == want.tolist()
        for g in range(G):
            r0, n = int(want[g]), int(want[g + 1] - want[g])
            loc = torch.empty(n + 1, dtype=torch.int32, device=device)
            capi.check(lib.mcsparseB200ShardLocalRowOffsets(handle.h, C.c_void_p(d_rp.data_ptr()), r0, n, base,
                                                            C.c_void_p(loc.data_ptr())))
            torch.cuda.synchronize()
            np.testing.assert_array_equal(loc.cpu().numpy(), oracle.shard_local_row_offsets(rp, r0, n, base))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, factor, chunks, out, mode="peer", store="crew", sync="flags"):
    """One rank of a two-GPU run. A comparison that fails is recorded in out[rank] and the rank still walks
    through every barrier and the tear-down of its peer mappings (job.close()), so that the other rank is
    never left waiting and no memory stays bound to a multicast object; the parent asserts on `out`."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), MCSPARSE_B200_PUSH_CHUNKS=str(chunks),
                      MCSPARSE_B200_PUSH_MODE=mode, MCSPARSE_B200_PUSH_STORE=store, MCSPARSE_B200_PUSH_SYNC=sync)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    errors = []

    def check(fn):
        try:
            fn()
        except AssertionError as e:
            errors.append(str(e)[:500])

    job = None
    try:
        cfg = workloads.scaled(name, factor)
        lengths = workloads.row_lengths(cfg, dev)
        bounds, nnz = sharding.shard_bounds(lengths, world)
        r0, r1 = bounds[rank], bounds[rank + 1]
        w = workloads.generate(cfg, dev, row_range=(r0, r1))
        h = mc.Handle()
        A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
        whole = workloads.generate(cfg, "cpu")
        alpha, beta = 1.5, 0.5
        ref, d = oracle.spmv(whole.row_ptr, whole.col, whole.val, whole.x, alpha, beta, whole.y0)

        # product path: rows pushed to the peers by the kernel, then the GPUs are ordered
        try:
            job = sharding.ShardedSpmv(h, A, w.x, r0, cfg.rows)
        except RuntimeError as e:  # no multicast mapping on this system: the same on every rank
            if mode != "multicast":
                raise
            out[rank] = f"skipped: {e}"
            return
        check(lambda: _assert(job.mode == mode, "push mode"))
        for _ in range(2):  # second step: the work buffer and the peer mappings are reused
            job.y.tensor.fill_(float("nan"))
            job.y_local.copy_(w.y0)
            torch.cuda.synchronize()
            dist.barrier()
            job.step(alpha, beta)
            torch.cuda.synchronize()
            got = job.y.tensor.cpu().numpy()
            check(lambda: assert_close(got, ref, d, TOL[cfg.dtype], f"push, rank {rank}"))
        dist.barrier()

        # baseline path: local SpMV, then a ragged NCCL all-gather
        y_full = torch.zeros(cfg.rows, dtype=cfg.dtype, device=dev)
        y_loc = y_full[r0:r1]
        y_loc.copy_(w.y0)
        X, Y = mc.DnVec(w.x), mc.DnVec(y_loc)
        buf = torch.empty(mc.spmv_buffer_size(h, A, X, Y), dtype=torch.uint8, device=dev)
        mc.spmv(h, A, X, Y, buf, alpha=alpha, beta=beta)
        sharding.all_gather_ragged([y_full[bounds[g]:bounds[g + 1]] for g in range(world)], y_loc)
        torch.cuda.synchronize()
        check(lambda: assert_close(y_full.cpu().numpy(), ref, d, TOL[cfg.dtype], f"all-gather, rank {rank}"))
        check(lambda: _assert(torch.equal(y_full, job.y.tensor), "both assemblies hold the very same bits"))
        out[rank] = "; ".join(errors) if errors else 1
    finally:
        try:
            if job is not None:
                job.close()  # two barriers inside: peers are unmapped before anyone frees
        finally:
            dist.destroy_process_group()


def _assert(cond, what):
    assert cond, what


# chunks 0: rows stored to the peers by the tile kernel (bulk copies from shared memory, or ordinary stores);
# 4: pipelined row copies. The GPUs are ordered by device-side arrival flags, or by a 4-byte all-reduce.
@pytest.mark.parametrize("chunks,store,sync", [(0, "crew", "flags"), (0, "bulk", "flags"), (0, "lsu", "collective"),
                                               (4, "crew", "flags")])
@pytest.mark.parametrize("name,factor", [("C5", 512), ("C3", 256)])
def test_sharded_spmv_push_and_allgather_two_gpus(name, factor, chunks, store, sync):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    env = {"NCCL_NVLS_ENABLE": "0"}
    os.environ.update(env)
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, port, name, factor, chunks, out, "peer", store, sync), nprocs=2, join=True)
        assert dict(out) == {0: 1, 1: 1}


@pytest.mark.parametrize("name,factor", [("C5", 512), ("C3", 256)])
def test_sharded_spmv_multicast_push_two_gpus(name, factor):
    """Rows stored once into an NVSwitch multicast mapping (multimem.st) instead of once per peer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, port, name, factor, 0, out, "multicast"), nprocs=2, join=True)
        assert sorted(out.keys()) == [0, 1]
        if any(isinstance(v, str) and v.startswith("skipped") for v in out.values()):
            pytest.skip(str(out[0]))
        assert dict(out) == {0: 1, 1: 1}


@pytest.mark.parametrize("chunks,store", [(0, "crew"), (0, "bulk"), (0, "lsu"), (1, "crew"), (4, "crew"), (8, "crew")])
@pytest.mark.parametrize("offset", [5, 8])
@pytest.mark.parametrize("name,factor", [("C3", 256), ("C5", 512), ("C2", 512)])
def test_push_to_a_second_local_buffer_matches_plain_spmv(handle, device, name, factor, chunks, store, offset,
                                                          monkeypatch):
    """One-GPU stand-in for a peer: the push destination is another buffer on the same device. The
    pushed copy, the local result and plain mcsparseSpMV must agree bit for bit, with the pushed
    rows landing at rowOffset + row."""
    from mcsparse_b200 import host

    monkeypatch.setenv("MCSPARSE_B200_PUSH_CHUNKS", str(chunks))
    monkeypatch.setenv("MCSPARSE_B200_PUSH_STORE", store)
    cfg = workloads.scaled(name, factor)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    y_plain, y_push = w.y0.clone(), w.y0.clone()
    peer = torch.full((w.rows + 2 * offset,), float("nan"), dtype=cfg.dtype, device=device)
    X, Y1, Y2 = mc.DnVec(w.x), mc.DnVec(y_plain), mc.DnVec(y_push)
    buf = torch.empty(mc.spmv_buffer_size(handle, A, X, Y1), dtype=torch.uint8, device=device)
    mc.spmv(handle, A, X, Y1, buf, alpha=1.5, beta=0.5)
    pa, pb, keep = host._scalars(handle, 1.5, 0.5, cfg.dtype)
    arr = (C.c_void_p * 1)(peer.data_ptr())
    capi.check(lib.mcsparseB200SpMVPush(handle.h, 0, pa, A.d, X.d, pb, Y2.d, host._DTYPE[cfg.dtype], 0,
                                        host._ptr(buf), 1, arr, offset))
    torch.cuda.synchronize()
    assert torch.equal(y_plain, y_push)
    assert torch.equal(peer[offset:offset + w.rows], y_push)
    assert torch.isnan(peer[:offset]).all() and torch.isnan(peer[offset + w.rows:]).all()
    assert lib.mcsparseB200SpMVPush(handle.h, 0, pa, A.d, X.d, pb, Y2.d, host._DTYPE[cfg.dtype], 0, host._ptr(buf),
                                    8, arr, 0) == capi.MCSPARSE_STATUS_INVALID_VALUE


def test_pipelined_push_replays_with_alternating_vectors(handle, device, monkeypatch):
    """The pipelined push replays a captured graph per set of arguments and keeps a few of them: a caller that
    cycles through more vector pairs than are kept must still get every product right."""
    from mcsparse_b200 import host

    monkeypatch.setenv("MCSPARSE_B200_PUSH_CHUNKS", "4")
    cfg = workloads.scaled("C5", 512)
    w = workloads.generate(cfg, device)
    A = mc.CsrMatrix(w.rows, w.cols, w.row_ptr, w.col, w.val)
    pairs = 5
    xs = [workloads.dense_values(cfg, device, w.cols, 90 + i) for i in range(pairs)]
    ys = [torch.zeros(w.rows, dtype=cfg.dtype, device=device) for _ in range(pairs)]
    peers = [torch.zeros(w.rows, dtype=cfg.dtype, device=device) for _ in range(pairs)]
    expect = []
    buf = torch.empty(mc.spmv_buffer_size(handle, A, mc.DnVec(xs[0]), mc.DnVec(ys[0])), dtype=torch.uint8, device=device)
    for x in xs:
        y = torch.zeros(w.rows, dtype=cfg.dtype, device=device)
        mc.spmv(handle, A, mc.DnVec(x), mc.DnVec(y), buf, alpha=2.0, beta=0.0)
        expect.append(y)
    pa, pb, keep = host._scalars(handle, 2.0, 0.0, cfg.dtype)
    X = [mc.DnVec(x) for x in xs]
    Y = [mc.DnVec(y) for y in ys]
    for step in range(3 * pairs):
        i = step % pairs
        ys[i].fill_(float("nan"))
        peers[i].fill_(float("nan"))
        arr = (C.c_void_p * 1)(peers[i].data_ptr())
        capi.check(lib.mcsparseB200SpMVPush(handle.h, 0, pa, A.d, X[i].d, pb, Y[i].d, host._DTYPE[cfg.dtype], 0,
                                            host._ptr(buf), 1, arr, 0))
        torch.cuda.synchronize()
        assert torch.equal(ys[i], expect[i]) and torch.equal(peers[i], expect[i]), f"step {step}"


def test_peer_signal_wait_loopback_and_bounded_wait(device):
    """mcsparseB200PeerSignalWait on one GPU. Loopback: the "remote" slot is this rank's own slot, so the
    kernel's signal satisfies its own wait. Then a slot that nothing sets: the wait runs out after the
    handle's limit, the kernel returns by itself, the status word and the next compute call report it."""
    h = mc.Handle()
    try:
        flags = torch.zeros(capi.PEER_FLAG_INTS, dtype=torch.int32, device=device)
        slot0 = (C.c_void_p * 1)(flags.data_ptr())
        for epoch in (1, 2, 7):
            capi.check(lib.mcsparseB200PeerSignalWait(h.h, 1, slot0, C.c_void_p(flags.data_ptr()), epoch))
            torch.cuda.synchronize()
            assert flags[0].item() == epoch and flags[capi.PEER_FLAG_STATUS].item() == 0
        # signal goes to a slot elsewhere, the awaited slot 0 stays at 7 < 8: bounded wait, about 0.5 ms
        capi.check(lib.mcsparseB200SetDeviceWaitLimit(h.h, 20000, 0))
        other = torch.zeros(1, dtype=torch.int32, device=device)
        elsewhere = (C.c_void_p * 1)(other.data_ptr())
        capi.check(lib.mcsparseB200PeerSignalWait(h.h, 1, elsewhere, C.c_void_p(flags.data_ptr()), 8))
        torch.cuda.synchronize()
        assert other.item() == 8 and flags[capi.PEER_FLAG_STATUS].item() == 1
        assert lib.mcsparseB200PeerSignalWait(h.h, 1, slot0, C.c_void_p(flags.data_ptr()), 9) == \
            capi.MCSPARSE_STATUS_EXECUTION_FAILED  # reported once, by the next call on the handle
        capi.check(lib.mcsparseB200PeerSignalWait(h.h, 1, slot0, C.c_void_p(flags.data_ptr()), 9))
        torch.cuda.synchronize()
        assert flags[0].item() == 9
        assert lib.mcsparseB200PeerSignalWait(h.h, 8, slot0, C.c_void_p(flags.data_ptr()), 1) == \
            capi.MCSPARSE_STATUS_INVALID_VALUE
    finally:
        h.close()
