"""Host-side logic for running one CSR matrix on several GPUs, one process per GPU.

Rows are cut into contiguous blocks balanced by nonzeros (the rule of mcsparseB200ShardRowBounds
and of its CPU restatement); x is replicated; every rank runs the single-GPU kernels on its block;
the full y is then present on every GPU, either
  * pushed by the kernel itself into the peers' y through NVLink (`ShardedSpmv`, the product path:
    mcsparseB200SpMVPush + one tiny collective that orders the GPUs), or
  * assembled afterwards by a ragged all-gather (`all_gather_ragged`, the plain-collective baseline).
Only torch.distributed and the C ABI are used; there is no arithmetic here.
"""

import ctypes as C
import os

import torch
import torch.distributed as dist

from . import capi
from .capi import check, lib


def shard_bounds(row_lengths, world):
    """bounds[g] = first row whose starting nonzero index is >= floor(g * nnz / world);
    bounds[0] = 0, bounds[world] = rows. `row_lengths` is an integer tensor (any device)."""
    rows = int(row_lengths.numel())
    ptr = torch.zeros(rows + 1, dtype=torch.int64, device=row_lengths.device)
    torch.cumsum(row_lengths, 0, out=ptr[1:])
    nnz = int(ptr[-1].item())
    targets = torch.tensor([(g * nnz) // world for g in range(world + 1)], dtype=torch.int64, device=ptr.device)
    bounds = torch.searchsorted(ptr, targets, right=False).tolist()
    bounds[0], bounds[-1] = 0, rows
    return bounds, nnz


def all_gather_ragged(parts, local, group=None):
    """parts[g] (views into the full vector, ragged lengths) <- rank g's `local`, on every rank.
    NCCL gathers ragged lists natively; gloo needs equal sizes, so blocks are padded there."""
    world = dist.get_world_size(group)
    if world == 1:
        if parts[0].data_ptr() != local.data_ptr():
            parts[0].copy_(local)
        return
    if dist.get_backend(group) == "nccl":
        dist.all_gather(parts, local, group=group)
        return
    longest = max(p.numel() for p in parts)
    padded = torch.zeros(longest, dtype=local.dtype, device=local.device)
    padded[: local.numel()] = local
    gathered = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded, group=group)
    for p, g in zip(parts, gathered):
        p.copy_(g[: p.numel()])


class _DeviceArray:
    """Exposes a raw device pointer to torch through the CUDA array interface."""

    def __init__(self, ptr, numel, dtype):
        typestr = {torch.float32: "<f4", torch.float64: "<f8", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 2}


class PeerVector:
    """A full-length device vector that every rank of the node can write: allocated with
    mcsparseB200PeerAlloc, exported to the other ranks and mapped there with mcsparseB200PeerOpen."""

    def __init__(self, numel, dtype, group=None):
        self.group, self.numel, self.dtype = group, numel, dtype
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        itemsize = torch.empty(0, dtype=dtype).element_size()
        p = C.c_void_p()
        # behind the vector (256-byte aligned): the flag area of mcsparseB200PeerSignalWait
        self.flag_offset = (max(numel, 1) * itemsize + 255) & ~255
        check(lib.mcsparseB200PeerAlloc(C.byref(p), self.flag_offset + capi.PEER_FLAG_INTS * 4), "mcsparseB200PeerAlloc")
        self.ptr = p.value
        device = torch.device("cuda", torch.cuda.current_device())
        self.tensor = torch.as_tensor(_DeviceArray(self.ptr, numel, dtype), device=device)
        self.tensor.zero_()
        self.flags = torch.as_tensor(_DeviceArray(self.ptr + self.flag_offset, capi.PEER_FLAG_INTS, torch.int32), device=device)
        self.flags.zero_()
        torch.cuda.synchronize()
        handle = C.create_string_buffer(64)
        check(lib.mcsparseB200PeerExport(C.c_void_p(self.ptr), handle), "mcsparseB200PeerExport")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.peer_ptrs = {}
        for g, raw in enumerate(handles):
            if g == self.rank:
                continue
            mapped = C.c_void_p()
            check(lib.mcsparseB200PeerOpen(C.create_string_buffer(raw, 64), C.byref(mapped)), "mcsparseB200PeerOpen")
            self.peer_ptrs[g] = mapped.value
        # slot of source rank g inside a rank r's flag area: g's position among r's peers in rank order
        peers = sorted(self.peer_ptrs)
        self.remote_slots = (C.c_void_p * max(len(peers), 1))(*[
            self.peer_ptrs[g] + self.flag_offset + 4 * (self.rank if self.rank < g else self.rank - 1) for g in peers])
        dist.barrier(group=group)  # every rank's flag area is zeroed before anyone signals into it

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody unmaps or frees while a peer may still write
        for mapped in self.peer_ptrs.values():
            lib.mcsparseB200PeerClose(C.c_void_p(mapped))
        self.peer_ptrs = {}
        dist.barrier(group=self.group)
        if self.ptr:
            self.tensor = None
            self.flags = None
            lib.mcsparseB200PeerFree(C.c_void_p(self.ptr))
            self.ptr = 0


class MulticastVector:
    """A full-length device vector allocated on every rank by torch's symmetric-memory allocator and
    bound to one NVSwitch multicast mapping: a multimem store to `multicast_ptr + offset` lands at
    `offset` in every rank's copy. Raises RuntimeError when the GPUs offer no multicast mapping."""

    def __init__(self, numel, dtype, group=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.numel, self.dtype = numel, dtype
        device = torch.device("cuda", torch.cuda.current_device())
        self.tensor = symm.empty(max(numel, 1), dtype=dtype, device=device)[:numel]
        self.handle = symm.rendezvous(self.tensor, group=self.group)
        base = int(self.handle.multicast_ptr)
        if base == 0:
            raise RuntimeError("no NVSwitch multicast mapping available for symmetric memory on this system")
        # The multicast range mirrors this rank's allocation: same offset, same bytes.
        delta = self.tensor.data_ptr() - int(self.handle.buffer_ptrs[self.handle.rank])
        if not 0 <= delta < int(self.handle.buffer_size):
            raise RuntimeError("symmetric-memory tensor lies outside its allocation")
        self.multicast_ptr = base + delta
        self.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.group)  # nobody frees while a peer's kernel may still store
        self.handle = None
        self.tensor = None
        dist.barrier(group=self.group)


def push_mode(world):
    """How ShardedSpmv assembles y: MCSPARSE_B200_PUSH_MODE=peer|multicast, default peer stores."""
    mode = os.environ.get("MCSPARSE_B200_PUSH_MODE", "peer")
    return mode if mode in ("peer", "multicast") and world > 1 else "peer"


def destination_order(rank, world, mode=None):
    """The other ranks of the group in the order a rank lists them as push destinations: rank order, or with
    MCSPARSE_B200_PEER_ORDER=rotated (or mode="rotated") rank + 1, rank + 2, ... modulo the group."""
    mode = mode or os.environ.get("MCSPARSE_B200_PEER_ORDER", "ascending")
    others = [g for g in range(world) if g != rank]
    return sorted(others, key=lambda g: (g - rank) % world) if mode == "rotated" else others


class ShardedSpmv:
    """y = alpha * A @ x + beta * y for a row-sharded A with the full y left on every GPU.

    `A_local` is this rank's row block as a CsrMatrix (local row offsets, global columns), `x` the
    full-length input, `row_offset` the global index of the block's first row."""

    def __init__(self, handle, A_local, x, row_offset, total_rows, group=None):
        from . import host

        self.h, self.A, self.group = handle, A_local, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.row_offset = int(row_offset)
        self.mode = push_mode(self.world)
        if self.mode == "multicast":
            self.y = MulticastVector(total_rows, A_local.dtype, group)
        else:
            self.y = PeerVector(total_rows, A_local.dtype, group)
        self.y_local = self.y.tensor[self.row_offset:self.row_offset + A_local.rows]
        self.X, self.Y = host.DnVec(x), host.DnVec(self.y_local)
        self.buffer = torch.empty(host.spmv_buffer_size(handle, A_local, self.X, self.Y), dtype=torch.uint8,
                                  device=x.device)
        host.spmv_preprocess(handle, A_local, self.X, self.Y, self.buffer)
        # Destinations in rank order; MCSPARSE_B200_PEER_ORDER=rotated lists them as rank + 1, rank + 2, ... modulo the
        # group, so that at any moment the ranks aim at different GPUs instead of all starting with GPU 0.
        ptrs = [] if self.mode == "multicast" else [self.y.peer_ptrs[g] for g in destination_order(self.rank, self.world)]
        self.n_peers = len(ptrs)
        self.peer_array = (C.c_void_p * max(self.n_peers, 1))(*ptrs)
        self.token = torch.zeros(1, dtype=torch.int32, device=x.device)
        # After the push the GPUs are ordered by per-peer arrival flags written and awaited on the device
        # (mcsparseB200PeerSignalWait); MCSPARSE_B200_PUSH_SYNC=collective uses a 4-byte all-reduce instead,
        # as the multicast variant always does (its vector comes from another allocator).
        self.sync_flags = self.mode == "peer" and os.environ.get("MCSPARSE_B200_PUSH_SYNC", "flags") != "collective"
        self.epoch = 0

    def compute(self, alpha=1.0, beta=0.0):
        """Launches the local SpMV with the push of finished rows to the peers (asynchronous)."""
        from . import host

        pa, pb, keep = host._scalars(self.h, alpha, beta, self.A.dtype)
        if self.mode == "multicast":
            check(lib.mcsparseB200SpMVPushMulticast(self.h.h, capi.MCSPARSE_OPERATION_NON_TRANSPOSE, pa, self.A.d,
                                                    self.X.d, pb, self.Y.d, host._DTYPE[self.A.dtype],
                                                    capi.MCSPARSE_SPMV_ALG_DEFAULT, host._ptr(self.buffer),
                                                    C.c_void_p(self.y.multicast_ptr), self.row_offset),
                  "mcsparseB200SpMVPushMulticast")
            del keep
            return
        check(lib.mcsparseB200SpMVPush(self.h.h, capi.MCSPARSE_OPERATION_NON_TRANSPOSE, pa, self.A.d, self.X.d, pb,
                                       self.Y.d, host._DTYPE[self.A.dtype], capi.MCSPARSE_SPMV_ALG_DEFAULT,
                                       host._ptr(self.buffer), self.n_peers, self.peer_array, self.row_offset),
              "mcsparseB200SpMVPush")
        del keep

    def step(self, alpha=1.0, beta=0.0):
        """compute() and then the ordering collective: when it completes on this rank's stream, every
        rank's kernel has finished and therefore all pushes into this GPU's y have landed."""
        self.compute(alpha, beta)
        if self.world > 1:
            if self.sync_flags:
                self.epoch = (self.epoch + 1) & 0x7FFFFFFF
                check(lib.mcsparseB200PeerSignalWait(self.h.h, self.n_peers, self.y.remote_slots,
                                                     C.c_void_p(self.y.ptr + self.y.flag_offset), self.epoch),
                      "mcsparseB200PeerSignalWait")
            else:
                dist.all_reduce(self.token, group=self.group)

    def close(self):
        self.y.close()
