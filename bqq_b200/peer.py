"""Peer-to-peer column gather for row-patch sharded BinaryQuadratic layers (one node, one process
per GPU): the set-up around the C entry points bqq_peer_alloc / bqq_peer_open / bqq_peer_gather.

Every rank allocates one region through the library, the 64-byte IPC handles travel over the
torch.distributed group (host side, once), and from then on a gather is one kernel launch per rank
with no library collective: each rank stores its column slice into every peer's buffer over NVLink,
waits (bounded) for the other slices and copies the full rows into an ordinary tensor.  The gathered
values are the shards' values, bit for bit.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _cabi
from ._cabi import BqqPeerGroup, check, lib

_DTYPE_CODE = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


class PeerGatherGroup:
    """Gather buffers of one process group.  `max_bytes` is the largest gathered result
    (rows * world * n_local * element size) the group will carry.

    `wait_cycles` bounds every wait on a peer (GPU clock cycles; 0 = about one second).

    All ranks must create the group collectively and call gather() in the same order.  Gathers of one
    group are serialised by stream order on every rank; use one group per stream."""

    def __init__(self, max_bytes: int, device: torch.device, group=None, wait_cycles: int = 0):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > _cabi.MAX_PEERS:
            raise ValueError(f'at most {_cabi.MAX_PEERS} ranks per peer gather group')
        self.device = torch.device(device)
        self.max_bytes = int(max_bytes)
        self._regions = [None] * self.world
        error = None
        with torch.cuda.device(self.device):
            own = C.c_void_p()
            handle = C.create_string_buffer(_cabi.PEER_HANDLE_BYTES)
            rc = lib.bqq_peer_alloc(self.max_bytes, C.byref(own), handle)
            if rc:
                error = f'bqq_peer_alloc: {_cabi.strerror(rc)}'
            else:
                self._regions[self.rank] = own.value
            # every rank takes part in both exchanges whatever happened locally, so that a failure on one rank
            # becomes an exception on all of them instead of a hang
            handles = [None] * self.world
            dist.all_gather_object(handles, None if error else handle.raw, group=group)
            if error is None and any(h is None for h in handles):
                error = 'a peer could not allocate its region'
            if error is None:
                for q in range(self.world):
                    if q == self.rank:
                        continue
                    p = C.c_void_p()
                    rc = lib.bqq_peer_open(handles[q], C.byref(p))
                    if rc:
                        error = f'bqq_peer_open(rank {q}): {_cabi.strerror(rc)} (CUDA IPC between these processes?)'
                        break
                    self._regions[q] = p.value
                torch.cuda.synchronize(self.device)
            errors = [None] * self.world
            dist.all_gather_object(errors, error, group=group)     # also the barrier: every region is zeroed and mapped
            if any(errors):
                for q, p in enumerate(self._regions):
                    if p is not None:
                        (lib.bqq_peer_free if q == self.rank else lib.bqq_peer_close)(p)
                self._regions = None
                raise RuntimeError('bqq_b200: peer gather group could not be set up: '
                                   + '; '.join(f'rank {q}: {e}' for q, e in enumerate(errors) if e))
        self._desc = BqqPeerGroup(self.rank, self.world, (C.c_void_p * _cabi.MAX_PEERS)(*self._regions),
                                  self.max_bytes, int(wait_cycles))

    def descriptor(self):
        """ctypes reference to the BqqPeerGroup of this rank (for the C entry points)."""
        return C.byref(self._desc)

    def gather(self, y_local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """y_local [..., n] on every rank -> [..., world*n] (columns in rank order) on every rank."""
        lead, n = y_local.shape[:-1], y_local.shape[-1]
        flat = y_local.reshape(-1, n)
        if flat.stride(-1) != 1:
            flat = flat.contiguous()
        rows = flat.shape[0]
        if out is None:
            out = torch.empty((rows, self.world * n), dtype=flat.dtype, device=flat.device)
        o2 = out.reshape(rows, self.world * n)
        if o2.data_ptr() != out.data_ptr() or o2.stride(-1) != 1 or out.dtype != flat.dtype:
            raise RuntimeError('bqq_b200: `out` must be a [rows, world*n] tensor of the input dtype with unit inner stride')
        with torch.cuda.device(self.device):
            check(lib.bqq_peer_gather(C.byref(self._desc), flat.data_ptr(), _DTYPE_CODE[flat.dtype], rows, n,
                                      flat.stride(0), o2.data_ptr(), o2.stride(0),
                                      torch.cuda.current_stream(self.device).cuda_stream), 'bqq_peer_gather')
        return o2.reshape(*lead, self.world * n)

    def status(self) -> None:
        """Synchronise the current stream and raise if a bounded wait on a peer gave up since creation."""
        with torch.cuda.device(self.device):
            check(lib.bqq_peer_status(C.byref(self._desc), torch.cuda.current_stream(self.device).cuda_stream),
                  'peer gather')

    def close(self) -> None:
        """Collective: all ranks stop using the group, then unmap the peers' regions and free the own one."""
        if self._regions is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for q, p in enumerate(self._regions):
                if p is not None and q != self.rank:
                    lib.bqq_peer_close(p)
            lib.bqq_peer_free(self._regions[self.rank])
        self._regions = None
