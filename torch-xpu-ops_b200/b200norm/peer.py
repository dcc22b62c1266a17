"""Peer-memory plumbing for the fused weight-gradient fold + all-reduce kernel (b2n_norm_wgrad_fold_allreduce).

One process per GPU on one node.  Every rank lets the library allocate its exchange buffer, hands the buffer's
64-byte CUDA IPC handle to the others through the process group, and opens theirs with its own device current;
from then on the kernel does the whole exchange: flags and data move by plain peer stores and loads over NVLink,
nothing goes through a library collective.  torch.distributed carries the one-time exchange of the handles."""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import OK, B200NormError, load_library
from .capi import Prepared, _dt, _ptr, _stream


class WgradExchange:
    """The exchange buffers of one (N, CTA count) configuration, opened on every rank of `group`.

    Collective: every rank of the group constructs it at the same point, and afterwards makes the same sequence of
    fold_allreduce calls.  ctas: CTAs the kernel uses — about 128 when it runs in the stream of the row kernels
    and has the GPU to itself, as few as the SMs left free when it runs on a second stream beside them.
    close() (collective as well) unmaps and frees; the buffers otherwise live until the process exits."""

    def __init__(self, n: int, device: torch.device, group=None, ctas: int = 128):
        self.lib = load_library()
        self.n, self.ctas, self.device, self.group = int(n), int(ctas), device, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > 8:
            raise ValueError("WgradExchange: at most 8 ranks (one node)")
        self._local = ctypes.c_void_p()
        self._mapped = []
        with torch.cuda.device(device):
            handle = ctypes.create_string_buffer(64)
            self._check(self.lib.b2n_wgrad_exchange_alloc(self.n, ctypes.byref(self._local), handle), "b2n_wgrad_exchange_alloc")
            pointers = [self._local.value]
            if self.world > 1:
                everyone = [None] * self.world
                dist.all_gather_object(everyone, bytes(handle.raw), group=group)
                pointers = []
                for r, h in enumerate(everyone):
                    if r == self.rank:
                        pointers.append(self._local.value)
                        continue
                    mapped = ctypes.c_void_p()
                    # this rank's device is current: the mapping belongs to the context whose kernels will use it
                    self._check(self.lib.b2n_wgrad_exchange_open(h, ctypes.byref(mapped)), f"b2n_wgrad_exchange_open(rank {r})")
                    self._mapped.append(mapped)
                    pointers.append(mapped.value)
                torch.cuda.synchronize()
                dist.barrier(group=group)
        self._table = (ctypes.c_void_p * self.world)(*pointers)

    @staticmethod
    def _check(rc, what):
        if rc != OK:
            raise B200NormError(rc, what)

    def close(self):
        """Unmap the peers' buffers and free this rank's (every rank, after its last call has finished)."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)  # nobody unmaps while a peer's kernel may still be reading
            for m in self._mapped:
                self.lib.b2n_wgrad_exchange_close(m)
            self._mapped = []
            if self._local:
                self.lib.b2n_wgrad_exchange_free(self._local)
                self._local = ctypes.c_void_p()

    def _args(self, workspace, partial_rows, dgamma, dbeta):
        w = dgamma if dgamma is not None else dbeta
        if w is None or w.numel() != self.n:
            raise ValueError("WgradExchange: dgamma / dbeta must have the N this exchange was opened for")
        return (_ptr(workspace), int(partial_rows), self.n, self._table, self.n, self.rank, self.world, _ptr(dgamma),
                _ptr(dbeta), _dt(w.dtype), self.ctas, _stream(w))

    def fold_allreduce(self, workspace, partial_rows: int, dgamma=None, dbeta=None) -> None:
        """Fold this rank's partial sums and add all ranks' results, in one kernel on the current stream."""
        with torch.cuda.device(self.device):
            rc = self.lib.b2n_norm_wgrad_fold_allreduce(*self._args(workspace, partial_rows, dgamma, dbeta))
        self._check(rc, "b2n_norm_wgrad_fold_allreduce")

    def prepare(self, workspace, partial_rows: int, dgamma=None, dbeta=None) -> Prepared:
        """The same as a Prepared call bound to the current stream."""
        return Prepared(self.lib.b2n_norm_wgrad_fold_allreduce, self._args(workspace, partial_rows, dgamma, dbeta),
                        "b2n_norm_wgrad_fold_allreduce", (workspace, dgamma, dbeta, self))
