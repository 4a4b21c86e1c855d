"""Peer-memory plumbing for the one-shot all-reduce kernel (eptq_allreduce_push).

Each rank allocates a data and a flag buffer, shares them with the other ranks of the node through
CUDA IPC handles (exchanged over the process group), and keeps the peers' mapped pointers.  The
kernel then needs no library call per reduction: it stores into the peers' buffers directly.
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch
import torch.distributed as dist

from . import _lib


class PushAllReduce:
    """all_reduce_(t): in-place sum over the group of a contiguous fp16 CUDA tensor of at most
    `max_elems` elements (a multiple of 8).  Graph-capturable: the call counters live on the device."""

    def __init__(self, group, max_elems: int, device: torch.device):
        lib = _lib.load()
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_max = (int(max_elems) + 7) // 8 * 8
        nbytes = lib.eptq_allreduce_data_bytes(self.world, self.n_max)
        fbytes = lib.eptq_allreduce_flag_bytes(self.world)
        if nbytes == 0 or fbytes == 0:
            raise RuntimeError("eptq_b200: the push all-reduce supports 1..8 ranks")
        self.data = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.flags = torch.zeros(fbytes, dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        mine = (self.data.untyped_storage()._share_cuda_(), self.flags.untyped_storage()._share_cuda_())
        handles: List = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        self._peers = []                       # keeps the mapped storages alive
        data_ptrs, flag_ptrs = [], []
        failure = None
        try:
            for r, (hd, hf) in enumerate(handles):
                if r == self.rank:
                    data_ptrs.append(self.data.data_ptr())
                    flag_ptrs.append(self.flags.data_ptr())
                    continue
                # Open the handle in THIS GPU's context (not the owner's, which the handle tuple names): the
                # mapping is then addressable by this GPU's kernels, with peer access enabled by the open.
                here = device.index if device.index is not None else torch.cuda.current_device()
                with torch.cuda.device(here):
                    sd = torch.UntypedStorage._new_shared_cuda(here, *hd[1:])
                    sf = torch.UntypedStorage._new_shared_cuda(here, *hf[1:])
                self._peers.append((sd, sf))
                data_ptrs.append(sd.data_ptr())
                flag_ptrs.append(sf.data_ptr())
        except Exception as exc:               # no peer access, IPC not permitted, ...
            failure = exc
        # Every rank learns whether every rank succeeded, so that all of them take the same path afterwards.
        ok = torch.tensor([0 if failure is not None else 1], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise RuntimeError(f"eptq_b200: peer memory for the push all-reduce could not be mapped on every rank "
                               f"(this rank: {failure!r})")
        self._data_ptrs = (C.c_void_p * self.world)(*data_ptrs)
        self._flag_ptrs = (C.c_void_p * self.world)(*flag_ptrs)
        dist.barrier(group=group)              # everyone has mapped everyone before the first store

    def all_reduce_(self, t: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        """t <- sum over ranks of t; with `residual`: residual <- residual + sum (returned), t untouched."""
        for x in (t, residual):
            if x is not None and not (x.is_cuda and x.dtype == torch.float16 and x.is_contiguous()):
                raise RuntimeError("eptq_b200: push all-reduce takes contiguous fp16 CUDA tensors")
        n = t.numel()
        if n > self.n_max or n % 8 or (residual is not None and residual.numel() != n):
            raise RuntimeError(f"eptq_b200: push all-reduce of {n} elements (limit {self.n_max}, multiple of 8)")
        out = t if residual is None else residual
        st = _lib.load().eptq_allreduce_push(t.data_ptr(), out.data_ptr(),
                                             None if residual is None else residual.data_ptr(), n,
                                             self._data_ptrs, self._flag_ptrs, self.rank, self.world, self.n_max,
                                             torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(st, "eptq allreduce_push")
        return out

    def check(self) -> None:
        """Raise if any reduction so far ran into its wait limit (one device read)."""
        words = self.flags.view(torch.int32)
        status = int(words[2 * self.world * 8 + 8].item())
        if status != 0:
            _lib.check(status, "eptq allreduce_push (device wait)")
