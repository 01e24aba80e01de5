"""Small all-reduce over peer memory: the Python side of ``aoto_sm100_peer_sum``.

One :class:`PeerSum` per process group and maximum row length. It owns this
rank's receive buffer in symmetric memory (``torch.distributed._symmetric_memory``
maps every rank's buffer into every process), the device epoch word the kernel
advances, and a status word a timed-out poll sets. ``sum_`` is one kernel launch on
the current stream - no library collective - and can be recorded into a CUDA graph.
All ranks must make the same sequence of calls.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from . import _native as N
from .errors import DeviceError, PlanInputError


class PeerSum:
    def __init__(self, max_count: int, *, group: Any = None, device: Any = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.capacity_words = (int(max_count) + 1) // 2
        lib = N.load()
        nbytes = int(lib.aoto_sm100_peer_sum_buffer_bytes(self.world, self.capacity_words))
        if nbytes <= 0:
            raise PlanInputError(f"no peer exchange for a world of {self.world} ranks and {max_count} values")
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        pointers = [int(p) for p in self.handle.buffer_ptrs]
        if len(pointers) != self.world or any(p == 0 for p in pointers):
            raise DeviceError("symmetric memory did not return one mapped buffer per rank")
        self._pointers = (ctypes.c_void_p * self.world)(*pointers)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # every buffer is zero before any rank stores into it
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def sum_(self, tensor: torch.Tensor) -> torch.Tensor:
        """In-place sum of ``tensor`` (bf16, contiguous, at most ``max_count`` values) over the ranks."""

        if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous() or not tensor.is_cuda:
            raise PlanInputError("peer sum takes a contiguous bfloat16 CUDA tensor")
        count = tensor.numel()
        if (count + 1) // 2 > self.capacity_words:
            raise PlanInputError(f"{count} values exceed the exchange's capacity of {2 * self.capacity_words}")
        args = N.PeerSumArgs(self._pointers, tensor.data_ptr(), tensor.data_ptr(), self.epoch.data_ptr(),
                             self.status.data_ptr(), self.world, self.rank, count, self.capacity_words)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        N.check(N.load().aoto_sm100_peer_sum(ctypes.byref(args), stream), "aoto_sm100_peer_sum")
        return tensor

    def check(self) -> None:
        """Raise if a poll of an earlier call ran out (synchronises)."""

        if int(self.status.item()):
            self.status.zero_()
            raise DeviceError("a peer-exchange poll ran out: a rank did not deliver its contribution in time")
