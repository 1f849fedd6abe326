"""Tensor-parallel exchange for one process per GPU: the library's one-shot all-reduce over peer-mapped memory
(include/scrapgpu_sm100.h, sm100_allreduce_*).  torch.distributed is used only to pass the IPC handles around."""
from __future__ import annotations

import ctypes as C

import torch

from . import capi


class PeerAllReduce:
    """In-place sum of a short f32 vector over all ranks: `ar(t)` enqueues one kernel on the current torch stream.
    Every rank must make the same sequence of calls (it can be captured in a CUDA graph and replayed)."""

    def __init__(self, rank: int, world: int, device_index: int, capacity_floats: int, dist):
        self.L = capi.lib()
        self.rank, self.world = rank, world
        capi.check(self.L.sm100_set_device(device_index), "set_device")
        nbytes = int(self.L.sm100_allreduce_area_bytes(world, capacity_floats))
        self.area = capi.Buffer(nbytes, device_index)
        s = capi.Stream(device_index)
        self.area.fill(s, 0)
        s.sync()
        s.close()
        hb = int(self.L.sm100_ipc_handle_bytes())
        mine = (C.c_ubyte * hb)()
        capi.check(self.L.sm100_ipc_export(C.c_void_p(self.area.ptr), mine), "ipc_export")
        handles = [None] * world
        dist.all_gather_object(handles, bytes(mine))
        self.opened = []
        areas = (C.c_void_p * world)()
        for r in range(world):
            if r == rank:
                areas[r] = self.area.ptr
            else:
                p = C.c_void_p()
                capi.check(self.L.sm100_ipc_open((C.c_ubyte * hb).from_buffer_copy(handles[r]), C.byref(p)), "ipc_open")
                self.opened.append(p)
                areas[r] = p.value
        dist.barrier()   # every area is zeroed and mapped everywhere before the first store
        self.ctx = C.c_void_p()
        capi.check(self.L.sm100_allreduce_create(rank, world, capacity_floats, areas, C.byref(self.ctx)), "allreduce_create")

    def __call__(self, t: torch.Tensor) -> None:
        assert t.dtype == torch.float32 and t.is_contiguous()
        stream = C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)
        capi.check(self.L.sm100_allreduce_sum(self.ctx, stream, C.c_void_p(t.data_ptr()), t.numel()), "allreduce_sum")

    def fault(self) -> int:
        v = C.c_int(0)
        capi.check(self.L.sm100_allreduce_fault(self.ctx, C.byref(v)), "allreduce_fault")
        return int(v.value)
