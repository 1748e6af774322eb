"""Exchange buffers of a rank group over NVLink peer memory.

One process per GPU. Every rank allocates the same named buffers, exports them through CUDA IPC
(the handles travel as Python objects through the process group) and maps the other ranks'
buffers into its own address space. Kernels of this library then read a peer's partial sums with
plain loads over NVLink / NVSwitch: the reduce-scatter half of the reference's all-reduce
(racetrack/realistic_bench.py:315-316,351) becomes part of the kernel that consumes it
(rt_peer_reduce_residual_norm), after a device-side barrier (rt_peer_barrier). No multicast
object and no tensor map ever covers another GPU's memory.

Order of use for one exchange, on every rank and on one stream:
    write the local buffer  ->  barrier()  ->  read the peers' buffers
A buffer may be rewritten after the NEXT barrier of the group (by then every rank has finished
reading it, because it arrived at that barrier after its reads); the layer alternates two buffers,
so one barrier per exchange is enough.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, comm, ops


class PeerExchange:
    def __init__(self, group: comm.Group, device: torch.device, buffers: dict[str, tuple]):
        """buffers: name -> (shape, dtype) of the local tensor every rank allocates."""
        from torch.multiprocessing.reductions import reduce_tensor
        if group.world > 8:
            raise RuntimeError("peer exchange supports at most 8 ranks")
        self.group, self.rank, self.world = group, group.rank, group.world
        self.local = {name: torch.empty(shape, dtype=dtype, device=device)
                      for name, (shape, dtype) in buffers.items()}
        self.flags = torch.zeros(self.world + 1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        exported = {name: reduce_tensor(t) for name, t in {**self.local, "__flags__": self.flags}.items()}
        gathered = [None] * self.world
        dist.all_gather_object(gathered, exported, group=group.group)
        self.views: dict[str, list[torch.Tensor]] = {}
        for name in exported:
            views = []
            for q in range(self.world):
                if q == self.rank:
                    views.append(self.flags if name == "__flags__" else self.local[name])
                else:
                    rebuild, args = gathered[q][name]
                    views.append(rebuild(*args))
            self.views[name] = views
        self._ptrs = {name: (ctypes.c_void_p * self.world)(*[v.data_ptr() for v in views])
                      for name, views in self.views.items()}
        # every rank has mapped every buffer before anyone uses them
        dist.barrier(group=group.group)

    def barrier(self) -> None:
        """All ranks' work enqueued before this call (on the current stream of each) is complete
        and visible when the kernels enqueued after it run."""
        lib = _lib.load()
        _lib.check(lib.rt_peer_barrier(self._ptrs["__flags__"], self.rank, self.world, ops._stream()),
                   "rt_peer_barrier")

    def reduce_residual_norm(self, name: str, residual_rows: torch.Tensor, weight: torch.Tensor, *,
                             eps: float):
        """(normed, hidden) for this rank's rows: hidden = (sum over ranks of buffer `name`)[rows]
        + residual_rows, normed = rms_norm(hidden) * weight. Includes the barrier that makes
        every rank's partial sums visible."""
        part = self.local[name]
        return self.group._timed("peer_barrier+reduce_residual_norm", part,
                                 lambda: self._reduce_residual_norm(part, name, residual_rows, weight, eps))

    def _reduce_residual_norm(self, part, name, residual_rows, weight, eps):
        self.barrier()
        total_rows, cols = part.shape
        lo, hi = self.group.rows_of(total_rows)
        res = residual_rows if residual_rows.stride(-1) == 1 else residual_rows.contiguous()
        w = weight.contiguous()
        normed = torch.empty(hi - lo, cols, dtype=torch.bfloat16, device=part.device)
        hidden = torch.empty(hi - lo, cols, dtype=torch.bfloat16, device=part.device)
        lib = _lib.load()
        _lib.check(lib.rt_peer_reduce_residual_norm(
            self._ptrs[name], self.world, lo, part.stride(0), res.data_ptr(), w.data_ptr(),
            ops._weight_tag(w), normed.data_ptr(), hidden.data_ptr(), hi - lo, cols, res.stride(0),
            float(eps), ops._stream()), "rt_peer_reduce_residual_norm")
        return normed, hidden

    def check(self) -> None:
        """Synchronises and raises if a barrier gave up waiting for a rank."""
        torch.cuda.synchronize()
        _lib.check(_lib.load().rt_peer_error_state(), "peer barrier")
