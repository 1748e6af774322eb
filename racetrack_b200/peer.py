"""Exchange buffers of a rank group over NVLink peer memory.

One process per GPU. Every rank allocates the same named buffers, exports them through CUDA IPC
(the handles travel as Python objects through the process group) and maps the other ranks'
buffers into its own address space. Kernels of this library then read a peer's partial sums with
plain loads over NVLink / NVSwitch: the reduce-scatter half of the reference's all-reduce
(racetrack/realistic_bench.py:315-316,351) becomes part of the kernel that consumes it
(rt_peer_reduce_residual_norm), after a device-side barrier (rt_peer_barrier). No multicast
object and no tensor map ever covers another GPU's memory.

The buffers are cudaMalloc allocations of this library (rt_peer_alloc), not torch storage: a peer
opens them with its own device current (rt_peer_open), which is what lets kernels on that device
dereference the mapping; torch sees the local ones as tensors through __cuda_array_interface__.

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


class _RawCuda:
    """A device allocation of this library exposed through __cuda_array_interface__, so that torch
    can view it as a tensor without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class _Bytes:
    """Stands in for a payload tensor where the group's timing wants a byte count."""
    is_cuda = True

    def __init__(self, nbytes: int):
        self._n = int(nbytes)

    def numel(self) -> int:
        return self._n

    def element_size(self) -> int:
        return 1


def _as_tensor(ptr: int, shape: tuple, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    nbytes = int(torch.empty((), dtype=dtype).element_size())
    for d in shape:
        nbytes *= int(d)
    raw = torch.as_tensor(_RawCuda(ptr, nbytes), device=device)
    return raw.view(dtype).view(shape)


class PeerExchange:
    def __init__(self, group: comm.Group, device: torch.device, buffers: dict[str, tuple]):
        """buffers: name -> (shape, dtype) of the local tensor every rank allocates."""
        if group.world > 8:
            raise RuntimeError("peer exchange supports at most 8 ranks")
        self.group, self.rank, self.world, self.device = group, group.rank, group.world, device
        lib = _lib.load()
        specs = {**buffers, "__flags__": ((self.world + 1,), torch.int32)}
        self._own: dict[str, int] = {}
        handles: dict[str, bytes] = {}
        self.local: dict[str, torch.Tensor] = {}
        with torch.cuda.device(device):
            for name, (shape, dtype) in specs.items():
                nbytes = int(torch.empty((), dtype=dtype).element_size())
                for d in shape:
                    nbytes *= int(d)
                ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
                _lib.check(lib.rt_peer_alloc(max(nbytes, 16), ctypes.byref(ptr), handle), "rt_peer_alloc")
                self._own[name] = ptr.value
                handles[name] = bytes(handle)
                self.local[name] = _as_tensor(ptr.value, tuple(shape), dtype, device)
            gathered = [handles]
            if self.world > 1:
                gathered = [None] * self.world
                dist.all_gather_object(gathered, handles, group=group.group)
            # a peer's buffer is opened with THIS rank's device current: the mapping (and the
            # NVLink peer access behind it) then belongs to the device whose kernels will use it
            self._mapped: dict[str, list[int]] = {}
            for name in specs:
                ptrs = []
                for q in range(self.world):
                    if q == self.rank:
                        ptrs.append(self._own[name])
                        continue
                    ptr = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[q][name])
                    _lib.check(lib.rt_peer_open(buf, ctypes.byref(ptr)), "rt_peer_open")
                    ptrs.append(ptr.value)
                self._mapped[name] = ptrs
        self.flags = self.local.pop("__flags__")
        self._ptrs = {name: (ctypes.c_void_p * self.world)(*ptrs) for name, ptrs in self._mapped.items()}
        # every rank has mapped every buffer before anyone uses them
        if self.world > 1:
            dist.barrier(group=group.group)

    def close(self) -> None:
        """Unmaps the peers' buffers and, once every rank has done so, frees the own ones."""
        if not self._own:
            return
        lib = _lib.load()
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for name, ptrs in self._mapped.items():
                for q, ptr in enumerate(ptrs):
                    if q != self.rank:
                        lib.rt_peer_close(ctypes.c_void_p(ptr))
            if self.world > 1:
                dist.barrier(group=self.group.group)
            for ptr in self._own.values():
                lib.rt_peer_free(ctypes.c_void_p(ptr))
        self._own, self._mapped, self.local = {}, {}, {}

    def barrier(self) -> None:
        """All ranks' work enqueued before this call (on the current stream of each) is complete
        and visible when the kernels enqueued after it run."""
        lib = _lib.load()
        _lib.check(lib.rt_peer_barrier(self._ptrs["__flags__"], self.rank, self.world, ops._stream()),
                   "rt_peer_barrier")

    def reduce_residual_norm(self, name: str, residual_rows: torch.Tensor, weight: torch.Tensor, *,
                             eps: float, all_rows: bool = False):
        """(normed, hidden) for this rank's rows: hidden = (sum over ranks of buffer `name`)[rows]
        + residual_rows, normed = rms_norm(hidden) * weight. Includes the barrier that makes
        every rank's partial sums visible. all_rows=True: every rank reduces ALL rows (a one-shot
        all-reduce fused with the kernel that follows it, for the few rows of a decode step)."""
        part = self.local[name]
        # timed apart: the barrier's interval is the wait for the slowest rank (load imbalance),
        # the kernel's interval is the transfer itself
        self.group._timed("peer_barrier (wait for the slowest rank)", self.flags, self.barrier)
        return self.group._timed("peer_reduce_residual_norm", part,
                                 lambda: self._reduce_residual_norm(part, name, residual_rows, weight, eps, all_rows))

    def _reduce_residual_norm(self, part, name, residual_rows, weight, eps, all_rows=False):
        total_rows, cols = part.shape
        lo, hi = (0, total_rows) if all_rows else self.group.rows_of(total_rows)
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

    def gather(self, *names: str) -> None:
        """All-gather of the named row-sharded buffers (at most four): every rank has written its
        own rows [rows_of(T)] of its local copy; after the call the local copies hold all rows.
        Includes the barrier that makes every rank's rows visible."""
        lib = _lib.load()
        ptrs, slices = [], []
        for name in names:
            buf = self.local[name]
            nbytes = buf.numel() * buf.element_size()
            if buf.shape[0] % self.world or (nbytes // self.world) % 16:
                raise RuntimeError(f"peer gather: buffer {name!r} does not split into 16-byte aligned blocks")
            ptrs.extend(self._mapped[name])
            slices.append(nbytes // self.world)
        c_ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        c_slices = (ctypes.c_int64 * len(slices))(*slices)
        self.group._timed("peer_barrier (wait for the slowest rank)", self.flags, self.barrier)
        payload = _Bytes(sum(slices) * (self.world - 1))      # what crosses NVLink into this rank
        self.group._timed("peer_gather", payload, lambda: _lib.check(
            lib.rt_peer_gather(c_ptrs, c_slices, len(slices), self.rank, self.world, ops._stream()),
            "rt_peer_gather"))

    def gather_cols(self, names: tuple, row0: int, rows: int) -> list:
        """For each named buffer (every rank's copy holds THAT rank's column block [T, cols] for
        all rows): this rank's rows [row0, row0 + rows) of the whole [T, world * cols] matrix, as a
        new local tensor [rows, world * cols]. Includes the barrier."""
        lib = _lib.load()
        ptrs, outs, row_bytes = [], [], []
        for name in names:
            buf = self.local[name]
            cols = buf.shape[1]
            outs.append(torch.empty(rows, self.world * cols, dtype=buf.dtype, device=buf.device))
            ptrs.extend(self._mapped[name])
            row_bytes.append(cols * buf.element_size())
        c_ptrs = (ctypes.c_void_p * len(ptrs))(*ptrs)
        c_dst = (ctypes.c_void_p * len(outs))(*[o.data_ptr() for o in outs])
        c_rb = (ctypes.c_int64 * len(row_bytes))(*row_bytes)
        self.group._timed("peer_barrier (wait for the slowest rank)", self.flags, self.barrier)
        payload = _Bytes(sum(row_bytes) * rows * (self.world - 1))
        self.group._timed("peer_gather_cols", payload, lambda: _lib.check(
            lib.rt_peer_gather_cols(c_ptrs, c_dst, c_rb, len(outs), row0, rows, self.world, ops._stream()),
            "rt_peer_gather_cols"))
        return outs

    def allmax(self, name: str, value: torch.Tensor) -> torch.Tensor:
        """The maximum over ranks of a non-negative 1-element fp32 tensor, through the 16-byte
        buffer `name`: store, barrier, read every rank's slot. Every rank gets the same value."""
        self.local[name][:1].copy_(value.reshape(1))
        out = torch.empty(1, dtype=torch.float32, device=value.device)
        lib = _lib.load()
        self.group._timed("peer_barrier (wait for the slowest rank)", self.flags, self.barrier)
        self.group._timed("peer_allmax", out, lambda: _lib.check(
            lib.rt_peer_allmax(self._ptrs[name], self.world, out.data_ptr(), ops._stream()), "rt_peer_allmax"))
        return out

    def check(self) -> None:
        """Synchronises and raises if a barrier gave up waiting for a rank."""
        torch.cuda.synchronize()
        _lib.check(_lib.load().rt_peer_error_state(), "peer barrier")
