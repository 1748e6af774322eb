"""Collectives of the sharded layer: thin wrappers over torch.distributed.

One process per GPU, NCCL over NVLink. The layer exchanges activations in three ways only
(the counterpart of the two all-reduces of racetrack/realistic_bench.py:315-316,351):

  reduce_scatter_rows   partial sums [T, H] of every rank -> this rank's T / world rows of
                        their sum (the first half of an all-reduce; the token-wise kernels that
                        follow run on those rows only)
  all_gather_rows       this rank's rows -> all rows, in rank order (the second half, moved
                        behind the token-wise kernels and carrying their SMALLER outputs:
                        the [T, 2112] latent projection or NVFP4 codes instead of bf16 hidden
                        states)
  all_reduce_max        a one-element maximum (the tensor-wide amax of the NVFP4 global scale)

The gloo backend has no reduce-scatter; there (CPU tests of the host logic) it is an all-reduce
followed by taking the rank's rows, which is the same result.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class Group:
    """A process group with the rank / world size the layer was built for. world == 1 makes
    every collective the identity, so single-GPU code paths need no branches."""

    def __init__(self, rank: int = 0, world: int = 1, group: Optional["dist.ProcessGroup"] = None):
        self.rank, self.world, self.group = rank, world, group
        if world > 1 and not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("a sharded layer needs an initialised torch.distributed process group")
        self._no_reduce_scatter = world > 1 and dist.get_backend(group) == "gloo"
        self.events = None          # a list while timing: (name, bytes sent by this rank, start, end)
        self.nccl_calls = 0         # collectives handed to torch.distributed so far

    def start_timing(self, in_graph: bool = False) -> None:
        """From now on every collective is bracketed by CUDA events on the current stream (the
        interval includes the wait for the collective's input, as the layer experiences it).
        `in_graph`: the calls are about to be captured into a CUDA graph; the events become
        event-record nodes of the graph and are read after a replay."""
        self.events = []
        self._external = bool(in_graph)

    def stop_timing(self) -> dict:
        """{name: (calls, total ms, total payload bytes)} of the collectives since start_timing."""
        torch.cuda.synchronize()
        out: dict = {}
        for name, nbytes, start, end in self.events or []:
            calls, ms, total = out.get(name, (0, 0.0, 0))
            out[name] = (calls + 1, ms + start.elapsed_time(end), total + nbytes)
        self.events = None
        self._external = False
        return out

    def _timed(self, name: str, payload: torch.Tensor, fn):
        if not name.startswith("peer_"):
            self.nccl_calls += 1
        if self.events is None or not payload.is_cuda:
            return fn()
        ext = getattr(self, "_external", False)
        start = torch.cuda.Event(enable_timing=True, external=ext)
        end = torch.cuda.Event(enable_timing=True, external=ext)
        start.record()
        result = fn()
        end.record()
        self.events.append((name, payload.numel() * payload.element_size(), start, end))
        return result

    def rows_of(self, total_rows: int) -> tuple[int, int]:
        """[begin, end) of this rank's rows of a [total_rows, ...] tensor."""
        if total_rows % self.world:
            raise RuntimeError(f"{total_rows} rows do not divide over {self.world} ranks")
        per = total_rows // self.world
        return self.rank * per, (self.rank + 1) * per

    def reduce_scatter_rows(self, partial: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return partial
        lo, hi = self.rows_of(partial.shape[0])
        partial = partial.contiguous()
        if self._no_reduce_scatter:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
            return partial[lo:hi].clone()
        out = torch.empty((hi - lo, *partial.shape[1:]), dtype=partial.dtype, device=partial.device)
        self._timed("reduce_scatter", partial, lambda: dist.reduce_scatter_tensor(
            out, partial, op=dist.ReduceOp.SUM, group=self.group))
        return out

    def all_gather_rows(self, rows: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return rows
        rows = rows.contiguous()
        out = torch.empty((rows.shape[0] * self.world, *rows.shape[1:]), dtype=rows.dtype,
                          device=rows.device)
        src, dst = rows, out
        if rows.dtype == torch.float8_e4m3fn:       # collectives move bytes
            src, dst = rows.view(torch.uint8), out.view(torch.uint8)
        self._timed("all_gather", rows, lambda: dist.all_gather_into_tensor(dst, src, group=self.group))
        return out

    def all_reduce_max(self, value: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            self._timed("all_reduce_max", value,
                        lambda: dist.all_reduce(value, op=dist.ReduceOp.MAX, group=self.group))
        return value

    def all_reduce_sum(self, value: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            self._timed("all_reduce_sum", value,
                        lambda: dist.all_reduce(value, op=dist.ReduceOp.SUM, group=self.group))
        return value
