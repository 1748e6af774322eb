"""torch.compile backend driven by a PartitionSpec.

Mirror of racetrack/compile_backend.py:34-111: ``RacetrackBackend(spec)`` receives Dynamo's FX
GraphModules, rewrites them with the partition's fx_pattern ops and returns ``gm.forward`` for
eager execution (no Inductor; the kernels are the hand-written CUDA ones). ``compile_with_partition``
first applies the pre_trace / module_patch ops to the modules, then compiles; it returns the
compiled model and the originals needed by ``rollback_patches``.

    spec = load_spec("dsv3_2", "<hash>")
    compiled, originals = compile_with_partition(model, spec, backend_override="cuda")
    out = compiled(tokens)
"""
from __future__ import annotations

import os
from typing import Callable

import torch
import torch.nn as nn
from torch.fx import GraphModule

from .dispatch import KernelDispatcher
from .fx_patterns import rewrite_graph
from .partition_spec import BASELINE_SPEC, PartitionSpec
from .pre_trace import Originals, apply_pre_trace_patches


def _dispatcher_for(spec: PartitionSpec) -> KernelDispatcher:
    return KernelDispatcher(spec.kernel_root if spec.kernel_root.is_dir() else None)


class RacetrackBackend:
    def __init__(self, spec: PartitionSpec):
        self.spec = spec
        self.dispatcher = _dispatcher_for(spec)

    def __call__(self, gm: GraphModule, example_inputs):
        gm = rewrite_graph(gm, self.spec, self.dispatcher)
        gm.recompile()
        return gm.forward


def make_racetrack_backend(spec: PartitionSpec | None = None) -> Callable:
    return RacetrackBackend(BASELINE_SPEC if spec is None else spec)


def compile_with_partition(model: nn.Module, spec: PartitionSpec, *,
                           backend_override: str | None = None) -> tuple[nn.Module, Originals]:
    """Pre-trace patches, then torch.compile with RacetrackBackend. `backend_override` sets
    RACETRACK_KERNEL_BACKEND and leaves it set: compilation is lazy, so the variable is read
    when the compiled model first runs (racetrack/compile_backend.py:76-84)."""
    if backend_override is not None:
        os.environ["RACETRACK_KERNEL_BACKEND"] = backend_override
    originals = apply_pre_trace_patches(model, spec, _dispatcher_for(spec))
    compiled = torch.compile(model, backend=RacetrackBackend(spec))
    return compiled, originals


def cleanup_compile_state() -> None:
    dynamo = getattr(torch, "_dynamo", None)
    reset = getattr(dynamo, "reset", None)
    if callable(reset):
        reset()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


try:  # named backend, like the reference's "racetrack"
    from torch._dynamo import register_backend
    register_backend(name="racetrack_b200", compiler_fn=make_racetrack_backend())
except Exception:
    pass
