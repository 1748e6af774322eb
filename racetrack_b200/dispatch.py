"""Kernel dispatcher: op name -> callable of a partition's ``kernels/<backend>/*.py``.

Mirror of the part of racetrack/runtime/dispatch.py:18-143 that a partition with one native
backend needs: the ``RACETRACK_KERNEL_BACKEND`` switch (:39-44), ``call`` (:56-76), ``_resolve``
(:95-102), module loading by directory listing (:104-143), ``backend_status`` (:46-54) and the
missing-kernel error (:92-93). There is exactly one backend here, ``cuda``; ``best`` (the
reference's timing race between Triton / CuTe-DSL / Helion, :145-196) resolves to it directly,
and ``torch`` still means "run the caller's fallback", as in the reference.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path
from types import ModuleType
from typing import Any, Callable

import torch

Fallback = Callable[..., Any]


class KernelDispatcher:
    BACKENDS = ("cuda",)

    def __init__(self, kernel_root: str | Path | None = None):
        self.kernel_root = Path(kernel_root) if kernel_root is not None else None
        self._modules: dict[str, list[ModuleType]] = {}
        # kept for code that peeks at the reference's autoselect state
        self._best_fast_path: dict[str, str] = {}

    # -- backend selection --------------------------------------------------------------
    @staticmethod
    def selected_backend(default: str = "torch") -> str:
        raw = os.getenv("RACETRACK_KERNEL_BACKEND", default).strip().lower()
        return {"cutedl": "cutedsl", "b200": "cuda"}.get(raw, raw)

    def backend_status(self, backend: str) -> str:
        if backend == "torch":
            return "native"
        modules = self._load_backend_modules(backend)
        if any(bool(getattr(m, "BACKEND_AVAILABLE", False)) for m in modules):
            return "native"
        return "missing"

    def best_summary(self) -> str:
        return "mixed=cuda"

    # -- dispatch -----------------------------------------------------------------------------
    # Opaque to Dynamo: a dispatched kernel is host code around a C-ABI call (environment lookup,
    # module loading, raw pointers and the current stream's handle), none of which can be traced.
    # Under torch.compile a model that reaches its kernels through the dispatcher gets a graph
    # break here and the call runs as it does in eager mode.
    @torch.compiler.disable
    def call(self, op_name: str, fallback: Fallback, *args: Any, backend: str | None = None,
             **kwargs: Any) -> Any:
        selected = backend or self.selected_backend(default="torch")
        if selected in ("torch", "all"):
            return fallback(*args, **kwargs)
        if selected == "best":
            selected = "cuda"
        fn = self._resolve(selected, op_name)
        if fn is None:
            self._handle_missing(selected, op_name)
        return fn(*args, fallback=fallback, **kwargs)

    def _handle_missing(self, backend: str, op_name: str) -> None:
        raise RuntimeError(f"No available {backend} kernel found for {op_name}")

    def _resolve(self, backend: str, op_name: str) -> Callable[..., Any] | None:
        for module in self._load_backend_modules(backend):
            if not bool(getattr(module, "BACKEND_AVAILABLE", False)):
                continue
            fn = getattr(module, op_name, None)
            if callable(fn):
                return fn
        return None

    # -- module loading -----------------------------------------------------------------------
    def _load_backend_modules(self, backend: str) -> list[ModuleType]:
        cached = self._modules.get(backend)
        if cached is not None:
            return cached
        modules: list[ModuleType] = []
        if self.kernel_root is not None:
            directory = self.kernel_root / backend
            if directory.is_dir():
                for path in sorted(directory.glob("*.py")):
                    if not path.name.startswith("_"):
                        modules.append(self._import(backend, path))
        self._modules[backend] = modules
        return modules

    @staticmethod
    def _import(backend: str, path: Path) -> ModuleType:
        name = f"racetrack_partition_kernel_{abs(hash(str(path)))}_{backend}_{path.stem}"
        spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
        return module
