"""Partition specs: what a partition fuses and where its kernels live.

Mirror of racetrack/partition_spec.py:21-140 (same classes, fields, properties and functions),
so code written against racetrack's ``PartitionSpec`` / ``FusedOp`` / ``load_spec`` /
``discover_partitions`` / ``BASELINE_SPEC`` runs against this module unchanged. A partition is
``partitions/<model>/<hash>/spec.py`` (constants ``FUSED_OPS``, ``GRAPH_NODES``,
``PARTITION_NOTES``) plus ``kernels/<backend>/<op>.py``; ``<hash>`` is the first 8 hex digits of
the SHA-256 of the spec.py bytes. The partitions root defaults to the one shipped inside this
package and can be redirected with ``RACETRACK_PARTITIONS_ROOT`` (e.g. to a racetrack checkout).
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any

PROJECT_ROOT = Path(__file__).resolve().parent
KINDS = ("fx_pattern", "pre_trace", "module_patch")


def partitions_root() -> Path:
    override = os.environ.get("RACETRACK_PARTITIONS_ROOT")
    return Path(override) if override else PROJECT_ROOT / "partitions"


@dataclass(frozen=True)
class FusedOp:
    name: str
    kind: str  # one of KINDS

    def to_dict(self) -> dict[str, str]:
        return {"name": self.name, "kind": self.kind}


@dataclass(frozen=True)
class PartitionSpec:
    model: str
    partition_hash: str
    notes: str
    graph_nodes: dict[str, list[str]]
    fused_ops: tuple[FusedOp, ...]

    @property
    def partition_dir(self) -> Path:
        return partitions_root() / self.model / self.partition_hash

    @property
    def kernel_root(self) -> Path:
        return self.partition_dir / "kernels"

    @property
    def partition_id(self) -> str:
        """Directory-name hash: SHA-256 of the spec.py bytes, 8 hex digits. Specs that exist
        only in memory (BASELINE_SPEC) hash their fields instead."""
        spec_file = self.partition_dir / "spec.py"
        if spec_file.exists():
            digest = hashlib.sha256(spec_file.read_bytes())
        else:
            fields = repr((self.model, self.partition_hash, self.notes, self.graph_nodes, self.fused_ops))
            digest = hashlib.sha256(fields.encode("utf-8"))
        return digest.hexdigest()[:8]

    def _of_kind(self, kind: str) -> list[FusedOp]:
        return [op for op in self.fused_ops if op.kind == kind]

    @property
    def fx_ops(self) -> list[FusedOp]:
        return self._of_kind("fx_pattern")

    @property
    def pre_trace_ops(self) -> list[FusedOp]:
        return self._of_kind("pre_trace")

    @property
    def module_patch_ops(self) -> list[FusedOp]:
        return self._of_kind("module_patch")

    @property
    def op_names(self) -> tuple[str, ...]:
        return tuple(op.name for op in self.fused_ops)

    @property
    def label(self) -> str:
        return f"{self.model}/{self.partition_hash}"


def _exec_spec(path: Path) -> Any:
    spec = importlib.util.spec_from_file_location(f"spec_{path.parent.name}", str(path))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def load_spec(model: str, partition_hash: str) -> PartitionSpec:
    path = partitions_root() / model / partition_hash / "spec.py"
    if not path.exists():
        raise FileNotFoundError(f"No spec.py at {path}")
    module = _exec_spec(path)
    ops = tuple(FusedOp(name=o["name"], kind=o["kind"]) for o in getattr(module, "FUSED_OPS", []))
    return PartitionSpec(model=model, partition_hash=partition_hash,
                         notes=getattr(module, "PARTITION_NOTES", ""),
                         graph_nodes=getattr(module, "GRAPH_NODES", {}), fused_ops=ops)


def discover_partitions(model: str) -> list[PartitionSpec]:
    """Every partition directory of `model` that has both a spec.py and a kernels/ directory."""
    root = partitions_root() / model
    if not root.is_dir():
        return []
    found = []
    for entry in sorted(root.iterdir()):
        if not entry.is_dir() or entry.name.startswith("__"):
            continue
        if not (entry / "spec.py").exists() or not (entry / "kernels").is_dir():
            continue
        try:
            found.append(load_spec(model, entry.name))
        except Exception:
            continue
    return found


BASELINE_SPEC = PartitionSpec(model="baseline", partition_hash="baseline",
                              notes="No partition — pure torch fallback", graph_nodes={},
                              fused_ops=())
