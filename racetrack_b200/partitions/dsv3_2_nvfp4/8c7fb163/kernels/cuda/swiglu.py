"""fused_swiglu on the B200 backend.
Contract: racetrack/models/deepseek.py:850-853 — (gate, up, *, fallback) -> Tensor."""
from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

fused_swiglu = ops.fused_swiglu
