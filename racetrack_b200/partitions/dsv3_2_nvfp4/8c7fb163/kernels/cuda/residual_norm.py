"""fused_residual_norm on the B200 backend.
Contract: racetrack/models/deepseek.py:485-505 — (update, residual, weight, *, eps, fallback)
-> (normed, hidden)."""
from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

fused_residual_norm = ops.fused_residual_norm
fused_rms_norm = ops.fused_rms_norm
