"""fused_norm_rope (q_a / kv_a RMSNorm + k_pe RoPE) and fused_rope on the B200 backend.
Contracts: partitions/dsv3_2/model.py:84-99,333-344 and
partitions/dsv3_2/3336cdbd/kernels/triton/rope.py:57-62."""
from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

fused_norm_rope = ops.fused_norm_rope
fused_rope = ops.fused_rope
