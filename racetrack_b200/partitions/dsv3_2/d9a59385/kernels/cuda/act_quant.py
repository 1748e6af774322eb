"""Activation quantisers on the B200 backend: FP8 e4m3 per-128 group (racetrack/models/deepseek.py:85-107;
wrapper contracts partitions/dsv3_2/3336cdbd/kernels/triton/act_quant.py:61-85) and NVFP4."""
from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

fused_act_quant = ops.fused_act_quant
fused_swiglu_quant = ops.fused_swiglu_quant
fused_nvfp4_quant = ops.fused_nvfp4_quant
fused_swiglu_nvfp4_quant = ops.fused_swiglu_nvfp4_quant
