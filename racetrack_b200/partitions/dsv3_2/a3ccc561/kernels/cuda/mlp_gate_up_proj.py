"""fused_mlp_gate_up_proj on the B200 backend: gate and up projections of an MLP as ONE
tcgen05 GEMM against the concatenated [w1; w3] weight.
Contract: racetrack/pre_trace.py:216-220 — (x, w1_w, w1_s, w3_w, w3_s, *, scale_fmt, fallback)
-> (gate, up). bf16 weights only; FP8 block-scaled weights are refused."""
import torch

from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

_CAT: dict = {}


def fused_mlp_gate_up_proj(x, w1_w, w1_s, w3_w, w3_s, *, scale_fmt, fallback):
    del fallback, scale_fmt
    if w1_w.dtype != torch.bfloat16 or w1_s is not None or w3_s is not None:
        raise RuntimeError("fused_mlp_gate_up_proj: only bf16 weights are supported by this backend")
    key = (w1_w.data_ptr(), w3_w.data_ptr(), w1_w._version, w3_w._version)
    w13 = _CAT.get(key)
    if w13 is None:
        w13 = torch.cat((w1_w, w3_w)).contiguous()
        _CAT[key] = w13
    gate_up = ops.linear_bf16(x, w13)
    inter = w1_w.shape[0]
    return gate_up[..., :inter], gate_up[..., inter:]
