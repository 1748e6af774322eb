"""fused_mlp_gate_up_proj on the B200 backend: gate and up projections of an MLP as ONE
tcgen05 GEMM against the concatenated [w1; w3] weight - bf16 weights on the bf16 GEMM, FP8
e4m3 weights with 128 x 128 block scales on act_quant + the FP8 block-scaled GEMM.
Contract: racetrack/pre_trace.py:216-220 — (x, w1_w, w1_s, w3_w, w3_s, *, scale_fmt, fallback)
-> (gate, up)."""
import torch

from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

_CAT: dict = {}      # key -> ([w1; w3], its scales, w1, w3)


def _concat(w1_w, w1_s, w3_w, w3_s):
    key = (w1_w.data_ptr(), w3_w.data_ptr(), tuple(w1_w.shape), tuple(w3_w.shape), w1_w.dtype,
           w1_w._version, w3_w._version)
    hit = _CAT.get(key)
    if hit is None:
        w13 = torch.cat((w1_w, w3_w)).contiguous()
        s13 = None
        if w1_s is not None:
            if w1_w.shape[0] % 128:
                raise RuntimeError("fused_mlp_gate_up_proj: FP8 weights need out_features % 128 == 0")
            s13 = torch.cat((w1_s.float(), w3_s.float())).contiguous()
        # the entry holds the source weights, so their addresses stay theirs while it exists
        hit = (w13, s13, w1_w.detach(), w3_w.detach())
        while len(_CAT) >= 1024:
            _CAT.pop(next(iter(_CAT)))
        _CAT[key] = hit
    return hit[0], hit[1]


def fused_mlp_gate_up_proj(x, w1_w, w1_s, w3_w, w3_s, *, scale_fmt, fallback):
    del fallback, scale_fmt
    fp8 = w1_w.dtype == torch.float8_e4m3fn
    if fp8 != (w1_s is not None) or (not fp8 and w1_w.dtype != torch.bfloat16):
        raise RuntimeError("fused_mlp_gate_up_proj: weights must be bf16, or e4m3fn with block scales")
    w13, s13 = _concat(w1_w, w1_s, w3_w, w3_s)
    gate_up = ops.linear_fp8_act(x, w13, s13) if fp8 else ops.linear_bf16(x, w13)
    inter = w1_w.shape[0]
    return gate_up[..., :inter], gate_up[..., inter:]
