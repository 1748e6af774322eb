"""fused_single_token_moe on the B200 backend: the whole MoE.forward of
racetrack/models/deepseek.py:998-1022 (gate, expert loop, shared experts, all-reduce) for any
number of tokens, with the routed experts evaluated as NVFP4 grouped GEMMs.
Contract: racetrack/pre_trace.py:182-187 — (moe, x, *, fallback) -> Tensor."""
import torch

from racetrack_b200 import _lib, moe as rt_moe, ops

BACKEND_AVAILABLE = _lib.available()


def _experts_of(moe):
    """NVFP4 copy of the module's local experts, built on first use and cached on the module.
    FP8 checkpoint weights (e4m3 codes + 128 x 128 block scales, racetrack/models/deepseek.py:
    361-371) are dequantised first, as the reference's weight_dequant does."""
    cached = getattr(moe, "_rt_nvfp4_experts", None)
    if cached is None:
        local = [e for e in moe.experts if e is not None]
        wb = ops.module_weight_bf16
        w13 = torch.stack([torch.cat((wb(e.w1), wb(e.w3))) for e in local])
        w2 = torch.stack([wb(e.w2) for e in local])
        cached = rt_moe.quantize_experts(w13, w2)
        moe._rt_nvfp4_experts = cached
    return cached


def fused_single_token_moe(moe, x, *, fallback):
    del fallback
    shape = x.size()
    x2 = x.view(-1, moe.dim)
    gate = moe.gate
    shared = moe.shared_experts(x2) if getattr(moe, "shared_experts", None) is not None else None
    dist = torch.distributed
    sharded = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    # an expert-parallel rank all-reduces its fp32 sums and casts afterwards
    # (racetrack/models/deepseek.py:1019-1022)
    y = rt_moe.fused_moe_forward(
        x2, gate.weight, gate.bias, _experts_of(moe), n_experts=moe.n_routed_experts,
        n_groups=gate.n_groups, topk_groups=gate.topk_groups, topk=gate.topk,
        route_scale=gate.route_scale, score_func=gate.score_func,
        expert_begin=getattr(moe, "experts_start_idx", 0), shared=shared,
        out_dtype=torch.float32 if sharded else torch.bfloat16)
    if sharded:
        dist.all_reduce(y)
        y = y.type_as(x)
    return y.view(shape)
