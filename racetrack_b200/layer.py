"""Synthetic full-size DeepSeek-V3.2 layer on the B200 kernels: the counterpart of
racetrack/realistic_bench.py:118-427 (ShardedRealisticBlock / ShardedRealisticModel).

Same structure and sharding as the reference runner: one layer's weights reused for every layer
of the stack; attention heads tensor-parallel (w_q_b / w_kv_b column-sharded, w_o row-sharded,
all-reduce after w_o); routed experts expert-parallel (each rank owns a contiguous slice, tokens
replicated, all-reduce after the combine); router replicated. Per layer:

    rms_norm -> qkv_a GEMM -> fused q_a/kv_a RMSNorm + k_pe RoPE -> q_b GEMM -> q_pe RoPE (in place)
    -> kv_b GEMM -> causal attention over the local heads (tcgen05) -> w_o GEMM -> all-reduce
    -> fused residual-add + rms_norm -> router GEMM (fp32) -> routing kernel -> NVFP4 grouped
    expert GEMMs with SwiGLU -> weighted combine -> all-reduce -> residual add (fused with the
    next layer's first rms_norm)

Dense projections run on the bf16 tcgen05 GEMM, experts on the NVFP4 block-scaled grouped GEMM,
everything element-wise on the fused kernels of ops.py, the attention core (QK^T, softmax, PV) on
the causal attention kernel of this library (ops.attention_prefill).

Unlike the reference, which seeds each rank's weights with seed + rank (so a 2-rank model is a
different model from a 1-rank one), weights here are defined per shard unit (one eighth of the
heads, one expert) and a rank draws the units it owns: every world size computes the same layer.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import torch
import torch.nn.functional as F

from . import moe, ops


@dataclass(frozen=True)
class LayerShape:
    """Dimensions of racetrack/realistic_bench.py:62-82 (realistic_shape("dsv3_2"))."""
    name: str = "dsv3_2"
    hidden: int = 7168
    heads: int = 128
    q_lora: int = 1536
    kv_lora: int = 512
    nope: int = 128
    rope: int = 64
    v_dim: int = 128
    moe_inter: int = 2048
    n_experts: int = 256
    topk: int = 8
    dense_inter: int = 18432
    eps: float = 1.0e-6
    rope_base: float = 10000.0
    seed: int = 38595
    units: int = 8           # shard granularity of heads and of the dense FFN

    @property
    def qk_dim(self) -> int:
        return self.nope + self.rope

    def scaled(self, **kw) -> "LayerShape":
        return replace(self, **kw)


DSV32 = LayerShape()


def _draw(shape, seed: int, std: float, device, dtype) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.empty(shape, device=device, dtype=torch.float32 if str(device) == "cpu" else dtype)
    w.normal_(mean=0.0, std=std, generator=g)
    return w.to(dtype)


def draw_expert(shape: LayerShape, e: int, device, *, std: float = 0.02,
                dtype: torch.dtype = torch.bfloat16):
    """(w13 [2I, H], w2 [H, I]) of routed expert `e`; the same values whatever rank draws them."""
    s = shape
    return (_draw((2 * s.moe_inter, s.hidden), s.seed + 10000 + 2 * e, std, device, dtype),
            _draw((s.hidden, s.moe_inter), s.seed + 10001 + 2 * e, std, device, dtype))


def make_weights(shape: LayerShape, rank: int, world: int, device, *, ffn: str = "moe",
                 std: float = 0.02, dtype: torch.dtype = torch.bfloat16) -> dict:
    """The weights rank `rank` of `world` owns, drawn unit by unit (see the module docstring).
    Keys: w_qkv_a [q+kv+rope, H]; w_q_b [h_loc*(nope+rope), q]; w_kv_b [h_loc*(nope+v), kv];
    w_o [H, h_loc*v]; w_gate [E, H]; w13 [E_loc, 2I, H], w2 [E_loc, H, I] (ffn == "moe") or
    w1, w3 [I_loc, H], w2d [H, I_loc] (ffn == "dense")."""
    if shape.units % world or shape.n_experts % world:
        raise ValueError("world size must divide the shard units and the expert count")
    s = shape
    hpu = s.heads // s.units                     # heads per unit
    units = range(rank * s.units // world, (rank + 1) * s.units // world)
    seed = s.seed
    w = {"w_qkv_a": _draw((s.q_lora + s.kv_lora + s.rope, s.hidden), seed + 1, std, device, dtype),
         "w_gate": _draw((s.n_experts, s.hidden), seed + 100000, std, device, dtype)}
    w["w_q_b"] = torch.cat([_draw((hpu * s.qk_dim, s.q_lora), seed + 100 + u, std, device, dtype)
                            for u in units])
    w["w_kv_b"] = torch.cat([_draw((hpu * (s.nope + s.v_dim), s.kv_lora), seed + 200 + u, std, device, dtype)
                             for u in units])
    w["w_o"] = torch.cat([_draw((s.hidden, hpu * s.v_dim), seed + 300 + u, std, device, dtype)
                          for u in units], dim=1)
    if ffn == "moe":
        e_loc = s.n_experts // world
        experts = [draw_expert(s, e, device, std=std, dtype=dtype)
                   for e in range(rank * e_loc, (rank + 1) * e_loc)]
        w["w13"] = torch.stack([e[0] for e in experts])
        w["w2"] = torch.stack([e[1] for e in experts])
    elif ffn == "dense":
        ipu = s.dense_inter // s.units
        w["w1"] = torch.cat([_draw((ipu, s.hidden), seed + 400 + u, std, device, dtype) for u in units])
        w["w3"] = torch.cat([_draw((ipu, s.hidden), seed + 500 + u, std, device, dtype) for u in units])
        w["w2d"] = torch.cat([_draw((s.hidden, ipu), seed + 600 + u, std, device, dtype) for u in units], dim=1)
    return w


def make_nvfp4_experts(shape: LayerShape, rank: int, world: int, device, *,
                       std: float = 0.02) -> "moe.NVFP4Experts":
    """The rank's routed experts drawn and quantised one at a time, so that the bf16 weights of
    only one expert exist at any moment (all 256 experts in bf16 would take 22.5 GB)."""
    s = shape
    e_loc = s.n_experts // world
    parts13, parts2 = [], []
    for e in range(rank * e_loc, (rank + 1) * e_loc):
        w13, w2 = draw_expert(s, e, device, std=std)
        parts13.append(ops.fused_nvfp4_quant(w13, tiled_scales=True))
        parts2.append(ops.fused_nvfp4_quant(w2, tiled_scales=True))
    cat = torch.cat
    return moe.NVFP4Experts(
        e_loc, s.hidden, s.moe_inter,
        cat([p[0] for p in parts13]), cat([p[1].view(torch.uint8) for p in parts13]),
        cat([p[2] for p in parts13]),
        cat([p[0] for p in parts2]), cat([p[1].view(torch.uint8) for p in parts2]),
        cat([p[2] for p in parts2]))


# "rt": the causal attention kernel of this library (ops.attention_prefill, tcgen05);
# "sdpa": torch's scaled_dot_product_attention, kept only as the yardstick the kernel is
# measured against (a library kernel, not part of the backend).
ATTENTION_CORE = "rt"


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Causal softmax(q k^T / sqrt(d)) v over [T, H, D] tensors -> [T, H, Dv]
    (racetrack/runtime/torch_ops.py:97-110) through torch SDPA (the yardstick, see
    ATTENTION_CORE); when the value width differs from the query width and the fused kernels
    refuse that, v is zero-padded to the query width."""
    qt, kt, vt = (t.transpose(0, 1).unsqueeze(0) for t in (q, k, v))
    try:
        out = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
    except RuntimeError:
        pad = q.shape[-1] - v.shape[-1]
        out = F.scaled_dot_product_attention(qt, kt, F.pad(vt, (0, pad)), is_causal=True)[..., :v.shape[-1]]
    return out.squeeze(0).transpose(0, 1)


class Projection:
    """A dense projection y = x W^T held either in bf16 or as FP8 e4m3 with 128 x 128 block
    scales (racetrack/models/deepseek.py:316-345 `linear`: bf16 weights go to F.linear, FP8
    weights to act_quant + fp8_gemm). FP8 needs K % 128 == 0; other widths stay bf16.
    dtype "mixed" keeps FP8 for the long reductions only (K >= MIXED_FP8_MIN_K): the FP8 GEMM
    rescales every 128-wide K block in registers, which pays off against the bf16 CTA-pair
    GEMM only when the tensor core has long K loops to hide it behind."""

    MIXED_FP8_MIN_K = 4096

    def __init__(self, weight: torch.Tensor, dtype: str):
        k = weight.shape[1]
        self.fp8 = k % 128 == 0 and (dtype == "fp8" or (dtype == "mixed" and k >= self.MIXED_FP8_MIN_K))
        if self.fp8:
            self.codes, self.scales = ops.quantize_weight_fp8(weight)
        else:
            self.weight = weight.contiguous()

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.fp8:
            return ops.linear_fp8_act(x, self.codes, self.scales)
        return ops.linear_bf16(x, self.weight)


class RealisticLayer:
    """One rank's shard of the synthetic layer; `forward_stack` applies it `layers` times.
    proj = "bf16" | "fp8" | "mixed" selects the arithmetic of the dense projections."""

    def __init__(self, shape: LayerShape, weights: dict, rank: int = 0, world: int = 1, *,
                 ffn: str = "moe", route: str = "topk_softmax", proj: str = "bf16",
                 process_group=None):
        self.shape, self.rank, self.world, self.ffn, self.route = shape, rank, world, ffn, route
        self.group, self.proj = process_group, proj
        self.local_heads = shape.heads // world
        dev = weights["w_qkv_a"].device
        self.w_qkv_a = Projection(weights["w_qkv_a"], proj)
        self.w_q_b = Projection(weights["w_q_b"], proj)
        s = shape
        self.attn_core = ATTENTION_CORE
        if self.attn_core == "rt":
            # K and V are column slices of the kv_b output; the attention kernel takes the
            # rope key as an operand of its own, one row per token for all heads
            self.w_kv_b = Projection(weights["w_kv_b"], proj)
        else:
            # kv_b rows regrouped per head as [k_nope | rope-wide gap (zero rows) | v]: the GEMM
            # then leaves room for k_pe right behind k_nope (a whole-key tensor for SDPA)
            wkv = weights["w_kv_b"].view(self.local_heads, s.nope + s.v_dim, s.kv_lora)
            gap = torch.zeros(self.local_heads, s.rope, s.kv_lora, device=dev, dtype=wkv.dtype)
            self.w_kv_b = Projection(
                torch.cat((wkv[:, :s.nope], gap, wkv[:, s.nope:]), dim=1)
                .reshape(self.local_heads * (s.nope + s.rope + s.v_dim), s.kv_lora), proj)
        self.w_o = Projection(weights["w_o"], proj)
        self.w_gate = weights["w_gate"].contiguous()
        self.ones_h = torch.ones(shape.hidden, device=dev, dtype=torch.bfloat16)
        self.q_norm = torch.ones(shape.q_lora, device=dev, dtype=torch.bfloat16)
        self.kv_norm = torch.ones(shape.kv_lora, device=dev, dtype=torch.bfloat16)
        if ffn == "moe":
            self.local_experts = shape.n_experts // world
            self.experts = weights["experts"] if "experts" in weights else \
                moe.quantize_experts(weights["w13"], weights["w2"])
        else:
            self.w13d = Projection(torch.cat([weights["w1"], weights["w3"]]), proj)
            self.w2d = Projection(weights["w2d"], proj)

    # -- pieces ---------------------------------------------------------------------------
    reduce = True   # set False to get this rank's partial sums (single-process checks)

    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1 and self.reduce:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def attention(self, normed: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """racetrack/realistic_bench.py:286-317."""
        s, h = self.shape, self.local_heads
        tokens = normed.shape[0]
        qkv = self.w_qkv_a(normed)
        q_c, kv_c, k_pe = ops.fused_norm_rope(
            qkv[:, :s.q_lora], self.q_norm, qkv[:, s.q_lora:s.q_lora + s.kv_lora], self.kv_norm,
            qkv[:, s.q_lora + s.kv_lora:], positions, eps=s.eps, rope_base=s.rope_base)
        q = self.w_q_b(q_c).view(tokens, h, s.qk_dim)
        ops.fused_rope_half(q[..., s.nope:], positions, rope_base=s.rope_base, inplace=True)
        if self.attn_core == "rt":
            kv = self.w_kv_b(kv_c).view(tokens, h, s.nope + s.v_dim)
            local = ops.attention_prefill(q, kv[..., :s.nope], k_pe, kv[..., s.nope:])
        else:
            kv = self.w_kv_b(kv_c).view(tokens, h, s.qk_dim + s.v_dim)
            ops.head_broadcast_(kv[..., s.nope:s.qk_dim], k_pe)       # K = [k_nope | k_pe] in place
            local = attention_core(q, kv[..., :s.qk_dim], kv[..., s.qk_dim:])
        out = self.w_o(local.reshape(tokens, h * s.v_dim))
        return self._all_reduce(out)

    def ffn_forward(self, normed: torch.Tensor) -> torch.Tensor:
        """racetrack/realistic_bench.py:319-352 (routed experts) or a dense SwiGLU FFN."""
        s = self.shape
        if self.ffn == "moe":
            # fp32 router logits of bf16 operands: tensor cores with the fp32 accumulators kept
            logits = ops.linear_bf16(normed, self.w_gate, out_dtype=torch.float32)
            if self.route == "topk_softmax":
                weights, indices = ops.fused_moe_route(logits, None, n_groups=1, topk_groups=1,
                                                       topk=s.topk, route_scale=1.0,
                                                       score_func="topk_softmax")
            else:
                raise ValueError(f"unknown route {self.route!r}")
            out = moe.fused_moe_experts(normed, weights, indices, self.experts,
                                        n_experts=s.n_experts,
                                        expert_begin=self.rank * self.local_experts)
        else:
            gate_up = self.w13d(normed)
            inter = gate_up.shape[1] // 2
            if self.w2d.fp8:     # SwiGLU and the FP8 quantisation of its result in one kernel
                codes, scales = ops.fused_swiglu_quant(gate_up[:, :inter], gate_up[:, inter:])
                out = ops.linear_fp8(codes, scales, self.w2d.codes, self.w2d.scales)
            else:
                out = self.w2d(ops.fused_swiglu(gate_up[:, :inter], gate_up[:, inter:]))
        return self._all_reduce(out)

    # -- the stack ----------------------------------------------------------------------------
    def forward_stack(self, hidden: torch.Tensor, positions: torch.Tensor, layers: int) -> torch.Tensor:
        """hidden [T, H] bf16 -> hidden after `layers` applications of the layer
        (racetrack/realistic_bench.py:354-389,420-423)."""
        s = self.shape
        normed = ops.fused_rms_norm(hidden, self.ones_h, eps=s.eps)
        for layer in range(layers):
            attn = self.attention(normed, positions)
            normed, hidden = ops.fused_residual_norm(attn, hidden, self.ones_h, eps=s.eps)
            ffn = self.ffn_forward(normed)
            # the add closing this layer and the rms_norm opening the next one, in one pass
            normed, hidden = ops.fused_residual_norm(ffn, hidden, self.ones_h, eps=s.eps)
        return hidden
