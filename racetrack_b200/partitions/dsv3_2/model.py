"""Synthetic flattened DeepSeek-V3.2 baseline: the model a dsv3_2 partition is swapped into.

Counterpart of racetrack's partitions/dsv3_2/model.py (config :162-221, ops :27-126, modules
:229-563, ``build_model`` :566-568) with the same public surface - ``DeepSeekConfig``,
``DSV3_2_CONFIG``, ``FlattenedDeepSeekModel(config, partition_root=...)``, ``build_model(**overrides)``
- and the same dispatch point: the MLA block calls
``dispatcher.call("fused_norm_rope", fused_norm_rope, q_c, q_w, kv_c, kv_w, k_pe, positions, eps=, rope_base=)``
(:333-344). Without a partition root every op is the vanilla torch function below, which makes
this file the "torch" row a partition is raced against. The hyper-connection branch
(``hc_mult > 1``) of the reference is not carried: DeepSeek-V3.2 runs with hc_mult = 1.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from pathlib import Path

import torch
import torch.nn.functional as F
from torch import nn

from racetrack_b200.dispatch import KernelDispatcher

MODEL_NAME = "dsv3_2"


# ---------------------------------------------------------------------------
# vanilla torch ops (the fallbacks handed to the dispatcher)
# ---------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def rope_cache(positions: torch.Tensor, rotary_dim: int, *, base: float = 10000.0, dtype=None):
    half = rotary_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, device=positions.device, dtype=torch.float32)
                               / max(half, 1)))
    angles = positions.float().unsqueeze(-1) * inv_freq.unsqueeze(0)
    cos, sin = torch.cos(angles), torch.sin(angles)
    return (cos.to(dtype), sin.to(dtype)) if dtype is not None else (cos, sin)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, *, rotary_dim: int | None = None,
               base: float = 10000.0) -> torch.Tensor:
    rotary_dim = x.shape[-1] if rotary_dim is None else rotary_dim
    if rotary_dim == 0:
        return x
    if rotary_dim % 2 or rotary_dim > x.shape[-1]:
        raise ValueError(f"bad rotary_dim {rotary_dim} for a tensor of width {x.shape[-1]}")
    cos, sin = rope_cache(positions, rotary_dim, base=base, dtype=x.dtype)
    half = rotary_dim // 2
    x1, x2, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
    while cos.dim() < x1.dim():
        cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
    parts = [x1 * cos - x2 * sin, x2 * cos + x1 * sin]
    if rest.numel():
        parts.append(rest)
    return torch.cat(parts, dim=-1)


def fused_norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, positions, *, eps: float, rope_base: float):
    return (rms_norm(q_c, q_weight, eps), rms_norm(kv_c, kv_weight, eps),
            apply_rope(k_pe, positions, base=rope_base))


def causal_attention(q, k, v, *, softmax_scale: float | None = None, causal_mask=None):
    scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
    scores = torch.einsum("thd,shd->hts", q.float(), k.float()) * scale
    if causal_mask is None:
        t = q.shape[0]
        causal_mask = torch.ones(t, t, device=q.device, dtype=torch.bool).tril()
    scores = scores.masked_fill(~causal_mask.unsqueeze(0), -float("inf"))
    return torch.einsum("hts,shd->thd", torch.softmax(scores, dim=-1).to(v.dtype), v)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


# ---------------------------------------------------------------------------
# config
# ---------------------------------------------------------------------------

@dataclass(frozen=True)
class DeepSeekConfig:
    name: str
    source: str
    vocab_size: int = 8192
    hidden_size: int = 512
    num_layers: int = 2
    num_attention_heads: int = 8
    head_dim: int = 64
    qk_nope_head_dim: int | None = None
    v_head_dim: int | None = None
    q_lora_rank: int = 128
    kv_lora_rank: int = 128
    qk_rope_head_dim: int = 16
    intermediate_size: int = 1024
    moe_intermediate_size: int = 384
    n_routed_experts: int = 8
    num_experts_per_tok: int = 2
    n_shared_experts: int = 1
    rms_norm_eps: float = 1.0e-6
    rope_base: float = 10000.0
    routed_scaling_factor: float = 1.0
    hc_mult: int = 1
    seed: int = 1234

    @property
    def resolved_qk_nope_head_dim(self) -> int:
        return self.qk_nope_head_dim if self.qk_nope_head_dim is not None \
            else self.head_dim - self.qk_rope_head_dim

    @property
    def resolved_v_head_dim(self) -> int:
        return self.v_head_dim if self.v_head_dim is not None else self.head_dim

    def for_benchmark(self, **overrides) -> "DeepSeekConfig":
        return replace(self, **overrides)


DSV3_2_CONFIG = DeepSeekConfig(name="dsv3_2", source="synthetic DeepSeek-V3.2 shape, reduced width",
                               seed=38595)


# ---------------------------------------------------------------------------
# modules
# ---------------------------------------------------------------------------

class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x):
        return rms_norm(x, self.weight, self.eps)


class SwiGLUExpert(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.w1 = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.w3 = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.w2 = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class RoutedMoE(nn.Module):
    """Dense evaluation of every expert, weighted by the top-k softmax routing weights."""

    def __init__(self, config: DeepSeekConfig):
        super().__init__()
        self.config = config
        self.gate = nn.Linear(config.hidden_size, config.n_routed_experts, bias=False)
        self.experts = nn.ModuleList(SwiGLUExpert(config.hidden_size, config.moe_intermediate_size)
                                     for _ in range(config.n_routed_experts))
        self.shared = SwiGLUExpert(config.hidden_size,
                                   config.moe_intermediate_size * config.n_shared_experts) \
            if config.n_shared_experts else None

    def forward(self, hidden_states, input_ids=None):
        del input_ids
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        logits = F.linear(x.float(), self.gate.weight.float())
        top_logits, top_ids = torch.topk(logits, self.config.num_experts_per_tok, dim=-1)
        top_w = torch.softmax(top_logits, dim=-1).to(x.dtype)
        out = torch.zeros_like(x)
        for e, expert in enumerate(self.experts):
            w = ((top_ids == e).to(x.dtype) * top_w).sum(dim=-1, keepdim=True)
            out = out + expert(x) * w
        if self.shared is not None:
            out = out + self.shared(x)
        return (out * self.config.routed_scaling_factor).view(shape)


class FlattenedMLAAttention(nn.Module):
    def __init__(self, config: DeepSeekConfig, dispatcher: KernelDispatcher | None = None):
        super().__init__()
        self.config, self.dispatcher = config, dispatcher
        self.nope_dim = config.resolved_qk_nope_head_dim
        self.v_head_dim = config.resolved_v_head_dim
        self.qk_head_dim = self.nope_dim + config.qk_rope_head_dim
        heads = config.num_attention_heads
        self.fused_qkv_a_proj = nn.Linear(
            config.hidden_size, config.q_lora_rank + config.kv_lora_rank + config.qk_rope_head_dim,
            bias=False)
        self.q_a_layernorm_weight = nn.Parameter(torch.ones(config.q_lora_rank))
        self.kv_a_layernorm_weight = nn.Parameter(torch.ones(config.kv_lora_rank))
        self.q_b_proj = nn.Linear(config.q_lora_rank, heads * self.qk_head_dim, bias=False)
        self.kv_b_proj = nn.Linear(config.kv_lora_rank, heads * (self.nope_dim + self.v_head_dim),
                                   bias=False)
        self.o_proj = nn.Linear(heads * self.v_head_dim, config.hidden_size, bias=False)

    def forward(self, hidden_states, positions, causal_mask=None):
        c = self.config
        qkv = self.fused_qkv_a_proj(hidden_states)
        q_c, kv_c, k_pe = qkv.split([c.q_lora_rank, c.kv_lora_rank, c.qk_rope_head_dim], dim=-1)
        args = (q_c, self.q_a_layernorm_weight, kv_c, self.kv_a_layernorm_weight, k_pe, positions)
        kw = dict(eps=c.rms_norm_eps, rope_base=c.rope_base)
        if self.dispatcher is None:
            q_c, kv_c, k_pe = fused_norm_rope(*args, **kw)
        else:
            q_c, kv_c, k_pe = self.dispatcher.call("fused_norm_rope", fused_norm_rope, *args, **kw)
        tokens, heads = hidden_states.shape[0], c.num_attention_heads
        q = self.q_b_proj(q_c).view(tokens, heads, self.qk_head_dim)
        q_nope, q_pe = q.split([self.nope_dim, c.qk_rope_head_dim], dim=-1)
        q = torch.cat((q_nope, apply_rope(q_pe, positions, base=c.rope_base)), dim=-1)
        kv = self.kv_b_proj(kv_c).view(tokens, heads, self.nope_dim + self.v_head_dim)
        k_nope, v = kv.split([self.nope_dim, self.v_head_dim], dim=-1)
        k = torch.cat((k_nope, k_pe.unsqueeze(1).expand(-1, heads, -1)), dim=-1)
        out = causal_attention(q, k, v, causal_mask=causal_mask)
        return self.o_proj(out.reshape(tokens, heads * self.v_head_dim))


class FlattenedDeepSeekBlock(nn.Module):
    def __init__(self, config: DeepSeekConfig, dispatcher: KernelDispatcher | None = None):
        super().__init__()
        self.config, self.dispatcher = config, dispatcher
        self.attn_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.ffn_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.attn = FlattenedMLAAttention(config, dispatcher)
        self.ffn = RoutedMoE(config)

    def forward(self, hidden_states, positions, input_ids, causal_mask=None):
        hidden_states = hidden_states + self.attn(self.attn_norm(hidden_states), positions, causal_mask)
        return hidden_states + self.ffn(self.ffn_norm(hidden_states), input_ids)


class FlattenedDeepSeekModel(nn.Module):
    def __init__(self, config: DeepSeekConfig, *, partition_root: str | Path | None = None):
        super().__init__()
        self.config = config
        self.dispatcher = KernelDispatcher(Path(partition_root) / "kernels") \
            if partition_root is not None else None
        with torch.random.fork_rng(devices=[]):
            torch.manual_seed(config.seed)
            self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
            self.layers = nn.ModuleList(FlattenedDeepSeekBlock(config, self.dispatcher)
                                        for _ in range(config.num_layers))
            self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
            self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    @property
    def backend_status(self) -> dict[str, str]:
        status = {"torch": "native"}
        if self.dispatcher is not None:
            status["cuda"] = self.dispatcher.backend_status("cuda")
        return status

    def forward(self, input_ids, positions=None):
        flat = input_ids.reshape(-1)
        if positions is None:
            positions = torch.arange(flat.numel(), device=flat.device, dtype=torch.long)
        else:
            positions = positions.reshape(-1).to(device=flat.device, dtype=torch.long)
        hidden = self.embed_tokens(flat)
        for layer in self.layers:
            hidden = layer(hidden, positions, flat)
        return self.lm_head(self.norm(hidden))


def build_model(**overrides) -> FlattenedDeepSeekModel:
    return FlattenedDeepSeekModel(DSV3_2_CONFIG.for_benchmark(**overrides))
