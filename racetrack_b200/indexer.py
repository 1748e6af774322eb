"""The DeepSeek-V3.2 sparse-attention indexer on the B200 kernels.

Counterpart of `Indexer.forward` (racetrack/models/deepseek.py:656-686): which `index_topk`
cached keys each query attends to. The two projections are bf16 GEMMs (the fp32 head-weight
projection as two bf16 halves of its weight with fp32 accumulation), everything between them
and the scores is one fused kernel per operand (ops.index_prep), the scores come from the
tensor cores (ops.fp8_index) and the selection is an exact radix select (ops.index_topk).
Nothing reads device data back to the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


@dataclass
class IndexerWeights:
    """wq_b [heads * 128, q_lora] bf16, wk [128, dim] bf16, k_norm weight / bias fp32 [128],
    weights_proj [heads, dim] fp32 (racetrack/models/deepseek.py:644-648)."""
    wq_b: torch.Tensor
    wk: torch.Tensor
    k_norm_weight: torch.Tensor
    k_norm_bias: torch.Tensor
    weights_proj: torch.Tensor
    heads: int = 64
    head_dim: int = 128


def weights_of_module(indexer) -> IndexerWeights:
    """IndexerWeights of a racetrack `Indexer` module (racetrack/models/deepseek.py:634-654),
    converted once and cached on the module. FP8 checkpoint weights of wq_b / wk are dequantised
    with their block scales; weights_proj stays fp32 as the reference keeps it."""
    cached = getattr(indexer, "_rt_index_weights", None)
    if cached is None:
        cached = IndexerWeights(
            ops.module_weight_bf16(indexer.wq_b), ops.module_weight_bf16(indexer.wk),
            indexer.k_norm.weight.detach().float().contiguous(),
            indexer.k_norm.bias.detach().float().contiguous(),
            indexer.weights_proj.weight.detach().float().contiguous(),
            indexer.n_heads, indexer.head_dim)
        indexer._rt_index_weights = cached
    return cached


def write_k_cache(x: torch.Tensor, w: IndexerWeights, k_cache: torch.Tensor,
                  k_scale_cache: torch.Tensor, start_pos: int, freqs_cis: torch.Tensor,
                  positions: Optional[torch.Tensor] = None) -> None:
    """The key half of `Indexer.forward` alone (racetrack/models/deepseek.py:665-676): project,
    LayerNorm, non-interleaved RoPE, Hadamard rotation, FP8 quantisation, and the append to the
    caches at [start_pos, start_pos + S). x [B, S, dim] bf16; k_cache float8_e4m3fn
    [>= B, max_len, 128]; k_scale_cache fp32 [>= B, max_len] or [.., 1]; freqs_cis complex64
    [S, 32] (the rows of the tokens) unless `positions` names rows of a longer table. What the
    reference's full-top-k short-circuit runs so that later steps find valid cached keys
    (racetrack/pre_trace.py:82-112)."""
    bsz, s_len, _ = x.shape
    end_pos = start_pos + s_len
    if positions is None:
        positions = torch.arange(s_len, device=x.device, dtype=torch.int64)
    pos = positions.repeat(bsz) if positions.numel() == s_len else positions.reshape(-1)
    k = ops.linear_bf16(x.reshape(bsz * s_len, -1), w.wk).view(bsz * s_len, 1, w.head_dim)
    k_fp8, k_scale = ops.index_prep(k, freqs_cis, positions=pos, ln_weight=w.k_norm_weight,
                                    ln_bias=w.k_norm_bias)
    k_cache[:bsz, start_pos:end_pos] = k_fp8.view(bsz, s_len, w.head_dim)
    k_scale_cache[:bsz, start_pos:end_pos] = k_scale.view(bsz, s_len, *k_scale_cache.shape[2:])


def indexer_forward(x: torch.Tensor, qr: torch.Tensor, w: IndexerWeights, k_cache: torch.Tensor,
                    k_scale_cache: torch.Tensor, start_pos: int, freqs_cis: torch.Tensor,
                    index_topk: int, *, causal: bool = True,
                    positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [S, dim] and qr [S, q_lora] bf16 (one sequence); k_cache float8_e4m3fn [max_len, 128]
    and k_scale_cache fp32 [max_len] are updated in place at [start_pos, start_pos + S).
    freqs_cis complex64 [table, 32] for the whole position range. Returns int32
    [S, min(index_topk, start_pos + S)], ascending: the cached positions query s may attend to
    (with `causal`, only positions <= start_pos + s compete, as with the reference's mask)."""
    s_len = x.shape[0]
    end_pos = start_pos + s_len
    if positions is None:
        positions = torch.arange(start_pos, end_pos, device=x.device, dtype=torch.int64)
    q = ops.linear_bf16(qr, w.wq_b).view(s_len, w.heads, w.head_dim)
    q_fp8, q_scale = ops.index_prep(q, freqs_cis, positions=positions)
    k = ops.linear_bf16(x, w.wk).view(s_len, 1, w.head_dim)
    k_fp8, k_scale = ops.index_prep(k, freqs_cis, positions=positions,
                                    ln_weight=w.k_norm_weight, ln_bias=w.k_norm_bias)
    k_cache[start_pos:end_pos] = k_fp8.view(s_len, w.head_dim)
    k_scale_cache[start_pos:end_pos] = k_scale.view(s_len)
    # per-head weights in fp32, as the reference forms them (deepseek.py:677-678)
    head_w = ops.linear_f32_weight(x, w.weights_proj) * w.heads ** -0.5
    head_w = head_w * q_scale * w.head_dim ** -0.5
    scores = ops.fp8_index(q_fp8.unsqueeze(0), head_w.unsqueeze(0), k_cache[:end_pos].unsqueeze(0),
                           k_scale_cache[:end_pos].unsqueeze(0),
                           causal_offset=start_pos if causal else None)
    return ops.index_topk(scores[0], index_topk)



def indexer_decode(x: torch.Tensor, qr: torch.Tensor, w: IndexerWeights, k_cache: torch.Tensor,
                   k_scale_cache: torch.Tensor, start_pos: int, freqs_cis: torch.Tensor,
                   index_topk: int, *, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step of B sequences (the reference's bsz = B, seqlen = 1): x [B, dim] and qr
    [B, q_lora] bf16 hold the token of every sequence at position start_pos; k_cache
    float8_e4m3fn [B, max_len, 128] and k_scale_cache fp32 [B, max_len] are updated in place at
    start_pos. Returns int32 [B, min(index_topk, start_pos + 1)], ascending. Every kernel runs
    once for the whole batch. `positions` (int64 [B]) are the rows of freqs_cis to rotate by
    (default: start_pos for every sequence, i.e. freqs_cis is the whole table)."""
    batch = x.shape[0]
    end_pos = start_pos + 1
    if positions is None:
        positions = torch.full((batch,), start_pos, device=x.device, dtype=torch.int64)
    q = ops.linear_bf16(qr, w.wq_b).view(batch, w.heads, w.head_dim)
    q_fp8, q_scale = ops.index_prep(q, freqs_cis, positions=positions)
    k = ops.linear_bf16(x, w.wk).view(batch, 1, w.head_dim)
    k_fp8, k_scale = ops.index_prep(k, freqs_cis, positions=positions,
                                    ln_weight=w.k_norm_weight, ln_bias=w.k_norm_bias)
    k_cache[:, start_pos] = k_fp8.view(batch, w.head_dim)
    k_scale_cache[:, start_pos] = k_scale.view(batch)
    head_w = ops.linear_f32_weight(x, w.weights_proj) * w.heads ** -0.5
    head_w = head_w * q_scale.view(batch, w.heads) * w.head_dim ** -0.5
    scores = ops.fp8_index(q_fp8.view(batch, 1, w.heads, w.head_dim), head_w.view(batch, 1, w.heads),
                           k_cache[:, :end_pos], k_scale_cache[:, :end_pos])
    return ops.index_topk(scores.view(batch, end_pos), index_topk)
