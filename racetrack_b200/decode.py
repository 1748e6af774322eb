"""Decode step of the synthetic DeepSeek-V3.2 layer on the B200 kernels: B sequences, one new
token each, per-sequence caches of `cache_len` positions, DSA sparse attention.

Counterpart of the reference's "MQA decode" branch (racetrack/models/deepseek.py:766-778,793-811):
the latent and rope caches are appended, the query is absorbed through the key half of wkv_b,
the indexer (racetrack/models/deepseek.py:656-686) picks `index_topk` cached positions per
sequence, attention runs over those rows only (ops.mla_sparse_decode, tcgen05), the value half
of wkv_b and wo follow, and the head-parallel partial sums are all-reduced. The feed-forward
half is the routed NVFP4 expert MLP of racetrack_b200.layer, expert-parallel.

The two absorbed projections are per-head products of a [B, 128] by [128, 512] shape, all heads
in one launch of the batched bf16 GEMM (ops.linear_bf16_batched), on the raw bf16 halves of
w_kv_b whatever `proj` says (the reference dequantises wkv_b before its einsums too,
racetrack/models/deepseek.py:795-798). Nothing reads device data back to the host, so a step can
be captured in a CUDA graph.

RoPE conventions: the layer's own q_pe / k_pe use the half-split rotation of the synthetic runner
this layer mirrors (racetrack/realistic_bench.py:297-303, partitions/dsv3_2/model.py:27-81),
prefill and decode alike, so a cache written by one is read correctly by the other; the indexer
inside the same step uses the reference model's complex table (non-interleaved pairs,
racetrack/models/deepseek.py:662-669). The real model's MLA branch rotates interleaved pairs
(:769-773); `ops.fused_rope` / `ops.fused_norm_rope_interleaved` are that convention.
"""
from __future__ import annotations


import torch

from . import indexer, ops
from .layer import LayerShape, RealisticLayer, _draw

INDEX_HEADS = 64
INDEX_DIM = 128
INDEX_TOPK = 2048


def make_indexer_weights(shape: LayerShape, device, *, std: float = 0.02) -> indexer.IndexerWeights:
    """The indexer's weights (replicated on every rank, as in the reference where they are plain
    Linear layers): wq_b [64 * 128, q_lora], wk [128, hidden] bf16 ~ N(0, std), LayerNorm weight
    1 / bias 0, weights_proj [64, hidden] fp32 ~ N(0, std)."""
    s = shape
    return indexer.IndexerWeights(
        _draw((INDEX_HEADS * INDEX_DIM, s.q_lora), s.seed + 700001, std, device, torch.bfloat16),
        _draw((INDEX_DIM, s.hidden), s.seed + 700002, std, device, torch.bfloat16),
        torch.ones(INDEX_DIM, device=device), torch.zeros(INDEX_DIM, device=device),
        _draw((INDEX_HEADS, s.hidden), s.seed + 700003, std, device, torch.float32),
        INDEX_HEADS, INDEX_DIM)


def rope_table(rope_dim: int, positions: int, base: float, device) -> torch.Tensor:
    """complex64 [positions, rope_dim / 2]: e^(i p base^(-2j / rope_dim))
    (racetrack/models/deepseek.py:523-601 without the long-context correction, which only
    applies beyond 4096 positions)."""
    freqs = 1.0 / (base ** (torch.arange(0, rope_dim, 2, dtype=torch.float32, device=device) / rope_dim))
    ang = torch.outer(torch.arange(positions, dtype=torch.float32, device=device), freqs)
    return torch.polar(torch.ones_like(ang), ang)


class DecodeCaches:
    """Per-sequence caches of one layer: latent kv [B, L, kv_lora] and rope keys [B, L, rope] in
    bf16, the indexer's keys [B, L, 128] in e4m3 with one fp32 scale per key."""

    def __init__(self, shape: LayerShape, batch: int, cache_len: int, device, *, seed: int = 0,
                 fill: int = 0):
        s = shape
        self.kv = torch.zeros(batch, cache_len, s.kv_lora, device=device, dtype=torch.bfloat16)
        self.pe = torch.zeros(batch, cache_len, s.rope, device=device, dtype=torch.bfloat16)
        self.index_k = torch.zeros(batch, cache_len, INDEX_DIM, device=device, dtype=torch.float8_e4m3fn)
        self.index_scale = torch.zeros(batch, cache_len, device=device, dtype=torch.float32)
        if fill:
            # positions [0, fill) ~ N(0, 1), as a context that was decoded earlier
            g = torch.Generator(device=device)
            g.manual_seed(s.seed + 900000 + seed)
            self.kv[:, :fill].normal_(generator=g)
            self.pe[:, :fill].normal_(generator=g)
            keys = torch.empty(batch * fill, INDEX_DIM, device=device, dtype=torch.bfloat16)
            keys.normal_(generator=g)
            codes, scales = ops.fused_act_quant(keys)
            self.index_k[:, :fill] = codes.view(batch, fill, INDEX_DIM)
            self.index_scale[:, :fill] = scales.view(batch, fill)


class DecodeLayer(RealisticLayer):
    """One rank's shard of the layer in decode mode; `decode_stack` applies it `layers` times to
    the B new tokens at position `start_pos` (the reference reuses one layer for the whole stack,
    racetrack/realistic_bench.py:420-423, so the caches are this one layer's)."""

    def __init__(self, shape: LayerShape, weights: dict, rank: int = 0, world: int = 1, *,
                 index_weights: indexer.IndexerWeights, caches: DecodeCaches,
                 index_topk: int = INDEX_TOPK, route: str = "topk_softmax", proj: str = "bf16",
                 process_group=None):
        super().__init__(shape, weights, rank, world, ffn="moe", route=route, proj=proj,
                         process_group=process_group)
        s, h = shape, self.local_heads
        wkv = weights["w_kv_b"].view(h, s.nope + s.v_dim, s.kv_lora)
        # per-head operands of the two absorbed projections, K-major for the batched GEMM
        self.w_uk_t = wkv[:, :s.nope].transpose(1, 2).contiguous()    # [h, kv_lora, nope]: q_nope -> latent
        self.w_uv = wkv[:, s.nope:].contiguous()                       # [h, v, kv_lora]: latent -> v
        self.w_kv_b = None          # the prefill form of this projection is never used by a decode step
        self.index_weights, self.caches, self.index_topk = index_weights, caches, index_topk
        self.softmax_scale = s.qk_dim ** -0.5
        self.freqs = rope_table(s.rope, caches.kv.shape[1], s.rope_base, weights["w_qkv_a"].device)

    def decode_attention(self, normed: torch.Tensor, start_pos: int,
                         out: torch.Tensor | None = None) -> torch.Tensor:
        """The attention half of a decode step; with `out` (an exchange buffer the other ranks
        read) this rank's partial sum is left there and not reduced."""
        s, h, c = self.shape, self.local_heads, self.caches
        batch = normed.shape[0]
        end = start_pos + 1
        positions = torch.full((batch,), start_pos, device=normed.device, dtype=torch.int64)
        qkv = self.w_qkv_a(normed)
        q_c, kv_c, k_pe = ops.fused_norm_rope(
            qkv[:, :s.q_lora], self.q_norm, qkv[:, s.q_lora:s.q_lora + s.kv_lora], self.kv_norm,
            qkv[:, s.q_lora + s.kv_lora:], positions, eps=s.eps, rope_base=s.rope_base)
        q = self.w_q_b(q_c).view(batch, h, s.qk_dim)
        ops.fused_rope_half(q[..., s.nope:], positions, rope_base=s.rope_base, inplace=True)
        c.kv[:, start_pos] = kv_c
        c.pe[:, start_pos] = k_pe
        # absorbed query: q_nope . W_UK per head (deepseek.py:799)
        q_abs = ops.linear_bf16_batched(q[..., :s.nope], self.w_uk_t)                    # [B, h, kv_lora]
        picked = indexer.indexer_decode(normed, q_c, self.index_weights, c.index_k, c.index_scale,
                                        start_pos, self.freqs, self.index_topk)
        latent = ops.mla_sparse_decode(q_abs, q[..., s.nope:], c.kv[:, :end], c.pe[:, :end], picked,
                                       self.softmax_scale)                                 # [B, h, kv_lora]
        heads_out = ops.linear_bf16_batched(latent, self.w_uv)                          # [B, h, v]
        if out is not None:
            return self.w_o(heads_out.reshape(batch, h * s.v_dim), out=out)
        return self._all_reduce(self.w_o(heads_out.reshape(batch, h * s.v_dim)))

    def _decode_exchange(self, batch: int):
        """The two [B, H] partial-sum buffers of this batch size, mapped across the ranks once."""
        from . import peer
        key = ("decode", batch)
        px = self._peer.get(key)
        if px is None:
            shape = (batch, self.shape.hidden)
            px = peer.PeerExchange(self.comm, self.ones_h.device,
                                   {"attn": (shape, torch.bfloat16), "ffn": (shape, torch.bfloat16)})
            self._peer[key] = px
        return px

    def decode_stack(self, hidden: torch.Tensor, start_pos: int, layers: int) -> torch.Tensor:
        """hidden [B, H] bf16 (the new token of every sequence) -> hidden after `layers`
        applications of the layer."""
        s = self.shape
        normed = ops.fused_rms_norm(hidden, self.ones_h, eps=s.eps)
        px = None
        if self.world > 1 and self.reduce and self.peer_reduce and hidden.is_cuda:
            # the two all-reduces of a layer (racetrack/realistic_bench.py:315-316,351) for the few
            # rows of a decode step: every rank leaves its partial sums in a buffer its peers have
            # mapped, and after one device barrier every rank sums all of them, adds the residual
            # and normalises in ONE kernel (a one-shot all-reduce fused with its consumer)
            px = self._decode_exchange(hidden.shape[0])
        for _ in range(layers):
            if px is not None:
                self.decode_attention(normed, start_pos, out=px.local["attn"])
                normed, hidden = px.reduce_residual_norm("attn", hidden, self.ones_h, eps=s.eps, all_rows=True)
                self.ffn_partial(normed, out=px.local["ffn"])
                normed, hidden = px.reduce_residual_norm("ffn", hidden, self.ones_h, eps=s.eps, all_rows=True)
                continue
            attn = self.decode_attention(normed, start_pos)
            normed, hidden = ops.fused_residual_norm(attn, hidden, self.ones_h, eps=s.eps)
            ffn = self.ffn_forward(normed)
            normed, hidden = ops.fused_residual_norm(ffn, hidden, self.ones_h, eps=s.eps)
        return hidden
