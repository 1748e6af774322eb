"""CPU restatement of racetrack's sharded realistic layer (ShardedRealisticBlock /
ShardedRealisticModel, ref: racetrack/realistic_bench.py:286-389,420-423) in vanilla torch.

TEST INFRASTRUCTURE ONLY (see ref_ops.py). All ranks of a tensor/expert-parallel group are
evaluated in this one process; an all-reduce is the sum of the ranks' bf16 partial results.
Weights come in as one dict per rank with the keys racetrack_b200.layer.make_weights produces
(bf16 expert weights, i.e. the un-quantised model the reference runs).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ref_ops as R


def causal_attention(q, k, v):
    """ref: racetrack/runtime/torch_ops.py:97-110."""
    scale = q.shape[-1] ** -0.5
    scores = torch.einsum("thd,shd->hts", q.float(), k.float()) * scale
    t = q.shape[0]
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask.unsqueeze(0), -float("inf"))
    probs = torch.softmax(scores, dim=-1).to(v.dtype)
    return torch.einsum("hts,shd->thd", probs, v)


def _all_reduce(parts):
    total = parts[0].float()
    for p in parts[1:]:
        total = total + p.float()
    return total.to(parts[0].dtype)


def attention(hidden, positions, w, shape, local_heads):
    """One rank's attention partial. ref: racetrack/realistic_bench.py:286-315."""
    s = shape
    qkv = F.linear(hidden, w["w_qkv_a"])
    q_c, kv_c, k_pe = qkv.split([s.q_lora, s.kv_lora, s.rope], dim=-1)
    ones_q = torch.ones(s.q_lora, dtype=hidden.dtype)
    ones_kv = torch.ones(s.kv_lora, dtype=hidden.dtype)
    q_c, kv_c, k_pe = R.fused_norm_rope(q_c, ones_q, kv_c, ones_kv, k_pe, positions, eps=s.eps,
                                        rope_base=s.rope_base)
    tokens = hidden.shape[0]
    q = F.linear(q_c, w["w_q_b"]).view(tokens, local_heads, s.nope + s.rope)
    q_nope, q_pe = q.split([s.nope, s.rope], dim=-1)
    q = torch.cat((q_nope, R.apply_rope(q_pe, positions, base=s.rope_base)), dim=-1)
    kv = F.linear(kv_c, w["w_kv_b"]).view(tokens, local_heads, s.nope + s.v_dim)
    k_nope, v = kv.split([s.nope, s.v_dim], dim=-1)
    k = torch.cat((k_nope, k_pe.unsqueeze(1).expand(-1, local_heads, -1)), dim=-1)
    local = causal_attention(q, k, v)
    return F.linear(local.reshape(tokens, local_heads * s.v_dim), w["w_o"])


def moe(hidden, w, shape, rank, local_experts):
    """One rank's routed-expert partial. ref: racetrack/realistic_bench.py:319-350."""
    s = shape
    logits = F.linear(hidden.float(), w["w_gate"].float())
    topk_logits, topk_ids = torch.topk(logits, s.topk, dim=-1)
    topk_weights = torch.softmax(topk_logits, dim=-1).to(hidden.dtype)
    local = torch.zeros_like(hidden)
    start, end = rank * local_experts, (rank + 1) * local_experts
    for slot in range(s.topk):
        ids = topk_ids[:, slot]
        mask = (ids >= start) & (ids < end)
        if not bool(mask.any()):
            continue
        lids = (ids[mask] - start).long()
        x = hidden[mask]
        gate_up = torch.bmm(w["w13"][lids], x.unsqueeze(-1)).squeeze(-1)
        gate, up = gate_up.chunk(2, dim=-1)
        out = torch.bmm(w["w2"][lids], (F.silu(gate) * up).unsqueeze(-1)).squeeze(-1)
        local[mask] = local[mask] + out * topk_weights[mask, slot].unsqueeze(-1)
    return local


def moe_nvfp4(hidden, w, shape, rank, local_experts):
    """Same routing as `moe`, experts evaluated on NVFP4-quantised operands
    (ref_ops.moe_experts_nvfp4): what the B200 layer computes, for tight comparisons. The
    NVFP4 arithmetic has no reference counterpart (parity unpinned)."""
    s = shape
    logits = F.linear(hidden.float(), w["w_gate"].float())
    topk_logits, topk_ids = torch.topk(logits, s.topk, dim=-1)
    topk_weights = torch.softmax(topk_logits, dim=-1).to(hidden.dtype).float()
    n = s.n_experts
    w13 = torch.zeros(n, *w["w13"].shape[1:], dtype=w["w13"].dtype)
    w2 = torch.zeros(n, *w["w2"].shape[1:], dtype=w["w2"].dtype)
    lo, hi = rank * local_experts, (rank + 1) * local_experts
    w13[lo:hi], w2[lo:hi] = w["w13"], w["w2"]
    return R.moe_experts_nvfp4(hidden, topk_weights, topk_ids, w13, w2, expert_range=(lo, hi))


def dense_ffn(hidden, w):
    """Dense SwiGLU FFN shard (the first-layers variant): w2(silu(w1 x) * w3 x)."""
    return F.linear(F.silu(F.linear(hidden, w["w1"])) * F.linear(hidden, w["w3"]), w["w2d"])


def forward_stack(hidden, positions, rank_weights, shape, layers, ffn="moe", experts="bf16"):
    """ref: racetrack/realistic_bench.py:375-389 (hc_mult == 1 branch) applied `layers` times.
    experts="nvfp4" swaps the bf16 expert matmuls for their NVFP4-quantised evaluation."""
    moe_fn = moe if experts == "bf16" else moe_nvfp4
    world = len(rank_weights)
    ones = torch.ones(shape.hidden, dtype=hidden.dtype)
    local_heads = shape.heads // world
    local_experts = shape.n_experts // world
    for _ in range(layers):
        residual = hidden
        h = R.rms_norm(hidden, ones, shape.eps)
        attn = _all_reduce([attention(h, positions, w, shape, local_heads) for w in rank_weights])
        hidden = residual + attn
        residual = hidden
        h = R.rms_norm(hidden, ones, shape.eps)
        if ffn == "moe":
            out = _all_reduce([moe_fn(h, w, shape, r, local_experts) for r, w in enumerate(rank_weights)])
        else:
            out = _all_reduce([dense_ffn(h, w) for w in rank_weights])
        hidden = residual + out
    return hidden


# ---------------------------------------------------------------------------
# decode step: B sequences, one token each, per-sequence caches, sparse attention
# ---------------------------------------------------------------------------
def indexer_decode(h, q_c, iw, caches, start_pos, freqs, index_topk):
    """Indexer.forward for bsz = B, seqlen = 1 (ref: racetrack/models/deepseek.py:656-686).
    iw: dict with wq_b, wk, k_norm_weight, k_norm_bias, weights_proj; caches: dict with index_k
    [B, L, 128] e4m3 and index_scale [B, L]. Returns int64 [B, 1, k]."""
    batch = h.shape[0]
    heads = iw["weights_proj"].shape[0]
    fc = freqs[start_pos:start_pos + 1].expand(batch, -1)
    q = F.linear(q_c, iw["wq_b"]).view(batch, heads, 128)
    q_fp8, q_scale, _ = R.index_prep(q, fc)
    k = F.linear(h, iw["wk"]).view(batch, 1, 128)
    k_fp8, k_scale, _ = R.index_prep(k, fc, ln_weight=iw["k_norm_weight"], ln_bias=iw["k_norm_bias"])
    caches["index_k"][:, start_pos] = k_fp8.view(batch, 128)
    caches["index_scale"][:, start_pos] = k_scale.view(batch)
    head_w = F.linear(h.float(), iw["weights_proj"]) * heads ** -0.5 * q_scale * 128 ** -0.5
    end = start_pos + 1
    scores = R.fp8_index(q_fp8.unsqueeze(1), head_w.unsqueeze(1), caches["index_k"][:, :end],
                         caches["index_scale"][:, :end])
    return R.index_topk(scores, index_topk)


def decode_attention(h, start_pos, w, iw, caches, shape, local_heads, freqs, index_topk):
    """One rank's attention partial of the decode step: the synthetic layer's projections
    (racetrack/realistic_bench.py:286-303) followed by the reference's "MQA decode" branch with
    the indexer's mask (racetrack/models/deepseek.py:777-778,793-811). The caches (kv, pe: bf16
    [B, L, .]) are this rank's copies and are updated in place."""
    s = shape
    batch = h.shape[0]
    positions = torch.full((batch,), start_pos, dtype=torch.int64)
    qkv = F.linear(h, w["w_qkv_a"])
    q_c, kv_c, k_pe = qkv.split([s.q_lora, s.kv_lora, s.rope], dim=-1)
    ones_q = torch.ones(s.q_lora, dtype=h.dtype)
    ones_kv = torch.ones(s.kv_lora, dtype=h.dtype)
    q_c, kv_c, k_pe = R.fused_norm_rope(q_c, ones_q, kv_c, ones_kv, k_pe, positions, eps=s.eps,
                                        rope_base=s.rope_base)
    q = F.linear(q_c, w["w_q_b"]).view(batch, local_heads, s.nope + s.rope)
    q_nope, q_pe = q.split([s.nope, s.rope], dim=-1)
    q_pe = R.apply_rope(q_pe, positions, base=s.rope_base)
    caches["kv"][:, start_pos] = kv_c
    caches["pe"][:, start_pos] = k_pe
    picked = indexer_decode(h, q_c, iw, caches, start_pos, freqs, index_topk)
    end = start_pos + 1
    out = R.mla_decode_core(q_nope.unsqueeze(1), q_pe.unsqueeze(1), w["w_kv_b"], caches["kv"][:, :end],
                            caches["pe"][:, :end], picked, (s.nope + s.rope) ** -0.5, s.nope, s.v_dim)
    return F.linear(out.reshape(batch, local_heads * s.v_dim), w["w_o"])


def decode_stack(hidden, start_pos, rank_weights, iw, rank_caches, shape, layers, freqs, index_topk,
                 experts="bf16"):
    """The decode step applied `layers` times (one layer reused, as in forward_stack)."""
    moe_fn = moe if experts == "bf16" else moe_nvfp4
    world = len(rank_weights)
    ones = torch.ones(shape.hidden, dtype=hidden.dtype)
    local_heads = shape.heads // world
    local_experts = shape.n_experts // world
    for _ in range(layers):
        residual = hidden
        h = R.rms_norm(hidden, ones, shape.eps)
        attn = _all_reduce([decode_attention(h, start_pos, w, iw, c, shape, local_heads, freqs, index_topk)
                            for w, c in zip(rank_weights, rank_caches)])
        hidden = residual + attn
        residual = hidden
        h = R.rms_norm(hidden, ones, shape.eps)
        out = _all_reduce([moe_fn(h, w, shape, r, local_experts) for r, w in enumerate(rank_weights)])
        hidden = residual + out
    return hidden
