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


MIXED_FP8_MIN_K = 4096


def make_linear(proj: str = "bf16"):
    """The projection arithmetic of a stack: "bf16" = F.linear; "fp8" / "mixed" = the
    reference's own path for FP8 weights (act_quant + dequantise-then-matmul fp8_gemm, ref:
    racetrack/models/deepseek.py:316-345) for every projection whose K is a multiple of 128
    ("mixed": only where K >= 4096). Quantised weights are cached per weight tensor."""
    cache: dict = {}

    def linear(x, weight):
        k = weight.shape[1]
        fp8 = k % 128 == 0 and (proj == "fp8" or (proj == "mixed" and k >= MIXED_FP8_MIN_K))
        if not fp8:
            return F.linear(x, weight)
        key = (weight.data_ptr(), tuple(weight.shape))
        if key not in cache:
            cache[key] = R.quantize_weight_fp8(weight)
        return R.linear_fp8(x, *cache[key])
    return linear


def attention(hidden, positions, w, shape, local_heads, linear=F.linear):
    """One rank's attention partial. ref: racetrack/realistic_bench.py:286-315. `linear` swaps the
    four projections' arithmetic (make_linear)."""
    s = shape
    qkv = linear(hidden, w["w_qkv_a"])
    q_c, kv_c, k_pe = qkv.split([s.q_lora, s.kv_lora, s.rope], dim=-1)
    ones_q = torch.ones(s.q_lora, dtype=hidden.dtype)
    ones_kv = torch.ones(s.kv_lora, dtype=hidden.dtype)
    q_c, kv_c, k_pe = R.fused_norm_rope(q_c, ones_q, kv_c, ones_kv, k_pe, positions, eps=s.eps,
                                        rope_base=s.rope_base)
    tokens = hidden.shape[0]
    q = linear(q_c, w["w_q_b"]).view(tokens, local_heads, s.nope + s.rope)
    q_nope, q_pe = q.split([s.nope, s.rope], dim=-1)
    q = torch.cat((q_nope, R.apply_rope(q_pe, positions, base=s.rope_base)), dim=-1)
    kv = linear(kv_c, w["w_kv_b"]).view(tokens, local_heads, s.nope + s.v_dim)
    k_nope, v = kv.split([s.nope, s.v_dim], dim=-1)
    k = torch.cat((k_nope, k_pe.unsqueeze(1).expand(-1, local_heads, -1)), dim=-1)
    local = causal_attention(q, k, v)
    return linear(local.reshape(tokens, local_heads * s.v_dim), w["w_o"])


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
    NVFP4 arithmetic has no reference counterpart (parity unpinned). A weight dict that carries
    "w13_dq" / "w2_dq" ([E, ...] for ALL experts, values already dequant(NVFP4(w))) is used as
    is; otherwise the rank's bf16 "w13" / "w2" are quantised here."""
    if "w13_dq" in w:
        s = shape
        logits = F.linear(hidden.float(), w["w_gate"].float())
        topk_logits, topk_ids = torch.topk(logits, s.topk, dim=-1)
        topk_weights = torch.softmax(topk_logits, dim=-1).to(hidden.dtype).float()
        lo, hi = rank * local_experts, (rank + 1) * local_experts
        return R.moe_experts_nvfp4(hidden, topk_weights, topk_ids, w["w13_dq"], w["w2_dq"],
                                   expert_range=(lo, hi),
                                   weights_dequantised=(w["w13_gs"], w["w2_gs"]))
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


class ExpertBank:
    """Full-width expert weights for the oracle, materialised one expert at a time: only the
    experts a sample routes to exist (all 256 in bf16 would take 22.5 GB). `draw(e)` returns
    the bf16 (w13 [2I, H], w2 [H, I]) of expert e on any device; `quantise(t)` returns the NVFP4
    (codes, row-major block scales, global scale) of a matrix on that device (default: the
    CPU quantiser of ref_ops; a caller with a GPU passes a device quantiser that its own tests
    show bit-identical, because the CPU one takes about a second per expert). The dict
    `weights` gains "w13" / "w2" (bf16) and "w13_dq" / "w2_dq" / "w13_gs" / "w2_gs" (NVFP4 values
    code * block scale, exact in bf16, and the global scales) for forward_stack."""

    def __init__(self, shape, weights: dict, draw, quantise=None):
        s = shape
        self.shape, self.w, self.draw, self.drawn = shape, weights, draw, set()
        self.quantise = quantise if quantise is not None else R.nvfp4_quant
        e, i, h = s.n_experts, s.moe_inter, s.hidden
        for key, dims in (("w13", (e, 2 * i, h)), ("w2", (e, h, i))):
            weights[key] = torch.empty(dims, dtype=torch.bfloat16)
            weights[key + "_dq"] = torch.empty(dims, dtype=torch.bfloat16)
            weights[key + "_gs"] = torch.zeros(e, dtype=torch.float32)

    def need(self, experts) -> None:
        for e in sorted(set(int(x) for x in experts) - self.drawn):
            for key, t in zip(("w13", "w2"), self.draw(e)):
                codes, sf, gs = self.quantise(t)
                one = torch.ones((), dtype=torch.float32, device=codes.device)
                dq = R.nvfp4_dequant(codes, sf, one).to(torch.bfloat16)
                self.w[key][e], self.w[key + "_dq"][e] = t.cpu(), dq.cpu()
                self.w[key + "_gs"][e] = gs.reshape(()).float().cpu()
            self.drawn.add(e)

    def route(self, normed) -> None:
        """Materialises the experts the top-k router sends `normed` to (a near-tie may go the
        other way in another arithmetic, so the runner-up is drawn as well)."""
        logits = F.linear(normed.float(), self.w["w_gate"].float())
        self.need(torch.topk(logits, self.shape.topk + 1, dim=-1)[1].flatten().tolist())


def dense_ffn(hidden, w):
    """Dense SwiGLU FFN shard (the first-layers variant): w2(silu(w1 x) * w3 x)."""
    return F.linear(F.silu(F.linear(hidden, w["w1"])) * F.linear(hidden, w["w3"]), w["w2d"])


def dense_ffn_fp8(hidden, w, linear):
    """The dense FFN with the projections' arithmetic swapped (gate and up as one projection of
    the concatenated weight, as the product runs it; the FP8 block scales of w1 and w3 are
    per 128 rows, so the concatenation quantises exactly like the two halves)."""
    if "w13d" not in w:
        w["w13d"] = torch.cat([w["w1"], w["w3"]])
    gate_up = linear(hidden, w["w13d"])
    inter = gate_up.shape[1] // 2
    return linear(R.swiglu(gate_up[:, :inter], gate_up[:, inter:]), w["w2d"])


def forward_stack(hidden, positions, rank_weights, shape, layers, ffn="moe", experts="bf16",
                  proj="bf16", before_moe=None):
    """ref: racetrack/realistic_bench.py:375-389 (hc_mult == 1 branch) applied `layers` times.
    experts="nvfp4" swaps the bf16 expert matmuls for their NVFP4-quantised evaluation and
    proj="fp8" / "mixed" the projections for the reference's FP8 path (make_linear): the same
    model in the arithmetic the B200 layer runs. `before_moe(normed)` is called with the MoE's
    input of every layer (a full-width caller materialises the experts that input routes to)."""
    moe_fn = moe if experts == "bf16" else moe_nvfp4
    linear = make_linear(proj)
    world = len(rank_weights)
    ones = torch.ones(shape.hidden, dtype=hidden.dtype)
    local_heads = shape.heads // world
    local_experts = shape.n_experts // world
    for _ in range(layers):
        residual = hidden
        h = R.rms_norm(hidden, ones, shape.eps)
        attn = _all_reduce([attention(h, positions, w, shape, local_heads, linear) for w in rank_weights])
        hidden = residual + attn
        residual = hidden
        h = R.rms_norm(hidden, ones, shape.eps)
        if ffn == "moe":
            if before_moe is not None:
                before_moe(h)
            out = _all_reduce([moe_fn(h, w, shape, r, local_experts) for r, w in enumerate(rank_weights)])
        elif proj == "bf16":
            out = _all_reduce([dense_ffn(h, w) for w in rank_weights])
        else:
            out = _all_reduce([dense_ffn_fp8(h, w, linear) for w in rank_weights])
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
