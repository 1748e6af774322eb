"""The MLA-prologue ops of the dsv3_2_nvfp4 partitions on the B200 backend, with the signatures of
their torch definitions (scripts/recipes_nvfp4.py:38-151; the keyword `fallback` every dispatched
kernel receives is accepted and ignored):

  fused_ar_rms_qkv_proj   residual add + RMSNorm, then ONE bf16 GEMM against [wq_a; wkv_a; indexer
                          wk] whose output is sliced into q_c, kv_c, k_pe and the indexer's key
  fused_indexer_k_path    LayerNorm + non-interleaved RoPE + Hadamard rotation + FP8 quantisation of
                          the indexer keys in one kernel, and the cache append
  fused_q_indexer_score   ONE bf16 GEMM against [wq_b; indexer wq_b]; the absorbed query as a batched
                          per-head GEMM; the indexer query path in one kernel; the fp32 head-weight
                          projection on the tensor cores; FP8 index scores (tcgen05) and exact top-k
  fused_q_rope_quant      interleaved RoPE of q_pe

`H` (the Hadamard matrix the torch definitions multiply by) is accepted for the signature's sake:
the kernel applies the same Sylvester-ordered transform as butterflies.
"""
import torch

from racetrack_b200 import _lib, ops

BACKEND_AVAILABLE = _lib.available()

_CAT: dict = {}          # key -> (derived weight, the tensors it was made from)
_CAT_MAX = 1024


def _remember(key, entry):
    while len(_CAT) >= _CAT_MAX:
        _CAT.pop(next(iter(_CAT)))
    _CAT[key] = entry


def _cat_weights(*weights):
    """Row-wise concatenation of bf16 weights, cached per set of tensors (racetrack's own
    kernels cache the same way, partitions/dsv3_2_nvfp4/cd91301b/kernels/triton/qkv_proj.py:21-39)."""
    key = tuple((w.data_ptr(), tuple(w.shape), w._version) for w in weights)
    hit = _CAT.get(key)
    if hit is None:
        for w in weights:
            if w.dtype != torch.bfloat16:
                raise RuntimeError("the MLA prologue ops take bfloat16 weights")
        # the entry holds the source tensors, so their addresses stay theirs while it exists
        hit = (torch.cat(weights, dim=0).contiguous(), tuple(w.detach() for w in weights))
        _remember(key, hit)
    return hit[0]


def _uk_t(wkv_b_weight, n_heads, nope, kv_lora):
    """[heads, kv_lora, nope]: the key half of wkv_b transposed per head, the K-major B operand of
    q_nope -> latent."""
    key = ("uk_t", wkv_b_weight.data_ptr(), tuple(wkv_b_weight.shape), wkv_b_weight._version)
    hit = _CAT.get(key)
    if hit is None:
        hit = (wkv_b_weight.view(n_heads, -1, kv_lora)[:, :nope].transpose(1, 2).contiguous(),
               wkv_b_weight.detach())
        _remember(key, hit)
    return hit[0]


def fused_ar_rms_qkv_proj(x, residual, norm_weight, wq_a_weight, wkv_a_weight, indexer_wk_weight, *,
                          eps, q_lora_rank, kv_lora_rank, qk_rope_head_dim, fallback=None):
    del fallback
    lead, dim = x.shape[:-1], x.shape[-1]
    x2 = x.reshape(-1, dim)
    if residual is not None:
        normed, hidden = ops.fused_residual_norm(x2, residual.reshape(-1, dim), norm_weight, eps=eps)
    else:
        normed, hidden = ops.fused_rms_norm(x2, norm_weight, eps=eps), x2
    out = ops.linear_bf16(normed, _cat_weights(wq_a_weight, wkv_a_weight, indexer_wk_weight))
    out = out.view(*lead, out.shape[-1])
    a, b = q_lora_rank, q_lora_rank + kv_lora_rank
    c = b + qk_rope_head_dim
    if wq_a_weight.shape[0] + wkv_a_weight.shape[0] != c:
        raise RuntimeError("fused_ar_rms_qkv_proj: wq_a / wkv_a rows do not add up to q_lora + kv_lora + rope")
    return (hidden.view(*lead, dim), normed.view(*lead, dim), out[..., :a], out[..., a:b], out[..., b:c],
            out[..., c:])


def fused_indexer_k_path(k, ln_weight, ln_bias, freqs_cis, H, k_cache, k_scale_cache, *, ln_dim, ln_eps,
                         rope_head_dim, start_pos, block_size, fallback=None):
    del fallback, H
    bsz, seqlen, dim = k.shape
    if dim != 128 or ln_dim != 128 or rope_head_dim != 64 or block_size != 128:
        raise RuntimeError("fused_indexer_k_path: index head width 128, rope width 64, block 128 only")
    pos = torch.arange(seqlen, device=k.device, dtype=torch.int64).repeat(bsz)
    codes, scales = ops.index_prep(k.reshape(bsz * seqlen, 1, dim), freqs_cis, positions=pos,
                                   ln_weight=ln_weight, ln_bias=ln_bias, eps=ln_eps)
    k_fp8, k_scale = codes.view(bsz, seqlen, dim), scales.view(bsz, seqlen, 1)
    end_pos = start_pos + seqlen
    k_cache[:bsz, start_pos:end_pos] = k_fp8 if k_cache.dtype == k_fp8.dtype else k_fp8.to(k_cache.dtype)
    k_scale_cache[:bsz, start_pos:end_pos] = k_scale.view(bsz, seqlen, *k_scale_cache.shape[2:])
    return k_fp8, k_scale


def fused_q_indexer_score(qr, normed_x, wq_b_weight, idx_wq_b_weight, idx_weights_proj_weight, wkv_b_weight,
                          freqs_cis, H, k_cache, k_scale_cache, *, eps, n_heads, qk_head_dim,
                          qk_nope_head_dim, kv_lora_rank, idx_n_heads, idx_head_dim, rope_head_dim,
                          softmax_scale, idx_softmax_scale, index_topk, start_pos, end_pos, block_size,
                          fallback=None):
    del fallback, H, eps, softmax_scale, start_pos
    bsz, seqlen, _ = qr.shape
    if idx_head_dim != 128 or rope_head_dim != 64 or block_size != 128:
        raise RuntimeError("fused_q_indexer_score: index head width 128, rope width 64, block 128 only")
    tokens = bsz * seqlen
    q_dim = n_heads * qk_head_dim
    both = ops.linear_bf16(qr.reshape(tokens, -1), _cat_weights(wq_b_weight, idx_wq_b_weight))
    q = both[:, :q_dim].view(tokens, n_heads, qk_head_dim)
    q_nope, q_pe = q[..., :qk_nope_head_dim], q[..., qk_nope_head_dim:]
    q_abs = ops.linear_bf16_batched(q_nope, _uk_t(wkv_b_weight, n_heads, qk_nope_head_dim, kv_lora_rank))
    idx_q = both[:, q_dim:].view(tokens, idx_n_heads, idx_head_dim)
    pos = torch.arange(seqlen, device=qr.device, dtype=torch.int64).repeat(bsz)
    q_fp8, q_scale = ops.index_prep(idx_q, freqs_cis, positions=pos)
    weights = ops.linear_f32_weight(normed_x.reshape(tokens, -1), idx_weights_proj_weight.float()) \
        * idx_n_heads ** -0.5
    weights = weights * q_scale * idx_softmax_scale
    keys = k_cache[:bsz, :end_pos]
    if keys.dtype != torch.float8_e4m3fn:
        keys = keys.to(torch.float8_e4m3fn)              # a cache kept in a wider type holds e4m3 values
    scores = ops.fp8_index(q_fp8.view(bsz, seqlen, idx_n_heads, idx_head_dim),
                           weights.view(bsz, seqlen, idx_n_heads), keys,
                           k_scale_cache[:bsz, :end_pos].reshape(bsz, end_pos))
    picked = ops.index_topk(scores, min(index_topk, end_pos)).long()
    shape4 = (bsz, seqlen, n_heads)
    return (q_nope.reshape(*shape4, qk_nope_head_dim), q_abs.view(*shape4, kv_lora_rank),
            q_pe.reshape(*shape4, qk_head_dim - qk_nope_head_dim), picked)


def fused_q_rope_quant(q_pe, freqs_cis, *, block_size, fallback=None):
    del fallback, block_size
    return ops.fused_rope(q_pe, freqs_cis)
