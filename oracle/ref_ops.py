"""CPU restatement of racetrack's vanilla-torch DeepSeek-V3.2 hot path.

TEST INFRASTRUCTURE ONLY. This module is the checker, never the product: only
tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs may import
it. Nothing under racetrack_b200/ imports it.

Every function restates one reference function and cites it as ``ref: file:lines``
(paths inside the racetrack project). The restatements are pinned against outputs of
the reference itself: tests/golden/make_golden.py imports the reference, runs it on
seeded inputs and stores input/output pairs; tests/test_oracle_golden.py replays them
through this module and demands exact equality.

The NVFP4 functions have no counterpart in the reference (it has no e2m1 code at
all), so their parity is UNPINNED: they implement the format as the build's
configuration states it (16-element blocks, e4m3 block scale, fp32 global scale =
amax / (448 * 6)) and are checked only against hand-derived known answers.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

FP8_BLOCK = 128
FP8_MAX = 448.0
FP4_MAX = 6.0
NVFP4_BLOCK = 16


# ---------------------------------------------------------------------------
# norms
# ---------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ref: partitions/_base.py:24-28 (same math as racetrack/models/deepseek.py:478-483)."""
    dtype = x.dtype
    xf = x.float()
    scale = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return (xf * scale * weight.float()).to(dtype)


def residual_norm(update: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                  eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(normed, hidden). ref: racetrack/models/deepseek.py:485-495."""
    hidden = update.float() + residual.float()
    var = hidden.pow(2).mean(-1, keepdim=True)
    normed = hidden * torch.rsqrt(var + eps)
    return (weight * normed).to(update.dtype), hidden.to(update.dtype)


# ---------------------------------------------------------------------------
# RoPE
# ---------------------------------------------------------------------------

def rope_cache(positions: torch.Tensor, rotary_dim: int, base: float = 10000.0,
               dtype: Optional[torch.dtype] = None):
    """cos/sin tables [T, rotary_dim/2]. ref: partitions/dsv3_2/model.py:27-52."""
    half = rotary_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / max(half, 1)))
    freqs = positions.float().unsqueeze(-1) * inv_freq.unsqueeze(0)
    cos, sin = torch.cos(freqs), torch.sin(freqs)
    if dtype is not None:
        cos, sin = cos.to(dtype), sin.to(dtype)
    return cos, sin


def apply_rope(x: torch.Tensor, positions: torch.Tensor, base: float = 10000.0) -> torch.Tensor:
    """Half-split RoPE over the whole last dimension. ref: partitions/dsv3_2/model.py:55-81."""
    rotary_dim = x.shape[-1]
    cos, sin = rope_cache(positions, rotary_dim, base=base, dtype=x.dtype)
    half = rotary_dim // 2
    x1, x2 = x[..., :half], x[..., half:]
    while cos.dim() < x1.dim():
        cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def precompute_freqs_cis(rope_dim: int, seqlen: int, theta: float = 10000.0,
                         original_seq_len: int = 4096, rope_factor: float = 40.0,
                         beta_fast: int = 32, beta_slow: int = 1) -> torch.Tensor:
    """complex64 [seqlen, rope_dim/2], YaRN-corrected beyond original_seq_len.
    ref: racetrack/models/deepseek.py:523-601."""
    dim = rope_dim

    def corr_dim(num_rot):
        return dim * math.log(original_seq_len / (num_rot * 2 * math.pi)) / (2 * math.log(theta))

    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if seqlen > original_seq_len:
        low = max(math.floor(corr_dim(beta_fast)), 0)
        high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
        hi = high + 0.001 if low == high else high
        ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (hi - low), 0, 1)
        smooth = 1 - ramp
        freqs = freqs / rope_factor * (1 - smooth) + freqs * smooth
    t = torch.arange(seqlen)
    freqs = torch.outer(t, freqs)
    return torch.polar(torch.ones_like(freqs), freqs)


def apply_rotary_emb(x: torch.Tensor, freqs_cis: torch.Tensor,
                     interleaved: bool = True) -> torch.Tensor:
    """x [B, S, H, D] rotated by freqs_cis [S, D/2]. ref: racetrack/models/deepseek.py:604-624."""
    dtype, shape = x.dtype, x.shape
    if not interleaved:
        x = x.view(*shape[:-1], 2, -1).transpose(-1, -2).contiguous()
    xc = torch.view_as_complex(x.float().view(*shape[:-1], -1, 2))
    fc = freqs_cis.view(1, xc.size(1), 1, xc.size(-1))
    y = torch.view_as_real(xc * fc).flatten(3)
    if not interleaved:
        y = torch.cat([y[..., 0::2], y[..., 1::2]], dim=-1)
    return y.to(dtype)


def fused_norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, positions, *, eps: float,
                    rope_base: float):
    """ref: partitions/dsv3_2/model.py:84-99."""
    return (rms_norm(q_c, q_weight, eps), rms_norm(kv_c, kv_weight, eps),
            apply_rope(k_pe, positions, base=rope_base))


def mla_prologue(x, residual, w_attn, q_c, w_q, kv_c, w_kv, q_pe, k_pe, freqs_cis, eps: float):
    """The fused MLA prologue of the CPU-runnable configuration: residual-add + RMSNorm,
    q_a / kv_a RMSNorm and interleaved RoPE on q_pe [T, H, D] and k_pe [T, 1, D].
    ref: racetrack/models/deepseek.py:485-495, :478-483, :766-776."""
    normed, hidden = residual_norm(x, residual, w_attn, eps)
    qn = rms_norm(q_c, w_q, eps)
    kvn = rms_norm(kv_c, w_kv, eps)
    q_rot = apply_rotary_emb(q_pe.unsqueeze(0), freqs_cis).squeeze(0)
    k_rot = apply_rotary_emb(k_pe.unsqueeze(0), freqs_cis).squeeze(0)
    return normed, hidden, qn, kvn, q_rot, k_rot


# ---------------------------------------------------------------------------
# SwiGLU and FP8 activation quantisation
# ---------------------------------------------------------------------------

def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """ref: racetrack/models/deepseek.py:850-851 (MLP), :958-959 (Expert)."""
    return (F.silu(gate.float()) * up.float()).type_as(gate)


def act_quant(x: torch.Tensor, block_size: int = FP8_BLOCK):
    """(e4m3 codes, fp32 scales [..., N/block]). ref: racetrack/models/deepseek.py:85-107."""
    x = x.contiguous()
    n = x.size(-1)
    assert n % block_size == 0
    groups = n // block_size
    shape = x.shape
    xf = x.float().reshape(-1, groups, block_size)
    amax = xf.abs().amax(dim=-1).clamp(min=1e-4)
    scale = amax / FP8_MAX
    y = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(shape)
    return y, scale.view(*shape[:-1], groups)


def swiglu_quant(gate: torch.Tensor, up: torch.Tensor):
    """SwiGLU rounded to the activation dtype, then act_quant.
    ref: benchmarks/gsm8k/flat_decode.py:132-136."""
    return act_quant(swiglu(gate, up))


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """ref: racetrack/models/deepseek.py:508-520 (LayerNorm: fp32 F.layer_norm, cast back)."""
    return F.layer_norm(x.float(), (x.shape[-1],), weight, bias, eps).type_as(x)


def hadamard_matrix(n: int) -> torch.Tensor:
    """Sylvester Hadamard matrix of order n (a power of two), entries +-1, natural ordering:
    H[i, k] = (-1)^popcount(i & k)."""
    h = torch.ones(1, 1)
    while h.shape[0] < n:
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return h


def rotate_activation(x: torch.Tensor) -> torch.Tensor:
    """x @ H_n * n^-0.5 in fp32, rounded to x's dtype.
    ref: racetrack/models/deepseek.py:627-631, which calls hadamard_transform(x, scale) of the
    third-party package fast_hadamard_transform (Dao-AILab, not vendored in racetrack and not
    installed here: parity of this step is unpinned). Its documented contract is the product
    with the Sylvester Hadamard matrix times `scale`, accumulated in fp32."""
    n = x.shape[-1]
    return ((x.float() @ hadamard_matrix(n)) * n ** -0.5).to(x.dtype)


def index_prep(x: torch.Tensor, freqs_cis: torch.Tensor, *, rope_dim: int = 64,
               ln_weight: Optional[torch.Tensor] = None, ln_bias: Optional[torch.Tensor] = None,
               eps: float = 1e-6):
    """The indexer's path from a projected row to FP8 (racetrack/models/deepseek.py:659-676):
    (LayerNorm for keys) -> non-interleaved RoPE on the first rope_dim dims -> Hadamard rotation
    -> act_quant. x [S, H, D] bf16 (H = 1 for keys), freqs_cis complex [S, rope_dim/2].
    Returns (codes e4m3 [S, H, D], scales fp32 [S, H], rotated bf16 [S, H, D])."""
    if ln_weight is not None:
        x = layer_norm(x, ln_weight, ln_bias, eps)
    pe, nope = torch.split(x, [rope_dim, x.shape[-1] - rope_dim], dim=-1)
    pe = apply_rotary_emb(pe.unsqueeze(0).contiguous(), freqs_cis, False).squeeze(0)
    rotated = rotate_activation(torch.cat([pe, nope], dim=-1))
    codes, scales = act_quant(rotated)
    return codes, scales.squeeze(-1), rotated


def fp8_index(q: torch.Tensor, q_s: torch.Tensor, k: torch.Tensor, k_s: torch.Tensor) -> torch.Tensor:
    """Index scores of the sparse-attention indexer.
        score[b, m, n] = k_s[b, n] * sum_h q_s[b, m, h] * relu(q[b, m, h, :] . k[b, n, :])
    q [b, m, h, d] and k [b, n, d] are e4m3 codes, q_s [b, m, h] fp32 (per-head weight already
    multiplied by the query's quantisation scale and the softmax scale), k_s [b, n] fp32.
    ref: racetrack/models/deepseek.py:164-176 (fp8_index)."""
    logits = torch.einsum("bmhd,bnd->bmhn", q.float(), k.float())
    logits = torch.relu(logits) * q_s.unsqueeze(-1)
    return logits.sum(dim=2) * k_s.unsqueeze(1)


def index_topk(scores: torch.Tensor, topk: int, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Indices of the `min(topk, n)` largest scores per query, after adding the (causal)
    mask. ref: racetrack/models/deepseek.py:681-683."""
    if mask is not None:
        scores = scores + mask
    return scores.topk(min(topk, scores.shape[-1]), dim=-1)[1]


def mla_sparse_decode(q_abs: torch.Tensor, q_pe: torch.Tensor, kv_cache: torch.Tensor,
                      pe_cache: torch.Tensor, indices: torch.Tensor | None,
                      softmax_scale: float) -> torch.Tensor:
    """The attention core of the MLA decode branch in fp32: scores of the absorbed query against
    the latent and rope caches, the indexer's mask (0 on the selected keys, -inf elsewhere),
    softmax, weighted sum of the latent rows. q_abs [B,H,512], q_pe [B,H,64], kv_cache [B,S,512],
    pe_cache [B,S,64], indices [B,n] (entries < 0 are ignored) or None -> fp32 [B,H,512].
    ref: racetrack/models/deepseek.py:799-809 (the reference runs these einsums in bf16)."""
    scores = (torch.einsum("bhc,btc->bht", q_abs.float(), kv_cache.float()) +
              torch.einsum("bhr,btr->bht", q_pe.float(), pe_cache.float())) * softmax_scale
    if indices is not None:
        b, s = kv_cache.shape[0], kv_cache.shape[1]
        mask = torch.full((b, s + 1), float("-inf"))
        idx = indices.long().clone()
        idx[(idx < 0) | (idx >= s)] = s
        mask.scatter_(-1, idx, 0.0)
        scores = scores + mask[:, None, :s]
    return torch.einsum("bht,btc->bhc", scores.softmax(dim=-1), kv_cache.float())


def mla_decode_core(q_nope: torch.Tensor, q_pe: torch.Tensor, wkv_b: torch.Tensor,
                    kv_cache: torch.Tensor, pe_cache: torch.Tensor, topk_indices: torch.Tensor,
                    softmax_scale: float, nope: int, v_dim: int) -> torch.Tensor:
    """The "MQA decode" branch in the reference's own dtype flow (every einsum and the softmax in
    the tensors' dtype, bf16 in the model): absorb q_nope through the key half of wkv_b, score
    against the latent and rope caches, add the index mask, softmax, weight the latent rows, apply
    the value half of wkv_b. q_nope [B,S,H,nope], q_pe [B,S,H,rope], wkv_b [H*(nope+v), C],
    kv_cache [B,T,C], pe_cache [B,T,rope] (T = end_pos), topk_indices [B,S,k] -> [B,S,H,v].
    ref: racetrack/models/deepseek.py:794-810."""
    bsz, _, heads, _ = q_nope.shape
    end_pos = kv_cache.shape[1]
    w = wkv_b.view(heads, -1, kv_cache.shape[-1])
    q_abs = torch.einsum("bshd,hdc->bshc", q_nope, w[:, :nope])
    scores = (torch.einsum("bshc,btc->bsht", q_abs, kv_cache) +
              torch.einsum("bshr,btr->bsht", q_pe, pe_cache)) * softmax_scale
    index_mask = torch.full((bsz, 1, end_pos), float("-inf"), dtype=scores.dtype).scatter_(
        -1, topk_indices.long(), 0)
    scores = scores + index_mask.unsqueeze(2)
    scores = scores.softmax(dim=-1)
    x = torch.einsum("bsht,btc->bshc", scores, kv_cache)
    return torch.einsum("bshc,hdc->bshd", x, w[:, -v_dim:])


def mla_decode(x: torch.Tensor, start_pos: int, freqs_cis: torch.Tensor, w: dict,
               kv_cache: torch.Tensor, pe_cache: torch.Tensor, topk_indices: torch.Tensor, *,
               heads: int, nope: int, rope: int, v_dim: int, eps: float = 1e-6) -> torch.Tensor:
    """MLA.forward with mask=None (one new token per sequence): x [B,1,dim] bf16; w holds wq_a,
    q_norm, wq_b, wkv_a, kv_norm, wkv_b, wo; the caches [B, max_len, .] are updated in place at
    start_pos; topk_indices [B,1,k] is what the indexer returned. freqs_cis complex [1, rope/2]
    for this position. ref: racetrack/models/deepseek.py:765-811."""
    bsz, seqlen, _ = x.shape
    end_pos = start_pos + seqlen
    qr = rms_norm(F.linear(x, w["wq_a"]), w["q_norm"], eps)
    q = F.linear(qr, w["wq_b"]).view(bsz, seqlen, heads, nope + rope)
    q_nope, q_pe = torch.split(q, [nope, rope], dim=-1)
    q_pe = apply_rotary_emb(q_pe, freqs_cis)
    kv = F.linear(x, w["wkv_a"])
    kv, k_pe = torch.split(kv, [kv.shape[-1] - rope, rope], dim=-1)
    kv = rms_norm(kv, w["kv_norm"], eps)
    k_pe = apply_rotary_emb(k_pe.unsqueeze(2), freqs_cis)
    kv_cache[:bsz, start_pos:end_pos] = kv
    pe_cache[:bsz, start_pos:end_pos] = k_pe.squeeze(2)
    out = mla_decode_core(q_nope, q_pe, w["wkv_b"], kv_cache[:bsz, :end_pos], pe_cache[:bsz, :end_pos],
                          topk_indices, (nope + rope) ** -0.5, nope, v_dim)
    return F.linear(out.flatten(2), w["wo"])


def block_dequant(weight: torch.Tensor, scale: torch.Tensor, block: int = FP8_BLOCK) -> torch.Tensor:
    """FP8 weight [out, in] with [out/128, in/128] scales -> bf16.
    ref: racetrack/models/deepseek.py:148-161."""
    out_f, in_f = weight.shape
    s = scale.float().repeat_interleave(block, 0)[:out_f].repeat_interleave(block, 1)[:, :in_f]
    return (weight.float() * s).to(torch.bfloat16)


def quantize_weight_fp8(weight: torch.Tensor, block: int = FP8_BLOCK):
    """bf16 / fp32 weight [out, in] -> (e4m3fn codes, fp32 scales [ceil(out/128), in/128]): one
    scale = amax / 448 (amax clamped at 1e-4) per 128 x 128 block, the checkpoint layout that
    `Linear` holds (ref: racetrack/models/deepseek.py:361-371) and `block_dequant` inverts."""
    n, k = weight.shape
    nb = (n + block - 1) // block
    w = torch.zeros(nb * block, k, dtype=torch.float32)
    w[:n] = weight.float()
    blocks = w.view(nb, block, k // block, block)
    scale = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-4) / FP8_MAX
    codes = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return codes.view(nb * block, k)[:n].contiguous(), scale.contiguous()


def linear_fp8(x: torch.Tensor, w_codes: torch.Tensor, w_scales: torch.Tensor) -> torch.Tensor:
    """`linear(x, weight)` for an FP8 weight as the reference's torch path runs it: act_quant of
    the activations, then the dequantise-then-matmul fp8_gemm.
    ref: racetrack/models/deepseek.py:343-345, 113-121."""
    codes, scales = act_quant(x.contiguous())
    return fp8_gemm(codes, scales, w_codes, w_scales)


def fp8_gemm(a: torch.Tensor, a_s: torch.Tensor, b: torch.Tensor, b_s: torch.Tensor) -> torch.Tensor:
    """Dequantise-then-matmul fallback of the FP8 block-scaled GEMM.
    ref: racetrack/models/deepseek.py:113-121."""
    a_s_e = a_s.repeat_interleave(FP8_BLOCK, dim=-1)[..., : a.shape[-1]]
    a_bf = (a.to(torch.float32) * a_s_e).to(torch.bfloat16)
    return F.linear(a_bf, block_dequant(b, b_s))


# ---------------------------------------------------------------------------
# NVFP4 (no reference counterpart: parity unpinned)
# ---------------------------------------------------------------------------

_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def e2m1_encode(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit e2m1 code (uint8), round-to-nearest-even, saturating at +-6.
    A tie between two grid points goes to the even code."""
    a = v.abs()
    code = ((a > 0.25).to(torch.uint8) + (a >= 0.75).to(torch.uint8) + (a > 1.25).to(torch.uint8)
            + (a >= 1.75).to(torch.uint8) + (a > 2.5).to(torch.uint8) + (a >= 3.5).to(torch.uint8)
            + (a > 5.0).to(torch.uint8))
    sign = torch.signbit(v).to(torch.uint8) << 3
    return code | sign


def e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    mag = _E2M1_VALUES.to(code.device)[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def nvfp4_quant(x: torch.Tensor, amax: Optional[torch.Tensor] = None):
    """(codes uint8 [..., N/2], block scales float8_e4m3fn [..., N/16], global scale fp32 scalar).

    gs = amax / 2688 (1 when amax == 0); bs = e4m3_rne(min(block_amax / (6 * gs), 448));
    code = e2m1(x * (1 / (gs * float(bs)))), all in IEEE fp32; an all-zero block scale gives
    zero codes. Element 2i sits in the low nibble of byte i.
    """
    n = x.shape[-1]
    assert n % NVFP4_BLOCK == 0
    xf = x.float()
    if amax is None:
        amax = xf.abs().max()
    amax = amax.float().reshape(())
    gs = amax / 2688.0 if float(amax) > 0 else torch.tensor(1.0)
    blocks = xf.reshape(*x.shape[:-1], n // NVFP4_BLOCK, NVFP4_BLOCK)
    bmax = blocks.abs().amax(dim=-1)
    t = (bmax / (6.0 * gs)).clamp(max=FP8_MAX)
    bs = t.to(torch.float8_e4m3fn)
    denom = gs * bs.float()
    inv = torch.where(denom > 0, 1.0 / denom, torch.zeros_like(denom))
    v = blocks * inv.unsqueeze(-1)
    code = torch.where((denom > 0).unsqueeze(-1), e2m1_encode(v), torch.zeros((), dtype=torch.uint8))
    code = code.reshape(*x.shape[:-1], n // 2, 2)
    packed = code[..., 0] | (code[..., 1] << 4)
    return packed, bs, gs.reshape(1).float()


def nvfp4_dequant(codes: torch.Tensor, block_scales: torch.Tensor, gs: torch.Tensor) -> torch.Tensor:
    """Inverse of nvfp4_quant -> fp32 [..., N]."""
    lo, hi = codes & 0xF, codes >> 4
    vals = torch.stack((e2m1_decode(lo), e2m1_decode(hi)), dim=-1).reshape(*codes.shape[:-1], -1)
    n = vals.shape[-1]
    scale = (block_scales.float() * gs.float().reshape(())).repeat_interleave(NVFP4_BLOCK, dim=-1)
    return vals * scale[..., :n]


def sf_tiled_offsets(rows: int, nblk: int) -> torch.Tensor:
    """Byte offsets [rows, nblk] of block scales in the 128-row x 4-block tiled layout."""
    r = torch.arange(rows).unsqueeze(1)
    b = torch.arange(nblk).unsqueeze(0)
    kt = (nblk + 3) // 4
    return ((r // 128) * kt + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4


# ---------------------------------------------------------------------------
# MoE gate, permutation, experts
# ---------------------------------------------------------------------------

def gate_route(logits: torch.Tensor, bias: Optional[torch.Tensor], *, n_groups: int,
               topk_groups: int, topk: int, route_scale: float, score_func: str = "sigmoid"):
    """Everything in Gate.forward after the logits GEMM. ref: racetrack/models/deepseek.py:899-920."""
    tokens = logits.size(0)
    scores = logits.softmax(dim=-1) if score_func == "softmax" else logits.sigmoid()
    original = scores
    if bias is not None:
        scores = scores + bias
    if n_groups > 1:
        scores = scores.view(tokens, n_groups, -1)
        if bias is None:
            group_scores = scores.amax(dim=-1)
        else:
            group_scores = scores.topk(2, dim=-1)[0].sum(dim=-1)
        idx = group_scores.topk(topk_groups, dim=-1)[1]
        mask = scores.new_ones(tokens, n_groups, dtype=torch.bool).scatter_(1, idx, False)
        scores = scores.masked_fill(mask.unsqueeze(-1), float("-inf")).flatten(1)
    indices = scores.topk(topk, dim=-1)[1]
    weights = original.gather(1, indices)
    if score_func == "sigmoid":
        weights = weights / weights.sum(dim=-1, keepdim=True)
    weights = weights * route_scale
    return weights, indices


def gate_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], **kw):
    """ref: racetrack/models/deepseek.py:888-920 (logits GEMM in fp32 at :898)."""
    return gate_route(F.linear(x.float(), weight.float()), bias, **kw)


def moe_permute(indices: torch.Tensor, n_experts: int):
    """(expert_offsets, sorted_pairs, pair_pos) as the per-expert ``torch.where(indices == e)``
    loop orders them. ref: racetrack/models/deepseek.py:1011-1017."""
    tokens, topk = indices.shape
    counts = torch.bincount(indices.flatten(), minlength=n_experts)
    offsets = torch.zeros(n_experts + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    sorted_pairs = []
    for e in range(n_experts):
        idx, top = torch.where(indices == e)
        sorted_pairs.append(idx * topk + top)
    sorted_pairs = torch.cat(sorted_pairs).to(torch.int32)
    pair_pos = torch.empty(tokens * topk, dtype=torch.int32)
    pair_pos[sorted_pairs.long()] = torch.arange(tokens * topk, dtype=torch.int32)
    return offsets, sorted_pairs, pair_pos


def expert_mlp(x, w1, w2, w3):
    """One SwiGLU expert with bf16 weights. ref: racetrack/models/deepseek.py:944-962."""
    h = swiglu(F.linear(x, w1), F.linear(x, w3))
    return F.linear(h.type_as(x), w2)


def moe_forward(x, gate_w, gate_b, experts, shared, *, n_groups, topk_groups, topk, route_scale,
                score_func="sigmoid", expert_range=None):
    """x [T, dim]; experts = list of (w1, w2, w3) or None; shared = (w1, w2, w3) or None.
    ref: racetrack/models/deepseek.py:998-1022."""
    weights, indices = gate_forward(x, gate_w, gate_b, n_groups=n_groups, topk_groups=topk_groups,
                                    topk=topk, route_scale=route_scale, score_func=score_func)
    y = torch.zeros_like(x, dtype=torch.float32)
    counts = torch.bincount(indices.flatten(), minlength=len(experts)).tolist()
    lo, hi = expert_range if expert_range is not None else (0, len(experts))
    for i in range(lo, hi):
        if counts[i] == 0:
            continue
        idx, top = torch.where(indices == i)
        y[idx] += expert_mlp(x[idx], *experts[i]) * weights[idx, top, None]
    if shared is not None:
        y += expert_mlp(x, *shared)
    return y.type_as(x)


def nvfp4_roundtrip(x: torch.Tensor, amax: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dequant(quant(x)) in fp32: the values an NVFP4 tensor-core GEMM actually multiplies."""
    return nvfp4_dequant(*nvfp4_quant(x, amax))


def moe_experts_nvfp4(x, weights, indices, w13, w2, shared_out=None, expert_range=None,
                      weights_dequantised=False, x_amax=None, h_amax=None):
    """MoE.forward's expert loop (ref: racetrack/models/deepseek.py:1011-1022) with NVFP4
    operands: x and swiglu(h) quantised with one tensor-wide global scale each (over the rows
    routed to the experts in `expert_range`), every expert's w13 [2I, H] / w2 [H, I] with its own;
    products of dequantised operands accumulate in fp32, GEMM outputs round to bf16.
    NVFP4 itself has no reference counterpart (parity unpinned); the control flow follows the
    reference. With weights_dequantised = (w13_gs, w2_gs) (fp32 [E] global scales), w13 / w2 hold
    code * block_scale of the already quantised weights (exact in bf16) and the products are
    multiplied by the expert's global scale afterwards (a full-width caller quantises 256
    experts once instead of on every call). x_amax / h_amax override the two tensor-wide
    maxima (a caller that evaluates a few rows of a larger batch passes the batch's own).
    Returns bf16 [T, H]."""
    if weights_dequantised:
        gs13, gs2 = weights_dequantised
        mm13 = lambda a, e: (a @ w13[e].float().t()) * gs13[e]
        mm2 = lambda a, e: (a @ w2[e].float().t()) * gs2[e]
    else:
        mm13 = lambda a, e: a @ nvfp4_roundtrip(w13[e]).t()
        mm2 = lambda a, e: a @ nvfp4_roundtrip(w2[e]).t()
    tokens, hidden = x.shape
    n_experts = w13.shape[0]
    inter = w13.shape[1] // 2
    lo, hi = expert_range if expert_range is not None else (0, n_experts)
    xq = nvfp4_roundtrip(x, x_amax)               # global amax over the un-permuted activations
    rows = {}
    for e in range(lo, hi):
        idx, top = torch.where(indices == e)
        if idx.numel() == 0:
            continue
        gate_up = mm13(xq[idx], e).to(torch.bfloat16)
        rows[e] = (idx, top, swiglu(gate_up[:, :inter], gate_up[:, inter:]))
    y = torch.zeros(tokens, hidden, dtype=torch.float32)
    if rows:
        if h_amax is None:
            h_amax = torch.stack([h.float().abs().max() for (_, _, h) in rows.values()]).max()
        # fp32 accumulation in slot order, as the combine kernel does
        outs = torch.zeros(tokens, indices.shape[1], hidden, dtype=torch.float32)
        for e, (idx, top, h) in rows.items():
            out = mm2(nvfp4_roundtrip(h, h_amax), e).to(torch.bfloat16)
            outs[idx, top] = out.float() * weights[idx, top, None]
        for s in range(indices.shape[1]):
            y = y + outs[:, s]
    if shared_out is not None:
        y = y + shared_out.float()
    return y.to(torch.bfloat16)


# ---------------------------------------------------------------------------
# MLA prologue ops of the dsv3_2_nvfp4 partitions (torch definitions the partitions fall back to)
# ---------------------------------------------------------------------------
def fused_ar_rms_qkv_proj(x, residual, norm_weight, wq_a_weight, wkv_a_weight, indexer_wk_weight, *,
                          eps, q_lora_rank, kv_lora_rank, qk_rope_head_dim):
    """Residual add + RMSNorm, the fused q_a / kv_a projection and the indexer's key projection.
    Returns (residual_out, normed, q_c, kv_c, k_pe, indexer_k).
    ref: scripts/recipes_nvfp4.py:38-66."""
    hidden = x.float() + residual.float() if residual is not None else x.float()
    var = hidden.square().mean(dim=-1, keepdim=True)
    normed = (norm_weight.float() * hidden * torch.rsqrt(var + eps)).to(x.dtype)
    qkv = F.linear(normed, torch.cat([wq_a_weight, wkv_a_weight], dim=0))
    total = q_lora_rank + kv_lora_rank + qk_rope_head_dim
    return (hidden.to(x.dtype), normed, qkv[..., :q_lora_rank],
            qkv[..., q_lora_rank:q_lora_rank + kv_lora_rank],
            qkv[..., q_lora_rank + kv_lora_rank:total], F.linear(normed, indexer_wk_weight))


def fused_indexer_k_path(k, ln_weight, ln_bias, freqs_cis, k_cache, k_scale_cache, *, ln_eps,
                         rope_head_dim, start_pos):
    """Indexer key path: LayerNorm, non-interleaved RoPE, Hadamard rotation, FP8 quantisation and
    the cache append. k [bsz, seqlen, 128]; freqs_cis complex [seqlen, rope/2]. Returns (k_fp8,
    k_scale [bsz, seqlen, 1]). ref: scripts/recipes_nvfp4.py:68-94."""
    bsz, seqlen, dim = k.shape
    codes, scales = [], []
    for b in range(bsz):
        c, s, _ = index_prep(k[b].unsqueeze(1), freqs_cis, rope_dim=rope_head_dim, ln_weight=ln_weight,
                             ln_bias=ln_bias, eps=ln_eps)
        codes.append(c.squeeze(1))
        scales.append(s)
    k_fp8, k_scale = torch.stack(codes), torch.stack(scales)
    k_cache[:bsz, start_pos:start_pos + seqlen] = k_fp8.to(k_cache.dtype)
    k_scale_cache[:bsz, start_pos:start_pos + seqlen] = k_scale.view(bsz, seqlen, *k_scale_cache.shape[2:])
    return k_fp8, k_scale


def fused_q_indexer_score(qr, normed_x, wq_b_weight, idx_wq_b_weight, idx_weights_proj_weight, wkv_b_weight,
                          freqs_cis, k_cache, k_scale_cache, *, n_heads, qk_head_dim, qk_nope_head_dim,
                          kv_lora_rank, idx_n_heads, idx_head_dim, rope_head_dim, idx_softmax_scale,
                          index_topk, end_pos):
    """Query projection, absorbed nope query, indexer query path, index scores and top-k.
    Returns (q_nope, q_nope_absorbed, q_pe, topk_indices). ref: scripts/recipes_nvfp4.py:96-140."""
    bsz, seqlen, _ = qr.shape
    q = F.linear(qr, wq_b_weight).view(bsz, seqlen, n_heads, qk_head_dim)
    q_nope, q_pe = torch.split(q, [qk_nope_head_dim, qk_head_dim - qk_nope_head_dim], dim=-1)
    wkv_b = wkv_b_weight.view(n_heads, -1, kv_lora_rank)
    q_abs = torch.einsum("bshd,hdc->bshc", q_nope, wkv_b[:, :qk_nope_head_dim])
    idx_q = F.linear(qr, idx_wq_b_weight).view(bsz, seqlen, idx_n_heads, idx_head_dim)
    codes, scales = [], []
    for b in range(bsz):
        c, s, _ = index_prep(idx_q[b], freqs_cis, rope_dim=rope_head_dim)
        codes.append(c)
        scales.append(s)
    q_fp8, q_scale = torch.stack(codes), torch.stack(scales)             # [b, s, h, d], [b, s, h]
    weights = F.linear(normed_x.float(), idx_weights_proj_weight.float()) * idx_n_heads ** -0.5
    weights = weights * q_scale * idx_softmax_scale
    k_s = k_scale_cache[:bsz, :end_pos].reshape(bsz, end_pos).contiguous()
    k_cached = k_cache[:bsz, :end_pos].contiguous()
    score = fp8_index(q_fp8, weights, k_cached, k_s)
    return q_nope, q_abs, q_pe, score.topk(min(index_topk, end_pos), dim=-1)[1]


def fused_q_rope_quant(q_pe, freqs_cis):
    """Interleaved RoPE of the query's rope part. ref: scripts/recipes_nvfp4.py:142-151."""
    return apply_rotary_emb(q_pe, freqs_cis, True)
