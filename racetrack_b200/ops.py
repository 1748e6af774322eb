"""Tensor-level entry points of the B200 backend.

Every function here takes CUDA tensors, allocates its outputs with torch's caching
allocator, and enqueues hand-written sm_100a kernels from librt_b200.so on the
current CUDA stream through the C ABI (include/rt_b200.h). Signatures and argument
meaning follow racetrack's own kernel contracts (the file:line each one mirrors is
given in its docstring); the ``fallback`` keyword every racetrack kernel receives is
accepted and ignored - there is no torch or CPU fallback, unsupported inputs raise.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import _lib

_BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("racetrack_b200 ops need CUDA tensors (there is no CPU path)")


def _require_bf16(name: str, t: torch.Tensor) -> None:
    if t.dtype != _BF16:
        raise RuntimeError(f"{name}: expected a bfloat16 tensor, got {t.dtype}")


def _weight_tag(w: torch.Tensor) -> int:
    if w.dtype == torch.bfloat16:
        return _lib.RT_BF16
    if w.dtype == torch.float32:
        return _lib.RT_F32
    raise RuntimeError(f"norm weight must be bfloat16 or float32, got {w.dtype}")


def _rows_view(x: torch.Tensor) -> torch.Tensor:
    """2-D [rows, cols] view whose row stride the kernels can take as is.

    Column slices of a wider matrix are passed through untouched; anything whose
    last dimension is not unit-stride or whose rows are not 16-byte aligned is copied.
    """
    cols = x.shape[-1]
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if x.dim() > 2:
        x = x.reshape(-1, cols)
    if x.stride(-1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    return x


# ---------------------------------------------------------------------------
# residual add + RMSNorm
# ---------------------------------------------------------------------------

def fused_residual_norm(update: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, *,
                        eps: float, fallback: Optional[Callable] = None):
    """(normed, hidden) with hidden = update + residual, normed = rms_norm(hidden) * weight.

    Contract of racetrack/models/deepseek.py:485-505 (RMSNorm.forward fallback and its
    ``_kernel_call("fused_residual_norm", ...)``).
    """
    del fallback
    _require_cuda(update, residual, weight)
    _require_bf16("fused_residual_norm", update)
    _require_bf16("fused_residual_norm", residual)
    if update.shape != residual.shape:
        raise RuntimeError("fused_residual_norm: update and residual shapes differ")
    cols = update.shape[-1]
    if weight.numel() != cols:
        raise RuntimeError("fused_residual_norm: weight length does not match the last dimension")
    u2, r2 = _rows_view(update), _rows_view(residual)
    w = weight.contiguous()
    normed = torch.empty(update.shape, dtype=update.dtype, device=update.device)
    hidden = torch.empty(update.shape, dtype=update.dtype, device=update.device)
    lib = _lib.load()
    _lib.check(lib.rt_residual_norm(u2.data_ptr(), r2.data_ptr(), w.data_ptr(), _weight_tag(w),
                                    normed.data_ptr(), hidden.data_ptr(), u2.shape[0], cols,
                                    u2.stride(0), r2.stride(0), float(eps), _lib.RT_BF16,
                                    _stream()), "rt_residual_norm")
    return normed, hidden


def fused_residual_norm_legacy(residual: torch.Tensor, update: torch.Tensor, weight: torch.Tensor,
                               *, eps: float, fallback: Optional[Callable] = None):
    """Legacy argument/return order ``(residual, update, w) -> (hidden, normed)`` of
    racetrack/runtime/triton_kernels.py:195-233 and racetrack/fx_patterns.py:116-122."""
    normed, hidden = fused_residual_norm(update, residual, weight, eps=eps, fallback=fallback)
    return hidden, normed


def fused_rms_norm(x: torch.Tensor, weight: torch.Tensor, *, eps: float,
                   fallback: Optional[Callable] = None) -> torch.Tensor:
    """rms_norm(x) * weight; partitions/_base.py:24-28, racetrack/models/deepseek.py:478-483."""
    del fallback
    _require_cuda(x, weight)
    _require_bf16("fused_rms_norm", x)
    cols = x.shape[-1]
    x2 = _rows_view(x)
    w = weight.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_rms_norm(x2.data_ptr(), w.data_ptr(), _weight_tag(w), out.data_ptr(),
                               x2.shape[0], cols, x2.stride(0), cols, float(eps), _lib.RT_BF16,
                               _stream()), "rt_rms_norm")
    return out


# ---------------------------------------------------------------------------
# MLA prologue
# ---------------------------------------------------------------------------

_INV_FREQ: dict[tuple, torch.Tensor] = {}


def _inv_freq(half: int, base: float, device: torch.device) -> torch.Tensor:
    """1 / base**(i/half), formed with the same torch ops as
    partitions/dsv3_2/model.py:39-45. The table is evaluated once on the host (powf differs
    by an ulp between host and device libraries, and a one-ulp frequency error grows with
    the position) and cached on the device."""
    key = (half, float(base), str(device))
    t = _INV_FREQ.get(key)
    if t is None:
        host = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / max(half, 1)))
        t = host.to(device).contiguous()
        _INV_FREQ[key] = t
    return t


def _freqs_table(freqs_cis: torch.Tensor, half: int) -> torch.Tensor:
    """[rows, half, 2] fp32 view of a complex64 freqs_cis tensor (no copy when contiguous)."""
    if not freqs_cis.is_complex():
        raise RuntimeError("freqs_cis must be a complex tensor")
    table = torch.view_as_real(freqs_cis.reshape(-1, half).contiguous())
    if table.dtype != torch.float32:
        table = table.float()
    return table


def _norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, positions, table, table_rows, eps, mode):
    _require_cuda(q_c, kv_c, k_pe, q_weight, kv_weight)
    for name, t in (("q_c", q_c), ("kv_c", kv_c), ("k_pe", k_pe)):
        _require_bf16(f"fused_norm_rope {name}", t)
    q2, kv2, k2 = _rows_view(q_c), _rows_view(kv_c), k_pe.reshape(-1, k_pe.shape[-1])
    if k2.stride(-1) != 1:
        k2 = k2.contiguous()
    tokens = q2.shape[0]
    if kv2.shape[0] != tokens or k2.shape[0] != tokens:
        raise RuntimeError("fused_norm_rope: q_c, kv_c and k_pe disagree on the token count")
    qw, kvw = q_weight.contiguous(), kv_weight.contiguous()
    if qw.dtype != kvw.dtype:
        kvw = kvw.to(qw.dtype)
    q_out = torch.empty(q_c.shape, dtype=q_c.dtype, device=q_c.device)
    kv_out = torch.empty(kv_c.shape, dtype=kv_c.dtype, device=kv_c.device)
    k_out = torch.empty(k_pe.shape, dtype=k_pe.dtype, device=k_pe.device)
    lib = _lib.load()
    _lib.check(lib.rt_norm_rope(q2.data_ptr(), qw.data_ptr(), kv2.data_ptr(), kvw.data_ptr(),
                                _weight_tag(qw), k2.data_ptr(),
                                positions.data_ptr() if positions is not None else None,
                                table.data_ptr(), table_rows,
                                q_out.data_ptr(), kv_out.data_ptr(), k_out.data_ptr(),
                                tokens, q2.shape[1], kv2.shape[1], k2.shape[1],
                                q2.stride(0), kv2.stride(0), k2.stride(0),
                                float(eps), mode, _lib.RT_BF16, _stream()), "rt_norm_rope")
    return q_out, kv_out, k_out


def fused_norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, positions, *, eps: float,
                    rope_base: float, fallback: Optional[Callable] = None):
    """(rms_norm(q_c), rms_norm(kv_c), apply_rope(k_pe)) with half-split RoPE.

    Contract of partitions/dsv3_2/model.py:84-99 and its call site :333-344; the three
    inputs are normally column slices of one [T, q_lora+kv_lora+rope] projection output.
    """
    del fallback
    half = k_pe.shape[-1] // 2
    pos = positions.reshape(-1)
    if pos.dtype != torch.int64:
        pos = pos.to(torch.int64)
    pos = pos.contiguous()
    table = _inv_freq(half, rope_base, k_pe.device)
    return _norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, pos, table, 0, eps, _lib.RT_ROPE_HALF)


def fused_norm_rope_interleaved(q_c, q_weight, kv_c, kv_weight, k_pe, freqs_cis, *, eps: float,
                                fallback: Optional[Callable] = None):
    """q_norm / kv_norm / interleaved rotary of k_pe as MLA.forward does them
    (racetrack/models/deepseek.py:766-776). ``freqs_cis`` is the complex64
    [seqlen, rope_dim/2] slice for the tokens; rows wrap around per batch element."""
    del fallback
    half = k_pe.shape[-1] // 2
    table = _freqs_table(freqs_cis, half)
    return _norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, None, table, table.shape[0], eps,
                      _lib.RT_ROPE_INTERLEAVED)


def _rope_heads(x: torch.Tensor, positions, table, table_rows, mode, inplace: bool):
    _require_cuda(x)
    _require_bf16("fused_rope", x)
    if x.dim() < 2:
        raise RuntimeError("fused_rope: expected [..., heads, rope_dim]")
    d = x.shape[-1]
    heads = x.shape[-2]
    x3 = x.reshape(-1, heads, d) if x.dim() != 3 else x
    ok = (x3.stride(2) == 1 and x3.stride(0) % 8 == 0 and x3.stride(1) % 8 == 0
          and x3.data_ptr() % 16 == 0)
    if not ok:
        if inplace:
            raise RuntimeError("fused_rope: in-place rotation needs a 16-byte aligned strided view")
        x3 = x3.contiguous()
    out3 = x3 if inplace else torch.empty((x3.shape[0], heads, d), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_rope(x3.data_ptr(), positions.data_ptr() if positions is not None else None,
                           table.data_ptr(), table_rows, out3.data_ptr(),
                           x3.shape[0], heads, d, x3.stride(0), x3.stride(1),
                           out3.stride(0), out3.stride(1), mode, _lib.RT_BF16, _stream()),
               "rt_rope")
    return x if inplace else out3.view(x.shape)


def fused_rope(x: torch.Tensor, freqs_cis: torch.Tensor, *, inplace: bool = False,
               fallback: Optional[Callable] = None) -> torch.Tensor:
    """Interleaved rotary embedding of x [batch, seq, heads, rope_dim] (or [seq, heads, rope_dim])
    by freqs_cis [seq, rope_dim/2]; racetrack/models/deepseek.py:604-624 with interleaved=True
    (kernel name as in partitions/dsv3_2/3336cdbd/kernels/triton/rope.py:57-62)."""
    del fallback
    half = x.shape[-1] // 2
    table = _freqs_table(freqs_cis, half)
    return _rope_heads(x, None, table, table.shape[0], _lib.RT_ROPE_INTERLEAVED, inplace)


def fused_rope_half(x: torch.Tensor, positions: torch.Tensor, *, rope_base: float = 10000.0,
                    inplace: bool = False, fallback: Optional[Callable] = None) -> torch.Tensor:
    """Half-split RoPE of x [tokens, heads, rope_dim] at integer positions;
    partitions/dsv3_2/model.py:55-81 (apply_rope), racetrack/realistic_bench.py:297-302."""
    del fallback
    half = x.shape[-1] // 2
    pos = positions.reshape(-1).to(torch.int64).contiguous()
    return _rope_heads(x, pos, _inv_freq(half, rope_base, x.device), 0, _lib.RT_ROPE_HALF, inplace)


def head_broadcast_(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """dst[t, h, :] = src[t, :] in place; dst is a [tokens, heads, dim] view (typically a column
    slice of the kv_b projection output), src is [tokens, dim]. The k_pe broadcast of
    racetrack/realistic_bench.py:311 without the torch.cat."""
    _require_cuda(dst, src)
    _require_bf16("head_broadcast_", dst)
    _require_bf16("head_broadcast_", src)
    tokens, heads, dim = dst.shape
    if src.shape != (tokens, dim) or dst.stride(2) != 1 or src.stride(1) != 1:
        raise RuntimeError("head_broadcast_: expected dst [T, H, D] and src [T, D], unit inner stride")
    lib = _lib.load()
    _lib.check(lib.rt_head_broadcast(src.data_ptr(), dst.data_ptr(), tokens, heads, dim,
                                     src.stride(0), dst.stride(0), dst.stride(1), _lib.RT_BF16,
                                     _stream()), "rt_head_broadcast")
    return dst


# ---------------------------------------------------------------------------
# SwiGLU and activation quantisation
# ---------------------------------------------------------------------------

def _gate_up(gate: torch.Tensor, up: torch.Tensor, who: str):
    _require_cuda(gate, up)
    _require_bf16(who, gate)
    _require_bf16(who, up)
    if gate.shape != up.shape:
        raise RuntimeError(f"{who}: gate and up shapes differ")
    return _rows_view(gate), _rows_view(up)


def fused_swiglu(gate: torch.Tensor, up: torch.Tensor, *,
                 fallback: Optional[Callable] = None) -> torch.Tensor:
    """(silu(gate.float()) * up.float()).type_as(gate); racetrack/models/deepseek.py:850-853."""
    del fallback
    g2, u2 = _gate_up(gate, up, "fused_swiglu")
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    lib = _lib.load()
    _lib.check(lib.rt_swiglu(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), g2.shape[0],
                             g2.shape[1], g2.stride(0), u2.stride(0), _lib.RT_BF16, _stream()),
               "rt_swiglu")
    return out


def fused_act_quant(x: torch.Tensor, *, out: Optional[tuple] = None, fallback: Optional[Callable] = None):
    """FP8 e4m3 codes [..., N] and fp32 scales [..., N/128]; racetrack/models/deepseek.py:85-107.
    ``out`` = (codes, scales) contiguous tensors of those shapes to write into (codes as
    float8_e4m3fn or uint8)."""
    del fallback
    _require_cuda(x)
    _require_bf16("fused_act_quant", x)
    n = x.shape[-1]
    if n % 128 != 0:
        raise RuntimeError(f"fused_act_quant: last dim ({n}) must be a multiple of 128")
    x2 = _rows_view(x)
    if out is not None:
        codes, scales = out
        if (codes.element_size() != 1 or scales.dtype != torch.float32 or not codes.is_contiguous()
                or not scales.is_contiguous() or tuple(codes.shape) != tuple(x.shape)
                or tuple(scales.shape) != (*x.shape[:-1], n // 128)):
            raise RuntimeError("fused_act_quant: out must be contiguous (1-byte codes [..., N], fp32 scales [..., N/128])")
    else:
        codes = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        scales = torch.empty(*x.shape[:-1], n // 128, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_act_quant_fp8(x2.data_ptr(), codes.data_ptr(), scales.data_ptr(),
                                    x2.shape[0], n, x2.stride(0), _lib.RT_BF16, _stream()),
               "rt_act_quant_fp8")
    return codes, scales


def fused_swiglu_quant(gate: torch.Tensor, up: torch.Tensor, *,
                       fallback: Optional[Callable] = None):
    """act_quant(swiglu(gate, up)) without materialising the bf16 product;
    benchmarks/gsm8k/flat_decode.py:132-136."""
    del fallback
    g2, u2 = _gate_up(gate, up, "fused_swiglu_quant")
    n = gate.shape[-1]
    if n % 128 != 0:
        raise RuntimeError(f"fused_swiglu_quant: last dim ({n}) must be a multiple of 128")
    codes = torch.empty(gate.shape, dtype=torch.float8_e4m3fn, device=gate.device)
    scales = torch.empty(*gate.shape[:-1], n // 128, dtype=torch.float32, device=gate.device)
    lib = _lib.load()
    _lib.check(lib.rt_swiglu_quant_fp8(g2.data_ptr(), u2.data_ptr(), codes.data_ptr(),
                                       scales.data_ptr(), g2.shape[0], n, g2.stride(0),
                                       u2.stride(0), _lib.RT_BF16, _stream()),
               "rt_swiglu_quant_fp8")
    return codes, scales


def tensor_absmax(x: torch.Tensor, up: Optional[torch.Tensor] = None) -> torch.Tensor:
    """max(|x|) over the whole tensor as a 1-element fp32 CUDA tensor (of swiglu(x, up)
    when ``up`` is given). Feeds the NVFP4 global scale."""
    _require_cuda(x)
    _require_bf16("tensor_absmax", x)
    if x.shape[-1] % 16 != 0:
        raise RuntimeError("tensor_absmax: last dim must be a multiple of 16")
    x2 = _rows_view(x)
    u2 = _rows_view(up) if up is not None else None
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_absmax(x2.data_ptr(), u2.data_ptr() if u2 is not None else None,
                             out.data_ptr(), x2.shape[0], x2.shape[1], x2.stride(0),
                             u2.stride(0) if u2 is not None else 0, _lib.RT_BF16, _stream()),
               "rt_absmax")
    return out


def sf_tiled_bytes(rows: int, cols: int) -> int:
    """Size of a 128x4-tiled NVFP4 block-scale buffer for a [rows, cols] tensor."""
    return ((rows + 127) // 128) * ((cols // 16 + 3) // 4) * 512


def fused_nvfp4_quant(x: torch.Tensor, *, up: Optional[torch.Tensor] = None,
                      amax: Optional[torch.Tensor] = None, tiled_scales: bool = False,
                      out: Optional[tuple] = None, fallback: Optional[Callable] = None):
    """NVFP4 quantisation -> (codes uint8 [..., N/2], block_scales float8_e4m3fn, global_scale fp32[1]).

    16-element blocks, e2m1 codes (element 2i in the low nibble), e4m3 block scale and
    one fp32 global scale = amax / (448 * 6). ``amax`` (1-element fp32 CUDA tensor) skips the
    abs-max pass when the caller already knows it. With ``up`` the quantised tensor is
    swiglu(x, up). ``tiled_scales`` selects the 128x4-tiled scale layout the block-scaled
    tensor-core GEMM consumes; otherwise scales are [..., N/16] row-major. ``out`` = (codes, scales)
    uint8 tensors of exactly those shapes to write into (e.g. a rank's rows of an exchange buffer).
    racetrack has no NVFP4 arithmetic; the format follows the build's stated configuration.
    """
    del fallback
    _require_cuda(x)
    _require_bf16("fused_nvfp4_quant", x)
    n = x.shape[-1]
    if n % 16 != 0:
        raise RuntimeError(f"fused_nvfp4_quant: last dim ({n}) must be a multiple of 16")
    x2 = _rows_view(x)
    u2 = None
    if up is not None:
        x2, u2 = _gate_up(x, up, "fused_nvfp4_quant")
    if amax is None:
        amax = tensor_absmax(x, up)
    rows = x2.shape[0]
    if out is not None:
        codes, sf = out
        want_sf = (sf_tiled_bytes(rows, n),) if tiled_scales else (*x.shape[:-1], n // 16)
        if (codes.dtype != torch.uint8 or sf.dtype != torch.uint8 or not codes.is_contiguous()
                or not sf.is_contiguous() or tuple(codes.shape) != (*x.shape[:-1], n // 2)
                or tuple(sf.shape) != tuple(want_sf)):
            raise RuntimeError("fused_nvfp4_quant: out must be contiguous uint8 (codes [..., N/2], scales)")
    else:
        codes = torch.empty(*x.shape[:-1], n // 2, dtype=torch.uint8, device=x.device)
        if tiled_scales:
            sf = torch.empty(sf_tiled_bytes(rows, n), dtype=torch.uint8, device=x.device)
        else:
            sf = torch.empty(*x.shape[:-1], n // 16, dtype=torch.uint8, device=x.device)
    gs = torch.empty(1, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_nvfp4_quant(x2.data_ptr(), u2.data_ptr() if u2 is not None else None,
                                  amax.data_ptr(), codes.data_ptr(), sf.data_ptr(), gs.data_ptr(),
                                  rows, n, x2.stride(0), u2.stride(0) if u2 is not None else 0,
                                  _lib.RT_SF_TILED128x4 if tiled_scales else _lib.RT_SF_ROWMAJOR,
                                  _lib.RT_BF16, _stream()), "rt_nvfp4_quant")
    return codes, sf.view(torch.float8_e4m3fn), gs


def fused_swiglu_nvfp4_quant(gate: torch.Tensor, up: torch.Tensor, **kw):
    """fused_nvfp4_quant of swiglu(gate, up)."""
    return fused_nvfp4_quant(gate, up=up, **kw)


# ---------------------------------------------------------------------------
# MoE routing / permutation / combine
# ---------------------------------------------------------------------------

def fused_moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], *, n_groups: int,
                    topk_groups: int, topk: int, route_scale: float,
                    score_func: str = "sigmoid", out: Optional[tuple] = None,
                    fallback: Optional[Callable] = None):
    """(weights fp32 [T, topk], indices int64 [T, topk]) from fp32 router logits [T, E];
    everything in Gate.forward after the logits GEMM (racetrack/models/deepseek.py:899-920).
    ``out`` = (weights, indices) contiguous tensors of those shapes to write into."""
    del fallback
    _require_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise RuntimeError("fused_moe_route: logits must be a 2-D float32 tensor")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    tokens, n_experts = logits.shape
    if out is not None:
        weights, indices = out
        if (weights.dtype != torch.float32 or indices.dtype != torch.int64 or not weights.is_contiguous()
                or not indices.is_contiguous() or tuple(weights.shape) != (tokens, topk)
                or tuple(indices.shape) != (tokens, topk)):
            raise RuntimeError("fused_moe_route: out must be contiguous (fp32 [T, topk], int64 [T, topk])")
    else:
        weights = torch.empty(tokens, topk, dtype=torch.float32, device=logits.device)
        indices = torch.empty(tokens, topk, dtype=torch.int64, device=logits.device)
    func = {"sigmoid": _lib.RT_SCORE_SIGMOID, "softmax": _lib.RT_SCORE_SOFTMAX,
            "topk_softmax": _lib.RT_SCORE_TOPK_SOFTMAX}[score_func]
    lib = _lib.load()
    _lib.check(lib.rt_moe_route(logits.data_ptr(), bias.data_ptr() if bias is not None else None,
                                weights.data_ptr(), indices.data_ptr(), tokens, n_experts,
                                logits.stride(0), n_groups, topk_groups, topk, float(route_scale),
                                func, _stream()), "rt_moe_route")
    return weights, indices


def fused_moe_permute(indices: torch.Tensor, n_experts: int):
    """Stable sort of (token, slot) pairs by expert ->
    (expert_offsets int32 [E+1], sorted_pairs int32 [T*topk], pair_pos int32 [T*topk]);
    replaces bincount + per-expert torch.where of racetrack/models/deepseek.py:1011-1017."""
    _require_cuda(indices)
    if indices.dtype != torch.int64 or indices.dim() != 2:
        raise RuntimeError("fused_moe_permute: indices must be a 2-D int64 tensor")
    indices = indices.contiguous()
    tokens, topk = indices.shape
    dev = indices.device
    lib = _lib.load()
    ws_bytes = int(lib.rt_moe_permute_workspace_bytes(tokens, topk, n_experts))
    workspace = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    sorted_pairs = torch.empty(tokens * topk, dtype=torch.int32, device=dev)
    pair_pos = torch.empty(tokens * topk, dtype=torch.int32, device=dev)
    _lib.check(lib.rt_moe_permute(indices.data_ptr(), offsets.data_ptr(), sorted_pairs.data_ptr(),
                                  pair_pos.data_ptr(), workspace.data_ptr(), tokens, topk,
                                  n_experts, _stream()), "rt_moe_permute")
    return offsets, sorted_pairs, pair_pos


def fused_moe_gather(x: torch.Tensor, sorted_pairs: torch.Tensor, topk: int) -> torch.Tensor:
    """x[sorted_pairs // topk] -> [T*topk, cols]; the x[idx] gathers of deepseek.py:1017."""
    _require_cuda(x, sorted_pairs)
    _require_bf16("fused_moe_gather", x)
    x2 = _rows_view(x)
    n_pairs = sorted_pairs.numel()
    out = torch.empty(n_pairs, x2.shape[1], dtype=x.dtype, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_moe_gather(x2.data_ptr(), sorted_pairs.data_ptr(), out.data_ptr(), n_pairs,
                                 topk, x2.shape[1], x2.stride(0), _lib.RT_BF16, _stream()),
               "rt_moe_gather")
    return out


def fused_moe_combine(expert_out: torch.Tensor, pair_pos: torch.Tensor, weights: torch.Tensor,
                      shared: Optional[torch.Tensor] = None, *, pos_begin: int = 0,
                      pos_end: Optional[int] = None,
                      pos_window: Optional[tuple] = None,
                      out_dtype: torch.dtype = torch.bfloat16,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t] = sum_s weights[t, s] * expert_out[pair_pos[t, s]] (+ shared[t]);
    racetrack/models/deepseek.py:1018-1022. ``pos_window`` = (begin, end) as 1-element int32
    CUDA tensors (entries of expert_offsets) restricts the sum to an expert-parallel rank's
    slice of the sorted range without a host read-back. ``out_dtype=torch.float32`` returns the
    fp32 sums (what the reference all-reduces across expert-parallel ranks before its cast)."""
    _require_cuda(expert_out, pair_pos, weights)
    _require_bf16("fused_moe_combine", expert_out)
    tokens, topk = weights.shape
    cols = expert_out.shape[-1]
    expert_out = expert_out.contiguous()
    weights = weights.to(torch.float32).contiguous()
    if shared is not None:
        _require_bf16("fused_moe_combine", shared)
        shared = shared.reshape(tokens, cols).contiguous()
    if pos_end is None:
        pos_end = tokens * topk
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("fused_moe_combine: out_dtype must be bfloat16 or float32")
    y = _out_buffer(out, (tokens, cols), out_dtype, expert_out.device)
    lib = _lib.load()
    _lib.check(lib.rt_moe_combine(expert_out.data_ptr(), pair_pos.data_ptr(), weights.data_ptr(),
                                  shared.data_ptr() if shared is not None else None, y.data_ptr(),
                                  tokens, topk, cols, pos_begin, pos_end,
                                  pos_window[0].data_ptr() if pos_window is not None else None,
                                  pos_window[1].data_ptr() if pos_window is not None else None,
                                  _lib.RT_F32 if out_dtype == torch.float32 else _lib.RT_BF16,
                                  _stream()),
               "rt_moe_combine")
    return y


# ---------------------------------------------------------------------------
# tensor-core GEMMs
# ---------------------------------------------------------------------------

def tc_error_state() -> None:
    """Synchronises the device and raises if a tensor-core kernel abandoned a bounded wait."""
    torch.cuda.synchronize()
    _lib.check(_lib.load().rt_tc_error_state(), "tensor-core kernel")


SPLITK_MAX_ROWS = 128          # linear_bf16 splits K for at most this many rows ...
SPLITK_MIN_WEIGHT = 1 << 20    # ... against a weight matrix of at least this many elements


def _out_buffer(out: Optional[torch.Tensor], shape: tuple, dtype: torch.dtype, device) -> torch.Tensor:
    """The caller's output buffer when it fits (contiguous, right shape and type: e.g. a buffer
    other ranks read over NVLink), else a fresh tensor."""
    if out is None:
        return torch.empty(shape, dtype=dtype, device=device)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or not out.is_contiguous():
        raise RuntimeError(f"out must be a contiguous {dtype} tensor of shape {tuple(shape)}")
    return out


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, *,
                out_dtype: torch.dtype = torch.bfloat16,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """F.linear(x, weight) for bf16 x [..., K] and weight [N, K] on the tcgen05 tensor cores
    (the bf16 branch of racetrack/models/deepseek.py:316-345 `linear`). out_dtype=torch.float32
    returns the fp32 accumulators (router logits, racetrack/models/deepseek.py:898)."""
    _require_cuda(x, weight)
    _require_bf16("linear_bf16 x", x)
    _require_bf16("linear_bf16 weight", weight)
    k = x.shape[-1]
    if weight.dim() != 2 or weight.shape[1] != k:
        raise RuntimeError("linear_bf16: weight must be [N, K] with K matching x")
    x2 = _rows_view(x)
    w = weight if (weight.stride(1) == 1 and weight.stride(0) % 8 == 0
                   and weight.data_ptr() % 16 == 0) else weight.contiguous()
    n = w.shape[0]
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("linear_bf16: out_dtype must be bfloat16 or float32")
    lib = _lib.load()
    rows = x2.shape[0]
    if 0 < rows <= SPLITK_MAX_ROWS and n * k >= SPLITK_MIN_WEIGHT:
        # a few decode tokens against a whole weight matrix: split the K range over the SMs
        splits = int(lib.rt_gemm_bf16_splitk_splits(rows, n, k))
        if splits > 1:
            # partial products per K range, then their sum in a fixed order: bit-reproducible,
            # and identical on every rank that forms the same replicated projection
            part = torch.empty(splits, rows, n, dtype=torch.float32, device=x.device)
            out = _out_buffer(out, (*x.shape[:-1], n), out_dtype, x.device)
            _lib.check(lib.rt_gemm_bf16_splitk(
                x2.data_ptr(), w.data_ptr(), part.data_ptr(), out.data_ptr(), rows, n, k,
                x2.stride(0), w.stride(0), n, n, splits,
                _lib.RT_F32 if out_dtype == torch.float32 else _lib.RT_BF16, _stream()),
                "rt_gemm_bf16_splitk")
            return out
    out = _out_buffer(out, (*x.shape[:-1], n), out_dtype, x.device)
    _lib.check(lib.rt_gemm_bf16(x2.data_ptr(), w.data_ptr(), out.data_ptr(), x2.shape[0], n, k,
                                x2.stride(0), w.stride(0), n,
                                _lib.RT_F32 if out_dtype == torch.float32 else _lib.RT_BF16,
                                _stream()), "rt_gemm_bf16")
    return out


def linear_bf16_batched(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """out[t, h, :] = x[t, h, :] @ weight[h]^T for x bf16 [T, H, K] (any token / head strides, e.g.
    a column slice of a projection output) and weight bf16 [H, N, K] -> bf16 [T, H, N], one launch
    for all heads. The absorbed projections of the MLA decode branch
    (racetrack/models/deepseek.py:799,810)."""
    _require_cuda(x, weight)
    _require_bf16("linear_bf16_batched x", x)
    _require_bf16("linear_bf16_batched weight", weight)
    if x.dim() != 3 or weight.dim() != 3 or weight.shape[0] != x.shape[1] or weight.shape[2] != x.shape[2]:
        raise RuntimeError("linear_bf16_batched: expected x [T, H, K] and weight [H, N, K]")
    if x.stride(2) != 1 or x.stride(0) % 8 or x.stride(1) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    if weight.stride(2) != 1 or weight.stride(0) % 8 or weight.stride(1) % 8 or weight.data_ptr() % 16:
        weight = weight.contiguous()
    tokens, heads, k = x.shape
    n = weight.shape[1]
    out = torch.empty(tokens, heads, n, dtype=torch.bfloat16, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_gemm_bf16_batched(x.data_ptr(), weight.data_ptr(), out.data_ptr(), heads, tokens, n, k,
                                        x.stride(0), x.stride(1), weight.stride(1), weight.stride(0),
                                        out.stride(0), out.stride(1), _stream()), "rt_gemm_bf16_batched")
    return out


_SPLIT_WEIGHTS: dict[tuple, tuple] = {}     # key -> (hi | lo halves, the weight itself)
_SPLIT_WEIGHTS_MAX = 256


def linear_f32_weight(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """F.linear(x.float(), weight) for bf16 x [..., K] and an fp32 weight [N, K] -> fp32 [..., N] on
    the tensor cores: the weight is split once into two bf16 matrices hi + lo (exact to 16
    mantissa bits: a relative 2^-17 per weight, below the fp32 round-off of a K-long sum), both
    multiply x with fp32 accumulation in one launch, and the two halves are added. The fp32
    projections of the model: the indexer's weights_proj (racetrack/models/deepseek.py:677)."""
    _require_cuda(x, weight)
    _require_bf16("linear_f32_weight x", x)
    if weight.dtype != torch.float32 or weight.dim() != 2:
        raise RuntimeError("linear_f32_weight: weight must be a 2-D float32 tensor")
    # The entry keeps the weight's storage alive, so its address cannot be handed to another
    # tensor while the entry exists; the version counter catches in-place updates.
    key = (weight.data_ptr(), tuple(weight.shape), tuple(weight.stride()), weight._version)
    entry = _SPLIT_WEIGHTS.get(key)
    if entry is None:
        hi = weight.to(torch.bfloat16)
        lo = (weight - hi.float()).to(torch.bfloat16)
        entry = (torch.cat((hi, lo)).contiguous(), weight.detach())
        while len(_SPLIT_WEIGHTS) >= _SPLIT_WEIGHTS_MAX:
            _SPLIT_WEIGHTS.pop(next(iter(_SPLIT_WEIGHTS)))
        _SPLIT_WEIGHTS[key] = entry
    split = entry[0]
    n = weight.shape[0]
    both = linear_bf16(x, split, out_dtype=torch.float32)
    return both[..., :n] + both[..., n:]


def quantize_weight_fp8(weight: torch.Tensor):
    """bf16/fp32 weight [N, K] -> (e4m3fn codes [N, K], fp32 scales [ceil(N/128), K/128]) with one
    scale = amax / 448 per 128 x 128 block: the checkpoint layout `weight` / `weight.scale` of
    racetrack/models/deepseek.py:361-371 (dequantised by `_block_dequant`, :148-161).
    Set-up time helper in plain torch (weights are quantised once, not on the hot path)."""
    n, k = weight.shape
    if k % 128:
        raise RuntimeError("quantize_weight_fp8: K must be a multiple of 128")
    nb = (n + 127) // 128
    w = torch.zeros(nb * 128, k, dtype=torch.float32, device=weight.device)
    w[:n] = weight.float()
    blocks = w.view(nb, 128, k // 128, 128)
    scale = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-4) / 448.0
    codes = (blocks / scale[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return codes.view(nb * 128, k)[:n].contiguous(), scale.contiguous()


def dequant_weight_fp8(weight: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3fn codes [N, K] with fp32 scales [ceil(N/128), ceil(K/128)] (one per 128 x 128 block)
    -> bf16 [N, K]; `weight_dequant` / `_block_dequant` of racetrack/models/deepseek.py:148-161,
    689-694. Set-up time helper in plain torch (a weight is converted once)."""
    if weight.dtype != torch.float8_e4m3fn or weight.dim() != 2:
        raise RuntimeError("dequant_weight_fp8: expected a 2-D float8_e4m3fn weight")
    n, k = weight.shape
    nb, kb = (n + 127) // 128, (k + 127) // 128
    if scale is None or tuple(scale.shape) != (nb, kb):
        raise RuntimeError(f"dequant_weight_fp8: scale must be [{nb}, {kb}]")
    full = scale.float().repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)[:, :k]
    return (weight.float() * full).to(torch.bfloat16)


def module_weight_bf16(linear) -> torch.Tensor:
    """The weight of a racetrack `Linear` (racetrack/models/deepseek.py:361-371) as a contiguous
    bf16 matrix: bf16 / fp32 weights are cast, FP8 weights (element size 1) are dequantised with
    their `weight.scale` block scales; an FP8 weight without scales is an error."""
    w = linear.weight
    if w.element_size() == 1:
        scale = getattr(w, "scale", None)
        if scale is None:
            scale = getattr(linear, "scale", None)
        if scale is None:
            raise RuntimeError("an FP8 weight needs its 128 x 128 block scales (weight.scale)")
        return dequant_weight_fp8(w.detach(), scale.detach()).contiguous()
    return w.detach().to(torch.bfloat16).contiguous()


def linear_fp8(x_codes: torch.Tensor, x_scales: torch.Tensor, w_codes: torch.Tensor,
               w_scales: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """FP8 block-scaled linear: fp8_gemm(a, a_s, b, b_s) of racetrack/models/deepseek.py:110-145
    -> bf16 [..., N]. x_codes / x_scales as fused_act_quant returns them."""
    _require_cuda(x_codes, x_scales, w_codes, w_scales)
    k = x_codes.shape[-1]
    n = w_codes.shape[0]
    if w_codes.shape[1] != k or x_codes.dtype != torch.float8_e4m3fn or w_codes.dtype != torch.float8_e4m3fn:
        raise RuntimeError("linear_fp8: expected e4m3fn codes with matching K")
    xc = x_codes.reshape(-1, k)
    xs = x_scales.reshape(-1, k // 128)
    if not (xc.is_contiguous() and xs.is_contiguous() and w_codes.is_contiguous()
            and w_scales.is_contiguous()):
        raise RuntimeError("linear_fp8: operands must be contiguous")
    if xs.dtype != torch.float32 or w_scales.dtype != torch.float32 \
            or w_scales.shape != ((n + 127) // 128, k // 128):
        raise RuntimeError("linear_fp8: scales must be fp32 [M, K/128] and [ceil(N/128), K/128]")
    out = _out_buffer(out, (*x_codes.shape[:-1], n), torch.bfloat16, x_codes.device)
    lib = _lib.load()
    _lib.check(lib.rt_gemm_fp8(xc.data_ptr(), xs.data_ptr(), w_codes.data_ptr(), w_scales.data_ptr(),
                               out.data_ptr(), xc.shape[0], n, k, k, k, n, _stream()), "rt_gemm_fp8")
    return out


def linear_fp8_act(x: torch.Tensor, w_codes: torch.Tensor, w_scales: torch.Tensor,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`linear(x, weight)` with an FP8 weight as racetrack/models/deepseek.py:343-345 runs it:
    act_quant(x) then the FP8 block-scaled GEMM."""
    codes, scales = fused_act_quant(x)
    return linear_fp8(codes, scales, w_codes, w_scales, out=out)


def moe_tile_map(offsets: torch.Tensor, g_begin: int, g_end: int, max_tiles: int):
    """Device-side work lists of the grouped GEMM for groups [g_begin, g_end) of the row
    offsets written by fused_moe_permute -> (tile_map int32 [2 * max_tiles, 4], tile_base
    int32 [groups + 1], tile_count int32 [2]). Rows [0, tile_count[0]) of tile_map are the
    128-row tiles (one scale row tile each); rows [max_tiles, max_tiles + tile_count[1]) cut
    the same rows into tiles of up to 256 rows for the CTA-pair GEMM. No host
    synchronisation."""
    _require_cuda(offsets)
    if offsets.dtype != torch.int32:
        raise RuntimeError("moe_tile_map: offsets must be int32")
    dev = offsets.device
    tile_map = torch.empty(2 * max_tiles, 4, dtype=torch.int32, device=dev)
    tile_base = torch.empty(g_end - g_begin + 1, dtype=torch.int32, device=dev)
    tile_count = torch.empty(2, dtype=torch.int32, device=dev)
    lib = _lib.load()
    _lib.check(lib.rt_moe_tile_map(offsets.data_ptr(), g_begin, g_end, tile_map.data_ptr(),
                                   tile_base.data_ptr(), tile_count.data_ptr(), max_tiles,
                                   _stream()), "rt_moe_tile_map")
    return tile_map, tile_base, tile_count


def gemm_nvfp4_grouped(a_codes: torch.Tensor, a_sf: torch.Tensor, a_gs: torch.Tensor,
                       b_codes: torch.Tensor, b_sf: torch.Tensor, b_gs: torch.Tensor,
                       tile_map: torch.Tensor, tile_count: torch.Tensor, *, n: int,
                       groups: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Block-scaled NVFP4 grouped GEMM (see rt_gemm_nvfp4_grouped in include/rt_b200.h).

    a_codes uint8 [rows, K/2]; a_sf tiled e4m3 scales (bytes); a_gs fp32 [1];
    b_codes uint8 [groups * n, K/2]; b_sf tiled scales per group; b_gs fp32 [groups];
    tile_map / tile_count as moe_tile_map returns them.
    Returns bf16 [rows, n]; rows outside every tile are left untouched."""
    _require_cuda(a_codes, a_sf, a_gs, b_codes, b_sf, b_gs, tile_map, tile_count)
    rows, kh = a_codes.shape
    if b_codes.shape != (groups * n, kh):
        raise RuntimeError("gemm_nvfp4_grouped: b_codes must be [groups * n, K/2]")
    if not (a_codes.is_contiguous() and b_codes.is_contiguous()):
        raise RuntimeError("gemm_nvfp4_grouped: code tensors must be contiguous")
    if out is None:
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=a_codes.device)
    lib = _lib.load()
    _lib.check(lib.rt_gemm_nvfp4_grouped(a_codes.data_ptr(), a_sf.data_ptr(), a_gs.data_ptr(),
                                         b_codes.data_ptr(), b_sf.data_ptr(), b_gs.data_ptr(),
                                         out.data_ptr(), tile_map.data_ptr(),
                                         tile_count.data_ptr(), tile_map.shape[0] // 2, rows,
                                         groups,
                                         n, 2 * kh, out.stride(0), _stream()),
               "rt_gemm_nvfp4_grouped")
    return out


def index_prep(x: torch.Tensor, freqs_cis: torch.Tensor, *, positions: Optional[torch.Tensor] = None,
               ln_weight: Optional[torch.Tensor] = None, ln_bias: Optional[torch.Tensor] = None,
               eps: float = 1e-6, return_rotated: bool = False):
    """The indexer's path from projected rows to FP8 in one pass (racetrack/models/deepseek.py:
    659-676): [LayerNorm for keys] -> non-interleaved RoPE on the first 64 dims -> Hadamard
    rotation -> act_quant.

    x bf16 [S, H, 128] (H = 1 for keys); freqs_cis complex64 [table, 32]; positions int64 [S]
    (default 0..S-1). Returns (codes float8_e4m3fn [S, H, 128], scales fp32 [S, H]) and, on
    request, the rotated bf16 tensor that was quantised."""
    _require_cuda(x, freqs_cis)
    _require_bf16("index_prep", x)
    if x.dim() != 3 or x.shape[-1] != 128:
        raise RuntimeError("index_prep: x must be [S, H, 128]")
    s_len, heads, dim = x.shape
    x2 = x.reshape(s_len * heads, dim)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    fr = torch.view_as_real(freqs_cis).to(torch.float32).contiguous()
    if fr.shape[-2:] != (32, 2):
        raise RuntimeError("index_prep: freqs_cis must be [table, 32] complex")
    codes = torch.empty(s_len, heads, dim, dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty(s_len, heads, dtype=torch.float32, device=x.device)
    rotated = torch.empty(s_len, heads, dim, dtype=torch.bfloat16, device=x.device) \
        if return_rotated else None
    lw = ln_weight.to(torch.float32).contiguous() if ln_weight is not None else None
    lb = ln_bias.to(torch.float32).contiguous() if ln_bias is not None else None
    pos = positions.to(torch.int64).contiguous() if positions is not None else None
    lib = _lib.load()
    _lib.check(lib.rt_index_prep(
        x2.data_ptr(), lw.data_ptr() if lw is not None else None,
        lb.data_ptr() if lb is not None else None, pos.data_ptr() if pos is not None else None,
        fr.data_ptr(), fr.shape[0], heads, codes.data_ptr(), scales.data_ptr(),
        rotated.data_ptr() if rotated is not None else None, s_len * heads, dim, 64,
        x2.stride(0), float(eps), _lib.RT_BF16, _stream()), "rt_index_prep")
    return (codes, scales, rotated) if return_rotated else (codes, scales)


def fp8_index(q: torch.Tensor, weights: torch.Tensor, k: torch.Tensor, k_scale: torch.Tensor, *,
              causal_offset: Optional[int] = None) -> torch.Tensor:
    """Index scores of the sparse-attention indexer (racetrack/models/deepseek.py:164-176):
    scores[b, m, n] = k_scale[b, n] * sum_h weights[b, m, h] * relu(q[b, m, h, :] . k[b, n, :]).

    q float8_e4m3fn [B, M, H, 128], weights fp32 [B, M, H], k float8_e4m3fn [B, N, 128] (may be the
    first N rows of longer per-sequence caches), k_scale fp32 [B, N] or [B, N, 1]; the batch
    dimension may be missing. With causal_offset = c, keys n > m + c get -inf (the mask the
    reference adds before top-k). One launch for all sequences. Returns fp32 [B, M, N]."""
    _require_cuda(q, weights, k, k_scale)
    if q.dtype != torch.float8_e4m3fn or k.dtype != torch.float8_e4m3fn:
        raise RuntimeError("fp8_index: q and k must be float8_e4m3fn")
    m, h, d = q.shape[-3:]
    n = k.shape[-2]
    lead = q.shape[:-3]
    if k.shape[:-2] != lead or len(lead) > 1:
        raise RuntimeError("fp8_index: q [B, M, H, D] and k [B, N, D] must share at most one batch dim")
    batch = lead[0] if lead else 1
    q3 = q.reshape(batch, m, h, d).contiguous()
    k3 = k.reshape(batch, n, d)
    if k3.stride(2) != 1 or k3.stride(1) != d or (batch > 1 and k3.stride(0) % d):
        k3 = k3.contiguous()
    w3 = weights.reshape(batch, m, h).to(torch.float32).contiguous()
    ks = k_scale.reshape(batch, n).to(torch.float32)
    if ks.stride(1) != 1:
        ks = ks.contiguous()
    scores = torch.empty(batch, m, n, dtype=torch.float32, device=q.device)
    lib = _lib.load()
    _lib.check(lib.rt_fp8_index_batched(
        q3.data_ptr(), w3.data_ptr(), k3.data_ptr(), ks.data_ptr(), scores.data_ptr(), batch, m, h,
        n, d, scores.stride(1), -1 if causal_offset is None else int(causal_offset),
        (k3.stride(0) // d) if batch > 1 else n, ks.stride(0) if batch > 1 else n, scores.stride(0),
        _stream()), "rt_fp8_index_batched")
    return scores.reshape(*lead, m, n)


def index_topk(scores: torch.Tensor, topk: int) -> torch.Tensor:
    """Indices (int32 [..., M, min(topk, N)], ascending) of the largest scores of every row
    (racetrack/models/deepseek.py:683; the reference uses them as a set)."""
    _require_cuda(scores)
    if scores.dtype != torch.float32:
        raise RuntimeError("index_topk: scores must be float32")
    n = scores.shape[-1]
    s2 = scores.reshape(-1, n)
    if s2.stride(1) != 1:
        s2 = s2.contiguous()
    kk = min(int(topk), n)
    out = torch.empty(s2.shape[0], kk, dtype=torch.int32, device=scores.device)
    lib = _lib.load()
    _lib.check(lib.rt_index_topk(s2.data_ptr(), out.data_ptr(), s2.shape[0], n, s2.stride(0), kk,
                                 _stream()), "rt_index_topk")
    return out.reshape(*scores.shape[:-1], kk)


def mla_sparse_decode(q_abs: torch.Tensor, q_pe: torch.Tensor, kv_cache: torch.Tensor,
                      pe_cache: torch.Tensor, indices: Optional[torch.Tensor],
                      softmax_scale: float) -> torch.Tensor:
    """Sparse multi-query attention of the MLA decode step (racetrack/models/deepseek.py:793-810):
    q_abs bf16 [B, H, 512] (q_nope times the key half of wkv_b), q_pe bf16 [B, H, 64], kv_cache
    bf16 [B, S, 512], pe_cache bf16 [B, S, 64], indices int32 [B, n_sel] of the keys each sequence
    attends to (the indexer's top-k; None = all S keys) -> bf16 [B, H, 512], the softmax-weighted
    sum of the selected latent rows."""
    _require_cuda(q_abs)
    for name, t in (("q_abs", q_abs), ("q_pe", q_pe), ("kv_cache", kv_cache), ("pe_cache", pe_cache)):
        if t.dtype != torch.bfloat16 or t.dim() != 3 or t.stride(2) != 1:
            raise RuntimeError(f"mla_sparse_decode: {name} must be bf16 [*, *, d] with a contiguous last dim")
    batch, heads, dim = q_abs.shape
    keys = kv_cache.shape[1]
    if dim != 512 or kv_cache.shape[2] != 512 or q_pe.shape != (batch, heads, 64) or \
            pe_cache.shape != (batch, keys, 64) or kv_cache.shape[0] != batch:
        raise RuntimeError("mla_sparse_decode: shapes must be [B,H,512], [B,H,64], [B,S,512], [B,S,64]")
    if indices is not None:
        if indices.dtype != torch.int32 or indices.dim() != 2 or indices.shape[0] != batch:
            raise RuntimeError("mla_sparse_decode: indices must be int32 [B, n_sel]")
        if indices.stride(1) != 1:
            indices = indices.contiguous()
        n_sel = indices.shape[1]
    else:
        n_sel = keys
    lib = _lib.load()
    splits = int(lib.rt_mla_sparse_decode_splits(batch, heads, n_sel))
    dev = q_abs.device
    out = torch.empty(batch, heads, 512, dtype=torch.bfloat16, device=dev)
    part_o = torch.empty(batch * splits * heads * 512, dtype=torch.float32, device=dev)
    part_ml = torch.empty(batch * splits * heads * 2, dtype=torch.float32, device=dev)
    _lib.check(lib.rt_mla_sparse_decode(
        q_abs.data_ptr(), q_pe.data_ptr(), kv_cache.data_ptr(), pe_cache.data_ptr(),
        indices.data_ptr() if indices is not None else None, out.data_ptr(), part_o.data_ptr(),
        part_ml.data_ptr(), batch, heads, keys, n_sel, q_abs.stride(0), q_abs.stride(1),
        q_pe.stride(0), q_pe.stride(1), kv_cache.stride(0), kv_cache.stride(1), pe_cache.stride(0),
        pe_cache.stride(1), indices.stride(0) if indices is not None else 0, splits,
        float(softmax_scale), _stream()), "rt_mla_sparse_decode")
    return out


def attention_prefill(q: torch.Tensor, k_nope: torch.Tensor, k_pe: Optional[torch.Tensor],
                      v: torch.Tensor, softmax_scale: Optional[float] = None, *,
                      quantized: bool = False, out: Optional[tuple] = None):
    """Causal attention over [tokens, heads, dim] tensors on the tensor cores
    (racetrack/runtime/torch_ops.py:97-110; the attention core of
    racetrack/realistic_bench.py:304-313): q bf16 [T, H, nope + rope]; the key of head h is
    [k_nope[:, h] | k_pe] with k_nope [T, H, nope] and k_pe [T, rope] (one rope key per token for
    all heads, never broadcast in memory) or [T, H, rope], or None; v [T, H, v_dim]. Operands may
    be strided views (column slices of projection outputs). Returns bf16 [T, H, v_dim].

    quantized=True returns act_quant of that output instead, (FP8 codes [T, H * v_dim], fp32 scales
    [T, H]), bit for bit what fused_act_quant makes of it; for the 128 + 64 / 128 head shape the
    attention kernel writes them from its own epilogue, otherwise the quantiser runs behind it.
    ``out`` = (codes, scales) to write into (contiguous, 1-byte codes)."""
    _require_cuda(q, k_nope, v)
    tokens, heads, qk = q.shape
    nope = k_nope.shape[-1]
    rope = qk - nope
    v_dim = v.shape[-1]
    ok = k_nope.shape == (tokens, heads, nope) and v.shape == (tokens, heads, v_dim) and rope >= 0
    if rope:
        ok = ok and k_pe is not None and k_pe.shape in ((tokens, rope), (tokens, heads, rope))
    if not ok:
        raise RuntimeError("attention_prefill: expected q [T,H,nope+rope], k_nope [T,H,nope], "
                           "k_pe [T,rope] or [T,H,rope], v [T,H,v]")

    def view(t, name):
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"attention_prefill: {name} must be bfloat16")
        if t.stride(-1) != 1 or any(st % 8 for st in t.stride()[:-1]) or t.data_ptr() % 16:
            t = t.contiguous()
        return t
    q, k_nope, v = view(q, "q"), view(k_nope, "k_nope"), view(v, "v")
    kp_ts = kp_hs = 0
    if rope:
        k_pe = view(k_pe, "k_pe")
        kp_ts = k_pe.stride(0)
        kp_hs = k_pe.stride(1) if k_pe.dim() == 3 else 0
        if k_pe.dim() == 3 and kp_hs == 0:         # an expanded view: the shared form
            k_pe = k_pe[:, 0]
    if softmax_scale is None:
        softmax_scale = qk ** -0.5
    lib = _lib.load()
    if quantized:
        if out is not None:
            codes, scales = out
            if (codes.element_size() != 1 or scales.dtype != torch.float32 or not codes.is_contiguous()
                    or not scales.is_contiguous() or tuple(codes.shape) != (tokens, heads * v_dim)
                    or tuple(scales.shape) != (tokens, heads * v_dim // 128)):
                raise RuntimeError("attention_prefill: out must be contiguous (1-byte codes [T, H*v], fp32 scales [T, H*v/128])")
        if (nope, rope, v_dim) != (128, 64, 128):
            # no fused epilogue for this head shape: the quantiser runs behind the attention kernel
            return fused_act_quant(attention_prefill(q, k_nope, k_pe, v, softmax_scale)
                                   .view(tokens, heads * v_dim), out=out)
        if out is None:
            codes = torch.empty(tokens, heads * v_dim, dtype=torch.float8_e4m3fn, device=q.device)
            scales = torch.empty(tokens, heads, dtype=torch.float32, device=q.device)
        _lib.check(lib.rt_attn_causal_prefill_fp8(
            q.data_ptr(), k_nope.data_ptr(), k_pe.data_ptr(), v.data_ptr(), codes.data_ptr(),
            scales.data_ptr(), tokens, heads, nope, rope, v_dim, q.stride(0), q.stride(1),
            k_nope.stride(0), k_nope.stride(1), kp_ts, kp_hs, v.stride(0), v.stride(1),
            float(softmax_scale), _stream()), "rt_attn_causal_prefill_fp8")
        return codes, scales
    out = torch.empty(tokens, heads, v_dim, dtype=torch.bfloat16, device=q.device)
    _lib.check(lib.rt_attn_causal_prefill(
        q.data_ptr(), k_nope.data_ptr(), k_pe.data_ptr() if rope else None, v.data_ptr(),
        out.data_ptr(), tokens, heads, nope, rope, v_dim, q.stride(0), q.stride(1),
        k_nope.stride(0), k_nope.stride(1), kp_ts, kp_hs, v.stride(0), v.stride(1),
        out.stride(0), out.stride(1), float(softmax_scale), _stream()), "rt_attn_causal_prefill")
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """racetrack/runtime/torch_ops.py:97-110 with whole keys k [T, H, qk] (qk <= 192): the first
    min(qk, 128) dims take the place of the nope part, the rest that of a per-head rope part."""
    nope = min(k.shape[-1], 128)
    return attention_prefill(q, k[..., :nope], k[..., nope:] if k.shape[-1] > nope else None, v)


def attention_prefill_schedule(schedule: int) -> int:
    """Selects the schedule of attention_prefill for this process (0 default = by shape and length,
    1 one CTA per 256 query rows, 2 CTA pairs with key tiles of 256 where the head shape allows)
    and returns the previous setting."""
    return int(_lib.load().rt_attn_prefill_schedule(int(schedule)))


def gemm_bf16_schedule(schedule: int) -> int:
    """Selects the schedule of the bf16 GEMM for this process (0 default = by size, 1 single-CTA
    128 x 256 tiles, 2 CTA pairs with 256 x 256 tiles where K % 64 == 0) and returns the
    previous setting."""
    return int(_lib.load().rt_gemm_bf16_schedule(int(schedule)))


def gemm_nvfp4_schedule(schedule: int) -> int:
    """Selects the schedule of the NVFP4 GEMM for this process (0 default = CTA pairs,
    1 single-CTA 128 x 128 tiles, 2 CTA pairs) and returns the previous setting."""
    return int(_lib.load().rt_gemm_nvfp4_schedule(int(schedule)))


_DENSE_TILES: dict[tuple, tuple] = {}


def linear_nvfp4(x_codes: torch.Tensor, x_sf: torch.Tensor, x_gs: torch.Tensor,
                 w_codes: torch.Tensor, w_sf: torch.Tensor, w_gs: torch.Tensor) -> torch.Tensor:
    """Dense NVFP4 linear layer: operands as fused_nvfp4_quant(..., tiled_scales=True) returns
    them (x [M, K], weight [N, K]) -> bf16 [M, N]."""
    m = x_codes.shape[0]
    key = (m, str(x_codes.device))
    tiles = _DENSE_TILES.get(key)
    if tiles is None:
        offsets = torch.tensor([0, m], dtype=torch.int32, device=x_codes.device)
        tm, _, tc = moe_tile_map(offsets, 0, 1, (m + 127) // 128 + 1)
        tiles = (tm, tc)
        _DENSE_TILES[key] = tiles
    return gemm_nvfp4_grouped(x_codes, x_sf.view(torch.uint8), x_gs, w_codes,
                              w_sf.view(torch.uint8), w_gs.reshape(1), tiles[0], tiles[1],
                              n=w_codes.shape[0], groups=1)
