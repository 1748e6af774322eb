"""Routed mixture-of-experts on the B200 kernels: routing, stable permutation, NVFP4
block-scaled grouped GEMMs over the sorted tokens, SwiGLU, weighted combine.

Replaces the Python expert loop of racetrack/models/deepseek.py:998-1022 (MoE.forward: bincount
with a host read-back, per-expert torch.where / gather / three linears / scatter-add) and the
per-token gathered-weight bmm of racetrack/realistic_bench.py:319-352. Nothing here reads
device data back to the host: expert offsets, the grouped-GEMM work list and the row windows of
an expert-parallel rank all stay on the device.

Expert weights are NVFP4 (e2m1 codes, e4m3 scale per 16 elements, one fp32 global scale per
expert), quantised once from bf16 with the same kernel that quantises activations.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib, ops


@dataclass
class NVFP4Experts:
    """NVFP4 weights of `count` consecutive experts, stacked along rows.

    w13: [count * 2*inter, hidden/2] codes (rows [0, inter) of an expert = gate projection w1,
         rows [inter, 2*inter) = up projection w3), tiled block scales, fp32 global scale/expert
    w2:  [count * hidden, inter/2] codes, tiled block scales, global scales
    """
    count: int
    hidden: int
    inter: int
    w13_codes: torch.Tensor
    w13_sf: torch.Tensor
    w13_gs: torch.Tensor
    w2_codes: torch.Tensor
    w2_sf: torch.Tensor
    w2_gs: torch.Tensor

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.w13_codes, self.w13_sf, self.w13_gs, self.w2_codes, self.w2_sf, self.w2_gs))


def quantize_experts(w13: torch.Tensor, w2: torch.Tensor) -> NVFP4Experts:
    """bf16 expert weights w13 [E, 2*inter, hidden], w2 [E, hidden, inter] -> NVFP4Experts.
    Each expert gets its own global scale (amax of that expert's matrix / (448*6))."""
    count, two_inter, hidden = w13.shape
    inter = two_inter // 2
    if w2.shape != (count, hidden, inter):
        raise RuntimeError("quantize_experts: w2 must be [E, hidden, inter]")
    if hidden % 256 or inter % 256:
        raise RuntimeError("quantize_experts: hidden and inter must be multiples of 256")
    parts13, parts2 = [], []
    for e in range(count):
        parts13.append(ops.fused_nvfp4_quant(w13[e], tiled_scales=True))
        parts2.append(ops.fused_nvfp4_quant(w2[e], tiled_scales=True))
    cat = torch.cat
    return NVFP4Experts(
        count, hidden, inter,
        cat([p[0] for p in parts13]), cat([p[1].view(torch.uint8) for p in parts13]),
        cat([p[2] for p in parts13]),
        cat([p[0] for p in parts2]), cat([p[1].view(torch.uint8) for p in parts2]),
        cat([p[2] for p in parts2]))


def _absmax_rows(x: torch.Tensor, up: Optional[torch.Tensor], window) -> torch.Tensor:
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    _lib.check(lib.rt_absmax_rows(x.data_ptr(), up.data_ptr() if up is not None else None,
                                  out.data_ptr(), x.shape[0], x.shape[1], x.stride(0),
                                  up.stride(0) if up is not None else 0,
                                  window[0].data_ptr() if window is not None else None,
                                  window[1].data_ptr() if window is not None else None,
                                  _lib.RT_BF16, ops._stream()), "rt_absmax_rows")
    return out


def moe_gather_nvfp4(codes: torch.Tensor, sf: torch.Tensor, sorted_pairs: torch.Tensor, topk: int,
                     tile_map: torch.Tensor, tile_count: torch.Tensor, total_rows: int):
    """MoE dispatch of token rows quantised once (codes [T, cols/2], row-major scales
    [T, cols/16] from ops.fused_nvfp4_quant): (codes [total_rows, cols/2] in expert order,
    tile-aligned scales) for the rows of a tile map (rt_moe_gather_nvfp4)."""
    cols = codes.shape[1] * 2
    max_tiles = tile_map.shape[0] // 2
    dev = codes.device
    out = torch.empty(total_rows, cols // 2, dtype=torch.uint8, device=dev)
    sf_out = torch.empty(max_tiles * (cols // 64) * 512, dtype=torch.uint8, device=dev)
    lib = _lib.load()
    _lib.check(lib.rt_moe_gather_nvfp4(
        codes.data_ptr(), sf.data_ptr(), sorted_pairs.data_ptr(), topk, out.data_ptr(),
        sf_out.data_ptr(), tile_map.data_ptr(), tile_count.data_ptr(), max_tiles, cols,
        ops._stream()), "rt_moe_gather_nvfp4")
    return out, sf_out


def swiglu_absmax_rows(gate: torch.Tensor, up: torch.Tensor, window):
    """(h, amax): h = bf16(silu(gate) * up) and max |h| over the rows of `window` (a pair of
    one-element device tensors [begin], [end], or None for all rows); rows outside the window
    are not written (rt_swiglu_absmax_rows)."""
    h = torch.empty(gate.shape, dtype=torch.bfloat16, device=gate.device)
    out = torch.empty(1, dtype=torch.float32, device=gate.device)
    lib = _lib.load()
    _lib.check(lib.rt_swiglu_absmax_rows(
        gate.data_ptr(), up.data_ptr(), h.data_ptr(), out.data_ptr(), gate.shape[0], gate.shape[1],
        gate.stride(0), up.stride(0), h.stride(0),
        window[0].data_ptr() if window is not None else None,
        window[1].data_ptr() if window is not None else None, _lib.RT_BF16, ops._stream()),
        "rt_swiglu_absmax_rows")
    return h, out


def moe_quant_nvfp4(x: torch.Tensor, tile_map: torch.Tensor, tile_count: torch.Tensor,
                    total_rows: int, *, amax: torch.Tensor, sorted_pairs=None, topk: int = 1,
                    up: Optional[torch.Tensor] = None):
    """NVFP4 codes [total_rows, cols/2] + tile-aligned block scales for the rows of a tile map
    (rt_moe_quant_nvfp4): gathers token rows when sorted_pairs is given, applies SwiGLU when
    `up` is given. Rows outside every tile are left unwritten."""
    cols = x.shape[-1]
    max_tiles = tile_map.shape[0] // 2
    dev = x.device
    codes = torch.empty(total_rows, cols // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(max_tiles * (cols // 64) * 512, dtype=torch.uint8, device=dev)
    gs = torch.empty(1, dtype=torch.float32, device=dev)
    lib = _lib.load()
    _lib.check(lib.rt_moe_quant_nvfp4(
        x.data_ptr(), up.data_ptr() if up is not None else None,
        sorted_pairs.data_ptr() if sorted_pairs is not None else None, topk, amax.data_ptr(),
        codes.data_ptr(), sf.data_ptr(), gs.data_ptr(), tile_map.data_ptr(), tile_count.data_ptr(),
        max_tiles, cols, x.stride(0), up.stride(0) if up is not None else 0, _lib.RT_BF16,
        ops._stream()), "rt_moe_quant_nvfp4")
    return codes, sf, gs


def fused_moe_experts(x: Optional[torch.Tensor], weights: torch.Tensor, indices: torch.Tensor,
                      experts: NVFP4Experts, *, n_experts: int, expert_begin: int = 0,
                      shared: Optional[torch.Tensor] = None,
                      out_dtype: torch.dtype = torch.bfloat16,
                      parts: Optional[dict] = None,
                      x_quant: Optional[tuple] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t] = sum over the token's routed experts owned here of w * expert(x[t]) (+ shared[t]).

    x [T, hidden] bf16; weights fp32 [T, k] and indices int64 [T, k] from fused_moe_route;
    `experts` holds the experts [expert_begin, expert_begin + experts.count) of n_experts (an
    expert-parallel rank passes its own slice and all-reduces the result). Expert arithmetic:
    NVFP4(x) . NVFP4(w13)^T -> bf16 gate/up -> NVFP4(swiglu) . NVFP4(w2)^T -> bf16, fp32 combine.
    `x_quant` = (codes [T, hidden/2], row-major block scales [T, hidden/16] as bytes, global scale
    [1]) hands over token rows that are quantised already (x may then be None): ranks of a
    token-sharded layer quantise their own rows and all-gather the codes.
    A dict passed as `parts` receives the intermediates (expert offsets, permutation, the two
    tensor-wide amax values, gate_up, h and the per-pair expert outputs) for stage-wise checks.
    """
    if x_quant is not None:
        tokens, hidden = x_quant[0].shape[0], x_quant[0].shape[1] * 2
    else:
        tokens, hidden = x.shape
    topk = indices.shape[1]
    pairs = tokens * topk
    count = experts.count
    offsets, sorted_pairs, pair_pos = ops.fused_moe_permute(indices, n_experts)
    max_tiles = (pairs + 127) // 128 + count
    tile_map, _tile_base, tile_count = ops.moe_tile_map(offsets, expert_begin, expert_begin + count,
                                                        max_tiles)
    local = count != n_experts
    window = (offsets[expert_begin:expert_begin + 1], offsets[expert_begin + count:expert_begin + count + 1]) \
        if local else None
    # dispatch: every token row is quantised once, then its codes and scales are copied into
    # expert order (the bf16 rows are not read topk times)
    if x_quant is not None:
        x_codes, x_sf, a_gs = x_quant
        x_amax = None
    else:
        x_amax = ops.tensor_absmax(x)
        x_codes, x_sf, a_gs = ops.fused_nvfp4_quant(x, amax=x_amax)
    a_codes, a_sf = moe_gather_nvfp4(x_codes, x_sf.view(torch.uint8), sorted_pairs, topk, tile_map,
                                     tile_count, pairs)
    gate_up = ops.gemm_nvfp4_grouped(a_codes, a_sf, a_gs, experts.w13_codes, experts.w13_sf,
                                     experts.w13_gs, tile_map, tile_count, n=2 * experts.inter,
                                     groups=count)
    gate, up = gate_up[:, :experts.inter], gate_up[:, experts.inter:]
    # SwiGLU once: this pass writes h and finds the tensor-wide amax its quantisation needs
    h, h_amax = swiglu_absmax_rows(gate, up, window)
    h_codes, h_sf, h_gs = moe_quant_nvfp4(h, tile_map, tile_count, pairs, amax=h_amax)
    expert_out = ops.gemm_nvfp4_grouped(h_codes, h_sf, h_gs, experts.w2_codes, experts.w2_sf,
                                        experts.w2_gs, tile_map, tile_count, n=hidden, groups=count)
    if parts is not None:
        parts.update(offsets=offsets, sorted_pairs=sorted_pairs, pair_pos=pair_pos, x_gs=a_gs, x_amax=x_amax,
                     gate_up=gate_up, h=h, h_amax=h_amax, expert_out=expert_out)
    return ops.fused_moe_combine(expert_out, pair_pos, weights, shared, pos_window=window,
                                 out_dtype=out_dtype, out=out)


def fused_moe_forward(x: torch.Tensor, gate_weight: torch.Tensor, gate_bias: Optional[torch.Tensor],
                      experts: NVFP4Experts, *, n_experts: int, n_groups: int, topk_groups: int,
                      topk: int, route_scale: float, score_func: str = "sigmoid",
                      expert_begin: int = 0, shared: Optional[torch.Tensor] = None,
                      out_dtype: torch.dtype = torch.bfloat16,
                      parts: Optional[dict] = None) -> torch.Tensor:
    """Gate (fp32 logits as in racetrack/models/deepseek.py:898, formed on the tensor cores from
    the bf16 operands with the fp32 accumulators kept) + routing kernel + experts."""
    if gate_weight.dtype == torch.float32:
        # a gate kept in fp32 (a module built outside the model's bf16 default): both halves of
        # the weight go through the tensor cores, so near-tied experts are ranked as in fp32
        logits = ops.linear_f32_weight(x, gate_weight)
    else:
        logits = ops.linear_bf16(x, gate_weight.to(torch.bfloat16), out_dtype=torch.float32)
    weights, indices = ops.fused_moe_route(logits, gate_bias, n_groups=n_groups,
                                           topk_groups=topk_groups, topk=topk,
                                           route_scale=route_scale, score_func=score_func)
    if parts is not None:
        parts.update(logits=logits, weights=weights, indices=indices)
    return fused_moe_experts(x, weights, indices, experts, n_experts=n_experts,
                             expert_begin=expert_begin, shared=shared, out_dtype=out_dtype,
                             parts=parts)
