"""GPU parity of the routed-MoE path (routing -> permutation -> NVFP4 grouped GEMMs ->
SwiGLU -> combine) against the CPU oracle, which runs the reference's expert loop on
dequantised NVFP4 operands."""
from __future__ import annotations

import pytest
import torch

from oracle import inputs as I
from oracle import ref_ops as R
from helpers import assert_bit_exact, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    from racetrack_b200 import moe, ops
    return ops, moe


def _setup(tokens, hidden, inter, n_experts, topk, seed=0):
    x = I.randn((tokens, hidden), seed + 1)
    w13 = I.randn((n_experts, 2 * inter, hidden), seed + 2, std=0.05)
    w2 = I.randn((n_experts, hidden, inter), seed + 3, std=0.05)
    g = torch.Generator().manual_seed(seed + 4)
    indices = torch.rand(tokens, n_experts, generator=g).topk(topk, dim=-1)[1]
    weights = torch.rand(tokens, topk, generator=g) + 0.1
    return x, w13, w2, weights, indices


def test_moe_quant_nvfp4_matches_plain_quantiser(mods):
    """The tile-aware, gather-fused quantiser writes the same codes and scales as the plain one
    run on the gathered rows; scales land in each expert's own 128-row tiles."""
    ops, moe = mods
    tokens, hidden, n_experts, topk = 300, 512, 8, 2
    x, _, _, _, indices = _setup(tokens, hidden, 256, n_experts, topk)
    xc, idx = x.cuda(), indices.cuda()
    offsets, sorted_pairs, _ = ops.fused_moe_permute(idx, n_experts)
    pairs = tokens * topk
    tile_map, tile_base, tile_count = ops.moe_tile_map(offsets, 0, n_experts, pairs // 128 + n_experts + 1)
    amax = ops.tensor_absmax(xc)
    codes, sf, gs = moe.moe_quant_nvfp4(xc, tile_map, tile_count, pairs, amax=amax,
                                        sorted_pairs=sorted_pairs, topk=topk)
    gathered = xc[(sorted_pairs // topk).long()]
    ref_codes, ref_sf, ref_gs = ops.fused_nvfp4_quant(gathered, amax=amax)
    assert_bit_exact(codes, ref_codes, "codes")
    assert_bit_exact(gs, ref_gs, "global scale")
    off = offsets.cpu().tolist()
    tb = tile_base.cpu().tolist()
    sf_cpu, ref_sf_cpu = sf.cpu(), ref_sf.view(torch.uint8).cpu()
    kt = hidden // 64
    for e in range(n_experts):
        rows = off[e + 1] - off[e]
        if rows == 0:
            continue
        tiles = (rows + 127) // 128
        seg = sf_cpu[tb[e] * kt * 512:(tb[e] + tiles) * kt * 512]
        o = R.sf_tiled_offsets(rows, hidden // 16)
        assert torch.equal(seg[o], ref_sf_cpu[off[e]:off[e + 1]]), f"scales of expert {e}"
        pad = torch.ones(seg.numel(), dtype=torch.bool)
        pad[o.flatten()] = False
        assert int(seg[pad].sum()) == 0, "padding rows of a scale tile must be zero"


@pytest.mark.parametrize("tokens,hidden,inter,n_experts,topk", [
    (64, 512, 256, 16, 4),
    (300, 1024, 512, 8, 2),      # several m-tiles per expert
    (5, 512, 256, 16, 4),        # most experts empty
])
def test_fused_moe_experts_matches_oracle(mods, tokens, hidden, inter, n_experts, topk):
    ops, moe = mods
    x, w13, w2, weights, indices = _setup(tokens, hidden, inter, n_experts, topk, seed=tokens)
    shared = I.randn((tokens, hidden), 99)
    experts = moe.quantize_experts(w13.cuda(), w2.cuda())
    y = moe.fused_moe_experts(x.cuda(), weights.cuda(), indices.cuda(), experts,
                              n_experts=n_experts, shared=shared.cuda())
    ops.tc_error_state()
    ref = R.moe_experts_nvfp4(x, weights, indices, w13, w2, shared_out=shared)
    err = rel_err(y, ref)
    assert err <= 1e-2, f"relative error {err}"
    # expert parallelism: two ranks owning half of the experts each sum to the full result
    # (each rank quantises swiglu(h) with the amax of ITS rows, so a rank is checked against the
    # oracle restricted to the same experts, and the sum against the full result more loosely)
    half = n_experts // 2
    parts = []
    for r in range(2):
        lo, hi = r * half, (r + 1) * half
        ex = moe.quantize_experts(w13[lo:hi].cuda(), w2[lo:hi].cuda())
        part = moe.fused_moe_experts(x.cuda(), weights.cuda(), indices.cuda(), ex,
                                     n_experts=n_experts, expert_begin=lo)
        ops.tc_error_state()
        ref_r = R.moe_experts_nvfp4(x, weights, indices, w13, w2, expert_range=(lo, hi))
        assert rel_err(part, ref_r) <= 1e-2, f"rank {r}"
        parts.append(part.float())
    total = parts[0] + parts[1] + shared.cuda().float()
    assert rel_err(total, ref) <= 1e-1


def test_fused_moe_forward_routes_and_combines(mods):
    """Gate + routing + experts at DeepSeek-V3.2 routing shape (256 experts, 8 groups, top-8),
    small expert matrices."""
    ops, moe = mods
    tokens, hidden, inter = 256, 1024, 256
    d = I.gate_inputs(tokens, hidden=hidden)
    w13 = I.randn((I.N_EXPERTS, 2 * inter, hidden), 5, std=0.02)
    w2 = I.randn((I.N_EXPERTS, hidden, inter), 6, std=0.02)
    experts = moe.quantize_experts(w13.cuda(), w2.cuda())
    kw = dict(n_groups=d["n_groups"], topk_groups=d["topk_groups"], topk=d["topk"],
              route_scale=d["route_scale"])
    y = moe.fused_moe_forward(d["hidden"].cuda(), d["w_gate"].cuda(), d["bias"].cuda(), experts,
                              n_experts=I.N_EXPERTS, **kw)
    ops.tc_error_state()
    # the oracle gets the GPU's routing decision: the logits GEMM differs in summation order
    logits = torch.nn.functional.linear(d["hidden"].cuda().float(), d["w_gate"].cuda().float())
    w, idx = ops.fused_moe_route(logits, d["bias"].cuda(), **kw)
    ref = R.moe_experts_nvfp4(d["hidden"], w.cpu(), idx.cpu(), w13, w2)
    assert rel_err(y, ref) <= 1e-2


@pytest.mark.parametrize("window", [None, (37, 211)])
def test_swiglu_absmax_rows_writes_h_and_its_amax(mods, window):
    """One pass: h = bf16(silu(gate) * up) for the rows of the window and max |h| over them,
    bit for bit what the SwiGLU kernel and the windowed amax kernel give separately."""
    ops, moe = mods
    rows, inter = 300, 512
    gate_up = I.randn((rows, 2 * inter), 31, std=2.0).cuda()
    gate, up = gate_up[:, :inter], gate_up[:, inter:]
    win = None
    if window is not None:
        win = (torch.tensor([window[0]], dtype=torch.int32).cuda(),
               torch.tensor([window[1]], dtype=torch.int32).cuda())
    h, amax = moe.swiglu_absmax_rows(gate, up, win)
    lo, hi = window if window is not None else (0, rows)
    ref = ops.fused_swiglu(gate, up)
    assert_bit_exact(h[lo:hi], ref[lo:hi], "h")
    assert_bit_exact(amax, moe._absmax_rows(gate, up, win), "amax")
    assert_bit_exact(amax, ref[lo:hi].float().abs().max().reshape(1), "amax of h")


@pytest.mark.parametrize("tokens,hidden,n_experts,topk", [(300, 512, 8, 2), (5, 7168, 16, 4),
                                                           (1000, 1024, 4, 1)])
def test_moe_gather_nvfp4_equals_gather_fused_quantiser(mods, tokens, hidden, n_experts, topk):
    """Quantising every token once and copying codes and scales into expert order gives the
    bytes the gather-fused quantiser writes (quantisation is per row), padding rows included."""
    ops, moe = mods
    x, _, _, _, indices = _setup(tokens, hidden, 256, n_experts, topk, seed=tokens)
    xc = x.cuda()
    offsets, sorted_pairs, _ = ops.fused_moe_permute(indices.cuda(), n_experts)
    pairs = tokens * topk
    tile_map, _, tile_count = ops.moe_tile_map(offsets, 0, n_experts, pairs // 128 + n_experts + 1)
    amax = ops.tensor_absmax(xc)
    ref_codes, ref_sf, ref_gs = moe.moe_quant_nvfp4(xc, tile_map, tile_count, pairs, amax=amax,
                                                   sorted_pairs=sorted_pairs, topk=topk)
    q_codes, q_sf, q_gs = ops.fused_nvfp4_quant(xc, amax=amax)
    codes, sf = moe.moe_gather_nvfp4(q_codes, q_sf.view(torch.uint8), sorted_pairs, topk, tile_map,
                                     tile_count, pairs)
    assert_bit_exact(q_gs, ref_gs, "global scale")
    assert_bit_exact(codes, ref_codes, "codes")
    used = int(tile_count[0]) * (hidden // 64) * 512
    assert_bit_exact(sf[:used], ref_sf[:used], "tiled scales")
