"""GPU parity tests of the tcgen05 GEMMs against an fp32 torch matmul of the same operands."""
from __future__ import annotations

import pytest
import torch

from oracle import inputs as I
from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from racetrack_b200 import ops as _ops
    return _ops


def _ref(x, w):
    return x.float() @ w.float().t()


@pytest.fixture(params=[1, 2], ids=["single_cta", "cta_pair"])
def bf16_schedule(request, ops):
    """Runs a test under both schedules of the bf16 GEMM (single-CTA 128 x 256 tiles, CTA pairs
    with 256 x 256 tiles; a K that is not a multiple of 64 always takes the single-CTA path)
    and restores the default."""
    previous = ops.gemm_bf16_schedule(request.param)
    yield request.param
    ops.gemm_bf16_schedule(previous)


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 64),        # one tile, one K block
    (128, 256, 256),       # one wide tile
    (256, 512, 512),       # 2 x 2 tiles
    (1, 2112, 7168),       # decode row, ragged N
    (100, 136, 72),        # ragged everywhere (multiples of 8)
    (4096, 2112, 7168),    # qkv_a projection
    (2048, 24576, 1536),   # q_b projection, all 128 heads
    (1000, 7168, 2048),    # expert down projection
    (300, 264, 192),       # pair: odd number of K blocks (the second half of a stage is empty)
    (257, 520, 64),        # pair: one K block, tiles ragged in both directions
])
def test_linear_bf16(ops, bf16_schedule, m, n, k):
    x = I.randn((m, k), 100 + m).cuda()
    w = I.randn((n, k), 200 + n, std=0.05).cuda()
    out = ops.linear_bf16(x, w)
    ops.tc_error_state()
    ref = _ref(x, w)
    assert out.shape == (m, n)
    err = rel_err(out, ref)
    assert err <= 1e-2, f"relative error {err}"
    # element-wise: bf16 rounding of an fp32 accumulation, allow 1 ulp + accumulation noise
    diff = (out.float() - ref).abs()
    tol = 2.0 ** -7 * ref.abs() + 2e-3 * ref.abs().max()
    assert bool((diff <= tol).all()), f"worst {float(diff.max())}"


def test_linear_bf16_strided_inputs_and_linearity(ops, bf16_schedule):
    big = I.randn((300, 1024), 5).cuda()
    w = I.randn((512, 512), 6, std=0.05).cuda()
    x = big[:, 256:768]                      # column slice: row pitch 1024
    out = ops.linear_bf16(x, w)
    ops.tc_error_state()
    assert rel_err(out, _ref(x, w)) <= 1e-2
    # exact linearity in powers of two: (2x) W^T == 2 (x W^T) bit for bit
    out2 = ops.linear_bf16((x * 2).contiguous(), w)
    assert torch.equal(out2, out * 2)
    # leading dims
    out3 = ops.linear_bf16(x.contiguous().view(3, 100, 512), w)
    assert out3.shape == (3, 100, 512) and torch.equal(out3.view(300, 512), out)


@pytest.mark.parametrize("m", [4096, 1, 77])
def test_router_logits_fp32_output(ops, bf16_schedule, m):
    """fp32 logits of bf16 hidden states and gate weights ([256, 7168]): every product is exact
    in fp32; the tensor-core accumulator aligns addends with a few bits less than an IEEE fp32
    sum, which shows as ~1e-5 of the largest logit."""
    x = I.randn((m, I.HIDDEN), 9).cuda()
    w = I.randn((I.N_EXPERTS, I.HIDDEN), 10, std=0.02).cuda()
    out = ops.linear_bf16(x, w, out_dtype=torch.float32)
    ops.tc_error_state()
    assert out.dtype == torch.float32 and out.shape == (m, I.N_EXPERTS)
    ref = (x.double() @ w.double().t())
    err = float((out.double() - ref).abs().max() / ref.abs().max())
    assert err <= 3e-5, f"relative error {err}"
    # same top-8 as the fp32 reference GEMM except on near-ties
    ref32 = torch.nn.functional.linear(x.float(), w.float())
    same = (out.topk(8, dim=-1)[1] == ref32.topk(8, dim=-1)[1]).all(dim=-1).float().mean()
    assert float(same) >= 0.99


# ---------------------------------------------------------------------------
# FP8 block-scaled GEMM
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("m,n,k", [
    (128, 256, 128),       # one tile, one K block
    (128, 256, 1024),      # partial buffers alternate, stages wrap
    (256, 512, 512),
    (100, 2112, 7168),     # qkv_a: ragged M, N not a multiple of 128 or 256
    (1, 7168, 2048),       # decode row
    (2048, 24576, 1536),   # q_b
    (1024, 7168, 16384),   # w_o: 128 K blocks
    (300, 520, 384),       # three K blocks, tiles ragged in both directions
])
def test_linear_fp8_block_scaled(ops, m, n, k):
    from oracle import ref_ops as R
    x = I.randn((m, k), 500 + m).cuda()
    w = I.randn((n, k), 600 + n, std=0.05).cuda()
    wc, ws = ops.quantize_weight_fp8(w)
    xc, xs = ops.fused_act_quant(x)
    out = ops.linear_fp8(xc, xs, wc, ws)
    ops.tc_error_state()
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    # the formula of the reference's GPU kernel, in fp64
    a = xc.double().view(m, k // 128, 128) * xs.double().unsqueeze(-1)
    nb = ws.shape[0]
    wpad = torch.zeros(nb * 128, k, dtype=torch.float64, device="cuda")
    wpad[:n] = wc.double()
    b = (wpad.view(nb, 128, k // 128, 128) * ws.double()[:, None, :, None]).view(nb * 128, k)[:n]
    ref = a.view(m, k) @ b.t()
    assert rel_err(out, ref.float()) <= 1e-2
    diff = (out.float() - ref.float()).abs()
    assert bool((diff <= 2.0 ** -7 * ref.float().abs() + 1e-3 * ref.float().abs().max()).all())
    # weight codes/scales reproduce the reference's block dequantisation; its CPU fallback GEMM agrees
    if m * n <= 300000:
        deq = R.block_dequant(wc.cpu(), ws.cpu())
        assert rel_err(deq, w.cpu()) <= 0.08
        ref_cpu = R.fp8_gemm(xc.cpu(), xs.cpu(), wc.cpu(), ws.cpu())
        assert rel_err(out, ref_cpu) <= 2e-2
    # the composite the real model calls: act_quant + GEMM
    out2 = ops.linear_fp8_act(x, wc, ws)
    assert torch.equal(out2, out)


# ---------------------------------------------------------------------------
# NVFP4 block-scaled GEMM
# ---------------------------------------------------------------------------

def _dequant_gpu(ops, x):
    """fp64 dequantisation (on the GPU) of what fused_nvfp4_quant makes of x."""
    from oracle import ref_ops as R
    codes, sf, gs = ops.fused_nvfp4_quant(x)
    return R.nvfp4_dequant(codes.cpu(), sf.cpu(), gs.cpu()).cuda().double()


def _check_nvfp4(out, ref64):
    ref = ref64.float()
    err = rel_err(out, ref)
    assert err <= 1e-2, f"relative error {err}"
    diff = (out.float() - ref).abs()
    tol = 2.0 ** -7 * ref.abs() + 1e-3 * ref.abs().max()
    assert bool((diff <= tol).all()), f"worst {float(diff.max())} (max |ref| {float(ref.abs().max())})"


@pytest.fixture(params=[1, 2], ids=["single_cta", "cta_pair"])
def nvfp4_schedule(request, ops):
    """Runs a test under both schedules of the NVFP4 GEMM (single-CTA 128 x 128 tiles, CTA
    pairs with 256 weight rows x up to 256 token rows) and restores the default."""
    previous = ops.gemm_nvfp4_schedule(request.param)
    yield request.param
    ops.gemm_nvfp4_schedule(previous)


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 256),       # one tile, one K stage
    (128, 128, 1024),      # one tile, several stages (scale buffers alternate)
    (256, 256, 512),       # 2 x 2 tiles (one pair tile with both token scale tiles)
    (16, 256, 256),        # narrowest pair MMA (N = 16)
    (17, 256, 1536),       # 17 tokens -> N = 32, the stage ring wraps once
    (129, 512, 512),       # second token scale tile holds a single row
    (200, 384, 768),       # token halves of 104 rows (64 + 32 + 8 row boxes), weight rows past n
    (300, 256, 512),       # a full wide tile and a 44-row one
    (100, 2112, 7168),     # ragged M, N not a multiple of the tile
    (1, 4096, 7168),       # decode row
    (2048, 4096, 7168),    # expert up-projection shape, many tiles per CTA
])
def test_linear_nvfp4_dense(ops, nvfp4_schedule, m, n, k):
    x = I.randn((m, k), 300 + m).cuda()
    w = I.randn((n, k), 400 + n, std=0.05).cuda()
    xq = ops.fused_nvfp4_quant(x, tiled_scales=True)
    wq = ops.fused_nvfp4_quant(w, tiled_scales=True)
    out = ops.linear_nvfp4(*xq, *wq)
    ops.tc_error_state()
    assert out.shape == (m, n)
    ref = _dequant_gpu(ops, x) @ _dequant_gpu(ops, w).t()
    _check_nvfp4(out, ref)


def test_gemm_nvfp4_grouped_ragged(ops, nvfp4_schedule):
    """Five groups of 130, 0, 5, 256 and 1 rows: tiles never straddle groups, every group
    uses its own weights and global scale, empty groups cost nothing."""
    sizes = [130, 0, 5, 256, 1]
    n, k = 256, 512
    offsets = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32).cuda()
    rows = sum(sizes)
    x = I.randn((rows, k), 7).cuda()
    ws = [(I.randn((n, k), 50 + g, std=0.05) * (g + 1)).to(torch.bfloat16).cuda() for g in range(len(sizes))]
    amax = ops.tensor_absmax(x)
    a_codes = torch.empty(rows, k // 2, dtype=torch.uint8, device="cuda")
    sf_parts, r0 = [], 0
    for s in sizes:
        if s:
            c, sf, a_gs = ops.fused_nvfp4_quant(x[r0:r0 + s], amax=amax, tiled_scales=True)
            a_codes[r0:r0 + s] = c
            sf_parts.append(sf.view(torch.uint8))
        r0 += s
    a_sf = torch.cat(sf_parts)
    wq = [ops.fused_nvfp4_quant(w, tiled_scales=True) for w in ws]
    b_codes = torch.cat([q[0] for q in wq])
    b_sf = torch.cat([q[1].view(torch.uint8) for q in wq])
    b_gs = torch.cat([q[2] for q in wq])
    tile_map, tile_base, tile_count = ops.moe_tile_map(offsets, 0, len(sizes), rows // 128 + len(sizes) + 1)
    max_tiles = tile_map.shape[0] // 2
    assert tile_base.cpu().tolist() == [0, 2, 2, 3, 5, 6] and tile_count.cpu().tolist() == [6, 4]
    assert tile_map.cpu()[:6].tolist() == [[0, 0, 128, 0], [0, 128, 2, 1], [2, 130, 5, 2],
                                           [3, 135, 128, 3], [3, 263, 128, 4], [4, 391, 1, 5]]
    # the same rows in tiles of up to 256 (work list of the CTA-pair schedule)
    assert tile_map.cpu()[max_tiles:max_tiles + 4].tolist() == [[0, 0, 130, 0], [2, 130, 5, 2],
                                                                [3, 135, 256, 3], [4, 391, 1, 5]]
    out = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_nvfp4_grouped(a_codes, a_sf, a_gs, b_codes, b_sf, b_gs, tile_map, tile_count,
                           n=n, groups=len(sizes), out=out)
    ops.tc_error_state()
    assert not bool(out.isnan().any())
    xd = _dequant_gpu(ops, x)          # same global amax as the per-group calls
    r0 = 0
    for g, s in enumerate(sizes):
        if s:
            _check_nvfp4(out[r0:r0 + s], xd[r0:r0 + s] @ _dequant_gpu(ops, ws[g]).t())
        r0 += s
    # a sub-range of groups (an expert-parallel rank owning groups 2..4)
    tm2, tb2, tc2 = ops.moe_tile_map(offsets, 2, 5, 8)
    assert tc2.cpu().tolist() == [4, 3] and tm2.cpu()[0].tolist() == [0, 130, 5, 0]
    assert tm2.cpu()[8:11].tolist() == [[0, 130, 5, 0], [1, 135, 256, 1], [2, 391, 1, 3]]


@pytest.mark.parametrize("m,n,k,out_dtype", [
    (1, 2112, 7168, torch.bfloat16),       # one decode token, qkv_a
    (64, 7168, 16384, torch.bfloat16),     # the decode batch, w_o: 256 K blocks
    (64, 256, 7168, torch.float32),        # router logits of the decode batch, fp32 out
    (17, 8192, 1536, torch.bfloat16),      # the indexer's wq_b, ragged rows
    (128, 1024, 1032, torch.bfloat16),     # K not a multiple of 64: the last block is partial
])
def test_linear_bf16_split_k_for_few_rows(ops, m, n, k, out_dtype):
    """Few rows against a whole weight matrix take the split-K schedule (rt_gemm_bf16_splitk):
    same product, fp32 partial sums per K range added in a fixed order, one rounding at the
    end; two runs give the same bits."""
    from racetrack_b200 import _lib
    assert int(_lib.load().rt_gemm_bf16_splitk_splits(m, n, k)) > 1
    x = I.randn((m, k), 300 + m).cuda()
    w = I.randn((n, k), 400 + n, std=0.05).cuda()
    before = _lib.launch_count()
    out = ops.linear_bf16(x, w, out_dtype=out_dtype)
    ops.tc_error_state()
    assert _lib.launch_count() - before == 2 and out.dtype == out_dtype and out.shape == (m, n)
    again = ops.linear_bf16(x, w, out_dtype=out_dtype)
    assert torch.equal(out, again), "split-K must be bit-reproducible"
    ref = _ref(x, w)
    diff = (out.float() - ref).abs()
    tol = (2.0 ** -7 if out_dtype == torch.bfloat16 else 1e-5) * ref.abs() + 2e-3 * ref.abs().max()
    assert bool((diff <= tol).all()), f"worst {float(diff.max())}"
    # the single-pass kernel gives the same result to the last bf16 bit or one
    saved, ops.SPLITK_MAX_ROWS = ops.SPLITK_MAX_ROWS, 0
    try:
        one = ops.linear_bf16(x, w, out_dtype=out_dtype)
    finally:
        ops.SPLITK_MAX_ROWS = saved
    assert float((out.float() - one.float()).abs().max()) <= 2.0 ** -6 * float(ref.abs().max())
