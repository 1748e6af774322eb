"""GPU parity tests: the CUDA kernels (through the C ABI) against the CPU oracle and the
reference-made fixtures. Bit-exact for codes, scales, indices and permutations; <= 1e-2
relative error (in practice one bf16 ulp) for bf16 outputs."""
from __future__ import annotations

import pytest
import torch

from oracle import inputs as I
from oracle import ref_ops as R
from helpers import assert_bit_exact, assert_close_bf16, mismatch_fraction, rel_err

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2   # relative tolerance for single-op bf16 outputs


@pytest.fixture(scope="module")
def ops():
    from racetrack_b200 import ops as _ops
    return _ops


def cu(t):
    return t.cuda()


# ---------------------------------------------------------------------------
# residual add + RMSNorm / RMSNorm
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(128, 7168), (1, 7168), (3, 512), (127, 2048), (129, 1536),
                                       (5, 18432), (2, 8), (7, 24576)])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_residual_norm(ops, rows, cols, wdtype):
    u, r = I.randn((rows, cols), 1), I.randn((rows, cols), 2)
    w = I.randn((cols,), 3, mean=1.0, std=0.02, dtype=wdtype)
    n_ref, h_ref = R.residual_norm(u, r, w.float() if wdtype == torch.float32 else w, 1e-6)
    n, h = ops.fused_residual_norm(cu(u), cu(r), cu(w), eps=1e-6)
    torch.cuda.synchronize()
    assert_bit_exact(h, h_ref, "hidden")          # one fp32 add, one rounding
    assert rel_err(n, n_ref) <= REL_TOL
    assert_close_bf16(n, n_ref, "normed", ulps=1, max_frac=2e-2)


def test_residual_norm_fixture_and_layouts(ops, golden_small):
    d = I.mla_prologue_inputs(4)
    n, h = ops.fused_residual_norm(cu(d["x"]), cu(d["residual"]), cu(d["w_attn"]), eps=d["eps"])
    assert_bit_exact(h, golden_small["c1_small.hidden"], "hidden vs reference fixture")
    assert_close_bf16(n, golden_small["c1_small.normed"], "normed vs reference fixture", ulps=1)
    # leading dims, legacy argument order, strided (column-slice) inputs
    u3 = cu(d["x"]).view(2, 2, -1)
    h2, n2 = ops.fused_residual_norm_legacy(cu(d["residual"]).view(2, 2, -1), u3, cu(d["w_attn"]),
                                            eps=d["eps"])
    assert n2.shape == u3.shape
    assert_bit_exact(n2.view(4, -1), n, "legacy order")
    assert_bit_exact(h2.view(4, -1), h, "legacy order")
    wide_u, wide_r = cu(I.randn((6, 1024), 9)), cu(I.randn((6, 1024), 10))
    w = cu(I.randn((512,), 11, mean=1.0, std=0.02, dtype=torch.float32))
    n3, h3 = ops.fused_residual_norm(wide_u[:, 256:768], wide_r[:, 512:], w, eps=1e-6)
    n4, h4 = ops.fused_residual_norm(wide_u[:, 256:768].contiguous(), wide_r[:, 512:].contiguous(),
                                     w, eps=1e-6)
    assert_bit_exact(n3, n4, "strided normed")
    assert_bit_exact(h3, h4, "strided hidden")
    # empty batch
    n0, h0 = ops.fused_residual_norm(wide_u[:0, :512], wide_r[:0, :512], w, eps=1e-6)
    assert n0.shape == (0, 512) and h0.shape == (0, 512)


def test_residual_norm_rejects_what_it_cannot_do(ops):
    u = cu(I.randn((4, 12), 1))
    w = cu(torch.ones(12))
    with pytest.raises(RuntimeError):
        ops.fused_residual_norm(u, u, w, eps=1e-6)          # cols % 8 != 0
    with pytest.raises(RuntimeError):
        ops.fused_residual_norm(u.float(), u.float(), w, eps=1e-6)   # not bf16
    with pytest.raises(RuntimeError):
        ops.fused_residual_norm(I.randn((4, 16), 1), I.randn((4, 16), 1), torch.ones(16), eps=1e-6)


@pytest.mark.parametrize("rows,cols", [(128, 1536), (128, 512), (1, 7168), (33, 64)])
def test_rms_norm(ops, rows, cols):
    x = I.randn((rows, cols), 4)
    w = I.randn((cols,), 5, mean=1.0, std=0.02, dtype=torch.float32)
    ref = R.rms_norm(x, w, 1e-6)
    out = ops.fused_rms_norm(cu(x), cu(w), eps=1e-6)
    assert rel_err(out, ref) <= REL_TOL
    assert_close_bf16(out, ref, "rms_norm", ulps=1, max_frac=2e-2)


# ---------------------------------------------------------------------------
# MLA prologue
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("tokens", [128, 1, 3, 129])
def test_fused_norm_rope_half_split(ops, tokens):
    d = I.mla_prologue_inputs(tokens)
    ref_q, ref_kv, ref_k = R.fused_norm_rope(d["q_c"], d["w_q"], d["kv_c"], d["w_kv"], d["k_pe"],
                                             d["positions"], eps=d["eps"], rope_base=d["rope_theta"])
    qkv = cu(d["qkv"])
    q_c, kv_c, k_pe = qkv[:, :I.Q_LORA], qkv[:, I.Q_LORA:I.Q_LORA + I.KV_LORA], qkv[:, I.Q_LORA + I.KV_LORA:]
    q, kv, k = ops.fused_norm_rope(q_c, cu(d["w_q"]), kv_c, cu(d["w_kv"]), k_pe, cu(d["positions"]),
                                   eps=d["eps"], rope_base=d["rope_theta"])
    assert q.is_contiguous() and kv.is_contiguous() and k.is_contiguous()
    for got, ref, name in ((q, ref_q, "q"), (kv, ref_kv, "kv"), (k, ref_k, "k_pe")):
        assert rel_err(got, ref) <= REL_TOL, name
        assert_close_bf16(got, ref, name, ulps=2, max_frac=3e-2)


@pytest.mark.parametrize("q_cols,kv_cols", [(4096, 2048), (2048, 1024), (128, 64), (8, 8)])
def test_fused_norm_rope_other_widths(ops, q_cols, kv_cols):
    """Widths beyond the warp-per-token kernel (CTA-per-token path) and tiny ones."""
    tokens, rope = 19, 32
    x = I.randn((tokens, q_cols + kv_cols + rope), 41)
    wq = I.randn((q_cols,), 42, mean=1.0, std=0.02, dtype=torch.float32)
    wkv = I.randn((kv_cols,), 43, mean=1.0, std=0.02, dtype=torch.float32)
    pos = torch.arange(tokens, dtype=torch.int64) * 3
    ref = R.fused_norm_rope(x[:, :q_cols], wq, x[:, q_cols:q_cols + kv_cols], wkv,
                            x[:, q_cols + kv_cols:], pos, eps=1e-6, rope_base=10000.0)
    xc = cu(x)
    got = ops.fused_norm_rope(xc[:, :q_cols], cu(wq), xc[:, q_cols:q_cols + kv_cols], cu(wkv),
                              xc[:, q_cols + kv_cols:], cu(pos), eps=1e-6, rope_base=10000.0)
    for g, r, name in zip(got, ref, ("q", "kv", "k_pe")):
        assert rel_err(g, r) <= REL_TOL, name
        assert_close_bf16(g, r, name, ulps=2, max_frac=3e-2)


def test_fused_norm_rope_bf16_weights_and_fixture(ops, golden_small):
    d = I.mla_prologue_inputs(4)
    q, kv, k = ops.fused_norm_rope(cu(d["q_c"]), cu(d["w_q"]), cu(d["kv_c"]), cu(d["w_kv"]),
                                   cu(d["k_pe"]), cu(d["positions"]), eps=d["eps"],
                                   rope_base=d["rope_theta"])
    assert_close_bf16(q, golden_small["c1_small.fused_q"], "q vs fixture", ulps=1)
    assert_close_bf16(kv, golden_small["c1_small.fused_kv"], "kv vs fixture", ulps=1)
    assert_close_bf16(k, golden_small["c1_small.fused_k"], "k vs fixture", ulps=2)
    wq, wkv = d["w_q"].to(torch.bfloat16), d["w_kv"].to(torch.bfloat16)
    ref = R.fused_norm_rope(d["q_c"], wq, d["kv_c"], wkv, d["k_pe"], d["positions"], eps=d["eps"],
                            rope_base=d["rope_theta"])
    got = ops.fused_norm_rope(cu(d["q_c"]), cu(wq), cu(d["kv_c"]), cu(wkv), cu(d["k_pe"]),
                              cu(d["positions"]), eps=d["eps"], rope_base=d["rope_theta"])
    for g, r in zip(got, ref):
        assert_close_bf16(g, r, "bf16 weights", ulps=2)


@pytest.mark.parametrize("tokens", [128, 5])
def test_mla_prologue_interleaved(ops, tokens, golden_small):
    """The CPU-runnable configuration: residual-add+RMSNorm, q_a/kv_a RMSNorm, interleaved RoPE
    on q_pe [T,128,64] and k_pe [T,1,64], theta 10000, positions 0..T-1."""
    d = I.mla_prologue_inputs(tokens)
    freqs = R.precompute_freqs_cis(I.ROPE_DIM, tokens, d["rope_theta"])
    ref = R.mla_prologue(d["x"], d["residual"], d["w_attn"], d["q_c"], d["w_q"], d["kv_c"], d["w_kv"],
                         d["q_pe"], d["k_pe"].unsqueeze(1), freqs, d["eps"])
    normed, hidden = ops.fused_residual_norm(cu(d["x"]), cu(d["residual"]), cu(d["w_attn"]), eps=d["eps"])
    qn, kvn, k_rot = ops.fused_norm_rope_interleaved(cu(d["q_c"]), cu(d["w_q"]), cu(d["kv_c"]),
                                                     cu(d["w_kv"]), cu(d["k_pe"]), cu(freqs),
                                                     eps=d["eps"])
    q_rot = ops.fused_rope(cu(d["q_pe"]), cu(freqs))
    got = (normed, hidden, qn, kvn, q_rot, k_rot.unsqueeze(1))
    names = ("normed", "hidden", "q_norm", "kv_norm", "q_rot", "k_rot")
    for g, r, name in zip(got, ref, names):
        assert g.shape == r.shape, name
        assert rel_err(g, r) <= REL_TOL, name
        assert_close_bf16(g, r, name, ulps=1, max_frac=2e-2)
    assert_bit_exact(hidden, ref[1], "hidden")
    # the rotation itself is four IEEE products and two sums on table values: exact
    assert_bit_exact(q_rot, ref[4], "q_rot")
    assert_bit_exact(k_rot.unsqueeze(1), ref[5], "k_rot")


def test_rope_variants(ops):
    tokens, heads = 37, 16
    freqs = R.precompute_freqs_cis(64, tokens)
    # batch of 2 sequences: table rows wrap per batch element
    x = I.randn((2, tokens, heads, 64), 12)
    ref = R.apply_rotary_emb(x, freqs)
    assert_bit_exact(ops.fused_rope(cu(x), cu(freqs)), ref, "batched interleaved")
    # in place on the q_pe slice of q [T, H, 192]
    q = cu(I.randn((tokens, heads, 192), 13))
    q_ref = R.apply_rotary_emb(q[..., 128:].cpu().unsqueeze(0), freqs).squeeze(0)
    nope_before = q[..., :128].clone()
    ops.fused_rope(q[..., 128:], cu(freqs), inplace=True)
    assert_bit_exact(q[..., 128:], q_ref, "in-place slice")
    assert_bit_exact(q[..., :128], nope_before, "nope part untouched")
    # half-split convention at large positions
    pos = torch.arange(tokens, dtype=torch.int64) * 211 + 5
    xh = I.randn((tokens, heads, 64), 14)
    ref_h = R.apply_rope(xh, pos)
    got_h = ops.fused_rope_half(cu(xh), cu(pos))
    # positions up to ~7800: host and device cos/sin differ in the last fp32 ulp, which can
    # flip the bf16 rounding of a table entry; cancellation in x1*c - x2*s then rules out a
    # per-element ulp bound, so the check is relative to the tensor's magnitude
    assert rel_err(got_h, ref_h) <= REL_TOL
    assert mismatch_fraction(got_h, ref_h) <= 5e-2


# ---------------------------------------------------------------------------
# SwiGLU and FP8 quantisation
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("tokens,inter", [(16, 512), (64, I.DENSE_INTER), (1, 2048), (3, 128), (257, 1408 // 128 * 128)])
def test_swiglu(ops, tokens, inter):
    d = I.swiglu_quant_inputs(tokens, inter)
    ref = R.swiglu(d["gate"], d["up"])
    gu = cu(d["gate_up"])
    out = ops.fused_swiglu(gu[:, :inter], gu[:, inter:])
    assert rel_err(out, ref) <= REL_TOL
    assert_close_bf16(out, ref, "swiglu", ulps=1, max_frac=1e-3)
    # the same arithmetic evaluated by torch on this GPU agrees bit for bit
    g, u = gu[:, :inter], gu[:, inter:]
    same_gpu = (torch.nn.functional.silu(g.float()) * u.float()).type_as(g)
    assert_bit_exact(out, same_gpu, "swiglu vs torch on the same GPU")


@pytest.mark.parametrize("tokens,cols", [(16, 512), (64, I.DENSE_INTER), (1, 7168), (3, 128), (130, 2048)])
def test_act_quant_fp8_bit_exact(ops, tokens, cols, golden_small):
    x = I.swiglu_quant_inputs(tokens, cols)["gate"]
    ref_codes, ref_scales = R.act_quant(x)
    codes, scales = ops.fused_act_quant(cu(x))      # strided: gate is a column slice
    assert codes.dtype == torch.float8_e4m3fn and scales.shape == (tokens, cols // 128)
    assert_bit_exact(scales, ref_scales, "scales")
    assert_bit_exact(codes, ref_codes, "codes")
    if (tokens, cols) == (16, 512):
        assert_bit_exact(codes, golden_small["c2_small.codes"], "codes vs reference fixture")
        assert_bit_exact(scales, golden_small["c2_small.scales"], "scales vs reference fixture")


def test_act_quant_fp8_edge_values(ops):
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    x[0, 3] = -0.0                         # the sign of a zero survives (code 0x80)
    x[3, 200] = -0.0
    x[1, :128] = 1e-6                      # below the 1e-4 amax clamp
    x[2, 5] = 3.0e38                       # near bf16 max
    x[2, 130] = -448.0
    x[3] = I.randn((256,), 3) * 1e-3
    x[3, 7] = float("inf") * 0             # NaN stays out: replace by 0
    x = torch.nan_to_num(x)
    ref_codes, ref_scales = R.act_quant(x)
    codes, scales = ops.fused_act_quant(cu(x))
    assert_bit_exact(scales, ref_scales, "scales")
    assert_bit_exact(codes, ref_codes, "codes")
    with pytest.raises(RuntimeError):
        ops.fused_act_quant(cu(torch.zeros(2, 100, dtype=torch.bfloat16)))


@pytest.mark.parametrize("tokens,inter", [(16, 512), (64, I.DENSE_INTER)])
def test_swiglu_quant_fp8(ops, tokens, inter, golden_small):
    d = I.swiglu_quant_inputs(tokens, inter)
    gu = cu(d["gate_up"])
    g, u = gu[:, :inter], gu[:, inter:]
    codes, scales = ops.fused_swiglu_quant(g, u)
    # fused == unfused on the same device, bit for bit
    c2, s2 = ops.fused_act_quant(ops.fused_swiglu(g, u))
    assert_bit_exact(codes, c2, "fused vs two-step codes")
    assert_bit_exact(scales, s2, "fused vs two-step scales")
    # against the CPU oracle the only freedom is the last ulp of exp() before the bf16 rounding
    ref_codes, ref_scales = R.swiglu_quant(d["gate"], d["up"])
    assert mismatch_fraction(codes, ref_codes) <= 1e-3
    assert mismatch_fraction(scales, ref_scales) <= 1e-2
    # quantising the reference's own bf16 product is exact
    if (tokens, inter) == (16, 512):
        c3, s3 = ops.fused_act_quant(cu(golden_small["c2_small.swiglu"]))
        assert_bit_exact(c3, golden_small["c2_small.h_codes"], "h_codes vs reference fixture")
        assert_bit_exact(s3, golden_small["c2_small.h_scales"], "h_scales vs reference fixture")


# ---------------------------------------------------------------------------
# NVFP4
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("rows,cols", [(64, 1024), (1, 16), (130, 7168), (16, I.DENSE_INTER)])
def test_nvfp4_quant_bit_exact(ops, rows, cols):
    x = I.randn((rows, cols), 21)
    ref_codes, ref_bs, ref_gs = R.nvfp4_quant(x)
    codes, bs, gs = ops.fused_nvfp4_quant(cu(x))
    assert_bit_exact(gs, ref_gs, "global scale")
    assert_bit_exact(bs, ref_bs, "block scales")
    assert_bit_exact(codes, ref_codes, "codes")
    amax = ops.tensor_absmax(cu(x))
    assert float(amax) == float(x.float().abs().max())
    # tiled scale layout carries the same bytes at the tiled offsets, padding is zero
    codes_t, bs_t, _ = ops.fused_nvfp4_quant(cu(x), tiled_scales=True)
    assert_bit_exact(codes_t, ref_codes, "codes (tiled scales)")
    flat = bs_t.view(torch.uint8).cpu()
    off = R.sf_tiled_offsets(rows, cols // 16)
    assert torch.equal(flat[off], ref_bs.view(torch.uint8))
    mask = torch.ones(flat.numel(), dtype=torch.bool)
    mask[off.flatten()] = False
    assert int(flat[mask].sum()) == 0


def test_nvfp4_known_answers_on_gpu(ops):
    x = torch.zeros(2, 32, dtype=torch.bfloat16)
    x[0, :8] = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]).to(torch.bfloat16)
    x[0, 8:15] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]).to(torch.bfloat16)
    x[1, 16] = -3.0
    for t in (x, torch.zeros(1, 16, dtype=torch.bfloat16)):
        ref = R.nvfp4_quant(t)
        got = ops.fused_nvfp4_quant(cu(t))
        for g, r, n in zip(got, ref, ("codes", "scales", "gs")):
            assert_bit_exact(g, r, n)
    codes, bs, gs = ops.fused_nvfp4_quant(cu(x))
    deq = R.nvfp4_dequant(codes.cpu(), bs.cpu(), gs.cpu())
    assert torch.equal(deq[0, 8:15], torch.tensor([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]))


def test_swiglu_nvfp4_quant(ops):
    d = I.swiglu_quant_inputs(32, 2048)
    gu = cu(d["gate_up"])
    g, u = gu[:, :2048], gu[:, 2048:]
    h = ops.fused_swiglu(g, u)
    two = ops.fused_nvfp4_quant(h)
    one = ops.fused_swiglu_nvfp4_quant(g, u)
    for a, b, n in zip(one, two, ("codes", "scales", "gs")):
        assert_bit_exact(a, b, f"fused vs two-step {n}")
    ref = R.nvfp4_quant(h.cpu())
    for a, b, n in zip(two, ref, ("codes", "scales", "gs")):
        assert_bit_exact(a, b, f"oracle on the same bf16 product: {n}")


# ---------------------------------------------------------------------------
# MoE routing, permutation, combine
# ---------------------------------------------------------------------------

def _route_margin(logits, bias, n_groups, topk_groups, topk):
    """Smallest gap the selection depends on (group cut, expert cut, and order inside the
    selection); the exact-index check is only meaningful when this exceeds rounding noise."""
    s = logits.sigmoid()
    b = s + bias if bias is not None else s
    t = b.shape[0]
    gap = torch.full((t,), float("inf"))
    if n_groups > 1:
        gs = b.view(t, n_groups, -1).topk(2, dim=-1)[0].sum(-1)
        g_sorted = gs.sort(dim=-1, descending=True)[0]
        gap = torch.minimum(gap, (g_sorted[:, :-1] - g_sorted[:, 1:]).min(dim=-1)[0])
        keep = torch.zeros(t, n_groups, dtype=torch.bool).scatter_(1, gs.topk(topk_groups)[1], True)
        b = b.view(t, n_groups, -1).masked_fill(~keep.unsqueeze(-1), float("-inf")).flatten(1)
    top = b.topk(topk + 1, dim=-1)[0]
    gap = torch.minimum(gap, (top[:, :-1] - top[:, 1:]).min(dim=-1)[0])
    return gap


@pytest.mark.parametrize("tokens", [64, 4096, 1, 9])
def test_moe_route_matches_gate(ops, tokens, golden_small):
    d = I.gate_inputs(tokens)
    logits = torch.nn.functional.linear(d["hidden"].float(), d["w_gate"].float())
    kw = dict(n_groups=d["n_groups"], topk_groups=d["topk_groups"], topk=d["topk"],
              route_scale=d["route_scale"], score_func="sigmoid")
    w_ref, i_ref = R.gate_route(logits, d["bias"], **kw)
    w, i = ops.fused_moe_route(cu(logits), cu(d["bias"]), **kw)
    safe = _route_margin(logits, d["bias"], d["n_groups"], d["topk_groups"], d["topk"]) > 1e-6
    assert float(safe.float().mean()) > 0.99
    assert torch.equal(i.cpu()[safe], i_ref[safe]), "expert indices differ"
    torch.testing.assert_close(w.cpu()[safe], w_ref[safe], rtol=1e-5, atol=1e-7)
    # every row: a valid selection of distinct experts from at most topk_groups groups
    ic = i.cpu()
    assert int(ic.min()) >= 0 and int(ic.max()) < I.N_EXPERTS
    assert all(len(set(row.tolist())) == d["topk"] for row in ic[:64])
    assert int(((ic // 32).sort(dim=-1)[0].diff(dim=-1) != 0).sum(-1).max()) <= d["topk_groups"] - 1
    if tokens == 64:
        assert torch.equal(ic[safe], golden_small["gate.indices"][safe])
        torch.testing.assert_close(w.cpu()[safe], golden_small["gate.weights"][safe], rtol=1e-5, atol=1e-7)


def test_moe_route_softmax_small_and_no_bias(ops, golden_small):
    x, wg = I.randn((32, 64), I.SEED + 42), I.randn((8, 64), I.SEED + 41, std=0.2)
    logits = torch.nn.functional.linear(x.float(), wg.float())
    w, i = ops.fused_moe_route(cu(logits), None, n_groups=1, topk_groups=1, topk=2, route_scale=1.0,
                               score_func="softmax")
    assert torch.equal(i.cpu(), golden_small["gate_softmax.indices"])
    torch.testing.assert_close(w.cpu(), golden_small["gate_softmax.weights"], rtol=1e-5, atol=1e-7)
    # groups without bias use the group maximum
    logits = I.randn((100, 64), 77, dtype=torch.float32)
    kw = dict(n_groups=4, topk_groups=2, topk=4, route_scale=1.5, score_func="sigmoid")
    w_ref, i_ref = R.gate_route(logits, None, **kw)
    w, i = ops.fused_moe_route(cu(logits), None, **kw)
    assert torch.equal(i.cpu(), i_ref)
    torch.testing.assert_close(w.cpu(), w_ref, rtol=1e-5, atol=1e-7)
    with pytest.raises(RuntimeError):
        ops.fused_moe_route(cu(logits), None, n_groups=3, topk_groups=2, topk=4, route_scale=1.0)


@pytest.mark.parametrize("tokens,topk,n_experts", [(4096, 8, 256), (1, 8, 256), (37, 4, 16), (1025, 2, 8)])
def test_moe_permute_matches_where_loop(ops, tokens, topk, n_experts):
    g = torch.Generator().manual_seed(tokens)
    scores = torch.rand(tokens, n_experts, generator=g)
    idx = scores.topk(topk, dim=-1)[1]
    if tokens == 37:
        idx[:, 0] = 3          # a heavily loaded expert and several empty ones
    off_ref, sp_ref, pp_ref = R.moe_permute(idx, n_experts)
    off, sp, pp = ops.fused_moe_permute(cu(idx), n_experts)
    assert torch.equal(off.cpu(), off_ref)
    assert torch.equal(sp.cpu(), sp_ref)
    assert torch.equal(pp.cpu(), pp_ref)


def test_moe_gather_and_combine(ops):
    tokens, topk, n_experts, cols = 200, 4, 16, 512
    g = torch.Generator().manual_seed(3)
    idx = torch.rand(tokens, n_experts, generator=g).topk(topk, dim=-1)[1]
    weights = torch.rand(tokens, topk, generator=g)
    x = I.randn((tokens, cols), 31)
    off, sp, pp = ops.fused_moe_permute(cu(idx), n_experts)
    xg = ops.fused_moe_gather(cu(x), sp, topk)
    assert_bit_exact(xg, x[(sp.cpu() // topk).long()], "gather")
    eo = I.randn((tokens * topk, cols), 32)
    shared = I.randn((tokens, cols), 33)
    y = ops.fused_moe_combine(cu(eo), pp, cu(weights), cu(shared))
    ref = shared.float().clone()
    acc = torch.zeros(tokens, cols)
    for s in range(topk):
        acc = acc + eo[pp.cpu().view(tokens, topk)[:, s].long()].float() * weights[:, s:s + 1]
    ref = (acc + shared.float()).to(torch.bfloat16)
    assert_bit_exact(y, ref, "combine")
    # an expert-parallel rank owning experts [4, 8) only sums its slice of the sorted range
    lo, hi = int(off[4]), int(off[8])
    y_part = ops.fused_moe_combine(cu(eo), pp, cu(weights), None, pos_begin=lo, pos_end=hi)
    ppv = pp.cpu().view(tokens, topk)
    acc = torch.zeros(tokens, cols)
    for s in range(topk):
        m = ((ppv[:, s] >= lo) & (ppv[:, s] < hi)).float().unsqueeze(1)
        acc = acc + eo[ppv[:, s].long()].float() * weights[:, s:s + 1] * m
    assert_bit_exact(y_part, acc.to(torch.bfloat16), "combine on an expert slice")


# ---------------------------------------------------------------------------
# full-size, size-independent properties
# ---------------------------------------------------------------------------

def test_full_size_swiglu_quant_properties(ops):
    """T=4096 x 18432 (the SwiGLU+quant configuration): fused == two-step bit for bit, scales are
    amax/448 of the product, dequantised codes stay within half an e4m3 step of it."""
    tokens, inter = 4096, I.DENSE_INTER
    gen = torch.Generator(device="cuda").manual_seed(I.SEED)
    gu = torch.empty(tokens, 2 * inter, device="cuda", dtype=torch.bfloat16).normal_(generator=gen)
    g, u = gu[:, :inter], gu[:, inter:]
    codes, scales = ops.fused_swiglu_quant(g, u)
    h = ops.fused_swiglu(g, u)
    c2, s2 = ops.fused_act_quant(h)
    assert torch.equal(codes.view(torch.uint8), c2.view(torch.uint8))
    assert torch.equal(scales, s2)
    amax = h.float().view(tokens, inter // 128, 128).abs().amax(-1).clamp(min=1e-4)
    assert torch.equal(scales, (amax.double() / 448.0).float())      # correctly rounded quotient
    # codes: x / scale evaluated in float64 and rounded once to fp32 is the IEEE fp32 quotient
    # (a 53-bit quotient of 24-bit operands never lands on an fp32 rounding boundary)
    q = (h.double().view(tokens, -1, 128) / scales.double().unsqueeze(-1)).float()
    ref_codes = q.clamp(-448, 448).to(torch.float8_e4m3fn).view(tokens, inter)
    bad = int((codes.view(torch.uint8) != ref_codes.view(torch.uint8)).sum())
    assert bad == 0, f"{bad} of {codes.numel()} FP8 codes differ from the exact quotient"
    # informative: torch's own fp32 tensor/tensor division on this GPU
    gpu_codes = (h.float().view(tokens, -1, 128) / scales.unsqueeze(-1)).clamp(-448, 448) \
        .to(torch.float8_e4m3fn).view(tokens, inter)
    frac = float((codes.view(torch.uint8) != gpu_codes.view(torch.uint8)).float().mean())
    print(f"FP8 codes differing from torch-on-GPU fp32 division: {frac:.3e}")
    assert frac < 1e-3
    # NVFP4 at the same size: decode error bound and fused == two-step
    n1 = ops.fused_swiglu_nvfp4_quant(g, u)
    n2 = ops.fused_nvfp4_quant(h)
    for a, b in zip(n1, n2):
        assert torch.equal(a.view(torch.uint8) if a.dtype != torch.float32 else a,
                           b.view(torch.uint8) if b.dtype != torch.float32 else b)
