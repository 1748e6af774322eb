"""Pins the CPU oracle (oracle/ref_ops.py) against fixtures produced by racetrack itself
(tests/golden/make_golden.py). Runs without a GPU."""
from __future__ import annotations

import pytest
import torch

from oracle import inputs as I
from oracle import ref_ops as R
from helpers import assert_bit_exact, assert_close_bf16, sha


def _check(name, got, golden_small, golden_hashes, exact_host, *, pure_ieee=False):
    """Exact equality on the host class that produced the fixtures (always for results made of
    IEEE-exact operations only); one bf16 ulp elsewhere, where libm/vector widths may differ."""
    want_hash = golden_hashes["sha256"].get(name)
    want = golden_small.get(name)
    if exact_host or pure_ieee:
        if want_hash is not None:
            assert sha(got) == want_hash, f"{name}: SHA-256 differs from the reference output"
        if want is not None:
            assert_bit_exact(got, want, name)
    elif want is not None:
        if got.dtype in (torch.bfloat16, torch.float32):
            assert_close_bf16(got, want, name, ulps=1)
        else:
            assert_bit_exact(got, want, name)


@pytest.mark.parametrize("tag,tokens", [("c1", 128), ("c1_small", 4)])
def test_mla_prologue_matches_reference(tag, tokens, golden_small, golden_hashes, same_cpu_as_golden):
    d = I.mla_prologue_inputs(tokens)
    normed, hidden = R.residual_norm(d["x"], d["residual"], d["w_attn"], d["eps"])
    freqs = R.precompute_freqs_cis(I.ROPE_DIM, tokens, d["rope_theta"])
    fq, fkv, fk = R.fused_norm_rope(d["q_c"], d["w_q"], d["kv_c"], d["w_kv"], d["k_pe"],
                                    d["positions"], eps=d["eps"], rope_base=d["rope_theta"])
    outs = {
        "normed": normed, "hidden": hidden,
        "q_norm": R.rms_norm(d["q_c"], d["w_q"], d["eps"]),
        "kv_norm": R.rms_norm(d["kv_c"], d["w_kv"], d["eps"]),
        "q_norm_real": R.rms_norm(d["q_c"], d["w_q"], d["eps"]),
        "freqs_cis": torch.view_as_real(freqs),
        "q_rot": R.apply_rotary_emb(d["q_pe"].unsqueeze(0), freqs).squeeze(0),
        "k_rot": R.apply_rotary_emb(d["k_pe"].unsqueeze(0).unsqueeze(2), freqs).squeeze(0),
        "k_rot_noninterleaved": R.apply_rotary_emb(
            d["k_pe"].unsqueeze(0).unsqueeze(2).contiguous(), freqs, False).squeeze(0),
        "fused_q": fq, "fused_kv": fkv, "fused_k": fk,
        "q_half": R.apply_rope(d["q_pe"], d["positions"], base=d["rope_theta"]),
    }
    for k, v in outs.items():
        _check(f"{tag}.{k}", v, golden_small, golden_hashes, same_cpu_as_golden)
    # mla_prologue is the same functions strung together
    p = R.mla_prologue(d["x"], d["residual"], d["w_attn"], d["q_c"], d["w_q"], d["kv_c"], d["w_kv"],
                       d["q_pe"], d["k_pe"].unsqueeze(1), freqs, d["eps"])
    assert torch.equal(p[0], normed) and torch.equal(p[4], outs["q_rot"])
    assert torch.equal(p[5], outs["k_rot"])


def test_yarn_table_matches_reference(golden_small, golden_hashes, same_cpu_as_golden):
    freqs = torch.view_as_real(R.precompute_freqs_cis(I.ROPE_DIM, 8192))
    if same_cpu_as_golden:
        assert sha(freqs) == golden_hashes["sha256"]["yarn8192.freqs_cis"]
    rows = freqs[[0, 1, 4095, 4096, 8191]]
    torch.testing.assert_close(rows, golden_small["yarn8192.freqs_cis_rows"], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("tag,tokens,inter", [("c2_small", 16, 512), ("c2_mid", 64, I.DENSE_INTER)])
def test_swiglu_and_fp8_quant_match_reference(tag, tokens, inter, golden_small, golden_hashes,
                                              same_cpu_as_golden):
    d = I.swiglu_quant_inputs(tokens, inter)
    h = R.swiglu(d["gate"], d["up"])
    _check(f"{tag}.swiglu", h, golden_small, golden_hashes, same_cpu_as_golden)
    codes, scales = R.act_quant(d["gate"])
    # amax, two IEEE divisions, a clamp and a cast: identical on every host
    _check(f"{tag}.codes", codes, golden_small, golden_hashes, True, pure_ieee=True)
    _check(f"{tag}.scales", scales, golden_small, golden_hashes, True, pure_ieee=True)
    hc, hs = R.swiglu_quant(d["gate"], d["up"])
    _check(f"{tag}.h_codes", hc, golden_small, golden_hashes, same_cpu_as_golden)
    _check(f"{tag}.h_scales", hs, golden_small, golden_hashes, same_cpu_as_golden)
    if not same_cpu_as_golden and f"{tag}.swiglu" in golden_small:
        # quantising the stored reference product must still be exact
        hc2, hs2 = R.act_quant(golden_small[f"{tag}.swiglu"])
        assert_bit_exact(hc2, golden_small[f"{tag}.h_codes"], "h_codes from stored swiglu")
        assert_bit_exact(hs2, golden_small[f"{tag}.h_scales"], "h_scales from stored swiglu")


def test_mlp_module_matches_reference(golden_small):
    w = I.expert_weights(1, 64, 128, seed=I.SEED + 7)[0]
    x = I.randn((8, 64), I.SEED + 8)
    out = R.expert_mlp(x, *w)
    assert_close_bf16(out, golden_small["mlp_small.out"], "mlp", ulps=2)


def test_fp8_gemm_fallback_matches_reference(golden_small):
    a = I.randn((16, 256), I.SEED + 31)
    wfp = I.randn((384, 256), I.SEED + 32, std=0.02, dtype=torch.float32)
    wq = wfp.clamp(-448, 448).to(torch.float8_e4m3fn)
    ws = I.uniform((3, 2), I.SEED + 33, 0.5, 1.5)
    a_q, a_s = R.act_quant(a)
    assert_bit_exact(R.block_dequant(wq, ws), golden_small["fp8_gemm.dequant"], "block_dequant")
    assert_close_bf16(R.fp8_gemm(a_q, a_s, wq, ws), golden_small["fp8_gemm.out"], "fp8_gemm", ulps=2)


def test_gate_matches_reference(golden_small):
    d = I.gate_inputs(64)
    w, idx = R.gate_forward(d["hidden"], d["w_gate"], d["bias"], n_groups=d["n_groups"],
                            topk_groups=d["topk_groups"], topk=d["topk"],
                            route_scale=d["route_scale"], score_func="sigmoid")
    assert torch.equal(idx, golden_small["gate.indices"])
    torch.testing.assert_close(w, golden_small["gate.weights"], rtol=1e-6, atol=1e-7)
    w, idx = R.gate_forward(I.randn((32, 64), I.SEED + 42), I.randn((8, 64), I.SEED + 41, std=0.2),
                            None, n_groups=1, topk_groups=1, topk=2, route_scale=1.0,
                            score_func="softmax")
    assert torch.equal(idx, golden_small["gate_softmax.indices"])
    torch.testing.assert_close(w, golden_small["gate_softmax.weights"], rtol=1e-6, atol=1e-7)


def test_moe_forward_matches_reference(golden_small, golden_hashes, same_cpu_as_golden):
    ew = I.expert_weights(17, I.HIDDEN, 64, seed=I.SEED + 50)
    x = I.randn((32, I.HIDDEN), I.SEED + 53)
    y = R.moe_forward(x, I.randn((16, I.HIDDEN), I.SEED + 51, std=0.02),
                      I.uniform((16,), I.SEED + 52, -0.1, 0.1), ew[:16], ew[16],
                      n_groups=4, topk_groups=2, topk=4, route_scale=I.ROUTE_SCALE)
    if same_cpu_as_golden:
        assert sha(y) == golden_hashes["sha256"]["moe.out"]
    assert_close_bf16(y[:, :256], golden_small["moe.out_cols0_256"], "moe", ulps=2)


def test_moe_permute_is_a_stable_sort():
    g = torch.Generator().manual_seed(5)
    idx = torch.stack([torch.randperm(16, generator=g)[:4] for _ in range(50)])
    offsets, sorted_pairs, pair_pos = R.moe_permute(idx, 16)
    flat = idx.flatten()
    experts_sorted = flat[sorted_pairs.long()]
    assert torch.equal(experts_sorted, experts_sorted.sort(stable=True)[0])
    assert torch.equal(sorted_pairs.long(), flat.sort(stable=True)[1])
    assert torch.equal(pair_pos[sorted_pairs.long()].long(), torch.arange(200))
    assert int(offsets[-1]) == 200


# ---------------------------------------------------------------------------
# NVFP4: no reference implementation exists, so known answers stand in for fixtures.
# ---------------------------------------------------------------------------

def test_e2m1_grid_round_trips_and_ties_go_to_even():
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    both = torch.cat([grid, -grid])
    assert torch.equal(R.e2m1_decode(R.e2m1_encode(both)), both)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    want = torch.tensor([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0])
    assert torch.equal(R.e2m1_decode(R.e2m1_encode(ties)), want)
    assert torch.equal(R.e2m1_decode(R.e2m1_encode(-ties)), -want)
    assert torch.equal(R.e2m1_decode(R.e2m1_encode(torch.tensor([7.0, 100.0, -1e9]))),
                       torch.tensor([6.0, 6.0, -6.0]))


def test_nvfp4_known_answers():
    # A block holding the tensor amax: block scale 448, the amax element maps to +-6.
    x = torch.zeros(2, 32, dtype=torch.bfloat16)
    x[0, :8] = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]).to(torch.bfloat16)
    x[1, 16] = -3.0
    codes, bs, gs = R.nvfp4_quant(x)
    assert float(gs) == pytest.approx(6.0 / 2688.0)
    assert float(bs[0, 0].float()) == 448.0          # block_amax / (6 * gs) = 448
    assert float(bs[0, 1].float()) == 0.0 and int(codes[0, 8:].sum()) == 0   # all-zero block
    deq = R.nvfp4_dequant(codes, bs, gs)
    torch.testing.assert_close(deq[0, :8], x[0, :8].float(), rtol=1e-6, atol=0)
    assert float(bs[1, 1].float()) == 224.0          # 3 / (6 * gs)
    assert float(deq[1, 16]) == pytest.approx(-3.0, rel=1e-6)
    # element 2i in the low nibble
    assert int(codes[0, 0]) == (0 | (1 << 4)) and int(codes[0, 3]) == (6 | (7 << 4))
    # all-zero tensor: unit global scale, zero codes and scales
    z = torch.zeros(1, 16, dtype=torch.bfloat16)
    c, b, g = R.nvfp4_quant(z)
    assert float(g) == 1.0 and int(c.sum()) == 0 and float(b.float().sum()) == 0.0


def test_nvfp4_error_bound_on_gaussian_data():
    x = I.randn((64, 1024), 7)
    codes, bs, gs = R.nvfp4_quant(x)
    deq = R.nvfp4_dequant(codes, bs, gs)
    blocks = x.float().reshape(64, 64, 16)
    bmax = blocks.abs().amax(-1, keepdim=True)
    err = (deq.reshape(64, 64, 16) - blocks).abs()
    # half of the widest grid step (4 -> 6, i.e. 1/6 of the block range) stretched by the
    # e4m3 rounding of the block scale (2^-4), plus saturation when the scale rounded down
    assert bool((err <= bmax * ((1.0 / 6.0) * (1 + 1.0 / 16.0) + 1.0 / 16.0) + 1e-6).all())


def test_sf_tiled_offsets_are_a_bijection():
    off = R.sf_tiled_offsets(256, 8)
    assert off.numel() == off.unique().numel() == 256 * 8
    assert int(off.max()) == 2 * 2 * 512 - 1
    assert int(off[0, 1]) == 1 and int(off[1, 0]) == 16 and int(off[32, 0]) == 4
    assert int(off[128, 0]) == 2 * 512 and int(off[0, 4]) == 512


def test_indexer_scores_and_topk_match_reference(golden_small, golden_hashes, same_cpu_as_golden):
    """fp8_index and the top-k selection of the sparse indexer against racetrack's own
    functions. The fp32 head and dimension sums may be ordered differently on another CPU, so
    scores are compared to 1e-5 of the largest score and selections through the scores they
    pick (a near-tie at the k-th place may legitimately swap two indices)."""
    d = I.indexer_inputs(5, 300)
    scores = R.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
    want = golden_small["idx_small.scores"]
    tol = 1e-5 * float(want.abs().max())
    assert float((scores - want).abs().max()) <= tol
    got_idx = R.index_topk(scores, 64).sort(dim=-1)[0].to(torch.int32)
    if same_cpu_as_golden:
        assert_bit_exact(scores, want, "idx_small.scores")
        assert_bit_exact(got_idx, golden_small["idx_small.topk"], "idx_small.topk")
    picked = want.gather(2, got_idx.long()).sum(-1)
    best = want.gather(2, golden_small["idx_small.topk"].long()).sum(-1)
    assert float((picked - best).abs().max()) <= 64 * tol

    d = I.indexer_inputs(16, 4096)
    scores = R.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
    idx = R.index_topk(scores, I.INDEX_TOPK)
    assert idx.shape == (1, 16, I.INDEX_TOPK)
    kth = scores.gather(2, idx)[..., -1]
    tol = 1e-5 * float(scores.abs().max())
    assert float((kth - golden_small["idx_decode.kth_score"]).abs().max()) <= tol
    sel = torch.zeros(1, 16, 4096, dtype=torch.bool)
    sel.scatter_(2, idx, True)
    assert int(sel.sum()) == 16 * I.INDEX_TOPK
    ssum = (scores * sel).sum(-1)
    assert float((ssum - golden_small["idx_decode.score_sum_selected"]).abs().max()) <= 2048 * tol
    if same_cpu_as_golden:
        assert sha(sel.to(torch.uint8)) == golden_hashes["sha256"]["idx_decode.selected_mask"]
    # a causal mask removes later keys from the selection
    mask = torch.full((16, 4096), float("-inf")).triu_(1 + 4096 - 16)
    idx_m = R.index_topk(scores, I.INDEX_TOPK, mask)
    assert int((idx_m[0, 0] > 4096 - 16).sum()) == 0


def test_indexer_key_prologue_matches_reference(golden_small, same_cpu_as_golden):
    """LayerNorm + non-interleaved RoPE of the indexer's key path against racetrack's own
    LayerNorm / apply_rotary_emb; the Hadamard rotation that follows comes from a package
    racetrack does not vendor, so it is only checked against its definition."""
    k_in = I.randn((9, 1, 128), I.SEED + 710)
    w = I.randn((128,), I.SEED + 711, mean=1.0, std=0.02, dtype=torch.float32)
    b = I.randn((128,), I.SEED + 712, std=0.02, dtype=torch.float32)
    k_ln = R.layer_norm(k_in, w, b)
    pe, nope = torch.split(k_ln, [64, 64], dim=-1)
    fc = R.precompute_freqs_cis(64, 16384)[:9]     # ModelArgs(): max_seq_len 16384 (YaRN on)
    got = torch.cat([R.apply_rotary_emb(pe.unsqueeze(0), fc, False).squeeze(0), nope], dim=-1)
    if same_cpu_as_golden:
        assert_bit_exact(got, golden_small["idxprep.k_ln_rope"], "idxprep.k_ln_rope")
    else:
        assert_close_bf16(got, golden_small["idxprep.k_ln_rope"], "idxprep.k_ln_rope", ulps=1)
    # the rotation: orthonormal, an involution, and equal to the butterfly network
    h = R.hadamard_matrix(128)
    assert torch.equal(h @ h.t(), 128 * torch.eye(128))
    x = I.randn((5, 128), 3).float()
    y = x.clone().view(5, 128)
    step = 1
    while step < 128:                       # fast Walsh-Hadamard transform, natural order
        y = y.view(5, -1, 2, step)
        y = torch.cat((y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]), dim=-1).view(5, 128)
        step *= 2
    torch.testing.assert_close(y, x @ h, rtol=1e-5, atol=1e-4)
    codes, scales, rotated = R.index_prep(k_in, fc, ln_weight=w, ln_bias=b)
    assert codes.shape == (9, 1, 128) and scales.shape == (9, 1)
    c2, s2 = R.act_quant(rotated)
    assert torch.equal(codes.view(torch.uint8), c2.view(torch.uint8)) and torch.equal(scales, s2.squeeze(-1))


def test_mla_decode_matches_reference(golden_small, same_cpu_as_golden):
    """The whole decode branch of MLA.forward (projections, cache append, absorbed scores, index
    mask, softmax, value projection, wo) against racetrack's own module run with a fixed
    selection in place of the indexer; and the fp32 attention core the GPU kernel is tested
    against agrees with that bf16 flow to bf16 accuracy."""
    c = I.MLA_DECODE
    d = I.mla_decode_inputs()
    fc = R.precompute_freqs_cis(c["rope"], c["max_len"])[c["start_pos"]:c["start_pos"] + 1]
    kv_cache, pe_cache = d["kv_cache"].clone(), d["pe_cache"].clone()
    y = R.mla_decode(d["x"], c["start_pos"], fc, d["w"], kv_cache, pe_cache, d["topk_indices"],
                     heads=c["heads"], nope=c["nope"], rope=c["rope"], v_dim=c["v_dim"])
    for got, key in ((y, "mla_decode.out"), (kv_cache[:, c["start_pos"]], "mla_decode.kv_row"),
                     (pe_cache[:, c["start_pos"]], "mla_decode.pe_row")):
        if same_cpu_as_golden:
            assert_bit_exact(got, golden_small[key], key)
        else:
            assert_close_bf16(got, golden_small[key], key, ulps=2)
    # the fp32 core (oracle of rt_mla_sparse_decode) against the bf16 flow, value projection aside
    end = c["start_pos"] + 1
    g = torch.Generator().manual_seed(5)
    q_abs = torch.randn(c["batch"], c["heads"], c["kv_lora"], generator=g).mul(0.3).bfloat16()
    q_pe = torch.randn(c["batch"], c["heads"], c["rope"], generator=g).mul(0.3).bfloat16()
    scale = (c["nope"] + c["rope"]) ** -0.5
    core = R.mla_sparse_decode(q_abs, q_pe, kv_cache[:, :end], pe_cache[:, :end],
                               d["topk_indices"][:, 0], scale)
    scores = (torch.einsum("bhc,btc->bht", q_abs, kv_cache[:, :end]) +
              torch.einsum("bhr,btr->bht", q_pe, pe_cache[:, :end])) * scale
    mask = torch.full((c["batch"], 1, end), float("-inf"), dtype=scores.dtype).scatter_(
        -1, d["topk_indices"][:, 0:1, :].reshape(c["batch"], 1, -1), 0)
    flow = torch.einsum("bht,btc->bhc", (scores + mask).softmax(dim=-1), kv_cache[:, :end])
    assert float((core - flow.float()).abs().max()) <= 3e-2 * float(core.abs().max())


@pytest.mark.parametrize("world", [1, 2])
def test_layer_oracle_matches_reference_block(world, same_cpu_as_golden):
    """oracle/ref_layer.forward_stack against racetrack's own ShardedRealisticBlock / Model
    (racetrack/realistic_bench.py:118-427) run by tests/golden/make_golden.py on CPU in bf16:
    one process (world 1) and two gloo ranks (world 2; each rank's weights as the reference
    drew them from seed + rank). Exact on the host class that made the fixture, one bf16 ulp
    of the largest element elsewhere (the matmuls' summation order follows the vector width)."""
    from conftest import GOLDEN_DIR
    from oracle import ref_layer
    from racetrack_b200.layer import LayerShape
    fx = torch.load(GOLDEN_DIR / "golden_layer.pt")
    s = fx["shape"]
    shape = LayerShape(name="pin", hidden=s["hidden_size"], heads=s["num_attention_heads"],
                       q_lora=s["q_lora_rank"], kv_lora=s["kv_lora_rank"],
                       nope=s["qk_nope_head_dim"], rope=s["qk_rope_head_dim"],
                       v_dim=s["v_head_dim"], moe_inter=s["moe_intermediate_size"],
                       n_experts=s["n_routed_experts"], topk=s["num_experts_per_tok"],
                       seed=s["seed"])
    case = fx[f"world{world}"]
    positions = torch.arange(fx["tokens"], dtype=torch.int64)
    for layers in (1, 3):
        got = ref_layer.forward_stack(case["hidden"], positions, case["rank_weights"], shape, layers)
        want = case[f"out{layers}"]
        if same_cpu_as_golden:
            assert_bit_exact(got, want, f"world {world}, {layers} layer(s)")
        else:
            tol = 2.0 ** -7 * float(want.float().abs().max())
            assert float((got.float() - want.float()).abs().max()) <= tol * layers
