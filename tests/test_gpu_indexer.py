"""GPU parity of the sparse-attention indexer kernels (index scores on the tensor cores, exact
top-k selection) against the CPU restatement of racetrack's fp8_index / topk
(oracle/ref_ops.py) and against the fixtures racetrack itself produced."""
from __future__ import annotations

import pytest
import torch

from oracle import inputs as I
from oracle import ref_ops as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from racetrack_b200 import ops as _ops
    return _ops


def _cuda(d):
    return {k: v.cuda() for k, v in d.items()}


def _close_rotated(got, want, what, max_frac=2e-2):
    """One bf16 ulp, with an absolute floor: a Hadamard output is a sum of 128 terms of either
    sign, so next to zero the fp32 summation order alone moves it by more than its own ulp."""
    g, w = got.detach().float().cpu(), want.detach().float().cpu()
    bad = (g - w).abs() > 2.0 ** -7 * w.abs() + 1e-5
    assert not bool(bad.any()), f"{what}: {int(bad.sum())} elements off, worst {float((g - w).abs().max())}"
    frac = float((got.detach().cpu().view(torch.int16) != want.view(torch.int16)).float().mean())
    assert frac <= max_frac, f"{what}: {frac:.2e} of the elements differ"


@pytest.mark.parametrize("queries,keys,heads", [
    (5, 300, 64),          # ragged everywhere: 1.25 query blocks, 2.3 key tiles
    (1, 4096, 64),         # one decode query over a 4096-key cache
    (64, 4096, 64),        # decode batch: 16 query blocks x 2 key chunks
    (3, 128, 32),          # 8 queries per block
    (2, 200, 128),         # one query per column half
    (300, 2100, 64),       # several chunks, work items wrap over the CTAs
])
def test_fp8_index_scores(ops, queries, keys, heads):
    d = I.indexer_inputs(queries, keys, heads=heads)
    g = _cuda(d)
    scores = ops.fp8_index(g["q"], g["weights"], g["k"], g["k_scale"])
    ops.tc_error_state()
    assert scores.shape == (1, queries, keys) and scores.dtype == torch.float32
    # fp64 evaluation of the reference formula: products of e4m3 values are exact, the sums
    # differ only by fp32 summation order
    q, k = d["q"].double(), d["k"].double()
    logits = torch.einsum("bmhd,bnd->bmhn", q, k).clamp(min=0) * d["weights"].double().unsqueeze(-1)
    ref = logits.sum(2) * d["k_scale"].double().unsqueeze(1)
    tol = 2e-5 * float(ref.abs().max())
    assert float((scores.cpu().double() - ref).abs().max()) <= tol
    # and the reference's own fp32 path
    ref32 = R.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
    assert float((scores.cpu() - ref32).abs().max()) <= tol


def test_fp8_index_matches_racetrack_fixture(ops, golden_small):
    d = _cuda(I.indexer_inputs(5, 300))
    scores = ops.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
    want = golden_small["idx_small.scores"]
    assert float((scores.cpu() - want).abs().max()) <= 2e-5 * float(want.abs().max())


def test_fp8_index_causal_mask(ops):
    queries, keys = 40, 300
    d = _cuda(I.indexer_inputs(queries, keys))
    plain = ops.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])[0]
    off = keys - queries                      # the queries are the last positions of the sequence
    masked = ops.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"], causal_offset=off)[0]
    m = torch.arange(queries, device="cuda").unsqueeze(1)
    n = torch.arange(keys, device="cuda").unsqueeze(0)
    visible = n <= m + off
    assert torch.equal(masked[visible], plain[visible])
    assert bool(torch.isneginf(masked[~visible]).all())


def _check_selection(scores, idx, topk):
    """idx selects exactly the topk largest scores of every row (as a set), ascending."""
    s = scores.reshape(-1, scores.shape[-1])
    i = idx.reshape(-1, idx.shape[-1]).long()
    assert i.shape[1] == min(topk, s.shape[1])
    assert bool((i[:, 1:] > i[:, :-1]).all()), "indices must be strictly ascending"
    picked = s.gather(1, i).sort(dim=1, descending=True)[0]
    best = s.topk(i.shape[1], dim=1)[0]
    assert torch.equal(picked, best)


@pytest.mark.parametrize("rows,keys,topk", [(7, 300, 64), (16, 4096, 2048), (3, 5000, 5000),
                                            (2, 70, 1), (5, 1025, 512)])
def test_index_topk_selects_the_largest(ops, rows, keys, topk):
    g = torch.Generator().manual_seed(rows * 1000 + keys)
    scores = torch.randn(rows, keys, generator=g).cuda()
    idx = ops.index_topk(scores, topk)
    assert idx.dtype == torch.int32
    _check_selection(scores, idx, topk)


def test_index_topk_ties_and_masked_scores(ops):
    """Quantised scores (many equal values) and -inf entries: the selection is still exactly
    the k largest, ties at the k-th place going to the lower indices."""
    g = torch.Generator().manual_seed(5)
    scores = (torch.randn(6, 900, generator=g) * 2).round() / 2
    scores[:, 600:] = float("-inf")
    scores = scores.cuda()
    idx = ops.index_topk(scores, 256)
    _check_selection(scores, idx, 256)
    for r in range(6):
        row = scores[r]
        kth = row.topk(256)[0][-1]
        ties = torch.nonzero(row == kth).flatten()
        taken = torch.isin(ties, idx[r].long())
        n_taken = int(taken.sum())
        assert bool(taken[:n_taken].all()) and not bool(taken[n_taken:].any())
    # more requested than there are finite scores: -inf entries fill the rest
    idx2 = ops.index_topk(scores, 700)
    _check_selection(scores, idx2, 700)


def test_indexer_end_to_end_matches_reference_selection(ops, golden_small):
    """Scores + top-2048 of a 16-query decode step over 4096 keys: the selected set picks the
    same total score as racetrack's own selection (a near-tie may swap two indices)."""
    d = I.indexer_inputs(16, 4096)
    g = _cuda(d)
    scores = ops.fp8_index(g["q"], g["weights"], g["k"], g["k_scale"])
    idx = ops.index_topk(scores, I.INDEX_TOPK)
    ops.tc_error_state()
    assert idx.shape == (1, 16, I.INDEX_TOPK)
    ref = R.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
    tol = 2e-5 * float(ref.abs().max())
    picked = ref.gather(2, idx.cpu().long()).sum(-1)
    assert float((picked - golden_small["idx_decode.score_sum_selected"]).abs().max()) <= 2048 * tol
    kth = ref.gather(2, idx.cpu().long()).min(-1)[0]
    assert float((kth - golden_small["idx_decode.kth_score"]).abs().max()) <= tol


@pytest.mark.parametrize("rows,heads,with_ln", [(9, 1, True), (300, 1, True), (5, 64, False),
                                                (130, 64, False)])
def test_index_prep_matches_reference_chain(ops, rows, heads, with_ln):
    """[LayerNorm] -> non-interleaved RoPE -> Hadamard rotation -> act_quant in one kernel: the
    rotated tensor agrees with the op-by-op reference to one bf16 ulp (fp32 sums are ordered
    differently), and codes / scales are exactly act_quant of the kernel's own rotated tensor."""
    from helpers import assert_bit_exact
    x = I.randn((rows, heads, 128), 40 + rows)
    w = I.randn((128,), 41, mean=1.0, std=0.02, dtype=torch.float32) if with_ln else None
    b = I.randn((128,), 42, std=0.02, dtype=torch.float32) if with_ln else None
    table = R.precompute_freqs_cis(64, 16384)
    pos = (torch.arange(rows) * 37) % 5000            # arbitrary positions inside the table
    codes, scales, rotated = ops.index_prep(
        x.cuda(), table.cuda(), positions=pos.cuda(), ln_weight=w.cuda() if with_ln else None,
        ln_bias=b.cuda() if with_ln else None, return_rotated=True)
    ref_codes, ref_scales, ref_rot = R.index_prep(x, table[pos], ln_weight=w, ln_bias=b)
    _close_rotated(rotated, ref_rot, "rotated")
    c2, s2 = ops.fused_act_quant(rotated.reshape(rows * heads, 128))
    assert_bit_exact(codes.reshape(rows * heads, 128), c2, "codes")
    assert_bit_exact(scales.reshape(rows * heads, 1), s2, "scales")
    # where the rotated rows agree exactly, so do the quantised ones
    same = (rotated.cpu().view(torch.int16) == ref_rot.view(torch.int16)).all(dim=-1)
    assert float(same.float().mean()) >= 0.3
    assert torch.equal(codes.cpu().view(torch.uint8)[same], ref_codes.view(torch.uint8)[same])
    assert torch.equal(scales.cpu()[same], ref_scales[same])


def test_index_prep_default_positions_and_golden(ops, golden_small):
    """Keys at positions 0..8 with LayerNorm: the stage before the rotation is pinned by
    racetrack's own LayerNorm + apply_rotary_emb (fixture), the rotation by its definition."""
    k_in = I.randn((9, 1, 128), I.SEED + 710)
    w = I.randn((128,), I.SEED + 711, mean=1.0, std=0.02, dtype=torch.float32)
    b = I.randn((128,), I.SEED + 712, std=0.02, dtype=torch.float32)
    table = R.precompute_freqs_cis(64, 16384)
    _, _, rotated = ops.index_prep(k_in.cuda(), table.cuda(), ln_weight=w.cuda(), ln_bias=b.cuda(),
                                   return_rotated=True)
    want = R.rotate_activation(golden_small["idxprep.k_ln_rope"])
    _close_rotated(rotated, want, "rotated keys")
    # the rotation is an involution: rotating the result again returns its input, up to the
    # bf16 rounding of the intermediate
    back = R.rotate_activation(rotated.cpu()).float()
    src = golden_small["idxprep.k_ln_rope"].float()
    assert float((back - src).abs().max()) <= 0.05 * float(src.abs().max())


def test_indexer_forward_selects_like_the_reference_chain():
    """The whole indexer (projections, prologues, cache update, scores, top-k) for a prefill of
    300 tokens followed by a decode step, against the reference's op sequence on the CPU. The
    selection is compared through the reference scores it picks (a near-tie may swap two
    indices), the cache contents row by row where the rotated keys agree bit for bit."""
    from racetrack_b200 import indexer, ops
    dim, q_lora, heads, topk = 1024, 256, 64, 128
    prefill, max_len = 300, 512
    g = torch.Generator().manual_seed(77)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std)
    wq_b, wk = mk(heads * 128, q_lora, std=0.06).bfloat16(), mk(128, dim, std=0.03).bfloat16()
    lnw, lnb = 1 + mk(128, std=0.02), mk(128, std=0.02)
    wproj = mk(heads, dim, std=0.03)
    table = R.precompute_freqs_cis(64, 16384)
    w = indexer.IndexerWeights(wq_b.cuda(), wk.cuda(), lnw.cuda(), lnb.cuda(), wproj.cuda())
    k_cache = torch.zeros(max_len, 128, dtype=torch.float8_e4m3fn, device="cuda")
    ks_cache = torch.zeros(max_len, dtype=torch.float32, device="cuda")
    ref_k = torch.zeros(max_len, 128, dtype=torch.float8_e4m3fn)
    ref_ks = torch.zeros(max_len)

    def reference(x, qr, start):
        s_len, end = x.shape[0], start + x.shape[0]
        fc = table[start:end]
        q = torch.nn.functional.linear(qr, wq_b).view(s_len, heads, 128)
        q_fp8, q_scale, _ = R.index_prep(q, fc)
        k = torch.nn.functional.linear(x, wk).view(s_len, 1, 128)
        k_fp8, k_scale, _ = R.index_prep(k, fc, ln_weight=lnw, ln_bias=lnb)
        ref_k[start:end], ref_ks[start:end] = k_fp8.view(s_len, 128), k_scale.view(s_len)
        hw = torch.nn.functional.linear(x.float(), wproj) * heads ** -0.5 * q_scale * 128 ** -0.5
        scores = R.fp8_index(q_fp8.unsqueeze(0), hw.unsqueeze(0), ref_k[:end].unsqueeze(0),
                             ref_ks[:end].unsqueeze(0))[0]
        mask = torch.full((s_len, end), float("-inf")).triu_(1 + start)
        return scores + mask

    for start, s_len in ((0, prefill), (prefill, 1)):
        x, qr = mk(s_len, dim).bfloat16(), mk(s_len, q_lora).bfloat16()
        idx = indexer.indexer_forward(x.cuda(), qr.cuda(), w, k_cache, ks_cache, start, table.cuda(), topk)
        ops.tc_error_state()
        ref_scores = reference(x, qr, start)
        end = start + s_len
        kk = min(topk, end)
        assert idx.shape == (s_len, kk)
        i = idx.cpu().long()
        # rows that see fewer than kk keys also pick masked (-inf) entries, as the reference's
        # topk does; the others pick visible keys only
        full = torch.arange(start, end) + 1 >= kk
        assert bool((i[full] <= torch.arange(start, end)[full].unsqueeze(1)).all()), "causality"
        picked = ref_scores.gather(1, i).sum(1)[full]
        best = ref_scores.topk(kk, dim=1)[0].sum(1)[full]
        scale = float(ref_scores[torch.isfinite(ref_scores)].abs().max())
        assert float((picked - best).abs().max()) <= 2e-3 * kk * scale
        same = (k_cache[:end].cpu().view(torch.uint8) == ref_k[:end].view(torch.uint8)).all(dim=1)
        assert float(same.float().mean()) >= 0.5
        assert torch.equal(ks_cache[:end].cpu()[same], ref_ks[:end][same])


def test_fp8_index_batched_equals_one_call_per_sequence(ops):
    """Three sequences with caches of their own (rows of longer buffers) in one launch."""
    batch, keys, max_len, heads = 3, 300, 384, 64
    seqs = [_cuda(I.indexer_inputs(1, keys, heads=heads, seed=40 + b)) for b in range(batch)]
    q = torch.cat([d["q"] for d in seqs])                     # [B, 1, H, 128]
    wts = torch.cat([d["weights"] for d in seqs])             # [B, 1, H]
    k_cache = torch.zeros(batch, max_len, 128, dtype=torch.float8_e4m3fn, device="cuda")
    ks_cache = torch.zeros(batch, max_len, device="cuda")
    for b, d in enumerate(seqs):
        k_cache[b, :keys] = d["k"][0]
        ks_cache[b, :keys] = d["k_scale"][0]
    got = ops.fp8_index(q, wts, k_cache[:, :keys], ks_cache[:, :keys])
    ops.tc_error_state()
    assert got.shape == (batch, 1, keys)
    for b, d in enumerate(seqs):
        one = ops.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
        assert torch.equal(got[b], one[0])


def test_indexer_decode_equals_the_single_sequence_path():
    """A decode step of four sequences in one go picks what four single-sequence calls pick."""
    from racetrack_b200 import indexer, ops
    dim, q_lora, heads, topk, batch, start, max_len = 1024, 256, 64, 128, 4, 299, 384
    g = torch.Generator().manual_seed(78)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std)
    w = indexer.IndexerWeights(mk(heads * 128, q_lora, std=0.06).bfloat16().cuda(),
                               mk(128, dim, std=0.03).bfloat16().cuda(), (1 + mk(128, std=0.02)).cuda(),
                               mk(128, std=0.02).cuda(), mk(heads, dim, std=0.03).cuda())
    table = R.precompute_freqs_cis(64, 16384).cuda()
    k_cache = (mk(batch, max_len, 128) * 2).cuda().to(torch.float8_e4m3fn)
    ks_cache = (mk(batch, max_len).abs() * 0.01 + 0.005).cuda()
    x, qr = mk(batch, dim).bfloat16().cuda(), mk(batch, q_lora).bfloat16().cuda()
    k1, s1 = k_cache.clone(), ks_cache.clone()
    idx = indexer.indexer_decode(x, qr, w, k_cache, ks_cache, start, table, topk)
    ops.tc_error_state()
    assert idx.shape == (batch, topk) and idx.dtype == torch.int32
    for b in range(batch):
        one = indexer.indexer_forward(x[b:b + 1], qr[b:b + 1], w, k1[b], s1[b], start, table, topk)
        assert torch.equal(idx[b], one[0])
    assert torch.equal(k_cache.view(torch.uint8), k1.view(torch.uint8))
    assert torch.equal(ks_cache, s1)
