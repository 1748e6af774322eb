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
