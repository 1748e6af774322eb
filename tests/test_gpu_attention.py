"""GPU parity of the sparse MLA decode attention (tcgen05 kernel behind rt_mla_sparse_decode)
against the fp32 CPU restatement of the reference's decode branch (oracle/ref_ops.py)."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_ops as R

pytestmark = pytest.mark.gpu

SCALE = (128 + 64) ** -0.5


@pytest.fixture(scope="module")
def ops():
    from racetrack_b200 import ops as _ops
    return _ops


def _inputs(batch, heads, keys, seed, q_std=1.0):
    g = torch.Generator().manual_seed(seed)
    q_abs = (torch.randn(batch, heads, 512, generator=g) * q_std).bfloat16()
    q_pe = (torch.randn(batch, heads, 64, generator=g) * q_std).bfloat16()
    kv = torch.randn(batch, keys, 512, generator=g).bfloat16()
    pe = torch.randn(batch, keys, 64, generator=g).bfloat16()
    return q_abs, q_pe, kv, pe


def _select(batch, keys, n_sel, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.randperm(keys, generator=g)[:n_sel].sort().values for _ in range(batch)]).int()


def _check(got, want, what):
    """bf16 output of fp32 accumulation with bf16 probabilities: 1e-2 of the row's scale."""
    g, w = got.float().cpu(), want.float()
    err = (g - w).abs().amax(dim=-1)
    ref = w.abs().amax(dim=-1).clamp_min(1e-3)
    worst = float((err / ref).max())
    assert worst <= 1e-2, f"{what}: worst error {worst:.3e} of the row maximum"


@pytest.mark.parametrize("batch,heads,keys,n_sel", [
    (1, 16, 4096, 2048),      # one decode token of one rank of eight
    (3, 16, 300, 200),        # ragged: 3.1 tiles
    (2, 32, 1024, 512),
    (2, 128, 512, 320),       # four head groups
    (64, 16, 4096, 2048),     # the decode batch
    (1, 8, 64, 17),           # less than one tile
])
def test_sparse_decode_matches_the_oracle(ops, batch, heads, keys, n_sel):
    q_abs, q_pe, kv, pe = _inputs(batch, heads, keys, 100 + batch + heads, q_std=0.3)
    idx = _select(batch, keys, n_sel, 7)
    want = R.mla_sparse_decode(q_abs, q_pe, kv, pe, idx, SCALE)
    got = ops.mla_sparse_decode(q_abs.cuda(), q_pe.cuda(), kv.cuda(), pe.cuda(), idx.cuda(), SCALE)
    torch.cuda.synchronize()
    _check(got, want, f"B={batch} H={heads} S={keys} n={n_sel}")


def test_dense_mode_visits_every_key(ops):
    q_abs, q_pe, kv, pe = _inputs(2, 16, 700, 3, q_std=0.3)
    want = R.mla_sparse_decode(q_abs, q_pe, kv, pe, None, SCALE)
    got = ops.mla_sparse_decode(q_abs.cuda(), q_pe.cuda(), kv.cuda(), pe.cuda(), None, SCALE)
    _check(got, want, "dense")


def test_negative_indices_are_skipped(ops):
    q_abs, q_pe, kv, pe = _inputs(2, 16, 512, 4, q_std=0.3)
    idx = _select(2, 512, 256, 9)
    idx[0, 5::3] = -1
    idx[1, 100:] = -1
    want = R.mla_sparse_decode(q_abs, q_pe, kv, pe, idx, SCALE)
    got = ops.mla_sparse_decode(q_abs.cuda(), q_pe.cuda(), kv.cuda(), pe.cuda(), idx.cuda(), SCALE)
    _check(got, want, "skipped entries")


def test_growing_scores_exercise_the_rescale(ops):
    """Keys visited in order of increasing score: the running maximum grows by far more than
    2^8 between tiles, so the accumulator is rescaled in tensor memory again and again."""
    batch, heads, keys = 1, 16, 1024
    q_abs, q_pe, kv, pe = _inputs(batch, heads, keys, 5, q_std=1.0)
    # make the score of key t grow with t for every head: add a shared direction
    direction = torch.randn(512).bfloat16()
    q_abs = (q_abs.float() * 0.05 + direction.float() * 0.5).bfloat16()
    ramp = torch.linspace(-1.0, 1.0, keys)[None, :, None]
    kv = (kv.float() * 0.2 + ramp * direction.float()[None, None, :] * 0.3).bfloat16()
    want = R.mla_sparse_decode(q_abs, q_pe, kv, pe, None, SCALE)
    got = ops.mla_sparse_decode(q_abs.cuda(), q_pe.cuda(), kv.cuda(), pe.cuda(), None, SCALE)
    _check(got, want, "growing maximum")


def test_strided_query_views(ops):
    """q_pe as the rope slice of a [B, H, 192] projection output, caches as slices of a batch."""
    batch, heads, keys = 4, 16, 640
    q_abs, q_pe, kv, pe = _inputs(batch, heads, keys, 6, q_std=0.3)
    q_full = torch.zeros(batch, heads, 192, dtype=torch.bfloat16)
    q_full[..., 128:] = q_pe
    idx = _select(batch, keys, 384, 11)
    want = R.mla_sparse_decode(q_abs, q_pe, kv, pe, idx, SCALE)
    got = ops.mla_sparse_decode(q_abs.cuda(), q_full.cuda()[..., 128:], kv.cuda(), pe.cuda(),
                                idx.cuda(), SCALE)
    _check(got, want, "strided q_pe")


def test_no_wait_was_abandoned(ops):
    from racetrack_b200 import _lib
    torch.cuda.synchronize()
    _lib.check(_lib.load().rt_tc_error_state(), "rt_tc_error_state")
