"""GPU parity of the synthetic DeepSeek-V3.2 layer stack (racetrack_b200/layer.py) against the
CPU restatement of racetrack's sharded realistic layer (oracle/ref_layer.py), at reduced width.
Criterion of the reference runner: diff <= atol + rtol * max|ref| with atol 0.5, rtol 0.1
(racetrack/realistic_bench.py:530-538); a tighter bound is checked as well."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_layer
from helpers import rel_err

pytestmark = pytest.mark.gpu

ATOL, RTOL = 0.5, 0.1


@pytest.fixture(scope="module")
def L():
    from racetrack_b200 import layer, ops
    return layer, ops


def small_shape(layer):
    return layer.DSV32.scaled(name="small", hidden=512, heads=8, q_lora=128, kv_lora=64, nope=32,
                              rope=16, v_dim=32, moe_inter=256, n_experts=16, topk=4,
                              dense_inter=1024)


def _inputs(shape, tokens, seed=0):
    g = torch.Generator().manual_seed(shape.seed + seed)
    hidden = (torch.randn(tokens, shape.hidden, generator=g) * 0.5).to(torch.bfloat16)
    return hidden, torch.arange(tokens, dtype=torch.int64)


def _to_cuda(w):
    return {k: v.cuda() for k, v in w.items()}


def _check(out, ref, tight):
    diff = float((out.float().cpu() - ref.float()).abs().max())
    scale = float(ref.float().abs().max())
    assert diff <= ATOL + RTOL * scale, f"diff {diff} vs max|ref| {scale}"
    assert rel_err(out, ref) <= tight, f"relative error {rel_err(out, ref)}"


@pytest.mark.parametrize("ffn,tight", [("moe", 6e-2), ("dense", 2e-2)])
@pytest.mark.parametrize("tokens,layers", [(96, 2), (1, 1), (130, 3)])
def test_layer_stack_matches_reference_layer(L, ffn, tight, tokens, layers):
    layer, ops = L
    shape = small_shape(layer)
    w = layer.make_weights(shape, 0, 1, "cpu", ffn=ffn, std=0.05)
    hidden, pos = _inputs(shape, tokens)
    ref = ref_layer.forward_stack(hidden, pos, [w], shape, layers, ffn=ffn)
    model = layer.RealisticLayer(shape, _to_cuda(w), ffn=ffn)
    out = model.forward_stack(hidden.cuda(), pos.cuda(), layers)
    ops.tc_error_state()
    assert out.shape == ref.shape and out.dtype == torch.bfloat16
    _check(out, ref, tight)


def test_rank_partials_sum_to_the_unsharded_layer(L):
    """Tensor-parallel heads and expert-parallel experts: the partial results of the two ranks
    of a world of 2 add up to what a single rank computes (all-reduce emulated by a sum)."""
    layer, ops = L
    shape = small_shape(layer)
    tokens = 64
    hidden, pos = _inputs(shape, tokens, seed=3)
    full = layer.RealisticLayer(shape, _to_cuda(layer.make_weights(shape, 0, 1, "cpu", std=0.05)))
    ranks = []
    for r in range(2):
        m = layer.RealisticLayer(shape, _to_cuda(layer.make_weights(shape, r, 2, "cpu", std=0.05)), r, 2)
        m.reduce = False
        ranks.append(m)
    normed = ops.fused_rms_norm(hidden.cuda(), full.ones_h, eps=shape.eps)
    a_full = full.attention(normed, pos.cuda()).float()
    a_sum = sum(m.attention(normed, pos.cuda()).float() for m in ranks)
    assert rel_err(a_sum, a_full) <= 1e-2
    f_full = full.ffn_forward(normed).float()
    f_sum = sum(m.ffn_forward(normed).float() for m in ranks)
    ops.tc_error_state()
    # each rank quantises swiglu(h) with its own tensor-wide scale: close, not identical
    assert rel_err(f_sum, f_full) <= 5e-2
    # and the reference layer evaluated with two ranks agrees with the unsharded product
    ws = [layer.make_weights(shape, r, 2, "cpu", std=0.05) for r in range(2)]
    ref = ref_layer.forward_stack(hidden, pos, ws, shape, 1)
    out = full.forward_stack(hidden.cuda(), pos.cuda(), 1)
    _check(out, ref, 6e-2)
