"""GPU parity of the decode step of the synthetic DeepSeek-V3.2 layer (racetrack_b200/decode.py:
cache append, absorbed query, sparse indexer, tcgen05 sparse attention, value projection, NVFP4
experts) against the CPU restatement of the reference's decode branch (oracle/ref_layer.py), at
reduced width. Stack criterion of the reference runner: diff <= 0.5 + 0.1 * max|ref|."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_layer
from helpers import rel_err

pytestmark = pytest.mark.gpu

BATCH, CACHE_LEN, START, TOPK = 5, 320, 300, 128


@pytest.fixture(scope="module")
def D():
    from racetrack_b200 import decode, layer, ops
    return decode, layer, ops


def _shape(layer):
    # the attention kernel fixes the latent width (512) and the rope width (64)
    return layer.DSV32.scaled(name="small_decode", hidden=512, heads=16, q_lora=128, kv_lora=512,
                              nope=32, rope=64, v_dim=32, moe_inter=256, n_experts=16, topk=4)


def _setup(D, world=1, rank=0):
    decode, layer, ops = D
    shape = _shape(layer)
    w = layer.make_weights(shape, rank, world, "cpu", std=0.05)
    iw = decode.make_indexer_weights(shape, "cuda", std=0.05)
    caches = decode.DecodeCaches(shape, BATCH, CACHE_LEN, "cuda", fill=START)
    model = decode.DecodeLayer(shape, {k: v.cuda() for k, v in w.items()}, rank, world,
                               index_weights=iw, caches=caches, index_topk=TOPK)
    model.reduce = False
    iw_cpu = {"wq_b": iw.wq_b.cpu(), "wk": iw.wk.cpu(), "k_norm_weight": iw.k_norm_weight.cpu(),
              "k_norm_bias": iw.k_norm_bias.cpu(), "weights_proj": iw.weights_proj.cpu()}
    c_cpu = {"kv": caches.kv.cpu().clone(), "pe": caches.pe.cpu().clone(),
             "index_k": caches.index_k.cpu().clone(), "index_scale": caches.index_scale.cpu().clone()}
    g = torch.Generator().manual_seed(shape.seed + 5)
    hidden = (torch.randn(BATCH, shape.hidden, generator=g) * 0.5).to(torch.bfloat16)
    return shape, w, iw_cpu, c_cpu, model, hidden


def test_decode_attention_matches_the_reference_branch(D):
    decode, layer, ops = D
    shape, w, iw, c_cpu, model, hidden = _setup(D)
    from oracle import ref_ops as R
    normed = R.rms_norm(hidden, torch.ones(shape.hidden, dtype=hidden.dtype), shape.eps)
    want = ref_layer.decode_attention(normed, START, w, iw, c_cpu, shape, shape.heads,
                                      model.freqs.cpu(), TOPK)
    got = model.decode_attention(normed.cuda(), START)
    ops.tc_error_state()
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    assert rel_err(got, want) <= 2e-2, f"relative error {rel_err(got, want)}"
    # the appended cache rows
    assert rel_err(model.caches.kv[:, START], c_cpu["kv"][:, START]) <= 1e-2
    assert rel_err(model.caches.pe[:, START], c_cpu["pe"][:, START]) <= 1e-2
    same = (model.caches.index_k[:, START].cpu().view(torch.uint8) ==
            c_cpu["index_k"][:, START].view(torch.uint8)).float().mean()
    assert float(same) >= 0.9


@pytest.mark.parametrize("layers", [1, 2])
def test_decode_stack_meets_the_runner_criterion(D, layers):
    decode, layer, ops = D
    shape, w, iw, c_cpu, model, hidden = _setup(D)
    ref = ref_layer.decode_stack(hidden, START, [w], iw, [c_cpu], shape, layers, model.freqs.cpu(), TOPK)
    ref4 = ref_layer.decode_stack(hidden, START, [w], iw, [{k: v.clone() for k, v in c_cpu.items()}],
                                  shape, layers, model.freqs.cpu(), TOPK, experts="nvfp4")
    out = model.decode_stack(hidden.cuda(), START, layers)
    ops.tc_error_state()
    assert out.shape == ref.shape and out.dtype == torch.bfloat16
    for r in (ref, ref4):
        diff = float((out.float().cpu() - r.float()).abs().max())
        assert diff <= 0.5 + 0.1 * float(r.float().abs().max())
    assert rel_err(out, ref4) <= 0.25


def test_two_rank_partials_sum_to_the_single_rank_result(D):
    """Heads split over two ranks (evaluated one after the other on this GPU): the partial
    attention outputs add up to the one-rank result; every rank selects the same keys."""
    decode, layer, ops = D
    shape, w, iw, c_cpu, model, hidden = _setup(D)
    from oracle import ref_ops as R
    normed = R.rms_norm(hidden, torch.ones(shape.hidden, dtype=hidden.dtype), shape.eps).cuda()
    whole = model.decode_attention(normed, START).float()
    parts = []
    for rank in range(2):
        _, _, _, _, m, _ = _setup(D, world=2, rank=rank)
        parts.append(m.decode_attention(normed, START).float())
    ops.tc_error_state()
    assert rel_err(parts[0] + parts[1], whole) <= 2e-2


def test_replayed_cuda_graph_equals_the_eager_step(D):
    """The decode step as the benchmark runs it by default: captured once in a CUDA graph and
    replayed (racetrack/bench.py:98-111 does the same for its sweeps). No kernel of the step
    depends on launch timing (the split-K projections add their partial sums in a fixed
    order), so a replay must reproduce the eager result bit for bit, twice in a row, and leave
    the same cache rows behind."""
    decode, layer, ops = D
    shape, w, iw, c_cpu, model, hidden = _setup(D)
    x = hidden.cuda()
    eager = model.decode_stack(x, START, 2).clone()
    ops.tc_error_state()
    rows = [t[:, START].clone() for t in (model.caches.kv, model.caches.pe, model.caches.index_k.view(torch.uint8),
                                          model.caches.index_scale)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model.decode_stack(x, START, 2)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model.decode_stack(x, START, 2)
    for _ in range(2):
        model.caches.kv[:, START].zero_()
        model.caches.pe[:, START].zero_()
        graph.replay()
        ops.tc_error_state()
        assert torch.equal(out, eager), "graph replay differs from the eager step"
        now = [t[:, START] for t in (model.caches.kv, model.caches.pe, model.caches.index_k.view(torch.uint8),
                                     model.caches.index_scale)]
        for a, b in zip(now, rows):
            assert torch.equal(a, b), "cache rows after a replay differ from the eager step's"
