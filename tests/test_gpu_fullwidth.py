"""Parity at FULL width: the configurations the benchmark runs (hidden 7168, 128 heads, 256 NVFP4
experts of width 2048, FP8 / bf16 projections), not scaled-down copies of them.

* the prefill layer on a few dozen tokens against the CPU restatement of racetrack's
  ShardedRealisticBlock evaluated in the layer's own arithmetic (FP8 projections as the
  reference's torch path runs them, NVFP4 experts), under the reference runner's criterion
  diff <= 0.5 + 0.1 * max|ref| (racetrack/realistic_bench.py:530-538); the distance to the
  un-quantised bf16 layer is reported beside it, and the expert stage is compared tightly with
  the NVFP4 oracle on the rows of a handful of experts;
* the routed MoE layer at T = 4096 (sigmoid + bias gate, 8 groups / top-4 / top-8, shared expert):
  routing indices against racetrack's Gate, expert outputs against the NVFP4 oracle for a handful
  of experts, the combine against the slot-ordered fp32 sum.

Weights are drawn on the GPU one expert at a time and copied to the host for the oracle, so both
sides see the same values. Only the experts the sample routes to exist on the host.
"""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from oracle import ref_layer
from oracle import ref_ops as R
from helpers import rel_err

pytestmark = pytest.mark.gpu

ATOL, RTOL = 0.5, 0.1


def _expert_rows(parts, e, topk):
    """(token index, slot) of the rows of expert e in sorted order, and their range."""
    off = parts["offsets"]
    lo, hi = int(off[e]), int(off[e + 1])
    pairs = parts["sorted_pairs"][lo:hi].long()
    return lo, hi, pairs // topk, pairs % topk


def _oracle_expert(x_rt, rows, w13, w2, h_amax, inter):
    """One expert on NVFP4 operands, as oracle/ref_ops.moe_experts_nvfp4 evaluates it."""
    gate_up = (x_rt[rows] @ R.nvfp4_roundtrip(w13).t()).to(torch.bfloat16)
    h = R.swiglu(gate_up[:, :inter], gate_up[:, inter:])
    return (R.nvfp4_roundtrip(h, h_amax) @ R.nvfp4_roundtrip(w2).t()).to(torch.bfloat16)


@pytest.mark.parametrize("tokens,layers", [(16, 1), (8, 2)])
def test_full_width_prefill_layer_meets_the_runner_criterion(tokens, layers):
    """The benchmark's own model object (mixed FP8 / bf16 projections, NVFP4 experts, this
    backend's attention core) on a short sequence.

    The reference's torch path for a quantised linear layer quantises BOTH operands and multiplies
    the dequantised values (act_quant + fp8_gemm's dequantise-then-matmul, deepseek.py:113-121,
    343-345); the oracle evaluates the layer the same way for the FP8 projections and the NVFP4
    experts, and that is what the runner's criterion diff <= 0.5 + 0.1 * max|ref| is asserted
    against, together with a tighter bound. Against the UN-quantised bf16 layer the distance is
    reported and only loosely bounded: e2m1 keeps one mantissa bit, so NVFP4 weights alone move
    the expert outputs of this white-noise model by 17 % RMS and NVFP4 activations by as much
    again; no implementation of the format can meet a 10 % bound there (the oracle's own NVFP4
    evaluation sits as far from the bf16 layer as the GPU does)."""
    from racetrack_b200 import layer, ops
    shape = layer.DSV32
    dev = torch.device("cuda")
    w = layer.make_weights(shape, 0, 1, dev, ffn="none", std=0.02)
    g = torch.Generator(device=dev).manual_seed(shape.seed)
    hidden = torch.empty(tokens, shape.hidden, device=dev, dtype=torch.bfloat16)
    hidden.normal_(mean=0.0, std=0.01, generator=g)
    positions = torch.arange(tokens, device=dev)
    cpu_w = {k: v.cpu() for k, v in w.items()}
    bank = ref_layer.ExpertBank(shape, cpu_w, lambda e: layer.draw_expert(shape, e, dev, std=0.02),
                                quantise=lambda t: ops.fused_nvfp4_quant(t))
    h_cpu, pos_cpu = hidden.cpu(), positions.cpu()
    ref = ref_layer.forward_stack(h_cpu, pos_cpu, [cpu_w], shape, layers, experts="nvfp4", proj="mixed",
                                  before_moe=bank.route)
    ref_bf16 = ref_layer.forward_stack(h_cpu, pos_cpu, [cpu_w], shape, layers, before_moe=bank.route)

    # the device quantiser that filled the bank writes what the CPU oracle's quantiser writes
    e0 = min(bank.drawn)
    w2 = layer.draw_expert(shape, e0, dev, std=0.02)[1]
    codes, sf, gs = ops.fused_nvfp4_quant(w2)
    rc, rsf, rgs = R.nvfp4_quant(w2.cpu())
    assert torch.equal(codes.cpu(), rc) and torch.equal(gs.cpu(), rgs)
    assert torch.equal(sf.cpu().view(torch.uint8), rsf.view(torch.uint8))

    w["experts"] = layer.make_nvfp4_experts(shape, 0, 1, dev, std=0.02)
    model = layer.RealisticLayer(shape, w, proj="mixed")
    assert model.w_qkv_a.fp8 and model.w_o.fp8 and not model.w_q_b.fp8
    out = model.forward_stack(hidden, positions, layers)
    ops.tc_error_state()
    assert bool(torch.isfinite(out.float()).all())
    diff = float((out.float().cpu() - ref.float()).abs().max())
    scale = float(ref.float().abs().max())
    diff16 = float((out.float().cpu() - ref_bf16.float()).abs().max())
    scale16 = float(ref_bf16.float().abs().max())
    own16 = float((ref.float() - ref_bf16.float()).abs().max())
    print(f"full-width prefill layer: tokens={tokens} layers={layers} "
          f"vs quantised oracle diff={diff:.4f} max|ref|={scale:.4f} rel={diff / scale:.4f}; "
          f"vs bf16 layer diff={diff16:.4f} rel={diff16 / scale16:.4f} "
          f"(oracle's own NVFP4/FP8 evaluation vs bf16: {own16 / scale16:.4f})")
    assert diff <= ATOL + RTOL * scale, f"diff {diff} exceeds {ATOL} + {RTOL} * {scale}"
    assert diff <= 0.12 * scale, f"diff {diff} vs max|ref| {scale}"
    assert diff16 <= 0.6 * scale16, f"diff {diff16} vs the bf16 layer's max {scale16}"

    # the expert stage against the NVFP4 oracle, on identical inputs, for a handful of experts
    normed = ops.fused_rms_norm(hidden, model.ones_h, eps=shape.eps)
    attn = model.attention(normed, positions)
    n2, _ = ops.fused_residual_norm(attn, hidden, model.ones_h, eps=shape.eps)
    logits = ops.linear_bf16(n2, model.w_gate, out_dtype=torch.float32)
    weights, indices = ops.fused_moe_route(logits, None, n_groups=1, topk_groups=1, topk=shape.topk,
                                           route_scale=1.0, score_func="topk_softmax")
    parts: dict = {}
    from racetrack_b200 import moe
    moe.fused_moe_experts(n2, weights, indices, model.experts, n_experts=shape.n_experts, parts=parts)
    ops.tc_error_state()
    parts = {k: v.cpu() for k, v in parts.items()}
    x_rt = R.nvfp4_roundtrip(n2.cpu())
    counts = parts["offsets"][1:] - parts["offsets"][:-1]
    busiest = counts.topk(5)[1].tolist()
    bank.need(busiest)
    for e in busiest:
        lo, hi, rows, _ = _expert_rows(parts, e, shape.topk)
        want = _oracle_expert(x_rt, rows, cpu_w["w13"][e], cpu_w["w2"][e], parts["h_amax"], shape.moe_inter)
        got = parts["expert_out"][lo:hi]
        assert rel_err(got, want) <= 3e-2, f"expert {e}: {rel_err(got, want)}"


def test_c3_moe_layer_at_full_width():
    """T = 4096 tokens ~ N(0, 1), gate [256, 7168] with sigmoid scores + bias, 8 groups / top-4 /
    top-8, route scale 2.5, 256 NVFP4 experts (w13 [4096, 7168], w2 [7168, 2048]) + one bf16
    shared expert: the grouped GEMMs walk all 256 groups at K = 7168 and K = 2048."""
    from racetrack_b200 import layer, moe, ops
    shape = layer.DSV32
    dev = torch.device("cuda")
    tokens = 4096
    g = torch.Generator(device=dev).manual_seed(shape.seed + 7)
    x = torch.empty(tokens, shape.hidden, device=dev, dtype=torch.bfloat16).normal_(generator=g)
    w_gate = torch.empty(shape.n_experts, shape.hidden, device=dev, dtype=torch.bfloat16)
    w_gate.normal_(mean=0.0, std=0.02, generator=g)
    bias = torch.empty(shape.n_experts, device=dev).uniform_(-0.1, 0.1, generator=g)
    experts = layer.make_nvfp4_experts(shape, 0, 1, dev, std=0.02)
    sw13, sw2 = layer.draw_expert(shape, shape.n_experts, dev, std=0.02)
    gate_up = ops.linear_bf16(x, sw13)
    shared = ops.linear_bf16(ops.fused_swiglu(gate_up[:, :shape.moe_inter], gate_up[:, shape.moe_inter:]), sw2)
    kw = dict(n_groups=8, topk_groups=4, topk=shape.topk, route_scale=2.5)
    parts: dict = {}
    y = moe.fused_moe_forward(x, w_gate, bias, experts, n_experts=shape.n_experts,
                              score_func="sigmoid", shared=shared, parts=parts, **kw)
    ops.tc_error_state()
    assert bool(torch.isfinite(y.float()).all())

    # routing: racetrack's Gate on the CPU (fp32 logits of the same bf16 operands)
    x_cpu = x.cpu()
    w_ref, i_ref = R.gate_forward(x_cpu, w_gate.cpu(), bias.cpu(), **kw)
    idx = parts["indices"].cpu()
    same = (idx.sort(dim=-1)[0] == i_ref.sort(dim=-1)[0]).all(dim=-1)
    assert float(same.float().mean()) >= 0.99, f"{int((~same).sum())} of {tokens} rows route differently"
    wts = parts["weights"].cpu()
    order_g, order_r = idx.sort(dim=-1)[1], i_ref.sort(dim=-1)[1]
    assert float((wts.gather(1, order_g)[same] - w_ref.gather(1, order_r)[same]).abs().max()) <= 1e-4

    # shared expert against the bf16 reference MLP on a slice of the tokens
    sl = slice(0, 256)
    want_shared = F.linear(R.swiglu(*F.linear(x_cpu[sl], sw13.cpu()).chunk(2, dim=-1)), sw2.cpu())
    assert rel_err(shared[sl], want_shared) <= 2e-2

    # routed experts: the NVFP4 oracle on the rows of a handful of experts (first, last, busiest,
    # emptiest), identical inputs and the product's own tensor-wide scales
    cpu = {k: v.cpu() for k, v in parts.items()}
    counts = cpu["offsets"][1:] - cpu["offsets"][:-1]
    assert int(counts.sum()) == tokens * shape.topk
    picks = sorted({0, shape.n_experts - 1, int(counts.argmax()), int(counts.argmin())})
    x_rt = R.nvfp4_roundtrip(x_cpu)
    for e in picks:
        lo, hi, rows, slots = _expert_rows(cpu, e, shape.topk)
        if hi == lo:
            continue
        assert bool((idx[rows, slots] == e).all()), "permutation lists a pair under the wrong expert"
        w13, w2 = (t.cpu() for t in layer.draw_expert(shape, e, dev, std=0.02))
        want = _oracle_expert(x_rt, rows, w13, w2, cpu["h_amax"], shape.moe_inter)
        got = cpu["expert_out"][lo:hi]
        assert rel_err(got, want) <= 3e-2, f"expert {e} ({hi - lo} rows): {rel_err(got, want)}"
        # and against the un-quantised bf16 expert: e2m1's one mantissa bit, not a bug
        full = F.linear(R.swiglu(*F.linear(x_cpu[rows], w13).chunk(2, dim=-1)), w2)
        assert rel_err(got, full) <= 0.5

    # combine: fp32 sum in slot order + shared, rounded once (deepseek.py:1018-1022), every token
    eo, pp = parts["expert_out"], parts["pair_pos"].view(tokens, shape.topk).long()
    acc = torch.zeros(tokens, shape.hidden, device=dev, dtype=torch.float32)
    for s in range(shape.topk):
        acc = acc + eo[pp[:, s]].float() * parts["weights"][:, s:s + 1]
    want_y = (acc + shared.float()).to(torch.bfloat16)
    assert torch.equal(y, want_y)
