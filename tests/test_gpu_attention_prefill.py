"""GPU parity of the causal attention kernel of the prefill stack (rt_attn_causal_prefill, tcgen05:
scores and probabilities in tensor memory) against the CPU restatement of racetrack's
causal_attention (oracle/ref_layer.causal_attention, ref: racetrack/runtime/torch_ops.py:97-110).
Tolerance: 1e-2 of the largest reference element (bf16 outputs, bf16 probabilities)."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_layer
from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from racetrack_b200 import ops
    return ops


def _qkv(tokens, heads, nope, rope, v_dim, seed, shared_pe=True, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, generator=g) * scale).to(torch.bfloat16)
    q = mk(tokens, heads, nope + rope)
    k_nope = mk(tokens, heads, nope)
    k_pe = mk(tokens, rope) if shared_pe else mk(tokens, heads, rope)
    v = mk(tokens, heads, v_dim)
    return q, k_nope, k_pe, v


def _reference(q, k_nope, k_pe, v):
    heads = q.shape[1]
    pe = k_pe.unsqueeze(1).expand(-1, heads, -1) if k_pe.dim() == 2 else k_pe
    return ref_layer.causal_attention(q, torch.cat((k_nope, pe), dim=-1), v)


@pytest.mark.parametrize("schedule", [1, 2])
@pytest.mark.parametrize("tokens,heads", [(1, 1), (7, 2), (128, 1), (129, 3), (256, 2), (300, 4),
                                          (513, 2), (640, 1), (1000, 3), (1300, 2)])
def test_mla_shape_matches_the_reference(ops, tokens, heads, schedule):
    """The DeepSeek-V3.2 head: 128 nope + 64 shared rope dims, values of width 128; ragged
    lengths around the 128-row tiles, the 256-row blocks of the single-CTA schedule (1) and
    the 512-row blocks of the CTA-pair schedule (2)."""
    q, kn, kp, v = _qkv(tokens, heads, 128, 64, 128, 100 + tokens)
    want = _reference(q, kn, kp, v)
    prev = ops.attention_prefill_schedule(schedule)
    try:
        got = ops.attention_prefill(q.cuda(), kn.cuda(), kp.cuda(), v.cuda())
    finally:
        ops.attention_prefill_schedule(prev)
    ops.tc_error_state()
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    assert rel_err(got, want) <= 1e-2, f"relative error {rel_err(got, want)}"


@pytest.mark.parametrize("nope,rope,v_dim,shared", [(32, 16, 32, True), (64, 64, 64, False),
                                                    (128, 0, 128, True), (96, 32, 72, True),
                                                    (48, 0, 16, True)])
def test_other_head_shapes(ops, nope, rope, v_dim, shared):
    """Widths that are not multiples of 64 are zero-filled by the tensor maps; a per-head rope
    key and no rope key at all are the same kernel."""
    q, kn, kp, v = _qkv(200, 3, nope, max(rope, 8), v_dim, 7 + nope, shared_pe=shared)
    if rope == 0:
        q, kp = q[..., :nope].contiguous(), None
        want = ref_layer.causal_attention(q, kn, v)
    else:
        want = _reference(q, kn, kp, v)
    got = ops.attention_prefill(q.cuda(), kn.cuda(), kp.cuda() if kp is not None else None, v.cuda())
    ops.tc_error_state()
    assert rel_err(got, want) <= 1e-2, f"relative error {rel_err(got, want)}"


@pytest.mark.parametrize("schedule", [1, 2])
def test_strided_views_of_projection_outputs(ops, schedule):
    """q a view of the q_b output, k_nope / v column slices of one kv_b output [T, H, nope + v]:
    consumed in place; a per-head rope key as well."""
    tokens, heads = 333, 4
    prev = ops.attention_prefill_schedule(schedule)
    try:
        _strided_case(ops, tokens, heads)
        q, kn, kp, v = _qkv(700, 3, 128, 64, 128, 58, shared_pe=False)
        got = ops.attention_prefill(q.cuda(), kn.cuda(), kp.cuda(), v.cuda())
        ops.tc_error_state()
        assert rel_err(got, _reference(q, kn, kp, v)) <= 1e-2
    finally:
        ops.attention_prefill_schedule(prev)


def _strided_case(ops, tokens, heads):
    q, kn, kp, v = _qkv(tokens, heads, 128, 64, 128, 55)
    kv = torch.cat((kn, v), dim=-1).cuda()                    # [T, H, 256]
    qbuf = torch.zeros(tokens, heads * 192 + 64, dtype=torch.bfloat16, device="cuda")
    qv = qbuf[:, :heads * 192].view(tokens, heads, 192)
    qv.copy_(q)
    got = ops.attention_prefill(qv, kv[..., :128], kp.cuda(), kv[..., 128:])
    ops.tc_error_state()
    assert rel_err(got, _reference(q, kn, kp, v)) <= 1e-2


@pytest.mark.parametrize("schedule", [1, 2])
def test_growing_maxima_and_large_scores(ops, schedule):
    """Scores that grow along the sequence (the running maximum is replaced again and again,
    the accumulator rescaled) and a wide score range (exp2 underflow of the early keys)."""
    prev = ops.attention_prefill_schedule(schedule)
    try:
        _growing_case(ops)
    finally:
        ops.attention_prefill_schedule(prev)


def _growing_case(ops):
    tokens, heads = 640, 2
    q, kn, kp, v = _qkv(tokens, heads, 128, 64, 128, 91, scale=1.0)
    ramp = torch.linspace(0.2, 3.0, tokens).view(tokens, 1, 1)
    kn = (kn.float() * ramp).to(torch.bfloat16)
    want = _reference(q, kn, kp, v)
    got = ops.attention_prefill(q.cuda(), kn.cuda(), kp.cuda(), v.cuda())
    ops.tc_error_state()
    assert rel_err(got, want) <= 1e-2, f"relative error {rel_err(got, want)}"


def test_whole_key_form_and_scale(ops):
    """causal_attention(q, k, v) with whole keys, and an explicit softmax scale."""
    q, kn, kp, v = _qkv(150, 2, 128, 64, 128, 23, shared_pe=False)
    k = torch.cat((kn, kp), dim=-1)
    got = ops.causal_attention(q.cuda(), k.cuda(), v.cuda())
    ops.tc_error_state()
    assert rel_err(got, ref_layer.causal_attention(q, k, v)) <= 1e-2
    scaled = ops.attention_prefill(q.cuda(), kn.cuda(), kp.cuda(), v.cuda(), softmax_scale=0.05)
    want = ref_layer.causal_attention((q.float() * 0.05 * 192 ** 0.5).to(torch.bfloat16), k, v)
    assert rel_err(scaled, want) <= 2e-2


def test_longer_sequence_many_heads_against_the_same_math_on_the_gpu(ops):
    """T = 2048 x 16 heads: the CPU oracle on 4 of the heads, and all heads against an fp32
    evaluation of the same formula in torch on the GPU (a yardstick, not the oracle)."""
    tokens, heads = 2048, 16
    q, kn, kp, v = _qkv(tokens, heads, 128, 64, 128, 77, scale=0.5)
    qc, knc, kpc, vc = q.cuda(), kn.cuda(), kp.cuda(), v.cuda()
    got = ops.attention_prefill(qc, knc, kpc, vc)
    ops.tc_error_state()
    pick = [0, 5, 10, 15]
    want = _reference(q[:, pick], kn[:, pick], kp, v[:, pick])
    assert rel_err(got[:, pick], want) <= 1e-2
    k = torch.cat((knc, kpc.unsqueeze(1).expand(-1, heads, -1)), dim=-1)
    scores = torch.einsum("thd,shd->hts", qc.float(), k.float()) * 192 ** -0.5
    scores = scores.masked_fill(~torch.ones(tokens, tokens, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    full = torch.einsum("hts,shd->thd", torch.softmax(scores, dim=-1).to(torch.bfloat16).float(), vc.float())
    assert rel_err(got, full) <= 1e-2


@pytest.mark.parametrize("tokens,heads", [(300, 3), (1500, 2)])
def test_fp8_epilogue_equals_act_quant_of_the_bf16_output(tokens, heads):
    """attention_prefill(quantized=True): the codes and scales the kernel's own epilogue writes are
    those fused_act_quant makes of the bf16 output of the same schedule (racetrack/models/
    deepseek.py:85-107 applied to racetrack/runtime/torch_ops.py:97-110), bit for bit; other head
    shapes run the quantiser behind the kernel."""
    from racetrack_b200 import ops
    g = torch.Generator().manual_seed(tokens)
    q = (torch.randn(tokens, heads, 192, generator=g) * 0.4).bfloat16().cuda()
    kv = (torch.randn(tokens, heads, 256, generator=g) * 0.4).bfloat16().cuda()
    kpe = (torch.randn(tokens, 64, generator=g) * 0.4).bfloat16().cuda()
    prev = ops.attention_prefill_schedule(2)
    try:
        plain = ops.attention_prefill(q, kv[..., :128], kpe, kv[..., 128:])
    finally:
        ops.attention_prefill_schedule(prev)
    want_c, want_s = ops.fused_act_quant(plain.view(tokens, heads * 128))
    codes, scales = ops.attention_prefill(q, kv[..., :128], kpe, kv[..., 128:], quantized=True)
    assert torch.equal(codes.view(torch.uint8), want_c.view(torch.uint8))
    assert torch.equal(scales, want_s)
    buf = (torch.empty(tokens, heads * 128, dtype=torch.uint8, device="cuda"),
           torch.empty(tokens, heads, dtype=torch.float32, device="cuda"))
    ops.attention_prefill(q, kv[..., :128], kpe, kv[..., 128:], quantized=True, out=buf)
    assert torch.equal(buf[0], want_c.view(torch.uint8)) and torch.equal(buf[1], want_s)
    # another head shape: same contract through the two-kernel route
    q2, k2, v2 = q[..., :96].contiguous(), kv[..., :64].contiguous(), kv[..., 128:256].contiguous()
    c2, s2 = ops.attention_prefill(q2, k2, kpe[:, :32].contiguous(), v2, quantized=True)
    w2 = ops.fused_act_quant(ops.attention_prefill(q2, k2, kpe[:, :32].contiguous(), v2).view(tokens, heads * 128))
    assert torch.equal(c2.view(torch.uint8), w2[0].view(torch.uint8)) and torch.equal(s2, w2[1])
    ops.tc_error_state()
