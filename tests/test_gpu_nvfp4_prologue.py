"""The MLA-prologue ops of the dsv3_2_nvfp4 partition on the B200 kernels, resolved through the
partition's dispatcher as racetrack would, against the CPU restatement of their torch definitions
(oracle/ref_ops.py, ref: scripts/recipes_nvfp4.py:38-151). bf16 outputs within 1e-2 of the largest
reference element; FP8 codes and the selected index sets as the indexer tests compare them."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_ops as R
from helpers import rel_err

pytestmark = pytest.mark.gpu

DIM, Q_LORA, KV_LORA, ROPE, HEADS, NOPE, IDX_HEADS = 1024, 256, 512, 64, 16, 128, 64


@pytest.fixture
def ops_of_partition(monkeypatch):
    monkeypatch.setenv("RACETRACK_KERNEL_BACKEND", "cuda")
    from racetrack_b200.dispatch import KernelDispatcher
    from racetrack_b200.partition_spec import discover_partitions
    spec = discover_partitions("dsv3_2_nvfp4")[0]
    assert {"fused_ar_rms_qkv_proj", "fused_indexer_k_path", "fused_q_indexer_score",
            "fused_q_rope_quant"} <= set(spec.op_names)
    disp = KernelDispatcher(spec.kernel_root)

    def call(name, *a, **kw):
        def fallback(*_a, **_k):
            raise AssertionError("the torch fallback must not run with the cuda backend selected")
        return disp.call(name, fallback, *a, **kw)
    return call


def _mk(seed):
    g = torch.Generator().manual_seed(seed)
    return lambda *s, std=1.0: (torch.randn(*s, generator=g) * std)


def _cuda(*ts):
    return [t.cuda() if t is not None else None for t in ts]


@pytest.mark.parametrize("with_residual", [True, False])
def test_ar_rms_qkv_proj(ops_of_partition, with_residual):
    from racetrack_b200 import ops
    mk = _mk(1)
    x, res = mk(2, 9, DIM).bfloat16(), mk(2, 9, DIM).bfloat16() if with_residual else None
    nw = 1 + mk(DIM, std=0.02)
    wq_a, wkv_a, wk = (mk(n, DIM, std=0.03).bfloat16() for n in (Q_LORA, KV_LORA + ROPE, 128))
    kw = dict(eps=1e-6, q_lora_rank=Q_LORA, kv_lora_rank=KV_LORA, qk_rope_head_dim=ROPE)
    want = R.fused_ar_rms_qkv_proj(x, res, nw, wq_a, wkv_a, wk, **kw)
    got = ops_of_partition("fused_ar_rms_qkv_proj", *_cuda(x, res, nw, wq_a, wkv_a, wk), **kw)
    ops.tc_error_state()
    assert torch.equal(got[0].cpu(), want[0]), "residual_out must be exact"
    for name, g_, w_ in zip(("normed", "q_c", "kv_c", "k_pe", "indexer_k"), got[1:], want[1:]):
        assert g_.shape == w_.shape, name
        assert rel_err(g_, w_) <= 1e-2, f"{name}: {rel_err(g_, w_)}"


def test_indexer_k_path_appends_the_cache(ops_of_partition):
    mk = _mk(2)
    bsz, seqlen, start, max_len = 2, 11, 5, 32
    k = mk(bsz, seqlen, 128).bfloat16()
    lnw, lnb = 1 + mk(128, std=0.02), mk(128, std=0.02)
    fc = R.precompute_freqs_cis(ROPE, max_len)[start:start + seqlen]
    H = R.hadamard_matrix(128)
    kw = dict(ln_eps=1e-6, rope_head_dim=ROPE, start_pos=start)
    kc, ks = torch.zeros(bsz, max_len, 128, dtype=torch.float8_e4m3fn), torch.zeros(bsz, max_len, 1)
    want_codes, want_scale = R.fused_indexer_k_path(k, lnw, lnb, fc, kc, ks, **kw)
    kc_g, ks_g = torch.zeros_like(kc).cuda(), torch.zeros_like(ks).cuda()
    got_codes, got_scale = ops_of_partition("fused_indexer_k_path", *_cuda(k, lnw, lnb, fc, H), kc_g, ks_g,
                                            ln_dim=128, block_size=128, **kw)
    assert got_codes.shape == want_codes.shape and got_scale.shape == (bsz, seqlen, 1)
    same = (got_codes.cpu().view(torch.uint8) == want_codes.view(torch.uint8)).all(dim=-1)
    assert float(same.float().mean()) >= 0.8, "FP8 codes of most rows must be identical"
    assert torch.equal(got_scale.cpu()[same], want_scale[same])
    deq_g = got_codes.float().cpu() * got_scale.cpu()
    deq_w = want_codes.float() * want_scale
    assert rel_err(deq_g, deq_w) <= 7e-2          # one e4m3 step where a bf16 rounding flipped a code
    assert torch.equal(kc_g[:, start:start + seqlen].cpu().view(torch.uint8), got_codes.cpu().view(torch.uint8))
    assert torch.equal(ks_g[:, start:start + seqlen].cpu(), got_scale.cpu())
    assert float(ks_g[:, :start].abs().max()) == 0 and float(ks_g[:, start + seqlen:].abs().max()) == 0


def test_q_indexer_score(ops_of_partition):
    from racetrack_b200 import ops
    mk = _mk(3)
    bsz, seqlen, end_pos, topk = 2, 3, 200, 48
    qk = NOPE + ROPE
    qr, nx = mk(bsz, seqlen, Q_LORA).bfloat16(), mk(bsz, seqlen, DIM).bfloat16()
    wq_b = mk(HEADS * qk, Q_LORA, std=0.05).bfloat16()
    iwq_b = mk(IDX_HEADS * 128, Q_LORA, std=0.05).bfloat16()
    iwp = mk(IDX_HEADS, DIM, std=0.03)
    wkv_b = mk(HEADS * (NOPE + 128), KV_LORA, std=0.05).bfloat16()
    fc = R.precompute_freqs_cis(ROPE, 256)[end_pos - seqlen:end_pos]
    kc, ksc = R.act_quant(mk(bsz, 256, 128).bfloat16())
    kw = dict(n_heads=HEADS, qk_head_dim=qk, qk_nope_head_dim=NOPE, kv_lora_rank=KV_LORA, idx_n_heads=IDX_HEADS,
              idx_head_dim=128, rope_head_dim=ROPE, idx_softmax_scale=128 ** -0.5, index_topk=topk,
              end_pos=end_pos)
    want = R.fused_q_indexer_score(qr, nx, wq_b, iwq_b, iwp, wkv_b, fc, kc, ksc, **kw)
    got = ops_of_partition("fused_q_indexer_score", *_cuda(qr, nx, wq_b, iwq_b, iwp, wkv_b, fc,
                                                           R.hadamard_matrix(128), kc, ksc),
                           eps=1e-6, softmax_scale=qk ** -0.5, start_pos=end_pos - seqlen, block_size=128, **kw)
    ops.tc_error_state()
    for name, g_, w_ in zip(("q_nope", "q_nope_absorbed", "q_pe"), got[:3], want[:3]):
        assert g_.shape == w_.shape, name
        assert rel_err(g_, w_) <= 1e-2, f"{name}: {rel_err(g_, w_)}"
    picked = got[3].cpu()
    assert picked.shape == want[3].shape and picked.dtype == torch.int64
    # the selection must be (nearly) the best set under the oracle's own scores
    q_fp8, q_scale = [], []
    idx_q = torch.nn.functional.linear(qr, iwq_b).view(bsz, seqlen, IDX_HEADS, 128)
    for b in range(bsz):
        c, s, _ = R.index_prep(idx_q[b], fc, rope_dim=ROPE)
        q_fp8.append(c), q_scale.append(s)
    w_ = torch.nn.functional.linear(nx.float(), iwp) * IDX_HEADS ** -0.5 * torch.stack(q_scale) * 128 ** -0.5
    scores = R.fp8_index(torch.stack(q_fp8), w_, kc[:, :end_pos], ksc[:, :end_pos].reshape(bsz, end_pos))
    best = scores.topk(topk, dim=-1)[0].sum(-1)
    mine = scores.gather(-1, picked).sum(-1)
    assert float((best - mine).abs().max()) <= 2e-3 * topk * float(scores.abs().max())


def test_q_rope_quant(ops_of_partition):
    mk = _mk(4)
    q_pe = mk(2, 7, HEADS, ROPE).bfloat16()
    fc = R.precompute_freqs_cis(ROPE, 64)[20:27]
    want = R.fused_q_rope_quant(q_pe, fc)
    got = ops_of_partition("fused_q_rope_quant", q_pe.cuda(), fc.cuda(), block_size=128)
    assert torch.equal(got.cpu(), want), "interleaved RoPE is evaluated in fp32 exactly like the reference"


def test_batched_gemm_and_fp32_weight_projection():
    """The two building blocks the prologue ops add: the per-head batched bf16 GEMM (on strided
    [T, H, K] slices) and the fp32-weight projection as two bf16 halves."""
    from racetrack_b200 import ops
    mk = _mk(5)
    for tokens in (1, 64, 300):
        q = mk(tokens, 16, 192).bfloat16()
        w = mk(16, 512, 128, std=0.05).bfloat16()
        got = ops.linear_bf16_batched(q.cuda()[..., :128], w.cuda())
        want = torch.einsum("thk,hnk->thn", q[..., :128].float(), w.float())
        assert rel_err(got, want) <= 1e-2
    x = mk(77, 1024).bfloat16()
    w32 = mk(64, 1024, std=0.03)
    got = ops.linear_f32_weight(x.cuda(), w32.cuda())
    want = torch.nn.functional.linear(x.float(), w32)
    assert got.dtype == torch.float32 and float((got.cpu() - want).abs().max()) <= 2e-5 * float(want.abs().max()) + 1e-6
    ops.tc_error_state()
