"""The shipped dsv3_2 partition swapped into the synthetic baseline model on a GPU: dispatcher
path, torch.compile path (FX rewrite to the custom op) and the module patchers, all ending in
the CUDA kernels."""
from __future__ import annotations

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from helpers import rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture
def cuda_backend(monkeypatch):
    monkeypatch.setenv("RACETRACK_KERNEL_BACKEND", "cuda")


@pytest.fixture(scope="module")
def spec():
    from racetrack_b200.partition_spec import discover_partitions
    return discover_partitions("dsv3_2")[0]


def test_baseline_model_with_partition_matches_torch_baseline(spec, cuda_backend):
    """The reference's smoke criterion: max-abs-diff <= 5e-2 against the torch baseline
    (racetrack/bench.py:266-268,409)."""
    from racetrack_b200 import _lib
    from racetrack_b200.partitions.dsv3_2 import model as syn
    cfg = syn.DSV3_2_CONFIG
    base = syn.FlattenedDeepSeekModel(cfg).cuda().to(torch.bfloat16)
    part = syn.FlattenedDeepSeekModel(cfg, partition_root=spec.partition_dir).cuda().to(torch.bfloat16)
    part.load_state_dict(base.state_dict())
    tokens = torch.randint(0, cfg.vocab_size, (128,), device="cuda")
    with torch.no_grad():
        want = base(tokens)
        before = _lib.launch_count()
        got = part(tokens)
    assert _lib.launch_count() - before == cfg.num_layers      # one fused_norm_rope launch per layer
    assert float((got.float() - want.float()).abs().max()) <= 5e-2
    assert part.backend_status["cuda"] == "native"


def test_torch_compile_of_the_baseline_model_with_the_shipped_partition(spec, cuda_backend):
    """The partition swapped in for the dsv3_2 baseline model under torch.compile: the model is
    compiled with the partition's backend (pre-trace patches, Dynamo, FX rewrite of the SwiGLU
    pattern to the custom op) and must agree with the eager torch baseline within the
    reference's smoke criterion (racetrack/bench.py:266-268,409), running this library's
    kernels (fused_norm_rope through the dispatcher, fused_swiglu through the rewrite)."""
    from racetrack_b200 import _lib, compile_backend
    from racetrack_b200.partitions.dsv3_2 import model as syn
    cfg = syn.DSV3_2_CONFIG
    base = syn.FlattenedDeepSeekModel(cfg).cuda().to(torch.bfloat16)
    part = syn.FlattenedDeepSeekModel(cfg, partition_root=spec.partition_dir).cuda().to(torch.bfloat16)
    part.load_state_dict(base.state_dict())
    tokens = torch.randint(0, cfg.vocab_size, (64,), device="cuda")
    try:
        with torch.no_grad():
            want = base(tokens)
            compiled, originals = compile_backend.compile_with_partition(part, spec, backend_override="cuda")
            before = _lib.launch_count()
            got = compiled(tokens)
            launches = _lib.launch_count() - before
            again = compiled(tokens)
    finally:
        compile_backend.cleanup_compile_state()
    from racetrack_b200 import pre_trace
    pre_trace.rollback_patches(originals)
    assert launches >= cfg.num_layers, f"only {launches} kernel launches under torch.compile"
    assert float((got.float() - want.float()).abs().max()) <= 5e-2
    assert torch.equal(got, again)


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1, self.w3, self.w2 = (nn.Linear(512, 1024, bias=False), nn.Linear(512, 1024, bias=False),
                                     nn.Linear(1024, 512, bias=False))

    def forward(self, x):
        gate, up = self.w1(x), self.w3(x)
        return self.w2((F.silu(gate.float()) * up.float()).type_as(gate))


def test_torch_compile_rewrites_swiglu_to_the_cuda_kernel(spec, cuda_backend):
    from racetrack_b200 import _lib, compile_backend
    model = Block().cuda().to(torch.bfloat16)
    x = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = model(x)
        compiled, originals = compile_backend.compile_with_partition(model, spec, backend_override="cuda")
        before = _lib.launch_count()
        got = compiled(x)
        launches = _lib.launch_count() - before
    compile_backend.cleanup_compile_state()
    assert launches == 1, "the silu*mul pair should have become one swiglu kernel launch"
    assert rel_err(got, want) <= 1e-2
    assert hasattr(torch.ops.racetrack_b200, "fused_swiglu")
    assert hasattr(torch.ops.racetrack_b200, "fused_residual_norm")
    assert hasattr(torch.ops.racetrack_b200, "fused_act_quant")
    n, h = torch.ops.racetrack_b200.fused_residual_norm(x, x, torch.ones(512, device="cuda"), 1e-6)
    assert torch.equal(h, x + x)
    codes, scales = torch.ops.racetrack_b200.fused_act_quant(x)
    assert codes.dtype == torch.float8_e4m3fn and scales.shape == (64, 4)


class Expert(nn.Module):
    def __init__(self, dim, inter):
        super().__init__()
        self.w1, self.w2, self.w3 = (nn.Linear(dim, inter, bias=False), nn.Linear(inter, dim, bias=False),
                                     nn.Linear(dim, inter, bias=False))

    def forward(self, x):
        return self.w2((F.silu(self.w1(x).float()) * self.w3(x).float()).type_as(x))


class Gate(nn.Module):
    def __init__(self, dim, n_experts):
        super().__init__()
        self.topk, self.n_groups, self.topk_groups = 4, 4, 2
        self.score_func, self.route_scale = "sigmoid", 2.5
        self.weight = nn.Parameter(torch.randn(n_experts, dim) * 0.05)
        self.bias = nn.Parameter(torch.rand(n_experts) * 0.2 - 0.1)


class MoE(nn.Module):
    """Same attributes and control flow as racetrack/models/deepseek.py:965-1022."""

    def __init__(self, dim=512, inter=256, n_experts=16):
        super().__init__()
        self.dim, self.n_routed_experts, self.experts_start_idx = dim, n_experts, 0
        self.gate = Gate(dim, n_experts)
        self.experts = nn.ModuleList(Expert(dim, inter) for _ in range(n_experts))
        self.shared_experts = Expert(dim, inter)

    def forward(self, x):
        from oracle import ref_ops as R
        shape = x.size()
        x = x.view(-1, self.dim)
        weights, indices = R.gate_forward(x, self.gate.weight, self.gate.bias, n_groups=4,
                                          topk_groups=2, topk=4, route_scale=2.5)
        y = torch.zeros_like(x, dtype=torch.float32)
        for i, expert in enumerate(self.experts):
            idx, top = torch.where(indices == i)
            if idx.numel():
                y[idx] += expert(x[idx]) * weights[idx, top, None]
        y += self.shared_experts(x)
        return y.type_as(x).view(shape)


def test_moe_patcher_runs_the_nvfp4_expert_path(spec, cuda_backend):
    from racetrack_b200 import ops, pre_trace
    from racetrack_b200.dispatch import KernelDispatcher
    torch.manual_seed(1)
    moe = MoE().cuda().to(torch.bfloat16)
    moe.gate.bias.data = moe.gate.bias.data.float()
    x = torch.randn(2, 48, 512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        want = moe(x)
        originals = pre_trace.apply_pre_trace_patches(moe, spec, KernelDispatcher(spec.kernel_root))
        got = moe(x)
        ops.tc_error_state()
        pre_trace.rollback_patches(originals)
        again = moe(x)
    assert got.shape == want.shape
    assert torch.equal(again, want)
    # bf16 experts against NVFP4 experts: the format's rounding noise, not a wiring error
    assert rel_err(got, want) <= 0.35
    assert hasattr(moe, "_rt_nvfp4_experts")


def test_indexer_patcher_runs_the_b200_indexer(spec, cuda_backend):
    """An `Indexer` module with the reference's attributes (racetrack/models/deepseek.py:635-653),
    patched through the partition's pre_trace op: beyond index_topk positions the kernel wrapper
    answers (prefill of one chunk, then a decode step of both sequences), and its selections and
    cache updates are those of racetrack_b200.indexer called directly."""
    from racetrack_b200 import indexer as rt_indexer, ops, pre_trace
    from racetrack_b200.dispatch import KernelDispatcher
    from oracle import ref_ops as R
    dim, q_lora, heads, topk, max_len, bsz = 512, 128, 64, 32, 128, 2

    class Indexer(nn.Module):
        def __init__(self):
            super().__init__()
            self.n_heads, self.head_dim, self.index_topk = heads, 128, topk
            self.wq_b = nn.Linear(q_lora, heads * 128, bias=False)
            self.wk = nn.Linear(dim, 128, bias=False)
            self.k_norm = nn.LayerNorm(128)
            self.weights_proj = nn.Linear(dim, heads, bias=False)
            self.register_buffer("k_cache", torch.zeros(bsz, max_len, 128, dtype=torch.float8_e4m3fn))
            self.register_buffer("k_scale_cache", torch.zeros(bsz, max_len, 1))

        def forward(self, x, qr, start_pos, freqs_cis, mask):
            raise AssertionError("the original forward must not run beyond index_topk positions")

    torch.manual_seed(3)
    mod = Indexer().cuda()
    mod.wq_b.to(torch.bfloat16), mod.wk.to(torch.bfloat16)
    table = R.precompute_freqs_cis(64, max_len).cuda()
    w = rt_indexer.IndexerWeights(mod.wq_b.weight, mod.wk.weight, mod.k_norm.weight.float(),
                                  mod.k_norm.bias.float(), mod.weights_proj.weight.float(), heads, 128)
    ref_k = torch.zeros(bsz, max_len, 128, dtype=torch.float8_e4m3fn, device="cuda")
    ref_s = torch.zeros(bsz, max_len, device="cuda")
    originals = pre_trace.apply_pre_trace_patches(mod, spec, KernelDispatcher(spec.kernel_root))
    assert len(originals) == 1
    with torch.no_grad():
        for start, seqlen in ((0, 48), (48, 1)):
            x = torch.randn(bsz, seqlen, dim, device="cuda").bfloat16()
            qr = torch.randn(bsz, seqlen, q_lora, device="cuda").bfloat16()
            mask = torch.full((seqlen, seqlen), float("-inf"), device="cuda").triu_(1) if seqlen > 1 else None
            got = mod(x, qr, start, table[start:start + seqlen], mask)
            ops.tc_error_state()
            assert got.dtype == torch.int64 and got.shape == (bsz, seqlen, topk)
            for b in range(bsz):
                want = rt_indexer.indexer_forward(x[b], qr[b], w, ref_k[b], ref_s[b], start, table, topk,
                                                  causal=mask is not None)
                assert torch.equal(got[b], want.long())
        assert torch.equal(mod.k_cache.view(torch.uint8), ref_k.view(torch.uint8))
        assert torch.equal(mod.k_scale_cache.view(bsz, max_len), ref_s)
    pre_trace.rollback_patches(originals)


def test_indexer_short_circuit_fills_the_key_cache(spec, cuda_backend):
    """Prefill of at most index_topk tokens (the patcher answers arange without running the
    indexer), then decode steps that cross index_topk: the first step past the limit scores the
    WHOLE prefix from the module's key cache, so the short-circuit must have written it
    (racetrack/pre_trace.py:82-112,138). The caches must equal those of the indexer run on
    every chunk, the selection past the limit must equal the full indexer's, and it must pick
    (nearly) the best keys of the CPU oracle's scores over the whole context."""
    from racetrack_b200 import indexer as rt_indexer, ops, pre_trace
    from racetrack_b200.dispatch import KernelDispatcher
    from oracle import ref_ops as R
    dim, q_lora, heads, topk, max_len, bsz, prefill, last = 512, 128, 64, 64, 128, 2, 40, 70

    class Indexer(nn.Module):
        def __init__(self):
            super().__init__()
            self.n_heads, self.head_dim, self.index_topk = heads, 128, topk
            self.wq_b = nn.Linear(q_lora, heads * 128, bias=False)
            self.wk = nn.Linear(dim, 128, bias=False)
            self.k_norm = nn.LayerNorm(128)
            self.weights_proj = nn.Linear(dim, heads, bias=False)
            self.register_buffer("k_cache", torch.zeros(bsz, max_len, 128, dtype=torch.float8_e4m3fn))
            self.register_buffer("k_scale_cache", torch.zeros(bsz, max_len, 1))

        def forward(self, x, qr, start_pos, freqs_cis, mask):
            raise AssertionError("the original forward must not run: short-circuit or kernel")

    torch.manual_seed(5)
    mod = Indexer().cuda()
    mod.wq_b.to(torch.bfloat16), mod.wk.to(torch.bfloat16)
    with torch.no_grad():
        mod.k_norm.weight.add_(torch.randn(128, device="cuda") * 0.02)
        mod.k_norm.bias.add_(torch.randn(128, device="cuda") * 0.02)
    table = R.precompute_freqs_cis(64, max_len).cuda()
    w = rt_indexer.weights_of_module(mod)
    ref_k = torch.zeros(bsz, max_len, 128, dtype=torch.float8_e4m3fn, device="cuda")
    ref_s = torch.zeros(bsz, max_len, device="cuda")
    originals = pre_trace.apply_pre_trace_patches(mod, spec, KernelDispatcher(spec.kernel_root))
    xs, qrs = [], []
    with torch.no_grad():
        chunks = [(0, prefill)] + [(p, 1) for p in range(prefill, last)]
        for start, seqlen in chunks:
            x = torch.randn(bsz, seqlen, dim, device="cuda").bfloat16()
            qr = torch.randn(bsz, seqlen, q_lora, device="cuda").bfloat16()
            xs.append(x), qrs.append(qr)
            mask = torch.full((seqlen, seqlen), float("-inf"), device="cuda").triu_(1) if seqlen > 1 else None
            got = mod(x, qr, start, table[start:start + seqlen], mask)
            ops.tc_error_state()
            end = start + seqlen
            want = torch.stack([rt_indexer.indexer_forward(x[b], qr[b], w, ref_k[b], ref_s[b], start,
                                                           table, topk, causal=mask is not None)
                                for b in range(bsz)]).long()
            if end <= topk:
                assert torch.equal(got, torch.arange(end, device="cuda").view(1, 1, end).expand(bsz, seqlen, end))
            else:
                assert torch.equal(got, want), f"selection at position {start}"
            assert torch.equal(mod.k_cache[:, :end].view(torch.uint8), ref_k[:, :end].view(torch.uint8))
            assert torch.equal(mod.k_scale_cache.view(bsz, max_len)[:, :end], ref_s[:, :end])
        assert int((mod.k_scale_cache.view(bsz, max_len)[:, :last] > 0).sum()) == bsz * last
    pre_trace.rollback_patches(originals)
    # CPU oracle over the whole context of sequence 0: scores of the last query against keys
    # built by the reference chain (racetrack/models/deepseek.py:656-683)
    x_all = torch.cat([x[0] for x in xs]).cpu()
    qr_last, x_last = qrs[-1][0].cpu(), xs[-1][0].cpu()
    fc = table.cpu()
    k = F.linear(x_all, mod.wk.weight.cpu()).view(last, 1, 128)
    k_fp8, k_scale, _ = R.index_prep(k, fc[:last], ln_weight=mod.k_norm.weight.float().cpu(),
                                     ln_bias=mod.k_norm.bias.float().cpu())
    q = F.linear(qr_last, mod.wq_b.weight.cpu()).view(1, heads, 128)
    q_fp8, q_scale, _ = R.index_prep(q, fc[last - 1:last])
    hw = F.linear(x_last.float(), mod.weights_proj.weight.float().cpu()) * heads ** -0.5 * q_scale * 128 ** -0.5
    scores = R.fp8_index(q_fp8.unsqueeze(0), hw.unsqueeze(0), k_fp8.view(1, last, 128),
                         k_scale.view(1, last))[0, 0]
    picked = scores[got[0, 0].cpu()].sum()
    best = scores.topk(topk)[0].sum()
    assert float((picked - best).abs()) <= 2e-3 * topk * float(scores.abs().max())
