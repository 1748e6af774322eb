"""The plugin surface (PartitionSpec / KernelDispatcher / fx_patterns / pre_trace /
RacetrackBackend) behaves like racetrack's: contract tests in the style of the reference's
tests/test_smoke.py, tests/test_partition_lint.py and tests/test_gsm8k_real_kernels.py, on CPU with
fake kernel directories (no CUDA kernel is called here)."""
from __future__ import annotations

import hashlib
import os
import textwrap

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from racetrack_b200 import compile_backend, fx_patterns, pre_trace
from racetrack_b200.dispatch import KernelDispatcher
from racetrack_b200.partition_spec import (BASELINE_SPEC, FusedOp, PartitionSpec,
                                            discover_partitions, load_spec, partitions_root)


@pytest.fixture
def backend_env(monkeypatch):
    def set_backend(name):
        monkeypatch.setenv("RACETRACK_KERNEL_BACKEND", name)
    monkeypatch.delenv("RACETRACK_KERNEL_BACKEND", raising=False)
    return set_backend


def _fake_kernel_dir(tmp_path, body: str, backend: str = "cuda"):
    d = tmp_path / "kernels" / backend
    d.mkdir(parents=True)
    (d / "ops.py").write_text(textwrap.dedent(body))
    (d / "_private.py").write_text("raise RuntimeError('underscore modules are never imported')")
    return tmp_path / "kernels"


def test_shipped_partition_loads_and_its_hash_names_the_directory():
    specs = discover_partitions("dsv3_2")
    assert len(specs) == 1
    spec = specs[0]
    spec_bytes = (spec.partition_dir / "spec.py").read_bytes()
    assert spec.partition_hash == hashlib.sha256(spec_bytes).hexdigest()[:8] == spec.partition_id
    assert spec.label == f"dsv3_2/{spec.partition_hash}"
    assert [op.name for op in spec.fx_ops] == ["fused_norm_rope", "fused_swiglu",
                                               "fused_residual_norm", "fused_act_quant"]
    assert [op.name for op in spec.pre_trace_ops] == ["fused_single_token_moe", "fused_full_topk_indexer"]
    assert [op.name for op in spec.module_patch_ops] == ["fused_mlp_gate_up_proj"]
    assert spec.op_names == tuple(op.name for op in spec.fused_ops)
    assert load_spec("dsv3_2", spec.partition_hash) == spec
    assert FusedOp("a", "fx_pattern").to_dict() == {"name": "a", "kind": "fx_pattern"}
    assert BASELINE_SPEC.fused_ops == () and len(BASELINE_SPEC.partition_id) == 8
    with pytest.raises(FileNotFoundError):
        load_spec("dsv3_2", "deadbeef")
    assert discover_partitions("no_such_model") == []


def test_every_fused_op_has_a_cuda_kernel_of_that_name():
    """The reference's lint (tests/test_partition_lint.py:57-91) for the one backend here."""
    spec = discover_partitions("dsv3_2")[0]
    disp = KernelDispatcher(spec.kernel_root)
    names = set()
    for path in sorted((spec.kernel_root / "cuda").glob("*.py")):
        text = path.read_text()
        assert "BACKEND_AVAILABLE" in text
        names.update(line.split("=")[0].strip() for line in text.splitlines()
                     if line.startswith("fused_") and "=" in line)
        names.update(line.split("(")[0][4:] for line in text.splitlines() if line.startswith("def fused_"))
    for op in spec.fused_ops:
        assert op.name in names, f"no cuda kernel named {op.name}"
    assert disp.backend_status("torch") == "native"


def test_partitions_root_can_point_at_another_checkout(tmp_path, monkeypatch):
    p = tmp_path / "m" / "abcd1234"
    (p / "kernels").mkdir(parents=True)
    (p / "spec.py").write_text("FUSED_OPS = [{'name': 'fused_swiglu', 'kind': 'fx_pattern'}]\n")
    monkeypatch.setenv("RACETRACK_PARTITIONS_ROOT", str(tmp_path))
    assert partitions_root() == tmp_path
    specs = discover_partitions("m")
    assert [s.partition_hash for s in specs] == ["abcd1234"] and specs[0].op_names == ("fused_swiglu",)
    assert specs[0].partition_id != "abcd1234"      # the id is the hash of the bytes


def test_dispatcher_routes_by_env_and_never_degrades_silently(tmp_path, backend_env):
    root = _fake_kernel_dir(tmp_path, """
        BACKEND_AVAILABLE = True
        CALLS = []
        def fused_swiglu(gate, up, *, fallback):
            CALLS.append("cuda")
            return fallback(gate, up) + 1
    """)
    disp = KernelDispatcher(root)
    fallback = lambda g, u: g * u
    g, u = torch.ones(3), torch.full((3,), 2.0)
    assert torch.equal(disp.call("fused_swiglu", fallback, g, u), g * u)          # default: torch
    backend_env("cuda")
    assert torch.equal(disp.call("fused_swiglu", fallback, g, u), g * u + 1)
    backend_env("best")
    assert torch.equal(disp.call("fused_swiglu", fallback, g, u), g * u + 1)      # one backend
    backend_env("torch")
    assert torch.equal(disp.call("fused_swiglu", fallback, g, u), g * u)
    backend_env("cuda")
    with pytest.raises(RuntimeError, match="No available cuda kernel found for fused_norm_rope"):
        disp.call("fused_norm_rope", fallback, g, u)
    backend_env("cutedl")
    assert disp.selected_backend() == "cutedsl"
    with pytest.raises(RuntimeError, match="No available cutedsl kernel"):
        disp.call("fused_swiglu", fallback, g, u)
    assert disp.backend_status("cuda") == "native" and disp.backend_status("triton") == "missing"
    assert KernelDispatcher(None).backend_status("cuda") == "missing"


def test_unavailable_backend_modules_are_skipped(tmp_path, backend_env):
    root = _fake_kernel_dir(tmp_path, """
        BACKEND_AVAILABLE = False
        def fused_swiglu(gate, up, *, fallback):
            return gate
    """)
    backend_env("cuda")
    disp = KernelDispatcher(root)
    assert disp.backend_status("cuda") == "missing"
    with pytest.raises(RuntimeError):
        disp.call("fused_swiglu", lambda g, u: g, torch.ones(1), torch.ones(1))


class TinySwiGLU(nn.Module):
    def __init__(self, real_formulation: bool):
        super().__init__()
        self.w1, self.w3, self.w2 = nn.Linear(8, 16, bias=False), nn.Linear(8, 16, bias=False), \
            nn.Linear(16, 8, bias=False)
        self.real = real_formulation

    def forward(self, x):
        gate, up = self.w1(x), self.w3(x)
        if self.real:
            h = (F.silu(gate.float()) * up.float()).type_as(gate)
        else:
            h = F.silu(gate) * up
        return self.w2(h)


@pytest.mark.parametrize("real_formulation", [False, True])
def test_fx_rewrite_replaces_silu_mul_by_the_custom_op(tmp_path, backend_env, real_formulation):
    root = _fake_kernel_dir(tmp_path, """
        import torch
        BACKEND_AVAILABLE = True
        CALLS = []
        def fused_swiglu(gate, up, *, fallback):
            CALLS.append((gate.dtype, tuple(gate.shape)))
            return (torch.nn.functional.silu(gate.float()) * up.float()).type_as(gate)
    """)
    backend_env("cuda")
    disp = KernelDispatcher(root)
    spec = PartitionSpec("m", "h", "", {}, (FusedOp("fused_swiglu", "fx_pattern"),
                                             FusedOp("fused_residual_norm", "fx_pattern")))
    model = TinySwiGLU(real_formulation)
    x = torch.randn(4, 8)
    want = model(x)
    gm = torch.fx.symbolic_trace(model)
    n_before = len([n for n in gm.graph.nodes if "silu" in str(n.target)])
    gm = fx_patterns.rewrite_graph(gm, spec, disp)
    targets = [str(n.target) for n in gm.graph.nodes]
    assert n_before == 1 and not any("silu" in t for t in targets)
    assert any("racetrack_b200.fused_swiglu" in t for t in targets)
    assert not any(t == "float" for t in targets)        # the fp32 casts went with the pattern
    torch.testing.assert_close(gm(x), want)
    kernel_module = disp._load_backend_modules("cuda")[0]
    assert kernel_module.CALLS == [(torch.float32, (4, 16))]
    # torch backend: nothing is rewritten
    backend_env("torch")
    gm2 = fx_patterns.rewrite_graph(torch.fx.symbolic_trace(model), spec, disp)
    assert any("silu" in str(n.target) for n in gm2.graph.nodes)


class Gate(nn.Module):
    pass


class MoE(nn.Module):                      # recognised by class name, like rm.MoE
    def __init__(self):
        super().__init__()
        self.dim = 8

    def forward(self, x):
        return x * 2


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1, self.w3, self.w2 = nn.Linear(8, 16, bias=False), nn.Linear(8, 16, bias=False), \
            nn.Linear(16, 8, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class Holder(nn.Module):
    def __init__(self):
        super().__init__()
        self.moe, self.mlp = MoE(), MLP()

    def forward(self, x):
        return self.moe(x) + self.mlp(x)


def test_pre_trace_patches_call_kernels_with_the_reference_signatures_and_roll_back(tmp_path, backend_env):
    root = _fake_kernel_dir(tmp_path, """
        BACKEND_AVAILABLE = True
        CALLS = []
        def fused_single_token_moe(moe, x, *, fallback):
            CALLS.append(("moe", type(moe).__name__))
            return fallback(moe, x)
        def fused_mlp_gate_up_proj(x, w1_w, w1_s, w3_w, w3_s, *, scale_fmt, fallback):
            CALLS.append(("gate_up", w1_s, w3_s, scale_fmt))
            return fallback(x, w1_w, w1_s, w3_w, w3_s, scale_fmt=scale_fmt)
        def fused_swiglu(gate, up, *, fallback):
            CALLS.append(("swiglu",))
            return fallback(gate, up)
    """)
    backend_env("cuda")
    disp = KernelDispatcher(root)
    spec = PartitionSpec("m", "h", "", {}, (FusedOp("fused_single_token_moe", "pre_trace"),
                                             FusedOp("fused_mlp_gate_up_proj", "module_patch"),
                                             FusedOp("fused_full_topk_indexer", "pre_trace")))
    model = Holder()
    x = torch.randn(3, 8)
    want = model(x)
    moe_forward, mlp_forward = model.moe.forward, model.mlp.forward
    originals = pre_trace.apply_pre_trace_patches(model, spec, disp)
    assert len(originals) == 2
    torch.testing.assert_close(model(x), want)
    calls = disp._load_backend_modules("cuda")[0].CALLS
    assert calls == [("moe", "MoE"), ("gate_up", None, None, None), ("swiglu",)]
    pre_trace.rollback_patches(originals)
    assert model.moe.forward == moe_forward and model.mlp.forward == mlp_forward
    torch.testing.assert_close(model(x), want)
    # torch backend: no patcher touches the model
    backend_env("torch")
    assert pre_trace.apply_pre_trace_patches(model, spec, disp) == []


def test_compile_with_partition_on_cpu_with_a_fake_backend(tmp_path, backend_env, monkeypatch):
    part = tmp_path / "m" / "p1"
    _fake_kernel_dir(part, """
        import torch
        BACKEND_AVAILABLE = True
        CALLS = []
        def fused_swiglu(gate, up, *, fallback):
            CALLS.append(1)
            return torch.nn.functional.silu(gate) * up
    """)
    (part / "spec.py").write_text("FUSED_OPS = [{'name': 'fused_swiglu', 'kind': 'fx_pattern'}]\n")
    monkeypatch.setenv("RACETRACK_PARTITIONS_ROOT", str(tmp_path))
    spec = load_spec("m", "p1")
    model = TinySwiGLU(False)
    x = torch.randn(2, 8)
    want = model(x)
    compiled, originals = compile_backend.compile_with_partition(model, spec, backend_override="cuda")
    assert os.environ["RACETRACK_KERNEL_BACKEND"] == "cuda" and originals == []
    torch.testing.assert_close(compiled(x), want)
    compile_backend.cleanup_compile_state()
    assert callable(compile_backend.make_racetrack_backend())


def test_baseline_model_dispatches_fused_norm_rope(tmp_path, backend_env):
    from racetrack_b200.partitions.dsv3_2 import model as syn
    part = tmp_path / "part"
    _fake_kernel_dir(part, """
        BACKEND_AVAILABLE = True
        CALLS = []
        def fused_norm_rope(q_c, q_weight, kv_c, kv_weight, k_pe, positions, *, eps, rope_base, fallback):
            CALLS.append((tuple(q_c.shape), tuple(kv_c.shape), tuple(k_pe.shape), q_c.is_contiguous()))
            return fallback(q_c, q_weight, kv_c, kv_weight, k_pe, positions, eps=eps, rope_base=rope_base)
    """)
    cfg = syn.DSV3_2_CONFIG.for_benchmark(num_layers=1, vocab_size=64)
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (16,))
    base = syn.FlattenedDeepSeekModel(cfg)
    part_model = syn.FlattenedDeepSeekModel(cfg, partition_root=part)
    part_model.load_state_dict(base.state_dict())
    want = base(tokens)
    backend_env("cuda")
    got = part_model(tokens)
    torch.testing.assert_close(got, want)
    calls = part_model.dispatcher._load_backend_modules("cuda")[0].CALLS
    assert calls == [((16, 128), (16, 128), (16, 16), False)]     # column slices, not copies
    assert part_model.backend_status == {"torch": "native", "cuda": "native"}
    assert syn.build_model(num_layers=1).config.num_layers == 1


def test_fp8_module_weights_are_dequantised_with_their_block_scales():
    """A racetrack `Linear` holds float8_e4m3fn codes plus one fp32 scale per 128 x 128 block
    when its dtype is FP8 (racetrack/models/deepseek.py:361-371). The kernel wrappers that
    convert a module's weights (experts to NVFP4, indexer projections to bf16) must dequantise
    them as `weight_dequant` does (deepseek.py:689-694) instead of reading the codes as values,
    and must refuse an FP8 weight that has no scales."""
    import pytest
    from oracle import ref_ops as R
    from racetrack_b200 import ops
    g = torch.Generator().manual_seed(9)
    full = torch.randn(200, 384, generator=g) * 0.05
    scale = torch.rand(2, 3, generator=g) * 0.01 + 0.001
    codes = (full / scale.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)).clamp(-448, 448) \
        .to(torch.float8_e4m3fn)

    class Linear(torch.nn.Module):
        def __init__(self, weight, scale=None):
            super().__init__()
            self.weight = torch.nn.Parameter(weight, requires_grad=False)
            if scale is not None:
                self.weight.scale = self.scale = torch.nn.Parameter(scale, requires_grad=False)

    got = ops.module_weight_bf16(Linear(codes, scale))
    want = R.block_dequant(codes, scale)
    assert got.dtype == torch.bfloat16 and torch.equal(got, want.to(torch.bfloat16))
    assert float((got.float() - full).abs().max()) <= 0.07 * float(full.abs().max())
    plain = ops.module_weight_bf16(Linear(full))
    assert torch.equal(plain, full.to(torch.bfloat16))
    with pytest.raises(RuntimeError):
        ops.module_weight_bf16(Linear(codes))
