"""racetrack's OWN modules on this backend.

Where an install of the reference exists under baseline/_ref (git-ignored; made in the build
container with `pip install --no-deps --target baseline/_ref <reference checkout>`), its real
RMSNorm / MLP / Expert / MoE modules (racetrack/models/deepseek.py) are patched by its own
`apply_pre_trace_patches` (racetrack/pre_trace.py:34-47), through its own `patch_real_model`
(benchmarks/gsm8k/real_kernels.py:147-216), and dispatched by its own `KernelDispatcher`
(racetrack/runtime/dispatch.py) with RACETRACK_KERNEL_BACKEND=cuda and the kernel root pointed
at this repository's partition. The partition's spec.py is parsed by the reference's own loader.
This is the reference's contract test tests/test_gsm8k_real_kernels.py:36-99 with real kernels
in place of its pass-through stubs. Skipped where baseline/_ref is absent."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

from helpers import rel_err

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
PARTITION = ROOT / "racetrack_b200" / "partitions" / "dsv3_2" / "d9a59385"

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not (REF / "racetrack" / "pre_trace.py").is_file(),
                                 reason="no install of the reference under baseline/_ref")]


@pytest.fixture(scope="module")
def ref():
    """The reference's modules, imported from baseline/_ref for this test module only."""
    added = str(REF)
    sys.path.insert(0, added)
    try:
        import racetrack.models.deepseek as rm
        from racetrack import partition_spec as ps
        from benchmarks.gsm8k.real_kernels import RealKernelRow, patch_real_model
        spec = ps._spec_from_module(ps._load_module(PARTITION / "spec.py"), "dsv3_2", PARTITION.name)

        def row(ops):
            return RealKernelRow(partition_model="dsv3_2", partition=PARTITION.name, backend="cuda",
                                 kernel_root=PARTITION / "kernels", ops=tuple(ops), spec=spec)
        yield type("Ref", (), {"rm": rm, "spec": spec, "row": staticmethod(row),
                               "patch_real_model": staticmethod(patch_real_model)})
    finally:
        sys.path.remove(added)
        for name in list(sys.modules):
            if name.split(".")[0] in ("racetrack", "benchmarks", "partitions"):
                del sys.modules[name]


def _init(module: torch.nn.Module, seed: int) -> torch.nn.Module:
    g = torch.Generator(device="cuda").manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            p.normal_(mean=0.0, std=0.02, generator=g)
    return module.eval()


def test_reference_loader_and_dispatcher_accept_the_partition(ref):
    names = {op.name for op in ref.spec.fused_ops}
    assert {"fused_residual_norm", "fused_swiglu", "fused_single_token_moe", "fused_mlp_gate_up_proj"} <= names
    sys.path.insert(0, str(REF))
    try:
        from racetrack.runtime.dispatch import KernelDispatcher
    finally:
        sys.path.remove(str(REF))
    d = KernelDispatcher(PARTITION / "kernels")
    assert d.backend_status("cuda") == "native"
    for name in names:
        assert callable(d._resolve("cuda", name)), name
    with pytest.raises(RuntimeError, match="No available cuda kernel found for fused_nothing"):
        d.call("fused_nothing", lambda: None, backend="cuda")


def test_reference_rmsnorm_and_mlp_run_on_the_cuda_kernels(ref):
    rm = ref.rm

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = rm.RMSNorm(1024)
            self.mlp = rm.MLP(1024, 2048)

        def forward(self, x, residual):
            x, residual = self.norm(x, residual)
            return self.mlp(x), residual

    with torch.device("cuda"):
        model = _init(Tiny(), 3)
    with torch.no_grad():
        model.norm.weight.copy_(1 + 0.02 * torch.randn(1024, device="cuda"))
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(2, 37, 1024, device="cuda", generator=g).bfloat16()
    residual = torch.randn(2, 37, 1024, device="cuda", generator=g).bfloat16()
    with torch.no_grad():
        expected = model(x, residual)
        with ref.patch_real_model(model, ref.row(op.name for op in ref.spec.fused_ops)) as stats:
            actual = model(x, residual)
            assert hasattr(model.norm, "kernel_dispatcher") and hasattr(model.mlp, "kernel_dispatcher")
    assert stats.calls["fused_residual_norm"] == 1
    assert stats.used_partition_kernel
    # the residual stream is bit-exact; the MLP output differs by the summation order of two bf16 GEMMs
    assert torch.equal(actual[1], expected[1])
    assert rel_err(actual[0], expected[0]) <= 2e-2
    # rollback left the modules as they were
    assert not hasattr(model.norm, "kernel_dispatcher") and not hasattr(model.mlp, "kernel_dispatcher")
    with torch.no_grad():
        again = model(x, residual)
    assert torch.equal(again[0], expected[0]) and torch.equal(again[1], expected[1])


def test_reference_moe_runs_on_the_nvfp4_expert_path(ref):
    rm = ref.rm
    args = rm.ModelArgs(dim=1024, moe_inter_dim=512, n_routed_experts=16, n_shared_experts=1,
                        n_activated_experts=4, n_expert_groups=4, n_limited_groups=2,
                        score_func="sigmoid", route_scale=2.5)
    with torch.device("cuda"):
        moe = _init(rm.MoE(args), 5)
    g = torch.Generator(device="cuda").manual_seed(6)
    with torch.no_grad():
        # logits of about +-1.6: the routing spreads over the experts and no sigmoid saturates
        # (scores that round to 1.0 would tie, and tie order is not part of the contract)
        moe.gate.weight.normal_(mean=0.0, std=0.05, generator=g)
    x = torch.randn(3, 50, 1024, device="cuda", generator=g).bfloat16()
    with torch.no_grad():
        expected = moe(x)
        with ref.patch_real_model(moe, ref.row(op.name for op in ref.spec.fused_ops)) as stats:
            actual = moe(x)
        routing = moe.gate(x.view(-1, 1024))
        shared = moe.shared_experts(x.view(-1, 1024))
    assert stats.used_partition_kernel
    assert actual.shape == expected.shape and actual.dtype == expected.dtype
    assert bool(torch.isfinite(actual.float()).all())
    # The experts run in NVFP4 (e2m1 weights and activations): against the reference's bf16 experts
    # the routed part carries the format's noise (loose bound); against the CPU restatement of the
    # SAME arithmetic, fed the reference Gate's own routing and the module's own weights, it is tight.
    assert rel_err(actual, expected) <= 0.5
    from oracle import ref_ops as R
    w13 = torch.stack([torch.cat((e.w1.weight, e.w3.weight)) for e in moe.experts]).cpu()
    w2 = torch.stack([e.w2.weight for e in moe.experts]).cpu()
    want = R.moe_experts_nvfp4(x.view(-1, 1024).cpu(), routing[0].float().cpu(), routing[1].cpu(), w13, w2,
                               shared_out=shared.cpu())
    assert rel_err(actual.view(-1, 1024), want) <= 3e-2
    with torch.no_grad():
        assert torch.equal(moe(x), expected), "rollback restores the reference forward"
