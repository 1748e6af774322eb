"""The C-ABI library loads and exports every symbol include/rt_b200.h declares (no compute
calls: this runs without a GPU)."""
from __future__ import annotations

import ctypes

import pytest

import __graft_entry__ as entry
from racetrack_b200 import _lib, build as rt_build


@pytest.fixture(scope="module")
def lib():
    rt_build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = entry.declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in rt_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    for name in _lib.SIGNATURES:
        assert name in declared, f"{name} bound in _lib.py but not declared in rt_b200.h"


def test_version_and_error_reporting_without_a_gpu(lib):
    assert lib.rt_version() == 1
    assert lib.rt_launch_count() >= 0
    # argument validation happens before any CUDA call, so it works on a CPU-only host
    rc = lib.rt_residual_norm(None, None, None, 0, None, None, 1, 8, 8, 8, 1e-6, 0, None)
    assert rc == -1
    assert b"null pointer" in lib.rt_last_error()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf) // 16 * 16 + 16
    rc = lib.rt_act_quant_fp8(p, p, p, 4, 100, 104, 0, None)
    assert rc == -2 and b"multiple of 128" in lib.rt_last_error()
    rc = lib.rt_swiglu(p, p, p, 4, 16, 16, 16, 1, None)       # fp32 activations: not built
    assert rc == -2 and b"bf16" in lib.rt_last_error()
    rc = lib.rt_moe_route(p, None, p, p, 4, 96, 96, 8, 4, 8, 2.5, 0, None)
    assert rc == -2
    assert lib.rt_moe_permute_workspace_bytes(4096, 8, 256) == 32 * 256 * 4


def test_ops_refuse_cpu_tensors():
    import torch
    from racetrack_b200 import ops
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.fused_act_quant(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.fused_swiglu(x, x)
