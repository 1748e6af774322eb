"""Comparison helpers shared by the CPU and GPU tests."""
from __future__ import annotations

import hashlib

import torch


def sha(t: torch.Tensor) -> str:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float8_e4m3fn):
        raw = t.view(torch.uint8 if t.element_size() == 1 else torch.int16)
    else:
        raw = t
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


def bits(t: torch.Tensor) -> torch.Tensor:
    """Integer view of a tensor's bit patterns (for exact comparisons of fp8/bf16)."""
    t = t.detach().cpu().contiguous()
    if t.element_size() == 1:
        return t.view(torch.uint8)
    if t.element_size() == 2:
        return t.view(torch.int16)
    if t.element_size() == 4:
        return t.view(torch.int32)
    return t.view(torch.int64)


def mismatch_fraction(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((bits(a) != bits(b)).float().mean())


def assert_bit_exact(a: torch.Tensor, b: torch.Tensor, what: str = "") -> None:
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    bad = int((bits(a) != bits(b)).sum())
    assert bad == 0, f"{what}: {bad} of {a.numel()} elements differ bitwise"


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| / max |b| in fp32."""
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def assert_close_bf16(a: torch.Tensor, b: torch.Tensor, what: str = "", ulps: int = 1,
                      max_frac: float = 1.0) -> None:
    """Element-wise agreement to `ulps` bf16 units in the last place (relative 2^-8 each),
    and at most `max_frac` of the elements differing at all."""
    af, bf = a.detach().float().cpu(), b.detach().float().cpu()
    tol = ulps * (2.0 ** -7) * bf.abs().clamp_min(1e-30) + 1e-30
    bad = ((af - bf).abs() > tol)
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} elements off by more than {ulps} bf16 ulp; "
        f"worst |a-b|={float((af - bf).abs().max()):.4g}")
    frac = mismatch_fraction(a.to(torch.bfloat16), b.to(torch.bfloat16))
    assert frac <= max_frac, f"{what}: {frac:.2e} of the elements differ (limit {max_frac:.1e})"
