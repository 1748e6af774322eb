"""Offline conversion of block-scaled FP8 expert weights (the checkpoint layout of
racetrack/models/deepseek.py:361-371) to the NVFP4 operands of the grouped GEMM
(racetrack_b200/weights.py), checked by dequantising both sides on the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_ops as R
from helpers import rel_err

pytestmark = pytest.mark.gpu


def _checkpoint(n_experts, hidden, inter, hf_names, seed=3):
    g = torch.Generator().manual_seed(seed)
    state, full = {}, {}
    names = ("gate_proj", "up_proj", "down_proj") if hf_names else ("w1", "w3", "w2")
    suffix = "weight_scale_inv" if hf_names else "scale"
    prefix = "model.layers.4.mlp.experts.{e}." if hf_names else "layers.4.ffn.experts.{e}."
    for e in range(n_experts):
        for name in names:
            shape = (hidden, inter) if name in ("down_proj", "w2") else (inter, hidden)
            w = torch.randn(shape, generator=g) * 0.02
            codes, scale = R.quantize_weight_fp8(w)
            state[prefix.format(e=e) + name + ".weight"] = codes
            state[prefix.format(e=e) + name + "." + suffix] = scale
            full[(e, name)] = R.block_dequant(codes, scale)
    return state, full, names


@pytest.mark.parametrize("hf_names", [True, False])
def test_fp8_checkpoint_experts_become_nvfp4_operands(hf_names):
    from racetrack_b200 import moe, ops, weights
    n_experts, hidden, inter = 3, 512, 256
    state, full, names = _checkpoint(n_experts, hidden, inter, hf_names)
    assert weights.expert_ids(state, 4) == [0, 1, 2]
    ex = weights.experts_from_checkpoint(state, 4, range(n_experts), device="cuda")
    assert (ex.count, ex.hidden, ex.inter) == (n_experts, hidden, inter)
    kt13, kt2 = hidden // 64, inter // 64
    for e in range(n_experts):
        w13 = torch.cat((full[(e, names[0])], full[(e, names[1])]))          # bf16, FP8-dequantised
        w2 = full[(e, names[2])]
        for w, codes, sf, gs, kt in ((w13, ex.w13_codes, ex.w13_sf, ex.w13_gs, kt13),
                                     (w2, ex.w2_codes, ex.w2_sf, ex.w2_gs, kt2)):
            rows = w.shape[0]
            rc, rsf, rgs = R.nvfp4_quant(w)
            got_codes = codes[e * rows:(e + 1) * rows].cpu()
            assert torch.equal(got_codes, rc), "NVFP4 codes differ from the oracle's"
            assert torch.equal(gs[e:e + 1].cpu(), rgs)
            tiles = (rows + 127) // 128
            seg = sf.cpu()[e * tiles * kt * 512:(e + 1) * tiles * kt * 512]
            assert torch.equal(seg[R.sf_tiled_offsets(rows, w.shape[1] // 16)], rsf.view(torch.uint8))
            # both sides dequantised: NVFP4 keeps the FP8 weights to e2m1 accuracy
            back = R.nvfp4_dequant(got_codes, rsf, rgs)
            assert rel_err(back, w.float()) <= 0.3
            rms = float((back - w.float()).pow(2).mean().sqrt() / w.float().pow(2).mean().sqrt())
            assert rms <= 0.13, f"relative RMS error {rms}"
    # the converted experts run: a small MoE against the NVFP4 oracle on the FP8-dequantised weights
    g = torch.Generator().manual_seed(9)
    x = torch.randn(40, hidden, generator=g).bfloat16()
    idx = torch.rand(40, n_experts, generator=g).topk(2, dim=-1)[1]
    wts = torch.rand(40, 2, generator=g) + 0.1
    w13_all = torch.stack([torch.cat((full[(e, names[0])], full[(e, names[1])])) for e in range(n_experts)])
    w2_all = torch.stack([full[(e, names[2])] for e in range(n_experts)])
    want = R.moe_experts_nvfp4(x, wts, idx, w13_all, w2_all)
    got = moe.fused_moe_experts(x.cuda(), wts.cuda(), idx.cuda(), ex, n_experts=n_experts)
    ops.tc_error_state()
    assert rel_err(got, want) <= 3e-2


def test_conversion_refuses_fp8_without_scales_and_missing_projections():
    from racetrack_b200 import weights
    state, _, _ = _checkpoint(1, 512, 256, True)
    broken = {k: v for k, v in state.items() if not k.endswith("gate_proj.weight_scale_inv")}
    with pytest.raises(RuntimeError):
        weights.experts_from_checkpoint(broken, 4, [0], device="cuda")
    missing = {k: v for k, v in state.items() if "down_proj" not in k}
    with pytest.raises(KeyError):
        weights.experts_from_checkpoint(missing, 4, [0], device="cuda")
