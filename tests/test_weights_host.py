"""Host side of the checkpoint conversion (racetrack_b200/weights.py): tensor lookup under the
Hugging Face and the reference model's names, and the FP8 block dequantisation, on CPU."""
from __future__ import annotations

import pytest
import torch

from oracle import ref_ops as R
from racetrack_b200 import weights


def _state(prefix, names, suffix):
    g = torch.Generator().manual_seed(1)
    state = {}
    for e in (0, 1, 5):
        for name, shape in zip(names, ((256, 384), (256, 384), (384, 256))):
            codes, scale = R.quantize_weight_fp8(torch.randn(shape, generator=g) * 0.02)
            state[f"{prefix}{e}.{name}.weight"] = codes
            state[f"{prefix}{e}.{name}.{suffix}"] = scale
    state["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(4, 4)
    return state


@pytest.mark.parametrize("prefix,names,suffix", [
    ("model.layers.2.mlp.experts.", ("gate_proj", "up_proj", "down_proj"), "weight_scale_inv"),
    ("layers.2.ffn.experts.", ("w1", "w3", "w2"), "scale"),
])
def test_expert_lookup_and_dequantisation(prefix, names, suffix):
    state = _state(prefix, names, suffix)
    assert weights.expert_ids(state, 2) == [0, 1, 5] and weights.expert_ids(state, 3) == []
    t = weights.find_expert_tensors(state, 2, 5)
    assert set(t) == {"gate", "up", "down"}
    for proj, name in zip(("gate", "up", "down"), names):
        w, s = t[proj]
        assert w is state[f"{prefix}5.{name}.weight"] and s is state[f"{prefix}5.{name}.{suffix}"]
        assert torch.equal(weights.to_bf16(w, s), R.block_dequant(w, s))
    with pytest.raises(KeyError):
        weights.find_expert_tensors(state, 2, 3)
    with pytest.raises(RuntimeError):
        weights.to_bf16(t["gate"][0], None)
    plain = torch.randn(8, 8)
    assert torch.equal(weights.to_bf16(plain, None), plain.to(torch.bfloat16))
