"""Expert weights from a block-scaled FP8 checkpoint to the NVFP4 layout of the grouped GEMM.

DeepSeek-V3.2 checkpoints store every expert projection as float8_e4m3fn codes with one fp32
scale per 128 x 128 block (racetrack/models/deepseek.py:361-371 `Linear.weight` / `.scale`;
Hugging Face names `...weight` / `...weight_scale_inv`, partitions/dsv3_2/weight_mapper.py:36-66).
The expert GEMMs of this backend read NVFP4: e2m1 codes, one e4m3 scale per 16 elements stored
in the 128-row x 4-block tiles the tensor core's scale columns take unchanged, and one fp32
global scale per expert matrix. This module is the offline step between the two:

    FP8 codes * block scale  ->  bf16 (the reference's weight_dequant, deepseek.py:689-694)
    [gate; up] stacked to w13, down = w2
    NVFP4 quantisation with tiled scales (the same kernel that quantises activations)

Nothing here runs on the hot path; a model is converted once.
"""
from __future__ import annotations

import re
from typing import Iterable, Mapping, Optional

import torch

from . import moe, ops

# projection -> (checkpoint names, scale suffixes); first match wins
_NAMES = {
    "gate": ("gate_proj", "w1"),
    "up": ("up_proj", "w3"),
    "down": ("down_proj", "w2"),
}
_SCALE_SUFFIXES = ("weight_scale_inv", "scale", "weight_scale")

DEFAULT_PREFIXES = ("model.layers.{layer}.mlp.experts.{expert}.", "layers.{layer}.ffn.experts.{expert}.")


def find_expert_tensors(state: Mapping[str, torch.Tensor], layer: int, expert: int,
                        prefixes: Iterable[str] = DEFAULT_PREFIXES) -> dict:
    """{"gate" | "up" | "down": (weight, scale or None)} of one expert, looked up under the
    Hugging Face names (`gate_proj.weight`, `gate_proj.weight_scale_inv`, ...) or the
    reference model's own (`w1.weight`, `w1.scale`, ...). Raises KeyError when a projection is
    missing."""
    for prefix in prefixes:
        base = prefix.format(layer=layer, expert=expert)
        found = {}
        for proj, names in _NAMES.items():
            for name in names:
                w = state.get(f"{base}{name}.weight")
                if w is None:
                    continue
                scale = None
                for suffix in _SCALE_SUFFIXES:
                    scale = state.get(f"{base}{name}.{suffix}")
                    if scale is not None:
                        break
                found[proj] = (w, scale)
                break
        if len(found) == 3:
            return found
    raise KeyError(f"expert {expert} of layer {layer}: gate / up / down projections not found")


def expert_ids(state: Mapping[str, torch.Tensor], layer: int) -> list[int]:
    """Expert numbers present for a layer under any known prefix."""
    ids = set()
    for prefix in DEFAULT_PREFIXES:
        head = re.escape(prefix.split("{expert}")[0].format(layer=layer))
        pat = re.compile(head + r"(\d+)\.")
        for key in state:
            m = pat.match(key)
            if m:
                ids.add(int(m.group(1)))
    return sorted(ids)


def to_bf16(weight: torch.Tensor, scale: Optional[torch.Tensor]) -> torch.Tensor:
    """One checkpoint matrix as bf16: FP8 codes are multiplied by their block scales, bf16 / fp32
    weights are cast. An FP8 matrix without scales is refused."""
    if weight.element_size() == 1:
        if scale is None:
            raise RuntimeError("an FP8 checkpoint weight needs its 128 x 128 block scales")
        return ops.dequant_weight_fp8(weight.view(torch.float8_e4m3fn), scale)
    return weight.to(torch.bfloat16)


def experts_from_checkpoint(state: Mapping[str, torch.Tensor], layer: int, experts: Iterable[int], *,
                            device, prefixes: Iterable[str] = DEFAULT_PREFIXES) -> "moe.NVFP4Experts":
    """NVFP4Experts (racetrack_b200.moe) of the given experts of one layer, in the given order
    (an expert-parallel rank passes its own slice). One expert's bf16 weights exist at a time."""
    parts13, parts2 = [], []
    hidden = inter = None
    for e in experts:
        t = find_expert_tensors(state, layer, e, prefixes)
        gate, up, down = (to_bf16(w.to(device), s.to(device) if s is not None else None)
                          for w, s in (t["gate"], t["up"], t["down"]))
        if gate.shape != up.shape or down.shape != (gate.shape[1], gate.shape[0]):
            raise RuntimeError(f"expert {e}: inconsistent projection shapes")
        inter, hidden = gate.shape
        if hidden % 256 or inter % 256:
            raise RuntimeError("hidden and intermediate widths must be multiples of 256")
        parts13.append(ops.fused_nvfp4_quant(torch.cat((gate, up)), tiled_scales=True))
        parts2.append(ops.fused_nvfp4_quant(down.contiguous(), tiled_scales=True))
    if not parts13:
        raise RuntimeError("no experts given")
    cat = torch.cat
    return moe.NVFP4Experts(
        len(parts13), hidden, inter,
        cat([p[0] for p in parts13]), cat([p[1].view(torch.uint8) for p in parts13]),
        cat([p[2] for p in parts13]),
        cat([p[0] for p in parts2]), cat([p[1].view(torch.uint8) for p in parts2]),
        cat([p[2] for p in parts2]))
