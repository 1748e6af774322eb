"""FX graph rewrites: replace fusible op sequences of a Dynamo-traced graph by calls to the
partition's kernels, wrapped as ``torch.library`` custom ops with fake implementations so
tracing never touches the ctypes layer.

Mirror of racetrack/fx_patterns.py:19-202: same registry decorator, ``rewrite_graph(gm, spec,
dispatcher)`` entry point and per-op matchers keyed by FUSED_OPS names. As in the reference only
``fused_swiglu`` rewrites nodes (:65-102); ``fused_residual_norm`` and ``fused_act_quant`` register
their custom ops (callable as ``torch.ops.racetrack_b200.<op>``) and rewrite nothing (:110-133,
:156-175); ``fused_rms_norm`` / ``fused_norm_rope`` are reached through the dispatcher from the
model code, not through the graph (:141-148, :183-188). The SwiGLU matcher additionally sees
through the fp32 casts of the real model's formulation,
``(F.silu(gate.float()) * up.float()).type_as(gate)`` (racetrack/models/deepseek.py:850-851).
"""
from __future__ import annotations

from typing import Any, Callable

import torch
from torch.fx import GraphModule, Node

from .dispatch import KernelDispatcher
from .partition_spec import PartitionSpec

NAMESPACE = "racetrack_b200"
_PATTERN_REGISTRY: dict[str, Callable] = {}
_CUSTOM_OPS: dict[str, Any] = {}
_KERNELS: dict[str, Callable] = {}     # op name -> kernel the custom op forwards to


def register_pattern(name: str):
    def decorator(fn: Callable) -> Callable:
        _PATTERN_REGISTRY[name] = fn
        return fn
    return decorator


def _get_or_create_custom_op(name: str, impl_fn, fake_fn):
    if name not in _CUSTOM_OPS:
        op = torch.library.custom_op(f"{NAMESPACE}::{name}", mutates_args=())(impl_fn)
        op.register_fake(fake_fn)
        _CUSTOM_OPS[name] = op
    return _CUSTOM_OPS[name]


def rewrite_graph(gm: GraphModule, spec: PartitionSpec, dispatcher: KernelDispatcher) -> GraphModule:
    rewrites = 0
    for op in spec.fx_ops:
        matcher = _PATTERN_REGISTRY.get(op.name)
        if matcher is not None:
            rewrites += matcher(gm.graph, dispatcher)
    if rewrites:
        gm.graph.lint()
        gm.recompile()
    return gm


def _resolve(dispatcher: KernelDispatcher, op_name: str):
    backend = dispatcher.selected_backend(default="torch")
    if backend in ("torch", "all"):
        return None
    if backend == "best":
        backend = "cuda"
    return dispatcher._resolve(backend, op_name)


# ---------------------------------------------------------------------------
# fused_swiglu: silu(gate) * up
# ---------------------------------------------------------------------------

def _is_float_cast(node: Any) -> bool:
    if not isinstance(node, Node):
        return False
    if node.op == "call_method" and node.target == "float":
        return True
    if node.op == "call_method" and node.target == "to" and torch.float32 in node.args[1:]:
        return True
    return False


def _is_mul(node: Node) -> bool:
    return node.op == "call_function" and "mul" in str(node.target) or \
        (node.op == "call_method" and node.target == "mul")


@register_pattern("fused_swiglu")
def _match_and_replace_swiglu(graph: torch.fx.Graph, dispatcher: KernelDispatcher) -> int:
    kernel_fn = _resolve(dispatcher, "fused_swiglu")
    if kernel_fn is None:
        return 0
    _KERNELS["fused_swiglu"] = kernel_fn

    def _impl(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        return _KERNELS["fused_swiglu"](gate, up, fallback=None)

    def _fake(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        return torch.empty_like(gate)

    op_callable = _get_or_create_custom_op("fused_swiglu", _impl, _fake)._opoverload
    count = 0
    for node in list(graph.nodes):
        if node.op != "call_function" or getattr(node.target, "__name__", "") != "silu":
            continue
        for user in list(node.users):
            if not _is_mul(user):
                continue
            others = [a for a in user.args if a is not node]
            if not others or not isinstance(others[0], Node):
                continue
            gate_in, up_in, out_node = node.args[0], others[0], user
            if _is_float_cast(gate_in) and _is_float_cast(up_in) and len(user.users) == 1:
                # fp32 formulation: fuse from the un-cast tensors through to the cast back
                cast_back = next(iter(user.users))
                if cast_back.op == "call_method" and cast_back.target in ("type_as", "to"):
                    gate_in, up_in, out_node = gate_in.args[0], up_in.args[0], cast_back
            with graph.inserting_before(out_node):
                fused = graph.call_function(op_callable, args=(gate_in, up_in))
            out_node.replace_all_uses_with(fused)
            graph.erase_node(out_node)
            if out_node is not user and len(user.users) == 0:
                graph.erase_node(user)
            if len(node.users) == 0:
                graph.erase_node(node)
            count += 1
    if count:
        graph.eliminate_dead_code()
    return count


# ---------------------------------------------------------------------------
# fused_residual_norm / fused_act_quant: custom ops registered, no node rewrite
# ---------------------------------------------------------------------------

@register_pattern("fused_residual_norm")
def _match_and_replace_residual_norm(graph: torch.fx.Graph, dispatcher: KernelDispatcher) -> int:
    kernel_fn = _resolve(dispatcher, "fused_residual_norm")
    if kernel_fn is None:
        return 0
    _KERNELS["fused_residual_norm"] = kernel_fn

    # canonical contract (update, residual, weight) -> (normed, hidden)
    def _impl(update: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
              eps: float) -> tuple[torch.Tensor, torch.Tensor]:
        return _KERNELS["fused_residual_norm"](update, residual, weight, eps=eps, fallback=None)

    def _fake(update: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
              eps: float) -> tuple[torch.Tensor, torch.Tensor]:
        return torch.empty_like(update), torch.empty_like(update)

    _get_or_create_custom_op("fused_residual_norm", _impl, _fake)
    return 0


@register_pattern("fused_act_quant")
def _match_and_replace_act_quant(graph: torch.fx.Graph, dispatcher: KernelDispatcher) -> int:
    kernel_fn = _resolve(dispatcher, "fused_act_quant")
    if kernel_fn is None:
        return 0
    _KERNELS["fused_act_quant"] = kernel_fn

    def _impl(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return _KERNELS["fused_act_quant"](x, fallback=None)

    def _fake(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        groups = (x.shape[-1] + 127) // 128
        return (torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device),
                torch.empty(*x.shape[:-1], groups, dtype=torch.float32, device=x.device))

    _get_or_create_custom_op("fused_act_quant", _impl, _fake)
    return 0


@register_pattern("fused_rms_norm")
def _match_and_replace_rms_norm(graph: torch.fx.Graph, dispatcher: KernelDispatcher) -> int:
    return 0


@register_pattern("fused_norm_rope")
def _match_and_replace_norm_rope(graph: torch.fx.Graph, dispatcher: KernelDispatcher) -> int:
    return 0
