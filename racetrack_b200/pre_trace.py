"""Pre-trace patchers: swap or tag module forwards before Dynamo traces the model.

Mirror of racetrack/pre_trace.py:22-393: same registry decorator, ``apply_pre_trace_patches`` /
``rollback_patches`` pair, ``Originals`` bookkeeping ``(module, attribute, existed, original)`` and
patcher names (the FUSED_OPS of kind ``pre_trace`` / ``module_patch``). The reference recognises
modules with ``isinstance`` checks against racetrack/models/deepseek.py; this mirror recognises the
same modules by class name (``MoE``, ``MLP``, ``Indexer``, ``MLA``, ``RMSNorm``), so it patches the
reference's real model when both are installed and any model that follows its module interface.

Forward-replacing patchers hand the kernel the same arguments as the reference does:
  fused_full_topk_indexer(indexer, x, qr, start_pos, freqs_cis, mask, *, fallback)   (:132-143)
  fused_single_token_moe(moe, x, *, fallback)                                       (:182-187)
  fused_mlp_gate_up_proj(x, w1_w, w1_s, w3_w, w3_s, *, scale_fmt, fallback)         (:216-220)
"""
from __future__ import annotations

from typing import Any, Callable

import torch
import torch.nn as nn

from .dispatch import KernelDispatcher
from .partition_spec import PartitionSpec

_REGISTRY: dict[str, Callable] = {}
Originals = list[tuple[nn.Module, str, bool, Any]]


def register_patcher(name: str):
    def decorator(fn: Callable) -> Callable:
        _REGISTRY[name] = fn
        return fn
    return decorator


def apply_pre_trace_patches(model: nn.Module, spec: PartitionSpec,
                            dispatcher: KernelDispatcher) -> Originals:
    originals: Originals = []
    for op in spec.pre_trace_ops + spec.module_patch_ops:
        patcher = _REGISTRY.get(op.name)
        if patcher is not None:
            patcher(model, dispatcher, originals)
    return originals


def rollback_patches(originals: Originals) -> None:
    for module, name, existed, original in reversed(originals):
        if existed:
            setattr(module, name, original)
        else:
            delattr(module, name)


def _set_attr(module: nn.Module, name: str, value: Any, originals: Originals) -> None:
    originals.append((module, name, hasattr(module, name), getattr(module, name, None)))
    setattr(module, name, value)


def _resolve_kernel(dispatcher: KernelDispatcher, op_name: str):
    backend = dispatcher.selected_backend(default="torch")
    if backend in ("torch", "all"):
        return None
    if backend == "best":
        backend = "cuda"
    fn = dispatcher._resolve(backend, op_name)
    # host code around a C-ABI call (raw pointers, the current stream's handle): opaque to Dynamo,
    # which breaks the graph at the call and runs it as in eager mode
    return torch.compiler.disable(fn) if fn is not None else None


def _modules_named(model: nn.Module, *class_names: str):
    for module in model.modules():
        if type(module).__name__ in class_names:
            yield module


# ---------------------------------------------------------------------------
# forward replacements
# ---------------------------------------------------------------------------

def _write_indexer_k_cache(indexer, x, start_pos, freqs_cis) -> None:
    """Fills the indexer's key cache for positions the full-top-k short-circuit answers without
    running the indexer (racetrack/pre_trace.py:82-112): once the context outgrows index_topk
    the indexer scores the WHOLE prefix [0, end_pos) from this cache. Modules without a key
    cache (light stubs) have nothing to fill. The keys come from this backend's own kernels
    (projection GEMM + the fused LayerNorm / RoPE / Hadamard / FP8 pass)."""
    if not hasattr(indexer, "k_cache"):
        return
    from . import indexer as rt_indexer
    rt_indexer.write_k_cache(x, rt_indexer.weights_of_module(indexer), indexer.k_cache,
                             indexer.k_scale_cache, start_pos, freqs_cis)


@register_patcher("fused_full_topk_indexer")
def _patch_full_topk_indexer(model: nn.Module, dispatcher: KernelDispatcher,
                             originals: Originals) -> None:
    """When every cached position fits into index_topk the indexer's answer is arange(end_pos)
    (racetrack/pre_trace.py:114-158); longer contexts go to the kernel, or to the original
    forward when the backend has none."""
    kernel_fn = _resolve_kernel(dispatcher, "fused_full_topk_indexer")
    for module in _modules_named(model, "Indexer"):
        original = module.forward
        top_k = module.index_topk

        def make(orig, indexer, limit):
            def forward(x, qr, start_pos, freqs_cis, mask):
                bsz, seqlen, _ = x.size()
                end_pos = start_pos + seqlen
                if end_pos <= limit:
                    _write_indexer_k_cache(indexer, x, start_pos, freqs_cis)
                    return torch.arange(end_pos, device=x.device, dtype=torch.long) \
                        .view(1, 1, end_pos).expand(bsz, seqlen, end_pos)
                if kernel_fn is None:
                    return orig(x, qr, start_pos, freqs_cis, mask)

                def fallback(_indexer, hidden, q_residual, pos, freqs, attn_mask):
                    return orig(hidden, q_residual, pos, freqs, attn_mask)
                return kernel_fn(indexer, x, qr, start_pos, freqs_cis, mask, fallback=fallback)
            return forward
        _set_attr(module, "forward", make(original, module, top_k), originals)


@register_patcher("fused_single_token_moe")
def _patch_single_token_moe(model: nn.Module, dispatcher: KernelDispatcher,
                            originals: Originals) -> None:
    kernel_fn = _resolve_kernel(dispatcher, "fused_single_token_moe")
    if kernel_fn is None:
        return
    for module in _modules_named(model, "MoE"):
        original = module.forward

        def make(orig, moe_mod):
            def forward(x):
                def fallback(_moe, hidden):
                    return orig(hidden)
                return kernel_fn(moe_mod, x, fallback=fallback)
            return forward
        _set_attr(module, "forward", make(original, module), originals)


@register_patcher("fused_mlp_gate_up_proj")
def _patch_mlp_gate_up_proj(model: nn.Module, dispatcher: KernelDispatcher,
                            originals: Originals) -> None:
    gate_up_fn = _resolve_kernel(dispatcher, "fused_mlp_gate_up_proj")
    swiglu_fn = _resolve_kernel(dispatcher, "fused_swiglu")
    if gate_up_fn is None:
        return
    for module in _modules_named(model, "MLP"):
        def make(mlp):
            def forward(x):
                def gate_up_fallback(hidden, w1_w, w1_s, w3_w, w3_s, *, scale_fmt):
                    del w1_s, w3_s, scale_fmt
                    return (torch.nn.functional.linear(hidden, w1_w),
                            torch.nn.functional.linear(hidden, w3_w))

                def swiglu_fallback(g, u):
                    return (torch.nn.functional.silu(g.float()) * u.float()).type_as(g)
                gate, up = gate_up_fn(x, mlp.w1.weight, getattr(mlp.w1, "scale", None),
                                      mlp.w3.weight, getattr(mlp.w3, "scale", None),
                                      scale_fmt=getattr(mlp.w1, "scale_fmt", None),
                                      fallback=gate_up_fallback)
                if swiglu_fn is not None:
                    hidden = swiglu_fn(gate, up, fallback=swiglu_fallback)
                else:
                    hidden = swiglu_fallback(gate, up)
                return mlp.w2(hidden.type_as(x))
            return forward
        _set_attr(module, "forward", make(module), originals)


# ---------------------------------------------------------------------------
# attribute patchers: hand the module a dispatcher; its own forward calls the ops
# (racetrack/models/deepseek.py:183-196 `_kernel_call`)
# ---------------------------------------------------------------------------

def _attach_dispatcher(op_name: str, *class_names: str):
    def patcher(model: nn.Module, dispatcher: KernelDispatcher, originals: Originals) -> None:
        if _resolve_kernel(dispatcher, op_name) is None:
            return
        for module in _modules_named(model, *class_names):
            _set_attr(module, "kernel_dispatcher", dispatcher, originals)
            _set_attr(module, "kernel_stats", None, originals)
    return patcher


for _op, _classes in {
    "fused_attn_norm_qkv": ("RMSNorm", "MLA"),
    "fused_qkv_proj_rope": ("MLA",),
    "fused_ar_rms_qkv_proj": ("RMSNorm", "MLA"),
    "fused_indexer_k_path": ("Indexer",),
    "fused_q_indexer_score": ("MLA",),
    "fused_q_rope_quant": ("MLA",),
    "fused_prefill_qkv_b_rope_cache": ("MLA",),
    # ops the model reaches through `_kernel_call` once a dispatcher is attached
    "fused_residual_norm_attach": ("RMSNorm",),
    "fused_swiglu_attach": ("MLP", "Expert"),
}.items():
    register_patcher(_op)(_attach_dispatcher(_op.replace("_attach", ""), *_classes))


# The reference declares these four prefill patchers and leaves them empty
# (racetrack/pre_trace.py:360-393); they are kept so the same specs load.
for _op in ("fused_attn_norm_qkv_prefill", "fused_norms_rope_cache_prefill",
            "fused_q_prefill_proj", "fused_q_rope_prefill"):
    register_patcher(_op)(lambda model, dispatcher, originals: None)
