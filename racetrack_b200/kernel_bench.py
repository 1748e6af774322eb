"""Per-kernel micro-benchmark: CUDA-event time, achieved GB/s and fraction of the HBM peak.

    python -m racetrack_b200.kernel_bench [--tokens 4096] [--kernel NAME ...] [--json out.json]

Same role as racetrack's scripts/benchmark_kernel.py (shapes + byte formulas + median of
CUDA-event timings), for the sm_100a kernels of this package. Bytes are ALGORITHMIC bytes:
every input element read once, every output element written once. L2 (126 MB) is flushed
between timed iterations by reading a 512 MB buffer, so small working sets cannot hide
in cache.
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path
from typing import Callable

import torch

from . import _lib, ops

HIDDEN, Q_LORA, KV_LORA, ROPE, HEADS, INTER, EXPERTS, TOPK = 7168, 1536, 512, 64, 128, 18432, 256, 8
FALLBACK_HBM_GBS = 6650.0


def hbm_peak_gbs() -> tuple[float, str]:
    """Measured copy bandwidth of this pool's B200s when the driver recorded it, else the
    stated fallback."""
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class L2Flusher:
    """Evicts L2 by READING a buffer four times its size. (Overwriting a buffer instead
    would leave L2 full of dirty lines whose write-back lands in the next kernel's time.)"""

    def __init__(self, nbytes: int = 512 << 20):
        self.buf = torch.zeros(nbytes // 4, dtype=torch.int32, device="cuda")

    def __call__(self) -> None:
        self.buf.sum()


def time_kernel(fn: Callable[[], object], *, warmup: int = 5, iters: int = 20,
                flush: L2Flusher | None = None) -> dict:
    """Median / min per-call device time in microseconds."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    return {"median_us": statistics.median(times), "min_us": min(times)}


def _randn(*shape, dtype=torch.bfloat16):
    return torch.randn(*shape, device="cuda", dtype=torch.float32).to(dtype)


def cases(tokens: int) -> dict[str, tuple[Callable[[], object], int]]:
    """name -> (callable, algorithmic bytes per call)."""
    T = tokens
    out: dict[str, tuple[Callable[[], object], int]] = {}
    u, r = _randn(T, HIDDEN), _randn(T, HIDDEN)
    w = torch.ones(HIDDEN, device="cuda")
    out["fused_residual_norm"] = (lambda: ops.fused_residual_norm(u, r, w, eps=1e-6),
                                  4 * T * HIDDEN * 2 + HIDDEN * 4)
    out["fused_rms_norm"] = (lambda: ops.fused_rms_norm(u, w, eps=1e-6), 2 * T * HIDDEN * 2 + HIDDEN * 4)
    qkv = _randn(T, Q_LORA + KV_LORA + ROPE)
    wq, wkv = torch.ones(Q_LORA, device="cuda"), torch.ones(KV_LORA, device="cuda")
    pos = torch.arange(T, device="cuda")
    out["fused_norm_rope"] = (
        lambda: ops.fused_norm_rope(qkv[:, :Q_LORA], wq, qkv[:, Q_LORA:Q_LORA + KV_LORA], wkv,
                                    qkv[:, Q_LORA + KV_LORA:], pos, eps=1e-6, rope_base=10000.0),
        2 * T * (Q_LORA + KV_LORA + ROPE) * 2)
    q_pe = _randn(T, HEADS, ROPE)
    freqs = torch.polar(torch.ones(T, ROPE // 2, device="cuda"),
                        torch.rand(T, ROPE // 2, device="cuda"))
    out["fused_rope"] = (lambda: ops.fused_rope(q_pe, freqs), 2 * T * HEADS * ROPE * 2)
    gu = _randn(T, 2 * INTER)
    g, up = gu[:, :INTER], gu[:, INTER:]
    out["fused_swiglu"] = (lambda: ops.fused_swiglu(g, up), 3 * T * INTER * 2)
    x = _randn(T, INTER)
    q_out = T * INTER + T * (INTER // 128) * 4
    out["fused_act_quant"] = (lambda: ops.fused_act_quant(x), T * INTER * 2 + q_out)
    out["fused_swiglu_quant"] = (lambda: ops.fused_swiglu_quant(g, up), 2 * T * INTER * 2 + q_out)
    amax = ops.tensor_absmax(x)
    n_out = T * INTER // 2 + T * INTER // 16
    out["tensor_absmax"] = (lambda: ops.tensor_absmax(x), T * INTER * 2)
    out["fused_nvfp4_quant"] = (lambda: ops.fused_nvfp4_quant(x, amax=amax), T * INTER * 2 + n_out)
    amax_h = ops.tensor_absmax(g, up)
    out["fused_swiglu_nvfp4_quant"] = (lambda: ops.fused_swiglu_nvfp4_quant(g, up, amax=amax_h),
                                       2 * T * INTER * 2 + n_out)
    logits = torch.randn(T, EXPERTS, device="cuda")
    bias = torch.rand(EXPERTS, device="cuda") * 0.2 - 0.1
    out["fused_moe_route"] = (
        lambda: ops.fused_moe_route(logits, bias, n_groups=8, topk_groups=4, topk=TOPK,
                                    route_scale=2.5),
        T * EXPERTS * 4 + T * TOPK * 12)
    _, idx = ops.fused_moe_route(logits, bias, n_groups=8, topk_groups=4, topk=TOPK, route_scale=2.5)
    out["fused_moe_permute"] = (lambda: ops.fused_moe_permute(idx, EXPERTS),
                                T * TOPK * (8 + 4 + 4))
    off, sp, pp = ops.fused_moe_permute(idx, EXPERTS)
    out["fused_moe_gather"] = (lambda: ops.fused_moe_gather(u, sp, TOPK),
                               T * HIDDEN * 2 + T * TOPK * HIDDEN * 2)
    sc = torch.randn(min(T, 2048), 4096, device="cuda")
    out["index_topk[2048 of 4096]"] = (lambda: ops.index_topk(sc, 2048),
                                       sc.numel() * 4 + sc.shape[0] * 2048 * 4)
    # indexer prologue: LayerNorm + RoPE + Hadamard + FP8 quantisation of the keys (one 128-wide
    # row per token) and of the 64 index heads of every query
    table = torch.polar(torch.ones(max(T, 16), 32, device="cuda"), torch.rand(max(T, 16), 32, device="cuda"))
    xk, xq = _randn(T, 1, 128), _randn(T, 64, 128)
    lnw, lnb = torch.ones(128, device="cuda"), torch.zeros(128, device="cuda")
    out["index_prep[keys]"] = (lambda: ops.index_prep(xk, table, ln_weight=lnw, ln_bias=lnb),
                               T * (256 + 132))
    out["index_prep[queries x 64 heads]"] = (lambda: ops.index_prep(xq, table), T * 64 * (256 + 132))
    eo = _randn(T * TOPK, HIDDEN)
    wts = torch.rand(T, TOPK, device="cuda")
    out["fused_moe_combine"] = (lambda: ops.fused_moe_combine(eo, pp, wts, u),
                                T * TOPK * HIDDEN * 2 + 2 * T * HIDDEN * 2)
    # sparse MLA decode attention: min(T, 64) sequences, 2048 of 4096 cached positions each;
    # algorithmic bytes = every selected cache row once + queries + output
    B = min(T, 64)
    kv, pe = _randn(B, 4096, KV_LORA), _randn(B, 4096, ROPE)
    sel = torch.stack([torch.randperm(4096, device="cuda")[:2048].sort().values for _ in range(B)]).int()
    for heads in (16, 128):
        qa, qp = _randn(B, heads, KV_LORA) * 0.3, _randn(B, heads, ROPE) * 0.3
        out[f"mla_sparse_decode[{B} seq x {heads} heads]"] = (
            (lambda qa=qa, qp=qp: ops.mla_sparse_decode(qa, qp, kv, pe, sel, 192 ** -0.5)),
            B * 2048 * (KV_LORA + ROPE) * 2 + B * heads * (2 * KV_LORA + ROPE) * 2)
    return out


def gemm_cases(tokens: int) -> dict[str, tuple[Callable[[], object], int, int, str]]:
    """name -> (callable, flops, bytes, kind) for the tensor-core GEMMs."""
    T = tokens
    out = {}
    for name, n, k in (("qkv_a", Q_LORA + KV_LORA + ROPE, HIDDEN), ("q_b", HEADS * 192, Q_LORA),
                       ("kv_b", HEADS * 256, KV_LORA), ("w_o", HIDDEN, HEADS * 128)):
        x, w = _randn(T, k), _randn(n, k)
        for sched, tag in ((2, "pair"), (1, "single")):
            def run_bf16(x=x, w=w, sched=sched):
                ops.gemm_bf16_schedule(sched)
                try:
                    return ops.linear_bf16(x, w)
                finally:
                    ops.gemm_bf16_schedule(0)
            out[f"linear_bf16/{tag}[{name} {T}x{n}x{k}]"] = (
                run_bf16, 2 * T * n * k, (T * k + n * k + T * n) * 2, "bf16")
        wc, ws = ops.quantize_weight_fp8(w)
        xc, xs = ops.fused_act_quant(x)
        out[f"linear_fp8[{name} {T}x{n}x{k}]"] = (
            (lambda xc=xc, xs=xs, wc=wc, ws=ws: ops.linear_fp8(xc, xs, wc, ws)), 2 * T * n * k,
            T * k + n * k + T * n * 2, "fp8")
    # sparse indexer: index scores (64 heads x 128) of T queries over 4096 and T keys
    for keys in sorted({4096, max(T, 128)}):
        q = torch.randn(1, T, 64, 128, device="cuda").to(torch.float8_e4m3fn)
        kk = torch.randn(1, keys, 128, device="cuda").to(torch.float8_e4m3fn)
        wts = torch.randn(1, T, 64, device="cuda") * 0.01
        ksc = torch.rand(1, keys, device="cuda") * 0.01
        out[f"fp8_index[{T} queries x {keys} keys]"] = (
            (lambda q=q, wts=wts, kk=kk, ksc=ksc: ops.fp8_index(q, wts, kk, ksc)),
            2 * T * 64 * keys * 128, T * 64 * 128 + keys * 128 + T * keys * 4, "fp8")
    # causal attention of the prefill stack (128 nope + 64 shared rope dims, values of 128):
    # this library's kernel, and torch SDPA on whole keys as the yardstick
    for heads in (16, HEADS):
        q, kv, kpe = _randn(T, heads, 192) * 0.3, _randn(T, heads, 256) * 0.3, _randn(T, ROPE) * 0.3
        flops = 2 * heads * (T * (T + 1) // 2) * (192 + 128)
        nbytes = 2 * T * heads * (192 + 256 + 128) + 2 * T * ROPE
        out[f"attention_prefill[{T} tokens x {heads} heads]"] = (
            (lambda q=q, kv=kv, kpe=kpe: ops.attention_prefill(q, kv[..., :128], kpe, kv[..., 128:])),
            flops, nbytes, "bf16")

        def single(q=q, kv=kv, kpe=kpe):      # the single-CTA schedule whatever the length
            prev = ops.attention_prefill_schedule(1)
            try:
                return ops.attention_prefill(q, kv[..., :128], kpe, kv[..., 128:])
            finally:
                ops.attention_prefill_schedule(prev)
        out[f"attention_prefill/single[{T} tokens x {heads} heads]"] = (single, flops, nbytes, "bf16")
        k_full = torch.cat((kv[..., :128], kpe.unsqueeze(1).expand(-1, heads, -1)), dim=-1)

        def sdpa(q=q, k=k_full, v=kv[..., 128:]):
            qt, kt, vt = (t.transpose(0, 1).unsqueeze(0) for t in (q, k, v))
            return torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
        out[f"torch_sdpa_yardstick[{T} tokens x {heads} heads]"] = (sdpa, flops, nbytes, "bf16")
    for name, n, k in (("w13", 4096, HIDDEN), ("w2", HIDDEN, 2048)):
        x, w = _randn(T, k), _randn(n, k)
        xq = ops.fused_nvfp4_quant(x, tiled_scales=True)
        wq = ops.fused_nvfp4_quant(w, tiled_scales=True)
        for sched, tag in ((2, "pair"), (1, "single")):
            def run(xq=xq, wq=wq, sched=sched):
                ops.gemm_nvfp4_schedule(sched)
                try:
                    return ops.linear_nvfp4(*xq, *wq)
                finally:
                    ops.gemm_nvfp4_schedule(0)
            out[f"linear_nvfp4/{tag}[{name} {T}x{n}x{k}]"] = (
                run, 2 * T * n * k, (T * k + n * k) * 9 // 16 + T * n * 2, "nvfp4")
    return out


def run_gemms(tokens: int, iters: int, flush: "L2Flusher", only: str = "") -> list[dict]:
    peaks = {}
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        peaks = json.loads(p.read_text())
    bf16_peak = float(peaks.get("bf16_tflops", 1590.0))
    rows = []
    for name, (fn, flops, nbytes, kind) in gemm_cases(tokens).items():
        if only and only not in name:
            continue
        t = time_kernel(fn, iters=iters, flush=flush)
        tf = flops / (t["median_us"] * 1e-6) / 1e12
        # dense NVFP4 has no measured peak on this pool: quoted against the nominal 9 PFLOP/s
        # dense FP8 / NVFP4 have no measured peak on this pool: quoted against nominal 4.5 / 9 PFLOP/s
        peak = {"bf16": bf16_peak, "fp8": 4500.0}.get(kind, 9000.0)
        label = {"bf16": "measured bf16", "fp8": "nominal fp8"}.get(kind, "nominal nvfp4")
        rows.append({"kernel": name, **t, "tflops": tf, "frac_of_peak": tf / peak, "peak_tflops": peak,
                     "gbs": nbytes / (t["median_us"] * 1e-6) / 1e9})
        print(f"{name:40s} {t['median_us']:9.1f} us  {tf:8.1f} TFLOP/s  {100*tf/peak:5.1f}% of "
              f"{peak:.0f} ({label})  "
              f"{rows[-1]['gbs']:7.1f} GB/s", flush=True)
    ops.tc_error_state()
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--kernel", action="append", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--gemm", action="store_true", help="also time the tensor-core GEMMs")
    ap.add_argument("--gemm-filter", default="", help="only GEMM cases whose name contains this")
    ap.add_argument("--json", type=Path, default=None)
    args = ap.parse_args()
    peak, peak_src = hbm_peak_gbs()
    flush = L2Flusher()
    rows = []
    for name, (fn, nbytes) in cases(args.tokens).items():
        if args.kernel and name not in args.kernel:
            continue
        before = _lib.launch_count()
        fn()
        launches = _lib.launch_count() - before
        t = time_kernel(fn, iters=args.iters, flush=flush)
        gbs = nbytes / (t["median_us"] * 1e-6) / 1e9
        rows.append({"kernel": name, "tokens": args.tokens, "launches": launches,
                     "bytes": nbytes, **t, "gbs": gbs, "frac_of_hbm_peak": gbs / peak})
        print(f"{name:28s} T={args.tokens:<6d} {t['median_us']:9.1f} us  {nbytes/1e6:9.1f} MB  "
              f"{gbs:8.1f} GB/s  {100*gbs/peak:5.1f}% of {peak_src} {peak:.0f} GB/s  "
              f"({launches} launch{'es' if launches != 1 else ''})", flush=True)
    gemm_rows = []
    if args.gemm:
        gemm_rows = run_gemms(args.tokens, args.iters, flush, args.gemm_filter)
    if args.json:
        args.json.write_text(json.dumps({"hbm_peak_gbs": peak, "peak_source": peak_src,
                                         "rows": rows, "gemm_rows": gemm_rows}, indent=1) + "\n")


if __name__ == "__main__":
    main()
