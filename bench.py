"""Benchmark of the DeepSeek-V3.2 partition hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0). Default workload `dsv3_2_prefill_stack`: the realistic prefill
stack of racetrack/realistic_bench.py at T = 8192 tokens, hidden 7168, one synthetic
DeepSeek-V3.2 layer (MLA attention + 256-expert top-8 MoE, NVFP4 experts) reused for 61 layers;
a step is one forward of the whole stack. Metric: tokens * layers / second, the reference
runner's own figure (racetrack/realistic_bench.py:557). `value` has the input resident in HBM;
`e2e` moves the step's hidden states from pinned host memory and reads the result back inside
the timed region. Under torchrun (N > 1) attention heads are tensor-parallel and experts
expert-parallel with NCCL all-reduces, tokens replicated: total work is fixed (strong scaling).

`--impl reference` times racetrack's own vanilla-torch CPU path (restated in oracle/) on the
host cores, on a bounded sample (a few tokens, one layer) of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

UNIT = "tokens*layers/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1400.0     # sustained figure of the fallback measurement
CPU_SAMPLE_TOKENS = 8


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, dense bf16 TFLOP/s sustained under the power cap, source)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
    }

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz = None
        self._halt = threading.Event()
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def run(self):
        if self._nvml is None:
            return
        nv = self._nvml
        while not self._halt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self) -> dict:
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# workload: realistic prefill stack (default)
# ---------------------------------------------------------------------------

CHECK_ATOL, CHECK_RTOL = 0.5, 0.1     # racetrack/realistic_bench.py:538,645-646


def _criterion(out: torch.Tensor, ref: torch.Tensor, ref_bf16=None, **what) -> dict:
    """The reference runner's pass criterion for a configuration: max |out - ref| against
    atol + rtol * max |ref| (racetrack/realistic_bench.py:530-538). `ref` is the CPU
    restatement of the reference's torch path in the timed configuration's own arithmetic;
    `ref_bf16`, when given, the same layers with every weight and activation left in bf16."""
    def dist(r):
        diff = float((out.float().cpu() - r.float()).abs().max())
        scale = float(r.float().abs().max())
        return {"diff": diff, "rel": diff / max(scale, 1e-30), "max_abs_ref": scale,
                "ok": bool(diff <= CHECK_ATOL + CHECK_RTOL * scale)}
    res = dist(ref)
    res.update({"criterion": f"diff <= {CHECK_ATOL} + {CHECK_RTOL} * max|ref|",
                "against": "CPU restatement of the reference's torch path in the timed "
                           "configuration's arithmetic (both operands of a quantised linear "
                           "quantised, dequantised values multiplied), same weights", **what})
    if ref_bf16 is not None:
        res["vs_unquantised_bf16"] = dist(ref_bf16)
        own = float((ref.float() - ref_bf16.float()).abs().max()) / max(float(ref_bf16.float().abs().max()), 1e-30)
        res["vs_unquantised_bf16"]["oracle_own_rel"] = own
    return res


def layer_check(model, shape, sample, positions, n_layers, *, proj, ffn="moe", rank=0) -> dict | None:
    """Runs `model` (a racetrack_b200.layer.RealisticLayer; every rank of its group must call
    this) on `sample` [t, hidden] for `n_layers` layers and compares it, on rank 0, with the CPU
    restatement of the reference layer built from the same weights.

    The oracle evaluates the layer in the model's own arithmetic: the reference's torch path of
    a quantised linear quantises both operands and multiplies the dequantised values
    (racetrack/models/deepseek.py:113-121,343-345), which the oracle does for FP8 projections
    and NVFP4 experts. Two comparisons, both under the reference runner's criterion
    diff <= 0.5 + 0.1 * max|ref| (racetrack/realistic_bench.py:530-538):

    * "stages": every layer's attention half and feed-forward half, the oracle fed the very
      tensor the product fed its kernels. `ok` is the conjunction of these.
    * "end_to_end": the free-running stacks, against the same-arithmetic oracle and against the
      un-quantised bf16 layer. With NVFP4 experts this one cannot hold beyond a layer or so
      for ANY implementation of the format on white-noise weights: e2m1 keeps one mantissa
      bit, so a last-bit difference in a quantiser's input flips codes by whole quantisation
      steps; it is reported, not asserted ("oracle_own_rel" is how far the oracle's own
      quantised evaluation sits from the bf16 layer)."""
    from oracle import ref_layer, ref_ops as R
    from racetrack_b200 import layer, ops
    s, dev = shape, sample.device
    dense = ffn == "dense"
    hidden = sample
    normed = ops.fused_rms_norm(hidden, model.ones_h, eps=s.eps)
    taps = []
    for _ in range(n_layers):
        attn = model.attention(normed, positions)
        normed2, hidden = ops.fused_residual_norm(attn, hidden, model.ones_h, eps=s.eps)
        out_ffn = model.ffn_forward(normed2)
        taps.append((normed, attn, normed2, out_ffn))
        normed, hidden = ops.fused_residual_norm(out_ffn, hidden, model.ones_h, eps=s.eps)
    # on several ranks the timed forward runs the token-sharded schedule (reduce-scatter, token-wise
    # kernels on the rank's rows, all-gather of their compact outputs); the stages above ran the
    # replicated one (all-reduce): same sums, so ONE layer of each must agree closely
    sharded_vs_replicated = None
    if getattr(model, "world", 1) > 1:
        one = model.forward_stack(sample, positions, 1)
        n_a, h_a = taps[0][2], None
        _, h_mid = ops.fused_residual_norm(taps[0][1], sample, model.ones_h, eps=s.eps)
        _, h_a = ops.fused_residual_norm(taps[0][3], h_mid, model.ones_h, eps=s.eps)
        d = float((one.float() - h_a.float()).abs().max())
        sc = float(h_a.float().abs().max())
        sharded_vs_replicated = {"layers": 1, "diff": round(d, 5), "rel": round(d / max(sc, 1e-30), 5),
                                 "ok": bool(d <= CHECK_ATOL + CHECK_RTOL * sc)}
    ops.tc_error_state()
    if rank != 0:
        return None
    full = layer.make_weights(s, 0, 1, dev, ffn="dense" if dense else "none", std=0.02)
    w = {k: v.cpu() for k, v in full.items()}
    del full
    linear = ref_layer.make_linear(proj)
    pos = positions.cpu()
    bank = None
    if not dense:
        bank = ref_layer.ExpertBank(s, w, lambda e: layer.draw_expert(s, e, dev, std=0.02),
                                    quantise=lambda x: ops.fused_nvfp4_quant(x))

    def dist(got, ref):
        diff = float((got.float().cpu() - ref.float()).abs().max())
        scale = float(ref.float().abs().max())
        return {"diff": round(diff, 5), "rel": round(diff / max(scale, 1e-30), 5),
                "max_abs_ref": round(scale, 5), "ok": bool(diff <= CHECK_ATOL + CHECK_RTOL * scale)}

    stages = []
    for i, (n1, attn, n2, out_ffn) in enumerate(taps):
        ref_attn = ref_layer.attention(n1.cpu(), pos, w, s, s.heads, linear)
        stages.append({"layer": i, "stage": "attention", **dist(attn, ref_attn)})
        x = n2.cpu()
        if dense:
            ref_ffn = ref_layer.dense_ffn(x, w) if proj == "bf16" else ref_layer.dense_ffn_fp8(x, w, linear)
        else:
            bank.route(x)
            ref_ffn = ref_layer.moe_nvfp4(x, w, s, 0, s.n_experts)
        stages.append({"layer": i, "stage": "ffn", **dist(out_ffn, ref_ffn)})
    h = sample.cpu()
    kw = dict(ffn="dense") if dense else dict(before_moe=bank.route)
    ref = ref_layer.forward_stack(h, pos, [w], s, n_layers, proj=proj,
                                  **(kw if dense else dict(experts="nvfp4", **kw)))
    ref16 = ref_layer.forward_stack(h, pos, [w], s, n_layers, **kw)
    e2e = {"vs_same_arithmetic_oracle": dist(hidden, ref), "vs_unquantised_bf16": dist(hidden, ref16)}
    e2e["vs_unquantised_bf16"]["oracle_own_rel"] = round(
        float((ref.float() - ref16.float()).abs().max()) / max(float(ref16.float().abs().max()), 1e-30), 5)
    if sharded_vs_replicated is not None:
        e2e["token_sharded_vs_replicated_schedule"] = sharded_vs_replicated
        stages.append({"layer": 0, "stage": "token-sharded schedule vs replicated schedule",
                       **{k: sharded_vs_replicated[k] for k in ("diff", "rel", "ok")},
                       "max_abs_ref": None})
    return {"ok": all(st["ok"] for st in stages), "tokens": int(sample.shape[0]), "layers": n_layers,
            "criterion": f"diff <= {CHECK_ATOL} + {CHECK_RTOL} * max|ref|",
            "mode": "every layer's attention half and feed-forward half against the CPU restatement of "
                    "the reference's torch path in the same arithmetic, fed the product's own input",
            "worst_stage_rel": max(st["rel"] for st in stages), "stages": stages, "end_to_end": e2e}


class PrefillStackWorkload:
    """T tokens through `layers` applications of one synthetic DeepSeek-V3.2 layer."""
    name = "dsv3_2_prefill_stack"
    metric = "dsv3_2_layer_tokens_per_s"
    scaling = "strong"
    dominant = "gemm_nvfp4_kernel[experts w13]"
    ffn = "moe"          # "dense": the first-three-layers variant (SwiGLU FFN of width 18432)
    default_tokens = 8192
    # The stack is replayed from a CUDA graph (racetrack/bench.py:98-111 captures its sweeps the
    # same way): 61 layers x ~140 launches per step leave one Python thread per rank behind the
    # GPU once the per-rank work shrinks (4 ranks: 176 ms eager, 165 ms replayed). --no-graph
    # runs it eagerly.
    graph_default = True

    def __init__(self, device, rank: int, world: int, args):
        from racetrack_b200 import layer, moe, ops
        self.layer_mod, self.moe, self.ops = layer, moe, ops
        self.device, self.rank, self.world = device, rank, world
        layer.ATTENTION_CORE = args.attn_core
        ops.attention_prefill_schedule({"auto": 0, "single": 1, "pair": 2}[getattr(args, "attn_schedule", "auto")])
        self.tokens, self.layers = args.tokens, args.layers
        if self.default_tokens != 8192 and args.tokens == 8192:
            self.tokens = self.default_tokens         # --tokens was not given
        self.shape = layer.DSV32
        self.ffn = args.ffn
        # Experts: expert-parallel up to 4 groups; from 8 ranks on, pairs of ranks share a group's
        # experts and split their intermediate dimension. Under this runner's router (random gate,
        # one layer applied 61 times) a few experts attract most rows: the busiest of 8 single-rank
        # blocks receives 2.2 x the mean rows, the busiest of 4 groups 1.35 x.
        tp = getattr(args, "moe_tp", "auto")
        self.moe_tp = (2 if world >= 8 else 1) if tp == "auto" else int(tp)
        self.ep_world, self.ep_rank = world // self.moe_tp, rank // self.moe_tp
        # several ranks: every rank also holds the whole output projection, so the attention half
        # exchanges the heads' outputs instead of reducing partial sums (--reduce-w-o: the latter)
        full_w_o = world > 1 and not args.replicated and not getattr(args, "reduce_w_o", False) \
            and not args.nccl_reduce
        if self.ffn == "dense":
            w = layer.make_weights(self.shape, rank, world, device, ffn="dense", std=0.02, full_w_o=full_w_o)
        else:
            w = layer.make_weights(self.shape, rank, world, device, ffn="none", std=0.02, full_w_o=full_w_o)
            w["experts"] = layer.make_nvfp4_experts(self.shape, rank, world, device, std=0.02,
                                                    moe_tp=self.moe_tp)
        self.proj = args.proj
        self.schedule = args.nvfp4_schedule
        ops.gemm_nvfp4_schedule({"auto": 0, "single": 1, "pair": 2}[self.schedule])
        pairs_local = self.tokens * self.shape.topk // self.ep_world
        uses_pairs = self.schedule == "pair" or (
            self.schedule == "auto" and pairs_local >= 128 * (self.shape.n_experts // self.ep_world))
        self.dominant = ("gemm_nvfp4_pair_kernel" if uses_pairs else "gemm_nvfp4_kernel") + \
            "[experts w13]"
        if self.ffn == "dense":
            fp8 = args.proj in ("fp8", "mixed")
            self.dominant = ("gemm_fp8_kernel" if fp8 else "gemm_bf16_pair_kernel") + "[dense w13]"
        self.model = self._build_model(w, args)
        gen = torch.Generator(device=device)
        gen.manual_seed(self.shape.seed)
        self.hidden = torch.empty(self.tokens, self.shape.hidden, device=device, dtype=torch.bfloat16)
        self.hidden.normal_(mean=0.0, std=0.01, generator=gen)
        self.positions = torch.arange(self.tokens, device=device, dtype=torch.int64)
        self.dom_events = []
        self._wrap_dominant()

    def _build_model(self, w, args):
        return self.layer_mod.RealisticLayer(self.shape, w, self.rank, self.world, ffn=self.ffn,
                                             proj=args.proj, token_sharded=not args.replicated,
                                             peer_reduce=not args.nccl_reduce)

    def _forward(self, hidden):
        return self.model.forward_stack(hidden, self.positions, self.layers)

    def _wrap_dominant(self):
        """CUDA events around every first expert GEMM (w13) of the timed region."""
        ops, inter2 = self.ops, 2 * self.shape.moe_inter // getattr(self, "moe_tp", 1)
        inner = ops.gemm_nvfp4_grouped
        wl = self

        def timed(*a, **kw):
            if wl.recording and kw.get("n") == inter2:
                s, e = wl._event_pair()
                s.record()
                out = inner(*a, **kw)
                e.record()
                return out
            return inner(*a, **kw)

        self.recording = False
        ops.gemm_nvfp4_grouped = timed
        if self.ffn == "dense":
            # the gate-up projection [2 * 18432 / world, 7168] of the dense FFN
            rows13 = 2 * self.shape.dense_inter // self.world

            def timed_linear(inner_fn, weight_arg):
                def call(*a, **kw):
                    if wl.recording and a[weight_arg].shape[0] == rows13:
                        s, e = wl._event_pair()
                        s.record()
                        out = inner_fn(*a, **kw)
                        e.record()
                        return out
                    return inner_fn(*a, **kw)
                return call

            ops.linear_fp8 = timed_linear(ops.linear_fp8, 2)      # (codes, scales, w_codes, w_scales)
            ops.linear_bf16 = timed_linear(ops.linear_bf16, 1)    # (x, weight)
        # experts that actually receive tokens (their weights are what the GEMM reads)
        inner_permute = ops.fused_moe_permute
        self.touched = []
        self.rank_rows = []       # per recorded layer: routed rows of every rank's expert block

        def permute(indices, n_experts):
            out = inner_permute(indices, n_experts)
            if wl.recording and len(wl.touched) < 64:
                off = out[0]
                lo = wl.ep_rank * (n_experts // wl.ep_world)
                hi = lo + n_experts // wl.ep_world
                wl.touched.append(((off[lo + 1:hi + 1] - off[lo:hi]) > 0).sum())
                if wl.world > 1:
                    wl.rank_rows.append((off[1:] - off[:-1]).view(wl.ep_world, -1).sum(-1))
            return out

        ops.fused_moe_permute = permute

    @property
    def units_per_step(self) -> int:
        return self.tokens * self.layers

    @property
    def dominant_bytes(self) -> int:
        s = self.shape
        if self.ffn == "dense":
            n = 2 * s.dense_inter // self.world
            per = 1 if self.proj in ("fp8", "mixed") else 2
            return per * (self.tokens * s.hidden + n * s.hidden) + self.tokens * n * 2
        e_loc = s.n_experts // self.ep_world
        inter = s.moe_inter // self.moe_tp
        pairs_local = self.tokens * s.topk // self.ep_world    # expected rows of this rank's group
        # experts that receive at least one token (all of them at prefill sizes; at decode
        # sizes only the touched experts' weights are read): counted from the routing of the
        # timed layers, else the expectation under uniform routing
        if self.touched:
            touched = float(torch.stack(self.touched).float().mean())
        else:
            touched = e_loc * (1.0 - (1.0 - 1.0 / s.n_experts) ** (self.tokens * s.topk))
        weights = int(touched * 2 * inter * s.hidden * 9 // 16)   # e2m1 codes + e4m3 scales
        acts = pairs_local * s.hidden * 9 // 16
        out = pairs_local * 2 * inter * 2
        return weights + acts + out

    @property
    def dominant_bytes_all_experts(self) -> int:
        """Algorithmic bytes of a w13 launch in which every local expert receives tokens."""
        s = self.shape
        pairs_local = self.tokens * s.topk // self.ep_world
        inter = s.moe_inter // self.moe_tp
        return ((s.n_experts // self.ep_world) * 2 * inter * s.hidden * 9 // 16
                + pairs_local * s.hidden * 9 // 16 + pairs_local * 2 * inter * 2)

    @property
    def dominant_flops(self) -> int:
        s = self.shape
        if self.ffn == "dense":
            return 2 * self.tokens * (2 * s.dense_inter // self.world) * s.hidden
        return 2 * (self.tokens * s.topk // self.ep_world) * 2 * (s.moe_inter // self.moe_tp) * s.hidden

    @property
    def tensor_peak_factor(self) -> float:
        """Tensor ceiling of the dominant kernel in units of the measured bf16 rate (the nominal
        ratios of the part: e2m1 4 x, e4m3 2 x)."""
        if self.ffn == "dense":
            return 2.0 if self.proj in ("fp8", "mixed") else 1.0
        return 4.0

    @property
    def dominant_traffic(self):
        """dram__bytes_read.sum + dram__bytes_write.sum of one w13 launch, from a one-pass ncu
        capture of the layer-1 launch of this very configuration (all 256 experts receive
        tokens there: 5.03 GB of algorithmic bytes); other sizes were not captured."""
        if self.ffn == "moe" and self.tokens == 8192 and self.world == 1 and self.shape.n_experts == 256:
            return 4.82e9 + 0.60e9
        return None

    def config(self) -> dict:
        s = self.shape
        return {"workload": self.name, "tokens": self.tokens, "layers": self.layers,
                "hidden": s.hidden, "heads": s.heads, "experts": s.n_experts, "topk": s.topk,
                "moe_inter": s.moe_inter, "ffn": self.ffn, "experts_dtype": "nvfp4", "experts_gemm_schedule": self.schedule,
                "projections_dtype": self.proj,
                "attention_core": "rt_attn_causal_prefill (tcgen05, this backend)"
                if self.layer_mod.ATTENTION_CORE == "rt" else "torch sdpa (yardstick: not a kernel of this backend)",
                "routing": "topk_softmax (racetrack/realistic_bench.py:321-327)",
                "l2_policy": "inputs_exceed_l2 (6.3 GB of expert weights + 117 MB of hidden "
                             "states stream through the 126 MB L2 every layer)"}

    graph = None
    capturing = False

    def _event_pair(self):
        """Two timing events around a launch of the dominant kernel. While the stack is being
        captured they become event-record NODES of the graph (external events), so every replay
        inside the timed region stamps them."""
        s = torch.cuda.Event(enable_timing=True, external=self.capturing)
        e = torch.cuda.Event(enable_timing=True, external=self.capturing)
        (self.graph_events if self.capturing else self.dom_events).append((s, e))
        return s, e

    def capture_graph(self):
        """Captures one forward of the stack in a CUDA graph (what racetrack/bench.py:98-111
        does for its sweeps); steps then replay it. Every op only enqueues work on the current
        stream and allocates through torch, so the whole stack is capturable."""
        from racetrack_b200 import _lib
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward(self.hidden)
        torch.cuda.current_stream().wait_stream(side)
        before = _lib.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        self.graph_events = []
        self.capturing = self.recording = True
        group = getattr(getattr(self, "model", None), "comm", None)
        calls0 = group.nccl_calls if group is not None else 0
        try:
            with torch.cuda.graph(self.graph):
                self.graph_out = self._forward(self.hidden)
        finally:
            self.capturing = self.recording = False
        # whether the captured step holds library collectives (the peer-memory schedule has none)
        self.graph_has_nccl = group is not None and group.nccl_calls > calls0
        self.launches_per_replay = _lib.launch_count() - before

    def capture_timing_graph(self, group):
        """A second graph of the same forward with the group's timing events captured as nodes;
        returns the function that replays it."""
        g = torch.cuda.CUDAGraph()
        group.start_timing(in_graph=True)
        with torch.cuda.graph(g):
            self._timing_out = self._forward(self.hidden)
        self._timing_graph = g
        return g.replay

    def step(self, record: bool = False):
        if self.graph is not None and not record:
            self.graph.replay()
            return self.graph_out
        self.recording = record
        out = self._forward(self.hidden)
        self.recording = False
        return out

    CHECK_TOKENS, CHECK_LAYERS = 8, 2

    def check(self):
        """Validation of what is timed, outside the timed region (the reference runner validates
        every configuration it times, racetrack/realistic_bench.py:530-538): see layer_check."""
        t = min(self.CHECK_TOKENS, self.tokens)
        return layer_check(self.model, self.shape, self.hidden[:t].clone(), self.positions[:t],
                           self.CHECK_LAYERS, proj=self.proj, ffn=self.ffn, rank=self.rank)

    def e2e_setup(self):
        self.host_in = torch.empty(self.hidden.shape, dtype=torch.bfloat16, pin_memory=True)
        self.host_in.copy_(self.hidden)
        self.dev_in = torch.empty_like(self.hidden)
        self.host_out = torch.empty(self.hidden.shape, dtype=torch.bfloat16, pin_memory=True)

    def e2e_step(self):
        if self.graph is not None:       # the graph reads self.hidden: refresh it from the host
            self.hidden.copy_(self.host_in, non_blocking=True)
            self.graph.replay()
            self.host_out.copy_(self.graph_out, non_blocking=True)
            return self.graph_out
        self.dev_in.copy_(self.host_in, non_blocking=True)
        out = self._forward(self.dev_in)
        self.host_out.copy_(out, non_blocking=True)
        return out

    def e2e_bytes(self):
        n = self.host_in.numel() * self.host_in.element_size()
        return n, n

    @staticmethod
    def cpu_runner(sample_tokens: int):
        """The reference's vanilla-torch layer (oracle/ref_layer.py) on `sample_tokens` tokens,
        one layer, full width. Only the experts the sample routes to are materialised."""
        from oracle import ref_layer, ref_ops as R
        from racetrack_b200 import layer
        shape = layer.DSV32
        g = torch.Generator().manual_seed(shape.seed)
        hidden = (torch.randn(sample_tokens, shape.hidden, generator=g) * 0.01).to(torch.bfloat16)
        pos = torch.arange(sample_tokens, dtype=torch.int64)
        if PrefillStackWorkload.ffn == "dense":
            wd = layer.make_weights(shape, 0, 1, "cpu", ffn="dense", std=0.02)

            def run_dense():
                return ref_layer.forward_stack(hidden, pos, [wd], shape, 1, ffn="dense")
            return run_dense, sample_tokens * 1
        w = layer.make_weights(shape, 0, 1, "cpu", ffn="none", std=0.02)
        ones = torch.ones(shape.hidden, dtype=torch.bfloat16)
        # routing of the sample decides which experts need weights
        h = R.rms_norm(hidden, ones, shape.eps)
        mid = hidden + ref_layer.attention(h, pos, w, shape, shape.heads)
        logits = torch.nn.functional.linear(R.rms_norm(mid, ones, shape.eps).float(), w["w_gate"].float())
        used = sorted(set(torch.topk(logits, shape.topk, dim=-1)[1].flatten().tolist()))
        w["w13"] = torch.empty(shape.n_experts, 2 * shape.moe_inter, shape.hidden, dtype=torch.bfloat16)
        w["w2"] = torch.empty(shape.n_experts, shape.hidden, shape.moe_inter, dtype=torch.bfloat16)
        for e in used:
            w["w13"][e], w["w2"][e] = layer.draw_expert(shape, e, "cpu", std=0.02)

        def run():
            return ref_layer.forward_stack(hidden, pos, [w], shape, 1)
        return run, sample_tokens * 1


# ---------------------------------------------------------------------------
# workload: routed MoE layer at T=4096 (sigmoid + bias grouped top-k gate, NVFP4 experts, one
# bf16 shared expert)
# ---------------------------------------------------------------------------

class MoeLayerWorkload:
    """One routed-MoE layer of DeepSeek-V3.2 (racetrack/models/deepseek.py:998-1022): gate
    [256, 7168] with sigmoid scores + bias, 8 groups / top-4 groups / top-8 experts, route scale
    2.5, NVFP4 experts (w13 [4096, 7168], w2 [7168, 2048]), one shared expert in bf16.
    Experts are replicated work on N GPUs here (weak scaling: every rank runs its own tokens)."""
    name = "dsv3_2_moe_layer_T4096"
    metric = "dsv3_2_layer_tokens_per_s"
    scaling = "weak"

    def __init__(self, device, rank: int, world: int, args):
        from racetrack_b200 import layer, moe, ops
        self.ops, self.moe, self.rank, self.world = ops, moe, rank, world
        self.tokens = args.tokens if args.tokens != 8192 else 4096
        self.shape = s = layer.DSV32
        ops.gemm_nvfp4_schedule({"auto": 0, "single": 1, "pair": 2}[args.nvfp4_schedule])
        uses_pairs = args.nvfp4_schedule == "pair" or (
            args.nvfp4_schedule == "auto" and self.tokens * s.topk >= 128 * s.n_experts)
        self.dominant = ("gemm_nvfp4_pair_kernel" if uses_pairs else "gemm_nvfp4_kernel") + \
            "[experts w13]"
        self.experts = layer.make_nvfp4_experts(s, 0, 1, device, std=0.02)
        self.kw = dict(n_experts=s.n_experts, n_groups=8, topk_groups=4, topk=s.topk,
                       route_scale=2.5, score_func="sigmoid")
        gen = torch.Generator(device=device)
        gen.manual_seed(s.seed + 7 + rank)
        self.x = torch.empty(self.tokens, s.hidden, device=device, dtype=torch.bfloat16)
        self.x.normal_(mean=0.0, std=1.0, generator=gen)
        self.w_gate = torch.empty(s.n_experts, s.hidden, device=device, dtype=torch.bfloat16)
        self.w_gate.normal_(mean=0.0, std=0.02, generator=gen)
        self.bias = torch.empty(s.n_experts, device=device, dtype=torch.float32)
        self.bias.uniform_(-0.1, 0.1, generator=gen)
        sw13, sw2 = layer.draw_expert(s, s.n_experts, device, std=0.02)     # the shared expert
        self.sw13, self.sw2 = sw13.contiguous(), sw2.contiguous()
        self.dom_events, self.recording = [], False
        inner = ops.gemm_nvfp4_grouped
        wl = self

        def timed(*a, **kw):
            if wl.recording and kw.get("n") == 2 * s.moe_inter:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = inner(*a, **kw)
                e1.record()
                wl.dom_events.append((e0, e1))
                return out
            return inner(*a, **kw)

        ops.gemm_nvfp4_grouped = timed

    @property
    def units_per_step(self) -> int:
        return self.tokens

    @property
    def dominant_bytes(self) -> int:
        s = self.shape
        pairs = self.tokens * s.topk
        return (s.n_experts * 2 * s.moe_inter * s.hidden * 9 // 16 + pairs * s.hidden * 9 // 16
                + pairs * 2 * s.moe_inter * 2)

    @property
    def dominant_flops(self) -> int:
        s = self.shape
        return 2 * self.tokens * s.topk * 2 * s.moe_inter * s.hidden

    def config(self) -> dict:
        s = self.shape
        return {"workload": self.name, "tokens": self.tokens, "layers": 1, "hidden": s.hidden,
                "experts": s.n_experts, "topk": s.topk, "moe_inter": s.moe_inter,
                "experts_dtype": "nvfp4", "shared_expert": "bf16",
                "routing": "sigmoid + bias, 8 groups, top-4 groups, top-8 (deepseek.py:888-920)",
                "l2_policy": "inputs_exceed_l2 (6.3 GB of expert weights stream through the "
                             "126 MB L2 every step)"}

    def _run(self, x, record):
        ops, s = self.ops, self.shape
        self.recording = record
        gate_up = ops.linear_bf16(x, self.sw13)
        shared = ops.linear_bf16(ops.fused_swiglu(gate_up[:, :s.moe_inter], gate_up[:, s.moe_inter:]),
                                 self.sw2)
        out = self.moe.fused_moe_forward(x, self.w_gate, self.bias, self.experts, shared=shared,
                                         **self.kw)
        self.recording = False
        return out

    def step(self, record: bool = False):
        return self._run(self.x, record)

    def check(self):
        """The first 8 tokens of the timed input through the same code path, against
        racetrack's MoE.forward on the CPU (oracle/ref_ops: Gate.forward, the expert loop on
        NVFP4 operands, the bf16 shared expert); the un-quantised MoE.forward stands beside it."""
        from oracle import ref_ops as R
        from racetrack_b200 import layer
        s, t = self.shape, min(8, self.tokens)
        out = self._run(self.x[:t].clone(), False)
        if self.rank != 0:
            return None
        kw = dict(n_groups=8, topk_groups=4, topk=s.topk, route_scale=2.5)
        x, wg, b = self.x[:t].cpu(), self.w_gate.cpu(), self.bias.cpu()
        wts, idx = R.gate_forward(x, wg, b, **kw)
        inter, dev = s.moe_inter, self.x.device
        split = lambda w13, w2: (w13[:inter].cpu(), w2.cpu(), w13[inter:].cpu())     # (w1, w2, w3)
        experts = [None] * s.n_experts
        w13 = torch.empty(s.n_experts, 2 * inter, s.hidden, dtype=torch.bfloat16)
        w2 = torch.empty(s.n_experts, s.hidden, inter, dtype=torch.bfloat16)
        gs13, gs2 = torch.zeros(s.n_experts), torch.zeros(s.n_experts)
        one = torch.ones((), device=dev)
        for e in sorted(set(idx.flatten().tolist())):
            a, c = layer.draw_expert(s, e, dev, std=0.02)
            experts[e] = split(a, c)
            for dst, gsv, m in ((w13, gs13, a), (w2, gs2, c)):
                codes, sf, gs = self.ops.fused_nvfp4_quant(m)
                dst[e] = R.nvfp4_dequant(codes, sf, one).to(torch.bfloat16).cpu()
                gsv[e] = float(gs)
        shared = split(self.sw13, self.sw2)
        ref = R.moe_experts_nvfp4(x, wts.float(), idx, w13, w2, shared_out=R.expert_mlp(x, *shared),
                                  weights_dequantised=(gs13, gs2))
        ref16 = R.moe_forward(x, wg, b, experts, shared, **kw)
        return _criterion(out, ref, ref16, tokens=t, layers=1)

    def e2e_setup(self):
        self.host_in = torch.empty(self.x.shape, dtype=torch.bfloat16, pin_memory=True)
        self.host_in.copy_(self.x)
        self.dev_in = torch.empty_like(self.x)
        self.host_out = torch.empty(self.x.shape, dtype=torch.bfloat16, pin_memory=True)

    def e2e_step(self):
        self.dev_in.copy_(self.host_in, non_blocking=True)
        out = self._run(self.dev_in, False)
        self.host_out.copy_(out, non_blocking=True)
        return out

    def e2e_bytes(self):
        n = self.host_in.numel() * self.host_in.element_size()
        return n, n

    @staticmethod
    def cpu_runner(sample_tokens: int):
        """racetrack's MoE.forward (oracle/ref_ops.moe_forward) on `sample_tokens` tokens at full
        width, bf16 weights; only the experts the sample routes to are materialised."""
        from oracle import inputs as I, ref_ops as R
        from racetrack_b200 import layer
        s = layer.DSV32
        d = I.gate_inputs(sample_tokens)
        kw = dict(n_groups=d["n_groups"], topk_groups=d["topk_groups"], topk=d["topk"],
                  route_scale=d["route_scale"])
        _, idx = R.gate_forward(d["hidden"], d["w_gate"], d["bias"], **kw)
        experts = [None] * s.n_experts
        inter = s.moe_inter

        def split(w13, w2):
            return w13[:inter], w2, w13[inter:]          # (w1, w2, w3)
        for e in sorted(set(idx.flatten().tolist())):
            experts[e] = split(*layer.draw_expert(s, e, "cpu", std=0.02))
        shared = split(*layer.draw_expert(s, s.n_experts, "cpu", std=0.02))

        def run():
            return R.moe_forward(d["hidden"], d["w_gate"], d["bias"], experts, shared, **kw)
        return run, sample_tokens


# ---------------------------------------------------------------------------
# workload: SwiGLU + activation quantisation at T=4096 (gate_up [T, 2*18432] bf16)
# ---------------------------------------------------------------------------

class SwigluQuantWorkload:
    """silu(gate)*up -> FP8 e4m3 per-128 codes+scales and NVFP4 codes+block scales+global scale."""
    name = "swiglu_act_quant_T4096_I18432"
    metric = "dsv3_2_swiglu_quant_tokens_per_s"
    scaling = "weak"
    dominant = "quant_fp8_kernel<swiglu>"
    tokens_default = 4096
    inter = 18432

    def __init__(self, device, rank: int, world: int, args):
        from racetrack_b200 import ops
        self.ops = ops
        self.tokens, self.layers = self.tokens_default, 1
        gen = torch.Generator(device=device)
        gen.manual_seed(38595 + rank)
        self.gate_up = torch.empty(self.tokens, 2 * self.inter, device=device, dtype=torch.bfloat16)
        self.gate_up.normal_(generator=gen)
        self.dom_events = []

    @property
    def units_per_step(self) -> int:
        return self.tokens

    @property
    def dominant_bytes(self) -> int:
        t, i = self.tokens, self.inter
        return 2 * t * i * 2 + t * i + t * (i // 128) * 4

    def config(self) -> dict:
        return {"workload": self.name, "tokens": self.tokens, "inter": self.inter,
                "outputs": "fp8_e4m3_per128+nvfp4_block16",
                "l2_policy": "inputs_exceed_l2 (302 MB gate_up per step vs 126 MB L2)"}

    def _run(self, gate_up, record):
        ops, i = self.ops, self.inter
        g, u = gate_up[:, :i], gate_up[:, i:]
        if record:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        codes, scales = ops.fused_swiglu_quant(g, u)
        if record:
            e.record()
            self.dom_events.append((s, e))
        c4, sf, gs = ops.fused_swiglu_nvfp4_quant(g, u)
        return codes, scales, c4, sf, gs

    def step(self, record: bool = False):
        return self._run(self.gate_up, record)

    def check(self):
        """Codes and scales of the first 64 rows against act_quant(swiglu(.)) on the CPU
        (racetrack/models/deepseek.py:85-107): the fraction of FP8 codes that differ (the CPU's
        expf may differ from the GPU's in the last ulp before the bf16 rounding)."""
        from oracle import ref_ops as R
        rows = self.gate_up[:64]
        codes, scales, *_ = self._run(rows, False)
        g, u = rows[:, :self.inter].cpu(), rows[:, self.inter:].cpu()
        rc, rs = R.swiglu_quant(g, u)
        bad = float((codes.cpu().view(torch.uint8) != rc.view(torch.uint8)).float().mean())
        return {"fp8_codes_differing": bad, "scales_equal": bool(torch.equal(scales.cpu(), rs)),
                "ok": bad <= 1e-3, "tokens": 64, "layers": 1,
                "against": "CPU restatement of act_quant(swiglu(gate, up))"}

    def e2e_setup(self):
        self.host_in = torch.empty(self.gate_up.shape, dtype=torch.bfloat16, pin_memory=True)
        self.host_in.copy_(self.gate_up)
        self.dev_in = torch.empty_like(self.gate_up)
        self.host_out = [torch.empty(o.shape, dtype=o.dtype, pin_memory=True) for o in self.step()]

    def e2e_step(self):
        self.dev_in.copy_(self.host_in, non_blocking=True)
        outs = self._run(self.dev_in, False)
        for h, o in zip(self.host_out, outs):
            h.copy_(o, non_blocking=True)
        return outs

    def e2e_bytes(self):
        return (self.host_in.numel() * 2,
                sum(h.numel() * h.element_size() for h in self.host_out))

    @staticmethod
    def cpu_runner(sample_tokens: int):
        from oracle import inputs as I, ref_ops as R
        sample_tokens = 256
        d = I.swiglu_quant_inputs(sample_tokens, SwigluQuantWorkload.inter)

        def run():
            R.swiglu_quant(d["gate"], d["up"])
            R.nvfp4_quant(R.swiglu(d["gate"], d["up"]))
        return run, sample_tokens


# ---------------------------------------------------------------------------
# workload: decode step of the layer (B sequences, one token each, caches of 4096 positions,
# sparse indexer + sparse attention, NVFP4 experts)
# ---------------------------------------------------------------------------

class DecodeLayerWorkload(PrefillStackWorkload):
    """`tokens` sequences decode one token each through `layers` applications of the layer; every
    sequence has a latent / rope / indexer cache of `cache_len` positions ~ N(0, 1), the indexer
    keeps 2048 of them. Heads and experts are sharded as in the prefill stack; the token batch and
    the (head-shared) latent caches are replicated on every rank."""
    name = "dsv3_2_decode_layer"
    cache_len = 4096
    default_tokens = 64
    default_proj = "bf16"
    graph_default = True      # a decode step is replayed from a CUDA graph, as racetrack/bench.py:98-111 does
    comm_schedule = ("tokens replicated (a decode step has few rows); the two all-reduces of a layer as "
                     "one-shot reductions over peer memory fused with residual add + RMSNorm")

    def _build_model(self, w, args):
        from racetrack_b200 import decode
        self.decode = decode
        self.start_pos = self.cache_len - 1
        caches = decode.DecodeCaches(self.shape, self.tokens, self.cache_len, self.device,
                                     fill=self.start_pos)
        iw = decode.make_indexer_weights(self.shape, self.device, std=0.02)
        return decode.DecodeLayer(self.shape, w, self.rank, self.world, index_weights=iw,
                                  caches=caches, proj=args.proj)

    def _forward(self, hidden):
        return self.model.decode_stack(hidden, self.start_pos, self.layers)

    @property
    def dominant_traffic(self):
        return None

    def check(self):
        """One eager decode step of the whole batch through one layer, validated for the first two
        sequences against the CPU restatement of the reference's decode branch
        (oracle/ref_layer.py) on the same weights and cache contents, stage by stage on
        identical inputs: the attention half (cache append, indexer, sparse attention, wo) and
        the expert half (NVFP4 operands, the batch's own tensor-wide scales)."""
        from oracle import ref_layer, ref_ops as R
        layer, s, m, ops = self.layer_mod, self.shape, self.model, self.ops
        b = min(2, self.tokens)
        normed = ops.fused_rms_norm(self.hidden, m.ones_h, eps=s.eps)
        attn = m.decode_attention(normed, self.start_pos)
        n2, _ = ops.fused_residual_norm(attn, self.hidden, m.ones_h, eps=s.eps)
        logits = ops.linear_bf16(n2, m.w_gate, out_dtype=torch.float32)
        wts, idx = ops.fused_moe_route(logits, None, n_groups=1, topk_groups=1, topk=s.topk,
                                       route_scale=1.0, score_func="topk_softmax")
        parts: dict = {}
        ffn = self.moe.fused_moe_experts(n2, wts, idx, m.experts, n_experts=s.n_experts,
                                         expert_begin=m.expert_begin, parts=parts)
        ffn = m._all_reduce(ffn)
        ops.tc_error_state()
        if self.rank != 0:
            return None
        full = layer.make_weights(s, 0, 1, self.device, ffn="none", std=0.02)
        w = {k: v.cpu() for k, v in full.items()}
        del full
        iw_dev = m.index_weights
        iw = {"wq_b": iw_dev.wq_b.cpu(), "wk": iw_dev.wk.cpu(),
              "k_norm_weight": iw_dev.k_norm_weight.cpu(), "k_norm_bias": iw_dev.k_norm_bias.cpu(),
              "weights_proj": iw_dev.weights_proj.cpu()}
        c = m.caches
        caches = {"kv": c.kv[:b].cpu(), "pe": c.pe[:b].cpu(), "index_k": c.index_k[:b].cpu(),
                  "index_scale": c.index_scale[:b].cpu()}
        ref_attn = ref_layer.decode_attention(normed[:b].cpu(), self.start_pos, w, iw, caches, s, s.heads,
                                              m.freqs.cpu(), m.index_topk)
        stages = [{"stage": "attention", **_criterion(attn[:b], ref_attn)}]
        bank = ref_layer.ExpertBank(s, w, lambda e: layer.draw_expert(s, e, self.device, std=0.02),
                                    quantise=lambda x: ops.fused_nvfp4_quant(x))
        x = n2[:b].cpu()
        i_cpu, w_cpu = idx[:b].cpu(), wts[:b].cpu()
        bank.need(i_cpu.flatten().tolist())
        x_amax = parts["x_amax"].cpu() if self.world == 1 else None
        ref_ffn = R.moe_experts_nvfp4(x, w_cpu, i_cpu, w["w13_dq"], w["w2_dq"],
                                      weights_dequantised=(w["w13_gs"], w["w2_gs"]),
                                      x_amax=x_amax,
                                      h_amax=parts["h_amax"].cpu() if self.world == 1 else None)
        stages.append({"stage": "ffn", **_criterion(ffn[:b], ref_ffn)})
        keep = ("stage", "diff", "rel", "max_abs_ref", "ok")
        return {"ok": all(st["ok"] for st in stages), "tokens": b, "layers": 1,
                "criterion": f"diff <= {CHECK_ATOL} + {CHECK_RTOL} * max|ref|",
                "mode": "attention half and expert half of one decode step against the CPU restatement "
                        "of the reference's decode branch, fed the product's own input",
                "stages": [{k: st[k] for k in keep} for st in stages]}

    def config(self) -> dict:
        c = super().config()
        c.update({"workload": self.name, "sequences": self.tokens, "cache_len": self.cache_len,
                  "index_heads": self.decode.INDEX_HEADS, "index_topk": self.decode.INDEX_TOPK,
                  "attention_core": "rt_mla_sparse_decode (tcgen05, this backend)",
                  "l2_policy": "inputs_exceed_l2 at 64 sequences (every layer reads the touched "
                               "experts' weights, up to 6.3 GB, and 151 MB of selected cache rows); "
                               "below that the touched experts alone exceed the 126 MB L2 from "
                               "4 sequences on"})
        return c

    @staticmethod
    def cpu_runner(sample_tokens: int):
        """The reference's decode branch (oracle/ref_layer.py decode_stack) for `sample_tokens`
        sequences, one layer, full width, caches of 4096 positions."""
        from oracle import ref_layer, ref_ops as R
        from racetrack_b200 import layer
        shape = layer.DSV32
        L = DecodeLayerWorkload.cache_len
        start = L - 1
        g = torch.Generator().manual_seed(shape.seed)
        b = sample_tokens
        hidden = (torch.randn(b, shape.hidden, generator=g) * 0.01).to(torch.bfloat16)
        w = layer.make_weights(shape, 0, 1, "cpu", ffn="none", std=0.02)
        mk = lambda *s, std=1.0: torch.randn(*s, generator=g) * std
        iw = {"wq_b": mk(64 * 128, shape.q_lora, std=0.02).bfloat16(),
              "wk": mk(128, shape.hidden, std=0.02).bfloat16(), "k_norm_weight": torch.ones(128),
              "k_norm_bias": torch.zeros(128), "weights_proj": mk(64, shape.hidden, std=0.02)}
        keys, scales = R.act_quant(mk(b, L, 128).bfloat16())
        caches = {"kv": mk(b, L, shape.kv_lora).bfloat16(), "pe": mk(b, L, shape.rope).bfloat16(),
                  "index_k": keys, "index_scale": scales.squeeze(-1).contiguous()}
        freqs = R.precompute_freqs_cis(shape.rope, L)
        w["w13"] = torch.empty(shape.n_experts, 2 * shape.moe_inter, shape.hidden, dtype=torch.bfloat16)
        w["w2"] = torch.empty(shape.n_experts, shape.hidden, shape.moe_inter, dtype=torch.bfloat16)
        drawn = set()

        def run():
            # experts are drawn when the routing of this sample first asks for them
            ones = torch.ones(shape.hidden, dtype=torch.bfloat16)
            h = R.rms_norm(hidden, ones, shape.eps)
            mid = hidden + ref_layer.decode_attention(h, start, w, iw, caches, shape, shape.heads,
                                                      freqs, 2048)
            logits = torch.nn.functional.linear(R.rms_norm(mid, ones, shape.eps).float(), w["w_gate"].float())
            for e in set(torch.topk(logits, shape.topk, dim=-1)[1].flatten().tolist()) - drawn:
                w["w13"][e], w["w2"][e] = layer.draw_expert(shape, e, "cpu", std=0.02)
                drawn.add(e)
            return ref_layer.decode_stack(hidden, start, [w], iw, [caches], shape, 1, freqs, 2048)
        return run, sample_tokens * 1


WORKLOADS = {w.name: w for w in (PrefillStackWorkload, MoeLayerWorkload, SwigluQuantWorkload,
                                 DecodeLayerWorkload)}
DEFAULT_WORKLOAD = PrefillStackWorkload.name


def cpu_line(wl_cls, steps: int, warmup: int) -> dict:
    # all host threads, also under torchrun (which exports OMP_NUM_THREADS=1 to every rank)
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        torch.set_num_threads(os.cpu_count() or 1)
    run, units = wl_cls.cpu_runner(CPU_SAMPLE_TOKENS)
    for _ in range(max(warmup, 1)):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    cores = torch.get_num_threads()
    return {"value": units * steps / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "ms_per_step": 1e3 * dt / steps,
            "sample": f"{units} token(s) x 1 layer per step at full width, torch CPU "
                      f"(oracle/ref_layer.py), {cores} threads of {os.cpu_count()} logical cores"}


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = WORKLOADS[args.workload]
    cpu = cpu_line(wl, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": wl.metric, "value": cpu["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": cpu.pop("ms_per_step"), "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl.name, "device": "host CPU", "sample": cpu["sample"]},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    import torch.distributed as dist
    from racetrack_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        # NCCL writes its version banner to stdout when NCCL_DEBUG is set in the environment;
        # stdout carries the one JSON line only, so file descriptor 1 points at stderr while
        # the communicator comes up
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier(device_ids=[local_rank])
            torch.cuda.synchronize(device)
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    def barrier():
        if distributed:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(device)

    def max_over_ranks(ms: float) -> float:
        if not distributed:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    _lib.load()
    wl = WORKLOADS[args.workload](device, rank, world, args)

    use_graph = (args.graph or getattr(wl, "graph_default", False)) and not args.no_graph \
        and hasattr(wl, "capture_graph")
    if use_graph:
        wl.step()
        barrier()
        wl.capture_graph()
    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _lib.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.profiler_range:      # lets `ncu --profile-from-start off` see the timed steps only
        torch.cuda.profiler.start()
    start.record()
    for _ in range(args.steps):
        wl.step(record=not use_graph)
    end.record()
    barrier()
    if args.profiler_range:
        torch.cuda.profiler.stop()
    launches = _lib.launch_count() - launches0
    ms_total = max_over_ranks(start.elapsed_time(end))
    timed_in = None
    if use_graph:
        # a replayed graph runs no host code: launches are those recorded at capture. The dominant
        # kernel is timed by event-record nodes captured around each of its launches, read after
        # the last timed replay; a workload that captured none times it in two eager steps
        launches = wl.launches_per_replay * args.steps
        if getattr(wl, "graph_events", None):
            wl.dom_events = list(wl.graph_events)
            timed_in = "event-record nodes of the replayed graph (the last timed step)"
        else:
            for _ in range(2):
                wl.step(record=True)
            barrier()
            timed_in = "two eager steps after the replayed region"
    dom_us = statistics.mean(s.elapsed_time(e) for s, e in wl.dom_events) * 1e3
    # where the step's time goes between the ranks: one more eager step with CUDA events around
    # every collective (outside the timed region)
    comm_stats = None
    group = getattr(getattr(wl, "model", None), "comm", None)
    if distributed and group is not None:
        barrier()
        if use_graph and hasattr(wl, "capture_timing_graph"):
            # a second capture of the same stack with event-record nodes around every collective:
            # replayed like the timed steps, so the intervals carry no host launch skew
            replay = wl.capture_timing_graph(group)
            barrier()
            replay()
            replay()
        else:
            group.start_timing()
            wl.step(record=True)
        per = group.stop_timing()
        layers = max(getattr(wl, "layers", 1), 1)
        comm_ms = max_over_ranks(sum(ms for _, ms, _ in per.values())) / layers
        comm_stats = {"comm_ms_per_layer": comm_ms,
                      "collectives_per_layer": {k: {"calls": c / layers, "ms": ms / layers,
                                                    "payload_mb": b / layers / 1e6}
                                                for k, (c, ms, b) in per.items()},
                      "schedule": getattr(wl, "comm_schedule", None) or
                                  ("token-sharded: reduce-scatter -> token-wise kernels on T/N rows -> "
                                   "all-gather of their compact outputs"
                                   + ("; attention half: heads' outputs exchanged, whole w_o on the rank's rows"
                                      if getattr(wl.model, "w_o_full", None) is not None else ""))
                      if getattr(wl.model, "token_sharded", False) else "replicated tokens, all-reduce"}

    wl.e2e_setup()
    for _ in range(min(args.warmup, 2)):
        wl.e2e_step()
    barrier()
    e2e_steps = max(2, min(args.steps, 5))
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        wl.e2e_step()
    e2.record()
    barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2))
    clocks = sampler.stop()
    h2d, d2h = wl.e2e_bytes()
    # validation of the timed configuration (outside every timed region)
    check = None
    if not args.no_check and hasattr(wl, "check"):
        try:
            torch.set_num_threads(len(os.sched_getaffinity(0)))
        except (AttributeError, RuntimeError):
            pass
        check = wl.check()
        barrier()
    from racetrack_b200 import ops
    ops.tc_error_state()

    if rank == 0:
        hbm_peak, bf16_peak, peak_src = measured_peaks()
        roof = {"bound": "hbm", "kernel": wl.dominant,
                "achieved": wl.dominant_bytes / (dom_us * 1e-6) / 1e9, "peak": hbm_peak,
                "unit": "GB/s"}
        flops = getattr(wl, "dominant_flops", 0)
        if flops:
            # the kernel is a block-scaled e2m1 GEMM: its tensor ceiling is taken as 4 x the
            # measured bf16 cuBLAS throughput (the nominal e2m1 : bf16 ratio of the part); the
            # bound reported is whichever ideal time (bytes / HBM, flops / tensor) is longer
            factor = float(getattr(wl, "tensor_peak_factor", 4.0))
            tensor_peak = factor * bf16_peak
            tensor = {"bound": "tensor", "kernel": wl.dominant,
                      "achieved": flops / (dom_us * 1e-6) / 1e12, "peak": tensor_peak,
                      "unit": "TFLOP/s",
                      "peak_note": f"{factor:g} x measured sustained bf16 cuBLAS (nominal ratio "
                                   "of the operand format to bf16)"}
            if flops / (tensor_peak * 1e12) > wl.dominant_bytes / (hbm_peak * 1e9):
                roof, tensor = tensor, roof
            roof["other_bound"] = {k: tensor[k] for k in ("bound", "achieved", "peak", "unit")}
            roof["other_bound"]["frac"] = tensor["achieved"] / tensor["peak"]
            roof["algorithmic_flops"] = flops
        traffic = getattr(wl, "dominant_traffic", None)
        if traffic is not None:
            # the captured launch touches every expert; its own algorithmic bytes stand beside
            # the measured traffic (the average launch of the timed region touches fewer experts)
            roof["traffic_launch_algorithmic_bytes"] = wl.dominant_bytes_all_experts
        roof.update({"frac": roof["achieved"] / roof["peak"], "peak_source": peak_src,
                     "traffic": traffic, "avg_launch_us": dom_us,
                     "launches_timed": len(wl.dom_events),
                     "algorithmic_bytes": wl.dominant_bytes})
        line = {
            "metric": wl.metric,
            "value": wl.units_per_step * args.steps / (ms_total * 1e-3)
                     * (world if wl.scaling == "weak" else 1),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": wl.scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {**wl.config(),
                       "parallelism": (f"tp{world}(heads)+ep{getattr(wl, 'ep_world', world)}"
                                       + (f"xtp{wl.moe_tp}" if getattr(wl, "moe_tp", 1) > 1 else "")
                                       + "(experts)") if wl.scaling == "strong"
                       else f"replicated-stream x{world}"},
            "roofline": roof,
            "e2e": {"value": wl.units_per_step * e2e_steps / (e2e_ms * 1e-3)
                             * (world if wl.scaling == "weak" else 1),
                    "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        line["check"] = check
        if comm_stats is not None and getattr(wl, "rank_rows", None):
            rr = torch.stack(wl.rank_rows).float()
            ratio = rr.max(dim=1).values / rr.mean(dim=1).clamp_min(1.0)
            comm_stats["expert_rows_busiest_rank_over_mean"] = {
                "mean": round(float(ratio.mean()), 3), "worst_layer": round(float(ratio.max()), 3),
                "layers_sampled": int(rr.shape[0]),
                "note": "routed (token, expert) rows of the busiest rank's expert block over the mean "
                        "per rank: the feed-forward half runs at that rank's pace"}
        if comm_stats is not None:
            comm_stats["compute_ms_per_layer"] = ms_total / args.steps / max(getattr(wl, "layers", 1), 1) \
                - comm_stats["comm_ms_per_layer"]
            line["multi_gpu"] = comm_stats
        line["config"]["cuda_graph"] = bool(use_graph)
        if use_graph:
            line["roofline"]["timed_in"] = timed_in
        if world == 1 and not args.no_cpu:
            cpu = cpu_line(type(wl), 3, 1)
            cpu.pop("ms_per_step")
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if distributed and use_graph and getattr(wl, "graph_has_nccl", True):
        # A captured graph that holds NCCL kernels kept the interpreter from finishing its
        # teardown here (torch 2.11, NCCL 2.28): drop the graph, meet once more, and leave
        # without running the communicator's destructors. (A graph of this library's own
        # peer-memory collectives only is torn down normally, below.)
        wl.graph = None
        wl.graph_out = None
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    if distributed:
        # the line is printed; should the teardown of the group ever stall, leave anyway
        watchdog = threading.Timer(120.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        # graphs first (they reference the exchange buffers), then the peer mappings, then the group
        for attr in ("graph", "graph_out", "_timing_graph", "_timing_out"):
            if hasattr(wl, attr):
                setattr(wl, attr, None)
        torch.cuda.synchronize()
        for px in list(getattr(getattr(wl, "model", None), "_peer", {}).values()):
            px.close()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=61)
    ap.add_argument("--proj", default=None, choices=("mixed", "fp8", "bf16"),
                    help="arithmetic of the dense projections: FP8 e4m3 block-scaled, bf16, or "
                         "mixed (FP8 where K >= 4096, bf16 elsewhere)")
    ap.add_argument("--nvfp4-schedule", default="auto", choices=("auto", "pair", "single"),
                    help="schedule of the expert GEMMs: the library's choice by size, CTA pairs, "
                         "or single-CTA 128 x 128 tiles")
    ap.add_argument("--ffn", default="moe", choices=("moe", "dense"),
                    help="FFN of the layer: 256 routed NVFP4 experts, or the dense SwiGLU FFN of "
                         "width 18432 that the first three layers of the model use")
    ap.add_argument("--attn-core", default="rt", choices=("rt", "sdpa"),
                    help="attention core of the prefill layer: this backend's causal attention "
                         "kernel, or torch's SDPA as the yardstick it is measured against")
    ap.add_argument("--attn-schedule", default="auto", choices=("auto", "single", "pair"),
                    help="schedule of this backend's attention kernel: the library's choice by shape "
                         "and length, one CTA per 256 query rows, or CTA pairs with key tiles of 256")
    ap.add_argument("--replicated", action="store_true",
                    help="multi-GPU: the reference's schedule (all tokens on every rank, two "
                         "all-reduces per layer) instead of the token-sharded one")
    ap.add_argument("--moe-tp", default="auto", choices=("auto", "1", "2", "4"),
                    help="ranks that share one group's experts and split their intermediate dimension "
                         "(the expert-parallel degree is the world size over this); auto: 2 from 8 ranks on")
    ap.add_argument("--reduce-w-o", action="store_true",
                    help="multi-GPU: keep the output projection row-sharded and reduce its partial sums "
                         "(the reference's arithmetic) instead of exchanging the heads' attention outputs")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="multi-GPU: NCCL reduce-scatter + the plain residual-norm kernel instead of "
                         "the fused kernel that reads the peers' partial sums over NVLink")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true",
                    help="skip the validation of the timed configuration against the CPU oracle")
    ap.add_argument("--graph", action="store_true",
                    help="capture the stack in a CUDA graph and replay it (decode sizes)")
    ap.add_argument("--no-graph", action="store_true",
                    help="run eagerly even where the workload replays a CUDA graph by default (decode)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed steps with cudaProfilerStart/Stop")
    args = ap.parse_args()
    if args.proj is None:
        # prefill: FP8 where the reduction is long; decode: bf16 ("bf16 with NVFP4 experts" is
        # how the decode configuration is stated), where few rows take the split-K path
        args.proj = getattr(WORKLOADS[args.workload], "default_proj", "mixed")
    PrefillStackWorkload.ffn = args.ffn          # the CPU legs draw the same variant
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
