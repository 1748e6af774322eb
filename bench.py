"""Benchmark of the DeepSeek-V3.2 partition hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One JSON line on stdout (rank 0). A "step" is one pass of the hot path over one batch of
synthetic, seeded input. `value` is whole-job tokens/s with inputs resident in HBM; `e2e` is
the same metric through the public op API with HOST buffers (pinned host -> device copy of
the step's input and device -> host read of its result inside the timed region).
`--impl reference` times racetrack's own vanilla-torch CPU path (restated in oracle/) on the
host cores, on a bounded sample of the same workload.

Under torchrun (N > 1) every rank processes its own batch of the same shape (weak scaling,
no data-path collective: the workload is a row-partitioned stream); time is the max over ranks.
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

METRIC = "dsv3_2_hot_path_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------

def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


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
# workload: SwiGLU + activation quantisation at T=4096 (gate_up [T, 2*18432] bf16)
# ---------------------------------------------------------------------------

class SwigluQuantWorkload:
    """silu(gate)*up -> FP8 e4m3 per-128 codes+scales and NVFP4 codes+block scales+global scale.

    Per step (T tokens): one fused SwiGLU+FP8-quant launch, one abs-max launch pair and one
    fused SwiGLU+NVFP4-quant launch. Algorithmic bytes of the dominant kernel
    (swiglu_quant_fp8): 2*T*I*2 read + T*I + T*(I/128)*4 written.
    """
    name = "swiglu_act_quant_T4096_I18432"
    tokens = 4096
    inter = 18432
    dominant = "quant_fp8_kernel<swiglu>"

    def __init__(self, device: torch.device, seed: int):
        from racetrack_b200 import ops
        self.ops = ops
        self.device = device
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        self.gate_up = torch.empty(self.tokens, 2 * self.inter, device=device, dtype=torch.bfloat16)
        self.gate_up.normal_(generator=gen)
        self.dom_events: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []
        self.host_in = None

    @property
    def dominant_bytes(self) -> int:
        t, i = self.tokens, self.inter
        return 2 * t * i * 2 + t * i + t * (i // 128) * 4

    def config(self) -> dict:
        return {"workload": self.name, "tokens_per_step": self.tokens, "inter": self.inter,
                "outputs": "fp8_e4m3_per128+nvfp4_block16",
                "l2_policy": "inputs_exceed_l2 (302 MB gate_up per step vs 126 MB L2)"}

    def _run(self, gate_up: torch.Tensor, record: bool):
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

    # end to end: pinned host input -> device, kernels, results back to pinned host
    def e2e_setup(self):
        self.host_in = torch.empty(self.gate_up.shape, dtype=torch.bfloat16, pin_memory=True)
        self.host_in.copy_(self.gate_up)
        self.dev_in = torch.empty_like(self.gate_up)
        outs = self.step()
        self.host_out = [torch.empty(o.shape, dtype=o.dtype, pin_memory=True) for o in outs]

    def e2e_step(self):
        self.dev_in.copy_(self.host_in, non_blocking=True)
        outs = self._run(self.dev_in, False)
        for h, o in zip(self.host_out, outs):
            h.copy_(o, non_blocking=True)
        return outs

    def e2e_bytes(self) -> tuple[int, int]:
        h2d = self.host_in.numel() * self.host_in.element_size()
        d2h = sum(h.numel() * h.element_size() for h in self.host_out)
        return h2d, d2h

    # CPU legs (oracle = restated reference torch path)
    @staticmethod
    def cpu_step(sample_tokens: int, inter: int, seed: int):
        from oracle import inputs as I, ref_ops as R
        d = I.swiglu_quant_inputs(sample_tokens, inter, seed=seed)

        def run():
            R.swiglu_quant(d["gate"], d["up"])
            h = R.swiglu(d["gate"], d["up"])
            R.nvfp4_quant(h)
        return run


WORKLOADS = {SwigluQuantWorkload.name: SwigluQuantWorkload}
DEFAULT_WORKLOAD = SwigluQuantWorkload.name


def time_cpu(run, sample_tokens: int, min_seconds: float = 3.0, max_iters: int = 50):
    run()  # warm-up
    n, t0 = 0, time.perf_counter()
    while True:
        run()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or n >= max_iters:
            break
    return sample_tokens * n / dt, dt / n


# ---------------------------------------------------------------------------
# arms
# ---------------------------------------------------------------------------

def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    sample = 256
    run = wl.cpu_step(sample, wl.inter, 38595)
    for _ in range(max(args.warmup, 1) - 1):
        run()
    run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": wl.name, "tokens_per_step": sample, "inter": wl.inter,
                   "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} of {wl.tokens} tokens per step, torch CPU, "
                                   f"{cores} threads of {os.cpu_count()} logical cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
        dist.init_process_group("nccl", device_id=device)

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

    wl = WORKLOADS[args.workload](device, 38595 + rank)
    _lib.load()

    # ---- device-resident timing -------------------------------------------------
    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _lib.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        wl.step(record=True)
    end.record()
    barrier()
    launches = _lib.launch_count() - launches0
    ms_total = max_over_ranks(start.elapsed_time(end))
    dom_us = statistics.mean(s.elapsed_time(e) for s, e in wl.dom_events) * 1e3

    # ---- end to end (host buffers) ------------------------------------------------
    wl.e2e_setup()
    for _ in range(min(args.warmup, 3)):
        wl.e2e_step()
    barrier()
    e2e_steps = max(3, min(args.steps, 20))
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(e2e_steps):
        wl.e2e_step()
    e2.record()
    barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2))
    clocks = sampler.stop()
    h2d, d2h = wl.e2e_bytes()

    if rank == 0:
        peak, peak_src = measured_peaks()
        achieved = wl.dominant_bytes / (dom_us * 1e-6) / 1e9
        line = {
            "metric": METRIC,
            "value": world * wl.tokens * args.steps / (ms_total * 1e-3),
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {**wl.config(), "parallelism": f"replicated-stream x{world}"},
            "roofline": {"bound": "hbm", "kernel": wl.dominant, "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src,
                         "traffic": None, "avg_launch_us": dom_us,
                         "algorithmic_bytes": wl.dominant_bytes},
            "e2e": {"value": world * wl.tokens * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if world == 1:
            sample = 256
            run = wl.cpu_step(sample, wl.inter, 38595)
            cpu_value, _ = time_cpu(run, sample)
            cores = torch.get_num_threads()
            line["cpu_baseline"] = {
                "value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
                "sample": f"{sample} of {wl.tokens} tokens per step, torch CPU, {cores} threads "
                          f"of {os.cpu_count()} logical cores"}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
