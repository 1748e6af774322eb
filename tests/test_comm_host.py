"""Host-side logic of the token-sharded schedule, on CPU with two gloo ranks: the reduce-scatter /
all-gather pair of racetrack_b200.comm around a token-wise step gives what the reference's single
all-reduce followed by the same step on all tokens gives (racetrack/realistic_bench.py:315-316,
351), and the compact payloads (bytes of FP8 / NVFP4 codes, int64 routing) survive the gather."""
from __future__ import annotations

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_ops as R


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from racetrack_b200 import comm
        torch.set_num_threads(1)
        g = comm.Group(rank, world)
        tokens, hidden = 12, 64
        gen = torch.Generator().manual_seed(100 + rank)
        partial = torch.randn(tokens, hidden, generator=gen)            # this rank's partial sums
        residual = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
        ones = torch.ones(hidden, dtype=torch.bfloat16)
        # token-sharded: reduce-scatter, token-wise step on the rank's rows, all-gather
        lo, hi = g.rows_of(tokens)
        mine = g.reduce_scatter_rows(partial.clone())
        normed, summed = R.residual_norm(mine.bfloat16(), residual[lo:hi], ones, 1e-6)
        codes, scales = R.act_quant(normed.repeat(1, 2))                 # 128 columns: one FP8 group
        out = {"normed": g.all_gather_rows(normed), "summed": g.all_gather_rows(summed),
               "codes": g.all_gather_rows(codes), "scales": g.all_gather_rows(scales),
               "ids": g.all_gather_rows(torch.arange(lo, hi, dtype=torch.int64).view(-1, 1) * 7),
               "amax": g.all_reduce_max(normed.float().abs().max().reshape(1))}
        # replicated: all-reduce, the same step on all tokens
        full = g.all_reduce_sum(partial.clone())
        out["ref_normed"], out["ref_summed"] = R.residual_norm(full.bfloat16(), residual, ones, 1e-6)
        out["rows"] = (lo, hi)
        torch.save(out, f"{out_dir}/rank{rank}.pt")
    finally:
        dist.destroy_process_group()


def test_reduce_scatter_step_all_gather_equals_all_reduce_step(tmp_path):
    world = 2
    mp.spawn(_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    assert [o["rows"] for o in outs] == [(0, 6), (6, 12)]
    for o in outs:
        assert torch.equal(o["normed"], o["ref_normed"]) and torch.equal(o["summed"], o["ref_summed"])
        codes, scales = R.act_quant(o["ref_normed"].repeat(1, 2))
        assert torch.equal(o["codes"].view(torch.uint8), codes.view(torch.uint8))
        assert torch.equal(o["scales"], scales)
        assert torch.equal(o["ids"].flatten(), torch.arange(12) * 7)
        assert float(o["amax"]) == float(o["ref_normed"].float().abs().max())
    for key in ("normed", "codes", "ids"):
        assert torch.equal(outs[0][key].view(torch.uint8) if key == "codes" else outs[0][key],
                           outs[1][key].view(torch.uint8) if key == "codes" else outs[1][key])


def test_single_rank_group_is_the_identity():
    from racetrack_b200 import comm
    g = comm.Group()
    x = torch.randn(5, 3)
    assert g.reduce_scatter_rows(x) is x and g.all_gather_rows(x) is x
    assert g.rows_of(10) == (0, 10)
    assert torch.equal(g.all_reduce_max(x.clone()), x)
