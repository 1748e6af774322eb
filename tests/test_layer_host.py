"""Host-side logic of the sharded layer, on CPU: weight sharding by unit, the reference layer
evaluated with 1 and 2 ranks, and the same 2-rank evaluation over a real gloo process group."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_layer
from racetrack_b200 import layer


def small_shape():
    return layer.DSV32.scaled(name="small", hidden=256, heads=8, q_lora=64, kv_lora=32, nope=16,
                              rope=16, v_dim=16, moe_inter=64, n_experts=8, topk=2, dense_inter=512)


def _inputs(shape, tokens):
    g = torch.Generator().manual_seed(7)
    return ((torch.randn(tokens, shape.hidden, generator=g) * 0.5).to(torch.bfloat16),
            torch.arange(tokens, dtype=torch.int64))


def test_shards_are_slices_of_the_unsharded_weights():
    shape = small_shape()
    full = layer.make_weights(shape, 0, 1, "cpu")
    for world in (2, 4, 8):
        parts = [layer.make_weights(shape, r, world, "cpu") for r in range(world)]
        assert torch.equal(torch.cat([p["w_q_b"] for p in parts]), full["w_q_b"])
        assert torch.equal(torch.cat([p["w_kv_b"] for p in parts]), full["w_kv_b"])
        assert torch.equal(torch.cat([p["w_o"] for p in parts], dim=1), full["w_o"])
        assert torch.equal(torch.cat([p["w13"] for p in parts]), full["w13"])
        assert torch.equal(torch.cat([p["w2"] for p in parts]), full["w2"])
        for p in parts:
            assert torch.equal(p["w_gate"], full["w_gate"]) and torch.equal(p["w_qkv_a"], full["w_qkv_a"])
    dense = layer.make_weights(shape, 0, 1, "cpu", ffn="dense")
    halves = [layer.make_weights(shape, r, 2, "cpu", ffn="dense") for r in range(2)]
    assert torch.equal(torch.cat([h["w1"] for h in halves]), dense["w1"])
    assert torch.equal(torch.cat([h["w2d"] for h in halves], dim=1), dense["w2d"])
    with pytest.raises(ValueError):
        layer.make_weights(shape, 0, 3, "cpu")


@pytest.mark.parametrize("ffn", ["moe", "dense"])
def test_reference_layer_is_invariant_to_the_world_size(ffn):
    shape = small_shape()
    hidden, pos = _inputs(shape, 24)
    one = ref_layer.forward_stack(hidden, pos, [layer.make_weights(shape, 0, 1, "cpu", ffn=ffn)],
                                  shape, 2, ffn=ffn)
    two = ref_layer.forward_stack(hidden, pos,
                                  [layer.make_weights(shape, r, 2, "cpu", ffn=ffn) for r in range(2)],
                                  shape, 2, ffn=ffn)
    # only the order of the bf16 partial sums differs
    assert float((one.float() - two.float()).abs().max()) <= 0.05 * float(one.float().abs().max())


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_rank(rank: int, world: int, port: int, out_path: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        shape = small_shape()
        hidden, pos = _inputs(shape, 16)
        w = layer.make_weights(shape, rank, world, "cpu")
        ones = torch.ones(shape.hidden, dtype=hidden.dtype)
        from oracle import ref_ops as R
        h = R.rms_norm(hidden, ones, shape.eps)
        # one rank's partial results, reduced the way the GPU runner reduces them
        attn = ref_layer.attention(h, pos, w, shape, shape.heads // world).float()
        dist.all_reduce(attn, op=dist.ReduceOp.SUM)
        moe = ref_layer.moe(h, w, shape, rank, shape.n_experts // world).float()
        dist.all_reduce(moe, op=dist.ReduceOp.SUM)
        if rank == 0:
            torch.save({"attn": attn, "moe": moe}, out_path)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reduce_to_the_single_rank_result(tmp_path):
    out_path = str(tmp_path / "rank0.pt")
    mp.spawn(_gloo_rank, args=(2, _free_port(), out_path), nprocs=2, join=True)
    got = torch.load(out_path)
    shape = small_shape()
    hidden, pos = _inputs(shape, 16)
    w = layer.make_weights(shape, 0, 1, "cpu")
    from oracle import ref_ops as R
    h = R.rms_norm(hidden, torch.ones(shape.hidden, dtype=hidden.dtype), shape.eps)
    attn = ref_layer.attention(h, pos, w, shape, shape.heads).float()
    moe = ref_layer.moe(h, w, shape, 0, shape.n_experts).float()
    assert float((got["attn"] - attn).abs().max()) <= 0.03 * float(attn.abs().max()) + 1e-3
    assert float((got["moe"] - moe).abs().max()) <= 0.03 * float(moe.abs().max()) + 1e-3


def test_reference_decode_step_is_invariant_to_the_world_size():
    """The decode branch of the oracle (cache append, indexer, sparse attention, experts) with the
    heads and experts split over 1, 2 and 4 ranks: every rank appends the same cache rows and
    selects the same positions, and the partial sums add up to the one-rank result."""
    from oracle import ref_ops as R
    shape = layer.DSV32.scaled(name="small_decode", hidden=256, heads=8, q_lora=64, kv_lora=64,
                               nope=16, rope=64, v_dim=16, moe_inter=64, n_experts=8, topk=2)
    batch, cache_len, start, topk = 3, 80, 70, 24
    g = torch.Generator().manual_seed(3)
    mk = lambda *s, std=1.0: torch.randn(*s, generator=g) * std
    iw = {"wq_b": mk(64 * 128, shape.q_lora, std=0.05).bfloat16(),
          "wk": mk(128, shape.hidden, std=0.05).bfloat16(), "k_norm_weight": torch.ones(128),
          "k_norm_bias": torch.zeros(128), "weights_proj": mk(64, shape.hidden, std=0.05)}
    keys, scales = R.act_quant(mk(batch, cache_len, 128).bfloat16())
    base = {"kv": mk(batch, cache_len, shape.kv_lora).bfloat16(),
            "pe": mk(batch, cache_len, shape.rope).bfloat16(), "index_k": keys,
            "index_scale": scales.squeeze(-1).contiguous()}
    freqs = R.precompute_freqs_cis(shape.rope, cache_len)
    hidden = (mk(batch, shape.hidden) * 0.5).bfloat16()
    outs, caches = {}, {}
    for world in (1, 2, 4):
        weights = [layer.make_weights(shape, r, world, "cpu", std=0.05) for r in range(world)]
        rank_caches = [{k: v.clone() for k, v in base.items()} for _ in range(world)]
        outs[world] = ref_layer.decode_stack(hidden, start, weights, iw, rank_caches, shape, 2, freqs, topk)
        caches[world] = rank_caches
        for c in rank_caches[1:]:
            for k in base:
                assert torch.equal(c[k].view(torch.uint8), rank_caches[0][k].view(torch.uint8)), k
    scale = float(outs[1].float().abs().max())
    for world in (2, 4):
        assert float((outs[world].float() - outs[1].float()).abs().max()) <= 0.05 * scale
