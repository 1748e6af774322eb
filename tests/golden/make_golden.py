"""Generates the golden fixtures in this directory by running racetrack itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/racetrack

It imports the reference's own vanilla-torch functions (CPU), feeds them the seeded inputs
of oracle/inputs.py and writes
  * golden_small.pt    - input-free output tensors of small cases (inputs are regenerated
                         from their seeds by the tests), a few hundred KB;
  * golden_hashes.json - SHA-256 of the reference outputs at full hot-path sizes, plus the
                         torch version / CPU capability they were produced with;
  * golden_layer.pt    - racetrack's own ShardedRealisticBlock (racetrack/realistic_bench.py:
                         118-427) on a small shape, world sizes 1 and 2 (gloo ranks as threads of
                         this process are not possible, so the two ranks run as child processes):
                         the weights it drew, its input and its output after 1 and 3 layers.
The fixtures only ever travel as data: nothing at test time imports the reference.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import inputs as I  # noqa: E402


def sha(t: torch.Tensor) -> str:
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float8_e4m3fn):
        raw = t.view(torch.uint8 if t.element_size() == 1 else torch.int16)
    else:
        raw = t
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()


LAYER_SHAPE = dict(name="pin", source="fixture", vocab_size=1, hidden_size=64, num_layers=3,
                   num_attention_heads=4, q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=8,
                   qk_rope_head_dim=8, v_head_dim=8, moe_intermediate_size=32,
                   n_routed_experts=8, num_experts_per_tok=2, seed=38595)
LAYER_TOKENS = 24


def _layer_rank(rank: int, world: int, reference: str, port: int, out_path: str) -> None:
    """One gloo rank: builds racetrack's ShardedRealisticBlock (backend "torch", bf16, CPU), runs
    1 and 3 layers on the runner's own kind of input (racetrack/realistic_bench.py:495-505) and
    saves this rank's weights and outputs."""
    import os
    import torch.distributed as dist
    sys.path.insert(0, reference)
    from racetrack import realistic_bench as rb
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shape = rb.RealisticShape(**LAYER_SHAPE)
        dev = torch.device("cpu")
        g = torch.Generator().manual_seed(shape.seed + 17)
        hidden = torch.empty(LAYER_TOKENS, shape.hidden_size, dtype=torch.bfloat16)
        hidden.normal_(mean=0.0, std=0.5, generator=g)
        positions = torch.arange(LAYER_TOKENS, dtype=torch.int64)
        outs = {}
        for layers in (1, 3):
            model = rb.ShardedRealisticModel(shape, device=dev, dtype=torch.bfloat16, rank=rank,
                                             world_size=world, backend="torch", layers=layers)
            with torch.no_grad():
                outs[layers] = model.forward(hidden.clone(), positions).clone()
        b = model.block
        torch.save({"hidden": hidden, "out1": outs[1], "out3": outs[3],
                    "weights": {k: getattr(b, k).clone() for k in
                                ("w_qkv_a", "w_q_b", "w_kv_b", "w_o", "w_gate", "w13", "w2")}},
                   out_path)
    finally:
        dist.destroy_process_group()


def make_layer_fixture(reference: str) -> None:
    import tempfile
    import torch.multiprocessing as mp
    fixture = {"shape": dict(LAYER_SHAPE), "tokens": LAYER_TOKENS}
    with tempfile.TemporaryDirectory() as tmp:
        for world, port in ((1, 29611), (2, 29612)):
            paths = [f"{tmp}/w{world}_r{r}.pt" for r in range(world)]
            ctx = mp.get_context("spawn")
            procs = [ctx.Process(target=_layer_rank, args=(r, world, reference, port, paths[r]))
                     for r in range(world)]
            for p in procs:
                p.start()
            for p in procs:
                p.join()
                if p.exitcode != 0:
                    raise RuntimeError(f"layer fixture: a rank of world {world} failed")
            ranks = [torch.load(p) for p in paths]
            assert all(torch.equal(r["out3"], ranks[0]["out3"]) for r in ranks)
            fixture[f"world{world}"] = {
                "hidden": ranks[0]["hidden"], "out1": ranks[0]["out1"], "out3": ranks[0]["out3"],
                "rank_weights": [r["weights"] for r in ranks]}
    torch.save(fixture, HERE / "golden_layer.pt")
    size = (HERE / "golden_layer.pt").stat().st_size
    print(f"wrote golden_layer.pt ({size/1024:.0f} KiB)")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the racetrack checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)

    from racetrack.models import deepseek as rm          # noqa: E402
    from partitions import _base as rbase                 # noqa: E402
    from partitions.dsv3_2 import model as rsyn           # noqa: E402

    torch.manual_seed(0)
    small: dict[str, torch.Tensor] = {}
    hashes: dict[str, str] = {}

    # ---- fused MLA prologue, T=128 full width (hashes) and T=8 (tensors) ----
    for tag, tokens in (("c1", 128), ("c1_small", 4)):
        d = I.mla_prologue_inputs(tokens)
        norm = rm.RMSNorm(I.HIDDEN)
        with torch.no_grad():
            norm.weight.copy_(d["w_attn"])
            normed, hidden = norm(d["x"], d["residual"])
            qn = rbase.rms_norm(d["q_c"], d["w_q"], d["eps"])
            kvn = rbase.rms_norm(d["kv_c"], d["w_kv"], d["eps"])
            qn2 = rm.RMSNorm(I.Q_LORA)
            qn2.weight.copy_(d["w_q"])
            qn_real = qn2(d["q_c"])
            margs = rm.ModelArgs(max_seq_len=tokens, qk_rope_head_dim=I.ROPE_DIM,
                                 rope_theta=d["rope_theta"])
            freqs = rm.precompute_freqs_cis(margs)
            q_rot = rm.apply_rotary_emb(d["q_pe"].unsqueeze(0), freqs).squeeze(0)
            k_rot = rm.apply_rotary_emb(d["k_pe"].unsqueeze(0).unsqueeze(2), freqs).squeeze(0)
            k_rot_noninter = rm.apply_rotary_emb(d["k_pe"].unsqueeze(0).unsqueeze(2).contiguous(),
                                                 freqs, False).squeeze(0)
            fq, fkv, fk = rsyn.fused_norm_rope(d["q_c"], d["w_q"], d["kv_c"], d["w_kv"], d["k_pe"],
                                               d["positions"], eps=d["eps"],
                                               rope_base=d["rope_theta"])
            q_half = rsyn.apply_rope(d["q_pe"], d["positions"], base=d["rope_theta"])
        outs = {"normed": normed, "hidden": hidden, "q_norm": qn, "kv_norm": kvn,
                "q_norm_real": qn_real, "freqs_cis": torch.view_as_real(freqs),
                "q_rot": q_rot, "k_rot": k_rot, "k_rot_noninterleaved": k_rot_noninter,
                "fused_q": fq, "fused_kv": fkv, "fused_k": fk, "q_half": q_half}
        for k, v in outs.items():
            hashes[f"{tag}.{k}"] = sha(v)
            if tag == "c1_small":
                small[f"{tag}.{k}"] = v.clone()

    # ---- YaRN table beyond the original sequence length ----
    margs = rm.ModelArgs(max_seq_len=8192, qk_rope_head_dim=I.ROPE_DIM)
    freqs = rm.precompute_freqs_cis(margs)
    hashes["yarn8192.freqs_cis"] = sha(torch.view_as_real(freqs))
    small["yarn8192.freqs_cis_rows"] = torch.view_as_real(freqs)[[0, 1, 4095, 4096, 8191]].clone()

    # ---- SwiGLU / FP8 quant ----
    for tag, tokens, inter in (("c2_small", 16, 512), ("c2_mid", 64, I.DENSE_INTER)):
        d = I.swiglu_quant_inputs(tokens, inter)
        h = (torch.nn.functional.silu(d["gate"].float()) * d["up"].float()).type_as(d["gate"])
        codes, scales = rm.act_quant(d["gate"].contiguous())
        hcodes, hscales = rm.act_quant(h)
        outs = {"swiglu": h, "codes": codes, "scales": scales, "h_codes": hcodes,
                "h_scales": hscales}
        for k, v in outs.items():
            hashes[f"{tag}.{k}"] = sha(v)
            if tag == "c2_small":
                small[f"{tag}.{k}"] = v.clone()
    # MLP module end to end (bf16 weights) on a tiny shape
    mlp = rm.MLP(64, 128)
    w = I.expert_weights(1, 64, 128, seed=I.SEED + 7)[0]
    with torch.no_grad():
        mlp.w1.weight.copy_(w[0]); mlp.w2.weight.copy_(w[1]); mlp.w3.weight.copy_(w[2])
        x = I.randn((8, 64), I.SEED + 8)
        small["mlp_small.out"] = mlp(x).clone()

    # ---- FP8 block-scaled GEMM fallback ----
    a = I.randn((16, 256), I.SEED + 31)
    wfp = I.randn((384, 256), I.SEED + 32, std=0.02, dtype=torch.float32)
    wq = wfp.clamp(-448, 448).to(torch.float8_e4m3fn)
    ws = I.uniform((3, 2), I.SEED + 33, 0.5, 1.5)
    a_q, a_s = rm.act_quant(a)
    small["fp8_gemm.out"] = rm.fp8_gemm(a_q, a_s, wq, ws).clone()
    small["fp8_gemm.dequant"] = rm._block_dequant(wq, ws).clone()

    # ---- Gate (dim 7168 -> bias branch), 64 tokens; and a small softmax gate ----
    d = I.gate_inputs(64)
    margs = rm.ModelArgs(dim=I.HIDDEN, n_routed_experts=I.N_EXPERTS, n_activated_experts=I.TOPK,
                         n_expert_groups=I.N_GROUPS, n_limited_groups=I.TOPK_GROUPS,
                         score_func="sigmoid", route_scale=I.ROUTE_SCALE)
    gate = rm.Gate(margs)
    with torch.no_grad():
        gate.weight.copy_(d["w_gate"])
        gate.bias.copy_(d["bias"])
        gw, gi = gate(d["hidden"])
    small["gate.weights"], small["gate.indices"] = gw.clone(), gi.clone()
    margs = rm.ModelArgs(dim=64, n_routed_experts=8, n_activated_experts=2, score_func="softmax")
    gate = rm.Gate(margs)
    with torch.no_grad():
        gate.weight.copy_(I.randn((8, 64), I.SEED + 41, std=0.2))
        gw, gi = gate(I.randn((32, 64), I.SEED + 42))
    small["gate_softmax.weights"], small["gate_softmax.indices"] = gw.clone(), gi.clone()

    # ---- MoE forward: dim 7168 (bias), 16 experts in 4 groups, top-4, one shared expert ----
    margs = rm.ModelArgs(dim=I.HIDDEN, moe_inter_dim=64, n_routed_experts=16, n_shared_experts=1,
                         n_activated_experts=4, n_expert_groups=4, n_limited_groups=2,
                         score_func="sigmoid", route_scale=I.ROUTE_SCALE)
    moe = rm.MoE(margs)
    ew = I.expert_weights(17, I.HIDDEN, 64, seed=I.SEED + 50)
    with torch.no_grad():
        moe.gate.weight.copy_(I.randn((16, I.HIDDEN), I.SEED + 51, std=0.02))
        moe.gate.bias.copy_(I.uniform((16,), I.SEED + 52, -0.1, 0.1))
        for e in range(16):
            moe.experts[e].w1.weight.copy_(ew[e][0])
            moe.experts[e].w2.weight.copy_(ew[e][1])
            moe.experts[e].w3.weight.copy_(ew[e][2])
        moe.shared_experts.w1.weight.copy_(ew[16][0])
        moe.shared_experts.w2.weight.copy_(ew[16][1])
        moe.shared_experts.w3.weight.copy_(ew[16][2])
        x = I.randn((32, I.HIDDEN), I.SEED + 53)
        y = moe(x)
    small["moe.out_cols0_256"] = y[:, :256].clone()
    hashes["moe.out"] = sha(y)

    # ---- sparse indexer: fp8_index scores and the top-k selection (deepseek.py:164-176, 681-683)
    for tag, queries, keys, topk in (("idx_small", 5, 300, 64), ("idx_decode", 16, 4096, 2048)):
        d = I.indexer_inputs(queries, keys)
        scores = rm.fp8_index(d["q"], d["weights"], d["k"], d["k_scale"])
        if tag == "idx_small":
            small["idx_small.scores"] = scores.clone()
            small["idx_small.topk"] = scores.topk(topk, dim=-1)[1].sort(dim=-1)[0].to(torch.int32)
        else:
            # full decode width: the selected sets as a bit mask per query (512 bytes each)
            sel = torch.zeros(1, queries, keys, dtype=torch.bool)
            sel.scatter_(2, scores.topk(topk, dim=-1)[1], True)
            small["idx_decode.kth_score"] = scores.topk(topk, dim=-1)[0][..., -1].clone()
            small["idx_decode.score_sum_selected"] = (scores * sel).sum(-1)
            hashes["idx_decode.selected_mask"] = sha(sel.to(torch.uint8))

    # ---- indexer prologue of the key path: LayerNorm + non-interleaved RoPE (deepseek.py:665-670)
    k_in = I.randn((9, 1, 128), I.SEED + 710)
    ln = rm.LayerNorm(128)
    with torch.no_grad():
        ln.weight.copy_(I.randn((128,), I.SEED + 711, mean=1.0, std=0.02, dtype=torch.float32))
        ln.bias.copy_(I.randn((128,), I.SEED + 712, std=0.02, dtype=torch.float32))
        k_ln = ln(k_in)
        k_pe, k_nope = torch.split(k_ln, [64, 64], dim=-1)
        fc = rm.precompute_freqs_cis(rm.ModelArgs())[:9]
        k_pe = rm.apply_rotary_emb(k_pe.unsqueeze(0), fc, False).squeeze(0)
    small["idxprep.k_ln_rope"] = torch.cat([k_pe, k_nope], dim=-1).clone()

    # ---- MLA.forward, decode branch (deepseek.py:765-811), the indexer replaced by a fixed selection
    c = I.MLA_DECODE
    d = I.mla_decode_inputs()
    torch.set_default_dtype(torch.bfloat16)     # the model's caches take the default dtype (deepseek.py:1135)
    try:
        margs = rm.ModelArgs(max_batch_size=c["batch"], max_seq_len=c["max_len"], dim=c["dim"],
                             n_heads=c["heads"], q_lora_rank=c["q_lora"], kv_lora_rank=c["kv_lora"],
                             qk_nope_head_dim=c["nope"], qk_rope_head_dim=c["rope"],
                             v_head_dim=c["v_dim"])
        mla = rm.MLA(margs)
        picked = d["topk_indices"]

        class FixedSelection(torch.nn.Module):
            def forward(self, x, qr, start_pos, freqs_cis, mask):
                return picked

        mla.indexer = FixedSelection()
        with torch.no_grad():
            mla.wq_a.weight.copy_(d["w"]["wq_a"]); mla.q_norm.weight.copy_(d["w"]["q_norm"])
            mla.wq_b.weight.copy_(d["w"]["wq_b"]); mla.wkv_a.weight.copy_(d["w"]["wkv_a"])
            mla.kv_norm.weight.copy_(d["w"]["kv_norm"]); mla.wkv_b.weight.copy_(d["w"]["wkv_b"])
            mla.wo.weight.copy_(d["w"]["wo"])
            mla.kv_cache.copy_(d["kv_cache"]); mla.pe_cache.copy_(d["pe_cache"])
            fc = rm.precompute_freqs_cis(margs)[c["start_pos"]:c["start_pos"] + 1]
            y = mla(d["x"], c["start_pos"], fc, None)
        small["mla_decode.out"] = y.clone()
        small["mla_decode.kv_row"] = mla.kv_cache[:, c["start_pos"]].clone()
        small["mla_decode.pe_row"] = mla.pe_cache[:, c["start_pos"]].clone()
    finally:
        torch.set_default_dtype(torch.float32)

    make_layer_fixture(args.reference)

    meta = {"torch": torch.__version__, "cpu_capability": torch.backends.cpu.get_cpu_capability(),
            "threads": torch.get_num_threads()}
    torch.save(small, HERE / "golden_small.pt")
    (HERE / "golden_hashes.json").write_text(json.dumps({"meta": meta, "sha256": hashes}, indent=1,
                                                        sort_keys=True) + "\n")
    size = (HERE / "golden_small.pt").stat().st_size
    print(f"wrote {len(small)} tensors ({size/1024:.0f} KiB) and {len(hashes)} hashes; meta={meta}")


if __name__ == "__main__":
    main()
