"""Seeded synthetic inputs for the hot-path configurations.

TEST INFRASTRUCTURE ONLY (see ref_ops.py). All tensors are drawn on the CPU with a
``torch.Generator`` so that the golden-vector script, the CPU tests, the GPU parity tests
and the benchmark's CPU leg see identical values; GPU callers move them with ``.cuda()``.
Seed base 38595 is the one the reference uses for its DeepSeek-V3.2 shape
(racetrack/realistic_bench.py:80).
"""
from __future__ import annotations

import torch

SEED = 38595

# DeepSeek-V3.2 dimensions (racetrack/realistic_bench.py:62-82, racetrack/models/deepseek.py:199-272
# with the 671B values: benchmarks/common.py:25-54).
HIDDEN = 7168
Q_LORA = 1536
KV_LORA = 512
ROPE_DIM = 64
NOPE_DIM = 128
V_DIM = 128
N_HEADS = 128
N_EXPERTS = 256
N_GROUPS = 8
TOPK_GROUPS = 4
TOPK = 8
ROUTE_SCALE = 2.5
MOE_INTER = 2048
DENSE_INTER = 18432
EPS = 1e-6
ROPE_THETA = 10000.0


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def randn(shape, seed: int, *, mean: float = 0.0, std: float = 1.0,
          dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    t = torch.empty(shape, dtype=torch.float32)
    t.normal_(mean=mean, std=std, generator=_gen(seed))
    return t.to(dtype)


def uniform(shape, seed: int, lo: float, hi: float, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    t = torch.empty(shape, dtype=torch.float32)
    t.uniform_(lo, hi, generator=_gen(seed))
    return t.to(dtype)


def mla_prologue_inputs(tokens: int = 128, *, hidden: int = HIDDEN, q_lora: int = Q_LORA,
                        kv_lora: int = KV_LORA, heads: int = N_HEADS, rope_dim: int = ROPE_DIM,
                        dtype: torch.dtype = torch.bfloat16, seed: int = SEED) -> dict:
    """Fused MLA prologue: x/residual [T, hidden] ~ N(0,1); norm weights ~ N(1, 0.02) fp32;
    q_c / kv_c / k_pe are column slices of one [T, q_lora + kv_lora + rope_dim] buffer, as in
    partitions/dsv3_2/model.py:316-319; q_pe [T, heads, rope_dim]; positions 0..T-1."""
    qkv = randn((tokens, q_lora + kv_lora + rope_dim), seed + 3, dtype=dtype)
    return {
        "x": randn((tokens, hidden), seed + 1, dtype=dtype),
        "residual": randn((tokens, hidden), seed + 2, dtype=dtype),
        "w_attn": randn((hidden,), seed + 4, mean=1.0, std=0.02, dtype=torch.float32),
        "qkv": qkv,
        "q_c": qkv[:, :q_lora],
        "kv_c": qkv[:, q_lora:q_lora + kv_lora],
        "k_pe": qkv[:, q_lora + kv_lora:],
        "w_q": randn((q_lora,), seed + 5, mean=1.0, std=0.02, dtype=torch.float32),
        "w_kv": randn((kv_lora,), seed + 6, mean=1.0, std=0.02, dtype=torch.float32),
        "q_pe": randn((tokens, heads, rope_dim), seed + 7, dtype=dtype),
        "positions": torch.arange(tokens, dtype=torch.int64),
        "eps": EPS,
        "rope_theta": ROPE_THETA,
    }


def swiglu_quant_inputs(tokens: int = 4096, inter: int = DENSE_INTER, *, seed: int = SEED,
                        dtype: torch.dtype = torch.bfloat16) -> dict:
    """gate_up [T, 2*inter] ~ N(0,1); gate = first half of the columns."""
    gate_up = randn((tokens, 2 * inter), seed + 11, dtype=dtype)
    return {"gate_up": gate_up, "gate": gate_up[:, :inter], "up": gate_up[:, inter:]}


def gate_inputs(tokens: int = 4096, *, hidden: int = HIDDEN, n_experts: int = N_EXPERTS,
                seed: int = SEED, dtype: torch.dtype = torch.bfloat16) -> dict:
    """Router inputs: hidden ~ N(0,1), gate weight ~ N(0, 0.02), bias ~ U(-0.1, 0.1) fp32."""
    return {
        "hidden": randn((tokens, hidden), seed + 21, dtype=dtype),
        "w_gate": randn((n_experts, hidden), seed + 100000, std=0.02, dtype=dtype),
        "bias": uniform((n_experts,), seed + 22, -0.1, 0.1),
        "n_groups": N_GROUPS, "topk_groups": TOPK_GROUPS, "topk": TOPK,
        "route_scale": ROUTE_SCALE,
    }


INDEX_HEADS = 64
INDEX_DIM = 128
INDEX_TOPK = 2048


def indexer_inputs(queries: int, keys: int, *, heads: int = INDEX_HEADS, dim: int = INDEX_DIM,
                   seed: int = SEED) -> dict:
    """Operands of the sparse indexer's scoring step as the reference forms them
    (racetrack/models/deepseek.py:671-680): q [1, m, h, d] and k [1, n, d] N(0, 1) quantised
    per 128 to e4m3 (one group per head / key), weights = N(0, 1) * h^-0.5 * q_scale * d^-0.5."""
    from . import ref_ops as R
    q = randn((1, queries, heads, dim), seed + 700)
    k = randn((1, keys, dim), seed + 701)
    q_fp8, q_scale = R.act_quant(q)                       # scales [1, m, h, 1]
    k_fp8, k_scale = R.act_quant(k)                       # scales [1, n, 1]
    w = randn((1, queries, heads), seed + 702, dtype=torch.float32) * heads ** -0.5
    weights = (w.unsqueeze(-1) * q_scale * dim ** -0.5).squeeze(-1)
    return {"q": q_fp8, "weights": weights.contiguous(), "k": k_fp8,
            "k_scale": k_scale.squeeze(-1).contiguous()}


def expert_weights(n_experts: int, hidden: int, inter: int, *, seed: int = SEED,
                   dtype: torch.dtype = torch.bfloat16):
    """[(w1 [inter, hidden], w2 [hidden, inter], w3 [inter, hidden])] ~ N(0, 0.02)."""
    out = []
    for e in range(n_experts):
        out.append((randn((inter, hidden), seed + 1000 + 3 * e, std=0.02, dtype=dtype),
                    randn((hidden, inter), seed + 1001 + 3 * e, std=0.02, dtype=dtype),
                    randn((inter, hidden), seed + 1002 + 3 * e, std=0.02, dtype=dtype)))
    return out


MLA_DECODE = dict(dim=256, heads=4, q_lora=64, kv_lora=64, nope=32, rope=16, v_dim=32, batch=2,
                  max_len=64, start_pos=40, topk=16)


def mla_decode_inputs(seed: int = SEED) -> dict:
    """A small MLA module in decode mode (racetrack/models/deepseek.py:697-811): weights, the
    token of each of `batch` sequences, caches holding `start_pos` earlier positions ~ N(0, 1)
    and the positions the indexer is taken to have selected."""
    c = MLA_DECODE
    b, L = c["batch"], c["max_len"]
    w = {"wq_a": randn((c["q_lora"], c["dim"]), seed + 800, std=0.06),
         "q_norm": randn((c["q_lora"],), seed + 801, mean=1.0, std=0.02, dtype=torch.float32),
         "wq_b": randn((c["heads"] * (c["nope"] + c["rope"]), c["q_lora"]), seed + 802, std=0.12),
         "wkv_a": randn((c["kv_lora"] + c["rope"], c["dim"]), seed + 803, std=0.06),
         "kv_norm": randn((c["kv_lora"],), seed + 804, mean=1.0, std=0.02, dtype=torch.float32),
         "wkv_b": randn((c["heads"] * (c["nope"] + c["v_dim"]), c["kv_lora"]), seed + 805, std=0.12),
         "wo": randn((c["dim"], c["heads"] * c["v_dim"]), seed + 806, std=0.09)}
    kv_cache = torch.zeros(b, L, c["kv_lora"], dtype=torch.bfloat16)
    pe_cache = torch.zeros(b, L, c["rope"], dtype=torch.bfloat16)
    kv_cache[:, :c["start_pos"]] = randn((b, c["start_pos"], c["kv_lora"]), seed + 807)
    pe_cache[:, :c["start_pos"]] = randn((b, c["start_pos"], c["rope"]), seed + 808)
    g = _gen(seed + 809)
    topk = torch.stack([torch.randperm(c["start_pos"] + 1, generator=g)[:c["topk"]] for _ in range(b)])
    return {"w": w, "x": randn((b, 1, c["dim"]), seed + 810), "kv_cache": kv_cache,
            "pe_cache": pe_cache, "topk_indices": topk.view(b, 1, c["topk"])}
