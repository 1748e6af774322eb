"""Synthetic full-size DeepSeek-V3.2 layer on the B200 kernels: the counterpart of
racetrack/realistic_bench.py:118-427 (ShardedRealisticBlock / ShardedRealisticModel).

Same structure and sharding as the reference runner: one layer's weights reused for every layer
of the stack; attention heads tensor-parallel (w_q_b / w_kv_b column-sharded, w_o row-sharded);
routed experts expert-parallel (each rank owns a contiguous slice). The reference replicates all
tokens and all-reduces the partial sums twice per layer (racetrack/realistic_bench.py:315-316,
351); here each all-reduce is split into its two halves with the token-wise work in between:

    partial sums [T, H]  --reduce-scatter-->  this rank's T / world rows of the sum
    residual add + RMSNorm, qkv_a projection / router + routing + NVFP4 quantisation on those rows
    --all-gather-->  every rank holds the [T, 2112] latent projection / the NVFP4 codes, scales
    and routing of all tokens (0.3 / 0.56 bytes per hidden element instead of 2)

so nothing token-wise is computed world times and less than half the bytes cross NVLink; the sums
are the same sums (`token_sharded=False` keeps the reference's replicated schedule). When the
caller also provides the WHOLE output projection (`w_o_full`), the attention half needs no
reduction at all: the heads' attention outputs change hands (every rank collects all heads for
its own rows, as FP8 codes + scales when w_o is FP8) and w_o is applied to a rank's rows over all
heads, which is the single-GPU computation of those rows. Per layer:

    rms_norm -> qkv_a GEMM -> fused q_a/kv_a RMSNorm + k_pe RoPE -> q_b GEMM -> q_pe RoPE (in place)
    -> kv_b GEMM -> causal attention over the local heads (tcgen05) -> w_o GEMM -> all-reduce
    -> fused residual-add + rms_norm -> router GEMM (fp32) -> routing kernel -> NVFP4 grouped
    expert GEMMs with SwiGLU -> weighted combine -> all-reduce -> residual add (fused with the
    next layer's first rms_norm)

Dense projections run on the bf16 tcgen05 GEMM, experts on the NVFP4 block-scaled grouped GEMM,
everything element-wise on the fused kernels of ops.py, the attention core (QK^T, softmax, PV) on
the causal attention kernel of this library (ops.attention_prefill).

Unlike the reference, which seeds each rank's weights with seed + rank (so a 2-rank model is a
different model from a 1-rank one), weights here are defined per shard unit (one eighth of the
heads, one expert) and a rank draws the units it owns: every world size computes the same layer.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import torch
import torch.nn.functional as F

from . import comm, moe, ops


@dataclass(frozen=True)
class LayerShape:
    """Dimensions of racetrack/realistic_bench.py:62-82 (realistic_shape("dsv3_2"))."""
    name: str = "dsv3_2"
    hidden: int = 7168
    heads: int = 128
    q_lora: int = 1536
    kv_lora: int = 512
    nope: int = 128
    rope: int = 64
    v_dim: int = 128
    moe_inter: int = 2048
    n_experts: int = 256
    topk: int = 8
    dense_inter: int = 18432
    eps: float = 1.0e-6
    rope_base: float = 10000.0
    seed: int = 38595
    units: int = 8           # shard granularity of heads and of the dense FFN

    @property
    def qk_dim(self) -> int:
        return self.nope + self.rope

    def scaled(self, **kw) -> "LayerShape":
        return replace(self, **kw)


DSV32 = LayerShape()


def _draw(shape, seed: int, std: float, device, dtype) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    w = torch.empty(shape, device=device, dtype=torch.float32 if str(device) == "cpu" else dtype)
    w.normal_(mean=0.0, std=std, generator=g)
    return w.to(dtype)


def draw_expert(shape: LayerShape, e: int, device, *, std: float = 0.02,
                dtype: torch.dtype = torch.bfloat16):
    """(w13 [2I, H], w2 [H, I]) of routed expert `e`; the same values whatever rank draws them."""
    s = shape
    return (_draw((2 * s.moe_inter, s.hidden), s.seed + 10000 + 2 * e, std, device, dtype),
            _draw((s.hidden, s.moe_inter), s.seed + 10001 + 2 * e, std, device, dtype))


def make_weights(shape: LayerShape, rank: int, world: int, device, *, ffn: str = "moe",
                 std: float = 0.02, dtype: torch.dtype = torch.bfloat16, full_w_o: bool = False) -> dict:
    """The weights rank `rank` of `world` owns, drawn unit by unit (see the module docstring).
    Keys: w_qkv_a [q+kv+rope, H]; w_q_b [h_loc*(nope+rope), q]; w_kv_b [h_loc*(nope+v), kv];
    w_o [H, h_loc*v]; w_gate [E, H]; w13 [E_loc, 2I, H], w2 [E_loc, H, I] (ffn == "moe") or
    w1, w3 [I_loc, H], w2d [H, I_loc] (ffn == "dense")."""
    if shape.units % world or shape.n_experts % world:
        raise ValueError("world size must divide the shard units and the expert count")
    s = shape
    hpu = s.heads // s.units                     # heads per unit
    units = range(rank * s.units // world, (rank + 1) * s.units // world)
    seed = s.seed
    w = {"w_qkv_a": _draw((s.q_lora + s.kv_lora + s.rope, s.hidden), seed + 1, std, device, dtype),
         "w_gate": _draw((s.n_experts, s.hidden), seed + 100000, std, device, dtype)}
    w["w_q_b"] = torch.cat([_draw((hpu * s.qk_dim, s.q_lora), seed + 100 + u, std, device, dtype)
                            for u in units])
    w["w_kv_b"] = torch.cat([_draw((hpu * (s.nope + s.v_dim), s.kv_lora), seed + 200 + u, std, device, dtype)
                             for u in units])
    w["w_o"] = torch.cat([_draw((s.hidden, hpu * s.v_dim), seed + 300 + u, std, device, dtype)
                          for u in units], dim=1)
    if full_w_o and world > 1:
        # every unit's columns: the whole output projection, for the schedule that applies it to a
        # rank's own token rows after exchanging the heads' attention outputs (RealisticLayer)
        w["w_o_full"] = torch.cat([_draw((s.hidden, hpu * s.v_dim), seed + 300 + u, std, device, dtype)
                                   for u in range(s.units)], dim=1)
    if ffn == "moe":
        e_loc = s.n_experts // world
        experts = [draw_expert(s, e, device, std=std, dtype=dtype)
                   for e in range(rank * e_loc, (rank + 1) * e_loc)]
        w["w13"] = torch.stack([e[0] for e in experts])
        w["w2"] = torch.stack([e[1] for e in experts])
    elif ffn == "dense":
        ipu = s.dense_inter // s.units
        w["w1"] = torch.cat([_draw((ipu, s.hidden), seed + 400 + u, std, device, dtype) for u in units])
        w["w3"] = torch.cat([_draw((ipu, s.hidden), seed + 500 + u, std, device, dtype) for u in units])
        w["w2d"] = torch.cat([_draw((s.hidden, ipu), seed + 600 + u, std, device, dtype) for u in units], dim=1)
    return w


def make_nvfp4_experts(shape: LayerShape, rank: int, world: int, device, *,
                       std: float = 0.02, moe_tp: int = 1) -> "moe.NVFP4Experts":
    """The rank's routed experts drawn and quantised one at a time, so that the bf16 weights of
    only one expert exist at any moment (all 256 experts in bf16 would take 22.5 GB).

    moe_tp > 1 makes the expert split a hybrid: the ranks form world / moe_tp expert-parallel
    groups of moe_tp ranks (rank = group * moe_tp + member); a group owns a contiguous block of
    experts and member m holds columns [m, m + 1) * inter / moe_tp of every one of them (the
    matching rows of w1 and w3, the matching K range of w2). The quantised weights are those of
    the whole expert, cut afterwards (same codes, block scales and global scale at every world
    size); the members' partial sums add up in the reduction that follows the experts anyway.
    A group's load is the sum over more experts, so a router that favours a few experts leaves
    the groups less out of balance than single ranks would be."""
    s = shape
    if world % moe_tp or s.n_experts % (world // moe_tp) or s.moe_inter % (256 * moe_tp):
        raise ValueError("moe_tp must divide the world size and leave inter / moe_tp a multiple of 256")
    group, member = divmod(rank, moe_tp)
    e_loc = s.n_experts // (world // moe_tp)
    inter = s.moe_inter // moe_tp
    parts13, parts2 = [], []
    for e in range(group * e_loc, (group + 1) * e_loc):
        w13, w2 = draw_expert(s, e, device, std=std)
        c13, sf13, gs13 = ops.fused_nvfp4_quant(w13, tiled_scales=True)
        c2, sf2, gs2 = ops.fused_nvfp4_quant(w2, tiled_scales=True)
        if moe_tp > 1:
            rows = slice(member * inter, (member + 1) * inter)
            # w13 = [w1; w3]: the member's rows of each; scale tiles are 128 rows x 4 blocks of 16
            # elements, ordered (row tile, K tile)
            c13 = c13.view(2, s.moe_inter, -1)[:, rows].reshape(2 * inter, -1).contiguous()
            t13 = sf13.view(torch.uint8).view(2, s.moe_inter // 128, -1, 512)
            sf13 = t13[:, member * inter // 128:(member + 1) * inter // 128].reshape(-1).contiguous()
            # w2 [H, I]: the member's K range (bytes hold two elements, a K tile 64 of them)
            c2 = c2[:, member * inter // 2:(member + 1) * inter // 2].contiguous()
            t2 = sf2.view(torch.uint8).view(-1, s.moe_inter // 64, 512)
            sf2 = t2[:, member * inter // 64:(member + 1) * inter // 64].reshape(-1).contiguous()
        parts13.append((c13, sf13, gs13))
        parts2.append((c2, sf2, gs2))
    cat = torch.cat
    return moe.NVFP4Experts(
        e_loc, s.hidden, inter,
        cat([p[0] for p in parts13]), cat([p[1].view(torch.uint8) for p in parts13]),
        cat([p[2] for p in parts13]),
        cat([p[0] for p in parts2]), cat([p[1].view(torch.uint8) for p in parts2]),
        cat([p[2] for p in parts2]))


# "rt": the causal attention kernel of this library (ops.attention_prefill, tcgen05);
# "sdpa": torch's scaled_dot_product_attention, kept only as the yardstick the kernel is
# measured against (a library kernel, not part of the backend).
ATTENTION_CORE = "rt"


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Causal softmax(q k^T / sqrt(d)) v over [T, H, D] tensors -> [T, H, Dv]
    (racetrack/runtime/torch_ops.py:97-110) through torch SDPA (the yardstick, see
    ATTENTION_CORE); when the value width differs from the query width and the fused kernels
    refuse that, v is zero-padded to the query width."""
    qt, kt, vt = (t.transpose(0, 1).unsqueeze(0) for t in (q, k, v))
    try:
        out = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
    except RuntimeError:
        pad = q.shape[-1] - v.shape[-1]
        out = F.scaled_dot_product_attention(qt, kt, F.pad(vt, (0, pad)), is_causal=True)[..., :v.shape[-1]]
    return out.squeeze(0).transpose(0, 1)


class Projection:
    """A dense projection y = x W^T held either in bf16 or as FP8 e4m3 with 128 x 128 block
    scales (racetrack/models/deepseek.py:316-345 `linear`: bf16 weights go to F.linear, FP8
    weights to act_quant + fp8_gemm). FP8 needs K % 128 == 0; other widths stay bf16.
    dtype "mixed" keeps FP8 for the long reductions only (K >= MIXED_FP8_MIN_K): the FP8 GEMM
    rescales every 128-wide K block in registers, which pays off against the bf16 CTA-pair
    GEMM only when the tensor core has long K loops to hide it behind."""

    MIXED_FP8_MIN_K = 4096

    def __init__(self, weight: torch.Tensor, dtype: str):
        k = weight.shape[1]
        self.out_features = weight.shape[0]
        self.fp8 = k % 128 == 0 and (dtype == "fp8" or (dtype == "mixed" and k >= self.MIXED_FP8_MIN_K))
        if self.fp8:
            self.codes, self.scales = ops.quantize_weight_fp8(weight)
        else:
            self.weight = weight.contiguous()

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.fp8:
            return ops.linear_fp8_act(x, self.codes, self.scales, out=out)
        return ops.linear_bf16(x, self.weight, out=out)


class RealisticLayer:
    """One rank's shard of the synthetic layer; `forward_stack` applies it `layers` times.
    proj = "bf16" | "fp8" | "mixed" selects the arithmetic of the dense projections."""

    def __init__(self, shape: LayerShape, weights: dict, rank: int = 0, world: int = 1, *,
                 ffn: str = "moe", route: str = "topk_softmax", proj: str = "bf16",
                 process_group=None, token_sharded: bool = True, peer_reduce: bool = True):
        self.shape, self.rank, self.world, self.ffn, self.route = shape, rank, world, ffn, route
        self.group, self.proj = process_group, proj
        self.token_sharded = token_sharded
        # reduce-scatter by peer loads over NVLink fused into the residual-add + RMSNorm kernel
        # (False: NCCL reduce-scatter, then the plain kernel)
        self.peer_reduce = peer_reduce
        self._peer: dict = {}
        self._comm = None
        self.local_heads = shape.heads // world
        dev = weights["w_qkv_a"].device
        self.w_qkv_a = Projection(weights["w_qkv_a"], proj)
        self.w_q_b = Projection(weights["w_q_b"], proj)
        s = shape
        self.attn_core = ATTENTION_CORE
        if self.attn_core == "rt":
            # K and V are column slices of the kv_b output; the attention kernel takes the
            # rope key as an operand of its own, one row per token for all heads
            self.w_kv_b = Projection(weights["w_kv_b"], proj)
        else:
            # kv_b rows regrouped per head as [k_nope | rope-wide gap (zero rows) | v]: the GEMM
            # then leaves room for k_pe right behind k_nope (a whole-key tensor for SDPA)
            wkv = weights["w_kv_b"].view(self.local_heads, s.nope + s.v_dim, s.kv_lora)
            gap = torch.zeros(self.local_heads, s.rope, s.kv_lora, device=dev, dtype=wkv.dtype)
            self.w_kv_b = Projection(
                torch.cat((wkv[:, :s.nope], gap, wkv[:, s.nope:]), dim=1)
                .reshape(self.local_heads * (s.nope + s.rope + s.v_dim), s.kv_lora), proj)
        self.w_o = Projection(weights["w_o"], proj)
        # the whole output projection (all heads' columns), when the caller provides it: the
        # token-sharded schedule then exchanges attention outputs instead of reducing w_o's
        self.w_o_full = Projection(weights["w_o_full"], proj) if "w_o_full" in weights and world > 1 else None
        self.w_gate = weights["w_gate"].contiguous()
        self.ones_h = torch.ones(shape.hidden, device=dev, dtype=torch.bfloat16)
        self.q_norm = torch.ones(shape.q_lora, device=dev, dtype=torch.bfloat16)
        self.kv_norm = torch.ones(shape.kv_lora, device=dev, dtype=torch.bfloat16)
        if ffn == "moe":
            self.experts = weights["experts"] if "experts" in weights else \
                moe.quantize_experts(weights["w13"], weights["w2"])
            # experts cut along their intermediate dimension (make_nvfp4_experts, moe_tp) shrink
            # the expert-parallel degree: world / moe_tp groups of consecutive ranks
            self.moe_tp = max(1, shape.moe_inter // self.experts.inter)
            self.local_experts = shape.n_experts // (world // self.moe_tp)
            self.expert_begin = (rank // self.moe_tp) * self.local_experts
        else:
            self.w13d = Projection(torch.cat([weights["w1"], weights["w3"]]), proj)
            self.w2d = Projection(weights["w2d"], proj)

    # -- pieces ---------------------------------------------------------------------------
    reduce = True   # set False to get this rank's partial sums (single-process checks)

    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1 and self.reduce:
            self.comm.all_reduce_sum(t)
        return t

    @property
    def comm(self) -> "comm.Group":
        if self._comm is None:
            self._comm = comm.Group(self.rank, self.world if self.reduce else 1, self.group)
        return self._comm

    def attention(self, normed: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """racetrack/realistic_bench.py:286-317: all tokens in, all-reduced [T, H] out."""
        return self._all_reduce(self.attention_partial(self.w_qkv_a(normed), positions))

    def attention_partial(self, qkv: torch.Tensor, positions: torch.Tensor,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """From the latent projection qkv [T, q_lora + kv_lora + rope] of ALL tokens to this
        rank's partial sum of the attention output (its heads' share of w_o), written into `out`
        when given (a buffer the other ranks read)."""
        if self.w_o.fp8 and self.attn_core == "rt":
            # the attention kernel writes the FP8 codes + scales the output projection consumes
            codes, scales = self.attention_heads(qkv, positions, quantized=True)
            return ops.linear_fp8(codes, scales, self.w_o.codes, self.w_o.scales, out=out)
        local = self.attention_heads(qkv, positions)
        return self.w_o(local, out=out)

    def attention_heads(self, qkv: torch.Tensor, positions: torch.Tensor, quantized: bool = False,
                        out: Optional[tuple] = None):
        """From the latent projection of ALL tokens to the attention output of this rank's heads,
        [T, local_heads * v_dim] (what w_o consumes); quantized=True: as FP8 codes + scales
        (act_quant of it), written into `out` when given."""
        s, h = self.shape, self.local_heads
        tokens = qkv.shape[0]
        q_c, kv_c, k_pe = ops.fused_norm_rope(
            qkv[:, :s.q_lora], self.q_norm, qkv[:, s.q_lora:s.q_lora + s.kv_lora], self.kv_norm,
            qkv[:, s.q_lora + s.kv_lora:], positions, eps=s.eps, rope_base=s.rope_base)
        q = self.w_q_b(q_c).view(tokens, h, s.qk_dim)
        ops.fused_rope_half(q[..., s.nope:], positions, rope_base=s.rope_base, inplace=True)
        if self.attn_core == "rt":
            kv = self.w_kv_b(kv_c).view(tokens, h, s.nope + s.v_dim)
            if quantized:
                return ops.attention_prefill(q, kv[..., :s.nope], k_pe, kv[..., s.nope:], quantized=True, out=out)
            local = ops.attention_prefill(q, kv[..., :s.nope], k_pe, kv[..., s.nope:])
        else:
            kv = self.w_kv_b(kv_c).view(tokens, h, s.qk_dim + s.v_dim)
            ops.head_broadcast_(kv[..., s.nope:s.qk_dim], k_pe)       # K = [k_nope | k_pe] in place
            local = attention_core(q, kv[..., :s.qk_dim], kv[..., s.qk_dim:])
        local = local.reshape(tokens, h * s.v_dim)
        return ops.fused_act_quant(local, out=out) if quantized else local

    def attention_rows_from_heads(self, px, heads_out: Optional[torch.Tensor], lo: int, hi: int) -> torch.Tensor:
        """The output projection of this rank's token rows [lo, hi) over ALL heads: the heads'
        attention outputs are exchanged (as FP8 codes + scales when w_o is FP8: a 128-wide
        quantisation group is one head's v_dim columns and never spans two ranks, so each rank
        quantises its own columns exactly as the whole row would be) and the whole w_o is applied
        locally. The sum over heads happens inside one GEMM, as on a single GPU; nothing is
        reduced across ranks."""
        if self.w_o_full.fp8:
            if heads_out is not None:      # else the attention kernel wrote the exchange buffers itself
                ops.fused_act_quant(heads_out, out=(px.local["ao_codes"], px.local["ao_scales"]))
            codes, scales = px.gather_cols(("ao_codes", "ao_scales"), lo, hi - lo)
            return ops.linear_fp8(codes.view(torch.float8_e4m3fn), scales, self.w_o_full.codes,
                                  self.w_o_full.scales)
        px.local["ao"].copy_(heads_out)
        (rows,) = px.gather_cols(("ao",), lo, hi - lo)
        return ops.linear_bf16(rows, self.w_o_full.weight)

    def _route(self, normed: torch.Tensor, out: Optional[tuple] = None):
        """Router of racetrack/realistic_bench.py:321-327 for the given rows: fp32 logits of bf16
        operands (tensor cores, fp32 accumulators kept), top-k, softmax over the k logits."""
        logits = ops.linear_bf16(normed, self.w_gate, out_dtype=torch.float32)
        if self.route != "topk_softmax":
            raise ValueError(f"unknown route {self.route!r}")
        return ops.fused_moe_route(logits, None, n_groups=1, topk_groups=1, topk=self.shape.topk,
                                   route_scale=1.0, score_func="topk_softmax", out=out)

    def ffn_forward(self, normed: torch.Tensor) -> torch.Tensor:
        """racetrack/realistic_bench.py:319-352 (routed experts) or a dense SwiGLU FFN."""
        return self._all_reduce(self.ffn_partial(normed))

    def ffn_partial(self, normed: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The feed-forward half on all tokens, this rank's partial sum (its experts / its FFN
        columns), written into `out` when given (a buffer the other ranks read)."""
        s = self.shape
        if self.ffn == "moe":
            weights, indices = self._route(normed)
            return moe.fused_moe_experts(normed, weights, indices, self.experts,
                                         n_experts=s.n_experts,
                                         expert_begin=self.expert_begin, out=out)
        gate_up = self.w13d(normed)
        inter = gate_up.shape[1] // 2
        if self.w2d.fp8:     # SwiGLU and the FP8 quantisation of its result in one kernel
            codes, scales = ops.fused_swiglu_quant(gate_up[:, :inter], gate_up[:, inter:])
            return ops.linear_fp8(codes, scales, self.w2d.codes, self.w2d.scales, out=out)
        return self.w2d(ops.fused_swiglu(gate_up[:, :inter], gate_up[:, inter:]), out=out)

    def ffn_partial_from_rows(self, normed_rows: torch.Tensor, out: Optional[torch.Tensor] = None,
                              px=None) -> torch.Tensor:
        """Token-sharded feed-forward half: `normed_rows` are this rank's T / world rows of the
        normalised hidden states; returns this rank's partial sum [T, H] over ALL tokens (its
        experts' / its FFN columns' share). Routing and quantisation run on the rank's rows, their
        compact results are all-gathered: NVFP4 codes + block scales + routing (MoE) or FP8 codes +
        scales (dense FFN with FP8 weights) instead of bf16 hidden states."""
        s, c = self.shape, self.comm
        if self.ffn == "moe":
            # one tensor-wide NVFP4 scale whatever the world size: the maximum over all ranks' rows
            if px is not None:
                amax = px.allmax("amax", ops.tensor_absmax(normed_rows))
            else:
                amax = c.all_reduce_max(ops.tensor_absmax(normed_rows))
            if px is not None:
                # routing and quantisation write this rank's rows of the exchange buffers; one
                # device barrier and one kernel then pull the other ranks' rows over NVLink
                lo, hi = c.rows_of(px.local["moe_codes"].shape[0])
                self._route(normed_rows, out=(px.local["moe_w"][lo:hi], px.local["moe_i"][lo:hi]))
                _, _, gs = ops.fused_nvfp4_quant(normed_rows, amax=amax,
                                                 out=(px.local["moe_codes"][lo:hi], px.local["moe_sf"][lo:hi]))
                px.gather("moe_codes", "moe_sf", "moe_w", "moe_i")
                codes, sf = px.local["moe_codes"], px.local["moe_sf"]
                weights, indices = px.local["moe_w"], px.local["moe_i"]
            else:
                weights, indices = self._route(normed_rows)
                codes, sf, gs = ops.fused_nvfp4_quant(normed_rows, amax=amax)
                codes, sf = c.all_gather_rows(codes), c.all_gather_rows(sf.view(torch.uint8))
                weights, indices = c.all_gather_rows(weights), c.all_gather_rows(indices)
            return moe.fused_moe_experts(None, weights, indices, self.experts, n_experts=s.n_experts,
                                         expert_begin=self.expert_begin,
                                         x_quant=(codes, sf, gs), out=out)
        if self.w13d.fp8:
            codes, scales = ops.fused_act_quant(normed_rows)
            gate_up = ops.linear_fp8(c.all_gather_rows(codes), c.all_gather_rows(scales),
                                     self.w13d.codes, self.w13d.scales)
        else:
            gate_up = ops.linear_bf16(c.all_gather_rows(normed_rows), self.w13d.weight)
        inter = gate_up.shape[1] // 2
        if self.w2d.fp8:
            codes, scales = ops.fused_swiglu_quant(gate_up[:, :inter], gate_up[:, inter:])
            return ops.linear_fp8(codes, scales, self.w2d.codes, self.w2d.scales, out=out)
        return self.w2d(ops.fused_swiglu(gate_up[:, :inter], gate_up[:, inter:]), out=out)

    # -- the stack ----------------------------------------------------------------------------
    def forward_stack(self, hidden: torch.Tensor, positions: torch.Tensor, layers: int) -> torch.Tensor:
        """hidden [T, H] bf16 -> hidden after `layers` applications of the layer
        (racetrack/realistic_bench.py:354-389,420-423)."""
        if self.world > 1 and self.reduce and self.token_sharded and hidden.shape[0] % self.world == 0:
            return self._forward_stack_token_sharded(hidden, positions, layers)
        s = self.shape
        normed = ops.fused_rms_norm(hidden, self.ones_h, eps=s.eps)
        for layer in range(layers):
            attn = self.attention(normed, positions)
            normed, hidden = ops.fused_residual_norm(attn, hidden, self.ones_h, eps=s.eps)
            ffn = self.ffn_forward(normed)
            # the add closing this layer and the rms_norm opening the next one, in one pass
            normed, hidden = ops.fused_residual_norm(ffn, hidden, self.ones_h, eps=s.eps)
        return hidden

    def _forward_stack_token_sharded(self, hidden: torch.Tensor, positions: torch.Tensor,
                                     layers: int) -> torch.Tensor:
        """The same stack on more than one rank with every all-reduce split into reduce-scatter
        and all-gather around the token-wise kernels (module docstring): between the two sharded
        halves of a layer a rank holds only its own T / world rows of the hidden states."""
        s, c = self.shape, self.comm
        tokens = hidden.shape[0]
        lo, hi = c.rows_of(tokens)
        mine = hidden[lo:hi].contiguous()
        normed = ops.fused_rms_norm(mine, self.ones_h, eps=s.eps)
        px = self._peer_exchange(tokens) if self.peer_reduce and hidden.is_cuda else None
        for _ in range(layers):
            if px is not None:
                # every exchange goes through buffers the other ranks have mapped. All-gather: the
                # latent projection ([T, 2112]: 0.3 of a hidden row) lands in this rank's rows of
                # its copy and the peers' rows are pulled over NVLink. Reduce-scatter: the partial
                # sums stay where they are computed; reduce, residual add and RMSNorm are ONE
                # kernel that reads them from every rank.
                self.w_qkv_a(normed, out=px.local["qkv"][lo:hi])
                px.gather("qkv")
                if self.w_o_full is not None:
                    # the heads' outputs change hands, not w_o's partial sums: 1 / world of the bytes
                    # (half of that again in FP8), and this half of the layer equals the single-GPU
                    # evaluation bit for bit
                    if self.w_o_full.fp8:
                        self.attention_heads(px.local["qkv"], positions, quantized=True,
                                             out=(px.local["ao_codes"], px.local["ao_scales"]))
                        heads_out = None
                    else:
                        heads_out = self.attention_heads(px.local["qkv"], positions)
                    attn = self.attention_rows_from_heads(px, heads_out, lo, hi)
                    normed, mine = ops.fused_residual_norm(attn, mine, self.ones_h, eps=s.eps)
                else:
                    self.attention_partial(px.local["qkv"], positions, out=px.local["attn"])
                    normed, mine = px.reduce_residual_norm("attn", mine, self.ones_h, eps=s.eps)
                self.ffn_partial_from_rows(normed, out=px.local["ffn"],
                                           px=px if self.ffn == "moe" else None)
                normed, mine = px.reduce_residual_norm("ffn", mine, self.ones_h, eps=s.eps)
                continue
            qkv = c.all_gather_rows(self.w_qkv_a(normed))
            attn = c.reduce_scatter_rows(self.attention_partial(qkv, positions))
            normed, mine = ops.fused_residual_norm(attn, mine, self.ones_h, eps=s.eps)
            ffn = c.reduce_scatter_rows(self.ffn_partial_from_rows(normed))
            normed, mine = ops.fused_residual_norm(ffn, mine, self.ones_h, eps=s.eps)
        if px is not None:
            # the stack's result for all tokens: the ffn partial-sum buffer carries the final
            # all-gather (a rank overwrites only ITS rows of ITS copy, which nobody else reads in
            # the last reduce; the gather's barrier orders the writes before the pulls)
            px.local["ffn"][lo:hi].copy_(mine)
            px.gather("ffn")
            return px.local["ffn"].clone()
        return c.all_gather_rows(mine)

    def _peer_exchange(self, tokens: int):
        """The two [T, H] partial-sum buffers of this token count, mapped across the ranks once."""
        from . import peer
        px = self._peer.get(tokens)
        if px is None:
            s = self.shape
            shape = (tokens, s.hidden)
            buffers = {"ffn": (shape, torch.bfloat16),
                       "qkv": ((tokens, self.w_qkv_a.out_features), torch.bfloat16)}
            cols = self.local_heads * s.v_dim
            if self.w_o_full is None:
                buffers["attn"] = (shape, torch.bfloat16)
            elif self.w_o_full.fp8:
                buffers["ao_codes"] = ((tokens, cols), torch.uint8)
                buffers["ao_scales"] = ((tokens, cols // 128), torch.float32)
            else:
                buffers["ao"] = ((tokens, cols), torch.bfloat16)
            if self.ffn == "moe":
                buffers.update({"amax": ((4,), torch.float32),
                                "moe_codes": ((tokens, s.hidden // 2), torch.uint8),
                                "moe_sf": ((tokens, s.hidden // 16), torch.uint8),
                                "moe_w": ((tokens, s.topk), torch.float32),
                                "moe_i": ((tokens, s.topk), torch.int64)})
            px = peer.PeerExchange(self.comm, self.ones_h.device, buffers)
            self._peer[tokens] = px
        return px
