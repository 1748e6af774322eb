PARTITION_NOTES = 'B200 kernels: residual_norm + norm_rope + swiglu + act_quant (FP8 / NVFP4) + routed MoE on NVFP4 grouped GEMMs + gate-up proj + sparse-attention indexer'

GRAPH_NODES = {
    "fused_norm_rope": ["rms_norm_q", "rms_norm_kv", "rope_kpe"],
    "fused_residual_norm": ["res_add_attn", "ffn_norm"],
    "fused_swiglu": ["swiglu"],
    "fused_act_quant": ["act_quant"],
    "fused_single_token_moe": ["gate_router", "topk_softmax", "expert_sum"],
    "fused_mlp_gate_up_proj": ["w1_proj", "w3_proj"],
    "fused_full_topk_indexer": ["indexer_proj", "indexer_scores", "indexer_topk"],
}

FUSED_OPS = [
    {"name": "fused_norm_rope", "kind": "fx_pattern"},
    {"name": "fused_swiglu", "kind": "fx_pattern"},
    {"name": "fused_residual_norm", "kind": "fx_pattern"},
    {"name": "fused_act_quant", "kind": "fx_pattern"},
    {"name": "fused_single_token_moe", "kind": "pre_trace"},
    {"name": "fused_full_topk_indexer", "kind": "pre_trace"},
    {"name": "fused_mlp_gate_up_proj", "kind": "module_patch"},
]
