PARTITION_NOTES = 'B200 kernels for the MLA prologue of the NVFP4 model: residual_norm + qkv_a / indexer-k projection, indexer key path, q_b / absorbed-q / indexer-q projections with index scores and top-k, q_pe RoPE; plus residual_norm, swiglu, full-top-k indexer and routed MoE on NVFP4 grouped GEMMs'

GRAPH_NODES = {
    "fused_ar_rms_qkv_proj": ["attn_residual_add", "attn_rms", "qkv_a_proj", "indexer_k_proj"],
    "fused_indexer_k_path": ["indexer_ln", "indexer_rope", "indexer_hadamard", "indexer_quant_fp8", "indexer_cache"],
    "fused_q_indexer_score": ["q_b_proj", "w_uk_t", "indexer_q_proj", "indexer_q_rope", "indexer_q_fp8",
                              "indexer_w", "indexer_mqa", "logits_topk"],
    "fused_q_rope_quant": ["q_rope"],
    "fused_full_topk_indexer": ["indexer_mqa", "logits_topk", "topk_page_idx"],
    "fused_single_token_moe": ["gate_router", "topk_softmax", "expert_sum"],
    "fused_residual_norm": ["attn_residual_add", "ffn_rms"],
    "fused_swiglu": ["ffn_silu", "ffn_gate_up_mul"],
}

FUSED_OPS = [
    {"name": "fused_swiglu", "kind": "fx_pattern"},
    {"name": "fused_residual_norm", "kind": "fx_pattern"},
    {"name": "fused_full_topk_indexer", "kind": "pre_trace"},
    {"name": "fused_single_token_moe", "kind": "pre_trace"},
    {"name": "fused_ar_rms_qkv_proj", "kind": "module_patch"},
    {"name": "fused_indexer_k_path", "kind": "module_patch"},
    {"name": "fused_q_indexer_score", "kind": "module_patch"},
    {"name": "fused_q_rope_quant", "kind": "module_patch"},
]
