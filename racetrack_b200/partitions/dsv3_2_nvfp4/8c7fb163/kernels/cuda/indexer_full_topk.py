"""fused_full_topk_indexer on the B200 backend: Indexer.forward of
racetrack/models/deepseek.py:656-686 (projections, LayerNorm, non-interleaved RoPE, Hadamard
rotation, FP8 quantisation, cache append, index scores, top-k) on the kernels of this library.
Contract: racetrack/pre_trace.py:132-143 — (indexer, x, qr, start_pos, freqs_cis, mask, *,
fallback) -> int64 [bsz, seqlen, min(index_topk, end_pos)]; the patcher only calls it when the
context is longer than index_topk. The module's own caches are updated in place."""
import torch

from racetrack_b200 import _lib, indexer as rt_indexer

BACKEND_AVAILABLE = _lib.available()


def fused_full_topk_indexer(indexer, x, qr, start_pos, freqs_cis, mask, *, fallback):
    del fallback
    bsz, seqlen, _ = x.size()
    w = rt_indexer.weights_of_module(indexer)
    k_cache = indexer.k_cache[:bsz]
    k_scale = indexer.k_scale_cache[:bsz].view(bsz, -1)
    # freqs_cis is the slice of the table for positions [start_pos, start_pos + seqlen)
    if seqlen == 1:
        local = torch.zeros(bsz, device=x.device, dtype=torch.int64)
        picked = rt_indexer.indexer_decode(x[:, 0], qr[:, 0], w, k_cache, k_scale, start_pos, freqs_cis,
                                           indexer.index_topk, positions=local)
        picked = picked.long().unsqueeze(1)
    else:
        local = torch.arange(seqlen, device=x.device, dtype=torch.int64)
        rows = [rt_indexer.indexer_forward(x[b], qr[b], w, k_cache[b], k_scale[b], start_pos, freqs_cis,
                                           indexer.index_topk, causal=mask is not None, positions=local)
                for b in range(bsz)]
        picked = torch.stack(rows).long()
    # every rank computes the same scores from replicated inputs, but a split-K projection or
    # a different kernel schedule may round differently on a near tie: rank 0's selection wins,
    # as in the reference (racetrack/models/deepseek.py:684-685)
    dist = torch.distributed
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        picked = picked.contiguous()
        dist.broadcast(picked, src=0)
    return picked
