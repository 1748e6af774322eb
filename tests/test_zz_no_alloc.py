"""rt_moe_permute_static: the variant of the expert permutation for hosts that cannot give the
library scratch memory (a runtime that owns one pre-sized device arena and exposes no
allocator to plugins, or an operator signature with inputs and outputs only). Its histogram
scratch is a fixed array inside the library, so the call itself allocates nothing.

The test drives the C ABI directly and demands the same three outputs as rt_moe_permute (the
entry point with a caller workspace), exactly, on two calls in a row: the second call
reuses the array with the first call's contents still in it. The file name sorts last so a
run that stops at the first failure has already executed every other test.
"""
from __future__ import annotations

import pytest
import torch

from racetrack_b200 import _lib

pytestmark = pytest.mark.gpu


def _indices(tokens: int, topk: int, n_experts: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.rand(tokens, n_experts, generator=g).topk(topk, dim=-1)[1].cuda()


def _outputs(tokens: int, topk: int, n_experts: int):
    dev = "cuda"
    return (torch.full((n_experts + 1,), -1, dtype=torch.int32, device=dev),
            torch.full((tokens * topk,), -1, dtype=torch.int32, device=dev),
            torch.full((tokens * topk,), -1, dtype=torch.int32, device=dev))


def _with_workspace(lib, idx, n_experts):
    tokens, topk = idx.shape
    out = _outputs(tokens, topk, n_experts)
    ws = torch.empty(max(int(lib.rt_moe_permute_workspace_bytes(tokens, topk, n_experts)), 4),
                     dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.rt_moe_permute(idx.data_ptr(), out[0].data_ptr(), out[1].data_ptr(),
                                  out[2].data_ptr(), ws.data_ptr(), tokens, topk, n_experts, stream),
               "rt_moe_permute")
    return out


def _static(lib, idx, n_experts):
    tokens, topk = idx.shape
    out = _outputs(tokens, topk, n_experts)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.rt_moe_permute_static(idx.data_ptr(), out[0].data_ptr(), out[1].data_ptr(),
                                         out[2].data_ptr(), tokens, topk, n_experts, stream),
               "rt_moe_permute_static")
    return out


def test_static_scratch_permute_matches_workspace_permute_twice_in_a_row():
    lib = _lib.load()
    # first call: the DeepSeek-V3.2 routing shape; second call: a smaller problem with other
    # expert counts, so stale histogram entries from the first call would show up
    cases = [(4096, 8, 256, 1), (777, 4, 16, 2)]
    for tokens, topk, n_experts, seed in cases:
        idx = _indices(tokens, topk, n_experts, seed)
        got = _static(lib, idx, n_experts)
        want = _with_workspace(lib, idx, n_experts)
        torch.cuda.synchronize()
        for g, w, name in zip(got, want, ("expert_offsets", "sorted_pairs", "pair_pos")):
            assert torch.equal(g, w), f"{name} differs for tokens={tokens}"
        assert int(got[0][-1]) == tokens * topk
    # and once more on the first shape, after the array held the second call's data
    idx = _indices(*cases[0])
    for g, w in zip(_static(lib, idx, 256), _with_workspace(lib, idx, 256)):
        assert torch.equal(g, w)


def test_static_scratch_permute_refuses_what_does_not_fit():
    lib = _lib.load()
    limit = int(lib.rt_moe_permute_static_max_ints())
    assert limit == 65536
    tokens, topk, n_experts = 65536, 8, 256          # 512 blocks x 256 experts = 131072 entries
    idx = torch.zeros(tokens, topk, dtype=torch.int64, device="cuda")
    out = _outputs(tokens, topk, n_experts)
    rc = lib.rt_moe_permute_static(idx.data_ptr(), out[0].data_ptr(), out[1].data_ptr(),
                                   out[2].data_ptr(), tokens, topk, n_experts, None)
    assert rc == -2
    msg = lib.rt_last_error().decode()
    assert "scratch" in msg and "rt_moe_permute" in msg
    assert int(out[0][0]) == -1                      # nothing ran
