"""ctypes binding of librt_b200.so, the C-ABI kernel library (see include/rt_b200.h).

The library is loaded lazily on first use. There is no fallback: when the shared
object is missing or a call returns a non-zero status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "librt_b200.so"

RT_BF16, RT_F32, RT_F16 = 0, 1, 2
RT_ROPE_HALF, RT_ROPE_INTERLEAVED = 0, 1
RT_SF_ROWMAJOR, RT_SF_TILED128x4 = 0, 1
RT_SCORE_SIGMOID, RT_SCORE_SOFTMAX, RT_SCORE_TOPK_SOFTMAX = 0, 1, 2

_P, _I, _L, _F = c_void_p, c_int, c_int64, c_float

# name -> (restype, argtypes); must list every symbol include/rt_b200.h declares.
SIGNATURES: dict[str, tuple] = {
    "rt_version": (_I, []),
    "rt_last_error": (c_char_p, []),
    "rt_launch_count": (_L, []),
    "rt_residual_norm": (_I, [_P, _P, _P, _I, _P, _P, _L, _L, _L, _L, _F, _I, _P]),
    "rt_rms_norm": (_I, [_P, _P, _I, _P, _L, _L, _L, _L, _F, _I, _P]),
    "rt_norm_rope": (_I, [_P, _P, _P, _P, _I, _P, _P, _P, _L, _P, _P, _P,
                          _L, _L, _L, _L, _L, _L, _L, _F, _I, _I, _P]),
    "rt_rope": (_I, [_P, _P, _P, _L, _P, _L, _L, _L, _L, _L, _L, _L, _I, _I, _P]),
    "rt_head_broadcast": (_I, [_P, _P, _L, _L, _L, _L, _L, _L, _I, _P]),
    "rt_swiglu": (_I, [_P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "rt_act_quant_fp8": (_I, [_P, _P, _P, _L, _L, _L, _I, _P]),
    "rt_swiglu_quant_fp8": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "rt_absmax": (_I, [_P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "rt_nvfp4_quant": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P]),
    "rt_moe_route": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _F, _I, _P]),
    "rt_moe_permute_workspace_bytes": (_L, [_L, _L, _L]),
    "rt_moe_permute": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _P]),
    "rt_moe_permute_static_max_ints": (_L, []),
    "rt_moe_permute_static": (_I, [_P, _P, _P, _P, _L, _L, _L, _P]),
    "rt_moe_gather": (_I, [_P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "rt_moe_combine": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _P, _P, _I, _P]),
    "rt_absmax_rows": (_I, [_P, _P, _P, _L, _L, _L, _L, _P, _P, _I, _P]),
    "rt_swiglu_absmax_rows": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _P, _P, _I, _P]),
    "rt_moe_quant_nvfp4": (_I, [_P, _P, _P, _L, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P]),
    "rt_moe_gather_nvfp4": (_I, [_P, _P, _P, _L, _P, _P, _P, _P, _L, _L, _P]),
    "rt_gemm_bf16": (_I, [_P, _P, _P, _L, _L, _L, _L, _L, _L, _I, _P]),
    "rt_gemm_bf16_batched": (_I, [_P, _P, _P] + [_L] * 10 + [_P]),
    "rt_gemm_bf16_splitk_splits": (_L, [_L, _L, _L]),
    "rt_gemm_bf16_splitk": (_I, [_P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P]),
    "rt_gemm_fp8": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P]),
    "rt_tc_error_state": (_I, []),
    "rt_moe_tile_map": (_I, [_P, _L, _L, _P, _P, _P, _L, _P]),
    "rt_gemm_nvfp4_schedule": (_I, [_I]),
    "rt_index_prep": (_I, [_P, _P, _P, _P, _P, _L, _L, _P, _P, _P, _L, _L, _L, _L, _F, _I, _P]),
    "rt_fp8_index": (_I, [_P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P]),
    "rt_fp8_index_batched": (_I, [_P, _P, _P, _P, _P] + [_L] * 10 + [_P]),
    "rt_index_topk": (_I, [_P, _P, _L, _L, _L, _L, _P]),
    "rt_mla_sparse_decode_splits": (_L, [_L, _L, _L]),
    "rt_mla_sparse_decode": (_I, [_P] * 8 + [_L] * 14 + [_F, _P]),
    "rt_attn_causal_prefill": (_I, [_P] * 5 + [_L] * 15 + [_F, _P]),
    "rt_attn_causal_prefill_fp8": (_I, [_P] * 6 + [_L] * 13 + [_F, _P]),
    "rt_attn_prefill_schedule": (_I, [_I]),
    "rt_peer_alloc": (_I, [_L, _P, _P]),
    "rt_peer_open": (_I, [_P, _P]),
    "rt_peer_close": (_I, [_P]),
    "rt_peer_free": (_I, [_P]),
    "rt_peer_barrier": (_I, [_P, _L, _L, _P]),
    "rt_peer_error_state": (_I, []),
    "rt_peer_reduce_residual_norm": (_I, [_P, _L, _L, _L, _P, _P, _I, _P, _P, _L, _L, _L, _F, _P]),
    "rt_peer_gather": (_I, [_P, _P, _L, _L, _L, _P]),
    "rt_peer_gather_cols": (_I, [_P, _P, _P, _L, _L, _L, _L, _P]),
    "rt_peer_allmax": (_I, [_P, _L, _P, _P]),
    "rt_gemm_bf16_schedule": (_I, [_I]),
    "rt_gemm_nvfp4_grouped": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _L, _L, _P]),
}

_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Loads librt_b200.so once and attaches the signatures above."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"librt_b200.so not found at {LIB_PATH}; build it with `python -m racetrack_b200.build` "
            "(there is no CPU or torch fallback for these ops)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def available() -> bool:
    return LIB_PATH.exists()


def check(status: int, what: str) -> None:
    """Turns a non-zero rt_status into a RuntimeError carrying rt_last_error()."""
    if status != 0:
        msg = load().rt_last_error()
        text = msg.decode("utf-8", "replace") if msg else ""
        raise RuntimeError(f"{what} failed with status {status}: {text}")


def launch_count() -> int:
    return int(load().rt_launch_count())
