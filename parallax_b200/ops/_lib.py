"""ctypes binding of ``libpxl_kernels.so`` (the sm_100a kernel library).

The library is loaded lazily. On a machine with a CUDA device a missing library is a hard
error: the GPU path never falls back silently to PyTorch eager.
"""

from __future__ import annotations

import ctypes
from ctypes import c_uint32, c_float, c_int, c_int64, c_void_p
from functools import lru_cache

from parallax_b200 import _build

PXL_OK = 0
_ERRORS = {
    1: "invalid argument",
    2: "CUDA launch error",
    3: "tensor-map encode failed",
    4: "size beyond the supported maximum",
    101: "device wait timed out (TMA stage full)",
    102: "device wait timed out (TMA stage empty)",
    103: "device wait timed out (accumulator full)",
    104: "device wait timed out (accumulator empty)",
    105: "device wait timed out (peer flag)",
    106: "index out of range (block table / slot / expert / row id)",
    107: "KV-cache slot of a token outside the cache",
    108: "row id of a gather (token id / logit row) outside the table",
    109: "block-table entry read by decode attention outside the cache",
    110: "block-table entry read by prefill attention (or the cp.async decode path) outside the cache",
    112: "a token position outside the rotary table (longer than the engine's max_total_length)",
    111: "a row of logits had no finite value (NaN activations): token 0 was returned for it",
}

EPI_NONE, EPI_RESIDUAL, EPI_SILU_MUL, EPI_F32 = 0, 1, 2, 3


class KernelError(RuntimeError):
    pass


def describe(code: int) -> str:
    return _ERRORS.get(code, f"error {code}")


def check(code: int, what: str) -> None:
    if code != PXL_OK:
        raise KernelError(f"{what}: {describe(code)}")


_P = c_void_p
_SIGS = {
    "pxl_gemm_bf16": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "pxl_gemm_bf16_pick_bn": [c_int, c_int, c_int],
    "pxl_gemm_bf16_small_m": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "pxl_gemm_bf16_uses_small_m": [c_int, c_int, c_int, c_int],
    "pxl_gemm_bf16_mid_m_plan": [c_int, c_int, c_int, c_int],
    "pxl_gemm_bf16_mid_m": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "pxl_rmsnorm": [_P, _P, _P, _P, c_int, c_int, c_float, c_float, _P],
    "pxl_qk_norm_rope_cache": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int64, c_float, c_float, c_int, _P, _P],
    "pxl_reshape_and_cache": [_P, _P, c_int64, c_int64, _P, _P, _P, c_int, c_int, c_int, c_int,
                              c_int, c_int64, _P, _P],
    "pxl_qk_norm_rope_cache_fp8": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int64, c_float, c_float, c_float, c_float, c_int, _P, _P],
    "pxl_reshape_and_cache_fp8": [_P, _P, c_int64, c_int64, _P, _P, _P, c_int, c_int, c_int, c_int,
                                  c_int, c_int64, c_float, c_float, _P, _P],
    "pxl_attn_decode_fp8": [_P, c_int64, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int64, c_float, c_int, c_int, c_int, c_float, c_float, _P, _P],
    "pxl_attn_prefill_fp8": [_P, c_int64, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int64, c_float, c_int, c_float, c_float, _P, _P],
    "pxl_dsa_index_prep": [_P, c_int64, _P, c_int64, c_int, c_int, _P, _P, c_float, _P, _P, c_int, _P, _P, c_int64, _P,
                           c_float, c_int, c_int, c_int, c_int, _P, _P],
    "pxl_act_mul": [_P, _P, c_int, c_int, c_int, c_float, _P],
    "pxl_gather_rows": [_P, _P, _P, c_int, c_int, c_int64, c_int, _P, _P],
    "pxl_add_inplace": [_P, _P, c_int64, _P],
    "pxl_selftest_bounded_wait": [_P, c_uint32, _P, _P, _P],
    "pxl_patch_i32": [_P, _P, _P, _P, c_int, c_int, c_int, _P, _P],
    "pxl_attn_decode": [_P, c_int64, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_int64, c_float, c_int, c_int, c_int, _P, _P],
    "pxl_attn_decode_splits": [c_int, c_int, c_int],
    "pxl_attn_prefill": [_P, c_int64, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_int, c_int64, c_float, c_int, _P, _P],
    "pxl_attn_prefill_tc": [_P, c_int64, _P, _P, _P, _P, _P, _P, c_int64, _P, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_int, c_int64, c_float, c_int, _P, _P],
    "pxl_moe_route": [_P, c_int, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, _P, _P, _P],
    "pxl_moe_align": [_P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, _P],
    "pxl_moe_gather": [_P, _P, _P, _P, c_int, c_int, _P],
    "pxl_moe_combine": [_P, _P, _P, _P, _P, c_int, c_int, c_int, _P],
    "pxl_gemm_bf16_grouped": [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P,
                              c_int, c_int, c_int, _P, _P],
    "pxl_mla_kv_prep": [_P, c_int64, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int64, c_float, _P, _P],
    "pxl_mla_q_prep": [_P, c_int64, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P],
    "pxl_mla_attn": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_int, c_float, _P],
    "pxl_dsa_index_scores": [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P],
    "pxl_topk_select": [_P, c_int64, _P, c_int, c_int, _P, c_int64, _P],
    "pxl_store_rows": [_P, c_int64, _P, _P, c_int, c_int, c_int64, _P, _P],
    "pxl_gemm_fp8_block": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P],
    "pxl_gemm_fp8_block_grouped": [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P,
                                   c_int, c_int, _P, _P],
    "pxl_quant_fp8_rows": [_P, c_int64, _P, _P, c_int, c_int, _P],
    "pxl_causal_conv1d_silu": [_P, c_int64, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P],
    "pxl_gated_delta_rule": [_P, c_int64, _P, _P, c_int64, _P, _P, _P, c_int64, _P, _P, _P, _P, _P, _P, c_int64,
                             c_int, c_int, c_int, c_int, c_int, c_float, _P],
    "pxl_sigmoid_gate_mul": [_P, c_int64, _P, c_int64, _P, c_int64, c_int, c_int, _P],
    "pxl_gate_mul_grouped": [_P, c_int64, _P, c_int64, _P, c_int64, _P, c_int64, c_int, c_int, c_int, _P],
    "pxl_row_dot": [_P, c_int64, _P, _P, c_int, c_int, _P],
    "pxl_msa_block_scores": [_P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_float, _P],
    "pxl_msa_select": [_P, c_int64, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int64, _P, _P],
    "pxl_rmsnorm_strided": [_P, c_int64, _P, _P, c_int64, c_int, c_int, c_float, c_float, _P],
    "pxl_argmax": [_P, c_int, c_int64, c_int, c_int, _P, _P, _P, _P],
    "pxl_apply_penalties": [_P, c_int, c_int64, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P],
    "pxl_sample": [_P, c_int, c_int64, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P],
}


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    path = _build.lib_path()
    if not path.exists():
        raise KernelError(
            f"{path} is missing: run `python -m parallax_b200._build` (needs nvcc) before using "
            "the CUDA ops"
        )
    handle = ctypes.CDLL(str(path))
    for name, argtypes in _SIGS.items():
        fn = getattr(handle, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int
    return handle


def bind(name: str, argtypes: list) -> ctypes._CFuncPtr:
    """Bind a symbol that is not in the static table (used by optional kernels)."""
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = c_int
    return fn


def available() -> bool:
    try:
        lib()
        return True
    except (KernelError, OSError):
        return False
