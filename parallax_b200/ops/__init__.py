"""Operator layer.

``ops.<name>(...)`` runs the hand-written sm_100a kernel when the tensors live on a CUDA
device and the plain-PyTorch restatement (:mod:`.reference`) on CPU. The CPU path exists for
correctness checks only; there is no alternative GPU backend.
"""

from __future__ import annotations

import torch

from . import reference
from ._lib import EPI_F32, EPI_NONE, EPI_RESIDUAL, EPI_SILU_MUL, KernelError

_NAMES = [
    "linear", "rmsnorm", "qk_norm_rope_cache", "reshape_and_cache", "act_mul", "gather_rows",
    "add_inplace", "patch_ids", "attn_decode", "attn_prefill", "argmax", "apply_penalties", "sample", "moe_route", "moe_ffn",
    "mla_kv_prep", "mla_q_absorb", "mla_attn", "mla_unabsorb", "store_rows", "dsa_index_prep", "dsa_index_scores", "topk_select",
    "quant_fp8_rows", "linear_fp8", "moe_ffn_fp8", "causal_conv1d_silu", "gated_delta_rule", "sigmoid_gate_mul", "gate_mul_grouped", "row_dot", "msa_block_scores", "msa_select",
]


def _first_tensor(args, kwargs):
    for a in list(args) + list(kwargs.values()):
        if isinstance(a, torch.Tensor):
            return a
    raise TypeError("op called without tensor arguments")


def _make(name):
    ref_fn = getattr(reference, name)

    def op(*args, **kwargs):
        t = _first_tensor(args, kwargs)
        if t.is_cuda:
            from . import cuda

            return getattr(cuda, name)(*args, **kwargs)
        return ref_fn(*args, **kwargs)

    op.__name__ = name
    op.__doc__ = ref_fn.__doc__
    return op


for _n in _NAMES:
    globals()[_n] = _make(_n)

build_cos_sin = reference.build_cos_sin
interleave_gate_up = reference.interleave_gate_up

__all__ = _NAMES + ["build_cos_sin", "interleave_gate_up", "reference", "KernelError",
                    "EPI_NONE", "EPI_RESIDUAL", "EPI_SILU_MUL", "EPI_F32"]
