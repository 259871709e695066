"""Python entry points of the fused compute+collective kernels, and their NCCL baselines.

* :func:`gemm_rs` - ``out_shard = reduce_scatter(A_r @ W_r^T) (+ residual)`` in ONE kernel:
  tcgen05 tiles whose epilogue stores the partial sums straight into the owning rank's
  staging slot over NVLink and then reduces the rows this rank owns.
* :func:`gemm_ag` - ``C = all_gather(X_shard) @ W^T`` in ONE kernel: copy CTAs pull the peers'
  row shards while the tensor cores start on the local shard.
* ``*_nccl`` - the unfused baseline (library GEMM + NCCL collective), used by the benchmarks
  and as the numerical reference in tests. It is never used on the serving path.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from parallax_b200.ops import _lib, cuda as cu
from parallax_b200.ops._lib import EPI_NONE, EPI_SILU_MUL, check
from parallax_b200.parallel.symm import TPWorkspace

_bound = {}


def _fn(name: str, argtypes):
    if name not in _bound:
        _bound[name] = _lib.bind(name, argtypes)
    return _bound[name]


def _rs_fn():
    from ctypes import c_int, c_uint32, c_void_p as P

    return _fn("pxl_gemm_bf16_rs", [P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_uint32, c_int, P, P])


def _ag_fn():
    from ctypes import c_int, c_uint32, c_void_p as P

    return _fn("pxl_gemm_bf16_ag", [P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                    c_uint32, c_int, c_int, P, P])


def gemm_rs(ws: TPWorkspace, a: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    """a ``[tp*Rp, K_local]``, w ``[N, K_local]`` -> out ``[Rp, N]`` (rows owned by this rank)."""
    M, K = a.shape
    N = w.shape[0]
    Rp = M // ws.tp
    assert M == ws.tp * Rp and Rp % 128 == 0 and Rp <= ws.max_rows and N <= ws.max_n
    s, epoch = ws.next_set()
    if out is None:
        out = torch.empty((Rp, N), dtype=a.dtype, device=a.device)
    code = _rs_fn()(a.data_ptr(), w.data_ptr(), out.data_ptr(), None if residual is None else residual.data_ptr(),
                    ws.buf.ptr_array(ws.stage_off(s)), ws.buf.ptr_array(ws.rs_flag_off(s)), ws.rank, ws.tp, Rp, N, K,
                    a.stride(0), w.stride(0), out.stride(0), epoch, bn, cu.status_tensor(a.device).data_ptr(),
                    cu._stream(a.device))
    check(code, "pxl_gemm_bf16_rs")
    cu._count()
    return out


def gemm_ag_begin(ws: TPWorkspace, rows_per_rank: int, k: int):
    """Reserve a buffer set; returns ``(token, x_shard)``: write this rank's rows into
    ``x_shard`` (e.g. as the output of RMSNorm), then call :func:`gemm_ag` with the token."""
    s, epoch = ws.next_set()
    return (s, epoch, rows_per_rank, k), ws.x_shard(s, rows_per_rank, k)


def gemm_ag(ws: TPWorkspace, token, w: torch.Tensor, bias: Optional[torch.Tensor] = None, epi: int = EPI_NONE,
            ncopy: int = 0, bn: int = 0) -> torch.Tensor:
    s, epoch, Rp, K = token
    N = w.shape[0]
    M = ws.tp * Rp
    n_out = N // 2 if epi == EPI_SILU_MUL else N
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=w.device)
    code = _ag_fn()(ws.buf.ptr_array(ws.x_off(s)), ws.buf.ptr_array(ws.ag_flag_off(s)), ws.tile_flags[s].data_ptr(),
                    w.data_ptr(), out.data_ptr(), None if bias is None else bias.data_ptr(), ws.rank, ws.tp, Rp, N, K,
                    K, w.stride(0), out.stride(0), epi, epoch, ncopy, bn, cu.status_tensor(w.device).data_ptr(),
                    cu._stream(w.device))
    check(code, "pxl_gemm_bf16_ag")
    cu._count()
    return out


def gathered_input(ws: TPWorkspace, token) -> torch.Tensor:
    """The full gathered matrix of a finished :func:`gemm_ag` (valid after that kernel)."""
    s, _epoch, Rp, K = token
    return ws.x_full(s, Rp, K)


# ------------------------------------------------------------------ NCCL baselines
def gemm_rs_nccl(group, a: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    tp = dist.get_world_size(group)
    partial = torch.matmul(a, w.t())
    out = torch.empty((a.shape[0] // tp, w.shape[0]), dtype=a.dtype, device=a.device)
    dist.reduce_scatter_tensor(out, partial, group=group)
    if residual is not None:
        out += residual
    return out


def gemm_ag_nccl(group, x_shard: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 silu_mul: bool = False) -> torch.Tensor:
    tp = dist.get_world_size(group)
    full = torch.empty((x_shard.shape[0] * tp, x_shard.shape[1]), dtype=x_shard.dtype, device=x_shard.device)
    dist.all_gather_into_tensor(full, x_shard, group=group)
    y = torch.matmul(full, w.t())
    if bias is not None:
        y = y + bias
    if silu_mul:
        from parallax_b200.ops import reference as ref

        y = ref.linear(full, w, epi=EPI_SILU_MUL)
    return y
